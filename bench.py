#!/usr/bin/env python
"""bench.py — NVILA-8B single-image request (BASELINE.json configs[1]) on B200, plus the blocks the
other BASELINE configs need (all in ONE JSON line, printed by rank 0).

One "step" = one request through the hot path: 1 x 448^2 synthetic image -> SigLIP tower ->
mm_projector -> text/media splice -> Qwen2-7B prefill (S = 257 visual + 22 text = 279) -> first token
(TTFT) -> 127 more greedy tokens (CUDA-graph decode).  Random-init weights of the named architecture
(no checkpoints / network), bf16.

  value           decode tokens/s (README "decode throughput"), inputs resident in HBM, CUDA events
  ttft_ms         time to first token for the same request, inputs resident in HBM
  e2e             the same two numbers through the public API (LlavaLlamaModel.generate) with HOST
                  buffers: pinned pixels + ids copied H2D and the new ids read back D2H inside the region
  roofline        dominant kernel = the gate/up decode GEMV; algorithmic bytes = N*K*2 per launch
  decode_kernels  every kernel of the decode step timed live (CUDA events, back to back over all
                  layers' weights): achieved GB/s and fraction of the measured HBM peak
  ttft_roofline   flops / bytes / floor of the TTFT path and the achieved fraction
  video_decode    BASELINE configs[2] follow-up: 64-frame prefill (S = 16.5K) then 128 greedy tokens
                  through LlavaLlamaModel.generate: decode tok/s at ctx 16.5K with its HBM roofline
  batched_decode  serving follow-up: 8 concurrent copies of the request, continuous batching over one
                  shared paged pool (vila_b200/serving.py): aggregate tok/s
  tiled_image     BASELINE configs[3]: a dynamic-S2 tiled image (35 tiles of 448^2 -> tower -> S2 merge ->
                  projector) through encode_images, with its tensor-core floor (N = 1 runs only; last block of the run)
  sp_prefill      BASELINE configs[4]: LongVILA 256 frames (S = 65,814), sequence-parallel over ALL
                  ranks of this launch through LlavaLlamaModel.generate(max_new_tokens=1) with
                  vila_b200.sp enabled; first-token id + last-token logits top-5 / checksum so runs at
                  N = 1/2/4/8 can be compared from the driver's SCALE file alone (strong scaling)
  cpu_baseline    the oracle (PyTorch port of the reference's modules) on the host cores: the FULL
                  26-layer tower + projector + 28-layer prefill once, then a bounded number of decode
                  tokens through all 28 layers (no extrapolation); thread count swept and stated

`--impl reference`      the same CPU port as its own arm (rank 0 only).
`--impl reference_gpu`  informational: HF transformers (SigLIP + Qwen2, sdpa, bf16, eager) on the same
                        B200 for the same request — the library path the reference would run.
Launch with torchrun for N > 1: the decode request does not shard at bs=1 ("replicas only",
SURVEY §8e): every rank serves its own replica, value = all ranks' tokens / max-over-ranks time; the
sp_prefill block is the part that really shards.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

if "--impl" in sys.argv and "reference" in sys.argv and os.environ.get("OMP_NUM_THREADS") == "1":
    # torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm sets its thread count explicitly
    os.environ.pop("OMP_NUM_THREADS")

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_TEXT_TOKENS = 22
NEW_TOKENS = 128


# ------------------------------------------------------------------------------------------------
def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback (B200_PROFILING.md)"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled DURING the timed region."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period: float = 0.2):
        self.index = index
        self.period = period
        self.samples = []
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                self.samples.append([x.strip() for x in out.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=3)

    def summary(self):
        sm = sorted(int(float(s[0])) for s in self.samples if s and s[0].replace(".", "").isdigit())
        mx = [int(float(s[1])) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        pw = [float(s[2]) for s in self.samples if len(s) > 2 and s[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            for i, n in enumerate(names):
                if len(s) > 3 + i and s[3 + i].lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_mhz_min": sm[0] if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w_max": max(pw) if pw else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
def make_request(cfg, seed=1):
    import torch
    g = torch.Generator().manual_seed(seed)
    S = cfg.vision_tower_cfg.image_size
    pixels = torch.randn(3, S, S, generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 151643, (PROMPT_TEXT_TOKENS,), generator=g).tolist()
    ids.insert(14, cfg.image_token_id)  # "<system/user text> <image> <question>"
    return pixels, torch.tensor([ids], dtype=torch.long)


def llm_weight_bytes(lc):
    layer_w = (lc.hidden_size * (lc.num_attention_heads + 2 * lc.num_key_value_heads) * lc.head_dim
               + lc.hidden_size * lc.num_attention_heads * lc.head_dim + 3 * lc.hidden_size * lc.intermediate_size)
    return 2 * (lc.num_hidden_layers * layer_w + lc.vocab_size * lc.hidden_size)


def decode_kernel_ledger(model, peaks, ctx=280):
    """Every kernel of one decode step, timed live with CUDA events: each kernel is launched back to
    back over ALL layers' weights (7.6 GB of gate/up weights etc. >> the 126 MB L2, so every launch
    streams from HBM; PDL lets launch i+1 prefetch under launch i exactly as in the decode graph)."""
    import torch

    from vila_b200 import ops
    llm = model.llm
    lc = llm.config
    Hq, Hkv, D = lc.num_attention_heads, lc.num_key_value_heads, lc.head_dim
    dev = llm.device
    x = torch.randn(lc.hidden_size, device=dev).to(torch.bfloat16)
    xa = torch.randn(Hq * D, device=dev).to(torch.bfloat16)
    xi = torch.randn(lc.intermediate_size, device=dev).to(torch.bfloat16)
    qkv = torch.empty((Hq + 2 * Hkv) * D, device=dev, dtype=torch.bfloat16)
    y = torch.empty(lc.hidden_size, device=dev, dtype=torch.bfloat16)
    act = torch.empty(lc.intermediate_size, device=dev, dtype=torch.bfloat16)
    key = torch.zeros(1, device=dev, dtype=torch.int64)
    dec = llm.decoder(NEW_TOKENS)
    cache = dec.cache if dec.cache is not None else dec.cache_for(ctx + NEW_TOKENS)
    pos = torch.tensor([ctx], dtype=torch.int32, device=dev)
    layers = list(llm.model.layers)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def per_layer(fn, reps=4, n=None):
        for li, l in enumerate(layers):
            fn(li, l)
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(reps):
            for li, l in enumerate(layers):
                fn(li, l)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / (reps * (n or len(layers)))

    rows = []

    def add(name, nbytes, us):
        gbs = nbytes / us / 1e3
        rows.append({"kernel": name, "algorithmic_bytes": int(nbytes), "us": round(us, 2),
                     "gbs": round(gbs, 1), "frac": round(gbs / peaks["hbm_gbs"], 4)})

    nq = (Hq + 2 * Hkv) * D
    add("gemv qkv (+RMSNorm, +bias) N=%d K=%d" % (nq, lc.hidden_size), 2 * nq * lc.hidden_size,
        per_layer(lambda li, l: ops.gemv(x, l._qkv_w, bias=l._qkv_b, norm_w=l.input_layernorm.weight,
                                         norm_eps=lc.rms_norm_eps, out=qkv, static_w=True)))
    add("decode_attn ctx=%d splits=%d (RoPE + KV append + attention; 0 = one CTA per query head)" % (ctx, dec.num_splits),
        2 * 2 * (ctx + 1) * Hkv * D,
        per_layer(lambda li, l: ops.decode_attention(qkv, pos, cache.k(li), cache.v(li), cache.page_table,
                                                     xa, dec.ws, dec.counters, llm.inv_freq, Hq, Hkv, D,
                                                     dec.num_splits, D ** -0.5)))
    add("gemv o_proj (+residual) N=%d K=%d" % (lc.hidden_size, Hq * D), 2 * lc.hidden_size * Hq * D,
        per_layer(lambda li, l: ops.gemv(xa, l.self_attn.o_proj.weight, residual=x, out=y, static_w=True)))
    add("gemv gate/up (+RMSNorm, SwiGLU) N=%d K=%d" % (2 * lc.intermediate_size, lc.hidden_size),
        2 * 2 * lc.intermediate_size * lc.hidden_size,
        per_layer(lambda li, l: ops.gemv(x, l._gu_w, norm_w=l.post_attention_layernorm.weight,
                                         norm_eps=lc.rms_norm_eps, swiglu=True, out=act, static_w=True)))
    add("gemv down (+residual) N=%d K=%d" % (lc.hidden_size, lc.intermediate_size),
        2 * lc.hidden_size * lc.intermediate_size,
        per_layer(lambda li, l: ops.gemv(xi, l.mlp.down_proj.weight, residual=x, out=y, static_w=True)))
    add("gemv lm_head (+RMSNorm, argmax) N=%d K=%d" % (lc.vocab_size, lc.hidden_size),
        2 * lc.vocab_size * lc.hidden_size,
        per_layer(lambda li, l: ops.gemv(x, llm.lm_head.weight, norm_w=llm.model.norm.weight,
                                         norm_eps=lc.rms_norm_eps, argmax_key=key, write_out=False,
                                         static_w=True), reps=1, n=len(layers)))
    return rows


def video_decode_block(model, peaks, frames_n=64, reps=3):
    """NVILA-Video follow-up to the headline: decode right after a 64-frame prefill (ctx 16.5K).
    Through LlavaLlamaModel.generate with device-resident frames; decode tok/s = 127 tokens /
    (t(128 new tokens) - t(1 new token))."""
    import torch
    cfg = model.config
    lc = cfg.llm_cfg
    g = torch.Generator(device="cuda").manual_seed(77)
    S_img = cfg.vision_tower_cfg.image_size
    frames = torch.randn(frames_n, 3, S_img, S_img, device="cuda", generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 151643, (PROMPT_TEXT_TOKENS,), generator=torch.Generator().manual_seed(8)).tolist()
    ids.insert(14, cfg.video_token_id)
    ids = torch.tensor([ids], dtype=torch.long)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def run(n_new):
        a, b = ev(), ev()
        a.record()
        out = model.generate(input_ids=ids, media={"video": [frames]}, media_config={"video": {}},
                             max_new_tokens=n_new, eos_token_id=None)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b), out

    run(1); run(NEW_TOKENS)
    t1 = sum(run(1)[0] for _ in range(reps)) / reps
    tn = sum(run(NEW_TOKENS)[0] for _ in range(reps)) / reps
    S = frames_n * 257 + PROMPT_TEXT_TOKENS
    ms_tok = (tn - t1) / (NEW_TOKENS - 1)
    kv_bytes = 2 * 2 * (S + NEW_TOKENS // 2) * lc.num_key_value_heads * lc.head_dim * lc.num_hidden_layers
    byts = llm_weight_bytes(lc) + kv_bytes
    del frames
    return {"workload": "NVILA-Video-8B: %d frames x 448^2 -> S=%d prefill, then %d greedy tokens (bs=1)"
                        % (frames_n, S, NEW_TOKENS),
            "decode_tok_s": round(1e3 / ms_tok, 2), "decode_ms_per_token": round(ms_tok, 4),
            "ttft_ms": round(t1, 2), "splits": model.llm.decoder(NEW_TOKENS).num_splits,
            "bytes_per_token": int(byts), "kv_bytes_per_token": int(kv_bytes),
            "achieved_gbs": round(byts / ms_tok / 1e6, 1),
            "frac_of_hbm_peak": round(byts / ms_tok / 1e6 / peaks["hbm_gbs"], 4)}


def tiled_image_block(peaks, reps=5):
    """BASELINE.json configs[3]: one dynamic-S2 tiled image — 1 + 4 + 5x6 = 35 tiles of 448^2 (what the tiler
    makes of a wide 4K frame at max_tiles 12) -> SigLIP tower -> multi-scale merge to the
    largest scale (C = 3456) -> mm_projector -> re-stitched token grid [7680, 3584].  Vision + projector only:
    the model is built with the dynamic-S2 configuration and a 2-layer LLM stub (encode_images never touches
    the LLM layers).  Same call and shapes as tests/test_fullsize_gpu.py::test_cfg4_matches_oracle_full_depth."""
    import dataclasses

    import torch

    from vila_b200.model import LlavaLlamaModel, nvila_8b_dynamic_s2
    cfg = nvila_8b_dynamic_s2()
    cfg.llm_cfg = dataclasses.replace(cfg.llm_cfg, num_hidden_layers=2)
    model = LlavaLlamaModel(cfg, device="cuda").init_random(0, device_rng=True)
    bs = (5, 6)
    n_tiles = 1 + 4 + bs[0] * bs[1]
    g = torch.Generator(device="cuda").manual_seed(5)
    tiles = torch.randn(n_tiles, 3, 448, 448, device="cuda", generator=g).to(torch.bfloat16)
    tiles_pin = tiles.cpu().pin_memory()
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def run(from_host):
        a, b = ev(), ev()
        a.record()
        x = tiles_pin.to("cuda", non_blocking=True) if from_host else tiles
        out = model.encode_images(x, block_sizes=[bs])
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b), out

    for _ in range(3):
        run(False)
    ms = sum(run(False)[0] for _ in range(reps)) / reps
    ms_h2d, out = 0.0, None
    for _ in range(reps):
        t, out = run(True)
        ms_h2d += t / reps
    tokens = int(out.shape[1])
    C, Hd = cfg.vision_tower_cfg.hidden_size, cfg.llm_cfg.hidden_size
    flops = n_tiles * (936e9 + 1.39e9) + bs[0] * bs[1] * 256 * (2 * 12 * C * Hd + 2 * Hd * Hd)
    floor_ms = flops / (peaks["bf16_tflops_sustained"] * 1e12) * 1e3
    del model, tiles
    torch.cuda.empty_cache()
    return {"workload": "dynamic-S2 tiled image: %d tiles x 448^2 (1 + 2x2 + %dx%d) -> tower -> S2 merge (C=%d) -> projector "
                        "-> %d tokens (BASELINE.json configs[3])" % (n_tiles, bs[0], bs[1], 3 * C, tokens),
            "api": "LlavaLlamaModel.encode_images(tiles, block_sizes=[(5, 6)])", "tiles": n_tiles, "tokens_out": tokens,
            "ms": round(ms, 3), "ms_with_h2d_of_tiles": round(ms_h2d, 3), "h2d_bytes": int(tiles_pin.numel() * 2),
            "tiles_per_s": round(n_tiles / (ms / 1e3), 1), "flops": flops, "floor_ms": round(floor_ms, 3),
            "frac_of_sustained_tensor_peak": round(floor_ms / ms, 4), "finite": bool(torch.isfinite(out.float()).all())}


def batched_decode_block(model, peaks, ids_h, pixels_d, slots=8):
    """Serving follow-up: `slots` copies of the headline request decoded together with
    continuous batching over one shared paged pool (vila_b200/serving.py): aggregate tok/s; the weights
    are streamed once per step for all slots."""
    import torch

    from vila_b200.serving import BatchedDecoder
    lc = model.config.llm_cfg
    emb, _, _ = model._embed(ids_h, {"image": [pixels_d]}, {"image": {}}, None, None)
    prompt = emb[0].clone()
    S = prompt.shape[0]
    dec = BatchedDecoder(model.llm, slots=slots, max_tokens_per_slot=1024, max_new=NEW_TOKENS)
    dec.capture()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    times = []
    for rep in range(3):
        for s_ in range(slots):
            dec.admit(s_, prompt)
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        dec.run(NEW_TOKENS - 1)
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        first = [dec.generated(s_)[:4] for s_ in range(slots)]
        for s_ in range(slots):
            dec.release(s_)
    ms = sum(times[1:]) / len(times[1:])
    step_ms = ms / (NEW_TOKENS - 1)
    kv = 2 * 2 * (S + NEW_TOKENS // 2) * lc.num_key_value_heads * lc.head_dim * lc.num_hidden_layers * slots
    byts = llm_weight_bytes(lc) + kv
    del dec
    return {"workload": "%d concurrent copies of the headline request (S=%d, %d greedy tokens each), continuous "
                        "batching over one shared paged pool" % (slots, S, NEW_TOKENS),
            "slots": slots, "aggregate_tok_s": round(slots * (NEW_TOKENS - 1) / (ms / 1e3), 1),
            "ms_per_step": round(step_ms, 4), "per_request_tok_s": round(1e3 / step_ms, 1),
            "bytes_per_step": int(byts), "achieved_gbs": round(byts / step_ms / 1e6, 1),
            "frac_of_hbm_peak": round(byts / step_ms / 1e6 / peaks["hbm_gbs"], 4),
            "all_slots_agree": bool(all(f == first[0] for f in first))}


def sp_prefill_block(model, args, peaks, rank, world, local):
    """BASELINE configs[4] through the public API with sequence parallelism over this launch's ranks."""
    import torch
    import torch.distributed as dist

    from vila_b200 import sp
    cfg = model.config
    lc = cfg.llm_cfg
    F = args.frames
    S_img = cfg.vision_tower_cfg.image_size
    g = torch.Generator(device="cuda").manual_seed(1234)  # the SAME video on every rank and for every N
    frames = torch.randn(F, 3, S_img, S_img, device="cuda", generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 151643, (PROMPT_TEXT_TOKENS,), generator=torch.Generator().manual_seed(7)).tolist()
    ids.insert(14, cfg.video_token_id)
    ids = torch.tensor([ids], dtype=torch.long)
    S = F * 257 + PROMPT_TEXT_TOKENS
    sp.set_sequence_parallel_group(None)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    vis_events = []
    orig = model._encode_frames

    def timed_encode(fr, batch=32):
        a, b = ev(), ev()
        a.record()
        r = orig(fr, batch)
        b.record()
        vis_events.append((a, b))
        return r

    model._encode_frames = timed_encode
    runner = model._sp_runner()
    pre_events = []
    orig_prefill = runner.prefill_hidden

    def timed_prefill(*a, **k):
        e0, e1 = ev(), ev()
        e0.record()
        r = orig_prefill(*a, **k)
        e1.record()
        pre_events.append((e0, e1))
        return r

    runner.prefill_hidden = timed_prefill

    def step():
        a, b = ev(), ev()
        a.record()
        out = model.generate(input_ids=ids, media={"video": [frames]}, media_config={"video": {}},
                             max_new_tokens=1, eos_token_id=None)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b), int(out[0, 0])

    try:
        est = 0.0
        for _ in range(max(3, args.warmup) if not args.profile else 1):
            est = step()[0]
        # at least --sp-steps steps, and long enough for >= 20 nvidia-smi clock samples (a query takes
        # ~0.75 s on an 8-GPU box): ~20 s of timed steps, capped at 80 steps; same count on every rank
        n_steps = torch.tensor([max(args.sp_steps, min(80, int(20000.0 / max(est, 1.0)) + 1))], device="cuda")
        dist.all_reduce(n_steps, op=dist.ReduceOp.MAX)
        n_steps = int(n_steps)
        dist.barrier(); torch.cuda.synchronize()
        vis_events.clear()
        pre_events.clear()
        rows = []
        with ClockSampler(local, period=0.1) as clocks:
            for _ in range(n_steps):
                rows.append(step())
            dist.barrier(); torch.cuda.synchronize()
        tot = torch.tensor([sum(r[0] for r in rows) / len(rows),
                            sum(a.elapsed_time(b) for a, b in vis_events) / max(1, len(vis_events)),
                            sum(a.elapsed_time(b) for a, b in pre_events) / max(1, len(pre_events))],
                           device="cuda", dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.MAX)
        ms, vis_ms, pre_ms = float(tot[0]), float(tot[1]), float(tot[2])
        tok = rows[-1][1]
        toks = torch.tensor([tok], device="cuda")
        all_toks = [torch.zeros_like(toks) for _ in range(world)]
        dist.all_gather(all_toks, toks)
        logits = model.llm.logits_from_hidden(model.llm.last_prefill_hidden[None])[0].float()
        top = torch.topk(logits, 5)
    finally:
        model._encode_frames = orig
        runner.prefill_hidden = orig_prefill
        sp.set_sequence_parallel_group(None, enabled=False)
    gemm_flops = 2.0 * 6.525e9 * S
    attn_flops = 2.0 * S * S * lc.num_attention_heads * lc.head_dim * lc.num_hidden_layers
    vit_flops = F * 936e9
    tf_gpu = (gemm_flops + attn_flops + vit_flops) / world / (ms / 1e3) / 1e12
    plan = sp.make_plan(S, world, rank)
    return {"workload": "LongVILA-8B %d frames x 448^2, S=%d tokens: vision tower sharded by frames + zigzag "
                        "SP-%d prefill + first token (BASELINE.json configs[4])" % (F, S, world),
            "api": "vila_b200.sp.set_sequence_parallel_group(); LlavaLlamaModel.generate(media={'video': [...]}, max_new_tokens=1)",
            "scaling": "strong", "n_gpus": world, "steps": n_steps, "warmup": max(3, args.warmup),
            "ms_per_step": round(ms, 2), "tok_s": round(S / (ms / 1e3), 1),
            "phase_ms_max_over_ranks": {"vision_tower_projector_gather": round(vis_ms, 2),
                                        "sp_prefill_28_layers": round(pre_ms, 2),
                                        "splice_host_glue_first_token": round(ms - vis_ms - pre_ms, 2)},
            "padded_len": plan.padded_len, "chunk": plan.chunk,
            "first_token_id": tok, "first_token_ids_all_ranks": [int(t) for t in all_toks],
            "logits_top5_ids": [int(i) for i in top.indices], "logits_top5": [round(float(v), 4) for v in top.values],
            "logits_checksum": {"sum": round(float(logits.sum()), 3), "l2": round(float(logits.norm()), 4)},
            "achieved_tflops_per_gpu": round(tf_gpu, 1),
            "frac_of_sustained_bf16_peak": round(tf_gpu / peaks["bf16_tflops_sustained"], 4),
            "clocks": clocks.summary()}


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if "RANK" not in os.environ:  # plain `python bench.py`: a 1-rank group (the SP block needs one)
        os.environ.update({"RANK": "0", "WORLD_SIZE": "1", "MASTER_ADDR": "127.0.0.1",
                           "MASTER_PORT": os.environ.get("MASTER_PORT", "29533")})
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from vila_b200 import _lib, ops
    from vila_b200.model import LlavaLlamaModel, nvila_8b

    cfg = nvila_8b()
    model = LlavaLlamaModel(cfg, device="cuda").init_random(0, device_rng=True)
    llm = model.llm
    pixels_h, ids_h = make_request(cfg, seed=1 + rank)
    pixels_pin = pixels_h.pin_memory()
    ids_pin = ids_h.pin_memory()
    pixels_d = pixels_h.cuda()
    media_cfg = {"image": {}}
    ev = lambda: torch.cuda.Event(enable_timing=True)

    vision_ms = []

    def request_device():
        """inputs resident in HBM; returns (t_ttft_ms, t_decode_ms)."""
        e0, e1, e2, ea = ev(), ev(), ev(), ev()
        e0.record()
        emb, _, _ = model._embed(ids_h, {"image": [pixels_d]}, media_cfg, None, None)
        ea.record()
        dec = llm.decoder(NEW_TOKENS)
        cache = dec.cache_for(emb.shape[1] + NEW_TOKENS)
        hid = llm.prefill_hidden_graphed(emb[0], cache)
        dec.start(hid[-1], cache)
        e1.record()
        dec.run(NEW_TOKENS)
        e2.record()
        torch.cuda.synchronize()
        vision_ms.append(e0.elapsed_time(ea))  # SigLIP tower + projector + splice
        return e0.elapsed_time(e1), e1.elapsed_time(e2), emb.shape[1]

    def request_e2e(n_new):
        """public API with host buffers (pinned): H2D of pixels/ids and D2H of ids inside the region."""
        e0, e1 = ev(), ev()
        e0.record()
        out = model.generate(input_ids=ids_pin, media={"image": [pixels_pin]}, media_config=media_cfg,
                             max_new_tokens=n_new, eos_token_id=None)
        out_h = out.cpu()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), out_h

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (graph capture, allocator, TMA descriptors) ----
    n_warm = 1 if args.profile else max(3, args.warmup)
    for _ in range(n_warm):
        request_device()
    request_e2e(1)
    request_e2e(NEW_TOKENS)

    # ---- timed: exactly K steps, device-resident ----
    launches0 = _lib.LAUNCHES
    barrier()
    ttfts, decs = [], []
    vision_ms.clear()
    with ClockSampler(local) as clocks:
        t_wall0 = time.perf_counter()
        for _ in range(args.steps):
            a, b, S = request_device()
            ttfts.append(a)
            decs.append(b)
        barrier()
        t_wall = time.perf_counter() - t_wall0
        launches_timed = _lib.LAUNCHES - launches0
        # e2e through the public API (host buffers)
        e2e_full, e2e_first = [], []
        for _ in range(args.steps):
            t, _ = request_e2e(NEW_TOKENS)
            e2e_full.append(t)
            t1, _ = request_e2e(1)
            e2e_first.append(t1)
    clock_summary = clocks.summary()
    peaks = read_peaks()
    # TTFT anatomy (outside the timed region): each stage alone, 10 repetitions, CUDA events around
    # the host call (so host-side Python that is not hidden behind GPU work shows up)
    def stage(fn, reps=10):
        fn(); torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(reps):
            fn()
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / reps
    emb0, _, _ = model._embed(ids_h, {"image": [pixels_d]}, media_cfg, None, None)
    emb0 = emb0[0].clone()
    dec0 = llm.decoder(NEW_TOKENS)
    cache0 = dec0.cache_for(emb0.shape[0] + NEW_TOKENS)
    def _prefill():
        cache0.length = 0
        return llm.prefill_hidden_graphed(emb0, cache0)
    hid0 = _prefill()
    anatomy = {"encode_images_graph": round(stage(lambda: model.encode_images(pixels_d[None])), 3),
               "embed_total (encoders + host index table + splice)": round(stage(lambda: model._embed(ids_h, {"image": [pixels_d]}, media_cfg, None, None)), 3),
               "prefill_graph": round(stage(_prefill), 3),
               "first_token (lm_head GEMV + finalize)": round(stage(lambda: dec0.start(hid0[-1], cache0)), 3)}
    ledger = decode_kernel_ledger(model, peaks, ctx=S)
    video = None
    if not (args.profile or args.no_video):
        try:
            video = video_decode_block(model, peaks)
        except Exception as e:  # the headline line must survive a failure of an extra block
            video = {"error": "%s: %s" % (type(e).__name__, str(e)[:300])}
            torch.cuda.synchronize()

    batched = None
    if not (args.profile or args.no_video):
        try:
            batched = batched_decode_block(model, peaks, ids_h, pixels_d, slots=8)
            batched["more_slots"] = [
                {k: v for k, v in batched_decode_block(model, peaks, ids_h, pixels_d, slots=n).items()
                 if k in ("slots", "aggregate_tok_s", "ms_per_step", "frac_of_hbm_peak", "all_slots_agree")}
                for n in (32,)]
        except Exception as e:
            batched = {"error": "%s: %s" % (type(e).__name__, str(e)[:300])}
            torch.cuda.synchronize()

    step_ms = [a + b for a, b in zip(ttfts, decs)]
    local_stats = torch.tensor([sum(step_ms) / len(step_ms), sum(decs) / len(decs), sum(ttfts) / len(ttfts),
                                sum(e2e_full) / len(e2e_full), sum(e2e_first) / len(e2e_first)],
                               device="cuda", dtype=torch.float64)
    dist.all_reduce(local_stats, op=dist.ReduceOp.MAX)
    ms_step, ms_dec, ms_ttft, ms_e2e_full, ms_e2e_first = local_stats.tolist()

    sp_block = None
    if not args.no_sp and not args.profile:
        try:
            sp_block = sp_prefill_block(model, args, peaks, rank, world, local)
        except Exception as e:  # the headline line must survive a failure of the extra block
            sp_block = {"error": "%s: %s" % (type(e).__name__, str(e)[:300])}
            torch.cuda.synchronize()

    if rank != 0:
        dist.destroy_process_group()
        return
    decode_tok_s = world * (NEW_TOKENS - 1) / (ms_dec / 1e3)
    e2e_decode_tok_s = world * (NEW_TOKENS - 1) / ((ms_e2e_full - ms_e2e_first) / 1e3)
    lc = cfg.llm_cfg
    weight_bytes_token = llm_weight_bytes(lc)
    gu = next(r for r in ledger if r["kernel"].startswith("gemv gate/up"))
    gemv_bytes, gemv_ms, achieved = gu["algorithmic_bytes"], gu["us"] / 1e3, gu["gbs"]
    ncu_file = ROOT / "profiles" / "ncu_dominant_kernel.json"
    traffic = None
    if ncu_file.exists():
        try:
            traffic = json.loads(ncu_file.read_text()).get("dram_bytes_per_launch")
        except Exception:
            traffic = None
    vis_avg = sum(vision_ms[:args.steps]) / max(1, min(len(vision_ms), args.steps))
    # TTFT floor: tower (26 evaluated layers) + projector on the tensor pipe, prefill at the ridge
    vit_flops, proj_flops = 936e9 + 1.39e9, 15.0e9
    prefill_flops = 2.0 * 6.525e9 * S + 2.0 * lc.vocab_size * lc.hidden_size
    tf = peaks["bf16_tflops_sustained"] * 1e12
    floor_vis = (vit_flops + proj_flops) / tf * 1e3
    floor_llm = max(prefill_flops / tf, weight_bytes_token / (peaks["hbm_gbs"] * 1e9)) * 1e3
    cpu = None
    if not args.no_cpu and world == 1:
        cpu = cpu_reference(cfg, seconds_budget=args.cpu_budget)["cpu_baseline"]
    dec_obj = llm.decoder(NEW_TOKENS)
    tiled = None
    if world == 1 and not (args.profile or args.no_video):
        try:  # last GPU work of the run; the headline line must survive a failure of this extra block
            tiled = tiled_image_block(peaks)
        except Exception as e:
            tiled = {"error": "%s: %s" % (type(e).__name__, str(e)[:300])}
    line = {
        "metric": "NVILA-8B decode tokens/sec (1 img 448^2, bs=1, 128 new tokens); TTFT reported as ttft_ms",
        "value": round(decode_tok_s, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": round(ms_step, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": round(decode_tok_s / world / 82.1, 3),
        "baseline_ref": "BASELINE.md: NVILA-8B FP16 PyTorch decode 82.1 tok/s on A100 (README.md:65); other hardware",
        "dtype": "bf16", "data": "synthetic (random-init weights of the named architecture, randn pixels, random ids)",
        "ttft_ms": round(ms_ttft, 3), "decode_ms_per_token": round(ms_dec / (NEW_TOKENS - 1), 4),
        "ttft_breakdown_ms": {"vision_projector_splice": round(vis_avg, 3),
                              "llm_prefill_first_token": round(ms_ttft - vis_avg, 3)},
        "ttft_anatomy_ms": anatomy,
        "config": {"workload": "NVILA-8B bf16, 1x448^2 image, prefill S=%d + %d-token greedy decode, bs=1 "
                               "(BASELINE.json configs[1])" % (S, NEW_TOKENS),
                   "vision": "SigLIP-so400m/14-448 (26 of 27 layers evaluated: hidden_states[-2])",
                   "projector": cfg.mm_projector_type, "llm": "Qwen2.5-7B architecture",
                   "parallelism": "replicas x%d (decode does not shard at bs=1); sp_prefill block: sp%d" % (world, world),
                   "l2_policy": "no flush needed: each decode step streams %.2f GB of weights (>> 126 MB L2)"
                                % (weight_bytes_token / 1e9)},
        "e2e": {"value": round(e2e_decode_tok_s, 2), "unit": "tok/s",
                "ttft_ms": round(ms_e2e_first, 3), "request_ms": round(ms_e2e_full, 3),
                "request_tok_s": round(world * NEW_TOKENS / (ms_e2e_full / 1e3), 2),
                # pixels (bf16) + the int32 splice index table built from the host ids
                "h2d_bytes_per_step": int(pixels_pin.numel() * 2 + S * 4),
                # token history (int32) read back once at the end + the returned LongTensor copied to host
                "d2h_bytes_per_step": int(NEW_TOKENS * 4 + NEW_TOKENS * 8),
                "api": "LlavaLlamaModel.generate(input_ids=<pinned host>, media={'image': [<pinned host>]})"},
        "gpu_launches": int(launches_timed + args.steps * (NEW_TOKENS - 1) * dec_obj.launches_per_step),
        "gpu_launches_note": "timed region (K device-resident requests): %d C-ABI kernel launches issued from Python "
                             "(vision, projector, splice, first token; the prefill replays a CUDA graph of ~230 "
                             "more that are not counted) + CUDA-graph replays of %d kernels per decoded token"
                             % (launches_timed, dec_obj.launches_per_step),
        "clocks": clock_summary,
        "roofline": {"kernel": "gemv_tma_kernel (gate/up SwiGLU GEMV, N=%d K=%d, fused RMSNorm prologue)"
                               % (2 * lc.intermediate_size, lc.hidden_size),
                     "bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": traffic,
                     "peak_source": peaks["source"], "algorithmic_bytes_per_launch": gemv_bytes,
                     "launch_ms": round(gemv_ms, 5)},
        "decode_kernels": ledger,
        "decode_step_roofline": {"weight_bytes_per_token": weight_bytes_token,
                                 "achieved_gbs": round(weight_bytes_token / (ms_dec / (NEW_TOKENS - 1) / 1e3) / 1e9, 1),
                                 "frac_of_hbm_peak": round(weight_bytes_token / (ms_dec / (NEW_TOKENS - 1) / 1e3) / 1e9
                                                           / peaks["hbm_gbs"], 4)},
        "ttft_roofline": {"vit_projector_flops": vit_flops + proj_flops, "prefill_flops": prefill_flops,
                          "prefill_weight_bytes": weight_bytes_token,
                          "floor_ms": {"vision": round(floor_vis, 3), "llm_prefill": round(floor_llm, 3),
                                       "total": round(floor_vis + floor_llm, 3)},
                          "peaks": "sustained bf16 %.0f TFLOP/s, HBM %.0f GB/s" % (peaks["bf16_tflops_sustained"], peaks["hbm_gbs"]),
                          "frac": round((floor_vis + floor_llm) / ms_ttft, 4),
                          "frac_vision": round(floor_vis / vis_avg, 4),
                          "frac_llm": round(floor_llm / max(ms_ttft - vis_avg, 1e-6), 4)},
        "video_decode": video,
        "batched_decode": batched,
        "tiled_image": tiled,
        "sp_prefill": sp_block,
        "cpu_baseline": cpu,
        "wall_s_timed_region": round(t_wall, 3),
    }
    print(json.dumps(line))
    dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
class CpuReference:
    """The reference's PyTorch path (oracle port) on the host cores at FULL size: 26 SigLIP layers +
    projector + 28 Qwen2-7B layers + lm_head in fp32 (~36 GB).  Weights: one randomly initialised
    layer per module type, the other layers are scaled copies written by a parallel multiply (so
    every layer owns distinct, touched memory; initialising 8 G parameters with the serial CPU RNG
    would take minutes and is not what is being measured)."""

    def __init__(self, cfg):
        import torch

        from oracle import vila_oracle as O
        self.O, self.torch, self.cfg = O, torch, cfg
        lc, vc = cfg.llm_cfg, cfg.vision_tower_cfg
        g = torch.Generator().manual_seed(0)

        def w(*shape, std=0.02):
            return torch.randn(*shape, generator=g) * std

        D, Hq, Hkv, Hd, I = lc.head_dim, lc.num_attention_heads, lc.num_key_value_heads, lc.hidden_size, lc.intermediate_size
        base = {"self_attn.q_proj.weight": w(Hq * D, Hd), "self_attn.q_proj.bias": w(Hq * D),
                "self_attn.k_proj.weight": w(Hkv * D, Hd), "self_attn.k_proj.bias": w(Hkv * D),
                "self_attn.v_proj.weight": w(Hkv * D, Hd), "self_attn.v_proj.bias": w(Hkv * D),
                "self_attn.o_proj.weight": w(Hd, Hq * D), "mlp.gate_proj.weight": w(I, Hd),
                "mlp.up_proj.weight": w(I, Hd), "mlp.down_proj.weight": w(Hd, I),
                "input_layernorm.weight": torch.ones(Hd), "post_attention_layernorm.weight": torch.ones(Hd)}
        p = {}
        for i in range(lc.num_hidden_layers):
            f = 1.0 + 0.01 * ((i * 7) % 5 - 2)
            for k, v in base.items():
                p[f"model.layers.{i}.{k}"] = v if i == 0 else v * f
        p["model.norm.weight"] = torch.ones(Hd)
        head = w(8192, Hd)
        reps = (lc.vocab_size + 8191) // 8192
        p["lm_head.weight"] = torch.cat([head * (1.0 + 0.003 * r) for r in range(reps)])[:lc.vocab_size].contiguous()
        p["model.embed_tokens.weight"] = p["lm_head.weight"]
        self.llm = p
        self.lcfg = O.Qwen2Cfg(Hd, I, lc.num_hidden_layers, Hq, Hkv, lc.vocab_size, lc.rms_norm_eps,
                               lc.rope_theta, D)
        C, Iv = vc.hidden_size, vc.intermediate_size
        sc = (2.0 / (2 * C)) ** 0.5
        vbase = {}
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            vbase[f"self_attn.{n}.weight"], vbase[f"self_attn.{n}.bias"] = w(C, C, std=sc), w(C)
        vbase["layer_norm1.weight"] = vbase["layer_norm2.weight"] = torch.ones(C)
        vbase["layer_norm1.bias"] = vbase["layer_norm2.bias"] = torch.zeros(C)
        vbase["mlp.fc1.weight"], vbase["mlp.fc1.bias"] = w(Iv, C, std=sc), w(Iv)
        vbase["mlp.fc2.weight"], vbase["mlp.fc2.bias"] = w(C, Iv, std=sc), w(C)
        vp = {}
        for i in range(vc.num_hidden_layers):
            for k, v in vbase.items():
                vp[f"vision_model.encoder.layers.{i}.{k}"] = v if i == 0 else v * (1.0 + 0.01 * (i % 3))
        vp["vision_model.embeddings.patch_embedding.weight"] = w(C, 3, vc.patch_size, vc.patch_size)
        vp["vision_model.embeddings.patch_embedding.bias"] = w(C)
        vp["vision_model.embeddings.position_embedding.weight"] = w(vc.num_patches, C)
        self.vision = vp
        self.vcfg = O.SiglipCfg(C, Iv, vc.num_hidden_layers, vc.num_attention_heads, vc.image_size, vc.patch_size)
        mm = 4 * C
        self.proj = {"layers.1.weight": torch.ones(mm), "layers.1.bias": torch.zeros(mm),
                     "layers.2.weight": w(Hd, mm), "layers.2.bias": w(Hd),
                     "layers.4.weight": w(Hd, Hd), "layers.4.bias": w(Hd)}
        self.pixels = torch.randn(1, 3, vc.image_size, vc.image_size, generator=g)
        self.text = torch.randn(PROMPT_TEXT_TOKENS + 1, Hd, generator=g) * 0.02
        self.past = None
        self.x = torch.randn(1, Hd, generator=g) * 0.02

    def ttft(self):
        """tower + projector + splice + 28-layer prefill + first-token logits; returns seconds"""
        O, torch = self.O, self.torch
        t0 = time.perf_counter()
        with torch.no_grad():
            feats = O.siglip_tower(self.pixels, self.vision, self.vcfg, -2)
            tok = O.projector(feats, self.proj, "mlp_downsample")[0]
            emb = torch.cat([self.text[:14], tok, self.text[14:]], 0)
            logits, self.past = O.qwen2_forward(emb, self.llm, self.lcfg, last_only=True)
            int(torch.argmax(logits[-1]))
        return time.perf_counter() - t0, emb.shape[0]

    def decode(self, n_tokens):
        """n greedy-decode steps through all 28 layers at the current context; past is NOT grown across
        calls beyond n tokens (each call restarts from the prefill's cache) so every sample is the same work"""
        O, torch = self.O, self.torch
        past = self.past
        t0 = time.perf_counter()
        with torch.no_grad():
            x = self.x
            for _ in range(n_tokens):
                logits, past = O.qwen2_forward(x, self.llm, self.lcfg, past=past, last_only=True)
                tok = int(torch.argmax(logits[-1]))
                x = self.llm["model.embed_tokens.weight"][tok][None, :]
        return time.perf_counter() - t0


def pick_threads(ref, candidates=None):
    """CPU decode is a memory-bound GEMV chain: more threads than memory channels need only adds
    synchronisation cost (128 threads on the 128-CPU B200 host: 26 s per token; 16 threads: 0.18 s).
    Sweep thread counts upwards on one decode token each, keep the fastest, and stop as soon as a count
    is more than 2x slower than the best so far (so the sweep itself stays cheap)."""
    import torch
    n = os.cpu_count() or 1
    cand = candidates or sorted({c for c in (8, 16, 32, 64, n // 2, n) if 1 <= c <= n})
    timings = {}
    best_t = None
    for c in cand:
        torch.set_num_threads(c)
        t = ref.decode(1)            # first token at this count (also the warm-up)
        if best_t is None or t < 2.0 * best_t:
            t = min(t, ref.decode(1), ref.decode(1))
        timings[c] = t
        if best_t is not None and t > 2.0 * best_t:
            break
        best_t = t if best_t is None else min(best_t, t)
    best = min(timings, key=timings.get)
    torch.set_num_threads(best)
    return best, {str(k): round(v, 4) for k, v in timings.items()}


def cpu_reference(cfg, seconds_budget=25.0, steps=1, warmup=0, tokens_per_step=8):
    """Returns {"cpu_baseline": {...}, "ttft_s": ..., "tok_s": ...}: the full-size CPU port, measured."""
    import torch
    t_build0 = time.perf_counter()
    ref = CpuReference(cfg)
    t_build = time.perf_counter() - t_build0
    torch.set_num_threads(os.cpu_count() or 1)
    t_ttft, S = ref.ttft()       # also builds the KV cache the decode samples start from
    best, sweep = pick_threads(ref)
    t_ttft2, _ = ref.ttft()      # with the chosen thread count
    ttft = min(t_ttft, t_ttft2)
    per_tok = ref.decode(2) / 2
    tokens_per_step = max(2, min(tokens_per_step, int(seconds_budget / max(1, steps + warmup) / max(per_tok, 1e-3))))
    for _ in range(warmup):
        ref.decode(tokens_per_step)
    times = [ref.decode(tokens_per_step) for _ in range(max(1, steps))]
    tok_s = tokens_per_step * len(times) / sum(times)
    cb = {"value": round(tok_s, 4), "unit": "tok/s", "cores": best, "kind": "port",
          "host_cpus": os.cpu_count(), "thread_sweep_s_per_token": sweep,
          "ttft_s": round(ttft, 3), "weights_build_s": round(t_build, 1),
          "sample": "oracle (fp32 PyTorch port of the reference modules) at FULL size on the host: %d-layer SigLIP "
                    "tower + projector + %d-layer LLM prefill at S=%d measured once (ttft_s), then %d x %d greedy "
                    "decode tokens through all %d layers + full-vocab lm_head at ctx %d (no extrapolation); "
                    "threads = fastest of the sweep"
                    % (cfg.vision_tower_cfg.num_hidden_layers - 1, cfg.llm_cfg.num_hidden_layers, S, len(times),
                       tokens_per_step, cfg.llm_cfg.num_hidden_layers, S)}
    return {"cpu_baseline": cb, "ttft_s": ttft, "tok_s": tok_s, "tokens_per_step": tokens_per_step,
            "step_s": sum(times) / len(times)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from vila_b200.model import nvila_8b
    cfg = nvila_8b()
    r = cpu_reference(cfg, seconds_budget=max(60.0, args.cpu_budget * 4), steps=args.steps, warmup=args.warmup)
    cpu, v = r["cpu_baseline"], r["tok_s"]
    line = {
        "impl": "reference",
        "metric": "NVILA-8B decode tokens/sec (1 img 448^2, bs=1, 128 new tokens); TTFT reported as ttft_ms",
        "value": round(v, 4), "unit": "tok/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * r["step_s"], 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "ttft_ms": round(r["ttft_s"] * 1e3, 1),
        "config": {"workload": "NVILA-8B, 1x448^2 image, prefill S=279 + greedy decode, bs=1 (BASELINE.json "
                               "configs[1]); each step = %d decode tokens of the 128 (bounded CPU sample), TTFT "
                               "measured once at full size; see cpu_baseline.sample" % r["tokens_per_step"]},
        "cpu_baseline": cpu,
        "e2e": {"value": round(v, 4), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference CLI cannot run on CPU unmodified (flash-attn-only SigLIP, .cuda(), fp16; "
                "SURVEY §0.5) and llava.model does not import here; this arm is the oracle port of its modules",
    }
    print(json.dumps(line))


def run_reference_gpu(args):
    """Informational arm: the library path the reference runs (HF transformers SigLIP + Qwen2, torch
    sdpa attention, cuBLAS GEMMs, eager launches) on the same B200 for the same request.  The
    reference's own vendored SigLIP lives under /root/reference (absent on the GPU box); transformers'
    SiglipVisionModel is the same architecture.  Random-init weights on the device."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    try:
        import torch
        from transformers import Qwen2Config, Qwen2ForCausalLM, SiglipVisionConfig, SiglipVisionModel

        from oracle import vila_oracle as O
        from vila_b200.model import nvila_8b
        cfg = nvila_8b()
        lc, vc = cfg.llm_cfg, cfg.vision_tower_cfg
        torch.cuda.set_device(0)
        dev = torch.device("cuda")
        attn = "sdpa"
        with torch.device(dev):
            hf_l = Qwen2Config(hidden_size=lc.hidden_size, intermediate_size=lc.intermediate_size,
                               num_hidden_layers=lc.num_hidden_layers, num_attention_heads=lc.num_attention_heads,
                               num_key_value_heads=lc.num_key_value_heads, vocab_size=lc.vocab_size,
                               rms_norm_eps=lc.rms_norm_eps, rope_theta=lc.rope_theta,
                               max_position_embeddings=32768, tie_word_embeddings=False)
            hf_l._attn_implementation = attn
            llm = Qwen2ForCausalLM(hf_l).to(torch.bfloat16).eval()
            hf_v = SiglipVisionConfig(hidden_size=vc.hidden_size, intermediate_size=vc.intermediate_size,
                                      num_hidden_layers=vc.num_hidden_layers, num_attention_heads=vc.num_attention_heads,
                                      image_size=vc.image_size, patch_size=vc.patch_size)
            hf_v._attn_implementation = attn
            vit = SiglipVisionModel(hf_v).to(torch.bfloat16).eval()
            mm = 4 * vc.hidden_size
            proj = {"layers.1.weight": torch.ones(mm), "layers.1.bias": torch.zeros(mm),
                    "layers.2.weight": torch.randn(lc.hidden_size, mm) * 0.01, "layers.2.bias": torch.zeros(lc.hidden_size),
                    "layers.4.weight": torch.randn(lc.hidden_size, lc.hidden_size) * 0.01,
                    "layers.4.bias": torch.zeros(lc.hidden_size)}
            proj = {k: v.to(torch.bfloat16) for k, v in proj.items()}
        pixels_h, ids_h = make_request(cfg, seed=1)
        pixels = pixels_h.cuda()[None]
        text_ids = torch.tensor([i for i in ids_h[0].tolist() if i != cfg.image_token_id], device=dev)
        nl = torch.tensor(list(cfg.newline_token_ids), device=dev)
        ev = lambda: torch.cuda.Event(enable_timing=True)

        @torch.inference_mode()
        def request(n_new):
            a, b = ev(), ev()
            a.record()
            hs = vit(pixel_values=pixels, output_hidden_states=True).hidden_states[-2]
            tok = O.projector(hs, proj, "mlp_downsample")[0]
            table = llm.get_input_embeddings()
            emb = torch.cat([table(text_ids[:14]), tok, table(nl), table(text_ids[14:])], 0)[None]
            out = llm.generate(inputs_embeds=emb, attention_mask=torch.ones(emb.shape[:2], device=dev, dtype=torch.long),
                               max_new_tokens=n_new, min_new_tokens=n_new, do_sample=False, pad_token_id=0)
            out.cpu()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b), emb.shape[1]

        for _ in range(max(1, min(args.warmup, 3))):
            request(1); request(NEW_TOKENS)
        t1 = tn = 0.0
        reps = max(1, min(args.steps, 5))
        with ClockSampler(0) as clocks:
            for _ in range(reps):
                a, S = request(1)
                b, _ = request(NEW_TOKENS)
                t1 += a / reps
                tn += b / reps
        v = (NEW_TOKENS - 1) / ((tn - t1) / 1e3)
        line = {"impl": "reference_gpu",
                "metric": "NVILA-8B decode tokens/sec (1 img 448^2, bs=1, 128 new tokens); TTFT reported as ttft_ms",
                "value": round(v, 2), "unit": "tok/s", "n_gpus": 1, "steps": reps, "warmup": args.warmup,
                "ms_per_step": round(tn, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic", "ttft_ms": round(t1, 2),
                "config": {"workload": "NVILA-8B bf16, 1x448^2 image, prefill S=%d + %d greedy tokens, bs=1; HF transformers "
                                       "%s SiglipVisionModel + Qwen2ForCausalLM.generate(inputs_embeds=...), attn=%s, eager"
                                       % (S, NEW_TOKENS, __import__("transformers").__version__, attn)},
                "e2e": {"value": round(v, 2), "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": NEW_TOKENS * 8},
                "clocks": clocks.summary(),
                "note": "library baseline (cuBLAS / sdpa / ATen through HF eager), not the product"}
    except Exception as e:
        line = {"impl": "reference_gpu", "unavailable": "%s: %s" % (type(e).__name__, str(e)[:300])}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# --workload hybrid_lm: the Moronex hybrid language model next to Qwen2 (the closest model of the
# package) at equal width / depth / heads / vocabulary, random weights, bf16
# ------------------------------------------------------------------------------------------------
HYBRID_SIZES = {
    "w2048": dict(width=2048, vocab=32768, heads=16, kv_rank=512, q_rank=768, dense_ff=5632, experts=32, top=4,
                  expert_ff=704),
    "w4096": dict(width=4096, vocab=32768, heads=32, kv_rank=512, q_rank=1536, dense_ff=11008, experts=64, top=6,
                  expert_ff=1408),
}


def hybrid_lm_config(z):
    lat = dict(heads=z["heads"], dim=128, vdim=128, kv_rank=z["kv_rank"], q_rank=z["q_rank"], scale=128 ** -0.5)
    rec = dict(heads=z["heads"], dim=128, vdim=128)
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]}}
    layers = [{"type": "latent_attention", "mixer": dict(lat), "mlp": {"kind": "dense", "ff": z["dense_ff"]}},
              {"type": "hgrn2", "mixer": dict(rec), "mlp": moe}, {"type": "hgrn2", "mixer": dict(rec), "mlp": moe},
              {"type": "latent_attention", "mixer": dict(lat, kv_from=0), "mlp": moe}]
    return {"architecture": "Moronex", "layers": layers, "norm": {"eps": 1e-5}, "vocab": z["vocab"], "width": z["width"]}


def hybrid_lm_block(args, peaks):
    import torch

    from vila_b200 import ops
    from vila_b200.model import MoronexConfig, MoronexForCausalLM, Qwen2Config, Qwen2ForCausalLM
    from vila_b200.serving import BatchedDecoder, TokenEngine
    dev = torch.device("cuda:0")
    if os.environ.get("VILA_BENCH_WORKSPACE", "0") == "1":
        ops.ensure_workspace(dev)     # enables the stream-K / split-K schedules of vila_linear
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(fn, reps=args.steps, warm=max(3, args.warmup), setup=None):
        ts = []
        for i in range(warm + reps):
            if setup is not None:
                setup()
            flush.fill_(i & 255)     # evict L2 (126 MB) between iterations
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= warm:
                ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]

    S, B, CTX, NEW = 2048, 8, 1024, 32
    tf, gbs = peaks["bf16_tflops"], peaks["hbm_gbs"]
    out = {}
    t00 = time.time()

    def log(msg):
        print("[hybrid_lm %6.1fs] %s" % (time.time() - t00, msg), file=sys.stderr, flush=True)

    for name, z in HYBRID_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        log("size %s: weights" % name)
        cfgd = hybrid_lm_config(z)
        W, H, R = z["width"], z["heads"], z["kv_rank"]
        lm = MoronexForCausalLM(MoronexConfig.from_dict(cfgd), dev, torch.bfloat16).init_random(0, on_device=True)
        g = torch.Generator().manual_seed(0)
        prompt = torch.randint(0, z["vocab"], (S,), generator=g).tolist()
        # ---- end to end through the engine -----------------------------------------------------------
        log('engine prefill')
        eng = TokenEngine(lm, max_tokens=B * (CTX + 4 * NEW + 64), slots=B)
        t_pre = timed(lambda: eng.step([("p", prompt, [S - 1])]), setup=lambda: eng.release("p"))
        eng.release("p")
        log('engine decode')
        for b in range(B):
            eng.step([(b, prompt[:CTX], [])])
        step_in = [[(b, [int(prompt[(k * 7 + b) % S])], [0]) for b in range(B)] for k in range(NEW)]

        def decode_run():
            for k in range(NEW):
                eng.step(step_in[k])
        t_dec = timed(decode_run, reps=3, warm=1)     # contexts grow CTX .. CTX + 4 * NEW: fits the reserve
        for b in range(B):
            eng.release(b)
        # ---- Qwen2 at equal width / depth / heads / vocabulary ---------------------------------------
        log('qwen2')
        qc = Qwen2Config(hidden_size=W, intermediate_size=z["dense_ff"], num_hidden_layers=4, num_attention_heads=H,
                         num_key_value_heads=4, vocab_size=z["vocab"])
        qw = Qwen2ForCausalLM(qc, dev)
        for prm in qw.parameters():
            prm.data.normal_(0, 0.02)
        for lyr in qw.model.layers:
            lyr._qkv_w.normal_(0, 0.02); lyr._qkv_b.zero_(); lyr._gu_w.normal_(0, 0.02)
        emb = qw.model.embed_tokens(torch.tensor(prompt, device=dev))

        def q_prefill():
            cache = qw.new_cache(S)
            hid = qw.prefill_hidden(emb, cache)
            return qw.logits_from_hidden(hid[-1:])
        tq_pre = timed(q_prefill)
        bd = BatchedDecoder(qw, slots=B, max_tokens_per_slot=CTX + 4 * NEW + 64, max_new=4 * NEW + 8)
        bd.capture()
        for b in range(B):
            bd.admit(b, emb[:CTX])
        tq_dec = timed(lambda: bd.run(NEW), reps=3, warm=1)
        # ---- kernel against the like kernel, at this size ----------------------------------------------
        log('kernel ledger')
        bf = torch.bfloat16
        led = {}
        L0 = lm.layers[0]
        page = eng.cache.page
        pool = eng.cache.latent[0]
        pt = torch.arange(eng.cache.n_pages, dtype=torch.int32, device=dev).view(1, -1).repeat(B, 1).contiguous()
        qa = torch.randn(S, H * R, device=dev)
        gate = torch.randn(S, H, device=dev).to(bf)
        tiles = torch.tensor([(o, 16, o, 0) for o in range(0, S, 16)], dtype=torch.int32, device=dev)
        t = timed(lambda: ops.latent_attention(qa, pool, pt, tiles, heads=H, page=page, scale=0.088, sink=L0.sink, gate=gate))
        fl = H * (S * (S + 1) / 2) * 4 * R
        led["latent_attention prefill, folded over the latent (CUDA cores, fp32 scores and weights)"] = {"ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}
        kvb = torch.randn(S, H * 256, device=dev).to(bf)
        qb = torch.randn(S, H * 128, device=dev).to(bf)
        kvt = torch.tensor([(o, 16, o, 0) for o in range(0, S, 16)], dtype=torch.int32, device=dev)
        t = timed(lambda: ops.sink_attention(qb, kvb[:, :H * 128], kvb[:, H * 128:], kvt, heads=H, scale=0.088, sink=L0.sink, gate=gate))
        fl = H * (S * (S + 1) / 2) * 4 * 128
        led["sink_attention prefill, un-folded keys / values (CUDA cores, fp32 scores and weights)"] = {"ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}
        q3 = torch.randn(S, H + 8, 128, device=dev).to(bf)
        cache = qw.new_cache(S)
        t = timed(lambda: ops.fmha(q3[:, :H], cache.k(0), cache.v(0), B=1, Sq=S, Sk=S, causal=True, scale=0.088, page_table=cache.page_table))
        fl = H * (S * (S + 1) / 2) * 4 * 128
        led["qwen2 fmha prefill (tcgen05)"] = {"ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}
        dt_ = torch.tensor([(b, 1, CTX - 1, b) for b in range(B)], dtype=torch.int32, device=dev)
        pt2 = (torch.arange(B, device=dev, dtype=torch.int32)[:, None] * (CTX // page) + torch.arange(eng.cache.n_pages, device=dev, dtype=torch.int32)[None]) % eng.cache.n_pages
        t = timed(lambda: ops.latent_attention(qa[:B], pool, pt2.contiguous(), dt_, heads=H, page=page, scale=0.088, sink=L0.sink, gate=gate[:B], decode=True, nsplit=eng.cache.decode_splits))
        by = B * CTX * R * 2
        led["latent_attention decode (8 x 1024 tokens)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs,
                                                            "note": "unique latent bytes; each of the H head CTAs re-reads them through L2"}
        t = timed(lambda: bd._step(), reps=3, warm=1)
        led["qwen2 batched decode step, all kernels of 4 layers (for scale)"] = {"ms": t}
        L1 = lm.layers[1]
        hd = H * 128
        proj = torch.randn(S, L1.in_w.shape[0], device=dev).to(bf)
        state = torch.zeros(B, H, 128, 128, device=dev)
        sq = torch.tensor([[0, S, 0, 0]], dtype=torch.int32, device=dev)
        kw = dict(heads=H, dim=128, vdim=128, q_off=0, f_off=hd, v_off=2 * hd, f_bias=L1.f_bias, lower=L1.lower)
        t = timed(lambda: ops.hgrn2_scan(proj, state, sq, **kw))
        by = S * 3 * hd * 2 + S * hd * 4
        led["hgrn2_scan prefill (2048 rows, sequential in time)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs,
                                                                      "fp32_tflops": 4 * S * hd * 128 / t / 1e9}
        sq8 = torch.tensor([[b, 1, 5, b] for b in range(B)], dtype=torch.int32, device=dev)
        t = timed(lambda: ops.hgrn2_scan(proj[:B], state, sq8, **kw))
        by = B * H * 128 * 128 * 4 * 2
        led["hgrn2_scan decode (8 sequences)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        h = torch.randn(S, W, device=dev).to(bf)
        t = timed(lambda: lm._experts(L1, h))
        fl = 2 * 2 * S * z["top"] * z["expert_ff"] * W
        led["routed experts prefill: route + group + 2 grouped CUDA-core GEMMs"] = {"ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}
        t = timed(lambda: lm._lin(lm._lin(h, L0.gu, swiglu=True), L0.down))
        fl = 2 * 3 * S * z["dense_ff"] * W
        led["dense SwiGLU feed-forward prefill (tcgen05, shared with qwen2)"] = {"ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}
        t = timed(lambda: lm._experts(L1, h[:B]))
        by = 2 * min(z["experts"], B * z["top"]) * z["expert_ff"] * W * 2
        led["routed experts decode (8 rows)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        x = torch.randn(S, W, device=dev)
        y = torch.randn(S, W, device=dev).to(bf)
        gt = torch.randn(S, W, device=dev).to(bf)
        t = timed(lambda: ops.gated_norm_residual(x, y, gate=gt, gate_bias=L0.rg1_b, w=L0.norm1b, w_offset=1.0, eps=1e-5))
        by = S * W * (8 + 2 + 2)
        led["gated_norm_residual (2048 rows)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        xb = torch.randn(S, W, device=dev).to(bf)
        t = timed(lambda: ops.rmsnorm(xb, qw.model.norm.weight, 1e-6))
        by = S * W * 4
        led["qwen2 rmsnorm (2048 rows)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        n_lm = sum(v.numel() for v in lm.weights.values())
        n_qw = sum(p_.numel() for p_ in qw.parameters())
        out[name] = {
            "moronex": {"params_m": n_lm / 1e6, "prefill_tok_s": S / t_pre * 1e3, "prefill_ms": t_pre,
                        "decode_tok_s": B * NEW / t_dec * 1e3, "decode_ms_per_step": t_dec / NEW},
            "qwen2": {"params_m": n_qw / 1e6, "prefill_tok_s": S / tq_pre * 1e3, "prefill_ms": tq_pre,
                      "decode_tok_s": B * NEW / tq_dec * 1e3, "decode_ms_per_step": tq_dec / NEW},
            "kernels": led,
        }
        del lm, qw, bd, eng
        torch.cuda.empty_cache()
    return {"workload": "hybrid_lm: 4 layers (latent attention + dense, 2 x (HGRN2 + routed experts), latent attention "
                        "reading layer 0's latent + routed experts) vs 4 Qwen2 layers of equal width / heads / vocabulary; "
                        "prefill: one %d-token prompt; decode: %d sequences x %d-token context, %d steps" % (S, B, CTX, NEW),
            "dtype": "bf16", "data": "synthetic (random weights, random ids)", "l2_policy": "256 MB buffer written between timed iterations",
            "peaks": peaks, "sizes": out}


def run_hybrid_lm(args):
    import torch
    assert torch.cuda.is_available(), "bench.py --workload hybrid_lm needs a GPU"
    import faulthandler
    # a stuck run prints where it stands and ends instead of holding the GPU
    faulthandler.dump_traceback_later(int(os.environ.get("VILA_BENCH_WATCHDOG_S", "480")), exit=True)
    peaks = read_peaks()
    with ClockSampler(0) as cs:
        res = hybrid_lm_block(args, peaks)
    res["clocks"] = cs.summary()
    from vila_b200 import _lib
    res["gpu_launches"] = _lib.LAUNCHES
    print(json.dumps(res))


# ------------------------------------------------------------------------------------------------
# --workload parallel_lm: the Lufatar parallel-sublayer language model next to Moronex (the closest
# model of the package: same engine, fp32 residual, routed experts, sink softmax) at equal width /
# depth / heads / vocabulary / experts, random weights, bf16
# ------------------------------------------------------------------------------------------------
PARALLEL_SIZES = {
    "w1024": dict(width=1024, vocab=32768, heads=8, kv_heads=2, experts=16, top=2, expert_ff=512, side=64,
                  kv_rank=512, q_rank=384),
    "w2048": dict(width=2048, vocab=32768, heads=16, kv_heads=4, experts=32, top=4, expert_ff=704, side=128,
                  kv_rank=512, q_rank=768),
    "w4096": dict(width=4096, vocab=32768, heads=32, kv_heads=8, experts=64, top=6, expert_ff=1408, side=128,
                  kv_rank=512, q_rank=1536),
}


def parallel_lm_config(z):
    mix = dict(heads=z["heads"], kv_heads=z["kv_heads"], dim=128, vdim=128, rot={"base": 10000.0, "dims": 64},
               scale=128 ** -0.5)
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"], "limit": 7.0},
           "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": 4, "keep": 2}}}
    layers = [{"type": "attention", "mixer": dict(mix), "mlp": dict(moe)} for _ in range(4)]
    return {"architecture": "Lufatar", "canon": {"taps": 4},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 7919}},
            "layers": layers, "loop": {"start": 1, "stop": 3, "times": 1}, "norm": {"eps": 1e-5, "groups": 4},
            "residual_mult": 0.5, "token_side": {"dim": z["side"]}, "vocab": z["vocab"], "width": z["width"]}


def parallel_lm_twin(z):
    """Moronex with the same width / heads / vocabulary / experts: 4 latent-attention layers with routed experts"""
    lat = dict(heads=z["heads"], dim=128, vdim=128, kv_rank=z["kv_rank"], q_rank=z["q_rank"], scale=128 ** -0.5)
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]}}
    layers = [{"type": "latent_attention", "mixer": dict(lat), "mlp": dict(moe)} for _ in range(4)]
    return {"architecture": "Moronex", "layers": layers, "norm": {"eps": 1e-5}, "vocab": z["vocab"], "width": z["width"]}


def parallel_lm_block(args, peaks):
    import torch

    from vila_b200 import ops
    from vila_b200.model import LufatarConfig, LufatarForCausalLM, MoronexConfig, MoronexForCausalLM
    from vila_b200.serving import TokenEngine
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(fn, reps=args.steps, warm=max(3, args.warmup), setup=None):
        ts = []
        for i in range(warm + reps):
            if setup is not None:
                setup()
            flush.fill_(i & 255)     # evict L2 (126 MB) between iterations
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= warm:
                ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]

    def timed_op(fn):
        """a single op of the kernel ledger: captured once, timed as a graph replay, so that the number is
        the device time of its launches and not the host time of the Python call around them"""
        fn()
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return timed(g.replay)

    S, B, CTX, NEW = 2048, 8, 1024, 32
    tf, gbs = peaks["bf16_tflops"], peaks["hbm_gbs"]
    bf = torch.bfloat16
    out = {}
    t00 = time.time()

    def log(msg):
        print("[parallel_lm %6.1fs] %s" % (time.time() - t00, msg), file=sys.stderr, flush=True)

    def engine_numbers(lm, prompt):
        eng = TokenEngine(lm, max_tokens=B * (CTX + 4 * NEW + 64), slots=B)
        t_pre = timed(lambda: eng.step([("p", prompt, [S - 1])]), setup=lambda: eng.release("p"))
        eng.release("p")
        for b in range(B):
            eng.step([(b, prompt[:CTX], [])])
        step_in = [[(b, [int(prompt[(k * 7 + b) % S])], [0]) for b in range(B)] for k in range(NEW)]

        def decode_run():
            for k in range(NEW):
                eng.step(step_in[k])
        t_dec = timed(decode_run, reps=3, warm=1)     # contexts grow CTX .. CTX + 4 * NEW: fits the reserve
        for b in range(B):
            eng.release(b)
        n = sum(v.numel() for v in lm.weights.values())
        return eng, {"params_m": n / 1e6, "prefill_tok_s": S / t_pre * 1e3, "prefill_ms": t_pre,
                     "decode_tok_s": B * NEW / t_dec * 1e3, "decode_ms_per_step": t_dec / NEW}

    for name, z in PARALLEL_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        W, H, G, R = z["width"], z["heads"], z["kv_heads"], z["kv_rank"]
        g = torch.Generator().manual_seed(0)
        prompt = torch.randint(0, z["vocab"], (S,), generator=g).tolist()
        log("size %s: lufatar" % name)
        lm = LufatarForCausalLM(LufatarConfig.from_dict(parallel_lm_config(z)), dev, bf).init_random(0, on_device=True)
        eng, res_new = engine_numbers(lm, prompt)
        log("size %s: moronex" % name)
        tw = MoronexForCausalLM(MoronexConfig.from_dict(parallel_lm_twin(z)), dev, bf).init_random(0, on_device=True)
        eng2, res_old = engine_numbers(tw, prompt)
        # ---- kernel beside the like kernel ---------------------------------------------------------------
        log("kernel ledger")
        led = {}
        L0, M0 = lm.layers[0], tw.layers[0]
        page = eng.cache.page
        npg = eng.cache.n_pages
        pool = eng.cache.latent[0]
        pt = torch.arange(npg, dtype=torch.int32, device=dev).view(1, -1).repeat(B, 1).contiguous()
        tiles = torch.tensor([(o, 16, o, 0) for o in range(0, S, 16)], dtype=torch.int32, device=dev)
        q = torch.randn(S, H * 128, device=dev)
        akw = dict(heads=H, kv_heads=G, dim=128, vdim=128, page=page, scale=0.088, talk=L0.talk, sink=L0.sink)
        t = timed_op(lambda: ops.paged_attention(q, pool, pt, tiles, max_rows=16, **akw))
        fl = H * (S * (S + 1) / 2) * 4 * 128
        led["paged_attention prefill (head mixing, fp32 scores and weights, CUDA cores)"] = {
            "ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}
        kvb = torch.randn(S, H * 256, device=dev).to(bf)
        qb = torch.randn(S, H * 128, device=dev).to(bf)
        gate = torch.randn(S, H, device=dev).to(bf)
        t = timed_op(lambda: ops.sink_attention(qb, kvb[:, :H * 128], kvb[:, H * 128:], tiles, heads=H, scale=0.088,
                                             sink=M0.sink, gate=gate))
        led["moronex sink_attention prefill (un-folded, fp32 scores and weights, CUDA cores)"] = {
            "ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}
        dt_ = torch.tensor([(b, 1, CTX - 1, b) for b in range(B)], dtype=torch.int32, device=dev)
        pt2 = ((torch.arange(B, device=dev, dtype=torch.int32)[:, None] * (CTX // page) +
                torch.arange(npg, device=dev, dtype=torch.int32)[None]) % npg).contiguous()
        t = timed_op(lambda: ops.paged_attention(q[:B], pool, pt2, dt_, max_rows=1, nsplit=eng.cache.decode_splits, **akw))
        by = B * CTX * G * 256 * 2
        led["paged_attention decode (8 x 1024 tokens)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        qa = torch.randn(B, H * R, device=dev)
        pool2 = eng2.cache.latent[0]
        t = timed_op(lambda: ops.latent_attention(qa, pool2, pt2, dt_, heads=H, page=page, scale=0.088, sink=M0.sink,
                                               gate=gate[:B], decode=True, nsplit=eng2.cache.decode_splits))
        by2 = B * CTX * R * 2
        led["moronex latent_attention decode (8 x 1024 tokens)"] = {"ms": t, "gbs": by2 / t / 1e6, "of_hbm": by2 / t / 1e6 / gbs}
        h = torch.randn(S, W, device=dev).to(bf)
        fl_new = 2 * 3 * S * z["top"] * z["expert_ff"] * W
        fl_old = 2 * 2 * S * z["top"] * z["expert_ff"] * W
        t = timed_op(lambda: lm._experts(L0, h))
        led["routed experts prefill: sigmoid group router + group + 2 grouped GEMMs (gate|up, down)"] = {
            "ms": t, "tflops": fl_new / t / 1e9, "of_bf16_peak": fl_new / t / 1e9 / tf}
        t = timed_op(lambda: tw._experts(M0, h))
        led["moronex routed experts prefill: softmax router + group + 2 grouped GEMMs (up, down)"] = {
            "ms": t, "tflops": fl_old / t / 1e9, "of_bf16_peak": fl_old / t / 1e9 / tf}
        t = timed_op(lambda: lm._experts(L0, h[:B]))
        by = 3 * min(z["experts"], B * z["top"]) * z["expert_ff"] * W * 2
        led["routed experts decode (8 rows)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        t = timed_op(lambda: tw._experts(M0, h[:B]))
        by = 2 * min(z["experts"], B * z["top"]) * z["expert_ff"] * W * 2
        led["moronex routed experts decode (8 rows)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        x = torch.randn(S, W, device=dev)
        ar = torch.arange(S, dtype=torch.int32, device=dev)
        sq = torch.tensor([[0, S, 0, 0]], dtype=torch.int32, device=dev)
        rs = torch.zeros(S, dtype=torch.int32, device=dev)
        batch = type("B", (), dict(seqs=sq, row_seq=rs))
        cache1 = type("C", (), dict(state=eng.cache.state))
        t = timed_op(lambda: lm._sublayer_inputs(L0, x, batch, cache1, 0))
        by = S * W * (4 + 2)
        by = S * W * (4 + 2 * 2)
        led["sublayer inputs of mixer and experts: group norm + short convolution + state, fused (2048 rows)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        t = timed_op(lambda: ops.rmsnorm_rows(x, M0.norm1, 1e-5, w_offset=1.0, out_dtype=bf))
        by = S * W * (4 + 2)
        led["moronex rmsnorm_rows (2048 rows, one sublayer)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        qkv = torch.randn(S, (H + 2 * G) * 128, device=dev).to(bf)
        t = timed_op(lambda: ops.rope_append(qkv, ar, ar, pool, heads=H, kv_heads=G, dim=128, vdim=128, inv_freq=L0.inv_freq,
                                          unit_norm=True, eps=1e-5))
        by = S * ((H + 2 * G) * 128 * 2 + H * 128 * 4 + 2 * G * 128 * 2)
        led["rope_append: rotary + unit norm + K|V append (2048 rows)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        y = torch.randn(S, W, device=dev).to(bf)
        parts = torch.randn(S * z["top"], W, device=dev)
        t = timed_op(lambda: ops.residual_add_rows(x, y, parts, n_partials=z["top"], mult=0.5))
        by = S * W * (8 + 2 + 4 * z["top"])
        led["residual_add_rows: x += m (attention + sum of expert partials) (2048 rows)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        gt = torch.randn(S, W, device=dev).to(bf)
        t = timed_op(lambda: ops.gated_norm_residual(x, parts, n_partials=z["top"], gate=gt, gate_bias=M0.rg2_b, w=M0.norm2b, w_offset=1.0, eps=1e-5))
        by = S * W * (8 + 2 + 4 * z["top"])
        led["moronex gated_norm_residual with expert partials (2048 rows)"] = {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}
        xcb = x.to(bf)
        t = timed_op(lambda: lm._token_side(L0, x, xcb, type("B", (), dict(ids=ar))))
        led["token side input: gate GEMM + gelu x table + proj GEMM + normed update (2048 rows)"] = {"ms": t}
        out[name] = {"lufatar": res_new, "moronex": res_old, "kernels": led}
        del lm, tw, eng, eng2
        torch.cuda.empty_cache()
    return {"workload": "parallel_lm: 4 Lufatar layers (rotary GQA with head mixing + routed clamped-GLU experts in "
                        "parallel, short convolutions, token side input) vs 4 Moronex layers (latent attention + routed "
                        "experts) of equal width / heads / vocabulary / experts; prefill: one %d-token prompt; decode: %d "
                        "sequences x %d-token context, %d steps" % (S, B, CTX, NEW),
            "dtype": "bf16", "data": "synthetic (random weights, random ids)",
            "l2_policy": "256 MB buffer written between timed iterations",
            "kernel_ledger_timing": "each op captured in a CUDA graph, one replay per timed iteration", "peaks": peaks, "sizes": out}


def run_parallel_lm(args):
    import torch
    assert torch.cuda.is_available(), "bench.py --workload parallel_lm needs a GPU"
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("VILA_BENCH_WATCHDOG_S", "480")), exit=True)
    peaks = read_peaks()
    with ClockSampler(0) as cs:
        res = parallel_lm_block(args, peaks)
    res["clocks"] = cs.summary()
    from vila_b200 import _lib
    res["gpu_launches"] = _lib.LAUNCHES
    print(json.dumps(res))

# ------------------------------------------------------------------------------------------------
# --workload ssm_lm: the Nusovik state-space / chunked-attention language model next to Moronex (the
# closest model of the package: same engine, recurrent layers with an fp32 state per sequence beside
# attention with sink and output gate, dense feed-forward) at equal width / depth / vocabulary,
# random weights, bf16
# ------------------------------------------------------------------------------------------------
SSM_SIZES = {
    "w1024": dict(width=1024, vocab=32768, heads=8, kv_heads=2, chunk=512, ff=4096, kv_rank=512, q_rank=384),
    "w2048": dict(width=2048, vocab=32768, heads=16, kv_heads=4, chunk=512, ff=8192, kv_rank=512, q_rank=768),
    "w4096": dict(width=4096, vocab=32768, heads=32, kv_heads=8, chunk=512, ff=16384, kv_rank=512, q_rank=1536),
}


def ssm_lm_config(z):
    W = z["width"]
    sel = {"conv": 4, "dt_rank": W // 16, "inner": 2 * W, "state": 16}
    par = {"left": {"bias_max": 512, "dim": 128, "heads": z["heads"], "kv_heads": z["kv_heads"],
                    "mask": {"size": z["chunk"]}, "scale": 128 ** -0.5, "vdim": 128},
           "left_scale": 1.0,
           "right": {"conv": 4, "groups": 8, "heads": 2 * W // 64, "norm_groups": 8, "state": 128, "vdim": 64},
           "right_scale": 1.0}
    ff = {"ff": z["ff"], "kind": "dense"}
    layers = [{"type": "mamba1", "mixer": dict(sel), "mlp": None}, {"type": "parallel", "mixer": dict(par), "mlp": dict(ff)},
              {"type": "mamba1", "mixer": dict(sel), "mlp": None}, {"type": "parallel", "mixer": dict(par), "mlp": dict(ff)}]
    return {"architecture": "Nusovik", "embedding": {"scale": 1.0}, "layers": layers, "logit_scale": 1.0,
            "norm": {"eps": 1e-5}, "vocab": z["vocab"], "width": W}


def ssm_lm_twin(z):
    """Moronex with the same width / heads / vocabulary: recurrent (HGRN2) and latent-attention layers in the same order"""
    lat = dict(heads=z["heads"], dim=128, vdim=128, kv_rank=z["kv_rank"], q_rank=z["q_rank"], scale=128 ** -0.5)
    rec = dict(heads=z["heads"], dim=128, vdim=128)
    ff = {"kind": "dense", "ff": z["ff"] * 2 // 3 // 64 * 64}      # gated: three matrices of 2/3 the width
    layers = [{"type": "hgrn2", "mixer": dict(rec), "mlp": None}, {"type": "latent_attention", "mixer": dict(lat), "mlp": dict(ff)},
              {"type": "hgrn2", "mixer": dict(rec), "mlp": None}, {"type": "latent_attention", "mixer": dict(lat), "mlp": dict(ff)}]
    return {"architecture": "Moronex", "layers": layers, "norm": {"eps": 1e-5}, "vocab": z["vocab"], "width": z["width"]}


def ssm_lm_block(args, peaks):
    import torch

    from vila_b200 import ops
    from vila_b200.model import MoronexConfig, MoronexForCausalLM, NusovikConfig, NusovikForCausalLM
    from vila_b200.serving import TokenEngine
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(fn, reps=args.steps, warm=max(3, args.warmup), setup=None):
        ts = []
        for i in range(warm + reps):
            if setup is not None:
                setup()
            flush.fill_(i & 255)     # evict L2 (126 MB) between iterations
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= warm:
                ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]

    def timed_op(fn):
        """a single op of the kernel ledger: captured once, timed as a graph replay, so that the number is
        the device time of its launches and not the host time of the Python call around them"""
        fn()
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return timed(g.replay)

    S, B, CTX, NEW = 2048, 8, 1024, 32
    tf, gbs = peaks["bf16_tflops"], peaks["hbm_gbs"]
    bf, f32 = torch.bfloat16, torch.float32
    out = {}
    t00 = time.time()

    def log(msg):
        print("[ssm_lm %6.1fs] %s" % (time.time() - t00, msg), file=sys.stderr, flush=True)

    def engine_numbers(lm, prompt):
        eng = TokenEngine(lm, max_tokens=B * (CTX + 4 * NEW + 64), slots=B)
        t_pre = timed(lambda: eng.step([("p", prompt, [S - 1])]), setup=lambda: eng.release("p"))
        eng.release("p")
        for b in range(B):
            eng.step([(b, prompt[:CTX], [])])
        step_in = [[(b, [int(prompt[(k * 7 + b) % S])], [0]) for b in range(B)] for k in range(NEW)]

        def decode_run():
            for k in range(NEW):
                eng.step(step_in[k])
        t_dec = timed(decode_run, reps=3, warm=1)     # contexts grow CTX .. CTX + 4 * NEW: fits the reserve
        for b in range(B):
            eng.release(b)
        n = sum(v.numel() for v in lm.weights.values())
        return eng, {"params_m": n / 1e6, "prefill_tok_s": S / t_pre * 1e3, "prefill_ms": t_pre,
                     "decode_tok_s": B * NEW / t_dec * 1e3, "decode_ms_per_step": t_dec / NEW}

    def rate(t, flop=None, byts=None):
        r = {"ms": t}
        if flop is not None:
            r["tflops_fp32"] = flop / t / 1e9
        if byts is not None:
            r["gbs"], r["of_hbm"] = byts / t / 1e6, byts / t / 1e6 / gbs
        return r

    for name, z in SSM_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        W, H, G = z["width"], z["heads"], z["kv_heads"]
        g = torch.Generator().manual_seed(0)
        prompt = torch.randint(0, z["vocab"], (S,), generator=g).tolist()
        log("size %s: nusovik" % name)
        cfgd = ssm_lm_config(z)
        lm = NusovikForCausalLM(NusovikConfig.from_dict(cfgd), dev, bf).init_random(0, on_device=True)
        eng, res_new = engine_numbers(lm, prompt)
        log("size %s: moronex" % name)
        tw = MoronexForCausalLM(MoronexConfig.from_dict(ssm_lm_twin(z)), dev, bf).init_random(0, on_device=True)
        eng2, res_old = engine_numbers(tw, prompt)
        # ---- kernel beside the like kernel ---------------------------------------------------------------
        log("kernel ledger")
        led = {}
        Ls, Lp, Mr, Ma = lm.layers[0], lm.layers[1], tw.layers[0], tw.layers[1]
        sq1 = torch.tensor([[0, S, 0, 0]], dtype=torch.int32, device=dev)
        sqB = torch.tensor([(b, 1, CTX, b) for b in range(B)], dtype=torch.int32, device=dev)
        rs1 = torch.zeros(S, dtype=torch.int32, device=dev)
        # recurrences: one 2048-row prompt, and 8 decoded rows
        r = cfgd["layers"][1]["mixer"]["right"]
        Hs, P, N, Gs = r["heads"], r["vdim"], r["state"], r["groups"]
        inner, chans = Hs * P, Hs * P + 2 * Gs * N
        wide = (torch.randn(S, 2 * inner + 2 * Gs * N + Hs, device=dev) * 0.5).to(bf)
        st = eng.cache.state[(1, "ssm")]
        skw = dict(heads=Hs, vdim=P, nstate=N, groups=Gs, dt_bias=Lp.dt_bias, A_log=Lp.A_log, D=Lp.D)
        for rows, sq, tag in ((S, sq1, "prefill, one %d-row prompt" % S), (B, sqB, "decode, %d rows" % B)):
            t = timed_op(lambda: ops.ssd_scan(wide[:rows, inner:inner + chans], wide[:rows, inner + chans:inner + chans + Hs],
                                              wide[:rows, :inner], st, sq, **skw))
            nseq = sq.shape[0]
            led["ssd_scan " + tag] = rate(t, flop=6.0 * rows * Hs * P * N,
                                          byts=rows * (2 * inner + chans + Hs) * 2 + rows * inner * 4 + 2 * nseq * Hs * P * N * 4)
        m1 = cfgd["layers"][0]["mixer"]
        C1, N1 = m1["inner"], m1["state"]
        xs, dts, zs = [(torch.randn(S, C1, device=dev) * 0.5).to(bf) for _ in range(3)]
        bc = (torch.randn(S, 2 * N1, device=dev) * 0.5).to(bf)
        st1 = eng.cache.state[(0, "ssm")]
        for rows, sq, tag in ((S, sq1, "prefill, one %d-row prompt" % S), (B, sqB, "decode, %d rows" % B)):
            t = timed_op(lambda: ops.selective_scan(xs[:rows], dts[:rows], bc[:rows], zs[:rows], st1, sq, dt_bias=Ls.dt_bias,
                                                    A_log=Ls.A_log, D=Ls.D, out_dtype=bf))
            nseq = sq.shape[0]
            led["selective_scan " + tag] = rate(t, flop=6.0 * rows * C1 * N1,
                                                byts=rows * (4 * C1 + 2 * N1) * 2 + 2 * nseq * C1 * N1 * 4)
        proj = (torch.randn(S, 3 * H * 128 + W, device=dev) * 0.5).to(bf)
        st2 = eng2.cache.state[0]
        for rows, sq, tag in ((S, sq1, "prefill, one %d-row prompt" % S), (B, sqB, "decode, %d rows" % B)):
            t = timed_op(lambda: ops.hgrn2_scan(proj[:rows], st2, sq, heads=H, dim=128, vdim=128, q_off=0, f_off=H * 128,
                                                v_off=2 * H * 128, f_bias=Mr.f_bias, lower=Mr.lower))
            nseq = sq.shape[0]
            led["moronex hgrn2_scan " + tag] = rate(t, flop=6.0 * rows * H * 128 * 128,
                                                    byts=rows * 3 * H * 128 * 2 + rows * H * 128 * 4 + 2 * nseq * H * 128 * 128 * 4)
        # attention: the same paged kernel with and without this model's options, and Moronex's un-folded kernel
        page, npg = eng.cache.page, eng.cache.n_pages
        pool = eng.cache.latent[1]
        pt = torch.arange(npg, dtype=torch.int32, device=dev).view(1, -1).repeat(B, 1).contiguous()
        tiles = torch.tensor([(o, 16, o, 0) for o in range(0, S, 16)], dtype=torch.int32, device=dev)
        q = torch.randn(S, H * 128, device=dev)
        gate = torch.randn(S, H, device=dev).to(bf)
        akw = dict(heads=H, kv_heads=G, dim=128, vdim=128, page=page, scale=0.088, sink=Lp.sink)
        okw = dict(dist_bias=Lp.dist_bias, chunk=z["chunk"], gate=gate)
        ck = z["chunk"]
        pairs_chunk = sum((p % ck) + 1 for p in range(S))
        t = timed_op(lambda: ops.paged_attention(q, pool, pt, tiles, max_rows=16, **akw, **okw))
        led["paged_attention prefill, chunk %d + distance bias + gate" % ck] = rate(t, flop=H * pairs_chunk * 4.0 * 128)
        t = timed_op(lambda: ops.paged_attention(q, pool, pt, tiles, max_rows=16, **akw))
        led["paged_attention prefill, plain causal, heads not mixed"] = rate(
            t, flop=H * (S * (S + 1) / 2) * 4.0 * 128)
        kvb = torch.randn(S, H * 256, device=dev).to(bf)
        qb = torch.randn(S, H * 128, device=dev).to(bf)
        t = timed_op(lambda: ops.sink_attention(qb, kvb[:, :H * 128], kvb[:, H * 128:], tiles, heads=H, scale=0.088,
                                                sink=Ma.sink, gate=gate))
        led["moronex sink_attention prefill (un-folded, plain causal)"] = rate(t, flop=H * (S * (S + 1) / 2) * 4.0 * 128)
        dt_ = torch.tensor([(b, 1, CTX - 1, b) for b in range(B)], dtype=torch.int32, device=dev)
        pt2 = ((torch.arange(B, device=dev, dtype=torch.int32)[:, None] * (CTX // page) +
                torch.arange(npg, device=dev, dtype=torch.int32)[None]) % npg).contiguous()
        okd = dict(okw, gate=gate[:B])
        t = timed_op(lambda: ops.paged_attention(q[:B], pool, pt2, dt_, max_rows=1, nsplit=eng.cache.decode_splits, **akw, **okd))
        led["paged_attention decode, chunk %d (8 rows at position %d: %d keys each)" % (ck, CTX - 1, (CTX - 1) % ck + 1)] = rate(
            t, byts=B * ((CTX - 1) % ck + 1) * G * 256 * 2)
        t = timed_op(lambda: ops.paged_attention(q[:B], pool, pt2, dt_, max_rows=1, nsplit=eng.cache.decode_splits, **akw))
        led["paged_attention decode, plain causal (8 x 1024 keys)"] = rate(t, byts=B * CTX * G * 256 * 2)
        # row kernels
        x = torch.randn(S, W, device=dev)
        y1, y2 = torch.randn(S, W, device=dev).to(bf), torch.randn(S, W, device=dev).to(bf)
        t = timed_op(lambda: ops.branch_norm_residual(x, y1, Lp.norm1, 1e-5, a_scale=1.0, b=y2, b_scale=1.0, copy_dtype=bf))
        led["branch_norm_residual, two branches + bf16 copy (2048 rows)"] = rate(t, byts=S * W * (8 + 2 + 2 + 2))
        gt = torch.randn(S, W, device=dev).to(bf)
        t = timed_op(lambda: ops.gated_norm_residual(x, y1, gate=gt, gate_bias=Ma.rg1_b, w=Ma.norm1b, w_offset=1.0, eps=1e-5))
        led["moronex gated_norm_residual (2048 rows)"] = rate(t, byts=S * W * (8 + 2 + 2))
        cst = eng.cache.state[(1, "conv")]
        t = timed_op(lambda: ops.causal_conv_rows(wide[:, inner:inner + chans], Lp.ssd_conv, Lp.ssd_conv_b, cst, sq1, rs1,
                                                  act=ops.CONV_SILU, out_dtype=bf))
        led["causal_conv_rows + tail update, %d channels, 4 taps, SiLU (2048 rows)" % chans] = rate(t, byts=S * chans * 4)
        h32 = torch.randn(S, W, device=dev)
        cw = torch.randn(W, 4, device=dev)
        cst2 = torch.zeros(B, 3, W, device=dev)
        t = timed_op(lambda: ops.short_conv_rows(h32, cw, cst2, sq1, rs1, out_dtype=bf))
        led["short_conv_rows + state, %d channels, 4 taps (the parallel-sublayer model's, fp32 in, 2048 rows)" % W] = rate(
            t, byts=S * W * 6)
        ar = torch.arange(S, dtype=torch.int32, device=dev)
        t = timed_op(lambda: ops.embed_sincos_rows(lm.embed, ar, ar, lm.inv_freq, 1.0, copy_dtype=bf))
        led["embed_sincos_rows (2048 rows)"] = rate(t, byts=S * W * (2 + 4 + 2))
        t = timed_op(lambda: ops.embed_rows(tw.embed, ar))
        led["moronex embed_rows (2048 rows)"] = rate(t, byts=S * W * (2 + 4))
        qk = (torch.randn(S, (H + G) * 128 + 8, device=dev)).to(bf)
        t = timed_op(lambda: ops.rope_append(qk, ar, ar, pool, heads=H, kv_heads=G, dim=128, vdim=128, inv_freq=None,
                                             unit_norm=True, eps=1e-5, q_norm_w=Lp.q_norm, k_norm_w=Lp.k_norm, v_from_k=True))
        led["head norm + k | v append (2048 rows)"] = rate(t, byts=S * ((H + G) * 128 * 2 + H * 128 * 4 + 2 * G * 128 * 2))
        # feed-forward: the tensor-core GEMM with the squared-ReLU epilogue beside the gated one
        hb = torch.randn(S, W, device=dev).to(bf)
        t = timed_op(lambda: ops.linear_any(hb, Lp.up, act=ops.ACT_RELU2))
        fl = 2.0 * S * W * z["ff"]
        led["feed-forward up-projection, squared-ReLU epilogue (tcgen05)"] = {"ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}
        t = timed_op(lambda: ops.linear_any(hb, Ma.gu, swiglu=True))
        fl = 2.0 * S * W * Ma.gu.shape[0]
        led["moronex feed-forward gate|up projection, SwiGLU epilogue (tcgen05)"] = {"ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}
        out[name] = {"nusovik": res_new, "moronex": res_old, "kernels": led}
        del lm, tw, eng, eng2
        torch.cuda.empty_cache()
    return {"workload": "ssm_lm: 4 Nusovik layers (selective scan; chunked sink attention + scalar-decay scan in parallel + "
                        "squared-ReLU feed-forward; twice) vs 4 Moronex layers (HGRN2; latent attention + gated feed-forward; "
                        "twice) of equal width / heads / vocabulary; prefill: one %d-token prompt; decode: %d sequences x "
                        "%d-token context, %d steps" % (S, B, CTX, NEW),
            "dtype": "bf16", "data": "synthetic (random weights, random ids)",
            "l2_policy": "256 MB buffer written between timed iterations",
            "kernel_ledger_timing": "each op captured in a CUDA graph, one replay per timed iteration", "peaks": peaks, "sizes": out}


def run_ssm_lm(args):
    import torch
    assert torch.cuda.is_available(), "bench.py --workload ssm_lm needs a GPU"
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("VILA_BENCH_WATCHDOG_S", "480")), exit=True)
    peaks = read_peaks()
    with ClockSampler(0) as cs:
        res = ssm_lm_block(args, peaks)
    res["clocks"] = cs.summary()
    from vila_b200 import _lib
    res["gpu_launches"] = _lib.LAUNCHES
    print(json.dumps(res))



# ------------------------------------------------------------------------------------------------
# --workload window_lm: the Ludazen windowed-attention language model next to Lufatar (the closest model of
# the package: same engine, rotary grouped-query attention over a paged k | v pool with head mixing, sigmoid
# router, gated experts) at equal width / heads / vocabulary / experts, random weights, bf16.  The latent
# layers are set beside Moronex's latent-attention kernel in the ledger.
# ------------------------------------------------------------------------------------------------
WINDOW_LM = dict(window=1024, keep_first=64, kv_rank=384, rot_dim=64)


def window_lm_config(z):
    H, G, W = z["heads"], z["kv_heads"], z["width"]
    att = dict(heads=H, kv_heads=G, dim=128, vdim=128, scale=128 ** -0.5,
               rot={"base": 10000.0, "dims": 128, "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}},
               mask={"size": WINDOW_LM["window"], "keep_first": WINDOW_LM["keep_first"]})
    lat = dict(heads=H, dim=128, rot_dim=WINDOW_LM["rot_dim"], vdim=128, kv_rank=WINDOW_LM["kv_rank"], scale=192 ** -0.5,
               rot={"base": 10000.0, "dims": WINDOW_LM["rot_dim"]}, mask={"size": WINDOW_LM["window"]})
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["expert_ff"]}}
    dense = {"kind": "dense", "ff": 4 * W}
    layers = [{"type": "attention", "mixer": dict(att), "mlp": dict(dense)}, {"type": "attention", "mixer": dict(att), "mlp": dict(moe)},
              {"type": "latent_attention", "mixer": dict(lat), "mlp": dict(dense)},
              {"type": "latent_attention", "mixer": dict(lat, kv_from=2), "mlp": dict(moe)}]
    return {"architecture": "Ludazen", "layers": layers, "norm": {"eps": 1e-5}, "vocab": z["vocab"], "width": W}


def window_lm_block(args, peaks):
    import torch

    from vila_b200 import ops
    from vila_b200.model import LudazenConfig, LudazenForCausalLM, LufatarConfig, LufatarForCausalLM
    from vila_b200.serving import TokenEngine
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(fn, reps=args.steps, warm=max(3, args.warmup), setup=None):
        ts = []
        for i in range(warm + reps):
            if setup is not None:
                setup()
            flush.fill_(i & 255)     # evict L2 (126 MB) between iterations
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if i >= warm:
                ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]

    def timed_op(fn):
        """a single op of the kernel ledger: captured once, timed as a graph replay, so that the number is
        the device time of its launches and not the host time of the Python call around them"""
        fn()
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return timed(g.replay)

    S, B, CTX, NEW = 2048, 8, 1024, 32
    tf, gbs = peaks["bf16_tflops"], peaks["hbm_gbs"]
    bf = torch.bfloat16
    out = {}
    t00 = time.time()

    def log(msg):
        print("[window_lm %6.1fs] %s" % (time.time() - t00, msg), file=sys.stderr, flush=True)

    def engine_numbers(lm, prompt):
        eng = TokenEngine(lm, max_tokens=B * (CTX + 4 * NEW + 64), slots=B)
        t_pre = timed(lambda: eng.step([("p", prompt, [S - 1])]), setup=lambda: eng.release("p"))
        eng.release("p")
        for b in range(B):
            eng.step([(b, prompt[:CTX], [])])
        step_in = [[(b, [int(prompt[(k * 7 + b) % S])], [0]) for b in range(B)] for k in range(NEW)]

        def decode_run():
            for k in range(NEW):
                eng.step(step_in[k])
        t_dec = timed(decode_run, reps=3, warm=1)     # contexts grow CTX .. CTX + 4 * NEW: fits the reserve
        for b in range(B):
            eng.release(b)
        n = sum(v.numel() for v in lm.weights.values())
        return eng, {"params_m": n / 1e6, "prefill_tok_s": S / t_pre * 1e3, "prefill_ms": t_pre,
                     "decode_tok_s": B * NEW / t_dec * 1e3, "decode_ms_per_step": t_dec / NEW}

    def flops(t, fl):
        return {"ms": t, "tflops": fl / t / 1e9, "of_bf16_peak": fl / t / 1e9 / tf}

    def bytes_(t, by):
        return {"ms": t, "gbs": by / t / 1e6, "of_hbm": by / t / 1e6 / gbs}

    win, keep, R, Dr = WINDOW_LM["window"], WINDOW_LM["keep_first"], WINDOW_LM["kv_rank"], WINDOW_LM["rot_dim"]
    RW = R + Dr
    for name, z in PARALLEL_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        W, H, G = z["width"], z["heads"], z["kv_heads"]
        g = torch.Generator().manual_seed(0)
        prompt = torch.randint(0, z["vocab"], (S,), generator=g).tolist()
        log("size %s: ludazen" % name)
        lm = LudazenForCausalLM(LudazenConfig.from_dict(window_lm_config(z)), dev, bf).init_random(0, on_device=True)
        eng, res_new = engine_numbers(lm, prompt)
        log("size %s: lufatar" % name)
        tw = LufatarForCausalLM(LufatarConfig.from_dict(parallel_lm_config(z)), dev, bf).init_random(0, on_device=True)
        eng2, res_old = engine_numbers(tw, prompt)
        # ---- kernel beside the like kernel ---------------------------------------------------------------
        log("kernel ledger")
        led = {}
        La, Lm, Ll, T0 = lm.layers[0], lm.layers[1], lm.layers[2], tw.layers[0]
        page, npg = eng.cache.page, eng.cache.n_pages
        pool = eng.cache.latent[0]
        pt = torch.arange(npg, dtype=torch.int32, device=dev).view(1, -1).repeat(B, 1).contiguous()
        tiles = torch.tensor([(o, 16, o, 0) for o in range(0, S, 16)], dtype=torch.int32, device=dev)
        q = torch.randn(S, H * 128, device=dev)
        # (query, key) pairs a mask lets through
        pairs_win = sum(min(p + 1, win) + max(0, min(keep, p + 1 - win)) for p in range(S))
        pairs_all = S * (S + 1) // 2
        wkw = dict(heads=H, kv_heads=G, dim=128, vdim=128, page=page, scale=0.088, talk=La.talk, talk_after=True,
                   head_scale=La.temp, window=win, keep_first=keep)
        t = timed_op(lambda: ops.paged_attention(q, pool, pt, tiles, max_rows=16, **wkw))
        led["paged_attention prefill: window %d + %d kept, weights mixed after the softmax (two passes over the keys)" % (win, keep)] = \
            flops(t, H * pairs_win * 4.0 * 128)
        okw = dict(heads=H, kv_heads=G, dim=128, vdim=128, page=page, scale=0.088, talk=T0.talk, sink=T0.sink)
        t = timed_op(lambda: ops.paged_attention(q, pool, pt, tiles, max_rows=16, **okw))
        led["lufatar paged_attention prefill: plain causal, scores mixed before the softmax"] = flops(t, H * pairs_all * 4.0 * 128)
        t = timed_op(lambda: ops.paged_attention(q, pool, pt, tiles, max_rows=16, window=win, keep_first=keep, **okw))
        led["paged_attention prefill: the same window, scores mixed before the softmax (one pass)"] = flops(t, H * pairs_win * 4.0 * 128)
        dt_ = torch.tensor([(b, 1, CTX - 1, b) for b in range(B)], dtype=torch.int32, device=dev)
        pt2 = ((torch.arange(B, device=dev, dtype=torch.int32)[:, None] * (CTX // page) +
                torch.arange(npg, device=dev, dtype=torch.int32)[None]) % npg).contiguous()
        ns = lm._splits(eng.cache, win + keep)
        t = timed_op(lambda: ops.paged_attention(q[:B], pool, pt2, dt_, max_rows=1, nsplit=ns, **wkw))
        led["paged_attention decode: window, weights mixed after the softmax (8 x 1024 keys, %d CTAs per row)" % ns] = \
            bytes_(t, B * CTX * G * 256 * 2)
        t = timed_op(lambda: ops.paged_attention(q[:B], pool, pt2, dt_, max_rows=1, nsplit=eng2.cache.decode_splits, **okw))
        led["lufatar paged_attention decode (8 x 1024 keys, %d CTAs per row)" % eng2.cache.decode_splits] = bytes_(t, B * CTX * G * 256 * 2)
        # latent attention over (latent | rotated key part) rows, beside the same kernel without window and rotary part
        lpool = eng.cache.latent[2]
        qa = torch.randn(S, H * RW, device=dev)
        t = timed_op(lambda: ops.latent_attention(qa, lpool, pt, tiles, heads=H, page=page, scale=0.072, window=win))
        led["latent_attention prefill: rows of %d + %d, window %d" % (R, Dr, win)] = flops(t, H * sum(min(p + 1, win) for p in range(S)) * 4.0 * RW)
        t = timed_op(lambda: ops.latent_attention(qa, lpool, pt, tiles, heads=H, page=page, scale=0.072))
        led["moronex-style latent_attention prefill: the same rows, plain causal"] = flops(t, H * pairs_all * 4.0 * RW)
        ns = lm._splits(eng.cache, win)
        t = timed_op(lambda: ops.latent_attention(qa[:B], lpool, pt2, dt_, heads=H, page=page, scale=0.072, window=win, decode=True, nsplit=ns))
        led["latent_attention decode: window (8 x 1024 keys, %d CTAs per row)" % ns] = bytes_(t, B * CTX * RW * 2)
        t = timed_op(lambda: ops.latent_attention(qa[:B], lpool, pt2, dt_, heads=H, page=page, scale=0.072, decode=True,
                                                  nsplit=eng.cache.decode_splits))
        led["moronex-style latent_attention decode: plain causal (8 x 1024 keys, %d CTAs per row)" % eng.cache.decode_splits] = \
            bytes_(t, B * CTX * RW * 2)
        ar = torch.arange(S, dtype=torch.int32, device=dev)
        P = torch.randn(S, H * 192 + RW, device=dev).to(bf)
        t = timed_op(lambda: ops.latent_rope_append(ar, Ll.inv_freq, rank=R, kv=P[:, H * 192:], norm_w=Ll.dkv_norm, eps=1e-5,
                                                    pool=lpool, cache_rows=ar, q=P, qa=qa, heads=H, q_head=192, q_off=128))
        led["latent_rope_append: latent norm + rotary key part -> cache row, rotary query parts (2048 rows)"] = \
            bytes_(t, S * ((RW + H * Dr) * 2 + RW * 2 + H * Dr * 4))
        qkv = torch.randn(S, (H + 2 * G) * 128, device=dev).to(bf)
        t = timed_op(lambda: ops.rope_append(qkv, ar, ar, pool, heads=H, kv_heads=G, dim=128, vdim=128, inv_freq=La.inv_freq,
                                             unit_norm=False, eps=1e-5, halves=True, mscale=La.magnitude))
        by = S * ((H + 2 * G) * 128 * 2 + H * 128 * 4 + 2 * G * 128 * 2)
        led["rope_append: rotary in halves, rescaled frequencies + k | v append (2048 rows)"] = bytes_(t, by)
        t = timed_op(lambda: ops.rope_append(qkv, ar, ar, eng2.cache.latent[0], heads=H, kv_heads=G, dim=128, vdim=128,
                                             inv_freq=T0.inv_freq, unit_norm=True, eps=1e-5))
        led["lufatar rope_append: rotary in pairs + unit norm + k | v append (2048 rows)"] = bytes_(t, by)
        # feed-forwards
        h = torch.randn(S, W, device=dev).to(bf)
        fl = 2 * 3 * S * z["top"] * z["expert_ff"] * W
        t = timed_op(lambda: lm._experts(Lm, h))
        led["routed + shared experts prefill: sigmoid router + group + 2 grouped GEMMs (weight on the input) + shared gated unit"] = \
            flops(t, fl + 2 * 3 * S * z["expert_ff"] * W)
        t = timed_op(lambda: tw._experts(T0, h))
        led["lufatar routed experts prefill: group-limited sigmoid router + group + 2 grouped GEMMs"] = flops(t, fl)
        t = timed_op(lambda: lm._experts(Lm, h[:B]))
        by = 3 * min(z["experts"], B * z["top"]) * z["expert_ff"] * W * 2
        led["routed + shared experts decode (8 rows)"] = bytes_(t, by + 3 * z["expert_ff"] * W * 2)
        t = timed_op(lambda: tw._experts(T0, h[:B]))
        led["lufatar routed experts decode (8 rows)"] = bytes_(t, by)
        t = timed_op(lambda: ops.linear_any(h, La.up, bias=La.up_b, act=ops.ACT_XIELU, act_params=La.act))
        led["dense feed-forward up-projection, bias + two-sided quadratic/exponential epilogue (tcgen05)"] = flops(t, 2.0 * S * W * 4 * W)
        t = timed_op(lambda: ops.linear_any(h, La.up, bias=La.up_b, act=ops.ACT_RELU2))
        led["the same projection with the squared-ReLU epilogue (tcgen05)"] = flops(t, 2.0 * S * W * 4 * W)
        # residual stream
        x = torch.randn(S, W, device=dev)
        y = torch.randn(S, W, device=dev).to(bf)
        parts = torch.randn(S * z["top"], W, device=dev)
        t = timed_op(lambda: ops.residual_norm_rows(x, y, La.norm1, 1e-5, part=parts, n_partials=z["top"], out_dtype=bf))
        led["residual_norm_rows: x += shared + expert partials, then the next pre-norm (2048 rows)"] = \
            bytes_(t, S * W * (8 + 2 + 4 * z["top"] + 2))
        t = timed_op(lambda: ops.residual_add_rows(x, y, parts, n_partials=z["top"], mult=0.5))
        led["lufatar residual_add_rows: x += m (attention + expert partials) (2048 rows)"] = bytes_(t, S * W * (8 + 2 + 4 * z["top"]))
        out[name] = {"ludazen": res_new, "lufatar": res_old, "kernels": led}
        del lm, tw, eng, eng2
        torch.cuda.empty_cache()
    return {"workload": "window_lm: 4 Ludazen layers (windowed rotary GQA with weight mixing + dense / routed feed-forward, "
                        "windowed latent attention with a rotary part + dense / routed feed-forward, the second latent layer "
                        "on the first one's rows) vs 4 Lufatar layers (rotary GQA with score mixing + routed experts in "
                        "parallel) of equal width / heads / vocabulary / experts; prefill: one %d-token prompt; decode: %d "
                        "sequences x %d-token context, %d steps" % (S, B, CTX, NEW),
            "dtype": "bf16", "data": "synthetic (random weights, random ids)",
            "l2_policy": "256 MB buffer written between timed iterations",
            "kernel_ledger_timing": "each op captured in a CUDA graph, one replay per timed iteration", "peaks": peaks, "sizes": out}


def run_window_lm(args):
    import torch
    assert torch.cuda.is_available(), "bench.py --workload window_lm needs a GPU"
    import faulthandler
    faulthandler.dump_traceback_later(int(os.environ.get("VILA_BENCH_WATCHDOG_S", "480")), exit=True)
    peaks = read_peaks()
    with ClockSampler(0) as cs:
        res = window_lm_block(args, peaks)
    res["clocks"] = cs.summary()
    from vila_b200 import _lib
    res["gpu_launches"] = _lib.LAUNCHES
    print(json.dumps(res))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_gpu"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-sp", action="store_true", help="skip the sp_prefill block")
    ap.add_argument("--no-video", action="store_true", help="skip the video_decode block")
    ap.add_argument("--cpu-budget", type=float, default=25.0)
    ap.add_argument("--frames", type=int, default=256, help="frames of the sp_prefill block")
    ap.add_argument("--sp-steps", type=int, default=10)
    ap.add_argument("--profile", action="store_true",
                    help="profiling aid (ncu): 1 warm-up, 8 new tokens, no extra blocks; NOT a valid bench number")
    ap.add_argument("--sizes", default="", help="hybrid_lm / parallel_lm / ssm_lm / window_lm: comma-separated subset of the workload's sizes ("
                    + ",".join(HYBRID_SIZES) + " / " + ",".join(PARALLEL_SIZES) + ")")
    ap.add_argument("--workload", default="headline", choices=["headline", "hybrid_lm", "parallel_lm", "ssm_lm", "window_lm"],
                    help="headline (default): the NVILA-8B serving step; hybrid_lm: Moronex vs Qwen2 at equal size; "
                         "parallel_lm: Lufatar vs Moronex at equal size; ssm_lm: Nusovik vs Moronex at equal size; "
                         "window_lm: Ludazen vs Lufatar at equal size")
    args = ap.parse_args()
    if args.workload == "hybrid_lm":
        return run_hybrid_lm(args)
    if args.workload == "parallel_lm":
        return run_parallel_lm(args)
    if args.workload == "ssm_lm":
        return run_ssm_lm(args)
    if args.workload == "window_lm":
        return run_window_lm(args)
    if args.profile:
        global NEW_TOKENS
        NEW_TOKENS = 8
        args.no_cpu = True
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference_gpu":
        run_reference_gpu(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
