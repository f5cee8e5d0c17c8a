"""Ludazen: a pre-norm decoder-only language model of windowed attention mixers on the ragged-batch kernels.

Residual stream x (fp32).  Layer i:  x += mixer(rms(x) * norm1),  x += ff(rms(x) * norm2)  (a layer may have
no feed-forward), rms(v) = v / sqrt(mean(v^2) + eps).  Mixers (config `layers[i].type`):

  attention          grouped-query heads; rotary positions on the first `rot.dims` columns of q and k in the
                     halves layout (column i pairs with i + dims / 2), optionally with rescaled frequencies
                     (`rot.scaling`: slow pairs divided by `factor`, fast pairs kept, a linear ramp between, and
                     one magnitude 0.1 ln(factor) + 1 on cos and sin); scores times `scale` times a per-head
                     temperature; a sliding window of `mask.size` positions plus the first `mask.keep_first`
                     tokens of the sequence; softmax; then the heads' WEIGHTS are mixed by a [heads, heads]
                     matrix, and head a applies its mixed weights to the values of its own key/value head
  latent_attention   keys and values expanded per head from ONE cached, normed latent c per token; every query
                     head has `dim` unrotated columns that meet the expanded key and `rot_dim` rotated ones
                     (pairs (2i, 2i+1)) that meet one rotated key part shared by all heads; sliding window of
                     `mask.size` positions.  A layer with `kv_from` has no latent projection and reads the rows
                     another layer cached.  Run in the absorbed form: the key expansion is folded into the
                     queries, the value expansion applied after the attention, so the kernels read the cached
                     rows (latent | rotated key part) directly.

Feed-forwards (`layers[i].mlp.kind`): dense  down(xielu(up h + b) ) + b  with xielu(z) = a_p z^2 + z/2 (z > 0),
a_n (e^z - 1 - z) + z/2 (z <= 0), a_p = softplus(p), a_n = 1/2 + softplus(q) from the layer's two numbers;
moe  sigmoid router, the `top` best scores chosen, the plain scores as weights ON THE EXPERT'S INPUT
(sum of expert(w h)), SiLU-gated experts, plus an optional shared expert of the same form for every token.

One step takes a RaggedBatch and a HybridCache owned by the serving engine (vila_b200/serving.py): attention
layers keep k | v rows, latent layers latent | rotated-key rows in paged pools.  dtype bfloat16: projections on
the tcgen05 GEMM (shapes it does not take go to the CUDA-core grouped kernel); positions and angles, norms,
scores, softmax and weight mixing, the router and the residual sums in fp32.  dtype float32: the same kernels
with fp32 tensors and the CUDA-core linear layer throughout.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional

import torch

from .. import ops
from .moronex import read_safetensors
from .nusovik import _pad_rows

ARCHITECTURE = "Ludazen"
ROT_MAGNITUDE_SLOPE = 0.1   # fixed by the architecture: cos / sin of rescaled frequencies are multiplied by slope * ln(factor) + 1
ROT_RAMP_MIN = 0.001        # fixed by the architecture: smallest width of the ramp between kept and rescaled pairs


@dataclass
class FrequencyScaling:
    factor: float
    original: int     # the length the unscaled frequencies were made for
    fast: float       # pairs that turn at least this often over `original` keep their frequency
    slow: float       # pairs that turn at most this often are divided by `factor`


@dataclass
class RotaryConfig:
    dims: int
    base: float
    scaling: Optional[FrequencyScaling] = None

    @staticmethod
    def from_dict(d: dict) -> "RotaryConfig":
        sc = d.get("scaling")
        return RotaryConfig(dims=int(d["dims"]), base=float(d["base"]),
                            scaling=None if not sc else FrequencyScaling(float(sc["factor"]), int(sc["original"]),
                                                                         float(sc["fast"]), float(sc["slow"])))

    def to_dict(self) -> dict:
        d = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            s = self.scaling
            d["scaling"] = {"factor": s.factor, "fast": s.fast, "original": s.original, "slow": s.slow}
        return d

    def frequencies(self) -> List[float]:
        """angle per position of pair i = 0 .. dims / 2 - 1 (float64 arithmetic)"""
        n = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(n)]
        s = self.scaling
        if s is None:
            return f

        def pair_of(turns: float) -> float:   # the (fractional) pair that turns `turns` times over `original` positions
            return self.dims * math.log(s.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

        lo = max(math.floor(pair_of(s.fast)), 0)
        hi = min(math.ceil(pair_of(s.slow)), self.dims - 1)
        out = []
        for i in range(n):
            ramp = min(max((i - lo) / max(hi - lo, ROT_RAMP_MIN), 0.0), 1.0)
            out.append(f[i] / s.factor * ramp + f[i] * (1.0 - ramp))
        return out

    @property
    def magnitude(self) -> float:
        return 1.0 if self.scaling is None else ROT_MAGNITUDE_SLOPE * math.log(self.scaling.factor) + 1.0


@dataclass
class LudazenLayerConfig:
    type: str                       # "attention" | "latent_attention"
    heads: int
    dim: int
    vdim: int
    scale: float
    window: int                     # mask.size
    rot: RotaryConfig = None
    kv_heads: int = 0               # attention
    keep_first: int = 0             # attention: mask.keep_first
    kv_rank: int = 0                # latent_attention
    rot_dim: int = 0
    kv_from: Optional[int] = None
    mlp_kind: Optional[str] = None  # "dense" | "moe" | None
    ff: int = 0                     # dense: hidden size; moe: hidden size of one expert
    experts: int = 0
    top: int = 0
    shared_ff: int = 0              # moe: hidden size of the shared expert (0: none)


@dataclass
class LudazenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[LudazenLayerConfig] = field(default_factory=list)
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(d: dict) -> "LudazenConfig":
        layers = []
        for i, spec in enumerate(d["layers"]):
            m, kind = spec["mixer"], spec["type"]
            if kind not in ("attention", "latent_attention"):
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            lc = LudazenLayerConfig(type=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                    scale=float(m["scale"]), window=int(m["mask"]["size"]),
                                    rot=RotaryConfig.from_dict(m["rot"]))
            if kind == "attention":
                lc.kv_heads, lc.keep_first = int(m["kv_heads"]), int(m["mask"].get("keep_first", 0))
            else:
                lc.kv_rank, lc.rot_dim = int(m["kv_rank"]), int(m["rot_dim"])
                lc.kv_from = None if m.get("kv_from") is None else int(m["kv_from"])
            mlp = spec.get("mlp")
            if mlp is not None:
                lc.mlp_kind = mlp["kind"]
                if lc.mlp_kind == "dense":
                    lc.ff = int(mlp["ff"])
                elif lc.mlp_kind == "moe":
                    lc.ff = int(mlp["expert"]["ff"])
                    lc.experts, lc.top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
                    lc.shared_ff = int(mlp["shared"]["ff"]) if mlp.get("shared") else 0
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {lc.mlp_kind!r}")
            layers.append(lc)
        cfg = LudazenConfig(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]), layers=layers)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, lc in enumerate(self.layers):
            if lc.window < 1 or lc.keep_first < 0 or lc.heads < 1:
                raise ValueError(f"layer {i}: mask.size {lc.window}, keep_first {lc.keep_first}, heads {lc.heads}")
            if lc.type == "attention":
                if lc.kv_heads < 1 or lc.heads % lc.kv_heads or lc.rot.dims % 2 or lc.rot.dims > lc.dim:
                    raise ValueError(f"layer {i}: heads {lc.heads} / kv_heads {lc.kv_heads} / rot.dims {lc.rot.dims} of {lc.dim}")
            else:
                if lc.rot.dims != lc.rot_dim or lc.rot_dim % 2 or lc.kv_rank < 1:
                    raise ValueError(f"layer {i}: rot.dims {lc.rot.dims} must equal rot_dim {lc.rot_dim} (even); kv_rank {lc.kv_rank}")
                if lc.kv_from is not None:
                    src = self.layers[lc.kv_from] if 0 <= lc.kv_from < i else None
                    if src is None or src.type != "latent_attention" or src.kv_from is not None or \
                            (src.kv_rank, src.rot_dim, src.rot) != (lc.kv_rank, lc.rot_dim, lc.rot):
                        raise ValueError(f"layer {i}: kv_from={lc.kv_from} must name an earlier latent-attention layer "
                                         "with its own latent of the same width and rotation")
            if lc.mlp_kind == "moe" and not 1 <= lc.top <= lc.experts:
                raise ValueError(f"layer {i}: router top {lc.top} of {lc.experts} experts")

    def to_dict(self) -> dict:
        out = []
        for lc in self.layers:
            if lc.type == "attention":
                mask = {"keep_first": lc.keep_first, "size": lc.window} if lc.keep_first else {"size": lc.window}
                m = {"dim": lc.dim, "heads": lc.heads, "kv_heads": lc.kv_heads, "mask": mask, "rot": lc.rot.to_dict(),
                     "scale": lc.scale, "vdim": lc.vdim}
            else:
                m = {"dim": lc.dim, "heads": lc.heads, "kv_rank": lc.kv_rank, "mask": {"size": lc.window},
                     "rot": lc.rot.to_dict(), "rot_dim": lc.rot_dim, "scale": lc.scale, "vdim": lc.vdim}
                if lc.kv_from is not None:
                    m["kv_from"] = lc.kv_from
            mlp = None
            if lc.mlp_kind == "dense":
                mlp = {"ff": lc.ff, "kind": "dense"}
            elif lc.mlp_kind == "moe":
                mlp = {"expert": {"ff": lc.ff}, "kind": "moe", "router": {"experts": lc.experts, "top": lc.top}}
                if lc.shared_ff:
                    mlp["shared"] = {"ff": lc.shared_ff}
            out.append({"mixer": m, "mlp": mlp, "type": lc.type})
        return {"architecture": self.architecture, "layers": out, "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width}

    def tensor_shapes(self) -> Dict[str, tuple]:
        """name -> shape of every checkpoint tensor (the layout `load_weights` expects)."""
        W, s = self.width, {}
        s["embed"] = (self.vocab, W)
        for i, lc in enumerate(self.layers):
            p = f"l{i}."
            s[p + "norm1"] = (W,)
            if lc.type == "attention":
                s[p + "mix.q"], s[p + "mix.k"] = (lc.heads * lc.dim, W), (lc.kv_heads * lc.dim, W)
                s[p + "mix.v"] = (lc.kv_heads * lc.vdim, W)
                s[p + "mix.talk"], s[p + "mix.temp"] = (lc.heads, lc.heads), (lc.heads,)
            else:
                s[p + "mix.q"] = (lc.heads * (lc.dim + lc.rot_dim), W)
                if lc.kv_from is None:
                    s[p + "mix.dkv"], s[p + "mix.dkv.norm"] = (lc.kv_rank + lc.rot_dim, W), (lc.kv_rank,)
                s[p + "mix.uk"], s[p + "mix.uv"] = (lc.heads * lc.dim, lc.kv_rank), (lc.heads * lc.vdim, lc.kv_rank)
            s[p + "mix.o"] = (W, lc.heads * lc.vdim)
            if lc.mlp_kind is not None:
                s[p + "norm2"] = (W,)
            if lc.mlp_kind == "dense":
                s[p + "mlp.up"], s[p + "mlp.up.b"] = (lc.ff, W), (lc.ff,)
                s[p + "mlp.down"], s[p + "mlp.down.b"] = (W, lc.ff), (W,)
                s[p + "mlp.act"] = (2,)
            elif lc.mlp_kind == "moe":
                units = [(f"mlp.e{e}.", lc.ff) for e in range(lc.experts)]
                if lc.shared_ff:
                    units.append(("mlp.shared.", lc.shared_ff))
                for u, ff in units:
                    s[p + u + "gate"], s[p + u + "up"], s[p + u + "down"] = (ff, W), (ff, W), (W, ff)
                s[p + "mlp.router"] = (lc.experts, W)
        s["final.norm"], s["head"] = (W,), (self.vocab, W)
        return s


class _Layer:
    """Device tensors of one layer in the layout the kernels want."""


def _softplus(z: float) -> float:
    return math.log1p(math.exp(-abs(z))) + max(z, 0.0)


class LudazenForCausalLM:
    """Weights + the per-step compute of the architecture.  Sequences, pages, batching and sampling belong to
    `vila_b200.serving.TokenEngine`, which calls `forward_step` / `logits`."""

    def __init__(self, cfg: LudazenConfig, device="cuda", dtype=torch.bfloat16):
        assert dtype in (torch.bfloat16, torch.float32)
        cfg.validate()
        self.config, self.device, self.dtype = cfg, torch.device(device), dtype
        self.vocab_size = cfg.vocab
        self.weights: Dict[str, torch.Tensor] = {}
        self.layers: List[_Layer] = []

    # ---- weights ----------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir, device="cuda", dtype=torch.bfloat16) -> "LudazenForCausalLM":
        d = Path(model_dir)
        cfg = LudazenConfig.from_dict(json.loads((d / "config.json").read_text()))
        files = sorted(d.glob("*.safetensors"))
        if not files:
            raise FileNotFoundError(f"no *.safetensors under {d}")
        tensors: Dict[str, torch.Tensor] = {}
        for f in files:
            tensors.update(read_safetensors(f))
        return cls(cfg, device, dtype).load_weights(tensors)

    def init_random(self, seed: int = 0, scale: float = 1.0, on_device: bool = False) -> "LudazenForCausalLM":
        """Random bf16-representable weights.  on_device: draw them on the model's device (large models)."""
        dev = self.device if on_device else torch.device("cpu")
        g = torch.Generator(device=dev).manual_seed(seed)
        t = {}
        for name, shape in self.config.tensor_shapes().items():
            last = name.rsplit(".", 1)[-1]
            if last == "talk":
                v = torch.eye(shape[0], device=dev) + torch.randn(shape, generator=g, device=dev) * 0.3
            elif last == "temp":
                v = 1.0 + torch.randn(shape, generator=g, device=dev) * 0.2
            elif last == "act":
                v = torch.randn(shape, generator=g, device=dev) * 0.5
            elif len(shape) == 2:
                v = torch.randn(shape, generator=g, device=dev) * (scale / shape[1] ** 0.5)
            elif "norm" in name:
                v = 1.0 + torch.randn(shape, generator=g, device=dev) * 0.1
            else:
                v = torch.randn(shape, generator=g, device=dev) * 0.1
            t[name] = v.to(torch.bfloat16)
        return self.load_weights(t)

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> "LudazenForCausalLM":
        """tensors: checkpoint name -> tensor ([out, in] linear weights).  Sizes are checked against the
        config; the fused / transposed device layouts and the frequency tables are built here."""
        cfg, dev, dt = self.config, self.device, self.dtype
        want = cfg.tensor_shapes()
        missing = [n for n in want if n not in tensors]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:4]}{'...' if len(missing) > 4 else ''}")
        for n, shape in want.items():
            if tuple(tensors[n].shape) != tuple(shape):
                raise ValueError(f"{n}: checkpoint shape {tuple(tensors[n].shape)} != config shape {shape}")

        def w(name):  # compute-dtype copy
            return tensors[name].to(device=dev, dtype=dt).contiguous()

        def f32(name):
            return tensors[name].to(device=dev, dtype=torch.float32).contiguous()

        def gate_up(prefix):  # rows gate_0, up_0, gate_1, ...: the layout of the gated-unit epilogue
            g_, u_ = w(prefix + "gate"), w(prefix + "up")
            gu = torch.empty(2 * g_.shape[0], g_.shape[1], device=dev, dtype=dt)
            gu[0::2], gu[1::2] = g_, u_
            return gu

        self.weights = {n: tensors[n] for n in want}
        self.embed, self.head, self.final_norm = w("embed"), w("head"), f32("final.norm")
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            p, L = f"l{i}.", _Layer()
            L.cfg, L.index = lc, i
            L.norm1 = f32(p + "norm1")
            L.inv_freq = torch.tensor(lc.rot.frequencies(), dtype=torch.float64, device=dev) if lc.rot.dims else None
            L.magnitude = lc.rot.magnitude
            if lc.type == "attention":
                L.qkv = _pad_rows(torch.cat([w(p + "mix.q"), w(p + "mix.k"), w(p + "mix.v")], 0))
                L.talk, L.temp = f32(p + "mix.talk"), f32(p + "mix.temp")
            else:
                parts = [w(p + "mix.q")] + ([w(p + "mix.dkv")] if lc.kv_from is None else [])
                L.in_w = _pad_rows(torch.cat(parts, 0))
                L.dkv_norm = f32(p + "mix.dkv.norm") if lc.kv_from is None else None
                # key expansion per head, transposed: q'_h = uk_t[h] q_h, uk_t [H, kv_rank, dim]
                L.uk_t = w(p + "mix.uk").view(lc.heads, lc.dim, lc.kv_rank).transpose(1, 2).contiguous()
                L.uv = w(p + "mix.uv").view(lc.heads, lc.vdim, lc.kv_rank).contiguous()
                L.latent_layer = i if lc.kv_from is None else lc.kv_from
            L.o = w(p + "mix.o")
            if lc.mlp_kind is not None:
                L.norm2 = f32(p + "norm2")
            if lc.mlp_kind == "dense":
                L.up, L.down = _pad_rows(w(p + "mlp.up")), w(p + "mlp.down")
                L.up_b = torch.zeros(L.up.shape[0], device=dev, dtype=dt)
                L.up_b[:lc.ff] = w(p + "mlp.up.b")
                L.down_b = w(p + "mlp.down.b")
                a = tensors[p + "mlp.act"].to(torch.float64).tolist()
                L.act = (_softplus(a[0]), 0.5 + _softplus(a[1]))
            elif lc.mlp_kind == "moe":
                L.gu = torch.stack([gate_up(p + f"mlp.e{e}.") for e in range(lc.experts)]).contiguous()
                L.down = torch.stack([w(p + f"mlp.e{e}.down") for e in range(lc.experts)]).contiguous()
                L.router = f32(p + "mlp.router")
                if lc.shared_ff:
                    L.shared_gu, L.shared_down = gate_up(p + "mlp.shared."), w(p + "mlp.shared.down")
            self.layers.append(L)
        return self

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return dict(self.weights)

    def save_pretrained(self, model_dir) -> None:
        from safetensors.torch import save_file
        d = Path(model_dir)
        d.mkdir(parents=True, exist_ok=True)
        (d / "config.json").write_text(json.dumps(self.config.to_dict(), indent=1))
        save_file({k: v.detach().cpu().contiguous() for k, v in self.weights.items()}, str(d / "model.safetensors"))

    # ---- cache geometry (read by serving.HybridCache) ----------------------------------------------
    def latent_widths(self) -> Dict[int, int]:
        """layer -> width of its paged per-token row: k | v of all key/value heads (attention), or latent |
        rotated key part (latent attention with its own latent projection)"""
        out = {}
        for i, lc in enumerate(self.config.layers):
            if lc.type == "attention":
                out[i] = lc.kv_heads * (lc.dim + lc.vdim)
            elif lc.kv_from is None:
                out[i] = lc.kv_rank + lc.rot_dim
        return out

    def state_shapes(self) -> Dict[int, tuple]:
        return {}   # nothing recurrent: a sequence's memory is its pages

    # ---- compute --------------------------------------------------------------------------------------
    def _attention(self, L: _Layer, h, batch, cache):
        lc = L.cfg
        pool = cache.latent[L.index]
        qkv = ops.linear_any(h, L.qkv)
        q = ops.rope_append(qkv, batch.positions, batch.cache_rows, pool, heads=lc.heads, kv_heads=lc.kv_heads,
                            dim=lc.dim, vdim=lc.vdim, inv_freq=L.inv_freq, unit_norm=False, eps=self.config.norm_eps,
                            halves=True, mscale=L.magnitude)
        o = torch.empty(h.shape[0], lc.heads * lc.vdim, dtype=self.dtype, device=self.device)
        kw = dict(heads=lc.heads, kv_heads=lc.kv_heads, dim=lc.dim, vdim=lc.vdim, page=cache.page, scale=lc.scale,
                  talk=L.talk, talk_after=True, head_scale=L.temp, window=lc.window, keep_first=lc.keep_first, out=o)
        if batch.tiles is not None:
            ops.paged_attention(q, pool, cache.page_tables, batch.tiles, max_rows=16, **kw)
        if batch.decode_tiles is not None:
            ops.paged_attention(q, pool, cache.page_tables, batch.decode_tiles, max_rows=1,
                                nsplit=self._splits(cache, lc.window + lc.keep_first), **kw)
        return ops.linear_any(o, L.o)

    @staticmethod
    def _splits(cache, visible: int) -> int:
        """CTAs per decoded row: the pool's choice, but no more than one per 64 keys a window lets a row see"""
        return max(1, min(cache.decode_splits, (visible + 63) // 64))

    def _latent_attention(self, L: _Layer, h, batch, cache):
        lc, T = L.cfg, h.shape[0]
        R, Dr, qh = lc.kv_rank, lc.rot_dim, lc.dim + lc.rot_dim
        RW = R + Dr
        pool = cache.latent[L.latent_layer]
        P = ops.linear_any(h, L.in_w)                                    # q | (latent, key part to rotate)
        own = lc.kv_from is None
        # folded queries: head h's row is (W_uk,h^T q_h | rotated q part), dotted with the cached (latent | rotated key part)
        qa = torch.empty(T, lc.heads * RW, dtype=torch.float32, device=self.device)
        ops.glinear(P[:, :lc.heads * qh], L.uk_t, groups=lc.heads, a_group_off=qh, o_group_off=RW, out=qa)
        ops.latent_rope_append(batch.positions, L.inv_freq, rank=R, mscale=L.magnitude,
                               kv=P[:, lc.heads * qh:lc.heads * qh + RW] if own else None, norm_w=L.dkv_norm,
                               eps=self.config.norm_eps, pool=pool if own else None,
                               cache_rows=batch.cache_rows if own else None,
                               q=P, qa=qa, heads=lc.heads, q_head=qh, q_off=lc.dim)
        ol = torch.empty(T, lc.heads * RW, dtype=self.dtype, device=self.device)
        kw = dict(heads=lc.heads, page=cache.page, scale=lc.scale, window=lc.window, out=ol)
        if batch.tiles is not None:
            ops.latent_attention(qa, pool, cache.page_tables, batch.tiles, **kw)
        if batch.decode_tiles is not None:
            ops.latent_attention(qa, pool, cache.page_tables, batch.decode_tiles, decode=True,
                                 nsplit=self._splits(cache, lc.window), **kw)
        o = ops.glinear(ol, L.uv, groups=lc.heads, a_group_off=RW, o_group_off=lc.vdim)   # reads the latent columns only
        return ops.linear_any(o, L.o)

    def _dense(self, L: _Layer, h):
        u = ops.linear_any(h, L.up, bias=L.up_b, act=ops.ACT_XIELU, act_params=L.act)
        return ops.linear_any(u[:, :L.cfg.ff], L.down, bias=L.down_b), None

    def _experts(self, L: _Layer, h):
        lc, T = L.cfg, h.shape[0]
        idx, wt = ops.moe_route_sigmoid(h, L.router, None, lc.top)
        seg, srt = ops.moe_group(idx, lc.experts)
        act = ops.glinear(h, L.gu, groups=lc.experts, seg=seg, a_rows=srt, a_row_div=lc.top, swiglu=True,
                          in_scale=wt.view(-1))
        parts = ops.glinear(act, L.down, groups=lc.experts, seg=seg, o_rows=srt, out_dtype=torch.float32,
                            out_rows_total=T * lc.top)
        shared = None
        if lc.shared_ff:
            shared = ops.linear_any(ops.linear_any(h, L.shared_gu, swiglu=True), L.shared_down)
        return shared, parts

    def _add(self, x, a, parts, top, next_norm):
        """x += a + partials; -> the next sublayer's normed operand (None after the last one)"""
        if next_norm is None:
            ops.residual_add_rows(x, a, parts, n_partials=top)
            return None
        return ops.residual_norm_rows(x, a, next_norm, self.config.norm_eps, part=parts, n_partials=top,
                                      out_dtype=self.dtype)

    @torch.inference_mode()
    def forward_step(self, batch, cache, layer_outputs: Optional[list] = None) -> torch.Tensor:
        """Run the rows of `batch` through all layers on top of what `cache` holds; the k | v and latent rows of
        the batch are written to the cache.  -> residual stream fp32 [T, width]."""
        eps, n = self.config.norm_eps, len(self.layers)
        x = ops.embed_rows(self.embed, batch.ids)
        h = ops.rmsnorm_rows(x, self.layers[0].norm1, eps, out_dtype=self.dtype) if n else None
        for i, L in enumerate(self.layers):
            nxt = self.layers[i + 1].norm1 if i + 1 < n else None
            y = (self._attention if L.cfg.type == "attention" else self._latent_attention)(L, h, batch, cache)
            if L.cfg.mlp_kind is None:
                h = self._add(x, y, None, 1, nxt)
            else:
                h = self._add(x, y, None, 1, L.norm2)
                a, parts = (self._dense if L.cfg.mlp_kind == "dense" else self._experts)(L, h)
                h = self._add(x, a, parts, L.cfg.top if parts is not None else 1, nxt)
            if layer_outputs is not None:
                layer_outputs.append(x.clone())
        return x

    @torch.inference_mode()
    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """final norm + output head for the given residual rows fp32 [n, width] -> fp32 [n, vocab]"""
        h = ops.rmsnorm_rows(hidden_rows.contiguous(), self.final_norm, self.config.norm_eps, out_dtype=self.dtype)
        return ops.glinear(h, self.head, out_dtype=torch.float32)

    @torch.inference_mode()
    def generate(self, input_ids, max_new_tokens: int = 20, eos_token_id=None, do_sample: bool = False,
                 temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: Optional[int] = None,
                 slots: int = 4, **engine_kw) -> List[List[int]]:
        """input_ids: one prompt (list of ids) or a list of prompts -> new ids per prompt, through the
        continuous-batching scheduler (vila_b200.serving.generate_tokens)."""
        from ..serving import generate_tokens
        prompts = [list(map(int, input_ids))] if input_ids and not isinstance(input_ids[0], (list, tuple)) \
            else [list(map(int, p)) for p in input_ids]
        eos = [] if eos_token_id is None else ([eos_token_id] if isinstance(eos_token_id, int) else list(eos_token_id))
        return generate_tokens(self, prompts, max_new_tokens, eos, slots=slots, sample=do_sample,
                               temperature=temperature, top_k=top_k, top_p=top_p, seed=seed, **engine_kw)
