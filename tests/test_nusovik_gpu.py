"""Nusovik on the GPU against the plain float64 oracle (oracle/nusovik_oracle.py): every mechanism's
kernel alone against a direct float64 restatement written here, then whole models (own small
configurations, random weights) under every way the engine can be driven: whole prompts, token-by-token
decoding, portions down to two tokens, mixed batches of unequal requests, pages and slots that are freed
and reused, long decoding, greedy generation through the scheduler, the command line and the trace runner."""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from oracle import nusovik_oracle as O

pytestmark = pytest.mark.gpu
BF, F32, F64 = torch.bfloat16, torch.float32, torch.float64
ROOT = Path(__file__).resolve().parent.parent


def _ops():
    from vila_b200 import ops
    return ops


def rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def tol(dtype):
    return 2e-5 if dtype == F32 else 5e-2   # max abs error over the largest expected entry


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64) * scale


def dev(t, dtype=F32):
    return t.to(device="cuda", dtype=dtype).contiguous()


def i32(rows):
    return torch.tensor(rows, dtype=torch.int32, device="cuda")


# ------------------------------------------------------------------------------------------------
# configurations (none of them a size combination of a published or given model)
# ------------------------------------------------------------------------------------------------
def left(heads, kv_heads, dim, chunk, bias_max, scale=None):
    return {"bias_max": bias_max, "dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": chunk},
            "scale": scale if scale is not None else dim ** -0.5, "vdim": dim}


def right(heads, vdim, state, groups, norm_groups, conv):
    return {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim}


def parallel(lft, rgt, ls, rs, ff):
    return {"mixer": {"left": lft, "left_scale": ls, "right": rgt, "right_scale": rs},
            "mlp": {"ff": ff, "kind": "dense"} if ff else None, "type": "parallel"}


def mamba1(inner, state, dt_rank, conv, ff):
    return {"mixer": {"conv": conv, "dt_rank": dt_rank, "inner": inner, "state": state},
            "mlp": {"ff": ff, "kind": "dense"} if ff else None, "type": "mamba1"}


def config(width, vocab, layers, *, embed_scale, logit_scale, eps=1e-5):
    return {"architecture": "Nusovik", "embedding": {"scale": embed_scale}, "layers": layers,
            "logit_scale": logit_scale, "norm": {"eps": eps}, "vocab": vocab, "width": width}


# name -> (configuration, rows of the distance-bias tables)
CONFIGS = {
    # nothing is a multiple of 8: every projection runs on the CUDA-core kernel in both dtypes; a chunk that
    # is no multiple of the 16-row tile or the 64-token page; three taps, five taps; a layer without feed-forward
    "odd": (config(100, 131, [
        parallel(left(4, 2, 12, 24, 40), right(6, 10, 12, 3, 3, 3), 1.3, 0.7, 72),
        mamba1(56, 7, 5, 2, 40),
        parallel(left(3, 3, 20, 50, 33), right(2, 24, 40, 1, 1, 5), 0.6, 1.2, 0)], embed_scale=1.7, logit_scale=0.5), 10),
    # tensor-core shapes; a recurrent layer first; one key head for 8 query heads
    "aligned": (config(128, 256, [
        mamba1(256, 16, 8, 4, 0),
        parallel(left(8, 1, 32, 64, 100), right(4, 32, 64, 1, 4, 4), 1.0, 1.0, 256),
        mamba1(128, 24, 16, 3, 128)], embed_scale=1.0, logit_scale=1.0), 16),
    # values that other models make larger: one head, one group, one tap (no convolution tail), a state of one
    # entry, a step size of rank one, a chunk of ONE position (a query sees itself and the sink), a chunk longer
    # than any prompt (plain causal attention with far keys beyond bias_max), a state of 130 entries
    "ones": (config(64, 97, [
        parallel(left(1, 1, 8, 1000, 300), right(1, 16, 130, 1, 1, 1), 1.0, 0.5, 0),
        mamba1(40, 1, 1, 1, 8),
        parallel(left(2, 1, 5, 1, 9), right(4, 4, 8, 4, 2, 2), 2.0, 1.0, 24)], embed_scale=0.3, logit_scale=2.0), 6),
}


def build(name, dtype, seed=0):
    """name: a key of CONFIGS or a (configuration, bias rows) pair"""
    from vila_b200.model import NusovikConfig, NusovikForCausalLM
    cfg, rows = CONFIGS[name] if isinstance(name, str) else name
    model = NusovikForCausalLM(NusovikConfig.from_dict(cfg), "cuda", dtype).init_random(seed, scale=1.5, bias_rows=rows)
    return cfg, model


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def run_schedule(model, prompts, schedule, max_tokens, slots=4):
    """schedule: steps of [(name, rows)]; the logits of every row are collected per request; a request
    is released with its last row.  -> {name: [len, vocab] fp32 on the CPU}"""
    from vila_b200.serving import TokenEngine
    eng = TokenEngine(model, max_tokens=max_tokens, slots=slots)
    at = {k: 0 for k in prompts}
    got = {k: [] for k in prompts}
    for step in schedule:
        entries = []
        for name, n in step:
            entries.append((name, prompts[name][at[name]:at[name] + n], list(range(n))))
            at[name] += n
        lg = eng.step(entries).cpu()
        o = 0
        for name, n in step:
            got[name].append(lg[o:o + n])
            o += n
            if at[name] == len(prompts[name]):
                eng.release(name)
    assert not eng.seqs and eng.cache.allocator.available == eng.cache.n_pages
    return {k: torch.cat(v) for k, v in got.items()}


def rows_close(got, want, dtype, what=""):
    """every row within tolerance (relative to the largest entry of the expected tensor).  bfloat16: the norm
    sits on the OUTPUT of a sublayer, so a row whose mixer output nearly cancels (a sum over state entries
    several times smaller than its neighbours') has the bf16 noise of the projections multiplied by the
    normalisation; one row in 50 may leave the tolerance, none by more than 8 times.  float32 has no exception."""
    got, want = got.double().cpu(), want.double().cpu()
    assert bool(torch.isfinite(got).all()), what
    err = (got - want).abs().amax(-1) / want.abs().max()
    bad = int((err >= tol(dtype)).sum())
    allowed = 0 if dtype == F32 else max(1, err.numel() // 50)
    assert bad <= allowed and float(err.max()) < 8 * tol(dtype), (what, bad, err.numel(), float(err.max()))


def check_logits(cfg, model, prompts, got, dtype):
    for name, toks in prompts.items():
        want = O.forward(cfg, model.state_dict(), toks)
        assert got[name].shape == want.shape
        rows_close(got[name], want, dtype, name)


# ------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------
def test_embedding_with_sinusoidal_positions(cuda):
    ops = _ops()
    for cols, scale in ((7, 0.5), (64, 1.0), (130, 2.5), (1030, 1.0)):
        table = rnd(50, cols, seed=cols).to(BF)
        ids = torch.randint(0, 50, (9,), generator=torch.Generator().manual_seed(1))
        pos = torch.tensor([0, 1, 2, 63, 64, 1000, 4097, 123457, 5])
        inv = (torch.tensor(10000.0, dtype=F64) ** (-2.0 * torch.arange((cols + 1) // 2, dtype=F64) / cols))
        want = table.double()[ids] * scale
        for c in range(cols):
            ang = pos.double() * 10000.0 ** (-2.0 * (c // 2) / cols)
            want[:, c] += torch.cos(ang) if c % 2 else torch.sin(ang)
        x, xc = ops.embed_sincos_rows(dev(table, BF), i32(ids.tolist()), i32(pos.tolist()), inv.cuda(), scale, copy_dtype=BF)
        assert rel(x, want) < 1e-6 and rel(xc, want) < 1e-2
        assert torch.equal(xc, x.to(BF))


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("rows,cols", [(1, 7), (37, 96), (9, 2100), (300, 1030)])
def test_branch_norm_residual(cuda, dtype, rows, cols):
    ops = _ops()
    x0, a, b, w = rnd(rows, cols, seed=1), rnd(rows, cols, seed=2).to(dtype), rnd(rows, cols, seed=3).to(dtype), rnd(cols, seed=4)
    eps = 1e-3

    def rms(v):
        return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    x = dev(x0)
    copy = ops.branch_norm_residual(x, dev(a, dtype), dev(w), eps, a_scale=0.8, b=dev(b, dtype), b_scale=-1.1, copy_dtype=BF)
    want = x0.float().double() + rms(0.8 * a.double() - 1.1 * b.double()) * w.float().double()
    assert rel(x, want) < 1e-5 and torch.equal(copy, x.to(BF))
    x = dev(x0)
    wide = dev(torch.cat([a, b], 1), dtype)   # a branch that is a column slice of a wider tensor
    assert ops.branch_norm_residual(x, wide[:, :cols], None, eps) is None
    assert rel(x, x0.float().double() + rms(a.double())) < 1e-5


def conv_direct(u, w, b, silu):
    T, taps = u.shape[0], w.shape[1]
    out = b.expand(T, -1).clone()
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out * torch.sigmoid(out) if silu else out


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_conv_in_portions_through_reused_slots(cuda, dtype, taps):
    """two sequences fed in portions of 1 .. 17 rows (shorter and longer than the tail), the inputs a column
    slice of a wider tensor, slots that hold another sequence's tail before"""
    ops = _ops()
    Cc, lens = 37, {"a": 61, "b": 23}
    w, b = rnd(Cc, taps, seed=1, scale=0.5), rnd(Cc, seed=2)
    u = {k: rnd(n, Cc, seed=3 + i).to(dtype) for i, (k, n) in enumerate(lens.items())}
    want = {k: conv_direct(u[k].double(), w, b, True) for k in u}
    state = torch.full((3, max(taps - 1, 1), Cc), 77.0, device="cuda")[:, :taps - 1].contiguous() if taps > 1 else None
    slot, at, got = {"a": 2, "b": 0}, {"a": 0, "b": 0}, {"a": [], "b": []}
    plan = [[("a", 1), ("b", 2)], [("b", 1), ("a", 17)], [("a", 2)], [("a", 9), ("b", 9)], [("b", 11), ("a", 1)], [("a", 31)]]
    for step in plan:
        rows, seqs, row_seq = [], [], []
        for k, n in step:
            seqs.append((len(rows), n, at[k], slot[k]))
            row_seq += [len(seqs) - 1] * n
            rows += list(u[k][at[k]:at[k] + n])
        wide = torch.zeros(len(rows), Cc + 5, dtype=dtype)
        wide[:, 3:3 + Cc] = torch.stack(rows)
        out = ops.causal_conv_rows(dev(wide, dtype)[:, 3:3 + Cc], dev(w), dev(b), state, i32(seqs), i32(row_seq),
                                   act=ops.CONV_SILU, out_dtype=F32)
        o = 0
        for k, n in step:
            got[k].append(out[o:o + n].cpu())
            at[k] += n
            o += n
    for k in u:
        assert at[k] == lens[k] and rel(torch.cat(got[k]), want[k]) < 1e-5, k


def ssd_direct(x, B, C, dt, z, A_log, dt_bias, D, groups):
    """x [T, H, P], B / C [T, G, N], dt [T, H] raw, z [T, H, P] -> y [T, H, P], final state [H, P, N]"""
    T, H, P = x.shape
    N = B.shape[2]
    dt = O.softplus(dt + dt_bias)
    y, S = torch.zeros(T, H, P, dtype=F64), torch.zeros(H, P, N, dtype=F64)
    for t in range(T):
        for h in range(H):
            g = h // (H // groups)
            S[h] = torch.exp(-torch.exp(A_log[h]) * dt[t, h]) * S[h] + dt[t, h] * torch.outer(x[t, h], B[t, g])
            y[t, h] = S[h] @ C[t, g] + D[h] * x[t, h]
    return y * (z * torch.sigmoid(z)), S


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("H,P,N,G", [(6, 10, 12, 3), (2, 40, 40, 1), (4, 32, 64, 4), (1, 5, 130, 1), (3, 33, 1, 3)])
def test_ssd_scan_in_portions_through_stale_slots(cuda, dtype, H, P, N, G):
    ops = _ops()
    T, inner = 70, H * P
    x, B, C = rnd(T, H, P, seed=1).to(dtype), rnd(T, G, N, seed=2).to(dtype), rnd(T, G, N, seed=3).to(dtype)
    dt, z = rnd(T, H, seed=4).to(dtype), rnd(T, H, P, seed=5).to(dtype)
    A_log, dt_bias, D = rnd(H, seed=6, scale=0.5), rnd(H, seed=7) - 1.0, rnd(H, seed=8)
    want, S = ssd_direct(x.double(), B.double(), C.double(), dt.double(), z.double(), A_log.float().double(),
                         dt_bias.float().double(), D.float().double(), G)
    # one wide row per token, as a projection would leave it: z | x | B | C | dt (+ padding)
    wide = torch.cat([z.reshape(T, inner), x.reshape(T, inner), B.reshape(T, G * N), C.reshape(T, G * N), dt,
                      torch.zeros(T, 3, dtype=dtype)], 1)
    wd = dev(wide, dtype)
    chans = inner + 2 * G * N
    state = torch.full((2, H, P, N), 55.0, device="cuda")      # stale: a sequence at position 0 must not read it
    out, at = [], 0
    for n in (1, 2, 35, 1, 16, 15):
        seqs = i32([(at, n, at, 1)])
        out.append(ops.ssd_scan(wd[:, inner:inner + chans], wd[:, inner + chans:inner + chans + H], wd[:, :inner], state,
                                seqs, heads=H, vdim=P, nstate=N, groups=G, dt_bias=dev(dt_bias), A_log=dev(A_log),
                                D=dev(D))[at:at + n])
        at += n
    assert at == T
    assert rel(torch.cat(out).view(T, H, P), want) < 2e-5
    assert rel(state[1], S) < 2e-5 and bool((state[0] == 55.0).all())


def selective_direct(x, dt, B, C, z, A_log, dt_bias, D):
    T, Cc = x.shape
    dt = O.softplus(dt + dt_bias)
    A = -torch.exp(A_log)
    S, y = torch.zeros(Cc, A.shape[1], dtype=F64), torch.zeros(T, Cc, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y * (z * torch.sigmoid(z)), S


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("Cc,N", [(56, 7), (40, 1), (64, 16), (33, 33), (70, 100), (8, 200)])
def test_selective_scan_in_portions_through_stale_slots(cuda, dtype, Cc, N):
    ops = _ops()
    T = 70
    x, dt, z = rnd(T, Cc, seed=1).to(dtype), rnd(T, Cc, seed=2).to(dtype), rnd(T, Cc, seed=3).to(dtype)
    bc = rnd(T, 2 * N, seed=4).to(dtype)
    A_log, dt_bias, D = rnd(Cc, N, seed=5, scale=0.5), rnd(Cc, seed=6) - 1.0, rnd(Cc, seed=7)
    want, S = selective_direct(x.double(), dt.double(), bc.double()[:, :N], bc.double()[:, N:], z.double(),
                               A_log.float().double(), dt_bias.float().double(), D.float().double())
    low = dev(torch.cat([torch.zeros(T, 5, dtype=dtype), bc], 1), dtype)      # B | C behind a low-rank step-size block
    state = torch.full((3, Cc, N), -9.0, device="cuda")
    out, at = [], 0
    for n in (2, 1, 33, 1, 17, 16):
        out.append(ops.selective_scan(dev(x, dtype), dev(dt, dtype), low[:, 5:], dev(z, dtype), state, i32([(at, n, at, 2)]),
                                      dt_bias=dev(dt_bias), A_log=dev(A_log), D=dev(D))[at:at + n])
        at += n
    assert rel(torch.cat(out), want) < 2e-5
    assert rel(state[2], S) < 2e-5 and bool((state[:2] == -9.0).all())


def test_two_sequences_per_scan_launch(cuda):
    """a decoded token of one sequence beside a prompt portion of another, each with its own slot"""
    ops = _ops()
    H, P, N = 2, 8, 8
    xbc, dt = rnd(12, H * P + 2 * N, seed=1), rnd(12, H, seed=2)
    par = dict(heads=H, vdim=P, nstate=N, groups=1, dt_bias=dev(rnd(H, seed=3)), A_log=dev(rnd(H, seed=4)), D=dev(rnd(H, seed=5)))
    state = torch.zeros(2, H, P, N, device="cuda")
    both = ops.ssd_scan(dev(xbc), dev(dt), None, state, i32([(0, 11, 0, 0), (11, 1, 0, 1)]), **par)
    s2 = torch.zeros(2, H, P, N, device="cuda")
    a = ops.ssd_scan(dev(xbc[:11]), dev(dt[:11]), None, s2, i32([(0, 11, 0, 1)]), **par)
    b = ops.ssd_scan(dev(xbc[11:]), dev(dt[11:]), None, s2, i32([(0, 1, 0, 0)]), **par)
    assert torch.equal(both, torch.cat([a, b])) and torch.equal(state[0], s2[1]) and torch.equal(state[1], s2[0])


@pytest.mark.parametrize("dtype", [F32, BF])
def test_head_norm_with_weights_and_values_from_keys(cuda, dtype):
    ops = _ops()
    H, G, d, T, eps = 5, 1, 12, 9, 1e-4
    row = rnd(T, (H + G) * d + 3, seed=1).to(dtype)
    wq, wk = rnd(d, seed=2), rnd(d, seed=3)
    pool = torch.zeros(64, 2 * G * d, device="cuda", dtype=dtype)
    rows = [40, 3, 17, 63, 0, 1, 2, 33, 9]
    q = ops.rope_append(dev(row, dtype), i32(list(range(T))), i32(rows), pool, heads=H, kv_heads=G, dim=d, vdim=d,
                        inv_freq=None, unit_norm=True, eps=eps, q_norm_w=dev(wq), k_norm_w=dev(wk), v_from_k=True)

    def rms(v):
        return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    r = row.double()
    assert rel(q, (rms(r[:, :H * d].view(T, H, d)) * wq.float().double()).reshape(T, -1)) < 1e-5
    k = r[:, H * d:(H + G) * d].view(T, G, d)
    got = pool[torch.tensor(rows, device="cuda")]
    assert rel(got[:, :G * d], (rms(k) * wk.float().double()).reshape(T, -1)) < (1e-5 if dtype == F32 else 1e-2)
    assert torch.equal(got[:, G * d:].cpu(), row[:, H * d:(H + G) * d])     # the value is the key as it came in


def attend_direct(q, K, V, pos0, *, sink, scale, table, chunk, gate):
    """q [n, H, d] at positions pos0 .., K / V [ctx, G, d] -> [n, H, d]; table [rows, H] bias by distance"""
    n, H, _ = q.shape
    G = K.shape[1]
    out = torch.zeros(n, H, V.shape[2], dtype=F64)
    for i in range(n):
        pos = pos0 + i
        lo = (pos // chunk) * chunk if chunk else 0
        for h in range(H):
            g = h // (H // G)
            js = torch.arange(lo, pos + 1)
            s = K[lo:pos + 1, g] @ q[i, h] * scale
            if table is not None:
                s = s + table[torch.clamp(pos - js, max=table.shape[0] - 1), h]
            m = torch.maximum(s.max(), sink[h]) if sink is not None else s.max()
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = (e / den) @ V[lo:pos + 1, g]
            if gate is not None:
                out[i, h] *= torch.sigmoid(gate[i, h])
    return out


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("H,G,d,chunk", [(4, 2, 12, 24), (3, 3, 20, 50), (8, 1, 32, 64), (1, 1, 8, 0), (2, 1, 5, 1), (6, 2, 16, 7),
                                         (40, 1, 16, 24), (32, 8, 64, 80)])
def test_attention_with_distance_bias_chunks_sink_and_gate(cuda, dtype, H, G, d, chunk):
    """portions that start and end inside pages and chunks, shuffled physical pages, prompt tiles and decoded rows
    (1 / 3 key splits) in the same pool"""
    ops = _ops()
    ctx, page = 150, 64
    K, V = rnd(ctx, G, d, seed=1).to(dtype), rnd(ctx, G, d, seed=2).to(dtype)
    sink, table = rnd(H, seed=3), rnd(11, H, seed=4)
    pages = [5, 1, 3]
    pool = torch.zeros(6 * page, 2 * G * d, dtype=dtype)
    for j in range(ctx):
        pool[pages[j // page] * page + j % page] = torch.cat([K[j].reshape(-1), V[j].reshape(-1)])
    pt = torch.zeros(2, 6, dtype=torch.int32)
    pt[1, :3] = torch.tensor(pages)
    for pos0, n in ((0, 16), (17, 16), (40, 9), (60, 16), (96, 16), (134, 16), (149, 1), (23, 1), (24, 1), (64, 1)):
        q, gate = rnd(n, H, d, seed=10 + pos0), rnd(n, H + 2, seed=20 + pos0).to(dtype)
        want = attend_direct(q.float().double(), K.double(), V.double(), pos0, sink=sink.float().double(), scale=0.3,
                             table=table.float().double(), chunk=chunk, gate=gate.double())
        kw = dict(heads=H, kv_heads=G, dim=d, vdim=d, page=page, scale=0.3, sink=dev(sink), dist_bias=dev(table),
                  chunk=chunk, gate=dev(gate, dtype)[:, :H], out_dtype=F32)
        tiles = i32([(0, n, pos0, 1)])
        splits = (1, 3) if n == 1 else (1,)
        for ns in splits:
            got = ops.paged_attention(dev(q.reshape(n, -1)), dev(pool, dtype), pt.cuda(), tiles, max_rows=16 if n > 1 else 1,
                                      nsplit=ns, **kw)
            assert rel(got.view(n, H, d), want) < 2e-5, (pos0, n, ns)


@pytest.mark.parametrize("decode", [False, True])
def test_chunk_edges_far_keys_and_the_sink_show(cuda, decode):
    """One key gets a score far above all others.  Just inside the query's chunk it must take all the weight,
    just outside it must not be seen at all; a key hundreds of positions back must win when the chunk is long;
    a large bias at ONE distance must pick the key at that distance; a huge sink must empty the output."""
    ops = _ops()
    H, G, d, page, ctx = 2, 1, 16, 64, 700
    K, V = rnd(ctx, G, d, seed=1, scale=0.1), rnd(ctx, G, d, seed=2)
    big = rnd(d, seed=3)
    big = big * (4.0 / big.norm())            # the key that stands out: score 60 against about 10 at most
    pt = torch.arange(11, dtype=torch.int32)[None].cuda()
    n = 1 if decode else 5
    pos0 = ctx - n

    def run(q, chunk, keys=K, table=None, sink=None):
        pool = torch.cat([keys.reshape(ctx, -1), V.reshape(ctx, -1)], 1)
        pool = torch.cat([pool, torch.zeros(704 - ctx, 2 * G * d, dtype=F64)])
        return ops.paged_attention(dev(q.reshape(n, -1)), dev(pool), pt, i32([(0, n, pos0, 0)]), heads=H, kv_heads=G,
                                   dim=d, vdim=d, page=page, scale=1.0, chunk=chunk, max_rows=1 if decode else 16,
                                   nsplit=2 if decode else 1, dist_bias=None if table is None else dev(table),
                                   sink=None if sink is None else dev(sink), out_dtype=F32).view(n, H, d).cpu().double()

    def standing_out(j):       # keys with the big one at position j, and the query every row and head asks it with
        keys = K.clone()
        keys[j, 0] = big
        return keys, (big * (60.0 / 16.0)).expand(n, H, d).contiguous()

    # the chunk of the last rows starts at 672 (chunk 112) -> key 672 inside, key 671 outside
    keys, q = standing_out(672)
    assert rel(run(q, 112, keys), V[672, 0].expand(n, H, d)) < 1e-4
    keys, q = standing_out(671)
    out = run(q, 112, keys)
    want = attend_direct(q, keys, V, pos0, sink=None, scale=1.0, table=None, chunk=112, gate=None)
    assert rel(out, want) < 1e-4 and rel(out, V[671, 0].expand(n, H, d)) > 0.1
    # a far key with one long chunk, and without chunks
    keys, q = standing_out(13)
    assert rel(run(q, 1000, keys), V[13, 0].expand(n, H, d)) < 1e-4
    assert rel(run(q, 0, keys), V[13, 0].expand(n, H, d)) < 1e-4
    # bias: +40 at distance 5 exactly (rows 0..7, the last row serves all larger distances)
    table = torch.zeros(8, H, dtype=F64)
    table[5] = 40.0
    out = run(torch.zeros(n, H, d, dtype=F64), 0, table=table)
    for i in range(n):
        assert rel(out[i], V[pos0 + i - 5, 0].expand(H, d)) < 1e-4
    # the sink takes (nearly) all the weight of head 1 only
    out = run(torch.zeros(n, H, d, dtype=F64), 0, sink=torch.tensor([-30.0, 30.0], dtype=F64))
    assert float(out[:, 1].abs().max()) < 1e-6 and float(out[:, 0].abs().max()) > 1e-3


@pytest.mark.parametrize("M", [5, 200])
def test_squared_relu_epilogue_of_the_tensor_core_gemm(cuda, M):
    ops = _ops()
    x, w = rnd(M, 64, seed=1).to(BF), rnd(96, 64, seed=2, scale=0.2).to(BF)
    got = ops.linear(dev(x, BF), dev(w, BF), act=ops.ACT_RELU2)
    z = (x.double() @ w.double().T).to(BF).double()
    assert rel(got, torch.relu(z) ** 2) < 1e-2
    assert rel(ops.linear_any(dev(x, BF), dev(w, BF), act=ops.ACT_RELU2), got) < 1e-2


# ------------------------------------------------------------------------------------------------
# whole models
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_layers(cuda, name, dtype):
    from vila_b200.serving import TokenEngine
    cfg, model = build(name, dtype)
    toks = tokens_for(cfg, 150, 1)
    eng = TokenEngine(model, max_tokens=192, slots=1)
    layers, after = [], []
    lg = eng.step([("a", toks, list(range(len(toks))))], layer_outputs=layers)
    want = O.forward(cfg, model.state_dict(), toks, after)
    assert len(layers) == len(after) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(layers, after)):
        rows_close(a, b, dtype, f"after layer {i}")
    rows_close(lg, want, dtype, "logits")
    # a one-token sequence in the slot and pages the long one gave back
    eng.release("a")
    assert rel(eng.step([("b", toks[:1], [0])]), want[:1]) < 2 * tol(dtype)


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_decode_and_portions_match_whole(cuda, name, dtype):
    cfg, model = build(name, dtype, seed=3)
    prompts = {"p": tokens_for(cfg, 140, 2)}
    token_by_token = [[("p", 1)] for _ in range(140)]
    head_then_decode = [[("p", 70)]] + [[("p", 1)] for _ in range(70)]
    portions = [[("p", n)] for n in (2, 3, 2, 57, 1, 16, 17, 2, 33, 5, 2)]
    assert sum(s[0][1] for s in portions) == 140
    for schedule in (token_by_token, head_then_decode, portions):
        got = run_schedule(model, prompts, schedule, max_tokens=192, slots=1)
        check_logits(cfg, model, prompts, got, dtype)


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("name", ["odd", "aligned"])
def test_mixed_batches_reuse_pages_and_slots(cuda, name, dtype):
    """Four unequal requests share 2 slots and a pool that holds two of them: c and d run in the pages
    and slots a and b gave back; portions sit next to single tokens of the other request."""
    cfg, model = build(name, dtype, seed=4)
    prompts = {"a": tokens_for(cfg, 100, 5), "b": tokens_for(cfg, 37, 6), "c": tokens_for(cfg, 128, 7),
               "d": tokens_for(cfg, 3, 8)}
    schedule = [[("a", 30), ("b", 2)], [("a", 1), ("b", 1)], [("a", 1), ("b", 1)], [("a", 1), ("b", 1)],   # two-row
                [("a", 1), ("b", 30)], [("b", 1), ("a", 47)], [("a", 19), ("b", 1)],   # decode steps: eager, captured, replayed
                [("c", 63)], [("d", 1), ("c", 2)], [("c", 1), ("d", 2)], [("c", 62)]]
    got = run_schedule(model, prompts, schedule, max_tokens=192, slots=2)
    check_logits(cfg, model, prompts, got, dtype)
    if dtype == F32:   # batching must not change a sequence beyond rounding
        alone = run_schedule(model, {"c": prompts["c"]}, [[("c", 128)]], max_tokens=128, slots=1)
        assert rel(got["c"], alone["c"]) < 1e-5


def test_engine_refuses_what_does_not_fit(cuda):
    from vila_b200.serving import TokenEngine
    cfg, model = build("aligned", BF)
    eng = TokenEngine(model, max_tokens=128, slots=1)
    eng.step([("a", tokens_for(cfg, 100, 1), [])])
    with pytest.raises(MemoryError):
        eng.step([("b", [1, 2], [])])           # no slot
    with pytest.raises(MemoryError):
        eng.step([("a", tokens_for(cfg, 40, 2), [])])   # no page
    eng.release("a")
    assert eng.step([("b", [1, 2], [1])]).shape == (1, cfg["vocab"])


def test_long_decode_across_page_and_chunk_borders(cuda):
    """300 decoded tokens after a short prompt in fp32: k | v pages, convolution tails and recurrent states are
    carried across 300 steps (graph replays), five page borders and five chunk borders."""
    cfg, model = build("aligned", F32, seed=5)
    prompts = {"p": tokens_for(cfg, 330, 9)}
    got = run_schedule(model, prompts, [[("p", 30)]] + [[("p", 1)] for _ in range(300)], max_tokens=384, slots=1)
    check_logits(cfg, model, prompts, got, F32)


def test_sharp_attention_over_a_long_context(cuda):
    """With a large score scale the softmax of the first layer is sharp and its chunk is longer than the prompt:
    every row attends to the best-matching token among up to 700 earlier ones, most of them beyond bias_max.
    Whole prompt, decoded tail, 64-token portions."""
    cfg, rows = json.loads(json.dumps(CONFIGS["ones"]))
    cfg["layers"][0]["mixer"]["left"]["scale"] = 6.0
    cfg["layers"][0]["mixer"]["left_scale"] = 3.0
    cfg, model = build((cfg, rows), F32, seed=6)
    toks = tokens_for(cfg, 700, 11)
    for schedule in ([[("p", 700)]], [[("p", 690)]] + [[("p", 1)]] * 10, [[("p", 64)]] * 10 + [[("p", 58)], [("p", 2)]]):
        got = run_schedule(model, {"p": toks}, schedule, max_tokens=704, slots=1)
        check_logits(cfg, model, {"p": toks}, got, F32)


def test_generate_through_scheduler_matches_oracle_greedy(cuda):
    """Greedy generation through generate_tokens (continuous batching, chunked prefill, 2 slots for 3
    prompts, small step budget) against greedy decoding with the oracle."""
    from vila_b200.serving import generate_tokens
    cfg, model = build("odd", F32, seed=6)
    prompts = [tokens_for(cfg, n, 10 + n) for n in (41, 5, 70)]
    out = generate_tokens(model, prompts, max_new_tokens=12, slots=2, max_step_tokens=24)
    for p, ids in zip(prompts, out):
        want, margins = O.greedy(cfg, model.state_dict(), p, 12)
        for k, (a, b) in enumerate(zip(ids, want)):
            if margins[k] < 1e-3:
                break       # a tie in the oracle itself
            assert a == b, (k, ids, want)
    # EOS stops a request and frees its slot; sampling with a seed is reproducible
    eos = out[1][3]
    short = generate_tokens(model, prompts[1:2], max_new_tokens=12, eos_token_ids=[eos])
    assert short[0] == out[1][:out[1].index(eos) + 1]
    s1 = generate_tokens(model, prompts[:2], max_new_tokens=6, sample=True, temperature=0.9, top_k=20, top_p=0.9, seed=1)
    s2 = generate_tokens(model, prompts[:2], max_new_tokens=6, sample=True, temperature=0.9, top_k=20, top_p=0.9, seed=1)
    assert s1 == s2 and all(len(s) == 6 for s in s1)
    assert model.generate(prompts[1], max_new_tokens=12)[0] == out[1]


def test_checkpoint_round_trip_and_registry(cuda, tmp_path):
    from vila_b200.model import load_language_model
    from vila_b200.serving import TokenEngine
    cfg, model = build("aligned", BF, seed=7)
    model.save_pretrained(tmp_path / "m")
    again = load_language_model(tmp_path / "m", dtype="bfloat16")
    assert type(again) is type(model) and again.config.to_dict() == model.config.to_dict() == cfg
    toks = tokens_for(cfg, 20, 3)
    a = TokenEngine(model, 64, 1).step([("x", toks, [19])])
    b = TokenEngine(again, 64, 1).step([("x", toks, [19])])
    assert torch.equal(a, b)


def test_command_line_generates_ids(cuda, tmp_path, capsys):
    from llava.cli import infer
    cfg, model = build("ones", F32, seed=8)
    model.save_pretrained(tmp_path / "m")
    prompt = tokens_for(cfg, 9, 4)
    text = infer.main(["--model-path", str(tmp_path / "m"), "--token-ids", ",".join(map(str, prompt)),
                       "--max-new-tokens", "5", "--dtype", "float32"])
    assert [int(t) for t in text.split(",")] == model.generate(prompt, max_new_tokens=5)[0]
    assert text in capsys.readouterr().out


def test_trace_runner_replays_steps(cuda, tmp_path):
    """bin/trace_run on a saved model: three requests over two slots' worth of pages, portions beside
    single tokens, a step that wants nothing, ids released and their pages used again."""
    cfg, model = build("odd", F32, seed=9)
    model.save_pretrained(tmp_path / "m")
    p = {"a": tokens_for(cfg, 70, 1), "b": tokens_for(cfg, 9, 2), "c": tokens_for(cfg, 66, 3)}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": p["a"][:50], "want": [0, 49]}, {"id": "b", "tokens": p["b"][:2], "want": [1]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": p["b"][2:8], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": p["a"][50:51], "want": [0]}, {"id": "b", "tokens": p["b"][8:], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": p["a"][51:], "want": [18]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": p["c"], "want": [64, 65]}], "end": ["c"]},
    ]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done %d" % k for k in range(5)]
    assert not (out / "1.f32").exists()
    want = {k: O.forward(cfg, model.state_dict(), v) for k, v in p.items()}
    import numpy as np
    rows = {0: [want["a"][0], want["a"][49], want["b"][1]], 2: [want["a"][50], want["b"][8]], 3: [want["a"][69]],
            4: [want["c"][64], want["c"][65]]}
    for k, exp in rows.items():
        got = torch.from_numpy(np.fromfile(out / f"{k}.f32", dtype="<f4").reshape(len(exp), cfg["vocab"]))
        assert rel(got, torch.stack(exp)) < tol(F32), k
