"""Ludazen on the GPU against the plain float64 oracle (oracle/ludazen_oracle.py): every mechanism's kernel
alone, then whole models (own small configurations, random weights) under every way the engine can be
driven: whole prompts, token-by-token decoding, portions down to two tokens, mixed batches of unequal
requests, pages and slots that are freed and reused, long decoding, greedy generation through the
scheduler, the command line and the trace runner.  Where random weights would hide a fault (a key at a
window's edge, a kept first token, a far key) one query / key pair is scaled so that one score stands out."""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from oracle import ludazen_oracle as O

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


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


# ------------------------------------------------------------------------------------------------
# configurations (none of them a size combination of a published or given model)
# ------------------------------------------------------------------------------------------------
def att(heads, kv_heads, dim, vdim, rot_dims, base, scale, size, keep=None, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mask = {"size": size} if keep is None else {"keep_first": keep, "size": size}
    return {"type": "attention", "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=rot,
                                               scale=scale, mask=mask)}


def lat(heads, dim, rot_dim, vdim, rank, base, scale, size, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, rot={"base": base, "dims": rot_dim},
             scale=scale, mask={"size": size})
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=0):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def config(width, vocab, layers, eps=1e-5):
    return {"architecture": "Ludazen", "layers": [dict(l, mlp=m) for l, m in layers], "norm": {"eps": eps},
            "vocab": vocab, "width": width}


CONFIGS = {
    # nothing is a multiple of 8 where it need not be; a latent layer first, its rows used by a layer that is not
    # its neighbour; full multi-head, one shared key/value head; rotation of a part of the head and rescaled
    # frequencies; windows shorter and longer than a page, one without kept tokens; two and three experts
    # per token, with and without a shared expert; a layer without feed-forward
    "odd": config(72, 97, [
        (lat(3, 10, 6, 14, 20, 300.0, 0.3, 21), moe(6, 2, 20, shared=12)),
        (att(3, 3, 12, 20, 8, 100.0, 0.4, 70, keep=3, scaling=(4.0, 64, 8.0, 2.0)), dense(44)),
        (lat(2, 12, 6, 10, 20, 300.0, 0.25, 90, kv_from=0), None),
        (att(4, 1, 10, 6, 10, 10000.0, 0.3, 9), moe(5, 3, 12)),
    ], eps=1e-6),
    # sizes the tensor-core GEMM takes; a pair of query heads per key/value head; a window of one page exactly;
    # kept tokens that reach into the second page; every expert chosen
    "aligned": config(128, 256, [
        (att(8, 4, 32, 32, 16, 500000.0, 0.17, 64, keep=70), moe(8, 2, 64, shared=64)),
        (lat(4, 32, 16, 48, 64, 10000.0, 0.2, 33), dense(256)),
        (att(4, 4, 32, 64, 32, 10000.0, 0.2, 200, keep=1, scaling=(16.0, 128, 16.0, 1.0)), moe(4, 4, 32)),
        (lat(8, 16, 16, 16, 64, 10000.0, 0.2, 128, kv_from=1), dense(64)),
    ]),
    # the small ends: one head, one expert of which one is taken, a window of one token (a row sees itself only,
    # plus the kept first two), a window that no prompt here outgrows
    "plain": config(40, 61, [
        (att(1, 1, 24, 12, 12, 1000.0, 0.2, 1, keep=2), moe(1, 1, 16)),
        (lat(1, 8, 4, 8, 12, 100.0, 0.35, 1000), dense(24)),
        (att(2, 1, 8, 8, 8, 100.0, 0.35, 2), None),
    ]),
    # a width that is no multiple of 4 (no 16-byte rows anywhere)
    "narrow": config(42, 35, [
        (att(3, 1, 14, 9, 6, 300.0, 0.3, 17, keep=5), moe(6, 3, 10, shared=7)),
        (lat(2, 5, 2, 7, 9, 20.0, 0.45, 30), dense(13)),
        (lat(3, 6, 2, 3, 9, 20.0, 0.45, 5, kv_from=1), moe(2, 1, 6)),
    ]),
}


def build(name, dtype, seed=0):
    """name: a key of CONFIGS or a configuration dictionary"""
    from vila_b200.model import LudazenConfig, LudazenForCausalLM
    cfg = CONFIGS[name] if isinstance(name, str) else name
    model = LudazenForCausalLM(LudazenConfig.from_dict(cfg), "cuda", dtype).init_random(seed, scale=1.5)
    if dtype == BF:
        # Two router scores closer than the bf16 noise of the router's input would pick another expert than the
        # float64 oracle, and the changed token would then be seen by every later one.  The bf16 models get a
        # decisive router: channel 0 of the residual stream is a constant (every word row has 4 there and nothing
        # writes to it), so the normed input has a positive channel 0, and every router row reads it with its own
        # factor (0.5 apart) on top of a small random part.  The chosen set is then fixed per layer while the
        # weights still vary per token.  Routing that changes from token to token is covered by the fp32 models
        # and the router's own test.
        t = model.state_dict()
        g = torch.Generator().manual_seed(seed + 100)
        t["embed"][:, 0] = 4.0
        for n in list(t):
            if n.endswith("mix.o") or n.endswith(".down"):
                t[n][0, :] = 0.0
            elif n.endswith("down.b"):
                t[n][0] = 0.0
            elif n.endswith("mlp.router"):
                E = t[n].shape[0]
                r = t[n].float() * 0.25
                r[:, 0] = (torch.randperm(E, generator=g).float() - (E - 1) / 2.0) * 0.5
                t[n] = r.to(BF)
        model.load_weights(t)
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
    """every row within tolerance (relative to the largest entry of the expected tensor)"""
    got, want = got.double().cpu(), want.double().cpu()
    assert bool(torch.isfinite(got).all()), what
    err = (got - want).abs().amax(-1) / want.abs().max()
    bad = int((err >= tol(dtype)).sum())
    assert bad == 0, (what, bad, err.numel(), float(err.max()))


def check_logits(cfg, model, prompts, got, dtype):
    for name, toks in prompts.items():
        want = O.forward(cfg, model.state_dict(), toks)
        assert got[name].shape == want.shape
        rows_close(got[name], want, dtype, name)


# ------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("H,G,dim,vdim,rot,scaling", [(3, 3, 12, 20, 8, None), (4, 1, 10, 6, 10, (4.0, 64, 8.0, 2.0)),
                                                      (2, 2, 16, 16, 0, None), (10, 2, 64, 32, 32, (6.0, 256, 24.0, 1.5))])
def test_rotation_in_halves_with_rescaled_frequencies(cuda, dtype, H, G, dim, vdim, rot, scaling):
    """positions near 0, at a page border and far; q comes back rotated (fp32), k | v land in the named pool rows"""
    from vila_b200.model.ludazen import RotaryConfig
    ops = _ops()
    pos = [0, 1, 63, 64, 65, 1000, 54321]
    T = len(pos)
    qkv = rnd(T, H * dim + G * (dim + vdim), seed=6, scale=2.0).to(dtype)
    rows = i32([9, 3, 70, 0, 33, 12, 5])
    pool = torch.zeros(80, G * (dim + vdim), dtype=dtype, device="cuda")
    rd = {"base": 1000.0, "dims": rot}
    if scaling:
        rd["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    rc = RotaryConfig.from_dict(rd)
    if rot:
        assert torch.allclose(torch.tensor(rc.frequencies(), dtype=F64), O.rotary_frequencies(rd), rtol=1e-14)
        assert rc.magnitude == O.rotary_magnitude(rd)
    inv = torch.tensor(rc.frequencies(), dtype=F64).cuda() if rot else None
    q = ops.rope_append(qkv.cuda(), i32(pos), rows, pool, heads=H, kv_heads=G, dim=dim, vdim=vdim, inv_freq=inv,
                        unit_norm=False, eps=1e-6, halves=True, mscale=rc.magnitude)

    def turned(v, heads):   # the oracle turns by 0 .. T-1: one call per position, take the last row
        v = v.double().view(T, heads, dim)
        out = []
        for t, p in enumerate(pos):
            seq = torch.zeros(p + 1, heads, dim, dtype=F64)
            seq[p] = v[t]
            out.append(O.rotate(seq, rd, "halves")[p] if p < 2000 else None)
        return out

    qd, kd = qkv.double()[:, :H * dim], qkv.double()[:, H * dim:(H + G) * dim]
    for t, (a, b) in enumerate(zip(turned(qd, H), turned(kd, G))):
        if a is None:      # far position: same formula in float64 here (the oracle would build 54k rows)
            f, mag = O.rotary_frequencies(rd) if rot else torch.zeros(0, dtype=F64), O.rotary_magnitude(rd)
            c, s = torch.cos(pos[t] * f) * mag, torch.sin(pos[t] * f) * mag

            def one(v, heads):
                v = v.view(heads, dim).clone()
                x, y = v[:, :rot // 2].clone(), v[:, rot // 2:rot].clone()
                v[:, :rot // 2], v[:, rot // 2:rot] = x * c - y * s, y * c + x * s
                return v
            a, b = one(qd[t], H), one(kd[t], G)
        assert rel(q[t].view(H, dim), a) < 1e-5
        assert rel(pool[rows[t], :G * dim].view(G, dim), b) < (1e-5 if dtype == F32 else 1e-2)
    assert rel(pool[rows.long(), G * dim:], qkv[:, (H + G) * dim:]) < 1e-6


def windowed_attention(q, k, v, H, G, scale, size, keep, talk=None, temp=None):
    """float64, q [T, H, D] (already rotated), k [T, G, D], v [T, G, V]"""
    T = q.shape[0]
    grp = torch.arange(H) // (H // G)
    sc = torch.einsum("thd,shd->hts", q, k[:, grp]) * scale
    if temp is not None:
        sc = sc * temp[:, None, None]
    w = torch.softmax(sc.masked_fill(~O.window_mask(T, size, keep)[None], float("-inf")), -1)
    if talk is not None:
        w = torch.einsum("ab,bts->ats", talk, w)
    return torch.einsum("hts,shv->thv", w, v[:, grp]).reshape(T, -1)


def fill_pool(k, v, page, n_pages, dtype, seed=0):
    """scatter a sequence's k | v rows into shuffled pages of a pool -> (pool, page table [1, n_pages])"""
    T = k.shape[0]
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed))
    pool = torch.full((n_pages * page, k[0].numel() + v[0].numel()), 99.0, dtype=dtype)   # stale rows are garbage
    pos = torch.arange(T)
    pool[perm[pos // page] * page + pos % page] = torch.cat([k.reshape(T, -1), v.reshape(T, -1)], 1).to(dtype)
    return pool.cuda(), perm.to(torch.int32)[None].cuda()


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("H,G,dk,dv,size,keep", [(3, 3, 12, 20, 21, 3), (4, 1, 10, 6, 70, 0), (6, 2, 6, 10, 1, 2), (16, 4, 64, 64, 64, 70),
                                                 (1, 1, 130, 5, 33, 1), (40, 8, 16, 24, 100, 5), (8, 8, 32, 32, 300, 0)])
def test_windowed_attention_with_weight_mixing(cuda, dtype, H, G, dk, dv, size, keep):
    """a prompt in 16-row tiles, then single rows with the keys dealt to 1, 2 and 5 CTAs: window with kept first
    tokens, per-head temperature, weights mixed after the softmax; pages in shuffled order"""
    ops = _ops()
    T, page = 200, 64
    q, k, v = rnd(T, H, dk, seed=1), rnd(T, G, dk, seed=2).to(dtype).double(), rnd(T, G, dv, seed=3).to(dtype).double()
    talk = torch.eye(H, dtype=F64) + rnd(H, H, seed=4, scale=0.3)
    temp = 1.0 + rnd(H, seed=5, scale=0.3)
    want = windowed_attention(q.float().double(), k, v, H, G, 0.3, size, keep, talk, temp)
    pool, pt = fill_pool(k, v, page, 4, dtype)
    qf = q.float().reshape(T, -1).cuda()
    kw = dict(heads=H, kv_heads=G, dim=dk, vdim=dv, page=page, scale=0.3, talk=talk.float().cuda(), talk_after=True,
              head_scale=temp.float().cuda(), window=size, keep_first=keep, out_dtype=F32)
    tiles = i32([(o, min(16, T - o), o, 0) for o in range(0, T, 16)])
    got = ops.paged_attention(qf, pool, pt, tiles, max_rows=16, **kw)
    assert rel(got, want) < (2e-5 if dtype == F32 else 2e-2)
    ones = i32([(t, 1, t, 0) for t in range(T)])
    for ns in (1, 2, 5):
        got = ops.paged_attention(qf, pool, pt, ones, max_rows=1, nsplit=ns, **kw)
        assert rel(got, want) < (2e-5 if dtype == F32 else 2e-2), ns
    # a portion that starts in the middle (rows 37 .. 60 as tiles of 16 + 8)
    part = i32([(0, 16, 37, 0), (16, 8, 53, 0)])
    got = ops.paged_attention(qf[37:61].contiguous(), pool, pt, part, max_rows=16, **kw)
    assert rel(got, want[37:61]) < (2e-5 if dtype == F32 else 2e-2)


@pytest.mark.parametrize("decode", [False, True])
def test_window_edges_and_kept_tokens_show(cuda, decode):
    """Query 150 of a window of 40 with 4 kept tokens.  One key at a time is made to match the query strongly:
    inside the window (111, 150), among the kept ones (0, 3) the row must take that key's value; just outside
    (110, 4) or in the future (151) it must not notice it.  Also without mixing, through the K/V-head-split form."""
    ops = _ops()
    H, G, D, V, T, size, keep, page = 4, 2, 16, 8, 160, 40, 4, 64
    base_k, v = rnd(T, G, D, seed=2, scale=0.1), rnd(T, G, V, seed=3)
    q = rnd(T, H, D, seed=1, scale=0.1)
    q[150] = 0.0
    q[150, :, 0] = 6.0
    for talk in (None, torch.eye(H, dtype=F64) + rnd(H, H, seed=4, scale=0.2)):
        for j, seen in ((111, True), (150, True), (0, True), (3, True), (110, False), (4, False), (151, False), (60, False)):
            k = base_k.clone()
            k[j, :, 0] = 6.0            # score 36 * scale against ~0 elsewhere
            want = windowed_attention(q, k, v, H, G, 1.0, size, keep, talk)
            pool, pt = fill_pool(k, v, page, 3, F32, seed=j)
            kw = dict(heads=H, kv_heads=G, dim=D, vdim=V, page=page, scale=1.0, window=size, keep_first=keep, out_dtype=F32,
                      talk=None if talk is None else talk.float().cuda(), talk_after=talk is not None)
            if decode:
                got = ops.paged_attention(q[150:151].float().reshape(1, -1).cuda(), pool, pt, i32([(0, 1, 150, 0)]),
                                          max_rows=1, nsplit=3, **kw)[0]
            else:
                got = ops.paged_attention(q[144:160].float().reshape(16, -1).cuda(), pool, pt, i32([(0, 16, 144, 0)]),
                                          max_rows=16, **kw)[6]
            assert rel(got, want[150]) < 1e-5, (j, seen)
            if talk is None:
                took = rel(got.view(H, V), v[j][torch.arange(H) // (H // G)]) < 1e-3
                assert took == seen, (j, seen)


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("H,R,rot,size", [(3, 20, 6, 21), (1, 12, 4, 1000), (4, 64, 16, 33), (8, 64, 8, 128), (2, 9, 2, 1), (16, 40, 24, 64),
                                          (5, 560, 8, 70), (2, 530, 4, 40)])
def test_latent_rows_and_windowed_latent_attention(cuda, dtype, H, R, rot, size):
    """cache rows (normed latent | rotated key part) and folded queries from latent_rope_append, then the windowed
    attention over them in tiles and as single rows with split keys, against separate keys and values in float64"""
    ops = _ops()
    T, page, D, V = 150, 64, 10, 14
    qh = D + rot
    rd = {"base": 300.0, "dims": rot}
    m = dict(heads=H, dim=D, rot_dim=rot, vdim=V, kv_rank=R, rot=rd, scale=0.3, mask={"size": size})
    W = {"q": rnd(H * qh, 32, seed=1, scale=0.3), "dkv": rnd(R + rot, 32, seed=2, scale=0.3), "dkv.norm": 1 + rnd(R, seed=3, scale=0.1),
         "uk": rnd(H * D, R, seed=4, scale=0.3).to(dtype).double(), "uv": rnd(H * V, R, seed=5, scale=0.3).to(dtype).double(),
         "o": torch.eye(H * V, dtype=F64)}
    h = rnd(T, 32, seed=6)
    qp, kvp = (h @ W["q"].T).to(dtype), (h @ W["dkv"].T).to(dtype)
    # the oracle from the same (rounded) projections: make them reproduce with h = identity-like inputs
    Wq = {"q": torch.eye(H * qh, dtype=F64), "dkv": torch.eye(R + rot, dtype=F64), "dkv.norm": W["dkv.norm"], "uk": W["uk"],
          "uv": W["uv"], "o": W["o"]}
    c, kr = O.latent_rows({"dkv": Wq["dkv"], "dkv.norm": Wq["dkv.norm"]}, "", kvp.double(), m, 1e-6)
    perm = torch.randperm(3, generator=torch.Generator().manual_seed(1))
    pos = torch.arange(T)
    rows = (perm[pos // page] * page + pos % page).to(torch.int32).cuda()
    pool = torch.full((3 * page, R + rot), 77.0, dtype=dtype, device="cuda")
    qa = torch.zeros(T, H * (R + rot), dtype=F32, device="cuda")
    uk_t = W["uk"].view(H, D, R).transpose(1, 2).contiguous().to(dtype).cuda()
    ops.glinear(qp.cuda(), uk_t, groups=H, a_group_off=qh, o_group_off=R + rot, out=qa)
    inv = O.rotary_frequencies(rd).cuda()
    ops.latent_rope_append(i32(pos.tolist()), inv, rank=R, kv=kvp.cuda(), norm_w=W["dkv.norm"].float().cuda(), eps=1e-6, pool=pool,
                           cache_rows=rows, q=qp.cuda(), qa=qa, heads=H, q_head=qh, q_off=D)
    assert rel(pool[rows.long(), :R], c) < (1e-5 if dtype == F32 else 1e-2)
    assert rel(pool[rows.long(), R:], kr) < (1e-5 if dtype == F32 else 1e-2)
    # expected output from what the pool really holds (so the comparison is about the attention, not the rounding of rows)
    c2, kr2 = pool[rows.long(), :R].double().cpu(), pool[rows.long(), R:].double().cpu()
    want = O.latent_attention({"q": Wq["q"], "uk": W["uk"], "uv": W["uv"], "o": W["o"]}, "", qp.double(), m, c2, kr2)
    pt = perm.to(torch.int32)[None].cuda()
    uv = W["uv"].view(H, V, R).to(dtype).cuda()
    lim = 2e-5 if dtype == F32 else 2e-2
    tiles = i32([(o, min(16, T - o), o, 0) for o in range(0, T, 16)])
    ol = ops.latent_attention(qa, pool, pt, tiles, heads=H, page=page, scale=0.3, window=size, out_dtype=F32)
    got = ops.glinear(ol.to(dtype), uv, groups=H, a_group_off=R + rot, o_group_off=V, out_dtype=F32)
    assert rel(got, want) < lim
    ones = i32([(t, 1, t, 0) for t in range(T)])
    for ns in (1, 3):
        ol = ops.latent_attention(qa, pool, pt, ones, heads=H, page=page, scale=0.3, window=size, decode=True, nsplit=ns, out_dtype=F32)
        got = ops.glinear(ol.to(dtype), uv, groups=H, a_group_off=R + rot, o_group_off=V, out_dtype=F32)
        assert rel(got, want) < lim, ns


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("H", [2, 5])
def test_latent_window_edge_shows(cuda, decode, H):
    """query 100 with a window of 37: a cached row that matches its folded query strongly is taken at positions 64
    and 100 and not noticed at 63 and 101 (H = 2 takes the one-row kernel when decoding, H = 5 the head-rows one)"""
    ops = _ops()
    R, T, size, page = 12, 112, 37, 64
    base = rnd(T, R, seed=1, scale=0.1)
    qa = torch.zeros(T, H * R, dtype=F64)
    qa[:, 0::R] = 5.0
    for j, seen in ((64, True), (100, True), (63, False), (101, False), (3, False)):
        c = base.clone()
        c[j, 0] = 5.0
        sc = torch.einsum("thr,sr->hts", qa.view(T, H, R), c)
        w = torch.softmax(sc.masked_fill(~O.window_mask(T, size)[None], float("-inf")), -1)
        want = torch.einsum("hts,sr->thr", w, c).reshape(T, -1)
        pool, pt = c.float().cuda(), i32([[0, 1]])
        if decode:
            got = ops.latent_attention(qa[100:101].float().cuda(), pool, pt, i32([(0, 1, 100, 0)]), heads=H, page=page,
                                       scale=1.0, window=size, decode=True, nsplit=2, out_dtype=F32)[0]
        else:
            got = ops.latent_attention(qa[96:112].float().cuda(), pool, pt, i32([(0, 16, 96, 0)]), heads=H, page=page,
                                       scale=1.0, window=size, out_dtype=F32)[4]
        assert rel(got, want[100]) < 1e-5, (j, seen)
        assert (rel(got.view(H, R)[0], c[j]) < 1e-3) == seen, (j, seen)


@pytest.mark.parametrize("dtype", [F32, BF])
@pytest.mark.parametrize("M", [3, 40, 300])
def test_xielu_layer_and_input_weighted_experts(cuda, dtype, M):
    ops = _ops()
    K, ff, E, top = 48, 20, 5, 2
    x = rnd(M, K, seed=1).to(dtype)
    # dense layer with biases and the two-sided activation; the padded tensor-core form and the grouped form
    up, ub = rnd(24, K, seed=2, scale=0.3).to(dtype), rnd(24, seed=3, scale=0.3).to(dtype)
    for p, q in ((0.3, -0.7), (-2.0, 1.5)):
        ap, an = math.log1p(math.exp(p)), 0.5 + math.log1p(math.exp(q))
        want = O.xielu(x.double() @ up.double().T + ub.double(), p, q)
        got = ops.linear_any(x.cuda(), up.cuda(), bias=ub.cuda(), act=ops.ACT_XIELU, act_params=(ap, an))
        assert rel(got, want) < (1e-5 if dtype == F32 else 2e-2)
        got = ops.glinear(x.cuda(), up.cuda(), bias=ub.cuda(), act=ops.ACT_XIELU, act_params=(ap, an), out_dtype=F32)
        assert rel(got, want) < (1e-5 if dtype == F32 else 1e-2)
    # experts whose INPUT is scaled by the routing weight: silu(w g) * (w u), not w * silu(g) * u
    W = {"router": rnd(E, K, seed=4, scale=0.5)}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"] = rnd(ff, K, seed=10 + e, scale=0.4).to(dtype).double(), rnd(ff, K, seed=20 + e, scale=0.4).to(dtype).double()
        W[f"e{e}.down"] = rnd(K, ff, seed=30 + e, scale=0.4).to(dtype).double()
    idx, wt = ops.moe_route_sigmoid(x.cuda(), W["router"].float().cuda(), None, top)
    oidx, owt = O.route(W, "", x.double(), top)
    assert torch.equal(idx.cpu().long(), oidx) and rel(wt, owt) < 1e-5
    gu = torch.empty(E, 2 * ff, K, dtype=dtype)
    for e in range(E):
        gu[e, 0::2], gu[e, 1::2] = W[f"e{e}.gate"].to(dtype), W[f"e{e}.up"].to(dtype)
    down = torch.stack([W[f"e{e}.down"] for e in range(E)]).to(dtype)
    seg, srt = ops.moe_group(idx, E)
    act = ops.glinear(x.cuda(), gu.cuda(), groups=E, seg=seg, a_rows=srt, a_row_div=top, swiglu=True, in_scale=wt.view(-1))
    parts = ops.glinear(act, down.cuda(), groups=E, seg=seg, o_rows=srt, out_dtype=F32, out_rows_total=M * top)
    got = parts.view(M, top, K).sum(1)
    want = O.expert_ff(W, "", x.double(), {"router": {"top": top}})
    assert rel(got, want) < (2e-5 if dtype == F32 else 3e-2)
    wrong = sum(owt[:, j:j + 1] * torch.stack([O.gated_unit(W, f"e{int(e)}.", x[t:t + 1].double())[0] for t, e in enumerate(oidx[:, j])])
                for j in range(top))
    assert rel(wrong, want) > 10 * rel(got, want)      # the weight on the output is a different function


def test_residual_sum_with_following_norm(cuda):
    ops = _ops()
    for rows, cols, np_ in ((9, 20, 1), (70, 1100, 3), (1, 7, 2)):
        x0, a, part, w = rnd(rows, cols, seed=1), rnd(rows, cols, seed=2).to(BF), rnd(rows * np_, cols, seed=3), 1 + rnd(cols, seed=4, scale=0.2)
        x = x0.float().cuda()
        h = ops.residual_norm_rows(x, a.cuda(), w.float().cuda(), 1e-5, part=part.float().cuda(), n_partials=np_, out_dtype=F32)
        s = x0 + a.double() + part.view(rows, np_, cols).sum(1)
        assert rel(x, s) < 1e-6 and rel(h, O.unit(s, 1e-5) * w) < 1e-5


# ------------------------------------------------------------------------------------------------
# whole models through the engine
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
    cfg, model = build("plain", BF)
    eng = TokenEngine(model, max_tokens=128, slots=1)
    eng.step([("a", tokens_for(cfg, 100, 1), [])])
    with pytest.raises(MemoryError):
        eng.step([("b", [1, 2], [])])           # no slot
    with pytest.raises(MemoryError):
        eng.step([("a", tokens_for(cfg, 40, 2), [])])   # no page
    eng.release("a")
    assert eng.step([("b", [1, 2], [1])]).shape == (1, cfg["vocab"])


def test_long_decode_past_every_window(cuda):
    """300 decoded tokens after a short prompt in fp32: every window (9 .. 200 positions) passes over decoded
    tokens, kept first tokens stay in sight, across 300 steps (graph replays) and five page borders."""
    cfg, model = build("aligned", F32, seed=5)
    prompts = {"p": tokens_for(cfg, 330, 9)}
    got = run_schedule(model, prompts, [[("p", 30)]] + [[("p", 1)] for _ in range(300)], max_tokens=384, slots=1)
    check_logits(cfg, model, prompts, got, F32)


def test_sharp_attention_over_a_long_context(cuda):
    """With a large score scale the softmax is sharp: every row attends to the one best-matching token its mask
    lets it see (a window of 500 with 30 kept tokens; a latent window of 300), so a far key that is missed, a
    key just outside that is taken, or a kept token that is lost changes the logits.  Whole prompt, decoded
    tail, 64-token portions."""
    cfg = config(40, 61, [
        (att(2, 1, 8, 8, 8, 100.0, 1.5, 500, keep=30), dense(24)),
        (lat(2, 8, 4, 8, 12, 100.0, 1.5, 300), None),
    ])
    cfg, model = build(cfg, F32, seed=6)
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
        seq = list(p)
        for k, a in enumerate(ids):
            lg = O.forward(cfg, model.state_dict(), seq)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) < 1e-3:
                break       # a tie in the oracle itself
            assert a == int(lg.argmax()), (k, ids)
            seq.append(a)
    # EOS stops a request and frees its slot; sampling with a seed is reproducible
    eos = out[1][3]
    short = generate_tokens(model, prompts[1:2], max_new_tokens=12, eos_token_ids=[eos])
    assert short[0] == out[1][:out[1].index(eos) + 1]
    s1 = generate_tokens(model, prompts[:2], max_new_tokens=6, sample=True, temperature=0.9, top_k=20, top_p=0.9, seed=1)
    s2 = generate_tokens(model, prompts[:2], max_new_tokens=6, sample=True, temperature=0.9, top_k=20, top_p=0.9, seed=1)
    assert s1 == s2 and all(len(s) == 6 for s in s1)


def test_checkpoint_round_trip_and_registry(cuda, tmp_path):
    from vila_b200.model import load_language_model
    from vila_b200.serving import TokenEngine
    cfg, model = build("narrow", BF, seed=7)
    model.save_pretrained(tmp_path / "m")
    again = load_language_model(tmp_path / "m", dtype="bfloat16")
    assert type(again) is type(model) and again.config.to_dict() == model.config.to_dict()
    toks = tokens_for(cfg, 20, 3)
    a = TokenEngine(model, 64, 1).step([("x", toks, [19])])
    b = TokenEngine(again, 64, 1).step([("x", toks, [19])])
    assert torch.equal(a, b)


def test_command_line_generates_ids(cuda, tmp_path, capsys):
    from llava.cli import infer
    cfg, model = build("plain", F32, seed=8)
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
