"""Tensor-level wrappers over the C-ABI (include/vila_b200.h).

PyTorch is used only for device memory (torch.empty), the current CUDA stream and dtype bookkeeping;
every operation below is one call into libvila_b200.so.  No function here has an eager fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import DecodeAttnParams, DecodeAttnSplitParams, FmhaParams, GemvParams, check

ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF, ACT_SILU = 0, 1, 2, 3


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _chk(t: torch.Tensor, name: str, dtype=torch.bfloat16) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"vila_b200.ops: {name} must be a CUDA tensor (no CPU fallback exists)")
    if t.dtype != dtype:
        raise RuntimeError(f"vila_b200.ops: {name} must be {dtype}, got {t.dtype}")


_WORKSPACE = {}


def ensure_workspace(device, nbytes: int = 96 << 20) -> torch.Tensor:
    """Allocate (once per device) and register the zero-initialised stream-K scratch."""
    key = torch.device(device).index or 0
    ws = _WORKSPACE.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _WORKSPACE[key] = ws
    check(_lib.load().vila_set_workspace(ws.data_ptr(), ws.numel()), "vila_set_workspace")
    return ws


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
           act: int = ACT_NONE, residual: Optional[torch.Tensor] = None, res_row_mod: int = 0,
           swiglu: bool = False, out: Optional[torch.Tensor] = None,
           block_n: Optional[int] = None, static_w: bool = False,
           act_params: Optional[Tuple[float, float]] = None) -> torch.Tensor:
    """out = epilogue(x @ w.T).  x [M,K] (row stride arbitrary), w [N,K].
    static_w: w is a parameter (VILA_FLAG_STATIC_W): it may be fetched before the PDL wait.
    act_params: the two coefficients of ACT_XIELU (positive side, negative side)."""
    _chk(x, "x"); _chk(w, "w")
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], (x.shape, w.shape)
    assert x.stride(1) == 1 and w.stride(1) == 1
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    else:
        assert out.shape == (M, n_out) and out.stride(1) == 1
    if M == 0:
        return out
    ld_res = 0
    if residual is not None:
        _chk(residual, "residual")
        assert residual.dim() == 2 and residual.stride(1) == 1 and residual.shape[1] == N
        ld_res = residual.stride(0)
    lib = _lib.load()
    args = (_p(x), x.stride(0), _p(w), w.stride(0), _p(bias), _p(residual), ld_res, res_row_mod,
            _p(out), out.stride(0), M, N, K, act, (1 if swiglu else 0) | (2 if static_w else 0), _stream())
    if act_params is not None:
        assert residual is None and block_n is None
        check(lib.vila_linear_act(_p(x), x.stride(0), _p(w), w.stride(0), _p(bias), _p(out), out.stride(0), M, N, K,
                                  act, float(act_params[0]), float(act_params[1]),
                                  (1 if swiglu else 0) | (2 if static_w else 0), _stream()), "vila_linear_act")
    elif block_n is None:
        check(lib.vila_linear(*args), "vila_linear")
    else:
        check(lib.vila_linear_cfg(block_n, *args), "vila_linear_cfg")
    return out


def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    _chk(x, "x")
    cols = x.shape[-1]
    x2 = x.reshape(-1, cols)
    assert x2.is_contiguous()
    out = torch.empty_like(x2)
    check(_lib.load().vila_layernorm(_p(x2), _p(w), _p(b), _p(out), x2.shape[0], cols, eps,
                                     _stream()), "vila_layernorm")
    return out.view(x.shape)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float,
            residual_add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Qwen2RMSNorm.  With residual_add: x += residual_add (in place) before normalising."""
    _chk(x, "x")
    cols = x.shape[-1]
    x2 = x.view(-1, cols)
    assert x2.is_contiguous()
    out = torch.empty_like(x2)
    check(_lib.load().vila_rmsnorm(_p(x2), _p(residual_add), _p(w), _p(out), x2.shape[0], cols,
                                   eps, _stream()), "vila_rmsnorm")
    return out.view(x.shape)


def fmha(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, B: int, Sq: int, Sk: int,
         causal: bool, scale: float, out: Optional[torch.Tensor] = None,
         page_table: Optional[torch.Tensor] = None, variant: int = 0) -> torch.Tensor:
    """q [B*Sq, Hq, D] view; k/v either [B*Sk, Hkv, D] views or paged pools [P, 128, Hkv, D].
    variant (test hook, vila_fmha_cfg): 0 heuristic, 1 one-tile kernel, 2 two-tile kernel."""
    _chk(q, "q"); _chk(k, "k"); _chk(v, "v")
    assert q.dim() == 3 and q.stride(2) == 1
    Hq, D = q.shape[1], q.shape[2]
    if out is None:
        out = torch.empty((B * Sq, Hq, D), dtype=torch.bfloat16, device=q.device)
    p = FmhaParams()
    p.q, p.q_tok_stride, p.q_head_stride = q.data_ptr(), q.stride(0), q.stride(1)
    p.k, p.v = k.data_ptr(), v.data_ptr()
    if k.dim() == 4:  # paged [P, 128, Hkv, D]
        assert k.shape[1] == 128 and k.stride() == v.stride() and k.stride(3) == 1
        Hkv = k.shape[2]
        p.kv_page_stride, p.kv_tok_stride, p.kv_head_stride = k.stride(0), k.stride(1), k.stride(2)
        p.kv_num_pages = k.shape[0]
        if page_table is not None:
            assert page_table.dtype == torch.int32 and page_table.is_cuda
            pt = page_table.view(B, -1)
            p.page_table, p.page_table_stride = pt.data_ptr(), pt.stride(0)
        else:
            assert B == 1
            p.page_table, p.page_table_stride = None, 0
    else:
        assert k.dim() == 3 and k.stride() == v.stride() and k.stride(2) == 1
        Hkv = k.shape[1]
        p.kv_page_stride, p.kv_tok_stride, p.kv_head_stride = 0, k.stride(0), k.stride(1)
        p.kv_num_pages = 0
        p.page_table, p.page_table_stride = None, 0
    p.o, p.o_tok_stride, p.o_head_stride = out.data_ptr(), out.stride(0), out.stride(1)
    p.B, p.Sq, p.Sk, p.Hq, p.Hkv, p.D = B, Sq, Sk, Hq, Hkv, D
    p.causal = 1 if causal else 0
    p.scale = scale
    if variant == 0:
        check(_lib.load().vila_fmha(C.byref(p), _stream()), "vila_fmha")
    else:
        check(_lib.load().vila_fmha_cfg(variant, C.byref(p), _stream()), "vila_fmha_cfg")
    return out


def patch_im2col(pixels: torch.Tensor, patch: int, k_pad: int) -> torch.Tensor:
    _chk(pixels, "pixels")
    assert pixels.is_contiguous() and pixels.dim() == 4
    B, Cc, H, W = pixels.shape
    out = torch.empty((B * (H // patch) * (W // patch), k_pad), dtype=torch.bfloat16,
                      device=pixels.device)
    check(_lib.load().vila_patch_im2col(_p(pixels), _p(out), B, Cc, H, W, patch, k_pad, _stream()),
          "vila_patch_im2col")
    return out


_COEFF_CACHE = {}


def _bicubic_tables(in_size: int, out_size: int, device):
    key = (in_size, out_size, str(device))
    ent = _COEFF_CACHE.get(key)
    if ent is None:
        from .model.media import bicubic_coeffs
        ksize, bounds, coeffs = bicubic_coeffs(in_size, out_size)
        if len(_COEFF_CACHE) > 64:
            _COEFF_CACHE.clear()
        ent = (ksize, bounds.to(device), coeffs.to(device))
        _COEFF_CACHE[key] = ent
    return ent


def resize_bicubic_tiles(src: torch.Tensor, out_w: int, out_h: int, out: torch.Tensor, tile: int,
                         tile_index0: int, mean: float, std: float) -> torch.Tensor:
    """src uint8 [H, W, 3] (device) -> PIL-exact bicubic resize to (out_w, out_h), rescale, normalise,
    cut into tile x tile blocks written to out[tile_index0 ...] (bf16 [n, 3, tile, tile])."""
    _chk(src, "src", torch.uint8); _chk(out, "out")
    assert src.dim() == 3 and src.shape[2] == 3 and src.is_contiguous() and out.is_contiguous()
    H, W = int(src.shape[0]), int(src.shape[1])
    n = (out_w // tile) * (out_h // tile)
    assert out.shape[1:] == (3, tile, tile) and tile_index0 + n <= out.shape[0]
    kx, bx, cx = _bicubic_tables(W, out_w, src.device)
    ky, by, cy = _bicubic_tables(H, out_h, src.device)
    tmp = torch.empty((H, out_w, 3), dtype=torch.uint8, device=src.device)
    check(_lib.load().vila_resize_bicubic_tiles(_p(src), H, W, out_w, out_h, _p(cx), _p(bx), kx, _p(cy),
                                                _p(by), ky, _p(tmp), _p(out), tile, tile_index0, mean,
                                                std, _stream()), "vila_resize_bicubic_tiles")
    return out


def space_to_depth(x: torch.Tensor, h: int, w: int, r: int) -> torch.Tensor:
    """x [B, h*w, C] -> [B, ceil(h/r)*ceil(w/r), r*r*C]"""
    _chk(x, "x")
    assert x.is_contiguous() and x.dim() == 3 and x.shape[1] == h * w
    B, _, Cc = x.shape
    ho, wo = (h + r - 1) // r, (w + r - 1) // r
    out = torch.empty((B, ho * wo, r * r * Cc), dtype=torch.bfloat16, device=x.device)
    check(_lib.load().vila_space_to_depth(_p(x), _p(out), B, h, w, Cc, r, _stream()),
          "vila_space_to_depth")
    return out


def s2_merge(tiles: torch.Tensor, splits_h: Sequence[int], splits_w: Sequence[int], out_bh: int,
             out_bw: int, share_tile: bool = False) -> torch.Tensor:
    """tiles [n_tiles, side*side, C] of ONE image -> [out_bh*out_bw, side*side, n_scales*C]"""
    _chk(tiles, "tiles")
    assert tiles.is_contiguous() and tiles.dim() == 3
    n, N, Cc = tiles.shape
    side = int(round(N ** 0.5))
    ns = len(splits_h)
    out = torch.empty((out_bh * out_bw, N, ns * Cc), dtype=torch.bfloat16, device=tiles.device)
    sh = (C.c_int * ns)(*splits_h)
    sw = (C.c_int * ns)(*splits_w)
    check(_lib.load().vila_s2_merge(_p(tiles), _p(out), side, Cc, ns, sh, sw, out_bh, out_bw,
                                    1 if share_tile else 0, _stream()), "vila_s2_merge")
    return out


def chessboard_merge(tiles: torch.Tensor, bh: int, bw: int) -> torch.Tensor:
    """[bh*bw, s*s, C] -> [(bh*s)*(bw*s), C]"""
    _chk(tiles, "tiles")
    assert tiles.is_contiguous() and tiles.shape[0] == bh * bw
    _, N, Cc = tiles.shape
    s = int(round(N ** 0.5))
    out = torch.empty((bh * s * bw * s, Cc), dtype=torch.bfloat16, device=tiles.device)
    check(_lib.load().vila_chessboard_merge(_p(tiles), _p(out), bh, bw, s, Cc, _stream()),
          "vila_chessboard_merge")
    return out


def tsp_pool(x: torch.Tensor, pt: int, ph: int, pw: int) -> torch.Tensor:
    """x [T, h, w, C] -> [T/pt, h/ph, w/pw, C]"""
    _chk(x, "x")
    assert x.is_contiguous() and x.dim() == 4
    T, h, w, Cc = x.shape
    out = torch.empty((T // pt, h // ph, w // pw, Cc), dtype=torch.bfloat16, device=x.device)
    check(_lib.load().vila_tsp_pool(_p(x), _p(out), T, h, w, Cc, pt, ph, pw, _stream()),
          "vila_tsp_pool")
    return out


def embed_splice(table: torch.Tensor, media: Optional[torch.Tensor], src: torch.Tensor) -> torch.Tensor:
    _chk(table, "table")
    assert src.dtype == torch.int32 and src.is_cuda and table.is_contiguous()
    if media is not None:
        assert media.is_contiguous() and media.shape[-1] == table.shape[1]
    rows, cols = src.numel(), table.shape[1]
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device=table.device)
    check(_lib.load().vila_embed_splice(_p(table), _p(media), _p(src), _p(out), rows, cols,
                                        _stream()), "vila_embed_splice")
    return out


def rope_kv_append(qkv: torch.Tensor, positions: torch.Tensor, Hq: int, Hkv: int, D: int,
                   inv_freq: torch.Tensor, k_pool: Optional[torch.Tensor] = None,
                   v_pool: Optional[torch.Tensor] = None, page_table: Optional[torch.Tensor] = None,
                   cache_pos0: int = 0) -> None:
    _chk(qkv, "qkv")
    assert qkv.is_contiguous() and qkv.shape[-1] == (Hq + 2 * Hkv) * D
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32
    S = qkv.shape[0]
    check(_lib.load().vila_rope_kv_append(_p(qkv), _p(positions), S, Hq, Hkv, D, _p(inv_freq),
                                          _p(k_pool), _p(v_pool), _p(page_table), cache_pos0,
                                          _stream()), "vila_rope_kv_append")


def rope_kv_append_table(qkv: torch.Tensor, table: torch.Tensor, Hq: int, Hkv: int, D: int,
                         k_pool: Optional[torch.Tensor] = None, v_pool: Optional[torch.Tensor] = None,
                         page_table: Optional[torch.Tensor] = None, cache_pos0: int = 0) -> None:
    """rope_kv_append with the cos | sin table of rope_table(positions) (long prefills)."""
    _chk(qkv, "qkv"); _chk(table, "table")
    assert qkv.is_contiguous() and qkv.shape[-1] == (Hq + 2 * Hkv) * D
    S = qkv.shape[0]
    assert table.shape == (S, D) and table.is_contiguous()
    check(_lib.load().vila_rope_kv_append_table(_p(qkv), _p(table), S, Hq, Hkv, D, _p(k_pool), _p(v_pool),
                                                _p(page_table), cache_pos0, _stream()),
          "vila_rope_kv_append_table")


def rope_table(positions: torch.Tensor, D: int, inv_freq: torch.Tensor) -> torch.Tensor:
    """cos | sin table [S, D] bf16 of a request's positions (shared by all layers and heads)."""
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32 and positions.is_cuda
    S = positions.numel()
    table = torch.empty((S, D), dtype=torch.bfloat16, device=positions.device)
    check(_lib.load().vila_rope_table(_p(positions), S, D, _p(inv_freq), _p(table), _stream()),
          "vila_rope_table")
    return table


def linear_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                    table: torch.Tensor, Hq: int, Hkv: int, D: int,
                    k_pool: Optional[torch.Tensor] = None, v_pool: Optional[torch.Tensor] = None,
                    page_table: Optional[torch.Tensor] = None, cache_pos0: int = 0,
                    static_w: bool = False) -> Optional[torch.Tensor]:
    """q/k/v projection + RoPE + KV-cache append in one kernel (short prefill chunks: M <= 384,
    head_dim 128; table = rope_table(positions)).  Returns qkv [M, (Hq+2Hkv)*D] whose q heads are
    rotated (k / v heads live in the pools when given), or None when the shape is not covered
    (caller: linear + rope_kv_append)."""
    _chk(x, "x"); _chk(w, "w")
    M, K = x.shape
    N = (Hq + 2 * Hkv) * D
    if D != 128 or M > 384 or M == 0:
        return None
    assert w.shape == (N, K) and x.stride(1) == 1 and w.stride(1) == 1
    assert table.shape == (M, D) and table.dtype == torch.bfloat16 and table.is_contiguous()
    ensure_workspace(x.device)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    rc = _lib.load().vila_linear_qkv_rope(_p(x), x.stride(0), _p(w), w.stride(0), _p(bias), _p(out),
                                          out.stride(0), M, K, Hq, Hkv, D, _p(table),
                                          _p(k_pool), _p(v_pool), _p(page_table), cache_pos0,
                                          2 if static_w else 0, _stream())
    if rc == 3:
        return None
    check(rc, "vila_linear_qkv_rope")
    return out


def gemv(x: torch.Tensor, w: torch.Tensor, *, bias=None, norm_w=None, norm_eps: float = 1e-6,
         residual=None, swiglu: bool = False, out: Optional[torch.Tensor] = None,
         argmax_key: Optional[torch.Tensor] = None, write_out: bool = True,
         static_w: bool = False, variant: int = 0) -> Optional[torch.Tensor]:
    _chk(x, "x"); _chk(w, "w")
    N, K = w.shape
    assert x.numel() == K and w.is_contiguous()
    if out is None and write_out:
        out = torch.empty((N // 2 if swiglu else N,), dtype=torch.bfloat16, device=x.device)
    p = GemvParams()
    p.x, p.w, p.bias, p.norm_w = _p(x), _p(w), _p(bias), _p(norm_w)
    p.norm_eps = norm_eps
    p.residual, p.y = _p(residual), _p(out)
    p.N, p.K, p.flags = N, K, (1 if swiglu else 0) | (2 if static_w else 0) | (4 if variant == 1 else 0)
    p.argmax_key = _p(argmax_key)
    check(_lib.load().vila_gemv(C.byref(p), _stream()), "vila_gemv")
    return out


def argmax_finalize(key: torch.Tensor, token_out: torch.Tensor, token_hist=None, step_counter=None,
                    position=None, embed_table=None, x_next=None) -> None:
    hidden = embed_table.shape[1] if embed_table is not None else 0
    check(_lib.load().vila_argmax_finalize(_p(key), _p(token_out), _p(token_hist),
                                           _p(step_counter), _p(position), _p(embed_table),
                                           _p(x_next), hidden, _stream()), "vila_argmax_finalize")


def decode_attention(qkv: torch.Tensor, position: torch.Tensor, k_pool: torch.Tensor,
                     v_pool: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor,
                     ws: torch.Tensor, counters: torch.Tensor, inv_freq: torch.Tensor, Hq: int,
                     Hkv: int, D: int, num_splits: int, scale: float) -> None:
    p = DecodeAttnParams()
    p.qkv, p.position, p.k_pool, p.v_pool = _p(qkv), _p(position), _p(k_pool), _p(v_pool)
    p.page_table, p.out, p.ws, p.counters = _p(page_table), _p(out), _p(ws), _p(counters)
    p.inv_freq = _p(inv_freq)
    p.Hq, p.Hkv, p.D, p.num_splits, p.scale = Hq, Hkv, D, num_splits, scale
    check(_lib.load().vila_decode_attention(C.byref(p), _stream()), "vila_decode_attention")


def decode_attention_split(qkv: torch.Tensor, position: torch.Tensor, k_pool: torch.Tensor,
                           v_pool: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor,
                           o_partial: torch.Tensor, lse: torch.Tensor, inv_freq: torch.Tensor, Hq: int,
                           Hkv: int, D: int, num_splits: int, split_tokens: int, scale: float,
                           counters: Optional[torch.Tensor] = None) -> None:
    """Long-context decode attention: RoPE + KV append, tcgen05 FMHA in split-KV mode, combine
    (counters int32 [Hkv], zeroed once: the combine is fused into the split kernel)."""
    assert o_partial.dtype == torch.float32 and o_partial.numel() >= num_splits * Hq * D
    assert lse.dtype == torch.float32 and lse.numel() >= num_splits * Hq
    p = DecodeAttnSplitParams()
    p.qkv, p.position, p.k_pool, p.v_pool = _p(qkv), _p(position), _p(k_pool), _p(v_pool)
    p.page_table, p.kv_num_pages, p.out = _p(page_table), k_pool.shape[0], _p(out)
    p.o_partial, p.lse, p.inv_freq = _p(o_partial), _p(lse), _p(inv_freq)
    p.counters = _p(counters)
    p.Hq, p.Hkv, p.D, p.num_splits, p.split_tokens, p.scale = Hq, Hkv, D, num_splits, split_tokens, scale
    check(_lib.load().vila_decode_attention_split(C.byref(p), _stream()), "vila_decode_attention_split")


def decode_attention_batch(qkv: torch.Tensor, positions: torch.Tensor, k_pool: torch.Tensor,
                           v_pool: torch.Tensor, page_tables: torch.Tensor, out: torch.Tensor,
                           inv_freq: torch.Tensor, Hq: int, Hkv: int, D: int, scale: float) -> None:
    """qkv [B, (Hq+2Hkv)*D], positions int32 [B] (< 0: idle slot), page_tables int32 [B, max_pages],
    out [B, Hq*D]; one shared paged pool [P, 128, Hkv, D]."""
    _chk(qkv, "qkv"); _chk(out, "out")
    B = qkv.shape[0]
    assert qkv.dim() == 2 and out.shape == (B, Hq * D) and qkv.stride(1) == 1 and out.stride(1) == 1
    assert positions.dtype == torch.int32 and positions.numel() == B and positions.is_contiguous()
    assert page_tables.dtype == torch.int32 and page_tables.dim() == 2 and page_tables.shape[0] == B
    p = DecodeAttnParams()
    p.qkv, p.position, p.k_pool, p.v_pool = _p(qkv), _p(positions), _p(k_pool), _p(v_pool)
    p.page_table, p.out, p.ws, p.counters = _p(page_tables), _p(out), None, None
    p.inv_freq = _p(inv_freq)
    p.Hq, p.Hkv, p.D, p.num_splits, p.scale = Hq, Hkv, D, 0, scale
    check(_lib.load().vila_decode_attention_batch(C.byref(p), B, qkv.stride(0), out.stride(0),
                                                  page_tables.stride(0), min(32, page_tables.shape[1]),
                                                  _stream()), "vila_decode_attention_batch")


# ---- ragged-batch language-model blocks (fp32 residual stream) -------------------------------------
DT_BF16, DT_F32 = 0, 1
ACT_RELU2 = 4
ACT_XIELU = 5   # z > 0: a_pos z^2 + z / 2;  z <= 0: a_neg (e^z - 1 - z) + z / 2  (act_params = (a_pos, a_neg))
_DT = {torch.bfloat16: DT_BF16, torch.float32: DT_F32}


def _dt(t: torch.Tensor, name: str) -> int:
    if not t.is_cuda:
        raise RuntimeError(f"vila_b200.ops: {name} must be a CUDA tensor (no CPU fallback exists)")
    if t.dtype not in _DT:
        raise RuntimeError(f"vila_b200.ops: {name} must be bfloat16 or float32, got {t.dtype}")
    return _DT[t.dtype]


def _i32(t: Optional[torch.Tensor], name: str) -> Optional[int]:
    if t is None:
        return None
    assert t.is_cuda and t.dtype == torch.int32 and t.is_contiguous(), name
    return t.data_ptr()


def _f32(t: Optional[torch.Tensor], name: str) -> Optional[int]:
    if t is None:
        return None
    assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous(), name
    return t.data_ptr()


def embed_rows(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """fp32 rows table[ids] (ids int32 [T])."""
    out = torch.empty(ids.numel(), table.shape[1], dtype=torch.float32, device=table.device)
    check(_lib.load().vila_embed_rows(_p(table), _dt(table, "table"), _i32(ids, "ids"), _p(out),
                                      ids.numel(), table.shape[1], _stream()), "vila_embed_rows")
    return out


def rmsnorm_rows(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, *, w_offset: float = 0.0,
                 out: Optional[torch.Tensor] = None, out_dtype=None,
                 out_rows: Optional[torch.Tensor] = None, groups: int = 1) -> torch.Tensor:
    """x [rows, cols] (row stride arbitrary) -> x / sqrt(mean(x^2) + eps) * (w + w_offset).  out_rows
    (int32 [rows]) scatters the result rows into `out` (a paged pool viewed as [pool rows, cols]).
    groups > 1: every one of `groups` equal consecutive pieces of a row has its own root mean square."""
    assert x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    if out is None:
        assert out_rows is None
        out = torch.empty(rows, cols, dtype=out_dtype or x.dtype, device=x.device)
    assert out.dim() == 2 and out.stride(1) == 1 and out.shape[1] == cols
    if groups != 1:
        assert out_rows is None and cols % groups == 0
        check(_lib.load().vila_group_rmsnorm_rows(_p(x), _dt(x, "x"), x.stride(0), _p(w),
                                                  _dt(w, "w") if w is not None else 0, w_offset, eps, _p(out),
                                                  _dt(out, "out"), out.stride(0), rows, cols, groups, _stream()),
              "vila_group_rmsnorm_rows")
        return out
    check(_lib.load().vila_rmsnorm_rows(_p(x), _dt(x, "x"), x.stride(0), _p(w), _dt(w, "w") if w is not None else 0,
                                        w_offset, eps, _p(out), _dt(out, "out"), out.stride(0),
                                        _i32(out_rows, "out_rows"), rows, cols, _stream()), "vila_rmsnorm_rows")
    return out


def gated_norm_residual(x: torch.Tensor, part: torch.Tensor, *, n_partials: int = 1,
                        gate: Optional[torch.Tensor] = None, gate_bias: Optional[torch.Tensor] = None,
                        w: Optional[torch.Tensor] = None, w_offset: float = 0.0, eps: float = 1e-6,
                        mult: float = 1.0) -> None:
    """x (fp32 [rows, cols], in place) += mult * rmsnorm(sum_j part[r * n_partials + j] * sigmoid(gate + bias)) * (w + w_offset)."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    rows, cols = x.shape
    assert part.dim() == 2 and part.stride(1) == 1 and part.shape == (rows * n_partials, cols)
    if gate is not None:
        assert gate.shape == (rows, cols) and gate.stride(1) == 1
    check(_lib.load().vila_gated_norm_residual_scaled(
        _p(x), _p(part), _dt(part, "part"), part.stride(0), n_partials,
        _p(gate), _dt(gate, "gate") if gate is not None else 0, gate.stride(0) if gate is not None else 0,
        _p(gate_bias), _dt(gate_bias, "gate_bias") if gate_bias is not None else 0,
        _p(w), _dt(w, "w") if w is not None else 0, w_offset, eps, mult, rows, cols, _stream()),
        "vila_gated_norm_residual_scaled")


def glinear(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None, out_dtype=None,
            bias: Optional[torch.Tensor] = None, act: int = ACT_NONE, swiglu: bool = False,
            groups: int = 1, a_group_off: int = 0, o_group_off: int = 0,
            seg: Optional[torch.Tensor] = None, a_rows: Optional[torch.Tensor] = None, a_row_div: int = 1,
            o_rows: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
            out_rows_total: Optional[int] = None, glu_clamp: Optional[Tuple[float, float]] = None,
            act_params: Optional[Tuple[float, float]] = None, in_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Any-shape (grouped) linear layer, fp32 accumulation on the CUDA cores (vila_glinear).
    w [N, K] (groups == 1) or [groups, N, K].  Batched groups (seg None): group g reads the A columns
    [g * a_group_off, + K) and writes the output columns [g * o_group_off, + N).  Segmented (seg int32
    [groups + 1]): the rows of group g are the sorted positions seg[g]..seg[g+1]; see the header.
    act_params: the coefficients of ACT_XIELU.  in_scale fp32: sorted position i is computed from its input row
    times in_scale[a_rows[i]] (a_rows None: in_scale[i]): the scale enters before bias and activation."""
    assert a.dim() == 2 and a.stride(1) == 1
    if w.dim() == 2:
        w = w[None]
    assert w.dim() == 3 and w.stride(2) == 1 and w.shape[0] == groups, (w.shape, groups)
    N, K = w.shape[1], w.shape[2]
    n_out = N // 2 if (swiglu or glu_clamp is not None) else N   # glu_clamp = (alpha, limit): see VILA_FLAG_GLU_CLAMP
    M = a.shape[0] if a_rows is None else a_rows.numel()
    if out is None:
        cols = n_out if seg is not None or groups == 1 else o_group_off * (groups - 1) + n_out
        out = torch.empty(out_rows_total if out_rows_total is not None else M, cols,
                          dtype=out_dtype or a.dtype, device=a.device)
    assert out.dim() == 2 and out.stride(1) == 1
    p = _lib.GLinearParams()
    p.a, p.lda = _p(a), a.stride(0)
    p.w, p.ldw, p.w_group_stride = _p(w), w.stride(1), w.stride(0)
    p.bias = _p(bias)
    p.bias_group_stride = N if bias is not None and bias.numel() > N else 0
    p.out, p.ldo = _p(out), out.stride(0)
    p.a_group_off, p.o_group_off = a_group_off, o_group_off
    p.seg, p.a_rows, p.o_rows = _i32(seg, "seg"), _i32(a_rows, "a_rows"), _i32(o_rows, "o_rows")
    p.row_scale = _f32(row_scale, "row_scale")
    p.a_dtype, p.w_dtype, p.out_dtype = _dt(a, "a"), _dt(w, "w"), _dt(out, "out")
    if bias is not None:
        assert bias.dtype == w.dtype
    p.M, p.N, p.K, p.groups = M, N, K, groups
    p.mode = 0 if seg is None else 1
    p.a_row_div, p.act, p.flags = a_row_div, act, (1 if swiglu else 0) | (4 if glu_clamp is not None else 0)
    if glu_clamp is not None or act_params is not None or in_scale is not None:
        assert in_scale is None or o_rows is None
        ext = _lib.GLinearExt(float(glu_clamp[0]) if glu_clamp else 1.0, float(glu_clamp[1]) if glu_clamp else float("inf"),
                              float(act_params[0]) if act_params else 0.0, float(act_params[1]) if act_params else 0.0,
                              _f32(in_scale, "in_scale"))
        check(_lib.load().vila_glinear_x(C.byref(p), C.byref(ext), _stream()), "vila_glinear_x")
    else:
        check(_lib.load().vila_glinear(C.byref(p), _stream()), "vila_glinear")
    return out


def latent_attention(q: torch.Tensor, cache: torch.Tensor, page_tables: torch.Tensor, tiles: torch.Tensor,
                     *, heads: int, page: int, scale: float, sink: Optional[torch.Tensor] = None,
                     gate: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, out_dtype=None,
                     decode: bool = False, nsplit: int = 1, window: int = 0) -> torch.Tensor:
    """q fp32 [T, heads * R] (key expansion already folded in), cache [pool rows, R], page_tables int32
    [slots, max_pages], tiles int32 [ntiles, 4] (row0, rows, pos0, slot) -> [T, heads * R].
    decode: one-row tiles; nsplit > 1 spreads the keys of every row over nsplit CTAs + a merge kernel.
    window > 0: a row sees itself and the window - 1 tokens before it only."""
    assert q.dtype == torch.float32 and q.is_contiguous() and q.dim() == 2
    assert cache.dim() == 2 and cache.is_contiguous()
    R = cache.shape[1]
    assert q.shape[1] == heads * R
    if out is None:
        out = torch.empty(q.shape, dtype=out_dtype or cache.dtype, device=q.device)
    assert out.shape == q.shape and out.is_contiguous()
    p = _lib.LatentAttnParams()
    p.q, p.cache, p.out = _p(q), _p(cache), _p(out)
    p.page_tables, p.tiles = _i32(page_tables, "page_tables"), _i32(tiles, "tiles")
    p.sink = _f32(sink, "sink")
    p.gate = _p(gate)
    p.ldg = gate.stride(0) if gate is not None else 0
    p.cache_dtype, p.out_dtype = _dt(cache, "cache"), _dt(out, "out")
    p.gate_dtype = _dt(gate, "gate") if gate is not None else 0
    p.ntiles, p.pt_stride = tiles.shape[0], page_tables.stride(0)
    p.H, p.R, p.page, p.decode, p.scale = heads, R, page, 1 if decode else 0, scale
    p.nsplit = max(1, int(nsplit)) if decode else 1
    p.window = int(window)
    partial = None
    if p.nsplit > 1:
        partial = torch.empty(q.shape[0] * heads * p.nsplit * (R + 2), dtype=torch.float32, device=q.device)
        p.partial = partial.data_ptr()
    check(_lib.load().vila_latent_attention(C.byref(p), _stream()), "vila_latent_attention")
    return out


def latent_rope_append(positions: torch.Tensor, inv_freq: Optional[torch.Tensor], *, rank: int, layout: int = 0,
                       mscale: float = 1.0, kv: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                       eps: float = 1e-6, pool: Optional[torch.Tensor] = None,
                       cache_rows: Optional[torch.Tensor] = None, q: Optional[torch.Tensor] = None,
                       qa: Optional[torch.Tensor] = None, heads: int = 0, q_head: int = 0, q_off: int = 0) -> None:
    """Cache rows and query parts of latent attention with a decoupled rotary part (rot = 2 * inv_freq.numel();
    inv_freq None: no rotary part, only the normed latent is written).
    kv [T, >= rank + rot]: pool row cache_rows[t] = rmsnorm(kv[t, :rank]) * norm_w | rotate(kv[t, rank : rank + rot]).
    q [T, >= heads * q_head]: qa[t, h, rank : rank + rot] = rotate(q[t, h * q_head + q_off : + rot]) (qa fp32
    [T, heads * (rank + rot)], its other columns are left alone).  layout 0: pairs (2i, 2i + 1), 1: (i, i + rot / 2)."""
    assert inv_freq is None or (inv_freq.dtype == torch.float64 and inv_freq.is_cuda and inv_freq.is_contiguous())
    rot = 0 if inv_freq is None else 2 * inv_freq.numel()
    p = _lib.LatentRopeParams()
    p.positions, p.inv_freq = _i32(positions, "positions"), _p(inv_freq)
    p.T, p.R, p.rot, p.layout, p.eps, p.mscale = positions.numel(), rank, rot, layout, eps, mscale
    if kv is not None:
        assert kv.dim() == 2 and kv.stride(1) == 1 and kv.shape[1] >= rank + rot and kv.shape[0] == p.T
        assert pool.dim() == 2 and pool.is_contiguous() and pool.shape[1] == rank + rot
        p.kv, p.ld_kv, p.kv_dtype = _p(kv), kv.stride(0), _dt(kv, "kv")
        p.norm_w, p.pool, p.pool_dtype = _f32(norm_w, "norm_w"), _p(pool), _dt(pool, "pool")
        p.cache_rows = _i32(cache_rows, "cache_rows")
    if q is not None:
        assert q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= heads * q_head and q.shape[0] == p.T
        assert qa.dtype == torch.float32 and qa.is_contiguous() and qa.shape == (p.T, heads * (rank + rot))
        p.q, p.ld_q, p.q_dtype, p.qa = _p(q), q.stride(0), _dt(q, "q"), _p(qa)
        p.H, p.q_head, p.q_off = heads, q_head, q_off
    check(_lib.load().vila_latent_rope_append(C.byref(p), _stream()), "vila_latent_rope_append")


def hgrn2_scan(proj: torch.Tensor, state: torch.Tensor, seqs: torch.Tensor, *, heads: int, dim: int, vdim: int,
               q_off: int, f_off: int, v_off: int, f_bias: Optional[torch.Tensor] = None,
               lower: Optional[torch.Tensor] = None) -> torch.Tensor:
    """proj [T, >= ...] holds the pre-activations of q | f | v; state fp32 [slots, heads, dim, vdim]
    (updated in place); seqs int32 [nseq, 4] (row0, rows, pos0, slot) -> o fp32 [T, heads * vdim]."""
    assert proj.dim() == 2 and proj.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (heads, dim, vdim)
    out = torch.empty(proj.shape[0], heads * vdim, dtype=torch.float32, device=proj.device)
    p = _lib.Hgrn2Params()
    p.proj, p.ldp, p.proj_dtype = _p(proj), proj.stride(0), _dt(proj, "proj")
    p.f_bias, p.lower = _f32(f_bias, "f_bias"), _f32(lower, "lower")
    p.state, p.seqs, p.out = _p(state), _i32(seqs, "seqs"), _p(out)
    p.q_off, p.f_off, p.v_off = q_off, f_off, v_off
    p.nseq, p.H, p.dim, p.vdim = seqs.shape[0], heads, dim, vdim
    check(_lib.load().vila_hgrn2_scan(C.byref(p), _stream()), "vila_hgrn2_scan")
    return out


def moe_route(x: torch.Tensor, w_router: torch.Tensor, bias: Optional[torch.Tensor], top: int):
    """-> (idx int32 [rows, top], weight fp32 [rows, top]); router weights / bias fp32."""
    assert x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    E = w_router.shape[0]
    idx = torch.empty(rows, top, dtype=torch.int32, device=x.device)
    wt = torch.empty(rows, top, dtype=torch.float32, device=x.device)
    check(_lib.load().vila_moe_route(_p(x), _dt(x, "x"), x.stride(0), _f32(w_router, "w_router"),
                                     _f32(bias, "bias"), _p(idx), _p(wt), rows, cols, E, top, _stream()),
          "vila_moe_route")
    return idx, wt


def moe_group(idx: torch.Tensor, experts: int):
    """-> (seg int32 [experts + 1], sorted int32 [pairs]): the (token, choice) pairs grouped by expert."""
    pairs = idx.numel()
    seg = torch.empty(experts + 1, dtype=torch.int32, device=idx.device)
    srt = torch.empty(max(pairs, 1), dtype=torch.int32, device=idx.device)
    check(_lib.load().vila_moe_group(_i32(idx, "idx"), _p(seg), _p(srt), pairs, experts, _stream()),
          "vila_moe_group")
    return seg, srt[:pairs]


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """src [N, C] contiguous, rows int32 [n] -> src[rows] (any dtype)."""
    assert src.dim() == 2 and src.is_contiguous() and src.is_cuda
    out = torch.empty(rows.numel(), src.shape[1], dtype=src.dtype, device=src.device)
    check(_lib.load().vila_gather_rows(_p(src), _i32(rows, "rows"), _p(out), rows.numel(),
                                       src.shape[1] * src.element_size(), _stream()), "vila_gather_rows")
    return out


def sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tiles: torch.Tensor, *, heads: int,
                   scale: float, sink: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None, out_dtype=None) -> torch.Tensor:
    """Causal attention with separate keys / values, fp32 softmax, optional sink and output gate.
    q [T, heads * dim]; k [rows, heads * dim], v [rows, heads * vdim] (views with a row stride are fine):
    every sequence's positions 0.. contiguous from its kv_row0; tiles int32 [n, 4] = (row0, rows, pos0,
    kv_row0) -> [T, heads * vdim]."""
    assert q.dim() == 2 and k.dim() == 2 and v.dim() == 2 and q.stride(1) == k.stride(1) == v.stride(1) == 1
    assert k.dtype == v.dtype and q.shape[1] == k.shape[1] and k.shape[1] % heads == 0 and v.shape[1] % heads == 0
    dim, vdim = k.shape[1] // heads, v.shape[1] // heads
    if out is None:
        out = torch.empty(q.shape[0], heads * vdim, dtype=out_dtype or q.dtype, device=q.device)
    assert out.shape == (q.shape[0], heads * vdim) and out.stride(1) == 1
    p = _lib.SinkAttnParams()
    p.q, p.k, p.v, p.out = _p(q), _p(k), _p(v), _p(out)
    p.tiles, p.sink, p.gate = _i32(tiles, "tiles"), _f32(sink, "sink"), _p(gate)
    p.ldq, p.ldk, p.ldv, p.ldo = q.stride(0), k.stride(0), v.stride(0), out.stride(0)
    p.ldg = gate.stride(0) if gate is not None else 0
    p.q_dtype, p.kv_dtype, p.out_dtype = _dt(q, "q"), _dt(k, "k"), _dt(out, "out")
    p.gate_dtype = _dt(gate, "gate") if gate is not None else 0
    p.ntiles, p.H, p.dim, p.vdim, p.scale = tiles.shape[0], heads, dim, vdim, scale
    check(_lib.load().vila_sink_attention(C.byref(p), _stream()), "vila_sink_attention")
    return out


# ---- parallel-sublayer decoders: pair embedding, short convolution, rotary GQA over a paged pool, sigmoid router ----
def linear_any(x: torch.Tensor, w: torch.Tensor, *, swiglu: bool = False, out_dtype=None,
               bias: Optional[torch.Tensor] = None, act: int = ACT_NONE,
               act_params: Optional[Tuple[float, float]] = None) -> torch.Tensor:
    """act(x [M, K] · w[N, K]^T + bias): bf16 operands with 16-byte aligned rows go to the tcgen05 GEMM,
    everything else (fp32 tensors, odd shapes, an fp32 result) to the CUDA-core grouped kernel."""
    N, K = w.shape
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out_dtype in (None, torch.bfloat16)
            and K % 8 == 0 and N % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and (not swiglu or N % 32 == 0)):
        return linear(x, w, bias, act=act, swiglu=swiglu, static_w=True, act_params=act_params)
    return glinear(x, w, swiglu=swiglu, out_dtype=out_dtype, bias=bias, act=act, act_params=act_params)


def embed_pair_rows(table: torch.Tensor, pair_table: torch.Tensor, ids: torch.Tensor, prev_ids: torch.Tensor,
                    mul_prev: int, mul_cur: int, buckets: int) -> torch.Tensor:
    """fp32 rows table[ids] + pair_table[(prev * mul_prev + id * mul_cur) mod buckets]; a token whose
    prev id is negative (the first of its sequence) reads row `buckets` of pair_table."""
    assert pair_table.shape == (buckets + 1, table.shape[1]) and table.is_contiguous() and pair_table.is_contiguous()
    out = torch.empty(ids.numel(), table.shape[1], dtype=torch.float32, device=table.device)
    check(_lib.load().vila_embed_pair_rows(_p(table), _dt(table, "table"), _p(pair_table), _dt(pair_table, "pair_table"),
                                           _i32(ids, "ids"), _i32(prev_ids, "prev_ids"), mul_prev, mul_cur, buckets,
                                           _p(out), ids.numel(), table.shape[1], _stream()), "vila_embed_pair_rows")
    return out


def add_row_vector(x: torch.Tensor, vec: torch.Tensor) -> None:
    """x fp32 [rows, cols] (in place) += vec [cols]"""
    assert x.dtype == torch.float32 and x.is_contiguous() and vec.is_contiguous() and vec.numel() == x.shape[1]
    check(_lib.load().vila_add_row_vector(_p(x), _p(vec), _dt(vec, "vec"), x.shape[0], x.shape[1], _stream()),
          "vila_add_row_vector")


def short_conv_rows(h: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor], seqs: torch.Tensor,
                    row_seq: torch.Tensor, *, out_dtype=None, update_state: bool = True) -> torch.Tensor:
    """h fp32 [T, C] -> h + causal convolution over time with w [C, taps]; state fp32 [slots, taps - 1, C]
    holds every sequence's last taps - 1 inputs (read for the taps that reach before the portion, then
    replaced by this portion's last inputs); seqs int32 [n, 4] = (row0, rows, pos0, slot), row_seq int32 [T]."""
    assert h.dtype == torch.float32 and h.is_contiguous() and h.dim() == 2
    T, Cc = h.shape
    taps = w.shape[1]
    assert w.shape == (Cc, taps) and w.is_contiguous()
    if taps > 1:
        assert state is not None and state.dtype == torch.float32 and state.is_contiguous() and \
            tuple(state.shape[1:]) == (taps - 1, Cc)
    out = torch.empty(T, Cc, dtype=out_dtype or h.dtype, device=h.device)
    lib = _lib.load()
    check(lib.vila_short_conv_rows(_p(h), _p(w), _dt(w, "w"), _p(state), _i32(seqs, "seqs"), _i32(row_seq, "row_seq"),
                                   _p(out), _dt(out, "out"), T, Cc, taps, _stream()), "vila_short_conv_rows")
    if update_state and taps > 1:
        check(lib.vila_short_conv_state(_p(h), _p(state), _i32(seqs, "seqs"), seqs.shape[0], Cc, taps, _stream()),
              "vila_short_conv_state")
    return out


def norm_conv_rows(x: torch.Tensor, norm_w: Sequence[torch.Tensor], conv_w: Sequence[torch.Tensor],
                   state: Sequence[Optional[torch.Tensor]], seqs: torch.Tensor, row_seq: torch.Tensor, *,
                   groups: int, eps: float, w_offset: float = 0.0, out_dtype=None):
    """Group RMS norm of x fp32 [T, C] followed by `h + short convolution(h)` for one or two sublayers that
    read the same rows (norm_w / conv_w / state per sublayer), in one pass; the states are advanced.
    -> list of outputs [T, C].  Equals rmsnorm_rows(groups=) + short_conv_rows per sublayer."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    T, Cc = x.shape
    nsub, taps = len(norm_w), conv_w[0].shape[1]
    assert nsub in (1, 2) and len(conv_w) == nsub and len(state) == nsub and Cc % groups == 0
    outs = [torch.empty(T, Cc, dtype=out_dtype or x.dtype, device=x.device) for _ in range(nsub)]
    p = _lib.NormConvParams()
    p.x = _p(x)
    for k in range(nsub):
        assert conv_w[k].shape == (Cc, taps) and conv_w[k].is_contiguous() and conv_w[k].dtype == conv_w[0].dtype
        p.norm_w[k], p.conv_w[k], p.out[k] = _f32(norm_w[k], "norm_w"), _p(conv_w[k]), _p(outs[k])
        if taps > 1:
            st = state[k]
            assert st is not None and st.dtype == torch.float32 and st.is_contiguous() and \
                tuple(st.shape[1:]) == (taps - 1, Cc)
            p.state[k] = _p(st)
    p.seqs, p.row_seq = _i32(seqs, "seqs"), _i32(row_seq, "row_seq")
    inv = torch.empty(T, groups, dtype=torch.float32, device=x.device)
    p.inv = _p(inv)
    p.conv_w_dtype, p.out_dtype = _dt(conv_w[0], "conv_w"), _dt(outs[0], "out")
    p.rows, p.nseq, p.cols, p.groups, p.taps, p.nsub = T, seqs.shape[0], Cc, groups, taps, nsub
    p.eps, p.w_offset = eps, w_offset
    check(_lib.load().vila_norm_conv_rows(C.byref(p), _stream()), "vila_norm_conv_rows")
    return outs


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, cache_rows: torch.Tensor, pool: torch.Tensor, *,
                heads: int, kv_heads: int, dim: int, vdim: int, inv_freq: Optional[torch.Tensor],
                unit_norm: bool, eps: float, q_norm_w: Optional[torch.Tensor] = None,
                k_norm_w: Optional[torch.Tensor] = None, v_from_k: bool = False, halves: bool = False,
                mscale: float = 1.0) -> torch.Tensor:
    """qkv [T, >= heads*dim + kv_heads*(dim+vdim)] -> q fp32 [T, heads*dim] (rotated, unit-normed); the
    token's k | v go to row cache_rows[t] of pool [pool rows, kv_heads*(dim+vdim)].  inv_freq float64
    [rot_dims / 2] (None: no rotation).  q_norm_w / k_norm_w fp32 [dim]: weights of the per-head norm.
    v_from_k: qkv holds q | k only, the cached value of a token is its incoming key (before rotation / norm).
    halves: column i of the rotated part pairs with i + rot_dims / 2 instead of 2i with 2i + 1; mscale multiplies
    cos and sin (a magnitude correction of rescaled frequencies)."""
    assert qkv.dim() == 2 and qkv.stride(1) == 1
    assert qkv.shape[1] >= heads * dim + kv_heads * (dim if v_from_k else dim + vdim)
    assert not v_from_k or vdim == dim
    assert pool.dim() == 2 and pool.is_contiguous() and pool.shape[1] == kv_heads * (dim + vdim)
    T = qkv.shape[0]
    q = torch.empty(T, heads * dim, dtype=torch.float32, device=qkv.device)
    p = _lib.RopeAppendParams()
    p.qkv, p.ldq = _p(qkv), qkv.stride(0)
    p.positions, p.cache_rows = _i32(positions, "positions"), _i32(cache_rows, "cache_rows")
    if inv_freq is not None:
        assert inv_freq.dtype == torch.float64 and inv_freq.is_cuda and inv_freq.is_contiguous()
    p.inv_freq = _p(inv_freq)
    p.q_out, p.pool = _p(q), _p(pool)
    p.qkv_dtype, p.pool_dtype = _dt(qkv, "qkv"), _dt(pool, "pool")
    p.T, p.H, p.G, p.dim, p.vdim = T, heads, kv_heads, dim, vdim
    p.rot_dims = 0 if inv_freq is None else 2 * inv_freq.numel()
    p.unit_norm, p.eps = 1 if unit_norm else 0, eps
    for t_ in (q_norm_w, k_norm_w):
        assert t_ is None or (unit_norm and t_.numel() == dim)
    p.q_norm_w, p.k_norm_w, p.v_from_k = _f32(q_norm_w, "q_norm_w"), _f32(k_norm_w, "k_norm_w"), 1 if v_from_k else 0
    p.rot_layout, p.rot_mscale = 1 if halves else 0, float(mscale)
    check(_lib.load().vila_rope_append(C.byref(p), _stream()), "vila_rope_append")
    return q


def paged_attention(q: torch.Tensor, pool: torch.Tensor, page_tables: torch.Tensor, tiles: torch.Tensor, *,
                    heads: int, kv_heads: int, dim: int, vdim: int, page: int, scale: float,
                    talk: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None,
                    out: Optional[torch.Tensor] = None, out_dtype=None, max_rows: int = 16,
                    nsplit: int = 1, dist_bias: Optional[torch.Tensor] = None, chunk: int = 0,
                    gate: Optional[torch.Tensor] = None, window: int = 0, keep_first: int = 0,
                    talk_after: bool = False, head_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal grouped-query attention of q fp32 [T, heads*dim] over the paged k | v pool, fp32 scores and
    softmax, optional mixing of the heads' scores (talk fp32 [heads, heads]) and per-head sink logit in
    the denominator.  tiles int32 [n, 4] = (row0, rows <= max_rows, pos0, slot) -> [T, heads*vdim].
    nsplit > 1 (one-row tiles only) spreads the keys of a row over nsplit CTAs + a merge kernel.
    dist_bias fp32 [rows, heads]: added to the score by distance (the last row for every larger one);
    chunk > 0: a query sees its own block of `chunk` positions only; gate [T, >= heads] (a view with a
    row stride is fine): the output of head h is multiplied by sigmoid(gate[t, h]).
    window > 0: a key is seen only when it is less than `window` positions back or among the first `keep_first`
    of its sequence.  talk_after: talk mixes the heads' softmax weights instead of their scores (no sink then).
    head_scale fp32 [heads]: per-head multiplier of the scores."""
    assert q.dtype == torch.float32 and q.is_contiguous() and q.shape[1] == heads * dim
    assert pool.dim() == 2 and pool.is_contiguous() and pool.shape[1] == kv_heads * (dim + vdim)
    if out is None:
        out = torch.empty(q.shape[0], heads * vdim, dtype=out_dtype or pool.dtype, device=q.device)
    assert out.shape == (q.shape[0], heads * vdim) and out.is_contiguous()
    if talk is not None:
        assert talk.shape == (heads, heads)
    p = _lib.PagedAttnParams()
    p.q, p.pool, p.out = _p(q), _p(pool), _p(out)
    p.page_tables, p.tiles = _i32(page_tables, "page_tables"), _i32(tiles, "tiles")
    p.talk, p.sink = _f32(talk, "talk"), _f32(sink, "sink")
    p.pool_dtype, p.out_dtype = _dt(pool, "pool"), _dt(out, "out")
    p.ntiles, p.pt_stride = tiles.shape[0], page_tables.stride(0)
    p.H, p.G, p.dim, p.vdim, p.page, p.scale = heads, kv_heads, dim, vdim, page, scale
    p.max_rows = max_rows
    if dist_bias is not None:
        assert dist_bias.dim() == 2 and dist_bias.shape[1] == heads
        p.dist_bias, p.dist_rows = _f32(dist_bias, "dist_bias"), dist_bias.shape[0]
    if gate is not None:
        assert gate.dim() == 2 and gate.shape[0] == q.shape[0] and gate.shape[1] >= heads and gate.stride(1) == 1
        p.gate, p.ldg, p.gate_dtype = _p(gate), gate.stride(0), _dt(gate, "gate")
    p.chunk = int(chunk)
    p.window, p.keep_first, p.talk_after = int(window), int(keep_first), 1 if talk_after else 0
    if head_scale is not None:
        assert head_scale.numel() == heads
        p.head_scale = _f32(head_scale, "head_scale")
    p.nsplit = max(1, int(nsplit)) if max_rows == 1 else 1
    partial = None
    if p.nsplit > 1:
        partial = torch.empty(q.shape[0] * p.nsplit * heads * (vdim + 2), dtype=torch.float32, device=q.device)
        p.partial = partial.data_ptr()
    check(_lib.load().vila_paged_attention(C.byref(p), _stream()), "vila_paged_attention")
    return out


def moe_route_sigmoid(x: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], top: int,
                      groups: int = 1, keep: int = 1):
    """Sigmoid router with group-limited choice -> (idx int32 [rows, top], weight fp32 [rows, top]):
    choice = sigmoid(w_router x) + correction, restricted to the `keep` groups (of `groups`) with the largest
    sum of their two best choice values; weights are the plain sigmoid scores of the chosen experts."""
    assert x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    E = w_router.shape[0]
    idx = torch.empty(rows, top, dtype=torch.int32, device=x.device)
    wt = torch.empty(rows, top, dtype=torch.float32, device=x.device)
    check(_lib.load().vila_moe_route_sigmoid(_p(x), _dt(x, "x"), x.stride(0), _f32(w_router, "w_router"),
                                             _f32(correction, "correction"), _p(idx), _p(wt), rows, cols, E, top,
                                             groups, keep, _stream()), "vila_moe_route_sigmoid")
    return idx, wt


def residual_add_rows(x: torch.Tensor, a: Optional[torch.Tensor] = None, part: Optional[torch.Tensor] = None, *,
                      n_partials: int = 1, mult: float = 1.0, copy_dtype=None) -> Optional[torch.Tensor]:
    """x fp32 [rows, cols] (in place) += mult * (a[r] + sum_j part[r * n_partials + j]); copy_dtype: also
    return the updated rows in that dtype (the operand of the projection that reads x next)."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    rows, cols = x.shape
    if a is not None:
        assert a.shape == (rows, cols) and a.stride(1) == 1
    if part is not None:
        assert part.shape == (rows * n_partials, cols) and part.stride(1) == 1
    copy = torch.empty(rows, cols, dtype=copy_dtype, device=x.device) if copy_dtype is not None else None
    check(_lib.load().vila_residual_add_rows(
        _p(x), _p(a), _dt(a, "a") if a is not None else 0, a.stride(0) if a is not None else 0,
        _p(part), _dt(part, "part") if part is not None else 0, part.stride(0) if part is not None else 0,
        n_partials, mult, _p(copy), _dt(copy, "copy") if copy is not None else 0, rows, cols, _stream()),
        "vila_residual_add_rows")
    return copy


def residual_norm_rows(x: torch.Tensor, a: Optional[torch.Tensor], w: Optional[torch.Tensor], eps: float, *,
                       part: Optional[torch.Tensor] = None, n_partials: int = 1, out_dtype=None) -> torch.Tensor:
    """x fp32 [rows, cols] (in place) += a[r] + sum_j part[r * n_partials + j]; -> rmsnorm(x) * w in out_dtype (the
    operand of the sublayer that reads x next): the residual sum and the following pre-norm in one pass."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    rows, cols = x.shape
    if a is not None:
        assert a.shape == (rows, cols) and a.stride(1) == 1
    if part is not None:
        assert part.shape == (rows * n_partials, cols) and part.stride(1) == 1
    out = torch.empty(rows, cols, dtype=out_dtype or x.dtype, device=x.device)
    check(_lib.load().vila_residual_norm_rows(
        _p(x), _p(a), _dt(a, "a") if a is not None else 0, a.stride(0) if a is not None else 0,
        _p(part), _dt(part, "part") if part is not None else 0, part.stride(0) if part is not None else 0,
        n_partials, _p(w), _dt(w, "w") if w is not None else 0, eps, _p(out), _dt(out, "out"), rows, cols, _stream()),
        "vila_residual_norm_rows")
    return out


def gelu_mul_gather(z: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, col0: int, *, out_dtype=None) -> torch.Tensor:
    """gelu_tanh(z [T, n]) * table[ids, col0 : col0 + n]"""
    assert z.is_contiguous() and z.dim() == 2
    assert table.dim() == 2 and table.stride(1) == 1 and col0 + z.shape[1] <= table.shape[1]
    out = torch.empty(z.shape, dtype=out_dtype or z.dtype, device=z.device)
    check(_lib.load().vila_gelu_mul_gather(_p(z), _dt(z, "z"), _p(table), _dt(table, "table"), table.stride(0), _i32(ids, "ids"),
                                           col0, _p(out), _dt(out, "out"), z.shape[0], z.shape[1], _stream()),
          "vila_gelu_mul_gather")
    return out


# ---- state-space mixers: sinusoidal embedding, causal convolution, scalar-decay and selective scans ----
def embed_sincos_rows(table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
                      scale: float, *, copy_dtype=None):
    """fp32 rows table[ids] * scale + sinusoid(positions): column 2i = sin, 2i + 1 = cos of position *
    inv_freq[i] (float64 [(cols + 1) // 2]).  -> (rows, the same rows in copy_dtype or None)"""
    T, cols = ids.numel(), table.shape[1]
    assert table.is_contiguous() and inv_freq.dtype == torch.float64 and inv_freq.is_cuda and \
        inv_freq.is_contiguous() and inv_freq.numel() == (cols + 1) // 2
    out = torch.empty(T, cols, dtype=torch.float32, device=table.device)
    copy = torch.empty(T, cols, dtype=copy_dtype, device=table.device) if copy_dtype is not None else None
    check(_lib.load().vila_embed_sincos_rows(_p(table), _dt(table, "table"), _i32(ids, "ids"),
                                             _i32(positions, "positions"), _p(inv_freq), scale, _p(out), _p(copy),
                                             _dt(copy, "copy") if copy is not None else 0, T, cols, _stream()),
          "vila_embed_sincos_rows")
    return out, copy


def branch_norm_residual(x: torch.Tensor, a: torch.Tensor, w: Optional[torch.Tensor], eps: float, *,
                         a_scale: float = 1.0, b: Optional[torch.Tensor] = None, b_scale: float = 1.0,
                         copy_dtype=None) -> Optional[torch.Tensor]:
    """x fp32 [rows, cols] (in place) += rms(a_scale * a + b_scale * b) * w, rms(v) = v / sqrt(mean(v^2) + eps):
    the post-normed residual update of one or two branches.  copy_dtype: also return the updated rows in
    that dtype (the operand of the projection that reads x next)."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2
    rows, cols = x.shape
    assert a.shape == (rows, cols) and a.stride(1) == 1
    if b is not None:
        assert b.shape == (rows, cols) and b.stride(1) == 1
    copy = torch.empty(rows, cols, dtype=copy_dtype, device=x.device) if copy_dtype is not None else None
    check(_lib.load().vila_branch_norm_residual(
        _p(x), _p(a), _dt(a, "a"), a.stride(0), a_scale, _p(b), _dt(b, "b") if b is not None else 0,
        b.stride(0) if b is not None else 0, b_scale, _p(w), _dt(w, "w") if w is not None else 0, eps,
        _p(copy), _dt(copy, "copy") if copy is not None else 0, rows, cols, _stream()), "vila_branch_norm_residual")
    return copy


CONV_NONE, CONV_SILU = 0, 1


def causal_conv_rows(u: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor],
                     seqs: torch.Tensor, row_seq: torch.Tensor, *, act: int = CONV_NONE, out_dtype=None,
                     update_state: bool = True) -> torch.Tensor:
    """u [T, C] (a column slice with a row stride is fine) -> act(bias + causal depthwise convolution over time
    with w [C, taps]; tap taps - 1 meets the newest input); state fp32 [slots, taps - 1, C] holds every sequence's
    last taps - 1 inputs (read for taps that reach before the portion, then replaced by this portion's last
    inputs); seqs int32 [n, 4] = (row0, rows, pos0, slot), row_seq int32 [T]."""
    assert u.dim() == 2 and u.stride(1) == 1
    T, Cc = u.shape
    taps = w.shape[1]
    assert w.shape == (Cc, taps) and w.is_contiguous()
    if bias is not None:
        assert bias.dtype == w.dtype and bias.numel() == Cc and bias.is_contiguous()
    if taps > 1:
        assert state is not None and state.dtype == torch.float32 and state.is_contiguous() and \
            tuple(state.shape[1:]) == (taps - 1, Cc)
    out = torch.empty(T, Cc, dtype=out_dtype or u.dtype, device=u.device)
    p = _lib.CausalConvParams()
    p.in_, p.ld_in, p.w, p.bias, p.state = _p(u), u.stride(0), _p(w), _p(bias), _p(state)
    p.seqs, p.row_seq, p.out, p.ld_out = _i32(seqs, "seqs"), _i32(row_seq, "row_seq"), _p(out), out.stride(0)
    p.in_dtype, p.w_dtype, p.out_dtype = _dt(u, "u"), _dt(w, "w"), _dt(out, "out")
    p.rows, p.nseq, p.cols, p.taps, p.act = T, seqs.shape[0], Cc, taps, act
    lib = _lib.load()
    check(lib.vila_causal_conv_rows(C.byref(p), _stream()), "vila_causal_conv_rows")
    if update_state and taps > 1:
        check(lib.vila_causal_conv_state(C.byref(p), _stream()), "vila_causal_conv_state")
    return out


def ssd_scan(xbc: torch.Tensor, dt: torch.Tensor, z: Optional[torch.Tensor], state: torch.Tensor, seqs: torch.Tensor,
             *, heads: int, vdim: int, nstate: int, groups: int, dt_bias: torch.Tensor, A_log: torch.Tensor,
             D: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    """Scalar-decay recurrence per head: S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t,
    dt_t = softplus(dt + dt_bias), out = y * silu(z).  xbc [T, heads*vdim + 2*groups*nstate] = x | B | C;
    dt [T, heads]; z [T, heads*vdim] or None (views with a row stride are fine, one dtype for the three);
    state fp32 [slots, heads, vdim, nstate], advanced in place; seqs int32 [n, 4] = (row0, rows, pos0, slot)."""
    T = xbc.shape[0]
    inner = heads * vdim
    assert xbc.dim() == 2 and xbc.stride(1) == 1 and xbc.shape[1] == inner + 2 * groups * nstate
    assert dt.shape == (T, heads) and dt.stride(1) == 1 and dt.dtype == xbc.dtype
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, vdim, nstate)
    out = torch.empty(T, inner, dtype=out_dtype, device=xbc.device)
    p = _lib.SsdScanParams()
    p.xbc, p.ld_xbc, p.dt, p.ld_dt = _p(xbc), xbc.stride(0), _p(dt), dt.stride(0)
    if z is not None:
        assert z.shape == (T, inner) and z.stride(1) == 1 and z.dtype == xbc.dtype
        p.z, p.ld_z = _p(z), z.stride(0)
    p.dt_bias, p.A_log, p.D = _f32(dt_bias, "dt_bias"), _f32(A_log, "A_log"), _f32(D, "D")
    assert dt_bias.numel() == heads and A_log.numel() == heads and D.numel() == heads
    p.state, p.seqs, p.out, p.ld_out = _p(state), _i32(seqs, "seqs"), _p(out), out.stride(0)
    p.in_dtype, p.out_dtype = _dt(xbc, "xbc"), _dt(out, "out")
    p.nseq, p.H, p.P, p.N, p.G = seqs.shape[0], heads, vdim, nstate, groups
    check(_lib.load().vila_ssd_scan(C.byref(p), _stream()), "vila_ssd_scan")
    return out


def selective_scan(x: torch.Tensor, dt: torch.Tensor, bc: torch.Tensor, z: Optional[torch.Tensor], state: torch.Tensor,
                   seqs: torch.Tensor, *, dt_bias: torch.Tensor, A_log: torch.Tensor, D: torch.Tensor,
                   out_dtype=torch.float32) -> torch.Tensor:
    """Per-channel selective recurrence: S_t[c, n] = exp(-exp(A_log[c, n]) dt_t,c) S_{t-1}[c, n] + dt_t,c x_t,c B_t,n,
    y_t,c = sum_n S_t[c, n] C_t,n + D_c x_t,c, dt = softplus(dt + dt_bias), out = y * silu(z).  x, dt, z [T, C];
    bc [T, 2 * N] = B | C (views with a row stride are fine, one dtype for all); state fp32 [slots, C, N]."""
    T, Cc = x.shape
    N = A_log.shape[1]
    assert x.stride(1) == 1 and dt.shape == (T, Cc) and dt.stride(1) == 1 and dt.dtype == x.dtype
    assert bc.shape == (T, 2 * N) and bc.stride(1) == 1 and bc.dtype == x.dtype
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (Cc, N)
    assert A_log.shape == (Cc, N) and dt_bias.numel() == Cc and D.numel() == Cc
    out = torch.empty(T, Cc, dtype=out_dtype, device=x.device)
    p = _lib.SelectiveScanParams()
    p.x, p.ld_x, p.dt, p.ld_dt, p.bc, p.ld_bc = _p(x), x.stride(0), _p(dt), dt.stride(0), _p(bc), bc.stride(0)
    if z is not None:
        assert z.shape == (T, Cc) and z.stride(1) == 1 and z.dtype == x.dtype
        p.z, p.ld_z = _p(z), z.stride(0)
    p.dt_bias, p.A_log, p.D = _f32(dt_bias, "dt_bias"), _f32(A_log, "A_log"), _f32(D, "D")
    p.state, p.seqs, p.out, p.ld_out = _p(state), _i32(seqs, "seqs"), _p(out), out.stride(0)
    p.in_dtype, p.out_dtype = _dt(x, "x"), _dt(out, "out")
    p.nseq, p.C, p.N = seqs.shape[0], Cc, N
    check(_lib.load().vila_selective_scan(C.byref(p), _stream()), "vila_selective_scan")
    return out
