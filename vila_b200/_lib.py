"""ctypes binding of libvila_b200.so (the C-ABI declared in include/vila_b200.h).

There is no fallback: if the shared library is missing or a call fails, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libvila_b200.so"

c_void_p, c_int, c_i64, c_float = C.c_void_p, C.c_int, C.c_int64, C.c_float
c_i32_p = C.POINTER(C.c_int32)


class FmhaParams(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("q_tok_stride", c_i64), ("q_head_stride", c_i64),
        ("k", c_void_p), ("v", c_void_p),
        ("kv_page_stride", c_i64), ("kv_tok_stride", c_i64), ("kv_head_stride", c_i64),
        ("kv_num_pages", c_i64),
        ("page_table", c_void_p), ("page_table_stride", C.c_int32),
        ("o", c_void_p), ("o_tok_stride", c_i64), ("o_head_stride", c_i64),
        ("B", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32), ("Hq", C.c_int32),
        ("Hkv", C.c_int32), ("D", C.c_int32), ("causal", C.c_int32),
        ("scale", c_float),
    ]


class GemvParams(C.Structure):
    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("norm_w", c_void_p),
        ("norm_eps", c_float), ("residual", c_void_p), ("y", c_void_p),
        ("N", C.c_int32), ("K", C.c_int32), ("flags", C.c_int32),
        ("argmax_key", c_void_p),
    ]


class DecodeAttnParams(C.Structure):
    _fields_ = [
        ("qkv", c_void_p), ("position", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p),
        ("page_table", c_void_p), ("out", c_void_p), ("ws", c_void_p), ("counters", c_void_p),
        ("inv_freq", c_void_p),
        ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32), ("num_splits", C.c_int32),
        ("scale", c_float),
    ]


class DecodeAttnSplitParams(C.Structure):
    _fields_ = [
        ("qkv", c_void_p), ("position", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p),
        ("page_table", c_void_p), ("kv_num_pages", c_i64), ("out", c_void_p), ("o_partial", c_void_p),
        ("lse", c_void_p), ("counters", c_void_p), ("inv_freq", c_void_p),
        ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32), ("num_splits", C.c_int32),
        ("split_tokens", C.c_int32), ("scale", c_float),
    ]


class MegaParams(C.Structure):
    _fields_ = [
        ("layers", c_void_p), ("num_layers", C.c_int32),
        ("final_norm_w", c_void_p), ("lm_head_w", c_void_p), ("embed", c_void_p),
        ("hidden", C.c_int32), ("inter", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32),
        ("vocab", C.c_int32), ("eps", c_float), ("scale", c_float),
        ("inv_freq", c_void_p), ("page_table", c_void_p),
        ("x", c_void_p), ("qkv", c_void_p), ("act", c_void_p), ("attn_ws", c_void_p), ("attn_counters", c_void_p),
        ("key", c_void_p), ("token", c_void_p), ("hist", c_void_p), ("step", c_void_p),
        ("position", c_void_p), ("barrier", c_void_p), ("epoch", c_void_p),
        ("n_tokens", C.c_int32), ("splits", C.c_int32),
    ]


class GLinearParams(C.Structure):
    _fields_ = [
        ("a", c_void_p), ("lda", c_i64), ("w", c_void_p), ("ldw", c_i64), ("w_group_stride", c_i64),
        ("bias", c_void_p), ("bias_group_stride", c_i64), ("out", c_void_p), ("ldo", c_i64),
        ("a_group_off", c_i64), ("o_group_off", c_i64), ("seg", c_void_p), ("a_rows", c_void_p),
        ("o_rows", c_void_p), ("row_scale", c_void_p),
        ("a_dtype", C.c_int32), ("w_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("groups", C.c_int32),
        ("mode", C.c_int32), ("a_row_div", C.c_int32), ("act", C.c_int32), ("flags", C.c_int32),
    ]


class LatentAttnParams(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("cache", c_void_p), ("page_tables", c_void_p), ("tiles", c_void_p),
        ("sink", c_void_p), ("gate", c_void_p), ("out", c_void_p), ("partial", c_void_p), ("ldg", c_i64),
        ("cache_dtype", C.c_int32), ("gate_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("ntiles", C.c_int32), ("pt_stride", C.c_int32), ("H", C.c_int32), ("R", C.c_int32),
        ("page", C.c_int32), ("decode", C.c_int32), ("nsplit", C.c_int32), ("scale", c_float),
        ("window", C.c_int32),
    ]


class LatentRopeParams(C.Structure):
    _fields_ = [
        ("kv", c_void_p), ("ld_kv", c_i64), ("norm_w", c_void_p), ("pool", c_void_p), ("cache_rows", c_void_p),
        ("q", c_void_p), ("ld_q", c_i64), ("qa", c_void_p), ("positions", c_void_p), ("inv_freq", c_void_p),
        ("kv_dtype", C.c_int32), ("pool_dtype", C.c_int32), ("q_dtype", C.c_int32), ("T", C.c_int32),
        ("H", C.c_int32), ("R", C.c_int32), ("rot", C.c_int32), ("q_head", C.c_int32), ("q_off", C.c_int32),
        ("layout", C.c_int32), ("eps", c_float), ("mscale", c_float),
    ]


class SinkAttnParams(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("tiles", c_void_p), ("sink", c_void_p),
        ("gate", c_void_p), ("out", c_void_p),
        ("ldq", c_i64), ("ldk", c_i64), ("ldv", c_i64), ("ldg", c_i64), ("ldo", c_i64),
        ("q_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("gate_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("ntiles", C.c_int32), ("H", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("scale", c_float),
    ]


class Hgrn2Params(C.Structure):
    _fields_ = [
        ("proj", c_void_p), ("ldp", c_i64), ("f_bias", c_void_p), ("lower", c_void_p),
        ("state", c_void_p), ("seqs", c_void_p), ("out", c_void_p),
        ("proj_dtype", C.c_int32), ("q_off", C.c_int32), ("f_off", C.c_int32), ("v_off", C.c_int32),
        ("nseq", C.c_int32), ("H", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32),
    ]


class GLinearExt(C.Structure):
    _fields_ = [("act_alpha", c_float), ("act_limit", c_float), ("act_pos", c_float), ("act_neg", c_float),
                ("in_scale", c_void_p)]


class RopeAppendParams(C.Structure):
    _fields_ = [
        ("qkv", c_void_p), ("ldq", c_i64), ("positions", c_void_p), ("cache_rows", c_void_p),
        ("inv_freq", c_void_p), ("q_out", c_void_p), ("pool", c_void_p),
        ("qkv_dtype", C.c_int32), ("pool_dtype", C.c_int32), ("T", C.c_int32), ("H", C.c_int32),
        ("G", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("rot_dims", C.c_int32),
        ("unit_norm", C.c_int32), ("eps", c_float),
        ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("v_from_k", C.c_int32),
        ("rot_layout", C.c_int32), ("rot_mscale", c_float),
    ]


class PagedAttnParams(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("pool", c_void_p), ("page_tables", c_void_p), ("tiles", c_void_p),
        ("talk", c_void_p), ("sink", c_void_p), ("out", c_void_p), ("partial", c_void_p),
        ("pool_dtype", C.c_int32), ("out_dtype", C.c_int32), ("ntiles", C.c_int32), ("pt_stride", C.c_int32),
        ("H", C.c_int32), ("G", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("page", C.c_int32),
        ("nsplit", C.c_int32), ("max_rows", C.c_int32), ("scale", c_float),
        ("dist_bias", c_void_p), ("gate", c_void_p), ("ldg", c_i64),
        ("dist_rows", C.c_int32), ("chunk", C.c_int32), ("gate_dtype", C.c_int32),
        ("window", C.c_int32), ("keep_first", C.c_int32), ("talk_after", C.c_int32), ("head_scale", c_void_p),
    ]


class CausalConvParams(C.Structure):
    _fields_ = [
        ("in_", c_void_p), ("ld_in", c_i64), ("w", c_void_p), ("bias", c_void_p), ("state", c_void_p),
        ("seqs", c_void_p), ("row_seq", c_void_p), ("out", c_void_p), ("ld_out", c_i64),
        ("in_dtype", C.c_int32), ("w_dtype", C.c_int32), ("out_dtype", C.c_int32), ("rows", C.c_int32),
        ("nseq", C.c_int32), ("cols", C.c_int32), ("taps", C.c_int32), ("act", C.c_int32),
    ]


class SsdScanParams(C.Structure):
    _fields_ = [
        ("xbc", c_void_p), ("ld_xbc", c_i64), ("dt", c_void_p), ("ld_dt", c_i64), ("z", c_void_p), ("ld_z", c_i64),
        ("dt_bias", c_void_p), ("A_log", c_void_p), ("D", c_void_p), ("state", c_void_p), ("seqs", c_void_p),
        ("out", c_void_p), ("ld_out", c_i64),
        ("in_dtype", C.c_int32), ("out_dtype", C.c_int32), ("nseq", C.c_int32), ("H", C.c_int32),
        ("P", C.c_int32), ("N", C.c_int32), ("G", C.c_int32),
    ]


class SelectiveScanParams(C.Structure):
    _fields_ = [
        ("x", c_void_p), ("ld_x", c_i64), ("dt", c_void_p), ("ld_dt", c_i64), ("bc", c_void_p), ("ld_bc", c_i64),
        ("z", c_void_p), ("ld_z", c_i64), ("dt_bias", c_void_p), ("A_log", c_void_p), ("D", c_void_p),
        ("state", c_void_p), ("seqs", c_void_p), ("out", c_void_p), ("ld_out", c_i64),
        ("in_dtype", C.c_int32), ("out_dtype", C.c_int32), ("nseq", C.c_int32), ("C", C.c_int32), ("N", C.c_int32),
    ]


class NormConvParams(C.Structure):
    _fields_ = [
        ("x", c_void_p), ("norm_w", c_void_p * 2), ("conv_w", c_void_p * 2), ("state", c_void_p * 2),
        ("out", c_void_p * 2), ("seqs", c_void_p), ("row_seq", c_void_p), ("inv", c_void_p),
        ("conv_w_dtype", C.c_int32), ("out_dtype", C.c_int32), ("rows", C.c_int32), ("nseq", C.c_int32),
        ("cols", C.c_int32), ("groups", C.c_int32), ("taps", C.c_int32), ("nsub", C.c_int32),
        ("eps", c_float), ("w_offset", c_float),
    ]


# name -> argtypes; every function returns int (0 == ok) unless listed in _RESTYPES
SIGNATURES = {
    "vila_abi_version": [],
    "vila_device_info": [C.POINTER(c_int)] * 3,
    "vila_set_workspace": [c_void_p, C.c_uint64],
    "vila_linear": [c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_void_p, c_i64, c_int, c_void_p,
                    c_i64, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "vila_linear_act": [c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_void_p, c_i64, c_int, c_int, c_int, c_int,
                        c_float, c_float, c_int, c_void_p],
    "vila_linear_cfg": [c_int, c_void_p, c_i64, c_void_p, c_i64, c_void_p, c_void_p, c_i64, c_int,
                        c_void_p, c_i64, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "vila_layernorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "vila_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "vila_fmha": [C.POINTER(FmhaParams), c_void_p],
    "vila_fmha_cfg": [c_int, C.POINTER(FmhaParams), c_void_p],
    "vila_patch_im2col": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "vila_resize_bicubic_tiles": [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                  c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p],
    "vila_space_to_depth": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "vila_s2_merge": [c_void_p, c_void_p, c_int, c_int, c_int, C.POINTER(c_int), C.POINTER(c_int),
                      c_int, c_int, c_int, c_void_p],
    "vila_chessboard_merge": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "vila_tsp_pool": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "vila_embed_splice": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "vila_rope_kv_append": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_int, c_void_p],
    "vila_rope_kv_append_table": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                  c_int, c_void_p],
    "vila_linear_qkv_rope": [c_void_p, C.c_int64, c_void_p, C.c_int64, c_void_p, c_void_p, C.c_int64,
                             c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_int, c_int, c_void_p],
    "vila_rope_table": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "vila_gemv": [C.POINTER(GemvParams), c_void_p],
    "vila_argmax_finalize": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int, c_void_p],
    "vila_decode_attention": [C.POINTER(DecodeAttnParams), c_void_p],
    "vila_decode_attention_batch": [C.POINTER(DecodeAttnParams), c_int, c_int, c_int, c_int, c_int, c_void_p],
    "vila_decode_attention_split": [C.POINTER(DecodeAttnSplitParams), c_void_p],
    "vila_decode_mega": [C.POINTER(MegaParams), c_void_p],
    "vila_embed_rows": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "vila_rmsnorm_rows": [c_void_p, c_int, c_i64, c_void_p, c_int, c_float, c_float, c_void_p, c_int, c_i64,
                          c_void_p, c_int, c_int, c_void_p],
    "vila_gated_norm_residual": [c_void_p, c_void_p, c_int, c_i64, c_int, c_void_p, c_int, c_i64, c_void_p,
                                 c_int, c_void_p, c_int, c_float, c_float, c_int, c_int, c_void_p],
    "vila_glinear": [C.POINTER(GLinearParams), c_void_p],
    "vila_latent_attention": [C.POINTER(LatentAttnParams), c_void_p],
    "vila_latent_rope_append": [C.POINTER(LatentRopeParams), c_void_p],
    "vila_hgrn2_scan": [C.POINTER(Hgrn2Params), c_void_p],
    "vila_sink_attention": [C.POINTER(SinkAttnParams), c_void_p],
    "vila_gather_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "vila_moe_route": [c_void_p, c_int, c_i64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                       c_int, c_void_p],
    "vila_moe_group": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "vila_glinear_x": [C.POINTER(GLinearParams), C.POINTER(GLinearExt), c_void_p],
    "vila_embed_pair_rows": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_i64, c_i64, c_i64, c_void_p,
                             c_int, c_int, c_void_p],
    "vila_add_row_vector": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "vila_group_rmsnorm_rows": [c_void_p, c_int, c_i64, c_void_p, c_int, c_float, c_float, c_void_p, c_int, c_i64,
                                c_int, c_int, c_int, c_void_p],
    "vila_short_conv_rows": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                             c_int, c_void_p],
    "vila_short_conv_state": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "vila_rope_append": [C.POINTER(RopeAppendParams), c_void_p],
    "vila_paged_attention": [C.POINTER(PagedAttnParams), c_void_p],
    "vila_moe_route_sigmoid": [c_void_p, c_int, c_i64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_void_p],
    "vila_residual_add_rows": [c_void_p, c_void_p, c_int, c_i64, c_void_p, c_int, c_i64, c_int, c_float, c_void_p,
                               c_int, c_int, c_int, c_void_p],
    "vila_residual_norm_rows": [c_void_p, c_void_p, c_int, c_i64, c_void_p, c_int, c_i64, c_int, c_void_p, c_int,
                                c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "vila_norm_conv_rows": [C.POINTER(NormConvParams), c_void_p],
    "vila_gated_norm_residual_scaled": [c_void_p, c_void_p, c_int, c_i64, c_int, c_void_p, c_int, c_i64, c_void_p,
                                        c_int, c_void_p, c_int, c_float, c_float, c_float, c_int, c_int, c_void_p],
    "vila_gelu_mul_gather": [c_void_p, c_int, c_void_p, c_int, c_i64, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                             c_void_p],
    "vila_embed_sincos_rows": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
                               c_int, c_int, c_void_p],
    "vila_branch_norm_residual": [c_void_p, c_void_p, c_int, c_i64, c_float, c_void_p, c_int, c_i64, c_float,
                                  c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "vila_causal_conv_rows": [C.POINTER(CausalConvParams), c_void_p],
    "vila_causal_conv_state": [C.POINTER(CausalConvParams), c_void_p],
    "vila_ssd_scan": [C.POINTER(SsdScanParams), c_void_p],
    "vila_selective_scan": [C.POINTER(SelectiveScanParams), c_void_p],
}
_RESTYPES = {"vila_last_error": C.c_char_p}

_lib = None


def lib_path() -> Path:
    return _LIB_PATH


def load() -> C.CDLL:
    """Load the shared library (raises if it has not been built)."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} not found: build it with `python -m vila_b200.build` "
            "(vila_b200 has no CPU / PyTorch fallback path)")
    lib = C.CDLL(str(_LIB_PATH))
    lib.vila_last_error.restype = C.c_char_p
    lib.vila_last_error.argtypes = []
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.argtypes = argtypes
        fn.restype = c_int
    _lib = lib
    return lib


LAUNCHES = 0  # number of C-ABI compute calls issued from this process (bench.py reports it)


def check(rc: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        msg = load().vila_last_error()
        raise RuntimeError(f"{what} failed (rc={rc}): {msg.decode() if msg else '?'}")
