"""Plain, slow restatement of the Ludazen architecture in float64 PyTorch (test infrastructure only;
the product never imports it).  One function per mechanism; whole sequences only: no cache, no
pages, no batching, no folded or fused forms, so every schedule of the engine can be compared
against it.

Notation: x residual [T, width]; W[name] checkpoint tensors (linear weights [out, in]); t, s query
and key positions (0-based inside the sequence); unit(v) = v / sqrt(mean(v^2) + eps)."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def unit(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-z.abs())) + z.clamp(min=0)


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2"""
    ap = softplus(torch.tensor(p, dtype=F64))
    an = 0.5 + softplus(torch.tensor(q, dtype=F64))
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(z.clamp(max=0)) - z) + 0.5 * z)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ---- rotary positions -----------------------------------------------------------------------------
def rotary_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i / dims); with `scaling`: the slow frequencies are divided by `factor`, the fast ones
    kept, a linear ramp over the pair index in between"""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f

    def pair_of(turns):   # the pair index whose wavelength fits `turns` times into the original length
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp)


def rotary_magnitude(rot: dict) -> float:
    sc = rot.get("scaling")
    return 0.1 * math.log(sc["factor"]) + 1.0 if sc else 1.0


def rotate(v: torch.Tensor, rot: dict, layout: str) -> torch.Tensor:
    """v [T, heads, dim]: the first rot.dims columns turn by t * f_i.  layout "halves": column i pairs with
    i + dims / 2; "pairs": column 2i with 2i + 1.  The rest passes unchanged."""
    T, dims = v.shape[0], int(rot["dims"])
    out = v.clone()
    if dims == 0:
        return out
    ang = torch.arange(T, dtype=F64)[:, None] * rotary_frequencies(rot)[None, :]
    mag = rotary_magnitude(rot)
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    if layout == "halves":
        a, b = v[..., :dims // 2], v[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = a * c - b * s, b * c + a * s
    else:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = a * c - b * s, b * c + a * s
    return out


# ---- masks ----------------------------------------------------------------------------------------
def window_mask(T: int, size: int, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: t sees s when s <= t and (t - s < size or s < keep_first)"""
    t = torch.arange(T)[:, None]
    s = torch.arange(T)[None, :]
    return (s <= t) & ((t - s < size) | (s < keep_first))


# ---- mixers ---------------------------------------------------------------------------------------
def attention(W, p: str, h: torch.Tensor, m: dict) -> torch.Tensor:
    """grouped-query heads, rotation in the halves layout, per-head temperature, window with kept first
    tokens, softmax, then the heads' WEIGHTS are mixed by `talk`; head a uses the values of its own group"""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate((h @ W[p + "q"].T).view(T, H, D), m["rot"], "halves")
    k = rotate((h @ W[p + "k"].T).view(T, G, D), m["rot"], "halves")
    v = (h @ W[p + "v"].T).view(T, G, V)
    grp = torch.arange(H) // (H // G)
    sc = torch.einsum("thd,shd->hts", q, k[:, grp]) * m["scale"] * W[p + "temp"][:, None, None]
    mask = window_mask(T, m["mask"]["size"], m["mask"].get("keep_first", 0))
    wts = torch.softmax(sc.masked_fill(~mask[None], float("-inf")), dim=-1)
    wts = torch.einsum("ab,bts->ats", W[p + "talk"], wts)
    o = torch.einsum("hts,shv->thv", wts, v[:, grp]).reshape(T, H * V)
    return o @ W[p + "o"].T


def latent_rows(W, p: str, h: torch.Tensor, m: dict, eps: float):
    """what a latent-attention layer keeps per token: the normed latent c [T, kv_rank] and the shared
    rotated key part [T, rot_dim]"""
    R = m["kv_rank"]
    d = h @ W[p + "dkv"].T
    c = unit(d[:, :R], eps) * W[p + "dkv.norm"]
    kr = rotate(d[:, None, R:], m["rot"], "pairs")[:, 0]
    return c, kr


def latent_attention(W, p: str, h: torch.Tensor, m: dict, c: torch.Tensor, kr: torch.Tensor) -> torch.Tensor:
    """keys and values expanded per head from the latent; every head's query has an unrotated part that
    meets the expanded key and a rotated part that meets the one shared rotated key part"""
    T = h.shape[0]
    H, D, Dr, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, D + Dr)
    qn, qr = q[..., :D], rotate(q[..., D:], m["rot"], "pairs")
    kn = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, V)
    sc = (torch.einsum("thd,shd->hts", qn, kn) + torch.einsum("thd,sd->hts", qr, kr)) * m["scale"]
    mask = window_mask(T, m["mask"]["size"])
    wts = torch.softmax(sc.masked_fill(~mask[None], float("-inf")), dim=-1)
    return torch.einsum("hts,shv->thv", wts, v).reshape(T, H * V) @ W[p + "o"].T


# ---- feed-forwards --------------------------------------------------------------------------------
def dense_ff(W, p: str, h: torch.Tensor) -> torch.Tensor:
    a = xielu(h @ W[p + "up"].T + W[p + "up.b"], float(W[p + "act"][0]), float(W[p + "act"][1]))
    return a @ W[p + "down"].T + W[p + "down.b"]


def gated_unit(W, p: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(W, p: str, h: torch.Tensor, top: int):
    """-> (chosen experts [T, top], their sigmoid scores [T, top]); the scores are the weights as they are"""
    s = torch.sigmoid(h @ W[p + "router"].T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


def expert_ff(W, p: str, h: torch.Tensor, mlp: dict) -> torch.Tensor:
    """sum over the chosen experts of expert(weight * h) (the weight scales the expert's INPUT) + shared expert"""
    idx, wt = route(W, p, h, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t].tolist(), wt[t]):
            out[t] += gated_unit(W, f"{p}e{e}.", (w * h[t])[None])[0]
    if mlp.get("shared"):
        out = out + gated_unit(W, p + "shared.", h)
    return out


# ---- the model ------------------------------------------------------------------------------------
def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens, layer_outputs: Optional[List] = None) -> torch.Tensor:
    """tokens of ONE sequence -> logits [T, vocab] (float64)"""
    W = {n: t.to(F64) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        h = unit(x, eps) * W[p + "norm1"]
        if spec["type"] == "attention":
            x = x + attention(W, p + "mix.", h, m)
        elif spec["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_rows(W, p + "mix.", h, m, eps)
            c, kr = kept[i if m.get("kv_from") is None else m["kv_from"]]
            x = x + latent_attention(W, p + "mix.", h, m, c, kr)
        else:
            raise ValueError(spec["type"])
        mlp = spec.get("mlp")
        if mlp is not None:
            h = unit(x, eps) * W[p + "norm2"]
            x = x + (dense_ff(W, p + "mlp.", h) if mlp["kind"] == "dense" else expert_ff(W, p + "mlp.", h, mlp))
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return (unit(x, eps) * W["final.norm"]) @ W["head"].T
