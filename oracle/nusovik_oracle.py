"""Plain, slow restatement of the Nusovik architecture in float64 PyTorch (test infrastructure only;
the product never imports it).  One function per mechanism; whole sequences only: no cache, no
pages, no state slots, no batching, no fused forms, so every schedule of the engine can be compared
against it.

Notation: x residual [T, width]; W[name] checkpoint tensors (linear weights [out, in]); t a position
(0-based inside its sequence); rms(v) = v / sqrt(mean(v^2) + eps)."""
from __future__ import annotations

import math
from typing import Dict, List

import torch

F64 = torch.float64


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)


def silu(v: torch.Tensor) -> torch.Tensor:
    return v * torch.sigmoid(v)


def softplus(v: torch.Tensor) -> torch.Tensor:
    return torch.where(v > 30.0, v, torch.log1p(torch.exp(torch.clamp_max(v, 30.0))))


def sinusoid(T: int, width: int) -> torch.Tensor:
    """row t: column 2i = sin(t * 10000^(-2i / width)), column 2i + 1 = cos of the same angle"""
    out = torch.zeros(T, width, dtype=F64)
    t = torch.arange(T, dtype=F64)
    for c in range(width):
        i = c // 2
        ang = t * (10000.0 ** (-2.0 * i / width))
        out[:, c] = torch.cos(ang) if c % 2 else torch.sin(ang)
    return out


def token_embedding(W, tokens, scale: float) -> torch.Tensor:
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = W["embed"][ids] * scale
    return x + sinusoid(len(ids), x.shape[1])


def distance_bucket(n: int, rows: int, far: int) -> int:
    """row of the distance-bias table for a key n >= 0 positions back: exact below rows // 2, then
    log-spaced up to distance `far`, the last row from there on"""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def causal_conv(u: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps] (tap taps - 1 meets the newest input), nothing before position 0"""
    T, taps = u.shape[0], w.shape[1]
    out = b.expand(T, -1).clone()
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out


def chunked_sink_attention(h, W, p, m, eps) -> torch.Tensor:
    """grouped-query heads, values = the un-normed keys, RMS-normed q / k, distance bias, a query sees
    the earlier keys of its own chunk of positions, softmax with a per-head sink, per-head output gate"""
    T, H, G, d = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, d)
    v = k
    q = rms(q, eps) * W[p + "q.norm"]
    k = rms(k, eps) * W[p + "k.norm"]
    rel, size = W[p + "rel"], m["mask"]["size"]
    gate = torch.sigmoid(h @ W[p + "g"].T)
    out = torch.zeros(T, H, d, dtype=h.dtype)
    row = torch.tensor([distance_bucket(n, rel.shape[0], m["bias_max"]) for n in range(T)], dtype=torch.long)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = (i // size) * size
            back = i - torch.arange(lo, i + 1)                     # distance of every visible key
            s = k[lo:i + 1, g] @ q[i, hd] * m["scale"] + rel[row[back], hd]
            mx = torch.maximum(s.max(), W[p + "sink"][hd])
            e = torch.exp(s - mx)
            wgt = e / (e.sum() + torch.exp(W[p + "sink"][hd] - mx))
            out[i, hd] = (wgt[:, None] * v[lo:i + 1, g]).sum(0) * gate[i, hd]
    return out.reshape(T, H * d) @ W[p + "o"].T


def ssd_mixer(h, W, p, m, eps) -> torch.Tensor:
    """state-space duality recurrence: scalar decay per head, state [N, vdim] per head"""
    T, H, P, N, G = h.shape[0], m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    u = h @ W[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        a = torch.exp(W[p + "A_log"][hd])
        for t in range(T):
            S = torch.exp(-a * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + W[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms(y.view(T, ng, inner // ng), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def selective_scan_mixer(h, W, p, m) -> torch.Tensor:
    """selective state-space recurrence: a state [inner, N], step size and decay per channel"""
    T, inner, N, R = h.shape[0], m["inner"], m["state"], m["dt_rank"]
    u = h @ W[p + "in"].T
    x, z = u[:, :inner], u[:, inner:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    r = x @ W[p + "x"].T
    dt = softplus(r[:, :R] @ W[p + "dt"].T + W[p + "dt.b"])
    B, C = r[:, R:R + N], r[:, R + N:]
    A = -torch.exp(W[p + "A_log"])
    S = torch.zeros(inner, N, dtype=h.dtype)
    y = torch.zeros(T, inner, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + W[p + "D"] * x[t]
    return (y * silu(z)) @ W[p + "o"].T


def feed_forward(h, W, p) -> torch.Tensor:
    return torch.relu(h @ W[p + "up"].T).pow(2) @ W[p + "down"].T


def mixer(x, W, p, spec, eps) -> torch.Tensor:
    m = spec["mixer"]
    if spec["type"] == "mamba1":
        return selective_scan_mixer(x, W, p, m)
    if spec["type"] == "parallel":
        return m["left_scale"] * chunked_sink_attention(x, W, p + "left.", m["left"], eps) + \
            m["right_scale"] * ssd_mixer(x, W, p + "right.", m["right"], eps)
    raise ValueError(spec["type"])


def layer(x, W, i, spec, config) -> torch.Tensor:
    """post-norm residual layer: a sublayer takes the un-normed stream, its result is normed and added"""
    eps, p = config["norm"]["eps"], f"l{i}."
    x = x + rms(mixer(x, W, p + "mix.", spec, eps), eps) * W[p + "norm1"]
    if spec.get("mlp") is not None:
        x = x + rms(feed_forward(x, W, p + "mlp."), eps) * W[p + "norm2"]
    return x


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, layer_outputs: List[torch.Tensor] = None):
    """-> logits [T, vocab] (float64) of one whole sequence"""
    W = {k: v.to(F64) for k, v in weights.items()}
    x = token_embedding(W, tokens, config["embedding"]["scale"])
    for i, spec in enumerate(config["layers"]):
        x = layer(x, W, i, spec, config)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    h = rms(x, config["norm"]["eps"]) * W["final.norm"]
    return h @ W["head"].T * config["logit_scale"]


def greedy(config, weights, prompt, n_new: int):
    """-> (new ids, top-2 logit margin of every choice)"""
    ids, out, margins = list(prompt), [], []
    for _ in range(n_new):
        last = forward(config, weights, ids)[-1]
        top = torch.topk(last, 2).values
        tok = int(last.argmax())
        out.append(tok)
        margins.append(float(top[0] - top[1]))
        ids.append(tok)
    return out, margins
