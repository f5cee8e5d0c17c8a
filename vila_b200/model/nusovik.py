"""Nusovik: a decoder-only language model of state-space mixers and chunked attention on the ragged-batch kernels.

Residual stream x (fp32).  A token enters as its word row times `embedding.scale` plus a sinusoidal
position vector (column 2i = sin, 2i + 1 = cos of position * 10000^(-2i / width)).  The norms sit on the
OUTPUT of every sublayer; a sublayer's input is the un-normed stream:

    x += rms(mixer(x)) * norm1,      x += rms(ff(x)) * norm2      (a layer may have no feed-forward)

  mixer "mamba1"    selective state-space recurrence: in -> x | z, causal convolution + SiLU on x, a low-rank
                    step size, a state [inner, N] per sequence, y * silu(z), out
  mixer "parallel"  left_scale * attention(x) + right_scale * ssd(x), both reading the same x
      left          grouped-query heads with biased q / k projections, a token's value is its key before the norm, RMS
                    norm of q and k per head (one weight vector for all heads), no rotation, a learned bias
                    looked up by log-spaced distance buckets, a query sees the keys of its own block of
                    `mask.size` positions, softmax with a per-head sink, per-head sigmoid output gate
      right         state-space duality recurrence: in -> z | x | B | C | dt, causal convolution + SiLU on
                    x | B | C, one decay per head, a state [N, vdim] per head, y * silu(z), RMS norm in
                    `norm_groups` pieces, out
  feed-forward      down(relu(up(x))^2)

One step takes a RaggedBatch and a HybridCache owned by the serving engine (vila_b200/serving.py): the
attention layers keep k | v rows in a paged pool, the recurrent mixers a convolution tail and a recurrent
state per sequence slot.  dtype bfloat16: projections on the tcgen05 GEMM (shapes it does not take go to
the CUDA-core grouped kernel), convolution outputs in bf16; positions and angles, norms, scores and softmax,
step sizes, decays, states and the residual sums in fp32.  dtype float32: the same kernels with fp32
tensors and the CUDA-core linear layer throughout.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from .moronex import read_safetensors

ARCHITECTURE = "Nusovik"
POSITION_BASE = 10000.0   # fixed by the architecture: base of the sinusoidal position vector


@dataclass
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: int          # distances from here on share the last row of the bias table
    chunk: int             # mask.size: a query sees the keys of its own block of this many positions
    bias_rows: int = 0     # rows of the bias table; 0: taken from the checkpoint tensor


@dataclass
class SsdConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state


@dataclass
class SelectiveConfig:
    inner: int
    state: int
    dt_rank: int
    conv: int


@dataclass
class NusovikLayerConfig:
    type: str                                   # "parallel" | "mamba1"
    left: Optional[ChunkedAttentionConfig] = None
    right: Optional[SsdConfig] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    selective: Optional[SelectiveConfig] = None
    ff: int = 0                                 # 0: no feed-forward


def distance_rows(bias_rows: int, bias_max: int) -> List[int]:
    """row of the bias table for every distance 0 .. bias_max (larger distances use the last entry):
    the distance itself below half the rows, then log-spaced up to bias_max"""
    half = bias_rows // 2
    out = []
    for n in range(bias_max + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(bias_rows - 1,
                           half + int(math.floor(math.log(n / half) / math.log(bias_max / half) * (bias_rows - half)))))
    return out


@dataclass
class NusovikConfig:
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    logit_scale: float
    layers: List[NusovikLayerConfig] = field(default_factory=list)
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(d: dict) -> "NusovikConfig":
        layers = []
        for i, spec in enumerate(d["layers"]):
            m, kind = spec["mixer"], spec["type"]
            if kind == "parallel":
                a, r = m["left"], m["right"]
                lc = NusovikLayerConfig(
                    type=kind,
                    left=ChunkedAttentionConfig(heads=int(a["heads"]), kv_heads=int(a["kv_heads"]), dim=int(a["dim"]),
                                                vdim=int(a["vdim"]), scale=float(a["scale"]),
                                                bias_max=int(a["bias_max"]), chunk=int(a["mask"]["size"]),
                                                bias_rows=int(a.get("bias_rows", 0))),
                    right=SsdConfig(heads=int(r["heads"]), vdim=int(r["vdim"]), state=int(r["state"]),
                                    groups=int(r["groups"]), norm_groups=int(r["norm_groups"]), conv=int(r["conv"])),
                    left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))
            elif kind == "mamba1":
                lc = NusovikLayerConfig(type=kind, selective=SelectiveConfig(
                    inner=int(m["inner"]), state=int(m["state"]), dt_rank=int(m["dt_rank"]), conv=int(m["conv"])))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            mlp = spec.get("mlp")
            if mlp is not None:
                if mlp["kind"] != "dense":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
                lc.ff = int(mlp["ff"])
            layers.append(lc)
        cfg = NusovikConfig(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                            embed_scale=float(d["embedding"]["scale"]), logit_scale=float(d["logit_scale"]),
                            layers=layers)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, lc in enumerate(self.layers):
            if lc.type == "parallel":
                a, r = lc.left, lc.right
                if a.heads % a.kv_heads or a.vdim != a.dim:
                    raise ValueError(f"layer {i}: heads {a.heads} / kv_heads {a.kv_heads}; the values are the keys, "
                                     f"so vdim {a.vdim} must equal dim {a.dim}")
                if a.chunk < 1 or (a.bias_rows and (a.bias_rows < 2 or a.bias_max <= a.bias_rows // 2)):
                    raise ValueError(f"layer {i}: mask.size {a.chunk}, bias rows {a.bias_rows}, bias_max {a.bias_max}")
                if r.heads % r.groups or r.inner % r.norm_groups or not 1 <= r.conv <= 16 or r.state > 256:
                    raise ValueError(f"layer {i}: ssd heads {r.heads} groups {r.groups} norm_groups {r.norm_groups} "
                                     f"conv {r.conv} state {r.state}")
            elif lc.type == "mamba1":
                s = lc.selective
                if not 1 <= s.conv <= 16 or s.state > 256 or s.dt_rank < 1:
                    raise ValueError(f"layer {i}: conv {s.conv} state {s.state} dt_rank {s.dt_rank}")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {lc.type!r}")

    def to_dict(self) -> dict:
        out = []
        for lc in self.layers:
            if lc.type == "parallel":
                a, r = lc.left, lc.right
                m = {"left": {"bias_max": a.bias_max, "dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads,
                              "mask": {"size": a.chunk}, "scale": a.scale, "vdim": a.vdim},
                     "left_scale": lc.left_scale,
                     "right": {"conv": r.conv, "groups": r.groups, "heads": r.heads, "norm_groups": r.norm_groups,
                               "state": r.state, "vdim": r.vdim},
                     "right_scale": lc.right_scale}
            else:
                s = lc.selective
                m = {"conv": s.conv, "dt_rank": s.dt_rank, "inner": s.inner, "state": s.state}
            out.append({"mixer": m, "mlp": {"ff": lc.ff, "kind": "dense"} if lc.ff else None, "type": lc.type})
        return {"architecture": self.architecture, "embedding": {"scale": self.embed_scale}, "layers": out,
                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
                "width": self.width}

    def tensor_shapes(self) -> Dict[str, tuple]:
        """name -> shape of every checkpoint tensor (the layout `load_weights` expects); the row count of
        a bias table whose `bias_rows` is 0 is reported as -1 (any)."""
        W, s = self.width, {}
        s["embed"] = (self.vocab, W)
        for i, lc in enumerate(self.layers):
            p = f"l{i}."
            s[p + "norm1"] = (W,)
            if lc.ff:
                s[p + "norm2"] = (W,)
            if lc.type == "parallel":
                a, r, q = lc.left, lc.right, p + "mix.left."
                s[q + "q"], s[q + "q.b"] = (a.heads * a.dim, W), (a.heads * a.dim,)
                s[q + "k"], s[q + "k.b"] = (a.kv_heads * a.dim, W), (a.kv_heads * a.dim,)
                s[q + "q.norm"], s[q + "k.norm"] = (a.dim,), (a.dim,)
                s[q + "rel"], s[q + "sink"] = (a.bias_rows or -1, a.heads), (a.heads,)
                s[q + "g"], s[q + "o"] = (a.heads, W), (W, a.heads * a.vdim)
                q = p + "mix.right."
                s[q + "in"] = (2 * r.inner + 2 * r.groups * r.state + r.heads, W)
                s[q + "conv"], s[q + "conv.b"] = (r.conv_channels, r.conv), (r.conv_channels,)
                s[q + "dt_bias"], s[q + "A_log"], s[q + "D"] = (r.heads,), (r.heads,), (r.heads,)
                s[q + "norm"], s[q + "o"] = (r.inner,), (W, r.inner)
            else:
                m, q = lc.selective, p + "mix."
                s[q + "in"] = (2 * m.inner, W)
                s[q + "conv"], s[q + "conv.b"] = (m.inner, m.conv), (m.inner,)
                s[q + "x"] = (m.dt_rank + 2 * m.state, m.inner)
                s[q + "dt"], s[q + "dt.b"] = (m.inner, m.dt_rank), (m.inner,)
                s[q + "A_log"], s[q + "D"] = (m.inner, m.state), (m.inner,)
                s[q + "o"] = (W, m.inner)
            if lc.ff:
                s[p + "mlp.up"], s[p + "mlp.down"] = (lc.ff, W), (W, lc.ff)
        s["final.norm"], s["head"] = (W,), (self.vocab, W)
        return s


class _Layer:
    """Device tensors of one layer in the layout the kernels want."""


def _pad_rows(w: torch.Tensor, mult: int = 8) -> torch.Tensor:
    """zero rows up to a multiple of `mult` output features (the tensor-core GEMM wants 16-byte output rows)"""
    extra = (-w.shape[0]) % mult
    if extra == 0:
        return w.contiguous()
    return torch.cat([w, w.new_zeros((extra,) + tuple(w.shape[1:]))], 0).contiguous()


class NusovikForCausalLM:
    """Weights + the per-step compute of the architecture.  Sequences, pages, state slots, batching and
    sampling belong to `vila_b200.serving.TokenEngine`, which calls `forward_step` / `logits`."""

    def __init__(self, cfg: NusovikConfig, device="cuda", dtype=torch.bfloat16):
        assert dtype in (torch.bfloat16, torch.float32)
        cfg.validate()
        self.config, self.device, self.dtype = cfg, torch.device(device), dtype
        self.vocab_size = cfg.vocab
        self.weights: Dict[str, torch.Tensor] = {}
        self.layers: List[_Layer] = []

    # ---- weights ----------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir, device="cuda", dtype=torch.bfloat16) -> "NusovikForCausalLM":
        d = Path(model_dir)
        cfg = NusovikConfig.from_dict(json.loads((d / "config.json").read_text()))
        files = sorted(d.glob("*.safetensors"))
        if not files:
            raise FileNotFoundError(f"no *.safetensors under {d}")
        tensors: Dict[str, torch.Tensor] = {}
        for f in files:
            tensors.update(read_safetensors(f))
        return cls(cfg, device, dtype).load_weights(tensors)

    def init_random(self, seed: int = 0, scale: float = 1.0, on_device: bool = False, bias_rows: int = 32
                    ) -> "NusovikForCausalLM":
        """Random bf16-representable weights.  on_device: draw them on the model's device (large models)."""
        dev = self.device if on_device else torch.device("cpu")
        g = torch.Generator(device=dev).manual_seed(seed)
        t = {}
        for name, shape in self.config.tensor_shapes().items():
            shape = tuple(bias_rows if n < 0 else n for n in shape)
            last = name.rsplit(".", 1)[-1]
            if last == "A_log":     # decay rates 1 .. 8
                v = torch.log(1.0 + 7.0 * torch.rand(shape, generator=g, device=dev))
            elif last == "dt_bias" or name.endswith("dt.b"):   # step sizes around 0.01 .. 0.1 after softplus
                v = -4.6 + 2.3 * torch.rand(shape, generator=g, device=dev)
            elif last == "conv":
                v = torch.randn(shape, generator=g, device=dev) * 0.4
            elif last == "rel":
                v = torch.randn(shape, generator=g, device=dev) * 0.5
            elif last == "sink":
                v = torch.randn(shape, generator=g, device=dev)
            elif last == "D":
                v = 1.0 + torch.randn(shape, generator=g, device=dev) * 0.2
            elif name.endswith("mix.dt"):   # small step-size pre-activations: a decay exp(-a dt) multiplies their error by a
                v = torch.randn(shape, generator=g, device=dev) * (0.2 / shape[1] ** 0.5)
            elif len(shape) == 2:
                v = torch.randn(shape, generator=g, device=dev) * (scale / shape[1] ** 0.5)
            elif "norm" in name:
                v = 1.0 + torch.randn(shape, generator=g, device=dev) * 0.1
            else:
                v = torch.randn(shape, generator=g, device=dev) * 0.1
            t[name] = v.to(torch.bfloat16)
        return self.load_weights(t)

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> "NusovikForCausalLM":
        """tensors: checkpoint name -> tensor ([out, in] linear weights).  Sizes are checked against the
        config; the fused device layouts and the distance-bias lookup are built here."""
        cfg, dev, dt = self.config, self.device, self.dtype
        want = cfg.tensor_shapes()
        missing = [n for n in want if n not in tensors]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:4]}{'...' if len(missing) > 4 else ''}")
        for n, shape in want.items():
            got = tuple(tensors[n].shape)
            if len(got) != len(shape) or any(b >= 0 and a != b for a, b in zip(got, shape)):
                raise ValueError(f"{n}: checkpoint shape {got} != config shape {shape}")

        def w(name):  # compute-dtype copy
            return tensors[name].to(device=dev, dtype=dt).contiguous()

        def f32(name):
            return tensors[name].to(device=dev, dtype=torch.float32).contiguous()

        self.weights = {n: tensors[n] for n in want}
        self.embed, self.head, self.final_norm = w("embed"), w("head"), f32("final.norm")
        half = (cfg.width + 1) // 2
        self.inv_freq = (torch.tensor(POSITION_BASE, dtype=torch.float64) **
                         (-2.0 * torch.arange(half, dtype=torch.float64) / cfg.width)).to(dev)
        self.layers = []
        for i, lc in enumerate(cfg.layers):
            p, L = f"l{i}.", _Layer()
            L.cfg, L.index = lc, i
            L.norm1 = f32(p + "norm1")
            if lc.type == "parallel":
                a, r, q = lc.left, lc.right, p + "mix.left."
                rows = tensors[q + "rel"].shape[0]
                if rows < 2 or a.bias_max <= rows // 2:
                    raise ValueError(f"{q}rel: {rows} rows with bias_max {a.bias_max}")
                # q | k | gate in one projection; the gate has no bias
                L.qkg = _pad_rows(torch.cat([w(q + "q"), w(q + "k"), w(q + "g")], 0))
                L.qkg_b = torch.zeros(L.qkg.shape[0], device=dev, dtype=dt)
                L.qkg_b[:(a.heads + a.kv_heads) * a.dim] = torch.cat([w(q + "q.b"), w(q + "k.b")])
                L.q_norm, L.k_norm, L.sink = f32(q + "q.norm"), f32(q + "k.norm"), f32(q + "sink")
                # bias by distance: the bucket rows laid out per distance 0 .. bias_max
                idx = torch.tensor(distance_rows(rows, a.bias_max), dtype=torch.long, device=dev)
                L.dist_bias = f32(q + "rel").index_select(0, idx).contiguous()
                L.attn_o = w(q + "o")
                q = p + "mix.right."
                L.ssd_in = _pad_rows(w(q + "in"))
                L.ssd_conv, L.ssd_conv_b = f32(q + "conv"), f32(q + "conv.b")
                L.dt_bias, L.A_log, L.D = f32(q + "dt_bias"), f32(q + "A_log"), f32(q + "D")
                L.ssd_norm, L.ssd_o = f32(q + "norm"), w(q + "o")
            else:
                q = p + "mix."
                L.sel_in = _pad_rows(w(q + "in"))
                L.sel_conv, L.sel_conv_b = f32(q + "conv"), f32(q + "conv.b")
                L.sel_x, L.sel_dt = _pad_rows(w(q + "x")), _pad_rows(w(q + "dt"))
                L.dt_bias, L.A_log, L.D = f32(q + "dt.b"), f32(q + "A_log"), f32(q + "D")
                L.sel_o = w(q + "o")
            if lc.ff:
                L.norm2 = f32(p + "norm2")
                L.up, L.down = _pad_rows(w(p + "mlp.up")), w(p + "mlp.down")
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
        """layer -> width of its paged per-token row: normed keys (kv_heads * dim) | values = raw keys"""
        return {i: lc.left.kv_heads * (lc.left.dim + lc.left.vdim)
                for i, lc in enumerate(self.config.layers) if lc.type == "parallel"}

    def state_shapes(self) -> Dict[Tuple[int, str], tuple]:
        """(layer, "conv") -> (taps - 1, channels): the convolution's last inputs; (layer, "ssm") -> the
        recurrent state ([heads, vdim, N] per head-wise mixer, [inner, N] per channel-wise one)"""
        out = {}
        for i, lc in enumerate(self.config.layers):
            if lc.type == "parallel":
                r = lc.right
                conv, chans, state = r.conv, r.conv_channels, (r.heads, r.vdim, r.state)
            else:
                m = lc.selective
                conv, chans, state = m.conv, m.inner, (m.inner, m.state)
            if conv > 1:
                out[(i, "conv")] = (conv - 1, chans)
            out[(i, "ssm")] = state
        return out

    # ---- compute --------------------------------------------------------------------------------------
    def _attention(self, L: _Layer, h, batch, cache):
        a = L.cfg.left
        pool = cache.latent[L.index]
        P = ops.linear_any(h, L.qkg, bias=L.qkg_b)                       # q | k | gate
        q = ops.rope_append(P, batch.positions, batch.cache_rows, pool, heads=a.heads, kv_heads=a.kv_heads,
                            dim=a.dim, vdim=a.vdim, inv_freq=None, unit_norm=True, eps=self.config.norm_eps,
                            q_norm_w=L.q_norm, k_norm_w=L.k_norm, v_from_k=True)
        g0 = (a.heads + a.kv_heads) * a.dim
        o = torch.empty(h.shape[0], a.heads * a.vdim, dtype=self.dtype, device=self.device)
        kw = dict(heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim, page=cache.page, scale=a.scale,
                  sink=L.sink, dist_bias=L.dist_bias, chunk=a.chunk, gate=P[:, g0:g0 + a.heads], out=o)
        if batch.tiles is not None:
            ops.paged_attention(q, pool, cache.page_tables, batch.tiles, max_rows=16, **kw)
        if batch.decode_tiles is not None:
            ops.paged_attention(q, pool, cache.page_tables, batch.decode_tiles, max_rows=1,
                                nsplit=cache.decode_splits, **kw)
        return ops.linear_any(o, L.attn_o)

    def _ssd(self, L: _Layer, h, batch, cache):
        r = L.cfg.right
        inner, chans = r.inner, r.conv_channels
        P = ops.linear_any(h, L.ssd_in)                                    # z | x | B | C | dt
        xbc = ops.causal_conv_rows(P[:, inner:inner + chans], L.ssd_conv, L.ssd_conv_b,
                                   cache.state.get((L.index, "conv")), batch.seqs, batch.row_seq,
                                   act=ops.CONV_SILU, out_dtype=self.dtype)
        y = ops.ssd_scan(xbc, P[:, inner + chans:inner + chans + r.heads], P[:, :inner],
                         cache.state[(L.index, "ssm")], batch.seqs, heads=r.heads, vdim=r.vdim, nstate=r.state,
                         groups=r.groups, dt_bias=L.dt_bias, A_log=L.A_log, D=L.D)
        yn = ops.rmsnorm_rows(y, L.ssd_norm, self.config.norm_eps, groups=r.norm_groups, out_dtype=self.dtype)
        return ops.linear_any(yn, L.ssd_o)

    def _selective(self, L: _Layer, h, batch, cache):
        m = L.cfg.selective
        P = ops.linear_any(h, L.sel_in)                                    # x | z
        x = ops.causal_conv_rows(P[:, :m.inner], L.sel_conv, L.sel_conv_b, cache.state.get((L.index, "conv")),
                                 batch.seqs, batch.row_seq, act=ops.CONV_SILU, out_dtype=self.dtype)
        r = ops.linear_any(x, L.sel_x)                                     # dt (low rank) | B | C
        dt = ops.linear_any(r[:, :m.dt_rank], L.sel_dt)
        y = ops.selective_scan(x, dt[:, :m.inner], r[:, m.dt_rank:m.dt_rank + 2 * m.state], P[:, m.inner:2 * m.inner],
                               cache.state[(L.index, "ssm")], batch.seqs, dt_bias=L.dt_bias, A_log=L.A_log, D=L.D,
                               out_dtype=self.dtype)
        return ops.linear_any(y, L.sel_o)

    @torch.inference_mode()
    def forward_step(self, batch, cache, layer_outputs: Optional[list] = None) -> torch.Tensor:
        """Run the rows of `batch` through all layers on top of what `cache` holds; k | v rows, convolution
        tails and recurrent states of the batch are written to the cache.  -> residual stream fp32 [T, width]."""
        cfg, eps = self.config, self.config.norm_eps
        copy = self.dtype if self.dtype != torch.float32 else None      # the projections' operand
        x, xc = ops.embed_sincos_rows(self.embed, batch.ids, batch.positions, self.inv_freq, cfg.embed_scale,
                                      copy_dtype=copy)
        for L in self.layers:
            h = x if copy is None else xc
            if L.cfg.type == "parallel":
                xc = ops.branch_norm_residual(x, self._attention(L, h, batch, cache), L.norm1, eps,
                                              a_scale=L.cfg.left_scale, b=self._ssd(L, h, batch, cache),
                                              b_scale=L.cfg.right_scale, copy_dtype=copy)
            else:
                xc = ops.branch_norm_residual(x, self._selective(L, h, batch, cache), L.norm1, eps, copy_dtype=copy)
            if L.cfg.ff:
                h = x if copy is None else xc
                u = ops.linear_any(h, L.up, act=ops.ACT_RELU2)
                xc = ops.branch_norm_residual(x, ops.linear_any(u[:, :L.cfg.ff], L.down), L.norm2, eps,
                                              copy_dtype=copy)
            if layer_outputs is not None:
                layer_outputs.append(x.clone())
        return x

    @torch.inference_mode()
    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        """final norm + output head for the given residual rows fp32 [n, width] -> fp32 [n, vocab]"""
        cfg = self.config
        h = ops.rmsnorm_rows(hidden_rows.contiguous(), self.final_norm, cfg.norm_eps, out_dtype=self.dtype)
        return ops.glinear(h, self.head, out_dtype=torch.float32).mul_(cfg.logit_scale)

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
