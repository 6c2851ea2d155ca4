"""GPU engine for layer-list models: a model directory (config.json + model.safetensors) whose configuration lists its
layers one by one, each a token mixer followed by an optional feed-forward, with dense bf16 weights.  How a sublayer
meets the residual stream is the architecture's ``residual`` style (``RESIDUAL_STYLES``), everything in f32:

    "sandwich":  x <- x + post_norm(sub(pre_norm(x)))                    norm weights stored around zero (Ribivik)
    "hyper":     u = sum_s in[s] x_s;  y = sub(norm(u));  x_t <- sum_s mix[s][t] x_s + m out[t] y      (Sunesun)
                 `streams` copies of the stream (hyper-connections); without them the plain x <- x + m sub(norm(x)),
                 which is how Venadra's pre-norm layers run (one stream, m = 1)
    "post":      x <- x + m * norm(sub(x))                               the sublayer reads the stream itself; the only
                 norm sits on its output (Darusun)

What a design fixes without saying it in config.json (how its attention masks, whether its experts are gated, ...) is
its entry of ``DESIGNS``; everything config.json gives is read from there.  A configuration with ``canon: {taps}`` puts a
short causal convolution in front of every mixer: h <- h + conv(h) on the normed input, the last taps - 1 inputs kept per
sequence slot and layer.

The mixers and feed-forwards are looked up by name (``MIXERS`` / ``FEED_FORWARDS`` below), so another design composes
the same mechanisms with its own sizes and order; ``ARCHITECTURES`` in models/registry.py maps an architecture name to
this engine.  Mixers here:

* ``latent_attention`` -- attention whose keys and values are up-projections of one small cached latent per token plus
  a rotated key part shared by all heads; a layer may read the cache another layer writes (``kv_from``);
* ``mamba2`` -- a gated selective state-space recurrence with a short causal convolution in front;
* ``attention`` -- grouped-query attention over a paged cache of one line per token and key/value head.  Per design:
  values that are the keys (one projection) or have a projection of their own; a sliding window or a chunked mask;
  interleaved rotary positions with optional frequency interpolation, or none; soft-capped scores; queries and keys
  divided by their root mean square; a sink per head in the softmax denominator; a sigmoid output gate; rotary in the
  rotate-half layout in front of the unit norm; scores mixed across heads by a matrix `talk` before the softmax (folded
  into the queries, see WindowAttentionMixer); a layer that reads another layer's keys and values (``kv_from``);
* ``lightning`` -- linear attention with a fixed decay per head and an f32 state [dim][vdim] per head and slot, SiLU on
  q, k and v, an RMS norm over the concatenated heads and a sigmoid output gate.

Feed-forwards: ``dense`` (squared ReLU, PolyNorm, or xIELU) and ``moe`` (sigmoid-scored, group-limited routing over small
squared-ReLU experts; or softmax-scored, renormalised routing over gated experts, with an optional router bias and a
shared expert behind a sigmoid gate per token).  A layer with ``weights_of: j`` runs
layer j's weights on a cache or state of its own (a looped layer).

What the engine shares with ``LlamaEngine`` is the serving surface (slots, rows with per-row positions, paged token
cache from ``PageAllocator``, ``forward`` / ``decode_step_greedy`` / ``prefill``), so the scheduler, the batching loop
and the command line drive it unchanged.  Per sequence slot it owns pages of every latent cache and one row of every
recurrent layer's state pools; a sequence that starts again at position 0 starts from zeros whatever its slot held.

Numerics: ``dtype="bfloat16"`` keeps weights and caches in bf16 and rounds the activation operand of every matrix
product to bf16 (f32 accumulation); norms, softmax, rotary angles, the residual stream, the recurrence with its decays
and step sizes are f32.  ``dtype="float32"`` widens weights and caches to f32 and rounds nothing.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..formats.safetensors import SafetensorsFile
from .memory import graph_capture
from .paging import PAGE, PageAllocator


# --------------------------------------------------------------------------------------------------
# configuration
# --------------------------------------------------------------------------------------------------
@dataclass
class LayerSpec:
    type: str
    mixer: dict
    mlp: Optional[dict]
    weights_of: Optional[int] = None       # run that layer's weights (norms, mixer, feed-forward) on a cache / state of its own


# What a design fixes outside its config.json, by architecture name.  residual: how sublayers meet the residual stream.
# attention: values ("keys": the keys as projected | "own": a projection v), mask (what mask.size means: "window" |
# "chunk"), qk_norm, sink (tensor `sink` [heads]), gate (tensor `g`: sigmoid output gate).  dense_act: "relu2" |
# "polynorm" (tensor `act` [4]) | "xielu" (tensor `act` [2]).  moe: score ("sigmoid" | "softmax"), renorm, gated (tensors
# e<n>.gate; True: a sigma(1.702 a) (1 + b) with expert.limit, "silu": silu(a) b), bias (tensor `router.b`), shared (entry
# `shared` of the mlp: one more gated expert for every token behind sigmoid(`shared.sg` . h)).  attention also: rot
# ("interleaved" | "half": the pair layout of the rotary, which own values otherwise exclude), talk (tensor `talk`
# [heads][heads] mixes the scores of the heads before the softmax).  latent: rot (the same), sink, gate ("full": one
# gate per output column | "head": one per head).  norm_weights "scalar": every norm over the width has one number.
DESIGNS = {
    "Ribivik": {"residual": "sandwich"},
    "Sunesun": {"residual": "hyper"},
    "Venadra": {"residual": "hyper",
                "attention": {"values": "own", "mask": "chunk", "qk_norm": True, "sink": True, "gate": True},
                "dense_act": "polynorm",
                "moe": {"score": "softmax", "renorm": True, "gated": True}},
    "Darusun": {"residual": "post", "norm_weights": "scalar",
                "attention": {"values": "own", "qk_norm": True, "rot": "half", "talk": True},
                "latent": {"rot": "interleaved", "sink": True, "gate": "head"},
                "dense_act": "xielu",
                "moe": {"score": "softmax", "renorm": True, "gated": "silu", "bias": True, "shared": True}},
}
RESIDUAL_STYLES = {name: d["residual"] for name, d in DESIGNS.items()}


@dataclass
class LayerListConfig:
    architecture: str
    width: int
    vocab: int
    norm_eps: float
    logit_softcap: float
    layers: List[LayerSpec] = field(default_factory=list)
    seq_len: int = 0
    residual: str = "sandwich"
    embed_scale: float = 1.0               # the embedding output is multiplied by it
    residual_mult: float = 1.0             # "hyper", "post": every sublayer output is multiplied by it on its way into the stream
    streams: int = 1                       # "hyper": copies of the residual stream
    hyper_weights: bool = False            # the layers bring hc<q>.in / .out / .mix tensors (else the plain sum)
    canon_taps: int = 0                    # > 0: h <- h + conv(h) over the last `taps` normed inputs, in front of every mixer
    traits: dict = field(default_factory=dict)      # the design's entry of DESIGNS

    # the serving code reads these names from every engine's header
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    @staticmethod
    def from_dict(c: dict) -> "LayerListConfig":
        layers = [LayerSpec(l["type"], dict(l["mixer"]), dict(l["mlp"]) if l.get("mlp") else None,
                            int(l["weights_of"]) if l.get("weights_of") is not None else None) for l in c["layers"]]
        for i, l in enumerate(layers):
            if l.weights_of is not None and (not 0 <= l.weights_of < len(layers) or layers[l.weights_of].weights_of is not None):
                raise ValueError(f"layer {i}: weights_of {l.weights_of} is not a layer with weights of its own")
        arch = c["architecture"]
        return LayerListConfig(architecture=arch, width=int(c["width"]), vocab=int(c["vocab"]),
                               norm_eps=float(c["norm"]["eps"]), logit_softcap=float(c.get("logit_softcap") or 0.0),
                               layers=layers, residual=RESIDUAL_STYLES.get(arch, "sandwich"),
                               embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)),
                               residual_mult=float(c.get("residual_mult", 1.0)),
                               streams=int(c.get("streams") or 1), hyper_weights=bool(c.get("streams")),
                               canon_taps=int((c.get("canon") or {}).get("taps") or 0), traits=DESIGNS.get(arch, {}))

    @staticmethod
    def load(model_dir: str) -> "LayerListConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return LayerListConfig.from_dict(json.load(f))

    def describe(self) -> str:
        kinds = ", ".join(f"{sum(1 for l in self.layers if l.type == t)} x {t}" for t in sorted({l.type for l in self.layers}))
        return (f"💡 Arch: {self.architecture}\n💡 Width: {self.width}\n💡 VocabSize: {self.vocab}\n"
                f"💡 nLayers: {len(self.layers)} ({kinds})\n💡 SeqLen: {self.seq_len}")


def rotary_frequencies(base: float, dims: int) -> torch.Tensor:
    """f_i = base^(-2 i / dims), i < dims / 2, in f64 (the kernels form pos * f_i in f64)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)


def interpolated_rotary(base: float, dims: int, scaling: Optional[dict]):
    """(frequencies f64 [dims / 2], magnitude).  Without `scaling`: the plain f_i and 1.  With scaling {factor, original,
    fast, slow} the slow frequencies are divided by `factor`, the fast ones kept and those between blended (YaRN):
    with d(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1),
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):  f_i' = f_i / factor * r_i + f_i (1 - r_i); cos and sin are
    multiplied by 0.1 ln(factor) + 1."""
    f = rotary_frequencies(base, dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def d(t):
        return dims * math.log(original / (2.0 * math.pi * float(t))) / (2.0 * math.log(base))

    lo, hi = max(math.floor(d(scaling["fast"])), 0), min(math.ceil(d(scaling["slow"])), dims - 1)
    i = torch.arange(dims // 2, dtype=torch.float64)
    r = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * r + f * (1.0 - r), 0.1 * math.log(factor) + 1.0


class DenseWeight:
    """A matrix [N][K] (or per-head matrices [H][N][K]) in the engine's weight type, plus -- in bf16 mode -- its image
    for the tensor-core GEMM (one per head), which serves batches of TC_MIN_ROWS rows and more."""

    def __init__(self, t: torch.Tensor, tc: bool):
        from ..ops import layers as L
        self.t = t
        self.N, self.K = int(t.shape[-2]), int(t.shape[-1])
        self.wh = None
        if tc and t.dtype == torch.bfloat16:
            self.wh = [L.make_wh(t[h]) for h in range(t.shape[0])] if t.dim() == 3 else L.make_wh(t)

    def nbytes(self) -> int:
        return self.t.numel() * self.t.element_size()


TC_MIN_ROWS = int(os.environ.get("DLLAMA_LAYERS_TC_MIN_ROWS", "32"))
CHUNKED_SCAN_MIN_ROWS = 256  # a batch holding this many rows of one sequence runs the recurrence chunk-parallel
LIGHTNING_CHUNKED_MIN_ROWS = 128     # the same for linear attention (chunks of 64 rows)
TC_HEADS_MIN_ROWS = 256      # per-head products (one small GEMM per head) take the tensor-core path from this many rows
GRAPH_MAX_ROWS = 64          # batches up to this many rows are replayed from CUDA graphs
WINDOW_MAX_SPLITS = 32       # most CTAs that share one tile's pages in the windowed-attention kernel
WINDOW_CTAS_PER_SM = 8       # pages are shared until about this many CTAs per SM run (one page in flight per CTA)


# --------------------------------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------------------------------
class LatentAttentionMixer:
    """Tensors <prefix>dq, dq.norm, uq, [dkv, dkv.norm], uk, uv, g, o.  Sizes from the layer's mixer entry: heads, dim
    (unrotated query / key dims per head), rot_dim (rotated dims per head, one shared key part), vdim, q_rank, kv_rank,
    scale, rot {base, dims}, mask.size (a sliding window; absent: all earlier positions) and kv_from (index of the layer
    whose cache this one reads).  The design's `latent` traits: rot "half" (default: dimension i pairs with i + dims / 2) |
    "interleaved" (2i with 2i + 1); sink: <prefix>sink [heads] joins the softmax denominator; gate "full" (default: <prefix>g
    [heads * vdim][width], one gate per output column) | "head" (<prefix>g [heads][width], one sigmoid gate per head)."""

    def __init__(self, eng: "LayerListEngine", index: int, m: dict, prefix: str):
        self.eng, self.index = eng, index
        tr = eng.cfg.traits.get("latent") or {}
        self.interleaved, self.head_gate = tr.get("rot", "half") == "interleaved", tr.get("gate", "full") == "head"
        self.window = int((m.get("mask") or {}).get("size") or 0)
        self.H, self.dn, self.dr, self.dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
        self.q_rank, self.rank = int(m["q_rank"]), int(m["kv_rank"])
        self.scale = float(m["scale"])
        self.rope_dims = int(m["rot"]["dims"])
        if self.rope_dims > self.dr or self.rope_dims % 2:
            raise ValueError(f"layer {index}: rotary dims {self.rope_dims} do not fit rot_dim {self.dr}")
        self.freqs = rotary_frequencies(float(m["rot"]["base"]), self.rope_dims).to(eng.device)
        self.kv_from = m.get("kv_from")
        W, V, D = eng.weight, eng.vector, eng.dense_weight
        self.w_dq, self.dq_norm, self.w_uq = D(W(prefix + "dq")), V(prefix + "dq.norm"), D(W(prefix + "uq"))
        self.w_g, self.w_o = D(W(prefix + "g")), D(W(prefix + "o"))
        H, dn, dv, r = self.H, self.dn, self.dv, self.rank
        if tuple(self.w_g.t.shape) != ((H if self.head_gate else H * dv), eng.cfg.width):
            raise ValueError(f"layer {index}: g has shape {tuple(self.w_g.t.shape)}")
        self.sink = V(prefix + "sink") if tr.get("sink") else None
        if self.sink is not None and tuple(self.sink.shape) != (H,):
            raise ValueError(f"layer {index}: sink has shape {tuple(self.sink.shape)}")
        # key up-projection per head, transposed, so that  q_lat[h] = U_k,h^T q_h  is a product against rows of K = dn
        self.w_uk_t = D(W(prefix + "uk").reshape(H, dn, r).transpose(1, 2).contiguous())
        self.w_uv = D(W(prefix + "uv").reshape(H, dv, r).contiguous())
        if self.kv_from is None:
            self.w_dkv, self.dkv_norm = D(W(prefix + "dkv")), V(prefix + "dkv.norm")
            self.cache = torch.zeros(eng.n_pages, PAGE, r + self.dr, dtype=eng.wdtype, device=eng.device)
        else:
            self.cache = None                      # bound to the owner's cache once all layers exist

    def scratch(self) -> Dict[str, int]:
        H = self.H
        return {"cq": self.q_rank, "q": H * (self.dn + self.dr), "kv": self.rank + self.dr, "q_lat": H * self.rank,
                "o_lat": H * self.rank, "o": H * self.dv, "og": H * self.dv, "gz": H}

    def bind(self, mixers: list):
        if self.kv_from is not None:
            src = mixers[int(self.kv_from)]
            if not isinstance(src, LatentAttentionMixer) or src.kv_from is not None:
                raise ValueError(f"layer {self.index}: kv_from {self.kv_from} is not a layer with a cache of its own")
            if (src.rank, src.dr, src.rope_dims, src.interleaved) != (self.rank, self.dr, self.rope_dims, self.interleaved):
                raise ValueError(f"layer {self.index}: cache shape differs from layer {self.kv_from}")
            self.cache = src.cache

    def weight_bytes(self) -> int:
        ts = [self.w_dq, self.w_uq, self.w_g, self.w_o, self.w_uk_t, self.w_uv] + ([self.w_dkv] if self.kv_from is None else [])
        return sum(t.nbytes() for t in ts)

    def forward(self, h: torch.Tensor, y: torch.Tensor, M: int):
        e, L = self.eng, self.eng.L
        H, dn, dr, dv, r = self.H, self.dn, self.dr, self.dv, self.rank
        cq, q, o, og = (e.buf(n) for n in ("cq", "q", "o", "og"))
        q_lat, o_lat = e.buf("q_lat", H * r), e.buf("o_lat", H * r)          # read as [M][H][rank], no row padding
        hd = dn + dr
        e.mm(self.w_dq, h, cq, M, src="h")
        L.rms_norm(cq, cq, M, self.q_rank, e.cfg.norm_eps, w=self.dq_norm)
        e.mm(self.w_uq, cq, q, M)
        L.rope_rows(q, M, H, hd, dn, self.rope_dims, self.freqs, e.pos, interleaved=self.interleaved)
        if self.kv_from is None:
            kv = e.buf("kv")
            e.mm(self.w_dkv, h, kv, M, src="h")
            L.latent_kv_write(kv, M, self.dkv_norm, e.cfg.norm_eps, r, dr, self.rope_dims, self.freqs, e.pos, e.slot,
                              e.block_table, self.cache, interleaved=self.interleaved)
        e.mm_heads(self.w_uk_t, q, q_lat, M, hd, r)
        gz = None
        if self.head_gate:          # one gate per head: a scalar commutes with the value up-projection, so the attention kernel applies it
            gz = e.buf("gz", H)
            e.mm(self.w_g, h, gz, M, src="h")
        L.latent_attention(q_lat, q, hd, dn, o_lat, M, H, r, dr, self.scale, e.pos, e.slot, e.block_table, self.cache,
                           tiles=e.latent_tiles(self), window=self.window, sink=self.sink, gate=gz)
        e.mm_heads(self.w_uv, o_lat, o, M, r, dv)
        if self.head_gate:
            e.mm(self.w_o, o, y, M)
            return
        e.mm(self.w_g, h, og, M, epi=L.DENSE_SIGMOID_MUL, aux=o, src="h")
        e.mm(self.w_o, og, y, M)


class Mamba2Mixer:
    """Tensors <prefix>in, conv, conv.b, dt_bias, A_log, D, norm, o.  Sizes: heads, vdim (inner = heads * vdim), state,
    groups (heads per B / C group = heads / groups), conv (taps), norm_groups."""

    def __init__(self, eng: "LayerListEngine", index: int, m: dict, prefix: str):
        self.eng, self.index = eng, index
        self.H, self.P, self.N, self.G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
        self.taps, self.norm_groups = int(m["conv"]), int(m["norm_groups"])
        self.inner = self.H * self.P
        self.channels = self.inner + 2 * self.G * self.N
        if self.H % self.G or self.inner % self.norm_groups:
            raise ValueError(f"layer {index}: heads / groups / norm_groups do not divide")
        W, V, D = eng.weight, eng.vector, eng.dense_weight
        self.w_in, self.w_o = D(W(prefix + "in")), D(W(prefix + "o"))
        self.w_conv, self.b_conv = W(prefix + "conv"), W(prefix + "conv.b")
        self.dt_bias, self.A_log, self.D, self.norm = (V(prefix + n) for n in ("dt_bias", "A_log", "D", "norm"))
        if tuple(self.w_in.t.shape) != (2 * self.inner + 2 * self.G * self.N + self.H, eng.cfg.width):
            raise ValueError(f"layer {index}: input projection has shape {tuple(self.w_in.t.shape)}")
        # the slot's recurrent state: S [heads][state][vdim] and the last taps-1 convolution inputs, both f32
        self.ssm_state = torch.zeros(eng.n_slots, self.H, self.N, self.P, dtype=torch.float32, device=eng.device)
        self.conv_state = torch.zeros(eng.n_slots, max(1, self.taps - 1), self.channels, dtype=torch.float32, device=eng.device)

    def scratch(self) -> Dict[str, int]:
        return {"zx": 2 * self.inner + 2 * self.G * self.N + self.H, "xbc": self.channels, "ys": self.inner, "yn": self.inner}

    def bind(self, mixers: list):
        pass

    def weight_bytes(self) -> int:
        return self.w_in.nbytes() + self.w_o.nbytes() + self.w_conv.numel() * self.w_conv.element_size()

    def forward(self, h: torch.Tensor, y: torch.Tensor, M: int):
        e, L = self.eng, self.eng.L
        zx, ys, yn = e.buf("zx"), e.buf("ys"), e.buf("yn")
        xbc = e.buf("xbc", self.channels)
        e.mm(self.w_in, h, zx, M, src="h")
        L.mamba_conv(e.mamba_batch, M, e.n_seq, zx, self.inner, self.w_conv, self.b_conv, self.conv_state, xbc)
        dt = zx[:, 2 * self.inner + 2 * self.G * self.N:]
        L.mamba_scan(e.mamba_batch, e.n_seq, xbc, dt, self.dt_bias, self.A_log, self.D, ys, self.ssm_state, self.H, self.P,
                     self.N, self.G, chunks=e.mamba_chunks(self))
        L.rms_norm(ys, yn, M, self.inner, e.cfg.norm_eps, w=self.norm, groups=self.norm_groups, gate=zx)
        e.mm(self.w_o, yn, y, M)


class DenseFeedForward:
    """Tensors <prefix>up, down:  W_down act(W_up h).  act = relu(.)^2, or (design trait dense_act "polynorm", tensor
    <prefix>act = [c1, c2, c3, c0]) PolyNorm: c0 + sum_p cp z^p / rms(z^p), p = 1..3, with the powers taken element-wise and
    the root mean square (eps inside) over a row; or ("xielu", tensor <prefix>act = [p, q]) xIELU: softplus(p) z^2 + z / 2 for
    z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 for z <= 0, in the up-projection's epilogue."""

    def __init__(self, eng: "LayerListEngine", index: int, m: dict, prefix: str):
        self.eng = eng
        self.ff = int(m["ff"])
        self.w_up, self.w_down = eng.dense_weight(eng.weight(prefix + "up")), eng.dense_weight(eng.weight(prefix + "down"))
        act = eng.cfg.traits.get("dense_act")
        self.poly = eng.vector(prefix + "act") if act == "polynorm" else None
        if self.poly is not None and tuple(self.poly.shape) != (4,):
            raise ValueError(f"layer {index}: {prefix}act has shape {tuple(self.poly.shape)}")
        self.xielu = None
        if act == "xielu":          # tensor act = [p, q]: the two constants softplus(p) and 1/2 + softplus(q), formed once in f32
            pq = eng.vector(prefix + "act")
            if tuple(pq.shape) != (2,):
                raise ValueError(f"layer {index}: {prefix}act has shape {tuple(pq.shape)}")
            sp = torch.nn.functional.softplus(pq.float().cpu())
            self.xielu = (float(sp[0]), float(torch.tensor(0.5, dtype=torch.float32) + sp[1]))

    def scratch(self) -> Dict[str, int]:
        return {"up": self.ff}

    def weight_bytes(self) -> int:
        return self.w_up.nbytes() + self.w_down.nbytes()

    def forward(self, h: torch.Tensor, y: torch.Tensor, M: int):
        e, L = self.eng, self.eng.L
        up = e.buf("up", self.ff)
        if self.poly is not None:
            e.mm(self.w_up, h, up, M, src="h")
            L.poly_norm(up, up, M, self.ff, self.poly, e.cfg.norm_eps)
        elif self.xielu is not None:
            e.mm(self.w_up, h, up, M, epi=L.DENSE_XIELU, param=self.xielu[0], param2=self.xielu[1], src="h")
        else:
            e.mm(self.w_up, h, up, M, epi=L.DENSE_RELU2, src="h")
        e.mm(self.w_down, up, y, M)


class WindowAttentionMixer:
    """Grouped-query attention over a paged cache.  Sizes: heads, kv_heads, dim (per-head query / key size), vdim, scale,
    softcap (0 / absent: none), mask.size, rot {base, dims, scaling} (absent: positions do not enter the scores).
    The design's `attention` traits choose the rest:
      values "keys" (default): tensors <prefix>q, k, o; the values are the keys as projected (vdim = dim), the cache line
             holds the rotated key followed by the unrotated head of k;
      values "own": a projection <prefix>v of vdim numbers per key/value head, the line holds key + value (no rotary);
      mask "window" (default): a position sees itself and the mask.size - 1 before it (absent: everything before it);
      mask "chunk": position i sees j <= i with floor(j / size) = floor(i / size): chunk borders are multiples of size in sequence positions;
      qk_norm: every query and key head is divided by its root mean square (eps of the model) before the scores;
      sink: <prefix>sink [heads], exp(sink_h) joins the softmax denominator without a key or a value;
      gate: <prefix>g, the concatenated heads are multiplied by sigmoid(W_g h) before the output projection;
      rot "half" | "interleaved" with values "own": rotary on the first rot.dims dimensions of every query and key head in
             that pair layout, BEFORE the unit norm;
      talk: <prefix>talk [heads][heads] mixes the heads' scaled scores before mask and softmax, score'_h = sum_g talk[h][g]
             score_g.  The mix is linear in the queries, so it is folded into them: with c(g) the key/value head of query
             head g,  score'_h = sum_c ( sum_{g: c(g) = c} talk[h][g] q_g ) . k_c  -- head h gets ONE query of kv_heads * dim
             numbers that meets the keys of all key/value heads side by side; the values stay those of its own group.
    A mixer entry with `kv_from: j` has no k / v tensors and no cache: it reads layer j's keys (as cached: rotated and
    normalised) and values with queries, mask and the rest of its own."""

    def __init__(self, eng: "LayerListEngine", index: int, m: dict, prefix: str, share: Optional["WindowAttentionMixer"] = None):
        self.eng, self.index = eng, index
        tr = eng.cfg.traits.get("attention") or {}
        self.own_v, self.qk_norm = tr.get("values", "keys") == "own", bool(tr.get("qk_norm"))
        self.H, self.G, self.dim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
        self.vdim = int(m.get("vdim", self.dim))
        if not self.own_v and self.vdim != self.dim:
            raise ValueError(f"layer {index}: the values are the keys, so vdim must equal dim")
        if self.H % self.G:
            raise ValueError(f"layer {index}: {self.H} heads do not divide into {self.G} key/value heads")
        self.scale, self.softcap = float(m["scale"]), float(m.get("softcap") or 0.0)
        size = int((m.get("mask") or {}).get("size") or 0)
        self.window, self.chunk = (0, size) if tr.get("mask", "window") == "chunk" else (size, 0)
        rot = m.get("rot") or {"base": 10000.0, "dims": 0}
        self.rope_dims = int(rot["dims"])
        self.own_rot = tr.get("rot")                      # own values: the pair layout of the rotary (None: no rotary with own values)
        self.kv_from = m.get("kv_from")
        if self.rope_dims > self.dim or self.rope_dims % 2 or (self.own_v and self.rope_dims and self.own_rot not in ("half", "interleaved")):
            raise ValueError(f"layer {index}: rotary dims {self.rope_dims} do not fit dim {self.dim}")
        if self.kv_from is not None and (not self.own_v or share is not None):
            raise ValueError(f"layer {index}: kv_from is known for attention with values of its own and weights of its own")
        freqs, self.rope_mag = interpolated_rotary(float(rot["base"]), self.rope_dims, rot.get("scaling"))
        self.freqs = freqs.to(eng.device) if self.rope_dims else torch.zeros(1, dtype=torch.float64, device=eng.device)
        H, G, d, dv = self.H, self.G, self.dim, self.vdim
        if share is None:
            W, D = eng.weight, eng.dense_weight
            wq = W(prefix + "q")
            wk = W(prefix + "k") if self.kv_from is None else None
            if tuple(wq.shape) != (H * d, eng.cfg.width) or (wk is not None and tuple(wk.shape) != (G * d, eng.cfg.width)):
                raise ValueError(f"layer {index}: q / k have shapes {tuple(wq.shape)} / {tuple(wk.shape) if wk is not None else None}")
            parts = [wq] + ([wk] if wk is not None else [])
            if self.own_v and self.kv_from is None:
                wv = W(prefix + "v")
                if tuple(wv.shape) != (G * dv, eng.cfg.width):
                    raise ValueError(f"layer {index}: v has shape {tuple(wv.shape)}")
                parts.append(wv)
            self.w_qk = D(torch.cat(parts, 0).contiguous())            # one product for queries, keys (and values)
            self.w_o = D(W(prefix + "o"))
            self.w_g = D(W(prefix + "g")) if tr.get("gate") else None
            self.sink = eng.vector(prefix + "sink") if tr.get("sink") else None
            if self.sink is not None and tuple(self.sink.shape) != (H,):
                raise ValueError(f"layer {index}: sink has shape {tuple(self.sink.shape)}")
            self.talk = eng.vector(prefix + "talk") if tr.get("talk") else None
            if self.talk is not None and tuple(self.talk.shape) != (H, H):
                raise ValueError(f"layer {index}: talk has shape {tuple(self.talk.shape)}")
        else:
            self.w_qk, self.w_o, self.w_g, self.sink, self.talk = share.w_qk, share.w_o, share.w_g, share.sink, share.talk
        self.owns_weights = share is None
        self.line = d + (dv if self.own_v else self.rope_dims)
        # a kv_from layer is bound to its owner's cache once all layers exist
        self.cache = torch.zeros(eng.n_pages, G, PAGE, self.line, dtype=eng.wdtype, device=eng.device) if self.kv_from is None else None
        # bf16 caches of sizes the tensor-core kernel takes: tiles of tc_rq consecutive rows of a sequence (0: per-row kernel)
        L = eng.L
        self.tc_rq, self.tc_rq_small, self.tc_talk = 0, 0, False
        self.partial_floats = 0                 # scratch of the page shares, if it is not the windowed kernel's
        attn_tc = eng.round_x and os.environ.get("DLLAMA_LAYERS_ATTN_TC", "1") != "0"
        if attn_tc and dv == d and self.talk is None and L.window_tc_supported(H, G, d, 0 if self.own_v else self.rope_dims, eng.wdtype):
            self.tc_rq = L.window_tc_rows(H, G)
        elif attn_tc and self.own_v and self.softcap == 0.0 and L.talk_tc_supported(H, G, d, dv, G if self.talk is not None else 0, eng.wdtype):
            # values wider or narrower than the keys, head-mixed scores: the tile kernel of talk_attention.cu
            # tiles of 128 stacked (row, head) pairs for long portions, of 16 for decoding, 64 where those do not fit
            kh = G if self.talk is not None else 0
            self.tc_rq, self.tc_rq_small, self.tc_talk = L.talk_tc_rows(H, G, d, dv, kh, 1 << 30), L.talk_tc_rows(H, G, d, dv, kh, 1), True
            self.partial_floats = L.talk_tc_partial_floats(WINDOW_CTAS_PER_SM * eng.n_sms, 1, 1, dv, self.tc_rq, H)

    def scratch(self) -> Dict[str, int]:
        n = {"qk": (self.H + self.G) * self.dim + (self.G * self.vdim if self.own_v else 0), "o": self.H * self.vdim}
        if self.w_g is not None:
            n["og"] = self.H * self.vdim
        if self.talk is not None:
            n["qmix"] = self.H * self.G * self.dim
        return n

    def bind(self, mixers: list):
        if self.kv_from is not None:
            src = mixers[int(self.kv_from)]
            if not isinstance(src, WindowAttentionMixer) or src.kv_from is not None:
                raise ValueError(f"layer {self.index}: kv_from {self.kv_from} is not an attention layer with a cache of its own")
            if (src.G, src.dim, src.vdim, src.rope_dims, src.own_v) != (self.G, self.dim, self.vdim, self.rope_dims, self.own_v):
                raise ValueError(f"layer {self.index}: key / value shapes differ from layer {self.kv_from}")
            self.cache = src.cache

    def weight_bytes(self) -> int:
        if not self.owns_weights:
            return 0
        return self.w_qk.nbytes() + self.w_o.nbytes() + (self.w_g.nbytes() if self.w_g is not None else 0)

    def forward(self, h: torch.Tensor, y: torch.Tensor, M: int):
        e, L = self.eng, self.eng.L
        H, G, d, dv, rd = self.H, self.G, self.dim, self.vdim, self.rope_dims
        nqk = (H + G) * d
        own_kv = self.kv_from is None
        qk, o = e.buf("qk", self.w_qk.N), e.buf("o", H * dv)
        e.mm(self.w_qk, h, qk, M, src="h")
        # one launch: the keys (and values) go into the cache and the queries are rotated / normalised in place (and mixed)
        q_in = qk
        if self.own_v:
            if self.talk is not None:
                q_in = e.buf("qmix", H * G * d)
            L.window_kv_write(qk[:, H * d:] if own_kv else None, M, G, d, rd, self.freqs, self.rope_mag, e.pos, e.slot, e.block_table,
                              self.cache, q=qk, q_heads=H, v=qk[:, nqk:] if own_kv else None, vdim=dv, qk_norm=self.qk_norm,
                              eps=e.cfg.norm_eps, rope_half=self.own_rot == "half", talk=self.talk, q_mixed=q_in if self.talk is not None else None)
            rd = 0                            # the attention kernels meet keys that are complete: nothing of a line is shared with its value
        else:
            L.window_kv_write(qk[:, H * d:], M, G, d, rd, self.freqs, self.rope_mag, e.pos, e.slot, e.block_table, self.cache,
                              q=qk, q_heads=H)
        opts = dict(vdim=dv if self.own_v else 0, chunk=self.chunk, sink=self.sink)
        if self.talk is not None:
            opts["key_heads"] = G
        if self.tc_rq:
            rq = self.tc_rq_small if self.tc_rq_small and e.longest <= self.tc_rq_small else self.tc_rq
            tile_rows, n_tiles = e.window_tiles(rq)
            # few tiles (decoding): several CTAs share a tile's pages.  The share count depends on the tiling only (not on
            # the positions), so a captured graph stays valid as the sequences grow
            span = self.window or self.chunk
            pages = (span + PAGE - 1) // PAGE + 1 if span else e.max_pages
            n_splits = 1
            # the tall tiles of long portions fill the SMs from one CTA each (page shares only add their merge: measured)
            if n_tiles * G <= (e.n_sms - 1 if self.tc_talk and rq > self.tc_rq_small else 2 * e.n_sms):
                n_splits = max(1, min(pages, WINDOW_MAX_SPLITS, (WINDOW_CTAS_PER_SM * e.n_sms) // (n_tiles * G)))
            partial = e.window_partial(d, self.partial_floats) if n_splits > 1 else None
            if self.tc_talk:
                L.talk_attention_tc(q_in, o, H, G, d, dv, self.scale, self.window, e.pos, e.slot, e.block_table, self.cache, tile_rows,
                                    n_tiles, rq, n_splits, partial, chunk=self.chunk, sink=self.sink, key_heads=opts.get("key_heads", 0))
            else:
                L.window_attention_tc(qk, o, H, G, d, rd, self.scale, self.softcap, self.window, e.pos, e.slot, e.block_table,
                                      self.cache, tile_rows, n_tiles, rq, n_splits, partial, **opts)
        else:
            L.window_attention(q_in, o, M, H, G, d, rd, self.scale, self.softcap, self.window, e.pos, e.slot, e.block_table,
                               self.cache, **opts)
        if self.w_g is not None:
            og = e.buf("og", H * dv)
            e.mm(self.w_g, h, og, M, epi=L.DENSE_SIGMOID_MUL, aux=o, src="h")
            o = og
        e.mm(self.w_o, o, y, M)


class LightningMixer:
    """Linear attention with a fixed decay per head.  Tensors <prefix>q, k, v, g, o, norm.  Sizes: heads, dim, vdim,
    decay [heads].  q, k, v = SiLU of their projections of h; per head S <- lambda S + k (x) v with lambda = decay_h (f32, one state
    [dim][vdim] per slot and head), o = S^T q; all heads' outputs side by side get ONE RMS norm (weight `norm` [heads * vdim]), are multiplied
    by sigmoid(W_g h) and projected by W_o."""

    def __init__(self, eng: "LayerListEngine", index: int, m: dict, prefix: str, share: Optional["LightningMixer"] = None):
        self.eng, self.index = eng, index
        self.H, self.dim, self.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        decay = [float(x) for x in m["decay"]] if isinstance(m["decay"], (list, tuple)) else [float(m["decay"])] * self.H
        if len(decay) != self.H or not all(0.0 <= x <= 1.0 for x in decay):
            raise ValueError(f"layer {index}: decay must give one number in [0, 1] per head")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=eng.device)
        H, d, dv = self.H, self.dim, self.vdim
        if share is None:
            W, D = eng.weight, eng.dense_weight
            wq, wk, wv = W(prefix + "q"), W(prefix + "k"), W(prefix + "v")
            if tuple(wq.shape) != (H * d, eng.cfg.width) or tuple(wk.shape) != (H * d, eng.cfg.width) or tuple(wv.shape) != (H * dv, eng.cfg.width):
                raise ValueError(f"layer {index}: q / k / v have shapes {tuple(wq.shape)} / {tuple(wk.shape)} / {tuple(wv.shape)}")
            self.w_qkv = D(torch.cat([wq, wk, wv], 0).contiguous())    # one product, SiLU in its epilogue
            self.w_g, self.w_o, self.norm = D(W(prefix + "g")), D(W(prefix + "o")), eng.vector(prefix + "norm")
            if tuple(self.norm.shape) != (H * dv,):
                raise ValueError(f"layer {index}: norm has shape {tuple(self.norm.shape)}")
        else:
            self.w_qkv, self.w_g, self.w_o, self.norm = share.w_qkv, share.w_g, share.w_o, share.norm
        self.owns_weights = share is None
        self.state = torch.zeros(eng.n_slots, H, d, dv, dtype=torch.float32, device=eng.device)
        self.chunked = eng.L.lightning_chunked_supported(d, dv)

    def scratch(self) -> Dict[str, int]:
        return {"lqkv": self.H * (2 * self.dim + self.vdim), "ys": self.H * self.vdim, "yn": self.H * self.vdim, "og": self.H * self.vdim}

    def bind(self, mixers: list):
        pass

    def weight_bytes(self) -> int:
        return self.w_qkv.nbytes() + self.w_g.nbytes() + self.w_o.nbytes() if self.owns_weights else 0

    def forward(self, h: torch.Tensor, y: torch.Tensor, M: int):
        e, L = self.eng, self.eng.L
        H, d, dv = self.H, self.dim, self.vdim
        qkv, ys, yn, og = e.buf("lqkv", H * (2 * d + dv)), e.buf("ys", H * dv), e.buf("yn", H * dv), e.buf("og", H * dv)
        e.mm(self.w_qkv, h, qkv, M, epi=L.DENSE_SILU, src="h")
        chunks = e.lightning_chunks if self.chunked else 0
        L.lightning_scan(e.mamba_batch, e.n_seq, qkv, qkv[:, H * d:], qkv[:, 2 * H * d:], self.decay, ys, self.state, H, d, dv,
                         max_chunks=chunks, scratch=e.lightning_scratch(self) if chunks else None)
        L.rms_norm(ys, yn, M, H * dv, e.cfg.norm_eps, w=self.norm)
        e.mm(self.w_g, h, og, M, epi=L.DENSE_SIGMOID_MUL, aux=yn, src="h")
        e.mm(self.w_o, og, y, M)


class RoutedExperts:
    """Tensors <prefix>router, e<n>.up, e<n>.down (gated experts: also e<n>.gate).  Sizes: expert.ff, router {experts,
    top, groups {count, keep}, scale}, expert.limit.  Router logits are f32.  The design's `moe` traits:
      score "sigmoid" (default): scores sigmoid(z); experts form `count` groups of neighbours scored by the sum of their
            two largest scores, only the `keep` best groups are eligible;  "softmax": scores softmax(z) over all experts;
      renorm: the chosen scores are divided by their sum (+ 1e-20); router.scale then multiplies the weights;
      gated:  an expert is W_down (a sigma(1.702 a) (1 + b)), a = min(gate . h, limit), b = clamp(up . h, +-limit);
              "silu": W_down (silu(gate . h) (up . h));  otherwise W_down relu(W_up h)^2;
      bias:   <prefix>router.b [experts] is added to the router logits;
      shared: an mlp entry `shared: {ff}` brings one more gated expert <prefix>shared.gate / up / down that every token runs;
              its output is multiplied by sigmoid(<prefix>shared.sg . h), one number per token, and added.
    The `top` best eligible experts run and their outputs are summed with the weights.  Softmax scores divided by the sum
    of the chosen ones are the softmax over the chosen logits alone."""

    def __init__(self, eng: "LayerListEngine", index: int, m: dict, prefix: str):
        self.eng = eng
        tr = eng.cfg.traits.get("moe") or {}
        self.softmax, self.renorm, self.gated = tr.get("score", "sigmoid") == "softmax", bool(tr.get("renorm")), bool(tr.get("gated"))
        self.gate_silu = tr.get("gated") == "silu"
        r = m["router"]
        self.E, self.top, self.ff = int(r["experts"]), int(r["top"]), int(m["expert"]["ff"])
        self.route_scale = float(r.get("scale") or 0.0)
        self.limit = float(m["expert"].get("limit") or 0.0)
        g = r.get("groups") or {"count": 1, "keep": 1}
        self.groups, self.keep = int(g["count"]), int(g["keep"])
        if self.E % self.groups or not 1 <= self.keep <= self.groups or not 1 <= self.top <= self.keep * (self.E // self.groups):
            raise ValueError(f"layer {index}: {self.E} experts, {self.groups} groups (keep {self.keep}), top {self.top}")
        wr = eng.weight(prefix + "router")
        if tuple(wr.shape) != (self.E, eng.cfg.width):
            raise ValueError(f"layer {index}: router has shape {tuple(wr.shape)}")
        self.router_b = eng.vector(prefix + "router.b") if tr.get("bias") else None
        if self.router_b is not None and tuple(self.router_b.shape) != (self.E,):
            raise ValueError(f"layer {index}: router.b has shape {tuple(self.router_b.shape)}")
        # a shared expert: its gate's row rides behind the router's rows (one product gives the logits and the gate);
        # gate and up rows interleaved in one matrix (gate_0, up_0, gate_1, ...): the tensor-core product forms
        # silu(gate) * up in its epilogue, the weight-streaming one reads the two strided halves
        sh = m.get("shared") if tr.get("shared") else None
        self.shared_ff = int(sh["ff"]) if sh else 0
        self.w_sgu = self.w_sdown = None
        if sh:
            wsg, sg_, su_, sd_ = (eng.weight(prefix + "shared." + n) for n in ("sg", "gate", "up", "down"))
            W_, F_ = eng.cfg.width, self.shared_ff
            if tuple(wsg.shape) != (1, W_) or tuple(sg_.shape) != (F_, W_) or tuple(su_.shape) != (F_, W_) or tuple(sd_.shape) != (W_, F_):
                raise ValueError(f"layer {index}: shared expert has shapes {tuple(wsg.shape)} / {tuple(sg_.shape)} / {tuple(su_.shape)} / {tuple(sd_.shape)}")
            wr = torch.cat([wr, wsg], 0).contiguous()
            self.w_sgu = eng.dense_weight(torch.stack([sg_, su_], dim=1).reshape(2 * F_, W_).contiguous())
            self.w_sdown = eng.dense_weight(sd_)
        self.router = eng.dense_weight(wr)
        self.w_up = torch.stack([eng.weight(f"{prefix}e{n}.up") for n in range(self.E)]).contiguous()        # [E][ff][W]
        self.w_down = torch.stack([eng.weight(f"{prefix}e{n}.down") for n in range(self.E)]).contiguous()    # [E][W][ff]
        self.w_gate = torch.stack([eng.weight(f"{prefix}e{n}.gate") for n in range(self.E)]).contiguous() if self.gated else None
        if tuple(self.w_up.shape) != (self.E, self.ff, eng.cfg.width) or tuple(self.w_down.shape) != (self.E, eng.cfg.width, self.ff) or \
                (self.gated and self.w_gate.shape != self.w_up.shape):
            raise ValueError(f"layer {index}: expert weights have shapes {tuple(self.w_up.shape)} / {tuple(self.w_down.shape)}")
        # bf16 mode: batches of TC_MIN_ROWS rows and more sort their (row, expert) pairs by expert and run all experts as
        # one grouped tensor-core GEMM per projection; fewer rows stream the chosen experts' weights pair by pair
        self.grouped = eng.L.MoeGrouped(self.w_up, self.w_down, self.top, eng.max_rows, w_gate=self.w_gate, limit=self.limit,
                                        gate_silu=self.gate_silu) if eng.tc else None

    def scratch(self) -> Dict[str, int]:
        n = {"router_z": self.router.N, "moe_act": self.top * self.ff, "moe_sel": self.top, "moe_wgt": self.top}
        if self.shared_ff:
            n["sh_g"], n["sh_a"] = self.shared_ff, self.shared_ff
        return n

    def weight_bytes(self) -> int:
        n = self.w_up.numel() + self.w_down.numel() + (self.w_gate.numel() if self.gated else 0)
        sh = self.w_sgu.nbytes() + self.w_sdown.nbytes() if self.shared_ff else 0
        return self.router.nbytes() + n * self.w_up.element_size() + sh

    def forward(self, h: torch.Tensor, y: torch.Tensor, M: int):
        e, L = self.eng, self.eng.L
        z, act = e.buf("router_z", self.router.N), e.buf("moe_act", self.top * self.ff)
        sel, wgt = e.buf("moe_sel", self.top).view(torch.int32), e.buf("moe_wgt", self.top)
        e.mm(self.router, h, z, M, src="h")
        L.moe_select(z, M, self.E, self.top, self.groups, self.keep, sel, wgt, renorm=self.renorm, softmax=self.softmax,
                     scale=self.route_scale, bias=self.router_b)
        if self.grouped is not None and M >= TC_MIN_ROWS:
            self.grouped.run(h, M, sel, wgt, y)
        else:
            L.moe_rows(self.w_up, self.w_down, h, M, self.top, sel, wgt, act, y, e.round_x, w_gate=self.w_gate, limit=self.limit,
                       gate_silu=self.gate_silu)
        if self.shared_ff:          # y += sigmoid(z[:, E]) * W_down (silu(W_gate h) * (W_up h))
            F = self.shared_ff
            sh_a = e.buf("sh_a", F)
            if self.w_sgu.wh is not None and M >= TC_MIN_ROWS:
                e.mm(self.w_sgu, h, sh_a, M, epi=L.DENSE_GLU_SILU, src="h")
            else:
                sh_g, gu = e.buf("sh_g", F), self.w_sgu.t
                L.dense(gu[0::2], h, sh_g, M, e.round_x, epi=L.DENSE_SILU)
                L.dense(gu[1::2], h, sh_a, M, e.round_x, epi=L.DENSE_MUL, aux=sh_g)
            e.mm(self.w_sdown, sh_a, y, M, epi=L.DENSE_ROWGATE_ADD, aux=z[:, self.E:])


MIXERS = {"latent_attention": LatentAttentionMixer, "mamba2": Mamba2Mixer, "attention": WindowAttentionMixer,
          "lightning": LightningMixer}
FEED_FORWARDS = {"dense": DenseFeedForward, "moe": RoutedExperts}


class _HyperWeights:
    """Read / write weights of one sublayer's hyper-connection: in [S], out [S], mix [S][S] (from, to), f32."""

    def __init__(self, eng: "LayerListEngine", prefix: Optional[str]):
        S = eng.cfg.streams
        if prefix is None:                      # the plain residual sum
            ones = torch.ones(S, dtype=torch.float32, device=eng.device)
            self.w_in, self.w_out, self.mix = ones, ones.clone(), torch.eye(S, dtype=torch.float32, device=eng.device).contiguous()
        else:
            self.w_in, self.w_out, self.mix = eng.vector(prefix + "in"), eng.vector(prefix + "out"), eng.vector(prefix + "mix")
            if tuple(self.w_in.shape) != (S,) or tuple(self.w_out.shape) != (S,) or tuple(self.mix.shape) != (S, S):
                raise ValueError(f"{prefix}*: shapes do not match {S} streams")


class _Layer:
    def __init__(self, eng: "LayerListEngine", i: int, spec: LayerSpec, owner: Optional["_Layer"] = None):
        p = f"l{i}."
        if spec.type not in MIXERS:
            raise ValueError(f"layer {i}: unknown mixer type {spec.type!r}")
        sandwich, post = eng.cfg.residual == "sandwich", eng.cfg.residual == "post"
        taps = eng.cfg.canon_taps
        # the last taps - 1 inputs of the convolution in front of the mixer: every layer's own, per sequence slot
        self.canon_state = torch.zeros(eng.n_slots, max(taps - 1, 1), eng.cfg.width, dtype=torch.float32, device=eng.device) if taps > 0 else None
        if owner is not None:
            # the owner's weights on a cache / state of this layer's own
            if spec.type not in ("attention", "lightning") or sandwich:
                raise ValueError(f"layer {i}: weights_of is only known for attention and lightning mixers of hyper-style models")
            self.mixer = MIXERS[spec.type](eng, i, spec.mixer, "", share=owner.mixer)
            self.ff = owner.ff
            for n in ("norm1", "norm1b", "norm2", "norm2b", "hc1", "hc2", "canon1"):
                setattr(self, n, getattr(owner, n, None))
            return
        self.mixer = MIXERS[spec.type](eng, i, spec.mixer, p + "mix.")
        # "post": the norm on a sublayer's output carries the residual multiplier, x <- x + (m g) * y / rms(y)
        norm_w = (lambda name: (eng.norm_weight(name) * eng.cfg.residual_mult).contiguous()) if post else eng.norm_weight
        self.norm1 = norm_w(p + "norm1")
        self.canon1 = None
        if taps > 0:
            self.canon1 = eng.weight(p + "canon1")
            if tuple(self.canon1.shape) != (eng.cfg.width, taps):
                raise ValueError(f"layer {i}: canon1 has shape {tuple(self.canon1.shape)}")
        self.norm1b = eng.vector(p + "norm1b") if sandwich else None
        self.hc1 = self.hc2 = None
        if not sandwich:
            self.hc1 = _HyperWeights(eng, p + "hc1." if eng.cfg.hyper_weights else None)
        self.ff = None
        if spec.mlp is not None:
            kind = spec.mlp.get("kind") or ("moe" if "router" in spec.mlp else "dense")
            if kind not in FEED_FORWARDS:
                raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")
            self.ff = FEED_FORWARDS[kind](eng, i, spec.mlp, p + "mlp.")
            self.norm2 = norm_w(p + "norm2")
            self.norm2b = eng.vector(p + "norm2b") if sandwich else None
            if not sandwich:
                self.hc2 = _HyperWeights(eng, p + "hc2." if eng.cfg.hyper_weights else None)


# --------------------------------------------------------------------------------------------------
# the engine
# --------------------------------------------------------------------------------------------------
class LayerListEngine:
    def __init__(self, model_path: str, rank: int = 0, world: int = 1, group=None, max_rows: int = 32, n_slots: int = 4,
                 max_seq_len: int = 2048, dtype: str = "bfloat16", n_pages: Optional[int] = None,
                 device: Optional[torch.device] = None, tensor_cores: Optional[bool] = None, use_graphs: bool = True,
                 **_unused):
        if world != 1:
            raise NotImplementedError("layer-list models run on one GPU (no tensor-parallel slicing of their mixers yet)")
        if dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype {dtype!r}: bfloat16 or float32")
        from ..ops import layers as L            # fails loudly if the CUDA library is missing
        L.layers_lib()
        self.L = L
        self.cfg = self.h = LayerListConfig.load(model_path)
        self.rank, self.world, self.group = 0, 1, None
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.dtype = dtype
        self.wdtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        self.round_x = dtype == "bfloat16"
        # bf16 mode: batches of TC_MIN_ROWS rows and more run their matrix products on the tcgen05 GEMM (operand images
        # made once per weight at load time, once per activation matrix at run time); fewer rows stream the weights
        if tensor_cores is None:
            tensor_cores = os.environ.get("DLLAMA_LAYERS_TC", "1") != "0"
        self.tc = bool(tensor_cores) and self.round_x and int(max_rows) >= TC_MIN_ROWS
        self._kmax = 0
        self.n_sms = L.sm_count()
        self.longest = 0                         # rows of the longest portion of the current batch
        self.max_rows, self.n_slots = int(max_rows), int(n_slots)
        self.seq_len = self.cfg.seq_len = int(max_seq_len)
        self.max_pages = (self.seq_len + PAGE - 1) // PAGE
        self.n_pages = int(n_pages) if n_pages else self.n_slots * self.max_pages
        self.pages = PageAllocator(self.n_pages, self.n_slots, self.max_pages)
        self._slot_len = np.zeros(self.n_slots, dtype=np.int64)       # tokens each slot has been fed (the state's position)
        dev, R = self.device, self.max_rows
        self._st = SafetensorsFile(os.path.join(model_path, "model.safetensors"))
        try:
            self.embed = self.weight("embed")
            if tuple(self.embed.shape) != (self.cfg.vocab, self.cfg.width):
                raise ValueError(f"embed has shape {tuple(self.embed.shape)}")
            # layers with weights of their own first: a looped layer may name a layer before or after itself
            built: Dict[int, _Layer] = {i: _Layer(self, i, spec) for i, spec in enumerate(self.cfg.layers) if spec.weights_of is None}
            for i, spec in enumerate(self.cfg.layers):
                if spec.weights_of is not None:
                    owner = built[spec.weights_of]
                    if (spec.type, spec.mlp is None) != (self.cfg.layers[spec.weights_of].type, owner.ff is None):
                        raise ValueError(f"layer {i}: its entry differs from layer {spec.weights_of}, whose weights it uses")
                    built[i] = _Layer(self, i, spec, owner)
            self.layers: List[_Layer] = [built[i] for i in range(len(self.cfg.layers))]
            self.final_norm, self.head = self.norm_weight("final.norm"), self.dense_weight(self.weight("head"))
        finally:
            self._st.close()
        mixers = [l.mixer for l in self.layers]
        for mx in mixers:
            mx.bind(mixers)
        # latent attention on the tensor cores (bf16 caches): rows of a sequence are tiled so that rows x heads <= 32
        att = [mx for mx in mixers if isinstance(mx, LatentAttentionMixer)]
        self.attn_rq = 0
        if att and self.round_x and os.environ.get("DLLAMA_LAYERS_ATTN_TC", "1") != "0":
            # decode-sized portions: tiles of 32 stacked rows (8 warps); longer ones: 64 (16 warps, half the page visits)
            hmax = max(mx.H for mx in att)
            rq = max(1, min(16, 32 // hmax))
            self._attn_rq_big = max(1, min(16, 64 // hmax))
            if any(L.latent_tc_supported(mx.H, mx.rank, mx.dr, self.wdtype, self._attn_rq_big) for mx in att):
                self.attn_rq = self._attn_rq_small = rq
        self._n_tiles = self._n_splits = 0
        self._attn_partial = None
        if self.attn_rq:
            rmax = max(mx.rank for mx in att)
            self._attn_partial = torch.zeros(L.latent_tc_partial_floats(3 * self.n_sms, 1, rmax), dtype=torch.float32, device=dev)
        # long prompt portions run the recurrence in chunks of L.MAMBA_CHUNK rows in parallel (two passes)
        mam = [mx for mx in mixers if isinstance(mx, Mamba2Mixer) and L.mamba_chunked_supported(mx.P, mx.N)]
        self._n_chunks, self._chunk_scratch = 0, None
        self._max_chunks = R // L.MAMBA_CHUNK + self.n_slots
        if mam and R >= CHUNKED_SCAN_MIN_ROWS and os.environ.get("DLLAMA_LAYERS_CHUNKED_SCAN", "1") != "0":
            self._chunk_scratch = (
                torch.zeros(self._max_chunks * max(mx.H * mx.N * mx.P for mx in mam), dtype=torch.float32, device=dev),
                torch.zeros(self._max_chunks * max(mx.H for mx in mam), dtype=torch.float32, device=dev),
                torch.zeros(R * max(mx.H for mx in mam), dtype=torch.float32, device=dev))
        # linear attention: portions of LIGHTNING_CHUNKED_MIN_ROWS rows and more run chunk-parallel (three launches)
        lt = [mx for mx in mixers if isinstance(mx, LightningMixer) and mx.chunked]
        self.lightning_chunks, self._lightning_scratch = 0, None
        if lt and R >= LIGHTNING_CHUNKED_MIN_ROWS and os.environ.get("DLLAMA_LAYERS_CHUNKED_SCAN", "1") != "0":
            self._lightning_scratch = torch.zeros(max(L.lightning_chunk_floats(R, self.n_slots, mx.H, mx.dim, mx.vdim) for mx in lt),
                                                  dtype=torch.float32, device=dev)
        if self.cfg.residual == "post" and self.cfg.streams != 1:
            raise ValueError("the post-norm residual style keeps one residual stream")
        if self.cfg.canon_taps and self.cfg.residual != "hyper":
            raise ValueError("a convolution in front of the mixers is only wired into the pre-norm / hyper residual style")
        # scratch: one f32 buffer per name, as wide as the widest user
        widths: Dict[str, int] = {}
        for l in self.layers:
            for part in (l.mixer, l.ff):
                if part is not None:
                    for name, w in part.scratch().items():
                        widths[name] = max(widths.get(name, 0), w)
        self._bufs = {n: torch.zeros(R * w, dtype=torch.float32, device=dev) for n, w in widths.items()}
        self._widths = widths
        self.ncap = (R + 7) // 8 * 8
        self._xh = {}
        if self.tc:       # activation slabs: one kept for a sublayer's input (several products read it), one for the rest
            n = L.xh_bytes(self._kmax, self.ncap)
            self._xh = {k: torch.zeros(n, dtype=torch.uint8, device=dev) for k in ("h", "tmp")}
        if self.cfg.streams > L.HC_MAX_STREAMS:
            raise ValueError(f"{self.cfg.streams} streams: the kernels keep at most {L.HC_MAX_STREAMS} copies of the residual stream")
        self.x = torch.zeros(R, self.cfg.streams * self.cfg.width, dtype=torch.float32, device=dev)      # row = [streams][width]
        self.hn = torch.zeros(R, self.cfg.width, dtype=torch.float32, device=dev)
        self.hc = torch.zeros(R, self.cfg.width, dtype=torch.float32, device=dev) if self.cfg.canon_taps else None
        self.y = torch.zeros(R, self.cfg.width, dtype=torch.float32, device=dev)
        self.logits = torch.zeros(R, self.cfg.vocab, dtype=torch.float32, device=dev)
        self.out_tokens = torch.zeros(R, dtype=torch.int32, device=dev)
        self.h_out_tokens = torch.zeros(R, dtype=torch.int32).pin_memory()
        # batch descriptor (one pinned -> device copy per step):
        #   tokens | pos | slot | row_seq | seq_rows | logit_rows   [R] each, then seq_start [S+1] | seq_slot [S] | seq_pos0 [S]
        S = self.n_slots
        self._tiles_off = 6 * R + 3 * S + 1                  # then tile_rows [n_tiles][rq] of the attention kernel
        self._chunks_off = self._tiles_off + R + 16 * S      # then chunk_seq | chunk_off [max_chunks] of the chunked scan
        self._desc_len = self._chunks_off + 2 * self._max_chunks
        # then, per tile height rq of the windowed-attention layers, tile_rows [tiles][rq] of their tensor-core kernel
        self._window_partial = None
        for mx in mixers:                              # allocated before any graph is captured
            if isinstance(mx, WindowAttentionMixer) and mx.tc_rq:
                self.window_partial(mx.dim, mx.partial_floats)
        self._wtile_off: Dict[int, int] = {}
        self._wtile_n: Dict[int, int] = {}
        for rq in sorted({r for mx in mixers if isinstance(mx, WindowAttentionMixer) for r in (mx.tc_rq, mx.tc_rq_small) if r}):
            self._wtile_off[rq] = self._desc_len
            self._desc_len += ((R + rq - 1) // rq + S) * rq
        self.tile_rows = None
        self.h_desc = torch.zeros(self._desc_len, dtype=torch.int32).pin_memory()
        self.desc = torch.zeros(self._desc_len, dtype=torch.int32, device=dev)
        d = self.desc
        self.tokens, self.pos, self.slot, self.row_seq, self.seq_rows, self.logit_rows = (d[i * R:(i + 1) * R] for i in range(6))
        o = 6 * R
        self.seq_start, self.seq_slot, self.seq_pos0 = d[o:o + S + 1], d[o + S + 1:o + 2 * S + 1], d[o + 2 * S + 1:o + 3 * S + 1]
        self.tile_rows = d[self._tiles_off:self._chunks_off]
        self.chunk_seq = d[self._chunks_off:self._chunks_off + self._max_chunks]
        self.chunk_off = d[self._chunks_off + self._max_chunks:]
        self.mamba_batch = L.mamba_batch(self.pos, self.row_seq, self.seq_start, self.seq_rows, self.seq_slot, self.seq_pos0)
        self.n_seq = 0
        self.block_table = torch.zeros(self.n_slots, self.max_pages, dtype=torch.int32, device=dev)
        self.h_block_table = torch.zeros(self.n_slots, self.max_pages, dtype=torch.int32).pin_memory()
        self._staging_ev: Optional[torch.cuda.Event] = None
        self._xh_h_ready = False
        # decode-sized batches replay a CUDA graph per batch shape (rows, sequences, wanted logits, attention tiling):
        # a step is ~25 small launches per layer, and the host cannot issue them as fast as the GPU retires them
        self.use_graphs = bool(use_graphs) and os.environ.get("DLLAMA_LAYERS_GRAPHS", "1") != "0"
        self._graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self._graph_launches: Dict[tuple, int] = {}
        self._graph_seen: Dict[tuple, int] = {}
        self._graph_stream = torch.cuda.Stream(device=dev)
        self.layer_probe = None              # a list: forward() appends a copy of the residual stream after every layer
        torch.cuda.synchronize()

    # ---- weights ---------------------------------------------------------------------------------
    def weight(self, name: str) -> torch.Tensor:
        """A matrix (or a convolution's taps and bias) in the engine's weight type."""
        if name not in self._st:
            raise KeyError(f"model.safetensors has no tensor {name!r}")
        return self._st.tensor(name).to(self.wdtype).to(self.device).contiguous()

    def vector(self, name: str) -> torch.Tensor:
        """A norm weight or a per-head constant: always f32 on the device."""
        if name not in self._st:
            raise KeyError(f"model.safetensors has no tensor {name!r}")
        return self._st.tensor(name).to(torch.float32).to(self.device).contiguous()

    def norm_weight(self, name: str) -> torch.Tensor:
        """The weight of a norm over the model's width: a vector, or one number for all coordinates (stored as a tensor
        without dimensions), which is widened here."""
        w = self.vector(name)
        if w.numel() == 1:
            return w.reshape(1).expand(self.cfg.width).contiguous()
        if tuple(w.shape) != (self.cfg.width,):
            raise ValueError(f"{name} has shape {tuple(w.shape)}")
        return w

    def dense_weight(self, t: torch.Tensor) -> DenseWeight:
        self._kmax = max(self._kmax, int(t.shape[-1]))
        return DenseWeight(t, self.tc)

    def mm(self, w: DenseWeight, x: torch.Tensor, y: torch.Tensor, M: int, epi: int = 0, aux=None, param: float = 0.0,
           src: str = "tmp", param2: float = 0.0):
        """y[:M] = epi(x[:M] @ w^T).  src="h": x is the current sublayer input; its tensor-core image is made by the
        first product that reads it (begin_sublayer() marks it stale) and shared by the others."""
        L = self.L
        if w.wh is None or M < TC_MIN_ROWS:
            L.dense(w.t, x, y, M, self.round_x, epi=epi, aux=aux, param=param, param2=param2)
            return
        xh = self._xh[src]
        if src != "h" or not self._xh_h_ready:
            L.xh_from_rows(x, M, w.K, self.ncap, xh)
            self._xh_h_ready = src == "h" or self._xh_h_ready
        L.dense_tc(w.wh, w.N, w.K, xh, self.ncap, y, M, epi=epi, aux=aux, param=param, param2=param2)

    def mm_heads(self, w: DenseWeight, x: torch.Tensor, y: torch.Tensor, M: int, x_head_stride: int, y_head_stride: int):
        """Per head h: y[:M, h*ys : h*ys+N] = x[:M, h*xs : h*xs+K] @ w[h]^T."""
        L = self.L
        if w.wh is None or M < TC_HEADS_MIN_ROWS:          # one batched launch (grid.z = heads) instead of two per head
            L.dense_heads(w.t, x, y, M, self.round_x, x_head_stride, y_head_stride)
            return
        for h in range(w.t.shape[0]):
            L.xh_from_rows(x[:, h * x_head_stride:], M, w.K, self.ncap, self._xh["tmp"])
            L.dense_tc(w.wh[h], w.N, w.K, self._xh["tmp"], self.ncap, y[:, h * y_head_stride:], M)

    def mamba_chunks(self, mx):
        """The chunking of this batch for the two-pass scan, or None where the token-by-token scan runs (short portions,
        decoding, sizes the chunked kernels do not take)."""
        if not self._n_chunks or not self.L.mamba_chunked_supported(mx.P, mx.N):
            return None
        return (self.chunk_seq, self.chunk_off, self._n_chunks) + self._chunk_scratch

    def lightning_scratch(self, mx):
        return self._lightning_scratch

    def latent_tiles(self, mx):
        """The row tiling of this batch for the tensor-core attention kernel, or None where the per-row kernel runs."""
        L = self.L
        if not self.attn_rq or not L.latent_tc_supported(mx.H, mx.rank, mx.dr, self.wdtype, self.attn_rq):
            return None
        return (self.tile_rows, self._n_tiles, self.attn_rq, self._n_splits, self._attn_partial)

    def window_partial(self, dim: int, floats: int = 0) -> torch.Tensor:
        """Scratch of the attention tile kernels' page shares: tiles x key/value heads x shares <= WINDOW_CTAS_PER_SM x SMs."""
        need = floats or self.L.window_tc_partial_floats(WINDOW_CTAS_PER_SM * self.n_sms, 1, 1, dim)
        if self._window_partial is None or self._window_partial.numel() < need:
            self._window_partial = torch.zeros(need, dtype=torch.float32, device=self.device)
        return self._window_partial

    def window_tiles(self, rq: int):
        """(tile_rows on the device, tiles) of this batch for windowed-attention layers with tiles of rq rows."""
        o = self._wtile_off[rq]
        return self.desc[o:], self._wtile_n[rq]

    def begin_sublayer(self):
        self._xh_h_ready = False

    def buf(self, name: str, width: Optional[int] = None) -> torch.Tensor:
        """Scratch `name` as [max_rows][width] (default: the width it was sized for)."""
        w = width or self._widths[name]
        return self._bufs[name][:self.max_rows * w].view(self.max_rows, w)

    def weight_bytes(self) -> int:
        n = sum(l.mixer.weight_bytes() for l in self.layers) + sum(f.weight_bytes() for f in {id(l.ff): l.ff for l in self.layers if l.ff}.values())
        return n + self.head.nbytes()

    # ---- slots / pages ---------------------------------------------------------------------------
    def usable_pages(self) -> int:
        return self.n_pages

    def alloc_slot(self) -> int:
        s = self.pages.alloc_slot()
        self._slot_len[s] = 0
        return s

    def free_slot(self, slot: int):
        self.pages.free_slot(slot)
        self._slot_len[slot] = 0

    def ensure_capacity(self, slot: int, n_tokens: int):
        self.pages.ensure(slot, n_tokens)

    # ---- one step ----------------------------------------------------------------------------------
    def set_batch(self, tokens: Sequence[int], positions: Sequence[int], slots: Sequence[int],
                  logit_rows: Sequence[int]) -> int:
        M, R, S = len(tokens), self.max_rows, self.n_slots
        if not 1 <= M <= R:
            raise ValueError(f"{M} rows in a batch of an engine built for {R}")
        by_slot: Dict[int, List[int]] = {}
        for m, s in enumerate(slots):
            by_slot.setdefault(int(s), []).append(m)
        if len(by_slot) > S:
            raise ValueError("more sequences in a batch than slots")
        if self._staging_ev is not None:
            self._staging_ev.synchronize()
        hd = self.h_desc.numpy()
        hd[0:M], hd[R:R + M], hd[2 * R:2 * R + M] = tokens, positions, slots
        o, at = 6 * R, 0
        for n, (s, rows) in enumerate(by_slot.items()):
            p0 = int(positions[rows[0]])
            for i, m in enumerate(rows):
                if int(positions[m]) != p0 + i:
                    raise ValueError(f"slot {s}: rows of a sequence must hold consecutive positions in order")
            # a recurrent state cannot be rewound: a sequence goes on where it stopped, or starts again at 0
            if p0 != 0 and p0 != int(self._slot_len[s]):
                raise ValueError(f"slot {s}: position {p0} does not continue the sequence (its state is at {int(self._slot_len[s])})")
            hd[3 * R + np.asarray(rows)] = n
            hd[4 * R + at:4 * R + at + len(rows)] = rows
            hd[o + n] = at
            hd[o + S + 1 + n] = s
            hd[o + 2 * S + 1 + n] = p0
            at += len(rows)
            self.pages.ensure(s, p0 + len(rows))
            self._slot_len[s] = p0 + len(rows)
        hd[o + len(by_slot)] = at
        if self.attn_rq:
            # attention tiles: up to rq rows of one sequence at consecutive positions; few tiles (decoding) share their
            # pages among several CTAs
            longest = max(len(r) for r in by_slot.values())
            self.attn_rq = self._attn_rq_big if longest > self._attn_rq_small else self._attn_rq_small
            rq, to, nt, pages = self.attn_rq, self._tiles_off, 0, 1
            for s, rows in by_slot.items():
                for i in range(0, len(rows), rq):
                    part = rows[i:i + rq]
                    hd[to + nt * rq:to + nt * rq + len(part)] = part
                    hd[to + nt * rq + len(part):to + (nt + 1) * rq] = -1
                    nt += 1
                pages = max(pages, (int(self._slot_len[s]) + PAGE - 1) // PAGE)
            self._n_tiles = nt
            self._n_splits = 1 if nt >= self.n_sms else max(1, min(32, (2 * self.n_sms) // nt, pages // 2))
        for rq, wo in self._wtile_off.items():       # tiles of up to rq rows of one sequence at consecutive positions
            nt = 0
            for rows in by_slot.values():
                for i in range(0, len(rows), rq):
                    part = rows[i:i + rq]
                    hd[wo + nt * rq:wo + nt * rq + len(part)] = part
                    hd[wo + nt * rq + len(part):wo + (nt + 1) * rq] = -1
                    nt += 1
            self._wtile_n[rq] = nt
        self.longest = longest = max(len(r) for r in by_slot.values())
        self.lightning_chunks = 0
        if self._lightning_scratch is not None and longest >= LIGHTNING_CHUNKED_MIN_ROWS:
            self.lightning_chunks = (longest + self.L.LIGHTNING_CHUNK - 1) // self.L.LIGHTNING_CHUNK
        self._n_chunks = 0
        if self._chunk_scratch is not None and longest >= CHUNKED_SCAN_MIN_ROWS:
            co, nc, ch = self._chunks_off, 0, self.L.MAMBA_CHUNK
            for n, rows in enumerate(by_slot.values()):
                for off in range(0, len(rows), ch):
                    hd[co + nc], hd[co + self._max_chunks + nc] = n, off
                    nc += 1
            self._n_chunks = nc
        nl = len(logit_rows)
        hd[5 * R:5 * R + nl] = logit_rows
        if self.pages.dirty:
            self.h_block_table.numpy()[:] = self.pages.table
            self.block_table.copy_(self.h_block_table, non_blocking=True)
            self.pages.dirty = False
        self.desc.copy_(self.h_desc, non_blocking=True)
        if self._staging_ev is None:
            self._staging_ev = torch.cuda.Event()
        self._staging_ev.record()
        self.n_seq = len(by_slot)
        return M

    def _launch_forward(self, M: int, n_logits: int):
        L, cfg, eps = self.L, self.cfg, self.cfg.norm_eps
        x, hn, y, W = self.x, self.hn, self.y, self.cfg.width
        L.embed_rows(self.embed, self.tokens, x, M, cfg.embed_scale, cfg.streams)
        if cfg.residual == "hyper":
            self._launch_hyper_layers(M)
            if n_logits:      # the copies summed, the model's norm, only the wanted rows
                L.hyper_step(x, n_logits, cfg.streams, W, h=hn, norm_w=self.final_norm, eps=eps, rows=self.logit_rows)
        elif cfg.residual == "post":
            # every sublayer reads the stream itself; the norm of its output, times the multiplier, is summed into the stream
            for l in self.layers:
                self.begin_sublayer()
                l.mixer.forward(x, y, M)
                L.rms_norm(y, x, M, W, eps, w=l.norm1, accumulate=True)
                if l.ff is not None:
                    self.begin_sublayer()
                    l.ff.forward(x, y, M)
                    L.rms_norm(y, x, M, W, eps, w=l.norm2, accumulate=True)
                if self.layer_probe is not None:
                    self.layer_probe.append(x[:M].clone())
            if n_logits:
                L.rms_norm(x, hn, n_logits, W, eps, w=self.final_norm, rows=self.logit_rows)
        else:
            for l in self.layers:
                L.rms_norm(x, hn, M, W, eps, w=l.norm1, plus_one=True)
                self.begin_sublayer()
                l.mixer.forward(hn, y, M)
                L.rms_norm(y, x, M, W, eps, w=l.norm1b, plus_one=True, accumulate=True)
                if l.ff is not None:
                    L.rms_norm(x, hn, M, W, eps, w=l.norm2, plus_one=True)
                    self.begin_sublayer()
                    l.ff.forward(hn, y, M)
                    L.rms_norm(y, x, M, W, eps, w=l.norm2b, plus_one=True, accumulate=True)
                if self.layer_probe is not None:
                    self.layer_probe.append(x[:M].clone())
            if n_logits:
                L.rms_norm(x, hn, n_logits, W, eps, w=self.final_norm, plus_one=True, rows=self.logit_rows)
        if n_logits:
            self.begin_sublayer()
            if cfg.logit_softcap > 0:
                self.mm(self.head, hn, self.logits, n_logits, epi=L.DENSE_SOFTCAP, param=cfg.logit_softcap)
            else:
                self.mm(self.head, hn, self.logits, n_logits)

    def _launch_hyper_layers(self, M: int):
        """Sublayer after sublayer on the copies of the residual stream.  The write of one sublayer's output and the read
        (mix + norm) of the next sublayer's input are one launch; only a probe of the stream after every layer splits
        them."""
        L, cfg = self.L, self.cfg
        x, hn, y, W, S, eps, mult = self.x, self.hn, self.y, cfg.width, cfg.streams, cfg.norm_eps, cfg.residual_mult
        pending = None                                  # hyper weights of the sublayer whose output waits in y
        for l in self.layers:
            for sub, hc, norm in ((l.mixer, l.hc1, l.norm1), (l.ff, l.hc2, getattr(l, "norm2", None))):
                if sub is None:
                    continue
                if pending is None:
                    L.hyper_step(x, M, S, W, h=hn, w_in=hc.w_in, norm_w=norm, eps=eps)
                else:
                    L.hyper_step(x, M, S, W, y=y, mix=pending.mix, w_out=pending.w_out, mult=mult,
                                 h=hn, w_in=hc.w_in, norm_w=norm, eps=eps)
                self.begin_sublayer()
                if sub is l.mixer and l.canon1 is not None:      # h <- h + conv(h) over the sequence's last inputs
                    L.causal_conv(self.mamba_batch, M, self.n_seq, hn, l.canon1, l.canon_state, self.hc, residual=True)
                    sub.forward(self.hc, y, M)
                else:
                    sub.forward(hn, y, M)
                pending = hc
            if self.layer_probe is not None:
                L.hyper_step(x, M, S, W, y=y, mix=pending.mix, w_out=pending.w_out, mult=mult)
                pending = None
                self.layer_probe.append(x[:M].view(M, S, W).sum(1))
        if pending is not None:
            L.hyper_step(x, M, S, W, y=y, mix=pending.mix, w_out=pending.w_out, mult=mult)

    def _run(self, M: int, n_logits: int, greedy: bool):
        """Eagerly, or -- for decode-sized batches -- from a CUDA graph.  A shape's first step runs eagerly (it loads
        modules and sets kernel attributes), its second is captured (capturing executes nothing: the recurrent state
        advances once per step) and replayed from then on."""
        from ..ops import lib as _lib
        key = (M, self.n_seq, n_logits, self._n_tiles, self._n_splits, greedy, tuple(self._wtile_n.values()))
        if not self.use_graphs or M > GRAPH_MAX_ROWS or self.layer_probe is not None:
            return self._launch_step(M, n_logits, greedy)
        g = self._graphs.get(key)
        if g is None:
            self._graph_seen[key] = self._graph_seen.get(key, 0) + 1
            if self._graph_seen[key] < 2:
                return self._launch_step(M, n_logits, greedy)
            torch.cuda.current_stream().synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = _lib.launch_count
            with graph_capture(g, self._graph_stream):
                self._launch_step(M, n_logits, greedy)
            self._graph_launches[key] = _lib.launch_count - n0
            _lib.launch_count = n0
            self._graphs[key] = g
        g.replay()
        _lib.count_launch(self._graph_launches[key])

    def _launch_step(self, M: int, n_logits: int, greedy: bool):
        self._launch_forward(M, n_logits)
        if greedy and n_logits:
            self.L.argmax(self.logits, n_logits, self.out_tokens)

    @torch.no_grad()
    def forward(self, tokens: Sequence[int], positions: Sequence[int], slots: Sequence[int], logits_from: int = 0,
                greedy: bool = False, logit_rows: Optional[Sequence[int]] = None) -> torch.Tensor:
        """One forward over a batch of rows: any mix of prompt portions and single decoded tokens; rows of one sequence
        hold consecutive positions in order.  Returns the device logits [n][vocab] of rows logits_from.. (or of
        `logit_rows`, any rows in any order), valid until the next forward."""
        rows = list(logit_rows) if logit_rows is not None else list(range(logits_from, len(tokens)))
        M = self.set_batch(tokens, positions, slots, rows)
        self._run(M, len(rows), greedy)
        return self.logits[:len(rows)]

    def prefill(self, slot: int, tokens: Sequence[int], start_pos: int = 0, chunk: Optional[int] = None):
        """Evaluate a prompt in portions of <= max_rows rows; returns the logits of the last token."""
        chunk = chunk or self.max_rows
        out = None
        for i in range(0, len(tokens), chunk):
            part = list(tokens[i:i + chunk])
            pos = list(range(start_pos + i, start_pos + i + len(part)))
            out = self.forward(part, pos, [slot] * len(part), logits_from=len(part) - 1)
        return out

    def decode_step_greedy(self, tokens, positions, slots, logits_from: int = 0) -> List[int]:
        n = len(tokens) - logits_from
        self.forward(tokens, positions, slots, logits_from, greedy=True)
        self.h_out_tokens.copy_(self.out_tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.h_out_tokens[:n].tolist()

    def decode_greedy_host(self, tokens, positions, slots) -> List[int]:
        return self.decode_step_greedy(tokens, positions, slots, 0)

    def sample_rows(self, logits, temperature, topp, coin, tokens_out):
        """Device sampler of the batching loop (temperature / top-p / coin per row), from this engine's library."""
        self.L.sample_rows(logits, temperature, topp, coin, tokens_out)

    def close(self):
        self._graphs.clear()
        torch.cuda.synchronize()


# --------------------------------------------------------------------------------------------------
# random models (tests, benchmarks, the smoke run): same files a trained model would come in
# --------------------------------------------------------------------------------------------------
def random_tensors(config: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16 weights for every tensor the configuration calls for (matrices ~ N(0, 1/in), norm weights small
    around zero, decays and step-size biases in the range where the recurrence neither dies nor saturates)."""
    g = torch.Generator().manual_seed(seed)
    W, V = int(config["width"]), int(config["vocab"])

    def mat(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain / math.sqrt(i)).to(torch.bfloat16)

    def small(n, s=0.1):
        return (torch.randn(n, generator=g) * s).to(torch.bfloat16)

    sandwich = RESIDUAL_STYLES.get(config["architecture"], "sandwich") == "sandwich"
    traits = DESIGNS.get(config["architecture"], {})
    att, moe, lat = traits.get("attention") or {}, traits.get("moe") or {}, traits.get("latent") or {}
    taps = int((config.get("canon") or {}).get("taps") or 0)
    S = int(config.get("streams") or 0)
    scalar_norms = config["architecture"] == "Venadra" or traits.get("norm_weights") == "scalar"          # one number per norm

    def norm_w():
        if scalar_norms:
            return (1 + torch.randn((), generator=g) * 0.1).to(torch.bfloat16)
        return small(W) if sandwich else 1 + small(W)

    t = {"embed": (torch.randn(V, W, generator=g)).to(torch.bfloat16), "head": mat(V, W), "final.norm": norm_w()}

    def hyper(prefix):
        # read weights around 1 / S, write weights around 1, a mixing matrix near the identity with some cross-talk
        t[prefix + "in"] = (1.0 / S + torch.randn(S, generator=g) * 0.1).to(torch.bfloat16)
        t[prefix + "out"] = (1.0 + torch.randn(S, generator=g) * 0.2).to(torch.bfloat16)
        t[prefix + "mix"] = (torch.eye(S) * 0.9 + torch.randn(S, S, generator=g) * 0.1).to(torch.bfloat16)

    for i, l in enumerate(config["layers"]):
        p, m = f"l{i}.", l["mixer"]
        if l.get("weights_of") is not None:
            continue
        t[p + "norm1"] = norm_w()
        if taps:
            t[p + "canon1"] = mat(W, taps, 0.5)
        if sandwich:
            t[p + "norm1b"] = small(W)
        elif S:
            hyper(p + "hc1.")
        if l["type"] == "latent_attention":
            H, dn, dr, dv, qr, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"] = mat(qr, W), 1 + small(qr)
            t[p + "mix.uq"] = mat(H * (dn + dr), qr, 2.0)
            if "kv_from" not in m:
                t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(r + dr, W), 1 + small(r)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * dn, r, 2.0), mat(H * dv, r)
            t[p + "mix.g"], t[p + "mix.o"] = mat(H if lat.get("gate") == "head" else H * dv, W), mat(W, H * dv)
            if lat.get("sink"):
                t[p + "mix.sink"] = (torch.randn(H, generator=g)).to(torch.bfloat16)
        elif l["type"] == "mamba2":
            H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * P, H * P + 2 * G * N
            t[p + "mix.in"] = mat(2 * inner + 2 * G * N + H, W)
            t[p + "mix.conv"], t[p + "mix.conv.b"] = mat(ch, taps, 1.5), small(ch)
            t[p + "mix.dt_bias"] = (torch.rand(H, generator=g) * 2 - 2).to(torch.bfloat16)
            t[p + "mix.A_log"] = torch.log(torch.rand(H, generator=g) * 1.5 + 0.25).to(torch.bfloat16)
            t[p + "mix.D"], t[p + "mix.norm"] = 1 + small(H), 1 + small(inner)
            t[p + "mix.o"] = mat(W, inner)
        elif l["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
            t[p + "mix.q"] = mat(H * d, W, 2.0)
            if m.get("kv_from") is None:
                t[p + "mix.k"] = mat(G * d, W, 2.0)
            t[p + "mix.o"] = mat(W, H * dv)
            if m.get("kv_from") is None and att.get("values") == "own":
                t[p + "mix.v"] = mat(G * dv, W)
            if att.get("talk"):     # near the identity, with cross-talk between all heads
                t[p + "mix.talk"] = (torch.eye(H) + torch.randn(H, H, generator=g) * 0.3).to(torch.bfloat16)
            if att.get("sink"):
                t[p + "mix.sink"] = (torch.randn(H, generator=g)).to(torch.bfloat16)
            if att.get("gate"):
                t[p + "mix.g"] = mat(H * dv, W)
        elif l["type"] == "lightning":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * d, W, 2.0), mat(H * d, W, 2.0), mat(H * dv, W, 2.0)
            t[p + "mix.g"], t[p + "mix.o"], t[p + "mix.norm"] = mat(H * dv, W), mat(W, H * dv), 1 + small(H * dv)
        else:
            raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
        if l.get("mlp"):
            t[p + "norm2"] = norm_w()
            if sandwich:
                t[p + "norm2b"] = small(W)
            elif S:
                hyper(p + "hc2.")
            if (l["mlp"].get("kind") or ("moe" if "router" in l["mlp"] else "dense")) == "moe":
                E, ff = l["mlp"]["router"]["experts"], l["mlp"]["expert"]["ff"]
                t[p + "mlp.router"] = mat(E, W, 2.0)
                if moe.get("bias"):
                    t[p + "mlp.router.b"] = (torch.randn(E, generator=g) * 0.5).to(torch.bfloat16)
                sh = l["mlp"].get("shared") if moe.get("shared") else None
                if sh:
                    t[p + "mlp.shared.gate"], t[p + "mlp.shared.up"] = mat(sh["ff"], W, 1.5), mat(sh["ff"], W, 1.5)
                    t[p + "mlp.shared.down"], t[p + "mlp.shared.sg"] = mat(W, sh["ff"]), mat(1, W, 2.0)
                for n in range(E):
                    t[p + f"mlp.e{n}.up"], t[p + f"mlp.e{n}.down"] = mat(ff, W, 1.5), mat(W, ff)
                    if moe.get("gated"):
                        t[p + f"mlp.e{n}.gate"] = mat(ff, W, 1.5)
            else:
                t[p + "mlp.up"], t[p + "mlp.down"] = mat(l["mlp"]["ff"], W), mat(W, l["mlp"]["ff"])
                if traits.get("dense_act") == "polynorm":
                    t[p + "mlp.act"] = torch.tensor([0.6, 0.3, 0.15, 0.05]).add(torch.randn(4, generator=g) * 0.05).to(torch.bfloat16)
                elif traits.get("dense_act") == "xielu":
                    t[p + "mlp.act"] = (torch.randn(2, generator=g) * 0.5).to(torch.bfloat16)
    return t


def write_random_model(model_dir: str, config: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """config.json + model.safetensors of a random model; returns the tensors written."""
    from ..formats.safetensors import write_safetensors
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    tensors = random_tensors(config, seed)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors)
    return tensors


def example_config(width: int = 192, vocab: int = 320, blocks: int = 2, heads: int = 4) -> dict:
    """A small Ribivik-shaped configuration: `blocks` x (latent-attention layer with a feed-forward, mamba2 layer, every
    second of them with a narrow feed-forward of its own); attention layers after the first read the first one's cache."""
    layers = []
    for b in range(blocks):
        mixer = {"heads": heads, "dim": 40, "rot_dim": 8, "vdim": 24, "q_rank": 48, "kv_rank": 56,
                 "scale": 1.0 / math.sqrt(48), "rot": {"base": 10000.0, "dims": 8}}
        if b >= 1:
            mixer["kv_from"] = 0
        layers.append({"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": 2 * width}})
        layers.append({"type": "mamba2", "mlp": {"kind": "dense", "ff": width // 2} if b % 2 else None,
                       "mixer": {"heads": heads, "vdim": 24, "state": 16, "groups": 2, "conv": 3, "norm_groups": 2}})
    return {"architecture": "Ribivik", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "logit_softcap": 25.0,
            "layers": layers}


def example_config_sunesun(width: int = 160, vocab: int = 320, layers: int = 3, heads: int = 6, kv_heads: int = 3,
                           window: int = 48, streams: int = 2) -> dict:
    """A small Sunesun-shaped configuration: windowed attention (values = keys) with routed experts on `streams`
    hyper-connected copies of the residual stream; the last layer runs the first layer's weights again."""
    def layer(i):
        l = {"type": "attention",
             "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 32, "vdim": 32, "scale": 1.0 / math.sqrt(32.0), "softcap": 30.0,
                       "mask": {"size": window},
                       "rot": {"base": 10000.0, "dims": 24, "scaling": {"factor": 8.0, "original": 512, "fast": 16.0, "slow": 2.0}}},
             "mlp": {"kind": "moe", "expert": {"ff": 64},
                     "router": {"experts": 12, "top": 3, "groups": {"count": 3, "keep": 2}}}}
        if i == layers - 1 and layers > 1:
            l["weights_of"] = 0
        return l
    return {"architecture": "Sunesun", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "residual_mult": 0.5, "streams": streams, "layers": [layer(i) for i in range(layers)]}


def example_config_venadra(width: int = 160, vocab: int = 320, heads: int = 3, chunk: int = 40) -> dict:
    """A small Venadra-shaped configuration: lightning layers (dense PolyNorm and gated-expert feed-forwards), one chunked
    sink-attention layer, a 3-tap convolution in front of every mixer; the last two layers run earlier layers' weights."""
    light = {"heads": heads, "dim": 16, "vdim": 24, "decay": [round(0.5 + 0.499 * i / max(heads - 1, 1), 4) for i in range(heads)]}
    attn = {"heads": 2 * heads, "kv_heads": heads, "dim": 32, "vdim": 32, "scale": 0.2, "mask": {"size": chunk}}
    dense = {"kind": "dense", "ff": 2 * width}
    moe = {"kind": "moe", "expert": {"ff": 48, "limit": 1.5}, "router": {"experts": 6, "top": 2, "scale": 1.25}}
    layers = [{"type": "lightning", "mixer": dict(light), "mlp": dict(dense)},
              {"type": "attention", "mixer": dict(attn), "mlp": dict(moe)},
              {"type": "lightning", "mixer": dict(light), "mlp": dict(moe)},
              {"type": "lightning", "mixer": dict(light), "mlp": dict(dense), "weights_of": 0},
              {"type": "attention", "mixer": dict(attn), "mlp": dict(moe), "weights_of": 1}]
    return {"architecture": "Venadra", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
            "canon": {"taps": 3}, "layers": layers}


def example_config_darusun(width: int = 160, vocab: int = 320, heads: int = 6, kv_heads: int = 3, window: int = 40) -> dict:
    """A small Darusun-shaped configuration: post-norm layers; grouped-query attention with rotate-half rotary, unit
    queries and keys, head-mixed scores and values wider than the keys (one layer reads the first layer's keys and
    values); a latent-attention layer with a sliding window, sinks and a gate per head; an xIELU feed-forward and routed
    experts with a router bias and a shared expert."""
    attn = {"heads": heads, "kv_heads": kv_heads, "dim": 32, "vdim": 48, "scale": 0.2, "rot": {"base": 10000.0, "dims": 16}}
    lat = {"heads": 4, "dim": 24, "rot_dim": 8, "vdim": 32, "q_rank": 40, "kv_rank": 48, "scale": 1.0 / math.sqrt(32.0),
           "rot": {"base": 10000.0, "dims": 8}, "mask": {"size": window}}
    moe = {"kind": "moe", "expert": {"ff": 48}, "router": {"experts": 6, "top": 2}, "shared": {"ff": 80}}
    layers = [{"type": "attention", "mixer": dict(attn), "mlp": {"kind": "dense", "ff": 2 * width}},
              {"type": "latent_attention", "mixer": dict(lat), "mlp": dict(moe)},
              {"type": "attention", "mixer": dict(attn, kv_from=0), "mlp": dict(moe)}]
    return {"architecture": "Darusun", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "residual_mult": 0.6, "layers": layers}
