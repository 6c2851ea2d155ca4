"""Slow, plain restatement of the Venadra mechanisms in float64 on the CPU, one function per mechanism, written from the
equations in this file's own notation.  It shares no code with the package: weights come as a dict of tensors,
sequences whole; it knows nothing of pages, slots, portions, batches or kernels.

Notation: T tokens at positions t = 0 .. T-1; unit(v) = v / sqrt(mean(v^2) + eps) along the last axis.
"""
import math

import torch

F64 = torch.float64


def unit(v, eps):
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def logistic(v):
    return 1.0 / (1.0 + torch.exp(-v))


def swish(v):
    return v * logistic(v)


def short_convolution(h, taps_w):
    """h [T, width], taps_w [width, taps]:  h_t + sum_j taps_w[:, j] h_(t - taps + 1 + j), nothing before t = 0."""
    T, taps = h.shape[0], taps_w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                out[t] += taps_w[:, j] * h[src]
    return out


def decayed_linear_attention(q, k, v, decay):
    """q, k [T, dim], v [T, vdim] of one head: the state starts at zero, S <- decay S + k_t v_t^T, o_t = S^T q_t."""
    S = torch.zeros(q.shape[1], v.shape[1], dtype=F64)
    out = torch.zeros(q.shape[0], v.shape[1], dtype=F64)
    for t in range(q.shape[0]):
        S = decay * S + k[t][:, None] * v[t][None, :]
        out[t] = q[t] @ S
    return out


def lightning_mixer(h, w, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = swish(h @ w["q"].T).reshape(T, H, d)
    k = swish(h @ w["k"].T).reshape(T, H, d)
    v = swish(h @ w["v"].T).reshape(T, H, dv)
    o = torch.cat([decayed_linear_attention(q[:, i], k[:, i], v[:, i], float(m["decay"][i])) for i in range(H)], dim=1)
    o = unit(o, eps) * w["norm"]
    return (o * logistic(h @ w["g"].T)) @ w["o"].T


def block_sink_softmax_rows(q, k, v, scale, block, sink, eps, first_position=0):
    """q [T, H, d], k [T, G, d], v [T, G, dv] at positions first_position .. : queries and keys made unit per head, key j
    visible to query i when j <= i and both lie in the same block of `block` positions (block 0: every j <= i); one extra
    term exp(sink_head) in the softmax denominator, which has no value."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    q, k = unit(q, eps), unit(k, eps)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(T):
        pi = first_position + i
        first = max((pi // block) * block - first_position, 0) if block else 0
        for a in range(H):
            g = a // (H // G)
            sc = (k[first:i + 1, g] @ q[i, a]) * scale
            top = max(float(sc.max()), float(sink[a]))
            e = torch.exp(sc - top)
            out[i, a] = (e / (e.sum() + math.exp(float(sink[a]) - top))) @ v[first:i + 1, g]
    return out


def chunk_sink_attention(h, w, m, eps):
    """Grouped-query attention without positions in the scores, with an element-wise logistic gate on the heads' outputs."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, G, d)
    v = (h @ w["v"].T).reshape(T, G, dv)
    out = block_sink_softmax_rows(q, k, v, m["scale"], (m.get("mask") or {}).get("size") or 0, w["sink"], eps)
    return (out.reshape(T, H * dv) * logistic(h @ w["g"].T)) @ w["o"].T


def poly_norm_feed_forward(h, w, eps):
    z = h @ w["up"].T
    a, b, c, e = (float(x) for x in w["act"])
    act = a * unit(z, eps) + b * unit(z ** 2, eps) + c * unit(z ** 3, eps) + e
    return act @ w["down"].T


def route(z, r):
    """z [experts] router logits of one token -> [(expert, weight)], best first."""
    s = torch.softmax(z, dim=0)
    chosen = sorted(range(r["experts"]), key=lambda e: (-float(s[e]), e))[:r["top"]]
    total = sum(float(s[e]) for e in chosen) + 1e-20
    return [(e, float(s[e]) / total * r.get("scale", 1.0)) for e in chosen]


def gated_expert(x, w, e, limit):
    g = torch.clamp(w[f"e{e}.gate"] @ x, max=limit)
    u = torch.clamp(w[f"e{e}.up"] @ x, min=-limit, max=limit)
    return w[f"e{e}.down"] @ (g * logistic(1.702 * g) * (u + 1.0))


def routed_experts(h, w, m):
    out = torch.zeros_like(h)
    z = h @ w["router"].T
    for t in range(h.shape[0]):
        for e, weight in route(z[t], m["router"]):
            out[t] += weight * gated_expert(h[t], w, e, m["expert"]["limit"])
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def model_logits(tensors, config, tokens, residual_out=None):
    """Logits [T, vocab] of one whole sequence; residual_out collects the residual stream after every layer."""
    eps = config["norm"]["eps"]
    W = {k: v.to(F64) for k, v in tensors.items()}
    x = W["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    for i, layer in enumerate(config["layers"]):
        j = layer.get("weights_of")
        p = f"l{i if j is None else j}."
        h = unit(x, eps) * W[p + "norm1"]
        if config.get("canon"):
            h = short_convolution(h, W[p + "canon1"])
        if layer["type"] == "lightning":
            x = x + lightning_mixer(h, sub(tensors, p + "mix."), layer["mixer"], eps)
        else:
            x = x + chunk_sink_attention(h, sub(tensors, p + "mix."), layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = unit(x, eps) * W[p + "norm2"]
            if mlp["kind"] == "dense":
                x = x + poly_norm_feed_forward(h, sub(tensors, p + "mlp."), eps)
            else:
                x = x + routed_experts(h, sub(tensors, p + "mlp."), mlp)
        if residual_out is not None:
            residual_out.append(x.clone())
    return (unit(x, eps) * W["final.norm"]) @ W["head"].T


def logit_error(got, want):
    """Per row: root mean square of the difference (mean taken off) over the root mean square of the wanted logits."""
    d = got.to(F64) - want.to(F64)
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / want.to(F64).pow(2).mean().sqrt()
