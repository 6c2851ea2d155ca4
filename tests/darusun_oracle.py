"""Darusun in float64, one plain function per mechanism, written from the equations; it shares no code with the package.

Notation: T tokens, W width, H query heads, G key/value heads (query head h reads key/value head h // (H // G)),
d key size, dv value size.  rms(x) = x / sqrt(mean(x^2) + eps) over the last axis.

  layer            x <- x + m * g1 * rms(mixer(x));  x <- x + m * g2 * rms(ff(x))      g1, g2: one number each, m: residual_mult
  attention        q, k, v = projections of x; rotary (pairs i, i + n/2) on the first n = rot.dims of every q and k head,
                   then q <- rms(q), k <- rms(k) per head;  s_h = scale * q_h . k_c(h);  s'_h = sum_g talk[h][g] s_g;
                   causal softmax over s';  o_h = sum_j p_h,j v_c(h),j;  y = W_o concat(o)
                   kv_from: j  -> k and v are those layer j made
  latent attention cq = w_dq * rms(W_dq x); q = W_uq cq, per head [d plain | r rotated]; W_dkv x = [kv_rank | r]:
                   c = w_dkv * rms(first part), kr = rotary(last part), shared by the heads; rotary pairs (2i, 2i + 1);
                   k_h = W_uk c, v_h = W_uv c;  s_h = scale * (q_plain . k_h + q_rot . kr); visible: 0 <= i - j < size;
                   softmax with exp(sink_h) added to the denominator;  o_h *= sigmoid(W_g x)_h;  y = W_o concat(o)
  dense ff         W_down xielu(W_up x);  xielu(z) = softplus(p) z^2 + z/2 (z > 0), (1/2 + softplus(q)) (e^z - 1 - z) + z/2 (z <= 0)
  experts          z = W_r x + b; the `top` largest z; weights = softmax over those z;  expert: W_down (silu(W_gate x) * W_up x);
                   + sigmoid(w_sg . x) * shared expert(x)
  output           logits = W_head (g * rms(x))
"""
import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def angles(positions, base, n):
    """[T, n / 2]: position * base^(-2 i / n)."""
    i = torch.arange(n // 2, dtype=F64)
    return positions.to(F64)[:, None] * torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / n)[None, :]


def rotate_half_pairs(x, positions, base, n):
    """x [T, heads, size]: dimension i < n / 2 is paired with i + n / 2; the rest passes."""
    a = angles(positions, base, n)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :n // 2], x[..., n // 2:n]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., n:]], -1)


def rotate_neighbour_pairs(x, positions, base, n):
    """x [T, heads, size]: dimension 2i is paired with 2i + 1, i < n / 2; the rest passes."""
    a = angles(positions, base, n)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def mixed_head_softmax_rows(q, k, v, scale, talk, first=0):
    """q [T, H, d] and k [S, G, d] as they meet (already rotated and normalised), v [S, G, dv]; query row t sits at
    position first + t and sees keys 0 .. first + t.  Scores of all heads are mixed by talk [H, H] before the softmax."""
    T, H, _ = q.shape
    S, G, dv = v.shape
    rep = H // G
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        n = first + t + 1
        raw = torch.stack([k[:n, h // rep] @ q[t, h] for h in range(H)]) * scale          # [H, n]
        mixed = talk @ raw
        p = torch.softmax(mixed, -1)
        for h in range(H):
            out[t, h] = p[h] @ v[:n, h // rep]
    return out


def attention_mixer(t, p, m, x, eps, kv=None, first=0):
    """Returns (y, (k, v)): k and v of all positions so far, for a layer that reads them."""
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(first, first + T)
    q = rms_unit(rotate_half_pairs((x @ t[p + "q"].T).reshape(T, H, d), pos, m["rot"]["base"], m["rot"]["dims"]), eps)
    if kv is None:
        k = rms_unit(rotate_half_pairs((x @ t[p + "k"].T).reshape(T, G, d), pos, m["rot"]["base"], m["rot"]["dims"]), eps)
        kv = (k, (x @ t[p + "v"].T).reshape(T, G, dv))
    o = mixed_head_softmax_rows(q, kv[0], kv[1], m["scale"], t[p + "talk"], first)
    return o.reshape(T, H * dv) @ t[p + "o"].T, kv


def window_sink_softmax_rows(scores, values, size, sink):
    """scores [H, T, T] (row i, key j), values [T, H, dv]; key j is visible to row i if 0 <= i - j < size (size 0: j <= i);
    exp(sink_h) joins the denominator."""
    H, T, _ = scores.shape
    out = torch.zeros(T, H, values.shape[-1], dtype=F64)
    for i in range(T):
        lo = max(0, i - size + 1) if size else 0
        for h in range(H):
            s = scores[h, i, lo:i + 1]
            mx = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - mx)
            out[i, h] = (e / (e.sum() + torch.exp(sink[h] - mx))) @ values[lo:i + 1, h]
    return out


def latent_mixer(t, p, m, x, eps):
    T = x.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_unit(x @ t[p + "dq"].T, eps) * t[p + "dq.norm"]
    q = (cq @ t[p + "uq"].T).reshape(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_neighbour_pairs(q[..., d:], pos, m["rot"]["base"], m["rot"]["dims"])
    down = x @ t[p + "dkv"].T
    c = rms_unit(down[:, :rank], eps) * t[p + "dkv.norm"]
    k_rot = rotate_neighbour_pairs(down[:, None, rank:], pos, m["rot"]["base"], m["rot"]["dims"])[:, 0]
    k = (c @ t[p + "uk"].T).reshape(T, H, d)
    v = (c @ t[p + "uv"].T).reshape(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    o = window_sink_softmax_rows(scores, v, int((m.get("mask") or {}).get("size") or 0), t[p + "sink"])
    o = o * torch.sigmoid(x @ t[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ t[p + "o"].T


def xielu(z, p, q):
    sp = lambda a: math.log1p(math.exp(-abs(a))) + max(a, 0.0)
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, sp(float(p)) * z * z + z / 2, (0.5 + sp(float(q))) * (torch.expm1(neg) - neg) + z / 2)


def dense_ff(t, p, x):
    return xielu(x @ t[p + "up"].T, t[p + "act"][0], t[p + "act"][1]) @ t[p + "down"].T


def route(z, top):
    """z [T, E] logits (bias included) -> (chosen experts [T, top] by falling logit, lower index first among equals;
    their weights: the softmax over the chosen logits)."""
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), -1)


def gated_unit(x, w_gate, w_up, w_down):
    g = x @ w_gate.T
    return (g * torch.sigmoid(g) * (x @ w_up.T)) @ w_down.T


def experts_ff(t, p, m, x):
    z = x @ t[p + "router"].T + t[p + "router.b"]
    sel, wgt = route(z, m["router"]["top"])
    y = torch.zeros_like(x)
    for i in range(x.shape[0]):
        for e, w in zip(sel[i].tolist(), wgt[i]):
            y[i] += w * gated_unit(x[i:i + 1], t[f"{p}e{e}.gate"], t[f"{p}e{e}.up"], t[f"{p}e{e}.down"])[0]
    if m.get("shared"):
        y = y + torch.sigmoid(x @ t[p + "shared.sg"].T) * gated_unit(x, t[p + "shared.gate"], t[p + "shared.up"], t[p + "shared.down"])
    return y


def model_logits(tensors, cfg, tokens, residual_out=None):
    t = {k: v.to(F64) for k, v in tensors.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = t["embed"][torch.tensor(tokens)]
    made = {}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        if l["type"] == "attention":
            src = l["mixer"].get("kv_from")
            y, made[i] = attention_mixer(t, p + "mix.", l["mixer"], x, eps, made[src] if src is not None else None)
        else:
            y = latent_mixer(t, p + "mix.", l["mixer"], x, eps)
        x = x + mult * t[p + "norm1"] * rms_unit(y, eps)
        if l.get("mlp"):
            f = dense_ff(t, p + "mlp.", x) if l["mlp"]["kind"] == "dense" else experts_ff(t, p + "mlp.", l["mlp"], x)
            x = x + mult * t[p + "norm2"] * rms_unit(f, eps)
        if residual_out is not None:
            residual_out.append(x.clone())
    return (t["final.norm"] * rms_unit(x, eps)) @ t["head"].T


def logit_error(got, want):
    """Per row: root mean square of the difference with its mean taken off, over the root mean square of the wanted row."""
    d = got.to(F64) - want.to(F64)
    d = d - d.mean(-1, keepdim=True)
    w = want.to(F64) - want.to(F64).mean(-1, keepdim=True)
    return torch.sqrt((d * d).mean(-1)) / torch.sqrt((w * w).mean(-1))
