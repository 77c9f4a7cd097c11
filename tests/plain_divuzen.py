"""A plain, slow implementation of the Divuzen design, written from its equations: float64, whole
sequences, explicit loops over tokens and heads, one function per mechanism.  It shares no code with
the package; the tests hold the package against it.

Notation: x the residual stream [T, d]; W tensors by their names in the weight file; positions count
from 0.  rms(v) = sqrt(mean(v^2) + eps).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def norm_one_plus(v, w, eps):
    """RMS norm whose stored weight lies around zero."""
    return rms_unit(v, eps) * (1.0 + w)


def norm_head(v, w, eps):
    """RMS norm over a head with a plain weight."""
    return rms_unit(v, eps) * w


def angles(T, dims, base, start=0):
    i = torch.arange(dims // 2, dtype=F64)
    f = torch.tensor(base, dtype=F64) ** (-2.0 * i / dims)
    p = torch.arange(start, start + T, dtype=F64)
    return p[:, None] * f[None, :]                       # [T, dims/2]


def rotate_pairs(v, dims, base, start=0):
    """v [T, heads, size]: entry 2i turns with entry 2i+1, i < dims/2; the rest passes."""
    a = angles(v.shape[0], dims, base, start)
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    out = v.clone()
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


def rotate_half(v, dims, base, start=0):
    """v [T, heads, size]: entry i turns with entry i + dims/2, i < dims/2; the rest passes."""
    a = angles(v.shape[0], dims, base, start)
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    h = dims // 2
    out = v.clone()
    u, w = v[..., :h], v[..., h:dims]
    out[..., :h] = u * c - w * s
    out[..., h:dims] = w * c + u * s
    return out


def attention_keys_values(h, W, p, mx, eps):
    """The keys (normed, rotated) and values of an attention layer that has its own."""
    T, G, dk, dv = h.shape[0], mx["kv_heads"], mx["dim"], mx["vdim"]
    k = norm_head((h @ W[p + "k"].T).view(T, G, dk), W[p + "k.norm"], eps)
    k = rotate_pairs(k, mx["rot"]["dims"], mx["rot"]["base"])
    v = (h @ W[p + "v"].T).view(T, G, dv)
    return k, v


def attention(h, W, p, mx, eps, k, v):
    """Causal softmax attention with a sink per head; k, v: this layer's or another layer's."""
    T, H, G, dk, dv = h.shape[0], mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = norm_head((h @ W[p + "q"].T).view(T, H, dk), W[p + "q.norm"], eps)
    q = rotate_pairs(q, mx["rot"]["dims"], mx["rot"]["base"])
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        sink = float(W[p + "sink"][head])
        for t in range(T):
            s = (k[: t + 1, g] @ q[t, head]) * mx["scale"]
            m = max(float(s.max()), sink)
            e = torch.exp(s - m)
            out[t, head] = (e[:, None] * v[: t + 1, g]).sum(0) / (e.sum() + math.exp(sink - m))
    return out.reshape(T, H * dv) @ W[p + "o"].T


def retention(h, W, p, mx, eps):
    """Linear attention with a fixed decay per head, token by token."""
    T, H, dk, dv = h.shape[0], mx["heads"], mx["dim"], mx["vdim"]
    q = rotate_half((h @ W[p + "q"].T).view(T, H, dk), mx["rot"]["dims"], mx["rot"]["base"])
    k = rotate_half((h @ W[p + "k"].T).view(T, H, dk), mx["rot"]["dims"], mx["rot"]["base"]) * dk ** -0.5
    v = (h @ W[p + "v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = mx["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = rms_unit(o, eps).reshape(T, H * dv)
    g = h @ W[p + "g"].T
    return (o * g * torch.sigmoid(g)) @ W[p + "o"].T


def dense_ff(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def expert(h, W, p):
    g = h @ W[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def choose(c, r):
    """The experts with the largest choice scores c inside the best groups (best first)."""
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = r["experts"] // groups["count"]
    by_group = c.view(groups["count"], per)
    score = by_group.sort(-1, descending=True).values[:, :2].sum(-1)
    kept = score.sort(descending=True, stable=True).indices[: groups["keep"]]
    masked = torch.full_like(by_group, -math.inf)
    masked[kept] = by_group[kept]
    order = masked.view(-1).sort(descending=True, stable=True)
    gaps = [math.inf]
    if r["top"] < groups["keep"] * per:
        gaps.append(float(order.values[r["top"] - 1] - order.values[r["top"]]))
    if groups["keep"] < groups["count"]:
        ranked = score.sort(descending=True).values
        gaps.append(float(ranked[groups["keep"] - 1] - ranked[groups["keep"]]))
    return order.indices[: r["top"]].tolist(), min(gaps)


def route(h_t, W, p, r, margin=None, given=None, slack=0.0):
    """One token: (chosen experts, their weights).  `margin`, a list, receives how far the choice is
    from another one: the gap between the last chosen and the first unchosen choice score, or between
    the last kept and the first dropped group's score, whichever is smaller.  `given`: experts that
    somebody else chose for this token; they are taken instead if they are what this router chooses
    once every choice score has moved by at most `slack` (theirs up, the others' down)."""
    s = torch.sigmoid(W[p + "router"] @ h_t)
    c = s + W[p + "correction"]
    chosen, gap = choose(c, r)
    if margin is not None:
        margin.append(gap)
    if given is not None and set(given) != set(chosen) and len(set(given)) == r["top"]:
        lift = torch.full_like(c, -slack)
        lift[list(given)] = slack
        if set(choose(c + lift, r)[0]) == set(given):
            chosen = list(given)
    w = s[chosen]
    return chosen, w / (w.sum() + 1e-20) * r["scale"]


def moe_ff(h, W, p, mlp, margins=None, given=None, slack=0.0):
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, w = route(h[t], W, p, mlp["router"], margins, (given or {}).get(t), slack)
        for j, e in enumerate(chosen):
            out[t] += w[j] * expert(h[t: t + 1], W, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + expert(h, W, p + "shared.") * torch.sigmoid(h @ W[p + "shared.sg"].T)
    return out


def forward(cfg, W, tokens, streams=None, mixers=None, margins=None, given=None, slack=0.0):
    """Logits [T, vocab] of one whole sequence.  `streams`, a list, receives the residual stream after
    every layer; `mixers` each mixer's output before its norm; `margins` one list per layer of routed
    experts with every token's distance from another choice of experts; `given` {layer: {position:
    experts}} and `slack`: choices to take over where they are as good as this router's own (see `route`)."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        h = norm_one_plus(x, W[p + "norm1"], eps)
        if layer["type"] == "attention":
            if mx.get("kv_from") is None:
                kept[i] = attention_keys_values(h, W, p + "mix.", mx, eps)
            a = attention(h, W, p + "mix.", mx, eps, *kept[i if mx.get("kv_from") is None else mx["kv_from"]])
        else:
            a = retention(h, W, p + "mix.", mx, eps)
        if mixers is not None:
            mixers.append(a)
        x = x + norm_one_plus(a, W[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = norm_one_plus(x, W[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                f = dense_ff(h, W, p + "mlp.", mlp["limit"])
            else:
                per_token = [] if margins is not None else None
                f = moe_ff(h, W, p + "mlp.", mlp, per_token, (given or {}).get(i), slack)
                if margins is not None:
                    margins.append(per_token)
            x = x + norm_one_plus(f, W[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return (norm_one_plus(x, W["final.norm"], eps) @ W["embed"].T) * cfg.get("logit_scale", 1.0)
