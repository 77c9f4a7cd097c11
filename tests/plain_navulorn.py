"""Navulorn, written out plainly: float64, one function per mechanism, whole sequences at once or
token by token with explicit Python loops.  Shares no code with the package; the tests compare the
engine with it.

The design: x = embed[token] * scale + bigram[row(previous token, token)]; every layer is
x <- norm(alpha x + mixer(x)), x <- norm(alpha x + ff(x)) with RMS norms AFTER the sums; mixers are
windowed grouped attention (norm over the whole query and key projections, partly rotated heads with
long-context frequency scaling, a sigmoid gate per head), windowed attention through a latent, and the
matrix-memory recurrence with exponential gates and a running maximum; feed-forwards are a tanh-gelu
gated unit or routed SiLU experts whose weights are a softmax over the chosen logits; the logits are
capped by a tanh.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token of one sequence from its start."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def embed(tokens, table, bigram, scale, buckets, mul_prev, mul_cur):
    idx = torch.tensor(list(tokens), dtype=torch.long)
    rows = torch.tensor(bigram_rows(list(tokens), buckets, mul_prev, mul_cur), dtype=torch.long)
    return table[idx] * scale + bigram[rows]


def frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims); with scaling {factor, low, high, original}: long wavelengths divided by the
    factor, short ones kept, a linear blend between."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / factor
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate(x, positions, freqs, dims, layout):
    """x [n, heads, dim]: the first `dims` entries of each head turn, the rest pass.  layout "half":
    entry i with entry i + dims/2; "pairs": entry 2i with entry 2i + 1."""
    out = x.clone()
    ang = positions.to(F64)[:, None] * freqs[None, :]             # [n, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    half = dims // 2
    if layout == "half":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    return out


def window_softmax_attention(q, k, v, scale, window, group):
    """q [n, H, dk], k [n, G, dk], v [n, G, dv] of one sequence from its start; token i sees j with
    0 <= i - j < window (window 0: all before it and itself).  Returns [n, H, dv]."""
    n, H, _ = q.shape
    out = torch.zeros((n, H, v.shape[-1]), dtype=F64)
    for i in range(n):
        lo = 0 if window <= 0 else max(0, i - window + 1)
        for h in range(H):
            g = h // group
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def attention(h, w, pre, mx, eps):
    """Grouped attention: norm over the whole q and k projections, rotation, window, gate per head."""
    n = h.shape[0]
    H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = rms_norm(h @ w[pre + "q"].T, w[pre + "q.norm"], eps).view(n, H, dk)
    k = rms_norm(h @ w[pre + "k"].T, w[pre + "k.norm"], eps).view(n, G, dk)
    v = (h @ w[pre + "v"].T).view(n, G, dv)
    rot = mx["rot"]
    f = frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    pos = torch.arange(n)
    q, k = rotate(q, pos, f, rot["dims"], "half"), rotate(k, pos, f, rot["dims"], "half")
    a = window_softmax_attention(q, k, v, mx["scale"], (mx.get("mask") or {}).get("size", 0), H // G)
    gate = torch.sigmoid(h @ w[pre + "g"].T)                      # [n, H]
    a = a * gate[:, :, None]
    return a.reshape(n, H * dv) @ w[pre + "o"].T


def latent_attention(h, w, pre, mx, eps):
    """Keys and values through a shared latent; one rotated key part for all heads."""
    n = h.shape[0]
    H, dk, r, dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = (h @ w[pre + "q"].T).view(n, H, dk + r)
    low = h @ w[pre + "dkv"].T
    c = rms_norm(low[:, :rank], w[pre + "dkv.norm"], eps)
    kr = low[:, rank:].view(n, 1, r)
    rot = mx["rot"]
    f = frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    pos = torch.arange(n)
    q_rot = rotate(q[..., dk:].contiguous(), pos, f, rot["dims"], "pairs")
    kr = rotate(kr, pos, f, rot["dims"], "pairs")
    k_plain = (c @ w[pre + "uk"].T).view(n, H, dk)
    v = (c @ w[pre + "uv"].T).view(n, H, dv)
    qq = torch.cat([q[..., :dk], q_rot], -1)
    kk = torch.cat([k_plain, kr.expand(n, H, r)], -1)
    a = window_softmax_attention(qq, kk, v, mx["scale"], (mx.get("mask") or {}).get("size", 0), 1)
    return a.reshape(n, H * dv) @ w[pre + "o"].T


def mlstm(h, w, pre, mx, eps):
    """The matrix memory, token by token, exactly as the recurrence reads."""
    n = h.shape[0]
    H, dk, dv, cap = mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"]
    q = (h @ w[pre + "q"].T).view(n, H, dk) * dk ** -0.5
    k = (h @ w[pre + "k"].T).view(n, H, dk)
    v = (h @ w[pre + "v"].T).view(n, H, dv)
    ig = cap * torch.tanh((h @ w[pre + "i"].T + w[pre + "i.b"]) / cap)                                  # [n, H]
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[pre + "f"].T + w[pre + "f.b"]) / cap))
    out = torch.zeros((n, H, dv), dtype=F64)
    for hd in range(H):
        S = torch.zeros((dk, dv), dtype=F64)
        nv = torch.zeros(dk, dtype=F64)
        m = 0.0
        for t in range(n):
            m_new = max(float(fg[t, hd]) + m, float(ig[t, hd]))
            a = math.exp(float(fg[t, hd]) + m - m_new)
            b = math.exp(float(ig[t, hd]) - m_new)
            S = a * S + b * torch.outer(k[t, hd], v[t, hd])
            nv = a * nv + b * k[t, hd]
            m = m_new
            den = max(abs(float(nv @ q[t, hd])), math.exp(-m)) + 1e-6
            out[t, hd] = (S.T @ q[t, hd]) / den
    o = rms(out, eps).reshape(n, H * dv) * w[pre + "norm"]
    o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def dense_ff(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, top, given=None, slack=0.0, margins=None):
    """(chosen experts [n, top], their weights [n, top]): the largest logits, softmax over them alone.
    `margins` (a list) takes, per token, how far the choice is from another one (the gap between the last
    chosen logit and the best one left out).  `given` {token index: experts}: somebody else's choice is taken
    over for a token when it is what this router gives after moving every logit by at most `slack`."""
    z = h @ w[pre + "router"].T + w[pre + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    E = z.shape[1]
    if margins is not None:
        rest = torch.topk(z, top + 1, dim=-1).values[:, -1] if top < E else torch.full((z.shape[0],), -math.inf, dtype=F64)
        margins.append([float(x) for x in (val[:, -1] - rest)])
    for t, cand in (given or {}).items():
        cand = [int(c) for c in cand]
        if t >= z.shape[0] or len(set(cand)) != top or sorted(cand) == sorted(idx[t].tolist()):
            continue
        out = [e for e in range(E) if e not in cand]
        if not out or float(z[t, cand].min()) + 2 * slack >= float(z[t, out].max()):
            idx[t] = torch.tensor(cand)
            val[t] = z[t, cand]
    return idx, torch.softmax(val, -1), z


def moe_ff(h, w, pre, mlp, given=None, slack=0.0, margins=None):
    top = mlp["router"]["top"]
    idx, wt, _ = route(h, w, pre, top, given, slack, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            p = f"{pre}e{e}."
            y = (silu(w[p + "gate"] @ h[t]) * (w[p + "up"] @ h[t])) @ w[p + "down"].T
            out[t] += wt[t, j] * y
    return out


MIXERS = {"attention": attention, "latent_attention": latent_attention, "mlstm": mlstm}


def layer(x, w, i, spec, cfg, given=None, slack=0.0, margins=None, coarse=None):
    """`coarse`, if given, is applied to what every sublayer reads and to what it returns: the stream as a
    sublayer with operands of fewer bits sees it (the stream itself and its sums keep their precision)."""
    eps, alpha = cfg["norm"]["eps"], cfg.get("postln_alpha", 1.0)
    see = coarse or (lambda t: t)
    a = see(MIXERS[spec["type"]](see(x), w, f"l{i}.mix.", spec["mixer"], eps))
    x = rms_norm(alpha * x + a, w[f"l{i}.norm1"], eps)
    mlp = spec.get("mlp")
    if mlp is not None:
        f = (dense_ff(see(x), w, f"l{i}.mlp.") if mlp["kind"] == "dense"
             else moe_ff(see(x), w, f"l{i}.mlp.", mlp, (given or {}).get(i), slack, margins))
        x = rms_norm(alpha * x + see(f), w[f"l{i}.norm2"], eps)
    return x


def forward(cfg, weights, tokens, streams=None, margins=None, given=None, slack=0.0, coarse=None):
    """Logits [n, vocab] (float64) of one sequence from its start.  `weights`: name -> tensor of any
    float type; `streams`, if a list, takes the stream after every layer; `margins`, `given`, `slack`: see
    `route` (`given` is {layer: {token index: experts}}); `coarse`: see `layer`."""
    w = {k: v.to(F64) for k, v in weights.items()}
    e = cfg.get("embedding") or {}
    b = e.get("bigram")
    if b:
        x = embed(tokens, w["embed"], w["bigram"], e.get("scale", 1.0), b["buckets"], b["mul_prev"], b["mul_cur"])
    else:
        x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)] * e.get("scale", 1.0)
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, w, i, spec, cfg, given, slack, margins, coarse)
        if streams is not None:
            streams.append(x.clone())
    x = rms_norm(x, w["final.norm"], cfg["norm"]["eps"])
    logits = (coarse(x) if coarse else x) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
