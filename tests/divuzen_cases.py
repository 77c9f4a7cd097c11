"""Small Divuzen configurations and random weights for the tests, made here (not by the package's
random-weights mode), and the glue that runs a schedule through the engine and the plain
implementation (tests/plain_divuzen.py).  The configurations differ from one another in every size;
between them they cover one and several query heads per key/value head, value heads smaller and
larger than key heads, rotation over a part of the head and over all of it in both layouts, layers
that read another layer's keys and values, decays from 0.5 to nearly 1, key heads of 8 to 128 and
value heads up to 136 entries in the retention layers, one and several groups of experts with one or
several kept, one expert per token and several, with and without a shared expert, layers without a
feed-forward, either mixer first, sizes that are no multiple of 8, and head sizes of 64 and 128.
"""
from __future__ import annotations

import copy
import math

import torch

import plain_divuzen


def rot(dims, base=10000.0):
    return {"dims": dims, "base": base}


def dense(ff, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top, count=1, keep=1, scale=1.0, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def att(heads, kv, dim, vdim, rdims, scale=None, base=10000.0, kv_from=None, mlp=None):
    mx = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": rot(rdims, base),
          "scale": scale if scale is not None else 2.0 / math.sqrt(dim)}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def ret(heads, dim, vdim, rdims, decay, base=500000.0, mlp=None):
    assert len(decay) == heads
    return {"type": "retention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "rot": rot(rdims, base), "decay": list(decay)}}


def config(layers, width, vocab, eps=1e-5, logit_scale=1.0):
    return {"architecture": "Divuzen", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
            "logit_scale": logit_scale}


CASES = {
    # one mechanism at a time
    "retention": config([ret(3, 8, 12, 4, [0.9, 0.97, 0.5], mlp=dense(40))], width=24, vocab=61, logit_scale=0.7),
    "retention_48": config([ret(2, 48, 40, 48, [0.99, 0.999], base=3000.0)], width=40, vocab=67, eps=3e-6),
    "retention_wide_values": config([ret(1, 16, 136, 8, [0.95], mlp=dense(24, 0.8))], width=32, vocab=53),
    "retention_128": config([ret(2, 128, 64, 64, [0.98, 0.9375])], width=48, vocab=71, logit_scale=2.0),
    "attention": config([att(4, 2, 16, 24, 8, mlp=dense(36, 2.5))], width=28, vocab=59),
    "attention_small_values": config([att(3, 3, 20, 6, 20, base=777.0)], width=36, vocab=73, eps=1e-6),
    "moe_groups": config([ret(2, 8, 8, 8, [0.8, 0.9], mlp=moe(12, 12, 4, count=3, keep=2, scale=1.7))], width=20,
                         vocab=47),
    "moe_one_each": config([att(2, 1, 12, 12, 6, mlp=moe(10, 5, 1, scale=0.6, shared=14))], width=22, vocab=43),
    "moe_groups_of_one": config([ret(1, 12, 20, 2, [0.75], mlp=moe(6, 6, 2, count=6, keep=3, shared=8))], width=18,
                                vocab=41, logit_scale=0.25),
    "retention_256_values": config([ret(1, 128, 256, 32, [0.9921875], mlp=dense(20))], width=24, vocab=37),
    # another layer's keys and values
    "shared_keys": config([att(4, 2, 12, 20, 4, mlp=dense(30)), ret(2, 8, 16, 8, [0.9, 0.99]),
                           att(4, 2, 12, 20, 4, scale=0.4, kv_from=0, mlp=moe(8, 8, 2, count=2, keep=1, shared=12))],
                          width=32, vocab=79),
    # head sizes 64 and 128 (the tensor-core attention kernels in bfloat16)
    "heads64": config([att(8, 2, 64, 64, 48, mlp=dense(72)), att(8, 2, 64, 64, 48, kv_from=0)], width=64, vocab=113),
    "heads128": config([att(2, 2, 128, 128, 64, base=50000.0), ret(2, 64, 128, 32, [0.96875, 0.999])], width=48,
                       vocab=103, logit_scale=1.5),
    # everything together, either mixer first
    "stack": config([ret(4, 16, 24, 16, [0.9, 0.95, 0.99, 0.999], mlp=dense(96, 1.2)),
                     att(6, 2, 32, 16, 16, mlp=moe(24, 8, 3, count=4, keep=2, scale=2.5, shared=40)),
                     ret(2, 24, 40, 12, [0.97, 0.6], mlp=moe(16, 6, 2, count=2, keep=2)),
                     att(6, 2, 32, 16, 16, kv_from=1, mlp=dense(80, 3.0)),
                     att(2, 1, 8, 8, 8)], width=64, vocab=131, logit_scale=0.4),
    "stack_attention_first": config([att(4, 4, 8, 10, 2, mlp=moe(20, 4, 2, shared=16)), ret(3, 12, 6, 10, [0.5, 0.9, 0.99]),
                                     att(3, 1, 20, 10, 10, mlp=dense(36))], width=40, vocab=89),
}


def tensor_shapes(cfg):
    """name -> (shape, kind) from the configuration alone, written out from the model's description."""
    d = cfg["width"]
    out = {"embed": ((cfg["vocab"], d), "embed"), "final.norm": ((d,), "norm")}
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = out[p + "norm1b"] = ((d,), "norm")
        H, dk, dv = mx["heads"], mx["dim"], mx["vdim"]
        if layer["type"] == "attention":
            out.update({p + "mix.q": ((H * dk, d), "matrix"), p + "mix.q.norm": ((dk,), "headnorm"),
                        p + "mix.sink": ((H,), "sink"), p + "mix.o": ((d, H * dv), "matrix")})
            if mx.get("kv_from") is None:
                G = mx["kv_heads"]
                out.update({p + "mix.k": ((G * dk, d), "matrix"), p + "mix.v": ((G * dv, d), "matrix"),
                            p + "mix.k.norm": ((dk,), "headnorm")})
        else:
            out.update({p + "mix.q": ((H * dk, d), "matrix"), p + "mix.k": ((H * dk, d), "matrix"),
                        p + "mix.v": ((H * dv, d), "matrix"), p + "mix.g": ((H * dv, d), "matrix"),
                        p + "mix.o": ((d, H * dv), "matrix")})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = out[p + "norm2b"] = ((d,), "norm")
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            out.update({p + "mlp.gate": ((F, d), "matrix"), p + "mlp.up": ((F, d), "matrix"),
                        p + "mlp.down": ((d, F), "matrix")})
            continue
        F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
        out[p + "mlp.router"] = ((E, d), "router")
        out[p + "mlp.correction"] = ((E,), "correction")
        for e in range(E):
            out.update({f"{p}mlp.e{e}.gate": ((F, d), "matrix"), f"{p}mlp.e{e}.up": ((F, d), "matrix"),
                        f"{p}mlp.e{e}.down": ((d, F), "matrix")})
        if mlp.get("shared"):
            S = mlp["shared"]["ff"]
            out.update({p + "mlp.shared.gate": ((S, d), "matrix"), p + "mlp.shared.up": ((S, d), "matrix"),
                        p + "mlp.shared.down": ((d, S), "matrix"), p + "mlp.shared.sg": ((1, d), "matrix")})
    return out


def make_weights(cfg, seed, dtype=torch.float32, gain=1.3):
    """Random tensors at which every mechanism moves the output: activations of order 1 (the clamps of
    the dense feed-forward bite now and then), sinks that take a visible share of a row, corrections
    that make some choice scores negative, and a router whose scores lie far enough apart that the
    choice does not hang on the last bits.  Stored in `dtype`."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if kind == "matrix":
            t = rnd(*shape) * gain / math.sqrt(shape[1])
        elif kind == "router":
            t = rnd(*shape) * 4.0 / math.sqrt(shape[1])
        elif kind == "embed":
            t = rnd(*shape)
        elif kind == "norm":
            t = 0.2 * rnd(*shape)                          # stored around zero
        elif kind == "headnorm":
            t = 1.0 + 0.2 * rnd(*shape)
        elif kind == "sink":
            t = 1.0 + rnd(*shape)
        elif kind == "correction":
            t = -0.8 + 0.5 * rnd(*shape)
        else:
            raise ValueError(kind)
        out[name] = t.to(dtype)
    return out


def oracle(cfg, weights, tokens, streams=None, given=None, slack=0.0):
    """float64 logits [T, vocab] of the plain implementation from the weights as stored.  The result
    carries `margin` [T], how far each token's choice of experts is from another choice (the smallest
    over the layers of routed experts, infinite without any), and `again(given, slack)`: the logits once
    more with somebody else's choices taken over where they are as good as the plain router's own."""
    margins = []
    logits = plain_divuzen.forward(cfg, weights, tokens, streams, margins=margins, given=given, slack=slack)
    m = torch.full((len(tokens),), math.inf, dtype=torch.float64)
    for per_token in margins:
        m = torch.minimum(m, torch.tensor(per_token, dtype=torch.float64))
    logits.margin = m
    logits.again = lambda given, slack: oracle(cfg, weights, tokens, given=given, slack=slack)
    return logits


def sharpened(cfg, factor, layers=None):
    cfg = copy.deepcopy(cfg)
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "attention" and (layers is None or i in layers):
            layer["mixer"]["scale"] *= factor
    return cfg


def _normed_embedding(cfg, w, token):
    return plain_divuzen.norm_one_plus(w["embed"].double()[token], w["l0.norm1"].double(), cfg["norm"]["eps"])


def _redirect(cfg, w, asker, target):
    """The map R on the normed stream with R x(asker) = x(target), identity across x(asker): a projection
    W R then gives the asker what W gives the target and leaves the other tokens nearly alone."""
    xa, xb = _normed_embedding(cfg, w, asker), _normed_embedding(cfg, w, target)
    return torch.eye(cfg["width"], dtype=torch.float64) + torch.outer(xb - xa, xa) / (xa @ xa)


def marked_attention(cfg, w, asker, target):
    """Layer 0 (an attention layer with keys of its own): every query head asks with its group's key
    projection and key norm, and the token `asker` asks as if it were `target`.  With a sharp scale, a
    row of `asker` hangs on the key of a `target` token when one is visible (on the part of the head
    that is not rotated; the rotated part adds or takes a little, by distance) and is spread over the
    other keys and the sink when none is."""
    w = dict(w)
    mx = cfg["layers"][0]["mixer"]
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    k = w["l0.mix.k"].double().view(G, d, -1)
    q = torch.stack([k[h // (H // G)] for h in range(H)]).reshape(H * d, -1) @ _redirect(cfg, w, asker, target)
    w["l0.mix.q"] = q.to(w["l0.mix.q"].dtype)
    w["l0.mix.q.norm"] = w["l0.mix.k.norm"].clone()
    return w


def build_engine(cfg, weights, dtype, max_tokens, block_size=8, max_requests=4, use_graphs=None, device="cuda:0"):
    """`use_graphs` None: replay from graphs in float32 only (a replayed step does not show which experts
    it chose, and in bfloat16 the comparison wants to know: see `oracle`)."""
    if use_graphs is None:
        use_graphs = dtype == "float32"
    from rllm_b200.config import config_from_dict
    from rllm_b200.engine import Engine
    from rllm_b200.models.model import DecoderModel, parse_dtype
    from rllm_b200.parts import Runtime
    model = DecoderModel(config_from_dict(cfg).model_spec(), Runtime(torch.device(device), parse_dtype(dtype)))
    model.load_tensors(dict(weights))
    return Engine(model, block_size=block_size, max_tokens=max_tokens, max_requests=max_requests,
                  use_graphs=use_graphs)


def tokens_for(cfg, n, seed, avoid=()):
    g = torch.Generator().manual_seed(2000 + seed)
    free = [t for t in range(cfg["vocab"]) if t not in avoid]
    return [free[int(i)] for i in torch.randint(0, len(free), (n,), generator=g)]


def row_error(row, ref):
    """max |row - ref| / max |ref| with the rows' means taken off (logits are defined up to a shift)."""
    row, ref = row.double() - row.double().mean(), ref.double() - ref.double().mean()
    return float((row - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
