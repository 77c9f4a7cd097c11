"""Small Navulorn configurations and random weights for the tests, made here (not by the package's
random-weights mode), and the glue that runs the plain implementation (tests/plain_navulorn.py).  The
configurations differ from one another in every size; between them they cover one and several query
heads per key/value head, value heads smaller and larger than key heads and equal to them, rotation over
a part of the head and over all of it, with and without the long-context frequency rule, windows from 1
key to more than the prompt, latents with rot_dim 2 and up, one head, one expert per token, all experts
per token, layers without a feed-forward, a model without a pair table, alpha 1, head sizes of 64 and 128
(the tensor-core attention kernels) and latents of 64 and 128 entries (the tensor-core latent kernel).
"""
from __future__ import annotations

import copy
import math

import torch

import plain_navulorn


def rot(dims, base=10000.0, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def att(heads, kv, dim, vdim, rdims, window, scale=None, base=10000.0, scaling=None, mlp=None):
    mx = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": rot(rdims, base, scaling),
          "scale": scale if scale is not None else 2.0 / math.sqrt(dim)}
    if window:
        mx["mask"] = {"size": window}
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def lat(heads, dim, rdim, vdim, rank, window, scale=None, base=5000.0, mlp=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rdim, "vdim": vdim, "kv_rank": rank, "rot": rot(rdim, base),
          "scale": scale if scale is not None else 2.0 / math.sqrt(dim + rdim)}
    if window:
        mx["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def mem(heads, dim, vdim, cap=8.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def config(layers, width, vocab, eps=1e-5, alpha=2.0, scale=1.5, bigram=(37, 5, 11), softcap=20.0):
    emb = {"scale": scale}
    if bigram:
        emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    return {"architecture": "Navulorn", "vocab": vocab, "width": width, "embedding": emb, "layers": layers,
            "norm": {"eps": eps}, "postln_alpha": alpha, "logit_softcap": softcap}


LLAMA = (8.0, 1.0, 4.0, 64)        # factor, low, high, original: wavelengths between 16 and 64 positions blend

CASES = {
    # one mechanism at a time
    "attention": config([att(4, 2, 16, 24, 8, 9, mlp=dense(36))], width=28, vocab=59),
    "attention_scaled": config([att(3, 3, 20, 6, 20, 5, base=50.0, scaling=LLAMA)], width=36, vocab=73, eps=1e-6,
                               alpha=0.5, bigram=(11, 3, 1)),
    "attention_window_1": config([att(2, 1, 8, 8, 4, 1, mlp=dense(20))], width=20, vocab=41, alpha=1.0),
    "attention_no_window": config([att(2, 2, 12, 4, 12, 0)], width=24, vocab=43, bigram=None, scale=1.0, softcap=0.0),
    "latent": config([lat(3, 12, 4, 10, 20, 7, mlp=dense(30))], width=32, vocab=61),
    "latent_one_head": config([lat(1, 6, 2, 14, 9, 33)], width=18, vocab=37, alpha=3.5, bigram=(5, 1, 1)),
    "memory": config([mem(3, 8, 12, mlp=dense(40))], width=24, vocab=53),
    "memory_48": config([mem(2, 48, 40, cap=15.0)], width=40, vocab=67, eps=3e-6),
    "memory_wide_values": config([mem(1, 16, 136, cap=4.0, mlp=moe(12, 3, 3))], width=32, vocab=47),
    "memory_128": config([mem(2, 128, 64)], width=48, vocab=71),
    "memory_one_wide_head": config([mem(1, 24, 272, cap=11.0, mlp=dense(28))], width=36, vocab=51, alpha=1.5),   # beyond the fast kernel
    "moe": config([mem(2, 8, 8, mlp=moe(12, 12, 4))], width=20, vocab=47, alpha=1.5),
    "moe_one_each": config([att(2, 1, 12, 12, 6, 6, mlp=moe(10, 5, 1))], width=22, vocab=43),
    # head sizes 64 and 128 with values of the same size (the tensor-core attention kernels in bfloat16) and
    # latents of 64 and 128 entries with key rows that are multiples of 16 (the tensor-core latent kernel)
    "heads64": config([att(8, 2, 64, 64, 48, 21, mlp=dense(72)), att(2, 2, 64, 64, 64, 44, scaling=LLAMA)], width=64,
                      vocab=113),
    "heads_tiny_windows": config([att(4, 2, 64, 64, 32, 3, mlp=dense(24)), att(2, 1, 128, 128, 128, 1), att(4, 4, 64, 64, 2, 130)],
                                 width=48, vocab=83, alpha=2.5, bigram=(29, 4, 9)),
    "heads128": config([att(2, 1, 128, 128, 64, 50, base=50000.0), mem(2, 64, 128)], width=48, vocab=103, alpha=4.0),
    "latent64": config([lat(4, 16, 16, 24, 64, 45, mlp=dense(40)), lat(2, 8, 32, 8, 128, 19)], width=64, vocab=97),
    # sizes that are no multiple of 2, 4 or 8 wherever the design allows it
    "odd_sizes": config([att(3, 1, 10, 7, 6, 4, mlp=moe(9, 3, 2)), lat(3, 5, 2, 3, 7, 5, mlp=dense(11)), mem(3, 5, 3, cap=5.0),
                         att(1, 1, 6, 9, 2, 3)], width=37, vocab=45, alpha=1.7, bigram=(13, 3, 2), softcap=9.0),
    # everything together, in two orders
    "stack": config([mem(4, 16, 24, mlp=dense(96)),
                     att(6, 2, 32, 16, 16, 13, scaling=LLAMA, base=300.0, mlp=moe(24, 8, 3)),
                     lat(4, 16, 8, 20, 24, 30, mlp=moe(16, 6, 2)),
                     att(6, 2, 32, 16, 16, 13, scaling=LLAMA, base=300.0, mlp=dense(80)),
                     mem(2, 24, 40, cap=10.0, mlp=moe(16, 6, 2)),
                     lat(2, 8, 8, 8, 16, 11)], width=64, vocab=131, alpha=2.5, scale=4.0),
    "stack_attention_first": config([att(4, 4, 8, 10, 2, 10, mlp=moe(20, 4, 2)), lat(3, 10, 6, 6, 12, 25, mlp=dense(36)),
                                     mem(3, 12, 18, cap=6.0), att(3, 1, 20, 10, 10, 44, mlp=dense(36))], width=40,
                                    vocab=89, alpha=2.0, bigram=(53, 2, 9)),
}


def tensor_shapes(cfg):
    """name -> (shape, kind) from the configuration alone, written out from the model's description."""
    d = cfg["width"]
    out = {"embed": ((cfg["vocab"], d), "embed"), "final.norm": ((d,), "norm"), "head": ((cfg["vocab"], d), "matrix")}
    b = (cfg.get("embedding") or {}).get("bigram")
    if b:
        out["bigram"] = ((b["buckets"] + 1, d), "embed")
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = ((d,), "norm")
        H, dk, dv = mx["heads"], mx["dim"], mx["vdim"]
        if layer["type"] == "attention":
            G = mx["kv_heads"]
            out.update({p + "mix.q": ((H * dk, d), "matrix"), p + "mix.k": ((G * dk, d), "matrix"),
                        p + "mix.v": ((G * dv, d), "matrix"), p + "mix.q.norm": ((H * dk,), "norm"),
                        p + "mix.k.norm": ((G * dk,), "norm"), p + "mix.g": ((H, d), "matrix"),
                        p + "mix.o": ((d, H * dv), "matrix")})
        elif layer["type"] == "latent_attention":
            r, rank = mx["rot_dim"], mx["kv_rank"]
            out.update({p + "mix.q": ((H * (dk + r), d), "matrix"), p + "mix.dkv": ((rank + r, d), "matrix"),
                        p + "mix.dkv.norm": ((rank,), "norm"), p + "mix.uk": ((H * dk, rank), "matrix"),
                        p + "mix.uv": ((H * dv, rank), "matrix"), p + "mix.o": ((d, H * dv), "matrix")})
        else:
            out.update({p + "mix.q": ((H * dk, d), "matrix"), p + "mix.k": ((H * dk, d), "matrix"),
                        p + "mix.v": ((H * dv, d), "matrix"), p + "mix.g": ((H * dv, d), "matrix"),
                        p + "mix.o": ((d, H * dv), "matrix"), p + "mix.norm": ((H * dv,), "norm"),
                        p + "mix.i": ((H, d), "gate"), p + "mix.f": ((H, d), "gate"),
                        p + "mix.i.b": ((H,), "gate_bias"), p + "mix.f.b": ((H,), "forget_bias")})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[p + "norm2"] = ((d,), "norm")
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            out.update({p + "mlp.gate": ((F, d), "matrix"), p + "mlp.up": ((F, d), "matrix"),
                        p + "mlp.down": ((d, F), "matrix")})
            continue
        F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
        out[p + "mlp.router"] = ((E, d), "router")
        out[p + "mlp.router.b"] = ((E,), "router_bias")
        for e in range(E):
            out.update({f"{p}mlp.e{e}.gate": ((F, d), "matrix"), f"{p}mlp.e{e}.up": ((F, d), "matrix"),
                        f"{p}mlp.e{e}.down": ((d, F), "matrix")})
    return out


def make_weights(cfg, seed, dtype=torch.float32, gain=1.3):
    """Random tensors at which every mechanism moves the output: the stream has entries of order 1 behind
    every norm, so products of order 1; gates whose caps bite now and then; forget gates between 0.5 and
    nearly 1; a router whose logits lie far enough apart that the choice seldom hangs on the last bits, with
    a bias that decides some of them.  Stored in `dtype`."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if kind == "matrix":
            t = rnd(*shape) * gain / math.sqrt(shape[1])
        elif kind == "router":
            t = rnd(*shape) * 4.0 / math.sqrt(shape[1])
        elif kind == "gate":
            t = rnd(*shape) * 3.0 / math.sqrt(shape[1])
        elif kind == "embed":
            t = rnd(*shape)
        elif kind == "norm":
            t = 1.0 + 0.2 * rnd(*shape)
        elif kind == "gate_bias":
            t = rnd(*shape)
        elif kind == "forget_bias":
            t = 2.0 + 2.0 * rnd(*shape)
        elif kind == "router_bias":
            t = 1.5 * rnd(*shape)
        else:
            raise ValueError(kind)
        out[name] = t.to(dtype)
    return out


def oracle(cfg, weights, tokens, streams=None, given=None, slack=0.0):
    """float64 logits [T, vocab] of the plain implementation from the weights as stored.  The result
    carries `margin` [T], how far each token's choice of experts is from another choice (the smallest
    over the layers of routed experts, infinite without any), and `again(given, slack)`: the logits once
    more with somebody else's choices taken over where they are as good as the plain router's own.  For
    weights stored in bfloat16 it also carries `noise` [T]: how far each row moves when every sublayer reads
    and returns rows rounded to bfloat16 (what rounding alone does to the row, with exact arithmetic)."""
    margins = []
    logits = plain_navulorn.forward(cfg, weights, tokens, streams, margins=margins, given=given, slack=slack)
    if weights["embed"].dtype == torch.bfloat16:
        coarse = plain_navulorn.forward(cfg, weights, tokens, given=given, slack=slack,
                                        coarse=lambda t: t.to(torch.bfloat16).to(torch.float64))
        logits.noise = [row_error(coarse[p], logits[p]) for p in range(len(tokens))]
    m = torch.full((len(tokens),), math.inf, dtype=torch.float64)
    for per_token in margins:
        m = torch.minimum(m, torch.tensor(per_token, dtype=torch.float64))
    logits.margin = m
    logits.again = lambda given, slack: oracle(cfg, weights, tokens, given=given, slack=slack)
    return logits


def sharpened(cfg, factor, layers=None):
    """The same model with the attention layers' scores multiplied by `factor`: rows then hang on few keys."""
    cfg = copy.deepcopy(cfg)
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "mlstm" and (layers is None or i in layers):
            layer["mixer"]["scale"] *= factor
    return cfg


def with_windows(cfg, delta):
    """The same model with every window `delta` keys longer: what a mask that is off by one would compute."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer["mixer"].get("mask"):
            layer["mixer"]["mask"]["size"] += delta
    return cfg


def marked_attention(cfg, w, asker, target, boost=12.0):
    """Layer 0 (an attention layer): every query head asks with its group's key projection and the key norm's
    weights, and the token `asker` asks as if it were `target` (the map R on the stream with R x(asker) =
    x(target) and the identity across x(asker), where x is the scaled embedding row, which the pair table
    moves only a little when the embedding's scale is large).  With a sharp scale, a row of `asker` hangs on
    the key of a `target` token when one is inside the window (on the part of the head that is not rotated;
    the rotated part adds or takes a little, by distance) and is spread over the other keys when none is.  The
    output projection is multiplied by `boost`, so that what attention finds is not drowned by the stream."""
    w = dict(w)
    mx = cfg["layers"][0]["mixer"]
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    p = "l0.mix."
    scale = cfg["embedding"]["scale"]
    xa, xb = w["embed"].double()[asker] * scale, w["embed"].double()[target] * scale
    R = torch.eye(cfg["width"], dtype=torch.float64) + torch.outer(xb - xa, xa) / (xa @ xa)
    k = w[p + "k"].double().view(G, d, -1)
    kn = w[p + "k.norm"].double().view(G, d)
    q = torch.stack([k[h // (H // G)] for h in range(H)]).reshape(H * d, -1) @ R
    w[p + "q"] = q.to(w[p + "q"].dtype)
    w[p + "q.norm"] = torch.stack([kn[h // (H // G)] for h in range(H)]).reshape(H * d).to(w[p + "q.norm"].dtype)
    w[p + "o"] = (w[p + "o"].double() * boost).to(w[p + "o"].dtype)
    return w


def marked_memory(cfg, w, marker, gate=16.0, boost=12.0):
    """Layer 0 (a matrix-memory layer): the input gate opens for the token `marker` alone (its row points along
    the marker's scaled embedding row, its bias is negative) and the forget gate stays open (no row, a large bias), so
    what the marker wrote stays the larger part of the memory for hundreds of tokens: a state that is lost,
    reset or carried wrongly between steps and segments changes every later row."""
    w = dict(w)
    H = cfg["layers"][0]["mixer"]["heads"]
    xa = w["embed"].double()[marker] * cfg["embedding"]["scale"]
    w["l0.mix.i"] = (torch.outer(torch.ones(H, dtype=torch.float64), xa) * gate / (xa @ xa)).to(w["l0.mix.i"].dtype)
    w["l0.mix.i.b"] = torch.full((H,), -6.0).to(w["l0.mix.i.b"].dtype)
    w["l0.mix.o"] = (w["l0.mix.o"].double() * boost).to(w["l0.mix.o"].dtype)     # not drowned by the stream
    w["l0.mix.f"] = torch.zeros_like(w["l0.mix.f"])
    w["l0.mix.f.b"] = torch.full((H,), 8.0).to(w["l0.mix.f.b"].dtype)
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
    g = torch.Generator().manual_seed(3000 + seed)
    free = [t for t in range(cfg["vocab"]) if t not in avoid]
    return [free[int(i)] for i in torch.randint(0, len(free), (n,), generator=g)]


def row_error(row, ref):
    """max |row - ref| / max |ref| with the rows' means taken off (logits are defined up to a shift)."""
    row, ref = row.double() - row.double().mean(), ref.double() - ref.double().mean()
    return float((row - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
