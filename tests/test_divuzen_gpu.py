"""Divuzen through the engine against the plain implementation (tests/plain_divuzen.py, float64).

Each mechanism's kernel alone against its plain function; whole prompts against token-by-token
decoding; portions down to two tokens; batches of unequal requests against each alone with pages and
state slots used again; a key far back among hundreds, at page borders, with sharp attention and a
check that a lost key or a forgotten sink would show; the first tokens of a sequence; long portions
that the retention kernel cuts along time; long decoding through CUDA-graph replay; sizes the
kernels' fast paths do not take; greedy generation through ``LLM.generate`` and the scheduler;
``bin/trace_run``.  The configurations and weights are made in tests/divuzen_cases.py.
"""
import json
import math

import pytest
import torch

import divuzen_cases as dc
import plain_divuzen as pd
from divuzen_cases import CASES, row_error

pytestmark = pytest.mark.gpu

# max |engine - plain| / max |plain| over a logits row (means taken off).  float32: the engine sums in
# another order than the float64 plain implementation.  bfloat16: weights, the operands of every product
# and the cache are rounded to 8 bits of mantissa (a lost key or sink moves rows by 0.1 to 1).
TOL = {"float32": 4e-5, "bfloat16": 6e-2}
# A token whose choice of experts hangs on less than this (a gap between choice scores, which lie in
# [-1, 2]) may take another expert when the router's input carries the rounding of the mode, and the rows
# after it then differ too.  So the comparison looks at which experts the engine chose: where the choice
# hangs on less than this, the plain implementation takes the engine's experts over if they are what its
# own router gives after moving every choice score by at most this much; everywhere else it keeps its own.
CLOSE = {"float32": 2e-5, "bfloat16": 3e-2}
DEV = "cuda:0"


def stored(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


class Rows(dict):
    """{(request, position): logits row}, and `chosen` {request: {layer: {position: experts}}}."""
    def __init__(self):
        super().__init__()
        self.chosen = {}


def watch(engine):
    """Records which experts every layer of routed experts chooses (eager steps only)."""
    if getattr(engine, "_watched", None) is None:
        engine._watched = []
        for li, block in enumerate(engine.model.blocks):
            ffn = getattr(block, "ffn", None)
            if ffn is None or not hasattr(ffn, "route"):
                continue
            seen = []

            def spy(h, _inner=ffn.route, _seen=seen):
                r = _inner(h)
                if not torch.cuda.is_current_stream_capturing():
                    _seen.append(r[0].detach().cpu())
                return r
            ffn.route = spy
            engine._watched.append((li, seen))
    return engine._watched


def run(engine, steps):
    """`steps`: list of (entries, end); an entry is (request, tokens, want).  Returns Rows."""
    from rllm_b200.engine import StepItem
    pos, out = {}, Rows()
    watched = watch(engine)
    for entries, end in steps:
        for _, seen in watched:
            seen.clear()
        logits = engine.step([StepItem(r, toks, want) for r, toks, want in entries])
        n = sum(len(toks) for _, toks, _ in entries)
        for li, seen in watched:
            idx = torch.cat(seen) if seen else None
            if idx is None or idx.shape[0] != n:
                continue                                   # a replayed step
            at = 0
            for r, toks, _ in entries:
                mine = out.chosen.setdefault(r, {}).setdefault(li, {})
                for j in range(len(toks)):
                    mine[pos.get(r, 0) + j] = idx[at + j].tolist()
                at += len(toks)
        row = 0
        for r, toks, want in entries:
            start = pos.get(r, 0)
            for w in want:
                out[(r, start + w)] = logits[row].detach().float().cpu()
                row += 1
            pos[r] = start + len(toks)
        for r in end:
            engine.finish(r)
            pos.pop(r, None)
    engine.check_device_errors()
    return out


def compare(out, refs, dtype, what, tol=None):
    tol = tol or TOL[dtype]
    assert out, what
    refs = dict(refs)
    for r, ref in refs.items():
        margin = getattr(ref, "margin", None)
        if margin is not None and float(margin.min()) < CLOSE[dtype] and getattr(out, "chosen", {}).get(r):
            refs[r] = ref.again(out.chosen[r], CLOSE[dtype])
    bad = []
    for (r, p), row in sorted(out.items()):
        e = row_error(row, refs[r][p])
        if not e <= tol:
            bad.append(f"request {r} position {p}: error {e:.3e} > {tol}")
    assert not bad, f"{what}: " + "; ".join(bad[:12]) + f" ({len(bad)} of {len(out)} rows)"


def cut(tokens, sizes):
    """Portions of the given sizes in turn (the last size repeats), every position wanted."""
    out, at, i = [], 0, 0
    while at < len(tokens):
        k = min(sizes[min(i, len(sizes) - 1)], len(tokens) - at)
        out.append((tokens[at:at + k], list(range(k))))
        at, i = at + k, i + 1
    return out


def one_by_one(r, toks, lo=0):
    return [([(r, [t], [0])], []) for t in toks[lo:]]


def closing(steps, r):
    steps[-1] = (steps[-1][0], [r])
    return steps


# ---------------------------------------------------------------- each kernel alone

def _angles_table(positions, dims, base):
    from rllm_b200.csrc import ops
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64).float().to(DEV)
    return ops.rope_table(positions, f)


def _rotate_at(v, positions, dims, base, pairs):
    """The plain rotation of rows that stand at the given positions (each row a sequence of its own)."""
    out = torch.empty_like(v)
    for t, p in enumerate(positions):
        fn = pd.rotate_pairs if pairs else pd.rotate_half
        out[t] = fn(v[t:t + 1], dims, base, start=p)[0]
    return out


@pytest.mark.parametrize("pairs,rot,hd,hdv,has_kv", [(True, 6, 10, 14, True), (False, 12, 12, 4, True),
                                                     (True, 40, 40, 40, False), (True, 0, 6, 6, True)])
def test_head_norm_rotation_store_kernel(pairs, rot, hd, hdv, has_kv):
    from rllm_b200.csrc import ops
    H, G, bs, n, eps = 5, 2, 4, 7, 3e-5
    g = torch.Generator().manual_seed(1)
    width = H * hd + (G * (hd + hdv) if has_kv else 0)
    rows = torch.randn(n, width + 3, generator=g).to(DEV)
    qw, kw = (1 + 0.3 * torch.randn(hd, generator=g)).to(DEV), (1 + 0.3 * torch.randn(hd, generator=g)).to(DEV)
    pos = [0, 1, 2, 40, 41, 300, 7]
    positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    slots = torch.tensor([3, 0, 5, -1, 9, 11, 6], dtype=torch.int32, device=DEV)
    q = torch.empty((n, H * hd), device=DEV)
    kc, vc = torch.zeros((3, G, bs, hd), device=DEV), torch.zeros((3, G, bs, hdv), device=DEV)
    cs = _angles_table(positions, rot, 300.0) if rot else None
    ops.head_norm_rope_store(rows[:, :width], qw, kw if has_kv else None, cs, rot, pairs, slots, q, kc, vc, H, G, hd,
                             hdv, bs, eps, has_kv=has_kv)
    r64 = rows.double().cpu()
    qh = pd.norm_head(r64[:, :H * hd].view(n, H, hd), qw.double().cpu(), eps)
    want_q = _rotate_at(qh, pos, rot, 300.0, pairs) if rot else qh
    assert torch.allclose(q.double().cpu().view(n, H, hd), want_q, atol=2e-5)
    if not has_kv:
        assert float(kc.abs().max()) == 0.0 and float(vc.abs().max()) == 0.0
        return
    kh = pd.norm_head(r64[:, H * hd:(H + G) * hd].view(n, G, hd), kw.double().cpu(), eps)
    want_k = _rotate_at(kh, pos, rot, 300.0, pairs) if rot else kh
    want_v = rows[:, (H + G) * hd:width].cpu().view(n, G, hdv)
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        assert torch.allclose(kc[s // bs, :, s % bs].double().cpu(), want_k[t], atol=2e-5)
        assert torch.equal(vc[s // bs, :, s % bs].cpu(), want_v[t])
    assert float(kc[0, :, 1].abs().max()) == 0.0 and float(vc[0, :, 2].abs().max()) == 0.0     # slots nobody named


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [50, 256])
def test_join_and_next_norm_kernel(dtype, d):
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    y = (3 * torch.randn(9, d + 20, generator=g)).to(DEV)
    x = torch.randn(9, d, generator=g).to(DEV)
    w1, w2 = (1 + 0.3 * torch.randn(d, generator=g)).to(DEV), (1 + 0.3 * torch.randn(d, generator=g)).to(DEV)
    out = torch.empty((9, d), dtype=dtype, device=DEV)
    want_x = x.double() + pd.rms_unit(y[:, 5:5 + d].double(), 1e-4) * w1.double()
    want_h = pd.rms_unit(want_x, 2e-6) * w2.double()
    ops.join_norm_rows(y[:, 5:5 + d], w1, 1e-4, x, w2, 2e-6, out)
    assert torch.allclose(x.double(), want_x, atol=1e-5)
    assert torch.allclose(out.double(), want_h, atol=1e-5 if dtype == torch.float32 else 3e-2)


def _paged(rows, bs, n_pages, g):
    """rows [T, heads, size] of one request laid into pages in a scrambled order: (cache, table row)."""
    T, heads, size = rows.shape
    used = -(-T // bs)
    pages = torch.randperm(n_pages, generator=g)[:used]
    cache = torch.zeros((n_pages, heads, bs, size), dtype=rows.dtype)
    for p in range(T):
        cache[pages[p // bs], :, p % bs] = rows[p]
    return cache, pages.to(torch.int32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,hdv", [(4, 2, 12, 20), (3, 3, 64, 64), (2, 1, 128, 128), (6, 2, 64, 32)])
def test_attention_kernel_with_sinks(dtype, H, G, hd, hdv):
    """Attention over pages with a sink per head (and value heads of their own size), a prompt's portion
    and single tokens: against the formula.  A sink of minus infinity gives plain attention; a large
    one takes the row."""
    from rllm_b200.csrc import ops
    from rllm_b200.engine.batch import StepContext
    bs, T, scale = 8, 77, 0.7 / math.sqrt(hd)
    g = torch.Generator().manual_seed(3)
    k, v = torch.randn(T, G, hd, generator=g).to(dtype), torch.randn(T, G, hdv, generator=g).to(dtype)
    q = (2 * torch.randn(T, H, hd, generator=g)).to(dtype)
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0, 1.0, -0.3][:H])
    kc, pages = _paged(k, bs, 13, g)
    vc = torch.zeros((13, G, bs, hdv), dtype=dtype)
    for p in range(T):
        vc[pages[p // bs], :, p % bs] = v[p]
    want = torch.zeros(T, H, hdv, dtype=torch.float64)
    for h in range(H):
        s = q[:, h].double() @ k[:, h // (H // G)].double().T * scale
        s = s.masked_fill(torch.ones(T, T).triu(1).bool(), -math.inf)
        m = torch.maximum(s.max(-1).values, sink[h].double())
        e = torch.exp(s - m[:, None])
        want[:, h] = (e @ v[:, h // (H // G)].double()) / (e.sum(-1) + torch.exp(sink[h].double() - m))[:, None]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    table = pages.view(1, -1).to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    for lo, hi in ((0, T), (40, T), (T - 1, T), (0, 1), (T - 5, T)):     # a whole prompt, a portion, single tokens, a few
        k_ = hi - lo
        ctx = StepContext(n_tokens=k_, n_requests=1, tokens=i32([0] * k_), positions=i32(list(range(lo, hi))),
                          seq_ids=i32([0] * k_), cu_q=i32([0, k_]), ctx_lens=i32([hi]), logit_rows=None, q_lens=[k_],
                          start_pos=[lo], ctx_lens_host=[hi], max_q_len=k_, max_ctx_len=hi)
        out = torch.empty((k_, H * hdv), dtype=dtype, device=DEV)
        qs = q[lo:hi].reshape(k_, -1).to(DEV)
        # the dispatcher (tensor-core kernels for bfloat16 heads of 64 and 128), and the plain kernel
        ops.paged_attention(qs, kc.to(DEV), vc.to(DEV), out, ctx, table, H, G, hd, bs, scale, v_head_dim=hdv,
                            sink=sink.to(DEV))
        plain = torch.empty_like(out)
        ops.paged_attention_generic(qs, kc.to(DEV), vc.to(DEV), plain, ctx.positions, ctx.seq_ids, table, H, G, hd, bs,
                                    scale, v_head_dim=hdv, sink=sink.to(DEV))
        ops.check_device_errors(DEV)
        for got in (out, plain):
            got = got.double().cpu().view(k_, H, hdv)
            assert float((got - want[lo:hi]).abs().max()) < tol, (lo, hi)
    # without the sink the rows are others (a forgotten sink would show)
    bare = torch.empty((T, H * hdv), dtype=dtype, device=DEV)
    ops.paged_attention_generic(q.reshape(T, -1).to(DEV), kc.to(DEV), vc.to(DEV), bare, i32(list(range(T))), i32([0] * T),
                                table, H, G, hd, bs, scale, v_head_dim=hdv)
    assert float((bare.double().cpu().view(T, H, hdv) - want).abs().max()) > 10 * tol
    # the first token sees one key: its row is that key's value times what the sink leaves
    s0 = (q[0].double() * k[0].double().repeat_interleave(H // G, 0)).sum(-1) * scale
    share = 1.0 / (1.0 + torch.exp(sink[:H].double() - s0))
    assert torch.allclose(want[0], v[0].double().repeat_interleave(H // G, 0) * share[:, None], atol=1e-9)


def _retention_weights(H, dk, dv, d, g):
    """Projections for the plain retention; the output projection is the identity, so its result is the
    gated, normed heads themselves."""
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    return {"m.q": rnd(H * dk, d) / math.sqrt(d), "m.k": rnd(H * dk, d) / math.sqrt(d), "m.v": rnd(H * dv, d) / math.sqrt(d),
            "m.g": rnd(H * dv, d) / math.sqrt(d), "m.o": torch.eye(H * dv, dtype=torch.float64)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv,rot", [(3, 8, 12, 4), (2, 48, 40, 48), (1, 16, 136, 0), (2, 128, 64, 64), (4, 32, 48, 16)])
def test_retention_kernel(dtype, H, dk, dv, rot):
    """Three requests of 37, 1 and 5 tokens in one launch, each in two calls (the state is carried in its
    slot), against the token-by-token recurrence; then a slot that was used is zeroed and used again."""
    from rllm_b200.csrc import ops
    d, eps, base = 24, 2e-5, 5000.0
    g = torch.Generator().manual_seed(4)
    W = _retention_weights(H, dk, dv, d, g)
    decay = [0.9, 0.999, 0.5, 0.97][:H]
    mx = {"heads": H, "dim": dk, "vdim": dv, "rot": {"dims": rot, "base": base}, "decay": decay}      # 0: nothing turns
    lens = [37, 1, 5]
    hs = [torch.randn(n, d, generator=g, dtype=torch.float64) for n in lens]
    want = [pd.retention(h, W, "m.", mx, eps) for h in hs]
    w_in = torch.cat([W["m.q"], W["m.k"], W["m.v"], W["m.g"]], 0).float().to(DEV)
    hk, hv = H * dk, H * dv
    state = torch.zeros((5, ops.retention_state_floats(H, dk, dv)), device=DEV)
    state[2].fill_(7.0)                                    # a slot the launch does not name stays as it is
    slots = torch.tensor([3, 0, 4], dtype=torch.int32, device=DEV)
    dec = torch.tensor(decay, dtype=torch.float64).float().to(DEV)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    got = [[] for _ in lens]
    at = [0, 0, 0]
    for part in ([20, 1, 2], [17, 0, 3]):
        live = [i for i, k in enumerate(part) if k]
        rows_h = torch.cat([hs[i][at[i]:at[i] + part[i]] for i in live])
        pos = torch.tensor([p for i in live for p in range(at[i], at[i] + part[i])], dtype=torch.int32, device=DEV)
        rows = (rows_h.float().to(DEV) @ w_in.T).contiguous()
        cu = torch.tensor([0] + list(torch.tensor([part[i] for i in live]).cumsum(0)), dtype=torch.int32, device=DEV)
        out = torch.empty((rows.shape[0], hv), dtype=dtype, device=DEV)
        cs = _angles_table(pos, rot, base) if rot else None
        ops.retention(rows, 0, hk, 2 * hk, 2 * hk + hv, cs, rot, False, dk ** -0.5, dec, eps, state, cu,
                      slots[live].contiguous(), out, len(live), H, dk, dv, gate="silu")
        o = 0
        for i in live:
            got[i].append(out[o:o + part[i]].double().cpu())
            o += part[i]
            at[i] += part[i]
    for i in range(3):
        assert float((torch.cat(got[i]) - want[i]).abs().max()) < tol * float(want[i].abs().max()), i
    assert float((state[2] - 7.0).abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0
    # the slot of the first request, zeroed as the cache manager does, runs the second request's token again
    state[3].zero_()
    rows = (hs[1].float().to(DEV) @ w_in.T).contiguous()
    out = torch.empty((1, hv), dtype=dtype, device=DEV)
    cs = _angles_table(torch.zeros(1, dtype=torch.int32, device=DEV), rot, base) if rot else None
    ops.retention(rows, 0, hk, 2 * hk, 2 * hk + hv, cs, rot, False, dk ** -0.5, dec, eps, state,
                  torch.tensor([0, 1], dtype=torch.int32, device=DEV), slots[:1].contiguous(), out, 1, H, dk, dv)
    assert float((out.double().cpu() - got[1][0]).abs().max()) < tol * float(got[1][0].abs().max())


@pytest.mark.parametrize("E,top,count,keep", [(16, 4, 2, 1), (12, 4, 3, 2), (6, 2, 6, 3), (5, 1, 1, 1), (64, 6, 8, 3)])
def test_router_kernel(E, top, count, keep):
    """The choice inside the best groups by corrected scores (some negative), the weights from the
    uncorrected ones: the same experts and weights as the plain router, token by token."""
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    n, d = 40, 16
    W = {"r.router": torch.randn(E, d, generator=g, dtype=torch.float64), "r.correction": -1.2 + 0.5 * torch.randn(E, generator=g, dtype=torch.float64)}
    h = torch.randn(n, d, generator=g, dtype=torch.float64)
    r = {"experts": E, "top": top, "scale": 1.7, "groups": {"count": count, "keep": keep}}
    logits = (h @ W["r.router"].T).float().to(DEV)
    logits = torch.cat([logits, torch.zeros(n, 2, device=DEV)], 1)[:, :E + 1]          # a column more, as with a shared gate
    idx = torch.empty((n, top), dtype=torch.int32, device=DEV)
    wt = torch.empty((n, top), dtype=torch.float32, device=DEV)
    ops.moe_route(logits, W["r.correction"].float().to(DEV), idx, wt, E, top, count, keep, 2, "sigmoid", True, 1e-20, 1.7)
    negative = 0
    for t in range(n):
        chosen, w = pd.route(h[t], W, "r.", r)
        negative += int((torch.sigmoid(W["r.router"] @ h[t]) + W["r.correction"])[chosen].min() < 0)
        got = dict(zip(idx[t].tolist(), wt[t].tolist()))
        assert sorted(got) == sorted(chosen), t
        for e, x in zip(chosen, w.tolist()):
            assert abs(got[e] - x) < 1e-5
    assert negative > 0                                    # zeros in place of minus infinity would have shown


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", [1, 9, 37, 150])
def test_routed_experts_part(dtype, n):
    """The feed-forward part alone, on few rows (every pair against its expert's matrices) and on many
    (pairs sorted by expert, each expert's rows through the products): against the plain sum."""
    from rllm_b200.models.model import parse_dtype
    from rllm_b200.parts import Runtime
    from rllm_b200.config.base import PartSpec
    from rllm_b200.parts.base import build_part
    g = torch.Generator().manual_seed(6)
    d, F, E, S = 40, 24, 12, 16
    mlp = dc.moe(F, E, 3, count=3, keep=2, scale=1.3, shared=S)
    cfg = dc.config([dc.ret(1, 8, 8, 2, [0.9], mlp=mlp)], width=d, vocab=11)
    W = {k[len("l0.mlp."):]: v for k, v in dc.make_weights(cfg, 7, stored(dtype)).items() if k.startswith("l0.mlp.")}
    part = build_part("ffn", PartSpec("routed_experts", {
        "hidden_size": d, "intermediate_size": F, "num_experts": E, "top_k": 3, "n_groups": 3, "keep_groups": 2,
        "group_best": 2, "score": "sigmoid", "correction": True, "normalize": True, "weight_eps": 1e-20,
        "route_scale": 1.3, "shared_size": S, "shared_gate": True}, "x."), Runtime(torch.device(DEV), parse_dtype(dtype)))
    part.load({"x." + k: v for k, v in W.items()})
    h = torch.randn(n, d, generator=g).to(stored(dtype))
    want = pd.moe_ff(h.double(), {"m." + k: v.double() for k, v in W.items()}, "m.", mlp)
    got = part.forward(h.to(DEV), None).double().cpu()
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert float((got - want).abs().max()) < tol * float(want.abs().max())


# ---------------------------------------------------------------- each configuration, each way of cutting

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_whole_prompt(name, dtype):
    cfg = CASES[name]
    w = dc.make_weights(cfg, 3, stored(dtype))
    toks = dc.tokens_for(cfg, 45, 1)
    ref = dc.oracle(cfg, w, toks)
    eng = dc.build_engine(cfg, w, dtype, max_tokens=64)
    out = run(eng, [([("a", toks, list(range(len(toks))))], ["a"])])
    compare(out, {"a": ref}, dtype, f"{name} whole")


def test_stream_after_every_layer():
    """The residual stream itself, layer by layer, in float32."""
    cfg = CASES["stack"]
    w = dc.make_weights(cfg, 8)
    toks = dc.tokens_for(cfg, 21, 9)
    want = []
    dc.oracle(cfg, w, toks, want)
    eng = dc.build_engine(cfg, w, "float32", max_tokens=32)
    seen = []
    for block in eng.model.blocks:
        inner = block.forward

        def spy(x, pending, ctx, cache, _inner=inner, **kw):
            out = _inner(x, pending, ctx, cache)          # without `next_entry`: the stream is complete on return
            seen.append(x.detach().double().cpu().clone())
            return out
        block.forward = spy
    run(eng, [([("a", toks, [20])], ["a"])])
    assert len(seen) == len(want) == 5
    for got, ref in zip(seen, want):
        assert float((got - ref).abs().max()) < 2e-5 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_token_by_token_and_portions(name, dtype):
    """The same prompt decoded one token a step from the first token on, and in portions of 2, 3, 2,
    17, 5, 2, 2, ... tokens: every row as the plain implementation has it from the whole sequence."""
    cfg = CASES[name]
    w = dc.make_weights(cfg, 4, stored(dtype))
    toks = dc.tokens_for(cfg, 52, 2)
    ref = {"a": dc.oracle(cfg, w, toks)}
    eng = dc.build_engine(cfg, w, dtype, max_tokens=128)
    compare(run(eng, closing(one_by_one("a", toks), "a")), ref, dtype, f"{name} one by one")
    steps = [([("a", p, want)], []) for p, want in cut(toks, [2, 3, 2, 17, 5, 2, 2, 9, 1, 1, 2])]
    compare(run(eng, closing(steps, "a")), ref, dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["stack", "stack_attention_first", "shared_keys", "moe_groups", "heads64", "heads128"])
def test_unequal_requests_in_one_batch_with_reuse(name, dtype):
    """Four requests of 61, 9, 33 and 2 tokens come and go in a pool of two request slots and few
    pages: portions of some beside single tokens of others; the pages and the state slot that a
    finished request gave back go to the next one.  Every row equals the request alone."""
    cfg = CASES[name]
    w = dc.make_weights(cfg, 5, stored(dtype))
    lens = {"a": 61, "b": 9, "c": 33, "d": 2}
    toks = {r: dc.tokens_for(cfg, n, 10 + i) for i, (r, n) in enumerate(lens.items())}
    refs = {r: dc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = dc.build_engine(cfg, w, dtype, max_tokens=96, block_size=8, max_requests=2)
    at = {r: 0 for r in toks}
    plan = [[("a", 7), ("b", 2)], [("a", 1), ("b", 5)], [("a", 16), ("b", 1)], [("a", 1), ("b", 1)],      # b ends
            [("a", 3), ("c", 9)], [("a", 1), ("c", 1)], [("a", 2), ("c", 17)], [("a", 30), ("c", 1)],     # a ends
            [("c", 1), ("d", 2)],                                                                         # d ends
            [("c", 4)]]
    steps = []
    for st in plan:
        entries = []
        for r, k in st:
            lo = at[r]
            at[r] = lo + k
            entries.append((r, toks[r][lo:lo + k], list(range(k))))
        steps.append((entries, [r for r, _ in st if at[r] == len(toks[r])]))
    assert all(at[r] == len(toks[r]) for r in toks)
    compare(run(eng, steps), refs, dtype, f"{name} mixed")
    eng.cache.check_invariants()
    assert not eng.cache.requests


def test_pages_and_slots_used_again_give_the_same_bits():
    """A request that runs on the pages and in the state slot another request just left has the bits it
    has in a fresh engine; a request that pauses for a step while another runs loses nothing."""
    cfg = CASES["stack"]
    w = dc.make_weights(cfg, 6)
    a, b = dc.tokens_for(cfg, 40, 20), dc.tokens_for(cfg, 37, 21)
    sched = [([("b", b[:20], [19])], []), ([("b", b[20:], list(range(17)))], ["b"])]
    fresh = run(dc.build_engine(cfg, w, "float32", max_tokens=48, max_requests=1), sched)
    eng = dc.build_engine(cfg, w, "float32", max_tokens=48, max_requests=1)
    run(eng, [([("a", a, [39])], ["a"])])
    again = run(eng, sched)
    for key, row in fresh.items():
        assert torch.equal(row, again[key]), key
    eng = dc.build_engine(cfg, w, "float32", max_tokens=96, max_requests=2)
    paused = run(eng, [([("b", b[:20], [19])], []), ([("a", a, [39])], ["a"]), ([("b", b[20:], list(range(17)))], ["b"])])
    for key, row in fresh.items():
        assert row_error(paused[key], row) < 1e-6, key


# ---------------------------------------------------------------- far keys, page borders, sinks, the first tokens

ASK, TARGET = 5, 6         # the asking token's queries are turned towards the target token's keys


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads", ["small", "64"])
def test_a_far_key_among_hundreds(dtype, heads):
    """Sharp attention: askers at places 300 to 429 hang on one target key at place 3 (its page is the
    first of fourteen; pages of 32), others on targets at the last place of a page and the first of the
    next, in a long portion, in short ones and decoded alone; a second layer reads the same keys.
    First a test of the test: without the target, and without the sinks, the askers' rows are others."""
    if heads == "small":
        layers = [dc.att(4, 2, 32, 20, 8, scale=1.5, mlp=dc.dense(30)), dc.ret(2, 8, 16, 8, [0.9, 0.99]),
                  dc.att(4, 2, 32, 20, 8, scale=0.15, kv_from=0)]
    else:
        layers = [dc.att(6, 2, 64, 64, 16, scale=1.0, mlp=dc.dense(30)), dc.att(6, 2, 64, 64, 16, scale=0.1, kv_from=0)]
    cfg = dc.config(layers, width=40, vocab=73)
    w = dc.marked_attention(cfg, dc.make_weights(cfg, 9, stored(dtype)), ASK, TARGET)
    last = f"l{len(layers) - 1}.mix.sink"
    w[last] = w[last] + 5.0                               # the last layer's rows are soft, and its sinks take a large share
    toks = dc.tokens_for(cfg, 430, 4, avoid=(ASK, TARGET))
    askers = [300, 333, 352, 383, 384, 401, 419, 420, 429]
    toks[3] = TARGET
    for a in askers:
        toks[a] = ASK
    ref = dc.oracle(cfg, w, toks)
    blind = dc.oracle(cfg, w, [7 if t == TARGET else t for t in toks])
    assert all(row_error(blind[a], ref[a]) > 3 * TOL[dtype] for a in askers)
    no_sink = dict(w)
    for i in (0, len(layers) - 1):
        no_sink[f"l{i}.mix.sink"] = torch.full_like(w[f"l{i}.mix.sink"], -30.0)
    bare = dc.oracle(cfg, no_sink, toks)
    assert sum(row_error(bare[p], ref[p]) > 3 * TOL[dtype] for p in range(len(toks))) > 30
    eng = dc.build_engine(cfg, w, dtype, max_tokens=448, block_size=32)
    steps = [([("a", toks[:340], [0, 1, 2, 3, 4, 31, 32, 33, 300, 333, 339])], []), ([("a", toks[340:353], [12])], []),
             ([("a", toks[353:355], [0, 1])], []), ([("a", toks[355:400], [28, 29])], [])]
    steps += one_by_one("a", toks, 400)
    compare(run(eng, closing(steps, "a")), {"a": ref}, dtype, "far key")
    # targets at a page's last place and the next page's first, askers a few places on and a page on
    toks2 = dc.tokens_for(cfg, 140, 5, avoid=(ASK, TARGET))
    for t, a in ((31, 33), (64, 66), (95, 130), (96, 97)):
        toks2[t], toks2[a] = TARGET, ASK
    ref2 = dc.oracle(cfg, w, toks2)
    steps = [([("b", toks2[:30], list(range(30)))], []), ([("b", toks2[30:34], [0, 1, 2, 3])], []),
             ([("b", toks2[34:96], list(range(62)))], [])] + one_by_one("b", toks2, 96)
    compare(run(eng, closing(steps, "b")), {"b": ref2}, dtype, "page borders")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens(dtype):
    """Requests of one, two and three tokens, alone and side by side: a first token sees one key and the
    sink, a retention state starts from zero."""
    cfg = CASES["stack"]
    w = dc.make_weights(cfg, 12, stored(dtype))
    toks = {r: dc.tokens_for(cfg, n, 50 + n) for r, n in (("a", 1), ("b", 2), ("c", 3))}
    refs = {r: dc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = dc.build_engine(cfg, w, dtype, max_tokens=64, max_requests=3)
    together = run(eng, [([(r, t, list(range(len(t)))) for r, t in toks.items()], list(toks))])
    compare(together, refs, dtype, "first tokens, one batch")
    for r, t in toks.items():
        compare(run(eng, closing(one_by_one(r, t), r)), refs, dtype, "first tokens, alone")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions(dtype):
    """Portions of 300 and 700 tokens (the retention kernel cuts them along time and joins the segments'
    states; the routed experts take their rows sorted by expert) beside a short request, then single
    tokens: rows near the cuts and at the end against the plain implementation, whose state after a
    thousand tokens is the decayed sum of all of them."""
    cfg = CASES["stack"]
    w = dc.make_weights(cfg, 13, stored(dtype))
    toks = {"a": dc.tokens_for(cfg, 1010, 60), "b": dc.tokens_for(cfg, 12, 61)}
    refs = {r: dc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = dc.build_engine(cfg, w, dtype, max_tokens=1088, block_size=16, max_requests=2)
    want = [0, 1, 127, 128, 129, 255, 256, 299]
    steps = [([("a", toks["a"][:300], want), ("b", toks["b"][:7], [6])], []),
             ([("b", toks["b"][7:8], [0]), ("a", toks["a"][300:1000], [0, 99, 100, 355, 356, 699])], [])]
    steps += [([("a", [toks["a"][1000 + i]], [0]), ("b", [toks["b"][8 + i]], [0])], []) for i in range(4)]
    steps += one_by_one("a", toks["a"], 1004)
    compare(run(eng, steps), refs, dtype, "long portions")


def test_long_portion_through_the_largest_retention_heads():
    """Value heads of 256 entries under keys of 128 (the retention kernel's largest blocks) in a portion
    long enough to be cut along time, then single tokens."""
    cfg = CASES["retention_256_values"]
    w = dc.make_weights(cfg, 14)
    toks = dc.tokens_for(cfg, 610, 62)
    ref = {"a": dc.oracle(cfg, w, toks)}
    eng = dc.build_engine(cfg, w, "float32", max_tokens=640, block_size=32, max_requests=1)
    steps = [([("a", toks[:600], [0, 127, 128, 300, 599])], [])] + one_by_one("a", toks, 600)
    compare(run(eng, steps), ref, "float32", "largest retention heads")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graph_replay(dtype):
    """200 single-token steps of three requests behind short prompts (graphs captured per context
    bucket, padded to a power of two of requests), every tenth row against the plain implementation;
    the replayed steps give what eager steps give."""
    cfg = CASES["stack"]
    w = dc.make_weights(cfg, 10, stored(dtype))
    reqs = {"a": dc.tokens_for(cfg, 215, 30), "b": dc.tokens_for(cfg, 203, 31), "c": dc.tokens_for(cfg, 206, 32)}
    refs = {r: dc.oracle(cfg, w, t) for r, t in reqs.items()}
    outs = []
    for graphs in (True, False):
        eng = dc.build_engine(cfg, w, dtype, max_tokens=768, block_size=16, use_graphs=graphs)
        steps = [([("a", reqs["a"][:15], [14]), ("b", reqs["b"][:3], [2]), ("c", reqs["c"][:6], [5])], [])]
        for i in range(200):
            steps.append(([(r, [t[len(t) - 200 + i]], [0] if i % 10 == 9 else []) for r, t in reqs.items()], []))
        outs.append(run(eng, steps))
        if graphs:
            assert eng.stats["graph_replays"] > 150
    outs[0].chosen = outs[1].chosen                        # a replayed step runs the kernels of an eager one
    compare(outs[0], refs, dtype, "long decoding, replayed")
    compare(outs[1], refs, dtype, "long decoding, eager")
    if dtype == "float32":
        for key, row in outs[0].items():
            assert row_error(row, outs[1][key]) < 1e-6, key


REAL = dc.config([dc.ret(8, 64, 128, 64, [1 - 2.0 ** -(3 + i) for i in range(8)], mlp=dc.dense(1536, 7.0)),
                  dc.att(8, 2, 128, 128, 64, mlp=dc.moe(256, 32, 4, count=4, keep=2, scale=2.0, shared=512)),
                  dc.att(8, 2, 128, 128, 64, kv_from=1, mlp=dc.dense(1024, 7.0)),
                  dc.att(16, 4, 64, 64, 64, mlp=dc.moe(384, 8, 2, scale=1.0))], width=1024, vocab=1531, logit_scale=0.5)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_layer_sizes_of_a_real_model(dtype):
    """Width 1,024 and layers of real sizes (retention heads of 64 x 128, attention heads of 128 and 64,
    32 experts): the products take the library, the tcgen05 and the weight-streaming kernels, attention the
    tensor-core kernels.  A prompt of 300 tokens, a portion of 40 beside another request's 20, then
    single tokens of both."""
    cfg = REAL
    w = dc.make_weights(cfg, 16, stored(dtype), gain=1.0)
    toks = {"a": dc.tokens_for(cfg, 352, 70), "b": dc.tokens_for(cfg, 32, 71)}
    refs = {r: dc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = dc.build_engine(cfg, w, dtype, max_tokens=512, block_size=32, max_requests=2)
    steps = [([("a", toks["a"][:300], list(range(0, 300, 23)) + [99, 100, 159, 160, 299])], []),
             ([("a", toks["a"][300:340], list(range(40))), ("b", toks["b"][:20], [0, 19])], [])]
    steps += [([("a", [toks["a"][340 + i]], [0]), ("b", [toks["b"][20 + i]], [0])], []) for i in range(12)]
    compare(run(eng, steps), refs, dtype, "real layer sizes")


# ---------------------------------------------------------------- the entry points a user calls

def write_folder(path, cfg, w):
    from rllm_b200.weights.safetensors_io import write_safetensors
    path.mkdir(exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", w)
    return path


def test_greedy_generation_through_the_scheduler(tmp_path):
    """LLM.generate (scheduler, continuous batching, prompts cut into portions of 16, device sampler)
    on a folder written in the stored format: the greedy continuation of each prompt is the plain
    implementation's."""
    from rllm_b200.llm import LLM
    cfg = CASES["stack"]
    w = dc.make_weights(cfg, 11)
    write_folder(tmp_path, cfg, w)
    prompts = [dc.tokens_for(cfg, n, 40 + i) for i, n in enumerate((37, 3, 21, 50, 9))]
    llm16 = LLM(str(tmp_path), dtype="bfloat16", ctx=128, block_size=8, prefill_chunk=16, parallel=3)
    got16 = llm16.generate(prompts, max_tokens=12, temperature=0.7, top_k=20, seed=5)
    assert all(len(g) == 12 and all(0 <= t < cfg["vocab"] for t in g) for g in got16)
    assert not llm16.engine.cache.requests
    del llm16
    llm = LLM(str(tmp_path), dtype="float32", ctx=128, block_size=8, prefill_chunk=16, parallel=3)
    got = llm.generate(prompts, max_tokens=12)
    checked = 0
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            logits = dc.oracle(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 1e-4:       # a tie at float32 precision decides nothing
                break
            assert int(logits.argmax()) == tok
            seq.append(tok)
            checked += 1
    assert all(len(g) == 12 for g in got) and checked > 40
    assert not llm.engine.cache.requests


def test_trace_replay_program_chooses_the_model_by_its_config(tmp_path):
    """bin/trace_run on a Divuzen folder: steps from standard input, rows out as little-endian float32; two
    requests share the steps, one pauses, pages and slots go back at the end."""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    cfg = CASES["stack_attention_first"]
    w = dc.make_weights(cfg, 12, torch.bfloat16)
    model = write_folder(tmp_path / "model", cfg, w)
    toks, other = dc.tokens_for(cfg, 30, 6), dc.tokens_for(cfg, 9, 7)
    lines = [json.dumps({"step": 0, "entries": [{"id": "x", "tokens": toks[:20], "want": [0, 19]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "y", "tokens": other[:8], "want": []}], "end": []}),
             json.dumps({"step": 2, "entries": [{"id": "x", "tokens": toks[20:], "want": [9]},
                                                {"id": "y", "tokens": other[8:], "want": [0]}], "end": ["x", "y"]})]
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model), "--dtype", "float32",
                           "--out", str(tmp_path / "out"), "--max-tokens", "128"], input="\n".join(lines) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    rows = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    ref, ref_other = dc.oracle(cfg, w, toks), dc.oracle(cfg, w, other)
    assert row_error(rows[0], ref[0]) < TOL["float32"] and row_error(rows[1], ref[19]) < TOL["float32"]
    assert not (tmp_path / "out" / "1.f32").exists()
    rows = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    assert row_error(rows[0], ref[29]) < TOL["float32"] and row_error(rows[1], ref_other[8]) < TOL["float32"]


def test_random_weights_mode_writes_a_folder_the_engine_loads(tmp_path):
    """The package's own random-weights mode knows the design's tensors."""
    from rllm_b200.config import config_from_dict
    from rllm_b200.models.model import load_model
    from rllm_b200.weights import write_random_model
    write_random_model(config_from_dict(CASES["stack"]), tmp_path, seed=3, dtype=torch.bfloat16)
    cfg, model = load_model(tmp_path, "bfloat16", DEV)
    assert cfg.to_dict() == CASES["stack"] and model.loaded
    from rllm_b200.engine import Engine, StepItem
    eng = Engine(model, block_size=16, max_tokens=64, max_requests=2)
    logits = eng.step([StepItem("a", [1, 2, 3, 4, 5], [4])])
    assert logits.shape == (1, CASES["stack"]["vocab"]) and bool(torch.isfinite(logits).all())
