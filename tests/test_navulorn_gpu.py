"""Navulorn through the engine against the plain implementation (tests/plain_navulorn.py, float64).

Each new kernel alone against its formula; each mechanism as a one-layer model; whole prompts against
token-by-token decoding; portions down to two tokens; batches of unequal requests against each alone with
pages and state slots used again; keys just inside and just outside every window, in prompts and in
decoding, with weights at which one key decides a row and a check that a window that is one key off
would show; the first tokens of a sequence; long portions that the matrix-memory kernel cuts along time;
long decoding through CUDA-graph replay; head sizes the tensor-core kernels take; layer sizes of a real
model; greedy generation through ``LLM.generate`` and the scheduler; ``bin/trace_run``; the random-weights
mode.  The configurations and weights are made in tests/navulorn_cases.py.
"""
import json
import math

import pytest
import torch

import navulorn_cases as nc
import plain_navulorn as pn
from navulorn_cases import CASES, row_error

pytestmark = pytest.mark.gpu

# max |engine - plain| / max |plain| over a logits row (means taken off).  float32: the engine sums in
# another order than the float64 plain implementation.  bfloat16: weights, the operands of every product
# and the cache are rounded to 8 bits of mantissa (a key lost at a window's edge moves rows by 0.1 to 1).
# How much rounding alone moves a row differs from row to row (a head of the matrix memory is divided by its
# root mean square, and where its sum nearly cancels the rounding of the terms is amplified; a small alpha
# lets a sublayer's rounding through to the stream): in bfloat16 a row's tolerance is this one plus three
# times what rounding the sublayers' inputs and outputs does to the row in the plain implementation
# (`oracle(...).noise`), and one row in fifty may pass it by less than a factor of two.  A lost key, state or
# token moves many rows, by more; the float32 runs of the same tests see it at 1e-4.
TOL = {"float32": 1e-4, "bfloat16": 7e-2}
STRAY = {"float32": 0, "bfloat16": 50}
# A token whose choice of experts hangs on less than this gap between router logits may take another
# expert when the router's input carries the rounding of the mode.  The comparison looks at which experts
# the engine chose: where the plain router's choice hangs on less than this, it takes the engine's experts
# over if they are what it gives itself after moving every logit by at most this much.
CLOSE = {"float32": 1e-4, "bfloat16": 0.15}
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
    bad, stray = [], 0
    for (r, p), row in sorted(out.items()):
        e = row_error(row, refs[r][p])
        noise = getattr(refs[r], "noise", None)
        tol_row = tol + (3 * noise[p] if noise is not None and dtype == "bfloat16" else 0.0)
        if not e <= tol_row:
            if e <= 2 * tol_row and STRAY[dtype] and stray < max(1, len(out) // STRAY[dtype]):
                stray += 1
                continue
            bad.append(f"request {r} position {p}: error {e:.3e} > {tol_row:.3e}")
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


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def step_context(lens, starts):
    """A StepContext of requests that bring `lens` tokens from positions `starts`."""
    from rllm_b200.engine.batch import StepContext
    n = sum(lens)
    cu = [0]
    for k in lens:
        cu.append(cu[-1] + k)
    pos = [s + j for k, s in zip(lens, starts) for j in range(k)]
    seq = [r for r, k in enumerate(lens) for _ in range(k)]
    ends = [s + k for k, s in zip(lens, starts)]
    return StepContext(n_tokens=n, n_requests=len(lens), tokens=i32([0] * n), positions=i32(pos), seq_ids=i32(seq),
                       cu_q=i32(cu), ctx_lens=i32(ends), logit_rows=None, q_lens=list(lens), start_pos=list(starts),
                       ctx_lens_host=ends, max_q_len=max(lens), max_ctx_len=max(ends))


def angles_table(positions, freqs):
    from rllm_b200.csrc import ops
    return ops.rope_table(positions, freqs.float().to(DEV))


# ---------------------------------------------------------------- each kernel alone

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,alpha", [(50, 3.0), (1300, 1.0), (8, 0.25)])
def test_norm_behind_the_sum_kernel(dtype, d, alpha):
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    y = (3 * torch.randn(9, d + 20, generator=g)).to(dtype).to(DEV)
    x = torch.randn(9, d, generator=g).to(DEV)
    w = (1 + 0.3 * torch.randn(d, generator=g)).to(DEV)
    low = torch.empty((9, d), dtype=dtype, device=DEV)
    want = pn.rms_norm(alpha * x.double() + y[:, 5:5 + d].double(), w.double(), 2e-6)
    ops.sum_norm_rows(x, y[:, 5:5 + d], alpha, w, 2e-6, low=low)
    assert torch.allclose(x.double(), want, atol=1e-5)
    assert torch.allclose(low.double(), want, atol=1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding_kernel_and_the_kept_last_token(dtype):
    """Three requests in two steps: the first row a request brings in the second step takes its previous
    token from the slot; a request's first token takes the table's last row; a slot used again starts anew."""
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    V, d, B, mp, mc, scale = 23, 12, 7, 5, 3, 2.5
    table, pair = torch.randn(V, d, generator=g).to(dtype), torch.randn(B + 1, d, generator=g).to(dtype)
    seqs = [[3, 20, 7, 7, 1, 22, 9], [5], [11, 0, 0, 4]]
    want = [pn.embed(s, table.double(), pair.double(), scale, B, mp, mc) for s in seqs]
    last = torch.full((5,), 99, dtype=torch.int32, device=DEV)          # a stale id that must never be read as is
    slots = i32([3, 0, 4])
    got = [[] for _ in seqs]
    at = [0, 0, 0]
    for part in ([4, 1, 1], [3, 0, 3]):
        live = [r for r, k in enumerate(part) if k]
        ctx = step_context([part[r] for r in live], [at[r] for r in live])
        toks = i32([t for r in live for t in seqs[r][at[r]:at[r] + part[r]]])
        out = torch.empty((toks.numel(), d), device=DEV)
        sl = slots[live].contiguous()
        ops.embed_pair(table.to(DEV), pair.to(DEV), toks, ctx.positions, ctx.seq_ids, ctx.cu_q, sl, last, out, scale, B,
                       mp, mc, ops.error_word(DEV))
        ops.keep_last_tokens(toks, ctx.cu_q, sl, last, len(live))
        o = 0
        for r in live:
            got[r].append(out[o:o + part[r]].double().cpu())
            o += part[r]
            at[r] += part[r]
    ops.check_device_errors(DEV)
    for r in range(3):
        assert torch.allclose(torch.cat(got[r]), want[r], atol=1e-6), r
    assert last.tolist() == [5, 99, 99, 9, 4]


@pytest.mark.parametrize("pairs,rot,H,G,dk,dv", [(False, 6, 5, 1, 10, 14), (True, 12, 4, 2, 12, 4), (False, 16, 2, 2, 16, 16),
                                                 (False, 0, 3, 1, 6, 6)])
def test_row_norm_rotation_store_kernel(pairs, rot, H, G, dk, dv):
    """Norm over the whole query row and the whole key row, then the rotation of each head's first entries."""
    from rllm_b200.csrc import ops
    bs, n, eps = 4, 7, 3e-5
    g = torch.Generator().manual_seed(3)
    width = H * dk + G * (dk + dv)
    rows = torch.randn(n, width + 3, generator=g).to(DEV)
    qw, kw = (1 + 0.3 * torch.randn(H * dk, generator=g)).to(DEV), (1 + 0.3 * torch.randn(G * dk, generator=g)).to(DEV)
    pos = [0, 1, 2, 40, 41, 300, 7]
    slots = i32([3, 0, 5, -1, 9, 11, 6])
    freqs = pn.frequencies(rot, 300.0) if rot else None
    cs = angles_table(i32(pos), freqs) if rot else None
    q = torch.empty((n, H * dk), device=DEV)
    kc, vc = torch.zeros((3, G, bs, dk), device=DEV), torch.zeros((3, G, bs, dv), device=DEV)
    ops.qkv_rownorm_store(rows[:, :width], None, qw, kw, slots, q, kc, vc, H, G, dk, dv, bs, eps, cs_table=cs, rot=rot,
                          pairs=pairs)
    ops.check_device_errors(DEV)
    r64 = rows.double().cpu()
    layout = "pairs" if pairs else "half"
    want_q = pn.rms_norm(r64[:, :H * dk], qw.double().cpu(), eps).view(n, H, dk)
    want_k = pn.rms_norm(r64[:, H * dk:(H + G) * dk], kw.double().cpu(), eps).view(n, G, dk)
    if rot:
        want_q = pn.rotate(want_q, torch.tensor(pos), freqs, rot, layout)
        want_k = pn.rotate(want_k, torch.tensor(pos), freqs, rot, layout)
    assert torch.allclose(q.double().cpu().view(n, H, dk), want_q, atol=3e-5)
    want_v = rows[:, (H + G) * dk:width].cpu().view(n, G, dv)
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        assert torch.allclose(kc[s // bs, :, s % bs].double().cpu(), want_k[t], atol=3e-5)
        assert torch.equal(vc[s // bs, :, s % bs].cpu(), want_v[t])
    assert float(kc[0, :, 1].abs().max()) == 0.0 and float(vc[0, :, 2].abs().max()) == 0.0     # slots nobody named


def test_one_gate_per_head_kernel():
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    a, gate = torch.randn(6, 3 * 5, generator=g).to(DEV), torch.randn(6, 3 + 2, generator=g).to(DEV)
    out = torch.empty_like(a)
    ops.rows_act(a, out, mul=gate[:, 1:4], mul_act="sigmoid", mul_group=5)
    want = a.double().view(6, 3, 5) * torch.sigmoid(gate[:, 1:4].double())[:, :, None]
    assert torch.allclose(out.double().view(6, 3, 5), want, atol=1e-6)


@pytest.mark.parametrize("pairs", [False, True])
def test_latent_store_kernel_in_both_layouts(pairs):
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(5)
    n, H, dq, r, rank, bs, eps = 5, 3, 6, 8, 10, 4, 1e-5
    q = torch.randn(n, H * (dq + r), generator=g).to(DEV)
    kv = torch.randn(n, rank + r + 2, generator=g).to(DEV)
    wn = (1 + 0.3 * torch.randn(rank, generator=g)).to(DEV)
    pos = [0, 3, 4, 90, 91]
    freqs = pn.frequencies(r, 700.0)
    cs = angles_table(i32(pos), freqs)
    q_att = torch.zeros((n, H * (rank + r)), device=DEV)
    cache = torch.zeros((3, 1, bs, rank + r), device=DEV)
    slots = i32([2, 7, -1, 11, 0])
    ops.latent_rope_store(q, kv[:, :rank + r], wn, cs, 1.0, slots, q_att, cache, H, dq, r, rank, bs, eps, pairs=pairs)
    layout = "pairs" if pairs else "half"
    want_q = pn.rotate(q.double().cpu().view(n, H, dq + r)[..., dq:].contiguous(), torch.tensor(pos), freqs, r, layout)
    assert torch.allclose(q_att.double().cpu().view(n, H, rank + r)[..., rank:], want_q, atol=2e-5)
    c = pn.rms_norm(kv[:, :rank].double().cpu(), wn.double().cpu(), eps)
    kr = pn.rotate(kv[:, rank:rank + r].double().cpu().view(n, 1, r), torch.tensor(pos), freqs, r, layout)[:, 0]
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            assert torch.allclose(cache.view(-1, rank + r)[s].double().cpu(), torch.cat([c[t], kr[t]]), atol=2e-5)


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
@pytest.mark.parametrize("H,W,V,window", [(3, 24, 16, 7), (5, 80, 64, 37), (2, 144, 128, 150), (4, 72, 64, 1), (2, 20, 12, 0)])
def test_shared_key_attention_with_a_window(dtype, H, W, V, window):
    """Attention of H heads over one shared key/value head whose values lie in the key rows, with a window:
    a whole prompt (the library products), a portion, few tokens and single tokens (the tensor-core decode
    kernel where the sizes allow it, else the plain kernel) against the formula; with the window one key
    longer the rows are others."""
    from rllm_b200.csrc import ops
    bs, T, scale = 8, 203, 1.2 / math.sqrt(W)
    g = torch.Generator().manual_seed(6)
    c = torch.randn(T, 1, W, generator=g).to(dtype)
    q = (2 * torch.randn(T, H, W, generator=g)).to(dtype)
    cache, pages = _paged(c, bs, 31, g)

    def formula(win):
        out = torch.zeros(T, H, V, dtype=torch.float64)
        for i in range(T):
            lo = max(0, i - win + 1) if win else 0
            s = (q[i].double() @ c[lo:i + 1, 0].double().T) * scale
            out[i] = torch.softmax(s, -1) @ c[lo:i + 1, 0, :V].double()
        return out
    want = formula(window)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    table = pages.view(1, -1).to(DEV)
    for lo, hi in ((0, T), (90, T), (T - 1, T), (0, 1), (T - 5, T), (60, 61)):
        k_ = hi - lo
        ctx = step_context([k_], [lo])
        out = torch.empty((k_, H * V), dtype=dtype, device=DEV)
        ops.shared_kv_attention(q[lo:hi].reshape(k_, -1).to(DEV), cache.to(DEV), out, ctx, table, H, W, V, bs, scale,
                                window=window)
        ops.check_device_errors(DEV)
        assert float((out.double().cpu().view(k_, H, V) - want[lo:hi]).abs().max()) < tol, (lo, hi)
    if window and window < T:
        assert float((formula(window + 1) - want).abs().max()) > 10 * tol


def _memory_weights(H, dk, dv, d, g):
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    return {"m.q": rnd(H * dk, d) / math.sqrt(d), "m.k": rnd(H * dk, d) / math.sqrt(d), "m.v": rnd(H * dv, d) / math.sqrt(d),
            "m.g": rnd(H * dv, d) / math.sqrt(d), "m.o": torch.eye(H * dv, dtype=torch.float64),
            "m.norm": 1 + 0.2 * rnd(H * dv), "m.i": 3 * rnd(H, d) / math.sqrt(d), "m.f": 3 * rnd(H, d) / math.sqrt(d),
            "m.i.b": rnd(H), "m.f.b": 2 + rnd(H)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv,cap", [(3, 8, 12, 8.0), (2, 48, 40, 15.0), (1, 16, 136, 3.0), (2, 128, 64, 6.0), (1, 200, 254, 9.0),
                                         (4, 33, 1, 2.0), (1, 16, 300, 5.0), (2, 260, 20, 7.0)])      # the last two: the plain kernel
def test_matrix_memory_kernel(dtype, H, dk, dv, cap):
    """Three requests of 37, 1 and 5 tokens in one launch, each in two calls (the state is carried in its
    slot), against the token-by-token recurrence; then a slot that was used is zeroed and used again."""
    from rllm_b200.csrc import ops
    d, eps = 24, 2e-5
    g = torch.Generator().manual_seed(7)
    W = _memory_weights(H, dk, dv, d, g)
    mx = {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}
    lens = [37, 1, 5]
    hs = [torch.randn(n, d, generator=g, dtype=torch.float64) for n in lens]
    want = [pn.mlstm(h, W, "m.", mx, eps) for h in hs]
    w_in = torch.cat([W["m.q"], W["m.k"], W["m.v"], W["m.g"], W["m.i"], W["m.f"]], 0).float().to(DEV)
    hk, hv = H * dk, H * dv
    state = torch.zeros((5, ops.mlstm_state_floats(H, dk, dv)), device=DEV)
    state[2].fill_(7.0)                                    # a slot the launch does not name stays as it is
    slots = i32([3, 0, 4])
    ib, fb, nw = (W[k].float().to(DEV) for k in ("m.i.b", "m.f.b", "m.norm"))
    tol = 5e-5 if dtype == torch.float32 else 2e-2

    def launch(rows_h, cu, sl, n_req):
        rows = (rows_h.float().to(DEV) @ w_in.T).contiguous()
        out = torch.empty((rows.shape[0], hv), dtype=dtype, device=DEV)
        ops.mlstm(rows, 0, hk, 2 * hk, 2 * hk + hv, 2 * hk + 2 * hv, 2 * hk + 2 * hv + H, ib, fb, cap, dk ** -0.5, nw, eps,
                  state, i32(cu), sl, out, n_req, H, dk, dv, gate="sigmoid")
        return out
    got = [[] for _ in lens]
    at = [0, 0, 0]
    for part in ([20, 1, 2], [17, 0, 3]):
        live = [i for i, k in enumerate(part) if k]
        rows_h = torch.cat([hs[i][at[i]:at[i] + part[i]] for i in live])
        cu = [0]
        for i in live:
            cu.append(cu[-1] + part[i])
        out = launch(rows_h, cu, slots[live].contiguous(), len(live))
        o = 0
        for i in live:
            got[i].append(out[o:o + part[i]].double().cpu())
            o += part[i]
            at[i] += part[i]
    for i in range(3):
        assert float((torch.cat(got[i]) - want[i]).abs().max()) < tol * float(want[i].abs().max()), i
    assert float((state[2] - 7.0).abs().max()) == 0.0 and float(state[1].abs().max()) == 0.0
    state[3].zero_()                                       # as the cache manager does when the slot is taken again
    out = launch(hs[1], [0, 1], slots[:1].contiguous(), 1)
    assert float((out.double().cpu() - got[1][0]).abs().max()) < tol * float(got[1][0].abs().max())


@pytest.mark.parametrize("dk,dv", [(16, 24), (128, 64), (64, 128)])
def test_matrix_memory_kernel_cut_along_time(dk, dv):
    """A portion of 700 tokens beside one of 3 and one of 300: the long ones are cut into segments (local
    passes, a combine step, a pass from the true start states) and give what the walk token by token gives,
    from a state that an earlier call left."""
    from rllm_b200.csrc import ops
    from rllm_b200.engine.batch import StepContext
    H, d, eps, cap = 2, 24, 1e-5, 10.0
    g = torch.Generator().manual_seed(8)
    W = _memory_weights(H, dk, dv, d, g)
    mx = {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}
    lens, first = [705, 3, 300], 5
    hs = [torch.randn(n, d, generator=g, dtype=torch.float64) for n in lens]
    want = [pn.mlstm(h, W, "m.", mx, eps) for h in hs]
    w_in = torch.cat([W["m.q"], W["m.k"], W["m.v"], W["m.g"], W["m.i"], W["m.f"]], 0).float().to(DEV)
    hk, hv = H * dk, H * dv
    state = torch.zeros((3, ops.mlstm_state_floats(H, dk, dv)), device=DEV)
    ib, fb, nw = (W[k].float().to(DEV) for k in ("m.i.b", "m.f.b", "m.norm"))
    slots = i32([2, 0, 1])
    outs = []
    for part, starts in (([first, 0, 0], [0]), ([lens[0] - first, 3, 300], [first, 0, 0])):
        live = [i for i, k in enumerate(part) if k]
        ctx = step_context([part[i] for i in live], starts)
        seg = ops.time_segments(ctx, DEV)
        assert (seg is not None) == (max(part) >= ops.SEGMENT_FROM)
        a0 = [0 if (len(outs) == 0 or i) else first for i in live]
        rows_h = torch.cat([hs[i][a:a + part[i]] for i, a in zip(live, a0)])
        rows = (rows_h.float().to(DEV) @ w_in.T).contiguous()
        out = torch.empty((rows.shape[0], hv), device=DEV)
        ops.mlstm(rows, 0, hk, 2 * hk, 2 * hk + hv, 2 * hk + 2 * hv, 2 * hk + 2 * hv + H, ib, fb, cap, dk ** -0.5, nw, eps,
                  state, ctx.cu_q, slots[live].contiguous(), out, len(live), H, dk, dv, gate="sigmoid", segments=seg)
        outs.append(out.double().cpu())
    got0 = torch.cat([outs[0], outs[1][:lens[0] - first]])
    assert float((got0 - want[0]).abs().max()) < 1e-4 * float(want[0].abs().max())
    o = lens[0] - first
    assert float((outs[1][o:o + 3] - want[1]).abs().max()) < 1e-4 * float(want[1].abs().max())
    assert float((outs[1][o + 3:] - want[2]).abs().max()) < 1e-4 * float(want[2].abs().max())


@pytest.mark.parametrize("n", [5, 300])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_unit_with_the_tanh_gelu(dtype, n):
    """The activation kernel and, for many bfloat16 rows, the tensor-core product with the form in its epilogue."""
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(9)
    d, F = 128, 256
    h = torch.randn(n, d, generator=g).to(dtype).to(DEV)
    w = (torch.randn(2 * F, d, generator=g) * 2 / math.sqrt(d)).to(dtype).to(DEV)
    out = torch.empty((n, F), dtype=dtype, device=DEV)
    ops.gate_up_swiglu(h, w, out, glu=ops.GLU_GELU_TANH)
    ops.check_device_errors(DEV)
    gu = h.double() @ w.double().T
    want = pn.gelu_tanh(gu[:, :F]) * gu[:, F:]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert float((out.double() - want).abs().max()) < tol * float(want.abs().max())
    if dtype == torch.float32:
        assert float((pn.silu(gu[:, :F]) * gu[:, F:] - want).abs().max()) > 100 * tol * float(want.abs().max())     # silu would show


@pytest.mark.parametrize("E,top", [(8, 3), (5, 1), (6, 6), (64, 6)])
def test_router_kernel_with_a_bias(E, top):
    from rllm_b200.csrc import ops
    g = torch.Generator().manual_seed(10)
    n = 33
    w = {"r.router": torch.eye(E, dtype=torch.float64), "r.router.b": torch.randn(E, generator=g, dtype=torch.float64) * 2}
    z = torch.randn(n, E + 3, generator=g) * 2
    idx = torch.empty((n, top), dtype=torch.int32, device=DEV)
    wt = torch.empty((n, top), dtype=torch.float32, device=DEV)
    ops.moe_route(z.to(DEV), None, idx, wt, E, top, score="softmax", normalize=True, bias=w["r.router.b"].float().to(DEV))
    want_idx, want_w, _ = pn.route(z[:, :E].double(), w, "r.", top)
    for t in range(n):
        got = dict(zip(idx[t].tolist(), wt[t].tolist()))
        assert set(got) == set(want_idx[t].tolist())
        for e, x in zip(want_idx[t].tolist(), want_w[t].tolist()):
            assert abs(got[e] - x) < 1e-6


# ---------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_whole_prompt(name, dtype):
    cfg = CASES[name]
    w = nc.make_weights(cfg, 1, stored(dtype))
    toks = nc.tokens_for(cfg, 61, 1)
    ref = nc.oracle(cfg, w, toks)
    eng = nc.build_engine(cfg, w, dtype, max_tokens=128)
    out = run(eng, [([("a", toks, list(range(61)))], ["a"])])
    compare(out, {"a": ref}, dtype, name)
    assert not eng.cache.requests


def test_stream_after_every_layer():
    """float32: the residual stream behind every layer of the stack is the plain implementation's."""
    cfg = CASES["stack"]
    w = nc.make_weights(cfg, 2)
    toks = nc.tokens_for(cfg, 40, 2)
    streams = []
    nc.oracle(cfg, w, toks, streams)
    eng = nc.build_engine(cfg, w, "float32", max_tokens=64)
    seen = []
    for b in eng.model.blocks:
        def wrapped(x, pending, ctx, cache, _f=b.forward, **kw):
            out = _f(x, pending, ctx, cache, **kw)
            seen.append(x.detach().double().cpu().clone())
            return out
        b.forward = wrapped
    run(eng, [([("a", toks, [39])], ["a"])])
    assert len(seen) == len(streams) == 6
    for i, (got, want) in enumerate(zip(seen, streams)):
        assert float((got - want).abs().max()) < 2e-5 * float(want.abs().max()), i


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CASES))
def test_token_by_token_and_portions(name, dtype):
    """The same prompt whole, token by token from the start, and in portions of 7, 2, 5, 3, 2, 2, 19, then 2s:
    every row against the plain implementation."""
    cfg = CASES[name]
    w = nc.make_weights(cfg, 3, stored(dtype))
    toks = nc.tokens_for(cfg, 58, 3)
    ref = {"a": nc.oracle(cfg, w, toks)}
    eng = nc.build_engine(cfg, w, dtype, max_tokens=128)
    compare(run(eng, closing(one_by_one("a", toks), "a")), ref, dtype, name + " token by token")
    steps = [([("a", t, want)], []) for t, want in cut(toks, [7, 2, 5, 3, 2, 2, 19, 2])]
    compare(run(eng, closing(steps, "a")), ref, dtype, name + " in portions")
    steps = [([("a", toks[:33], [0, 32])], [])] + one_by_one("a", toks, 33)
    compare(run(eng, closing(steps, "a")), ref, dtype, name + " prompt then single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["stack", "stack_attention_first", "heads64", "heads128", "latent64", "moe"])
def test_unequal_requests_in_one_batch_with_reuse(name, dtype):
    """Four requests of 70, 9, 31 and 2 tokens, portions of some beside single tokens of others, a fifth
    that takes over the pages and the slot of one that ended: every row is what the request gives alone."""
    cfg = CASES[name]
    w = nc.make_weights(cfg, 4, stored(dtype))
    lens = {"a": 70, "b": 9, "c": 31, "d": 2, "e": 26}
    toks = {r: nc.tokens_for(cfg, n, 10 + i) for i, (r, n) in enumerate(lens.items())}
    refs = {r: nc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = nc.build_engine(cfg, w, dtype, max_tokens=192, max_requests=4)
    T = toks
    all_ = lambda k: list(range(k))
    steps = [
        ([("a", T["a"][:40], all_(40)), ("b", T["b"][:3], all_(3))], []),
        ([("a", T["a"][40:41], [0]), ("b", T["b"][3:9], all_(6)), ("c", T["c"][:17], all_(17)), ("d", T["d"][:2], all_(2))], ["b", "d"]),
        ([("c", T["c"][17:18], [0]), ("e", T["e"][:11], all_(11)), ("a", T["a"][41:43], all_(2))], []),
        ([("e", T["e"][11:26], all_(15)), ("a", T["a"][43:44], [0]), ("c", T["c"][18:19], [0])], ["e"]),
        ([("a", T["a"][44:70], all_(26)), ("c", T["c"][19:31], all_(12))], ["a", "c"]),
    ]
    compare(run(eng, steps), refs, dtype, name)
    assert not eng.cache.requests
    eng.cache.check_invariants()


def test_pages_and_slots_used_again_give_the_same_bits():
    """A request run alone in a fresh engine, and again in an engine whose pages and slots other requests
    have used and given back: the same bits."""
    cfg = CASES["stack"]
    w = nc.make_weights(cfg, 5)
    toks, other = nc.tokens_for(cfg, 45, 20), nc.tokens_for(cfg, 60, 21)
    steps = lambda r, t: closing([([(r, t[:30], list(range(30)))], [])] + one_by_one(r, t, 30), r)
    fresh = run(nc.build_engine(cfg, w, "float32", max_tokens=64, max_requests=2), steps("a", toks))
    eng = nc.build_engine(cfg, w, "float32", max_tokens=64, max_requests=2)
    run(eng, steps("x", other))
    run(eng, steps("y", other[::-1]))
    again = run(eng, steps("a", toks))
    for key, row in fresh.items():
        assert torch.equal(row, again[key]), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention", "heads64", "heads128"])
def test_keys_at_the_windows_edges_decide_rows(name, dtype):
    """The marked attention layer with a sharp scale: the token `asker` asks for the keys of `target`.  A
    prompt in which an asker follows a target at every distance around the window (the last key inside, the
    first key outside, one further, the key right before), whole, in portions that cut the window, and
    decoded token by token across page borders: every row against the plain implementation, which itself
    changes by far more than the tolerance when its windows are one key longer."""
    cfg = nc.sharpened(CASES[name], 6.0, layers=[0])
    cfg["embedding"]["scale"] = 8.0                               # a token's row is its id's, whatever came before it
    window = cfg["layers"][0]["mixer"]["mask"]["size"]
    asker, target = 5, 9
    w = nc.marked_attention(cfg, nc.make_weights(cfg, 6, stored(dtype)), asker, target)
    toks = nc.tokens_for(cfg, 13 * window + 40, 30, avoid=(asker, target))
    asks = []
    at = 3
    for dist in (window - 1, window, window + 1, 1, window - 1, window):     # the asker comes `dist` tokens behind
        toks[at] = target
        at += dist
        toks[at] = asker
        asks.append(at)
        at += window + 2                                                 # the next pair starts with a clean window
    toks = toks[:at]
    ref = nc.oracle(cfg, w, toks)
    off = nc.oracle(nc.with_windows(cfg, 1), w, toks)
    moved = [row_error(off[a], ref[a]) for a in asks]
    assert min(moved[1], moved[5]) > 1.5 * TOL[dtype], moved           # the key just outside would be seen
    eng = nc.build_engine(cfg, w, dtype, max_tokens=2 * len(toks), block_size=8)
    refs = {"a": ref}
    compare(run(eng, [([("a", toks, list(range(len(toks))))], ["a"])]), refs, dtype, "whole")
    steps = [([("a", t, want)], []) for t, want in cut(toks, [window - 2, 3, 2, window + 1, 5])]
    compare(run(eng, closing(steps, "a")), refs, dtype, "portions")
    compare(run(eng, closing([([("a", toks[:2], [0, 1])], [])] + one_by_one("a", toks, 2), "a")), refs, dtype, "decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["latent", "latent64", "stack"])
def test_sharp_attention_over_every_window(name, dtype):
    """Every attention layer with a sharper scale, so that rows hang on fewer keys (four times as sharp in
    float32; in bfloat16 one and a half times, beyond which the rounding of the scores themselves moves the
    rows): a prompt several windows long whole, cut and decoded; the plain implementation with windows one key
    longer differs on many rows by more than the tolerance."""
    cfg = nc.sharpened(CASES[name], 4.0 if dtype == "float32" else 1.5)
    w = nc.make_weights(cfg, 7, stored(dtype))
    toks = nc.tokens_for(cfg, 150, 31)
    ref = nc.oracle(cfg, w, toks)
    off = nc.oracle(nc.with_windows(cfg, 1), w, toks)
    tol = 3 * TOL[dtype] if dtype == "float32" else TOL[dtype]
    moved = sum(row_error(off[p], ref[p]) > 2 * tol for p in range(60, 150))
    assert moved > 9, moved
    eng = nc.build_engine(cfg, w, dtype, max_tokens=192, block_size=8)
    refs = {"a": ref}
    compare(run(eng, [([("a", toks, list(range(150)))], ["a"])]), refs, dtype, "whole", tol)
    steps = [([("a", t, want)], []) for t, want in cut(toks, [29, 2, 31, 7, 2, 40, 3])]
    compare(run(eng, closing(steps, "a")), refs, dtype, "portions", tol)
    compare(run(eng, closing([([("a", toks[:50], [49])], [])] + one_by_one("a", toks, 50), "a")), refs, dtype, "decoded", tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["memory", "memory_128"])
def test_a_token_hundreds_of_places_back_decides_rows_through_the_memory(name, dtype):
    """The marked memory layer: one token near the start writes most of what the memory holds 600 tokens
    later.  The prompt whole (cut along time), in portions, and its last 60 tokens decoded: every row against the
    plain implementation, whose rows far behind the marker change by much more than the tolerance when the
    marker is another token."""
    cfg = dict(CASES[name], embedding=dict(CASES[name]["embedding"], scale=8.0))
    marker = 7
    w = nc.marked_memory(cfg, nc.make_weights(cfg, 13, stored(dtype)), marker)
    toks = nc.tokens_for(cfg, 650, 80, avoid=(marker,))
    without = list(toks)
    toks[5] = marker
    ref, other = nc.oracle(cfg, w, toks), nc.oracle(cfg, w, without)
    moved = [row_error(other[p], ref[p]) for p in range(300, 650)]
    assert min(moved) > 2 * TOL[dtype] and sorted(moved)[len(moved) // 2] > 5 * TOL[dtype], min(moved)
    want = list(range(0, 650, 41)) + list(range(600, 650))
    eng = nc.build_engine(cfg, w, dtype, max_tokens=1024, block_size=16)
    refs = {"a": ref}
    compare(run(eng, [([("a", toks, want)], ["a"])]), refs, dtype, "whole")
    steps = [([("a", t, [len(t) - 1])], []) for t, _ in cut(toks, [290, 2, 130, 7, 200, 21])]
    compare(run(eng, closing(steps, "a")), refs, dtype, "portions")
    compare(run(eng, closing([([("a", toks[:590], [589])], [])] + one_by_one("a", toks, 590), "a")), refs, dtype, "decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens(dtype):
    """Requests of 1, 2 and 3 tokens alone and together: the first token takes the pair table's last row, sees
    itself only, and meets an empty memory whose maximum starts at 0."""
    cfg = CASES["stack"]
    w = nc.make_weights(cfg, 8, stored(dtype))
    toks = {"a": nc.tokens_for(cfg, 1, 40), "b": nc.tokens_for(cfg, 2, 41), "c": nc.tokens_for(cfg, 3, 42)}
    refs = {r: nc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = nc.build_engine(cfg, w, dtype, max_tokens=64)
    steps = [([(r, t, list(range(len(t)))) for r, t in toks.items()], list(toks))]
    compare(run(eng, steps), refs, dtype, "together")
    for r, t in toks.items():
        compare(run(eng, closing(one_by_one(r, t), r)), refs, dtype, "alone " + r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions(dtype):
    """A prompt of 700 tokens in one step (the matrix memory is cut along time, the windows have long passed
    the first pages), the same in two steps of 411 and 289, and 20 more tokens one by one."""
    cfg = CASES["stack"]
    w = nc.make_weights(cfg, 9, stored(dtype))
    toks = nc.tokens_for(cfg, 720, 50)
    refs = {"a": nc.oracle(cfg, w, toks)}
    want = list(range(0, 700, 37)) + [255, 256, 257, 699]
    eng = nc.build_engine(cfg, w, dtype, max_tokens=1024, block_size=16)
    steps = [([("a", toks[:700], want)], [])] + one_by_one("a", toks, 700)
    compare(run(eng, closing(steps, "a")), refs, dtype, "one step")
    steps = [([("a", toks[:411], [0, 300, 410])], []), ([("a", toks[411:700], [0, 100, 288])], [])] + one_by_one("a", toks, 700)
    compare(run(eng, closing(steps, "a")), refs, dtype, "two steps")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graph_replay(dtype):
    """Two requests decode 150 tokens each after prompts of 20 and 3: replayed from CUDA graphs and launched
    one by one, both against the plain implementation (float32) and against each other."""
    cfg = CASES["stack_attention_first"]
    w = nc.make_weights(cfg, 10, stored(dtype))
    toks = {"a": nc.tokens_for(cfg, 170, 60), "b": nc.tokens_for(cfg, 153, 61)}
    steps = [([("a", toks["a"][:20], [19]), ("b", toks["b"][:3], [2])], [])]
    steps += [([("a", [toks["a"][20 + i]], [0]), ("b", [toks["b"][3 + i]], [0])], []) for i in range(150)]
    outs = []
    for graphs in (True, False):
        eng = nc.build_engine(cfg, w, dtype, max_tokens=512, use_graphs=graphs)
        outs.append(run(eng, steps))
        if graphs:
            assert eng.stats["graph_replays"] > 100
    if dtype == "float32":
        refs = {r: nc.oracle(cfg, w, t) for r, t in toks.items()}
        compare(outs[0], refs, dtype, "replayed")
        compare(outs[1], refs, dtype, "launched")
    for key, row in outs[0].items():
        assert row_error(row, outs[1][key]) < (1e-6 if dtype == "float32" else 2e-2), key


REAL = nc.config([nc.mem(8, 64, 128, mlp=nc.dense(1536)),
                  nc.att(8, 2, 128, 128, 64, 100, scaling=(8.0, 1.0, 4.0, 256), mlp=nc.moe(256, 32, 4)),
                  nc.lat(8, 64, 32, 64, 256, 70, mlp=nc.dense(1024)),
                  nc.att(16, 4, 64, 64, 64, 33, mlp=nc.moe(384, 8, 2))], width=1024, vocab=1531, scale=6.0, bigram=(997, 29, 5))


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_layer_sizes_of_a_real_model(dtype):
    """Width 1,024 and layers of real sizes (memory heads of 64 x 128, attention heads of 128 and 64, a latent
    of 256, 32 experts): the products take the library, the tcgen05 and the weight-streaming kernels, attention
    the tensor-core kernels.  A prompt of 300 tokens, a portion of 40 beside another request's 20, then single
    tokens of both."""
    cfg = REAL
    w = nc.make_weights(cfg, 16, stored(dtype), gain=1.0)
    toks = {"a": nc.tokens_for(cfg, 352, 70), "b": nc.tokens_for(cfg, 32, 71)}
    refs = {r: nc.oracle(cfg, w, t) for r, t in toks.items()}
    eng = nc.build_engine(cfg, w, dtype, max_tokens=512, block_size=32, max_requests=2)
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
    w = nc.make_weights(cfg, 11)
    write_folder(tmp_path, cfg, w)
    prompts = [nc.tokens_for(cfg, n, 40 + i) for i, n in enumerate((37, 3, 21, 50, 9))]
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
            logits = nc.oracle(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) < 1e-4:       # a tie at float32 precision decides nothing
                break
            assert int(logits.argmax()) == tok
            seq.append(tok)
            checked += 1
    assert all(len(g) == 12 for g in got) and checked > 40
    assert not llm.engine.cache.requests


def test_trace_replay_program_chooses_the_model_by_its_config(tmp_path):
    """bin/trace_run on a Navulorn folder: steps from standard input, rows out as little-endian float32; two
    requests share the steps, one pauses, pages and slots go back at the end."""
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    cfg = CASES["stack_attention_first"]
    w = nc.make_weights(cfg, 12, torch.bfloat16)
    model = write_folder(tmp_path / "model", cfg, w)
    toks, other = nc.tokens_for(cfg, 30, 6), nc.tokens_for(cfg, 9, 7)
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
    ref, ref_other = nc.oracle(cfg, w, toks), nc.oracle(cfg, w, other)
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
