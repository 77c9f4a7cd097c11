"""Python wrappers over the extern "C" kernel launchers.

Every wrapper takes CUDA torch tensors, checks what the kernel assumes (device,
dtype, contiguity, sizes) and launches on the current torch stream.  There is no
CPU or library fallback: a tensor that is not on a CUDA device, or a library that
cannot be built and loaded, raises.
"""
from __future__ import annotations

import ctypes
import os
import struct
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build, profiler

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {t.dtype}; kernels take float32 and bfloat16") from None


def _ptr(t):
    if t is None:
        return c_void_p(0)
    if _trace is not None:
        _trace.keep.append(t)                 # a traced launch names this memory: it stays alive with the trace
    return c_void_p(t.data_ptr())


# ------------------------------------------------------------------ trace and replay of launches
# A step that is not replayed from a CUDA graph launches its kernels from Python, and most of what a
# launch costs the host is the wrapper around it: checks, dispatch rules, argument conversion (7 to
# 13 us against 3.5 us for the call itself).  The layers of a model are alike: what one layer launches,
# the next launches too, with its own weights and cache planes in place of the first one's.  So the
# launches of one layer are recorded (`tracing`) and replayed for the layers of the same build
# (`Trace.replay`): the recorded calls again, argument for argument, with the pointers that belong to
# the layer swapped.  Whatever a wrapper decides from shapes and types it has decided once.
_trace = None


class Trace:
    """The launches recorded between `tracing()` and its end: (launcher, arguments) in order.
    `freeze(addresses)` names the addresses that belong to the layer, in the order in which
    `replay(addresses of another layer)` gives theirs; the calls then live in the C++ host runtime
    (host_runtime.cpp, rllm_trace_replay), which makes them again through the launchers'
    packed-argument forms, one call from Python for the whole layer."""

    def __init__(self):
        self.calls: list = []             # [library, launcher name, [ctypes arguments]]
        self.keep: list = []              # tensors (and ctypes objects) whose memory the arguments name
        self.own_launches = 0
        self._native = None
        self._n_roles = 0

    @staticmethod
    def _word(a) -> int:
        if isinstance(a, c_void_p):
            return a.value or 0
        if isinstance(a, c_float):
            return struct.unpack("<I", struct.pack("<f", a.value))[0]
        if isinstance(a, (c_int, c_longlong)):
            return a.value & 0xFFFFFFFFFFFFFFFF
        if isinstance(a, int):
            return a & 0xFFFFFFFFFFFFFFFF
        return ctypes.cast(a, c_void_p).value or 0          # byref(...) of an out parameter, a ctypes pointer

    def freeze(self, addresses) -> None:
        role_of = {}
        for i, addr in enumerate(addresses):
            role_of.setdefault(addr, i)
        self._n_roles = len(addresses)
        fns, n_args, words, swap_at, swap_role = [], [], [], [], []
        for lib, name, args in self.calls:
            fn = getattr(lib, name + "_packed")
            fns.append(ctypes.cast(fn, c_void_p).value)
            n_args.append(len(args))
            for a in args:
                if isinstance(a, c_void_p) and a.value in role_of:
                    swap_at.append(len(words))
                    swap_role.append(role_of[a.value])
                words.append(self._word(a))
        self.keep.append([a for _, _, args in self.calls for a in args])     # out parameters stay alive
        host = build.load("host")
        host.rllm_trace_create.restype = c_void_p
        host.rllm_trace_create.argtypes = [c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int),
                                           ctypes.POINTER(ctypes.c_ulonglong), c_int, ctypes.POINTER(c_int),
                                           ctypes.POINTER(c_int)]
        host.rllm_trace_replay.argtypes = [c_void_p, ctypes.POINTER(ctypes.c_ulonglong), c_int, ctypes.POINTER(c_int)]
        host.rllm_trace_destroy.argtypes = [c_void_p]
        n = len(fns)
        self._host = host
        self._native = host.rllm_trace_create(
            n, (c_void_p * max(n, 1))(*fns), (c_int * max(n, 1))(*n_args),
            (ctypes.c_ulonglong * max(len(words), 1))(*words), len(swap_at),
            (c_int * max(len(swap_at), 1))(*swap_at), (c_int * max(len(swap_role), 1))(*swap_role))
        if not self._native:
            raise KernelError("the host runtime refused a trace of launches")

    def replay(self, addresses) -> None:
        """Launches the recorded calls again with `addresses` (same order as at `freeze`) in place."""
        if len(addresses) != self._n_roles:
            raise KernelError("replay: other addresses than the trace was frozen with")
        failed = c_int(-1)
        status = self._host.rllm_trace_replay(self._native, (ctypes.c_ulonglong * max(self._n_roles, 1))(*addresses),
                                              self._n_roles, ctypes.byref(failed))
        if status:
            name = self.calls[failed.value][1] if 0 <= failed.value < len(self.calls) else "?"
            raise KernelError(f"replayed launch {name}: status {status}")
        add_launches(self.own_launches)

    def __del__(self):
        try:
            if self._native:
                self._host.rllm_trace_destroy(self._native)
                self._native = None
        except Exception:
            pass


class _RecordingLibrary:
    def __init__(self, lib, trace):
        self._lib, self._trace = lib, trace

    def __getattr__(self, name):
        lib, trace = self._lib, self._trace
        fn = getattr(lib, name)

        def call(*args):
            trace.calls.append((lib, name, list(args)))
            return fn(*args)
        return call


class tracing:
    """``with ops.tracing() as trace:`` every launch inside is recorded into `trace` (and made)."""

    def __enter__(self):
        global _trace
        if _trace is not None:
            raise KernelError("a trace is being recorded already")
        _trace = Trace()
        self._before = _launches
        return _trace

    def __exit__(self, *exc):
        global _trace
        trace, _trace = _trace, None
        trace.own_launches = _launches - self._before


class untraced:
    """``with ops.untraced():`` launches inside are made but not recorded (what one pass does once for
    all its layers, like the table of rotary angles)."""

    def __enter__(self):
        global _trace
        self._saved, _trace = _trace, None

    def __exit__(self, *exc):
        global _trace
        _trace = self._saved


def can_trace() -> bool:
    """Launches can be recorded (not while every launch is timed with events)."""
    return not profiler.enabled()


_raw_stream = torch._C._cuda_getCurrentRawStream
_current_device = torch._C._cuda_getDevice


def _stream():
    """The current stream of the current device, as the launchers take it (the raw handle: building a
    torch.cuda.Stream object for every launch costs more than the launch)."""
    return c_void_p(_raw_stream(_current_device()))


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("rllm_b200 kernels run on a CUDA device only; got a tensor on "
                              f"{t.device}. There is no CPU path.")


def _need_contig(**ts):
    for name, t in ts.items():
        if t is not None and not t.is_contiguous():
            raise KernelError(f"{name} must be contiguous")


_launches = 0


def launch_count() -> int:
    """Number of this package's own kernels launched so far (library products not counted)."""
    return _launches


def add_launches(n: int) -> None:
    """Counts kernels that ran from a replayed CUDA graph."""
    global _launches
    _launches += n


def _check(status: int, what: str, own: bool = True):
    global _launches
    if status != 0:
        raise KernelError(f"{what}: CUDA error {status} (cudaError_t)")
    if own:
        _launches += 1


_timed: dict = {}


def _lib(name: str):
    """The loaded library `name`; with RLLM_B200_PROFILE=1 its launchers are timed with CUDA events."""
    lib = _timed.get(name)
    if lib is None:
        lib = build.load(name)
        if profiler.enabled():
            lib = profiler.TimedLibrary(lib)
        _timed[name] = lib
    if _trace is not None:
        return _RecordingLibrary(lib, _trace)
    return lib


def core():
    return _lib("core")


# ------------------------------------------------------------------ elementwise

def embed(table, tokens, out, err=None):
    """out[t,:] = table[tokens[t],:] as float32.  table [V,d] f32/bf16, tokens int32 [n], out f32 [n,d]."""
    _need_cuda(table, tokens, out)
    _need_contig(table=table, tokens=tokens, out=out)
    n, d = out.shape
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32 and table.shape[1] == d
    _check(core().rllm_embed(_ptr(table), _code(table), _ptr(tokens), _ptr(out), c_int(n), c_int(d),
                             c_int(table.shape[0]), _ptr(err), _stream()), "embed")
    return out


def embed_pair(table, pair_table, ctx_tokens, positions, seq_ids, cu_q, slots, last_tok, out, scale, buckets,
               mul_prev, mul_cur, err=None):
    """out[t] = table[token] * scale + pair_table[(previous * mul_prev + token * mul_cur) mod buckets], and
    pair_table[buckets] for a request's first token; the previous token of the first row a request brings
    is last_tok[slots[request]] (int32, written by keep_last_tokens after the step before)."""
    _need_cuda(table, pair_table, ctx_tokens, positions, seq_ids, cu_q, slots, last_tok, out)
    _need_contig(table=table, pair_table=pair_table, tokens=ctx_tokens, out=out, last_tok=last_tok)
    n, d = out.shape
    assert out.dtype == torch.float32 and table.shape[1] == d and pair_table.shape == (buckets + 1, d)
    assert table.dtype == pair_table.dtype and last_tok.dtype == torch.int32
    _check(core().rllm_embed_pair(_ptr(table), _ptr(pair_table), c_int(_code(table)), _ptr(ctx_tokens), _ptr(positions),
                                  _ptr(seq_ids), _ptr(cu_q), _ptr(slots), _ptr(last_tok), _ptr(out), c_int(n), c_int(d),
                                  c_int(table.shape[0]), c_float(scale), c_int(buckets), c_longlong(mul_prev),
                                  c_longlong(mul_cur), _ptr(err), _stream()), "embed_pair")
    return out


def keep_last_tokens(ctx_tokens, cu_q, slots, last_tok, n_requests):
    """last_tok[slots[r]] = the last token that request r brings in this step."""
    _need_cuda(ctx_tokens, cu_q, slots, last_tok)
    _check(core().rllm_keep_last_tokens(_ptr(ctx_tokens), _ptr(cu_q), _ptr(slots), _ptr(last_tok), c_int(n_requests),
                                        _stream()), "keep_last_tokens")


def add_rms_norm(x, delta, weight, out, eps, rows=None, write_x=True, delta_scale=1.0):
    """out[r] = rmsnorm(x[src] (+ delta_scale * delta[src])) * weight with src = rows[r] if rows is given
    else r.  x is the float32 residual stream and receives the sum when write_x (and delta is given)."""
    _need_cuda(x, delta, weight, out, rows)
    _need_contig(x=x, delta=delta, weight=weight, out=out, rows=rows)
    d = x.shape[-1]
    n_rows = out.shape[0]
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == d
    assert out.shape[-1] == d
    if rows is None:
        assert x.shape[0] == n_rows
    else:
        assert rows.dtype == torch.int32 and rows.numel() == n_rows
    if delta is not None:
        assert delta.shape == x.shape
    _check(core().rllm_add_rms_norm(_ptr(x), _ptr(delta), c_int(_code(delta) if delta is not None else F32),
                                    _ptr(rows), _ptr(weight), _ptr(out), c_int(_code(out)), c_int(n_rows),
                                    c_int(d), c_float(eps), c_int(1 if write_x else 0), c_float(delta_scale),
                                    _stream()),
           "add_rms_norm")
    return out


def add_inplace(x, delta):
    _need_cuda(x, delta)
    _need_contig(x=x, delta=delta)
    assert x.dtype == torch.float32 and x.shape == delta.shape
    _check(core().rllm_add_inplace(_ptr(x), _ptr(delta), c_int(_code(delta)), c_longlong(x.numel()),
                                   _stream()), "add_inplace")
    return x


def silu_mul(gate_up, out):
    """gate_up [n, 2F] (gate columns then up columns) -> out [n, F] = silu(gate) * up."""
    _need_cuda(gate_up, out)
    _need_contig(gate_up=gate_up, out=out)
    n, F = out.shape
    assert gate_up.shape == (n, 2 * F)
    _check(core().rllm_silu_mul(_ptr(gate_up), c_int(_code(gate_up)), _ptr(out), c_int(_code(out)),
                                c_int(n), c_int(F), _stream()), "silu_mul")
    return out


def rope_table(positions, inv_freq):
    """(cos, sin) of positions[t] * inv_freq[i] as float32 [n, head_dim/2, 2]: the rotation angles of a
    step's tokens, worked out once and read by every layer's qk_norm_rope_store."""
    _need_cuda(positions, inv_freq)
    n, half = positions.numel(), inv_freq.numel()
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()
    out = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    _check(core().rllm_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(out), c_int(n), c_int(half), _stream()),
           "rope_table")
    return out


def qk_norm_rope_store(qkv, q_norm_w, k_norm_w, inv_freq, positions, slots, q_out, k_cache, v_cache,
                       H, K, hd, block_size, eps, write_kv=True, cs_table=None):
    """Fused per-head q/k RMSNorm, rotary embedding and paged K/V write; see elementwise.cu.
    The rotation takes its angles from `cs_table` (rope_table: made once per step and shared by the
    layers); given `inv_freq` alone, the table is made here; neither: no rotation."""
    _need_cuda(qkv, q_norm_w, k_norm_w, inv_freq, positions, slots, q_out, k_cache, v_cache)
    _need_contig(qkv=qkv, q_out=q_out, k_cache=k_cache, v_cache=v_cache, positions=positions, slots=slots)
    n = qkv.shape[0]
    assert qkv.shape[1] == (H + 2 * K) * hd and q_out.shape == (n, H * hd)
    assert positions.dtype == torch.int32 and slots.dtype == torch.int32
    assert positions.numel() == n and slots.numel() == n
    if hd % 4 or hd > 256:
        raise KernelError(f"head size {hd} is not supported: the q/k norm + rotary kernel takes multiples of 4 up to 256")
    for w in (q_norm_w, k_norm_w):
        assert w is None or (w.dtype == torch.float32 and w.numel() == hd)
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == hd // 2)
    assert k_cache.dtype == q_out.dtype == v_cache.dtype
    if cs_table is None and inv_freq is not None:
        cs_table = rope_table(positions, inv_freq)
    assert cs_table is None or (cs_table.dtype == torch.float32 and cs_table.shape == (n, hd // 2, 2)
                                and cs_table.is_contiguous())
    _check(core().rllm_qk_norm_rope_store(
        _ptr(qkv), c_int(_code(qkv)), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cs_table), _ptr(positions),
        _ptr(slots), _ptr(q_out), c_int(_code(q_out)), _ptr(k_cache), _ptr(v_cache), c_int(_code(k_cache)),
        c_int(n), c_int(H), c_int(K), c_int(hd), c_int(block_size), c_float(eps),
        c_int(1 if write_kv else 0), c_longlong(k_cache.shape[0] * block_size), _ptr(error_word(qkv.device)),
        _stream()), "qk_norm_rope_store")
    return q_out


# ------------------------------------------------------------------ attention

def paged_attention_generic(q, k_cache, v_cache, out, positions, seq_ids, block_table, H, K, hd,
                            block_size, scale, window=0, keep_first=0, v_head_dim=None, chunk=0, softcap=0.0,
                            sink=None):
    """Plain paged causal attention; q [n, H*hd], out [n, H*hdv], caches [pages, K, block_size, hd] and
    [pages, K, block_size, hdv] (hdv = v_head_dim, hd by default).  keep_first: the first keys of a
    request stay visible when the window has passed them.  chunk: a token sees only the keys of its
    own run of that many positions (counted from 0).  softcap: scores go through cap * tanh(s / cap).
    `v_cache is k_cache` with hdv < hd: the values are the first hdv entries of the key rows.
    sink (float32 [H]): exp(sink[h]) joins the softmax's denominator of head h, with no key and no value."""
    _need_cuda(q, k_cache, v_cache, out, positions, seq_ids, block_table, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H and sink.is_contiguous())
    _need_contig(q=q, k_cache=k_cache, v_cache=v_cache, out=out, positions=positions, seq_ids=seq_ids)
    n = q.shape[0]
    hdv = hd if not v_head_dim else int(v_head_dim)
    assert q.shape == (n, H * hd) and out.shape == (n, H * hdv)
    v_ld = hd if (v_cache.data_ptr() == k_cache.data_ptr() and hdv < hd) else hdv
    assert k_cache.shape[-1] == hd and v_cache.shape[-1] == v_ld >= hdv
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.stride(1) == 1
    assert positions.dtype == torch.int32 and seq_ids.dtype == torch.int32
    if hd > 2048 or hdv > 512:
        raise KernelError(f"head sizes {hd} (keys) and {hdv} (values) exceed the attention kernel's limits of 2048 and 512")
    if H % K:
        raise KernelError(f"{H} query heads are not a multiple of {K} key/value heads")
    _check(core().rllm_paged_attention_generic(
        _ptr(q), c_int(_code(q)), _ptr(k_cache), _ptr(v_cache), c_int(_code(k_cache)), _ptr(out),
        c_int(_code(out)), _ptr(positions), _ptr(seq_ids), _ptr(block_table), c_int(block_table.stride(0)),
        c_int(n), c_int(H), c_int(K), c_int(hd), c_int(hdv), c_int(block_size), c_float(scale), c_int(window),
        c_int(keep_first), c_int(min(k_cache.shape[0], 0x7fffffff)), _ptr(error_word(q.device)), c_int(chunk),
        c_float(softcap), c_int(v_ld), _ptr(sink), _stream()),
        "paged_attention_generic")
    return out


# ------------------------------------------------------------------ output norms, rotate-then-norm heads, latents (headwise.cu)

def norm_rows(rows, weight, eps, x=None, add=False, low=None):
    """v = rows / rms(rows) * weight (weight None: 1) (+ x when `add`); x (float32 [n, d], optional)
    takes v; `low` (optional, any row stride) takes v in its own type.  `rows` may be x itself, or
    columns of a wider matrix."""
    _need_cuda(rows, weight, x, low)
    _rows2d(rows, "rows")
    n, d = rows.shape
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == d and weight.is_contiguous())
    assert x is None or (x.dtype == torch.float32 and x.shape == (n, d) and x.is_contiguous())
    assert low is None or _rows2d(low, "low").shape == (n, d)
    if x is None and low is None:
        raise KernelError("norm_rows: nowhere to write")
    _check(core().rllm_norm_rows(_ptr(rows), c_int(_code(rows)), c_longlong(rows.stride(0)), _ptr(weight), _ptr(x),
                                 c_int(1 if add else 0), _ptr(low), c_int(_code(low) if low is not None else F32),
                                 c_longlong(low.stride(0) if low is not None else 0), c_int(n), c_int(d), c_float(eps),
                                 _stream()), "norm_rows")
    return low if low is not None else x


def sum_norm_rows(x, y, alpha, weight, eps, low=None):
    """x = (alpha * x + y) / rms(alpha * x + y) * weight in place (x: the float32 stream, y: a sublayer's
    output in any type); `low` (optional) takes the new rows in its own type."""
    _need_cuda(x, y, weight, low)
    _need_contig(x=x, weight=weight)
    _rows2d(y, "y")
    n, d = x.shape
    assert x.dtype == torch.float32 and y.shape == (n, d) and weight.dtype == torch.float32 and weight.numel() == d
    assert low is None or _rows2d(low, "low").shape == (n, d)
    _check(core().rllm_sum_norm_rows(_ptr(x), c_float(alpha), _ptr(y), c_int(_code(y)), c_longlong(y.stride(0)),
                                     _ptr(weight), _ptr(low), c_int(_code(low) if low is not None else F32),
                                     c_longlong(low.stride(0) if low is not None else 0), c_int(n), c_int(d),
                                     c_float(eps), _stream()), "sum_norm_rows")
    return x


def rope_unitnorm_store(rows, cs_table, rot, cs_mult, slots, q_out, k_cache, v_cache, H, G, hd, block_size, eps,
                        unit_norm=True, v_tied=True, write_kv=True):
    """rows [n, (H + G) * hd (+ G * hd values)] -> per head: the first `rot` entries rotated by the
    angles of cs_table [n, rot/2, 2] (cos and sin times cs_mult), then the head divided by its root mean
    square (unit_norm); queries to q_out, keys to the paged cache; the values stored are the key heads
    as projected (v_tied) or the row's value columns.  See headwise.cu."""
    _need_cuda(rows, cs_table, slots, q_out, k_cache, v_cache)
    _need_contig(q_out=q_out, k_cache=k_cache, v_cache=v_cache, slots=slots)
    _rows2d(rows, "rows")
    n = rows.shape[0]
    assert rows.shape[1] == (H + G * (1 if v_tied else 2)) * hd and q_out.shape == (n, H * hd)
    assert slots.dtype == torch.int32 and slots.numel() == n
    assert k_cache.shape[1:] == (G, block_size, hd) and v_cache.shape[1:] == (G, block_size, hd)
    assert k_cache.dtype == v_cache.dtype == q_out.dtype
    assert rot == 0 or (cs_table.dtype == torch.float32 and cs_table.shape == (n, rot // 2, 2) and cs_table.is_contiguous())
    _check(core().rllm_rope_unitnorm_store(
        _ptr(rows), c_int(_code(rows)), c_longlong(rows.stride(0)), _ptr(cs_table), c_int(rot), c_float(cs_mult),
        _ptr(slots), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), c_int(_code(q_out)), c_int(n), c_int(H), c_int(G),
        c_int(hd), c_int(block_size), c_float(eps), c_int(1 if unit_norm else 0), c_int(1 if v_tied else 0),
        c_int(1 if write_kv else 0), c_longlong(k_cache.shape[0] * block_size), _ptr(error_word(rows.device)),
        _stream()), "rope_unitnorm_store")
    return q_out


def head_norm_rope_store(rows, q_norm_w, k_norm_w, cs_table, rot, pairs, slots, q_out, k_cache, v_cache, H, G, hd, hdv,
                         block_size, eps, has_kv=True, write_kv=True):
    """rows [n, H*hd (+ G*hd + G*hdv when has_kv)] -> per query and key head: RMS norm with a weight of hd
    entries (None: no norm), then the first `rot` entries rotated by the angles of cs_table [n, rot/2, 2]
    (pairs (2i, 2i+1) when `pairs`, else (i, i + rot/2)); queries to q_out, keys and values (heads of hdv
    entries) into the paged cache.  See headwise.cu."""
    _need_cuda(rows, q_norm_w, k_norm_w, cs_table, slots, q_out, k_cache, v_cache)
    _need_contig(q_out=q_out, k_cache=k_cache, v_cache=v_cache, slots=slots)
    _rows2d(rows, "rows")
    n = rows.shape[0]
    assert rows.shape[1] == H * hd + (G * (hd + hdv) if has_kv else 0) and q_out.shape == (n, H * hd)
    assert slots.dtype == torch.int32 and slots.numel() == n
    assert k_cache.shape[1:] == (G, block_size, hd) and v_cache.shape[1:] == (G, block_size, hdv)
    assert k_cache.dtype == v_cache.dtype == q_out.dtype
    for w in (q_norm_w, k_norm_w):
        assert w is None or (w.dtype == torch.float32 and w.numel() == hd and w.is_contiguous())
    assert rot == 0 or (cs_table.dtype == torch.float32 and cs_table.shape == (n, rot // 2, 2) and cs_table.is_contiguous())
    _check(core().rllm_head_norm_rope_store(
        _ptr(rows), c_int(_code(rows)), c_longlong(rows.stride(0)), _ptr(q_norm_w), _ptr(k_norm_w),
        _ptr(cs_table if rot else None), c_int(rot), c_int(1 if pairs else 0), _ptr(slots), _ptr(q_out), _ptr(k_cache),
        _ptr(v_cache), c_int(_code(q_out)), c_int(n), c_int(H), c_int(G), c_int(hd), c_int(hdv), c_int(block_size),
        c_float(eps), c_int(1 if has_kv else 0), c_int(1 if (write_kv and has_kv) else 0),
        c_longlong(k_cache.shape[0] * block_size), _ptr(error_word(rows.device)), _stream()), "head_norm_rope_store")
    return q_out


def join_norm_rows(y, w_out, eps_out, x, w_next, eps_next, out):
    """x += y / rms(y) * w_out (x: the float32 stream, in place), out = x / rms(x) * w_next in out's type:
    one kernel for the norm on a sublayer's output and the norm in front of the next sublayer.  Rows
    too long for the kernel's shared memory take the two kernels it stands for."""
    _need_cuda(y, w_out, x, w_next, out)
    _need_contig(x=x, out=out, w_out=w_out, w_next=w_next)
    _rows2d(y, "y")
    n, d = x.shape
    assert x.dtype == torch.float32 and y.shape == (n, d) and out.shape == (n, d)
    assert w_out.dtype == w_next.dtype == torch.float32 and w_out.numel() == w_next.numel() == d
    if d * 4 > 48 * 1024:
        norm_rows(y, w_out, eps_out, x=x, add=True)
        return add_rms_norm(x, None, w_next, out, eps_next)
    _check(core().rllm_join_norm_rows(_ptr(y), c_int(_code(y)), c_longlong(y.stride(0)), _ptr(w_out), c_float(eps_out),
                                      _ptr(x), _ptr(w_next), c_float(eps_next), _ptr(out), c_int(_code(out)), c_int(n),
                                      c_int(d), _stream()), "join_norm_rows")
    return out


def latent_rope_store(q, kv, kv_norm_w, cs_table, cs_mult, slots, q_att, cache, H, dq, r, rank, block_size, eps,
                      write_kv=True, pairs=False):
    """Attention through latents, the step between the projections and the attention kernel: kv
    [n, rank + r] (float32, any row stride) -> cache row [normed latent | rotated shared key part];
    q [n, H * (dq + r)] -> the rotated part of every head into q_att[:, h, rank:rank + r].  `pairs`: entry 2i
    turns with 2i + 1 (else i with i + r/2).  See headwise.cu."""
    _need_cuda(q, kv, kv_norm_w, cs_table, slots, q_att, cache)
    _need_contig(q_att=q_att, cache=cache, slots=slots)
    _rows2d(q, "q"), _rows2d(kv, "kv")
    n = q.shape[0]
    assert q.shape[1] == H * (dq + r) and kv.shape == (n, rank + r) and kv.dtype == torch.float32
    assert q_att.shape == (n, H * (rank + r)) and cache.shape[1:] == (1, block_size, rank + r)
    assert cache.dtype == q_att.dtype and slots.dtype == torch.int32 and slots.numel() == n
    assert kv_norm_w.dtype == torch.float32 and kv_norm_w.numel() == rank and kv_norm_w.is_contiguous()
    assert cs_table.dtype == torch.float32 and cs_table.shape == (n, r // 2, 2) and cs_table.is_contiguous()
    _check(core().rllm_latent_rope_store(
        _ptr(q), c_int(_code(q)), c_longlong(q.stride(0)), _ptr(kv), c_longlong(kv.stride(0)), _ptr(kv_norm_w),
        _ptr(cs_table), c_float(cs_mult), _ptr(slots), _ptr(q_att), _ptr(cache), c_int(_code(q_att)), c_int(n),
        c_int(H), c_int(dq), c_int(r), c_int(rank), c_int(block_size), c_float(eps), c_int(1 if write_kv else 0),
        c_longlong(cache.shape[0] * block_size), _ptr(error_word(q.device)), c_int(1 if pairs else 0), _stream()),
        "latent_rope_store")
    return q_att


GLU_GELU_TANH = (0.0, 0.0, 0.0)     # the `glu` triple (limit, alpha, shift) of act = tanh-form gelu: alpha 0 selects it


def glu_clamped(gate_up, out, limit, alpha=1.0, shift=0.0):
    """gate_up [n, 2F] (gate columns, then up columns; float32 or bfloat16) -> out [n, F] =
    g * sigmoid(alpha * g) * (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit)
    (limit 0: no clamp)."""
    _need_cuda(gate_up, out)
    _need_contig(out=out)
    _rows2d(gate_up, "gate_up")
    n, F = out.shape
    assert gate_up.shape == (n, 2 * F)
    _check(core().rllm_glu_clamped(_ptr(gate_up), c_int(_code(gate_up)), c_longlong(gate_up.stride(0)), _ptr(out),
                                   c_int(_code(out)), c_int(n), c_int(F), c_float(limit), c_float(alpha),
                                   c_float(shift), _stream()), "glu_clamped")
    return out


def softcap_rows(x, cap):
    """x = cap * tanh(x / cap) in place (float32)."""
    _need_cuda(x)
    _need_contig(x=x)
    assert x.dtype == torch.float32
    _check(core().rllm_softcap_rows(_ptr(x), c_longlong(x.numel()), c_float(cap), _stream()), "softcap_rows")
    return x


# ------------------------------------------------------------------ row-wise helpers (rowwise.cu)

ACT = {None: 0, "none": 0, "silu": 1, "relu2": 2, "sigmoid": 3, "tanh": 4, "softplus": 5}


def _rows2d(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be a matrix whose rows are contiguous")
    return t


def rows_act(a, out, act=None, bias=None, mul=None, mul_act=None, mul_group=1):
    """out[t, c] = f(a[t, c] + bias[c]) * g(mul[t, c // mul_group]); a, mul, out may be column slices of
    wider matrices (any row stride), float32 or bfloat16; bias float32.  f, g by name (ACT).  mul_group > 1:
    one factor for each run of that many columns (a gate per head)."""
    _need_cuda(a, out, bias, mul)
    _rows2d(a, "a"), _rows2d(out, "out")
    n, cols = out.shape
    assert mul_group >= 1 and cols % mul_group == 0
    assert a.shape == (n, cols) and (mul is None or _rows2d(mul, "mul").shape == (n, cols // mul_group))
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == cols and bias.is_contiguous())
    _check(core().rllm_rows_act(_ptr(a), c_int(_code(a)), c_longlong(a.stride(0)), _ptr(bias), c_int(ACT[act]),
                                _ptr(mul), c_int(_code(mul) if mul is not None else F32),
                                c_longlong(mul.stride(0) if mul is not None else 0), c_int(ACT[mul_act]), _ptr(out),
                                c_int(_code(out)), c_longlong(out.stride(0)), c_int(n), c_int(cols), c_int(mul_group),
                                _stream()), "rows_act")
    return out


def axpby(a, x, b, y, out):
    """out = a * x + b * y over float32 tensors of one shape."""
    _need_cuda(x, y, out)
    _need_contig(x=x, y=y, out=out)
    assert x.dtype == y.dtype == out.dtype == torch.float32 and x.shape == y.shape == out.shape
    _check(core().rllm_axpby(c_float(a), _ptr(x), c_float(b), _ptr(y), _ptr(out), c_longlong(out.numel()),
                             _stream()), "axpby")
    return out


def cat2_cast(x, y, out, delta=None, delta_scale=1.0):
    """out[t] = [x[t] + delta_scale * delta[t] | y[t]]; x, y float32 [n, d], out [n, 2d]."""
    _need_cuda(x, y, out, delta)
    _need_contig(x=x, y=y, out=out, delta=delta)
    n, d = x.shape
    assert x.dtype == y.dtype == torch.float32 and y.shape == (n, d) and out.shape == (n, 2 * d)
    assert delta is None or delta.shape == (n, d)
    _check(core().rllm_cat2_cast(_ptr(x), _ptr(delta), c_int(_code(delta) if delta is not None else F32),
                                 c_float(delta_scale), _ptr(y), _ptr(out), c_int(_code(out)), c_int(n), c_int(d),
                                 _stream()), "cat2_cast")
    return out


def qkv_rownorm_store(qkv, bias, q_norm_w, k_norm_w, slots, q_out, k_cache, v_cache, H, G, dk, dv, block_size, eps,
                      write_kv=True, cs_table=None, rot=0, pairs=False):
    """Biased q/k/v row -> RMSNorm over the whole q row and the whole k row (weights per column, None:
    no norm) -> with `rot` > 0 the first rot entries of every query and key head rotated by the angles of
    cs_table [n, rot/2, 2] (entry i with i + rot/2, or 2i with 2i + 1 when `pairs`) -> queries out, keys and
    values into the paged cache; see rowwise.cu."""
    _need_cuda(qkv, bias, q_norm_w, k_norm_w, slots, q_out, k_cache, v_cache, cs_table)
    assert rot == 0 or (cs_table.dtype == torch.float32 and cs_table.shape == (qkv.shape[0], rot // 2, 2)
                        and cs_table.is_contiguous() and rot % 2 == 0 and rot <= dk)
    _need_contig(q_out=q_out, k_cache=k_cache, v_cache=v_cache, slots=slots)
    _rows2d(qkv, "qkv")                       # may be the leading columns of a wider projection
    n = qkv.shape[0]
    assert qkv.shape[1] == H * dk + G * dk + G * dv and q_out.shape == (n, H * dk)
    assert slots.dtype == torch.int32 and slots.numel() == n
    assert k_cache.shape[1:] == (G, block_size, dk) and v_cache.shape[1:] == (G, block_size, dv)
    assert k_cache.dtype == v_cache.dtype == q_out.dtype
    for w, size in ((bias, qkv.shape[1]), (q_norm_w, H * dk), (k_norm_w, G * dk)):
        assert w is None or (w.dtype == torch.float32 and w.numel() == size and w.is_contiguous())
    _check(core().rllm_qkv_rownorm_store(
        _ptr(qkv), c_int(_code(qkv)), c_longlong(qkv.stride(0)), _ptr(bias), _ptr(q_norm_w), _ptr(k_norm_w),
        _ptr(slots), _ptr(q_out),
        _ptr(k_cache), _ptr(v_cache), c_int(_code(q_out)), c_int(n), c_int(H), c_int(G), c_int(dk), c_int(dv),
        c_int(block_size), c_float(eps), c_int(1 if write_kv else 0), c_longlong(k_cache.shape[0] * block_size),
        _ptr(error_word(qkv.device)), _ptr(cs_table if rot else None), c_int(rot), c_int(1 if pairs else 0), _stream()),
        "qkv_rownorm_store")
    return q_out


# ------------------------------------------------------------------ layers with a state per request (recurrent.cu)

def _state2d(state):
    """The plane of state slots as [slots, floats per slot]."""
    assert state.dtype == torch.float32 and state.is_contiguous() and state.dim() == 2
    return state


def conv_silu(xz, weight, bias, state, conv_off, ctx_seq_ids, cu_q, slots, out, inner):
    """Causal per-channel convolution + silu over columns [0, inner) of xz (float32), reaching back into
    the request's kept inputs at state[slot, conv_off:]; weight [inner, taps] float32."""
    _need_cuda(xz, weight, bias, state, out)
    _rows2d(xz, "xz"), _need_contig(out=out, weight=weight)
    n = xz.shape[0]
    taps = weight.shape[1]
    assert xz.dtype == weight.dtype == torch.float32 and weight.shape[0] == inner and out.shape == (n, inner)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == inner)
    st = _state2d(state)
    assert conv_off + inner * (taps - 1) <= st.shape[1]
    _check(_lib("recur").rllm_conv_silu(_ptr(xz), c_longlong(xz.stride(0)), _ptr(weight), _ptr(bias), _ptr(st),
                                        c_longlong(st.stride(0)), c_longlong(conv_off), _ptr(ctx_seq_ids), _ptr(cu_q),
                                        _ptr(slots), _ptr(out), c_int(_code(out)), c_int(n), c_int(inner), c_int(taps),
                                        _stream()), "conv_silu")
    return out


def selective_scan(x, xz, low, b_off, c_off, dtr, dt_bias, A, D, state, conv_off, cu_q, slots, out, n_requests,
                   inner, N, taps, segments=None):
    """The selective scan over each request's tokens with its state in state[slot, :inner*N]; see
    recurrent.cu.  x, out: activation type [n, inner]; xz, low, dtr float32."""
    _need_cuda(x, xz, low, dtr, dt_bias, A, D, state, out)
    _need_contig(x=x, out=out, dtr=dtr, A=A)
    _rows2d(xz, "xz"), _rows2d(low, "low")
    n = x.shape[0]
    assert x.dtype == out.dtype and x.shape == out.shape == (n, inner) and dtr.shape == (n, inner)
    assert xz.dtype == low.dtype == dtr.dtype == torch.float32 and xz.shape[1] >= 2 * inner
    assert A.shape == (inner, N) and A.dtype == dt_bias.dtype == D.dtype == torch.float32
    assert dt_bias.numel() == inner and D.numel() == inner and max(b_off, c_off) + N <= low.shape[1]
    st = _state2d(state)
    assert conv_off >= inner * N and conv_off + inner * (taps - 1) <= st.shape[1]
    if N > 256:
        raise KernelError(f"state size {N} exceeds the scan kernel's limit of 256")
    sg = segments                              # TimeSegments of the step, or None (defined below)
    carry = decay = None
    if sg is not None:
        carry = torch.empty((sg.n_items, inner * N), dtype=torch.float32, device=out.device)
        decay = torch.empty((sg.n_items, inner), dtype=torch.float32, device=out.device)
    _check(_lib("recur").rllm_selective_scan(
        _ptr(x), c_int(_code(x)), _ptr(xz), c_longlong(xz.stride(0)), _ptr(low), c_longlong(low.stride(0)),
        c_int(b_off), c_int(c_off), _ptr(dtr), _ptr(dt_bias), _ptr(A), _ptr(D), _ptr(st), c_longlong(st.stride(0)),
        c_longlong(conv_off), _ptr(cu_q), _ptr(slots), _ptr(out), c_int(n_requests), c_int(inner), c_int(N),
        c_int(taps), _ptr(sg.t0 if sg else None), _ptr(sg.t1 if sg else None), _ptr(sg.req if sg else None),
        _ptr(sg.flags if sg else None), _ptr(sg.item0 if sg else None), _ptr(sg.items if sg else None),
        c_int(sg.n_items if sg else 0), _ptr(carry), _ptr(decay), _stream()), "selective_scan")
    if sg is not None:
        global _launches
        _launches += 2                         # the local pass and the combine kernel
    return out


def token_shift(h, mu, state, prev_off, seq_ids, cu_q, slots, out):
    """out[s] = h + (previous row - h) * mu[s]; mu float32 [streams, d], out [streams, n, d]; the row
    before a request's first token of the step is state[slot, prev_off:prev_off + d]."""
    _need_cuda(h, mu, state, out)
    _need_contig(h=h, mu=mu, out=out)
    n, d = h.shape
    S = mu.shape[0]
    assert mu.dtype == torch.float32 and mu.shape == (S, d) and out.shape == (S, n, d) and out.dtype == h.dtype
    st = _state2d(state)
    assert prev_off + d <= st.shape[1]
    _check(_lib("recur").rllm_token_shift(_ptr(h), c_int(_code(h)), _ptr(mu), _ptr(st), c_longlong(st.stride(0)),
                                          c_longlong(prev_off), _ptr(seq_ids), _ptr(cu_q), _ptr(slots), _ptr(out),
                                          c_int(n), c_int(d), c_int(S), _stream()), "token_shift")
    return out


def wkv_state_floats(H: int, D: int) -> int:
    """Floats of a request's WKV state (the kernel keeps each head's state padded to a power of two
    and in its threads' order; recurrent.cu).  No device needed."""
    dmax = 32 if D <= 32 else 64 if D <= 64 else 128 if D <= 128 else 256
    return H * dmax * dmax


SEGMENT_TOKENS = 128      # length of a segment when long portions are cut along time
SEGMENT_FROM = 256        # shortest portion that is cut
TIME_SEGMENTS = os.environ.get("RLLM_B200_NO_TIME_SEGMENTS", "0") in ("", "0")


class TimeSegments:
    """The step's requests cut along time for the recurrent kernels (recurrent.cu, TimeSegments): a
    request that brings fewer than SEGMENT_FROM tokens is one item, a longer one several of
    SEGMENT_TOKENS tokens (the last takes the remainder).  Built once per step on the host from the
    step's shape and shared by all layers."""

    def __init__(self, ctx, device):
        t0, t1, req, flags, item0, items = [], [], [], [], [], []
        base = 0
        for r, q in enumerate(ctx.q_lens):
            n = q // SEGMENT_TOKENS if q >= SEGMENT_FROM else 1
            item0.append(len(t0))
            items.append(n)
            for s in range(n):
                t0.append(base + s * SEGMENT_TOKENS)
                t1.append(base + (s + 1) * SEGMENT_TOKENS if s + 1 < n else base + q)
                req.append(r)
                flags.append((1 if s == 0 else 0) | (2 if s + 1 == n else 0))
            base += q
        self.n_items = len(t0)
        flat = torch.tensor(t0 + t1 + req + flags + item0 + items, dtype=torch.int32).to(device)
        n, R = self.n_items, len(items)
        self.t0, self.t1, self.req, self.flags = flat[:n], flat[n:2 * n], flat[2 * n:3 * n], flat[3 * n:4 * n]
        self.item0, self.items = flat[4 * n:4 * n + R], flat[4 * n + R:4 * n + 2 * R]


def time_segments(ctx, device):
    """The step's TimeSegments, or None when no request brings a portion long enough to cut."""
    if not TIME_SEGMENTS or ctx.max_q_len < SEGMENT_FROM:
        return None
    plan = ctx.plans.get("time_segments")
    if plan is None:
        plan = ctx.plans["time_segments"] = TimeSegments(ctx, device)
    return plan


def wkv(r, k, v, wraw, g, w0, u, norm_w, eps, state, prev_off, h, cu_q, slots, out, n_requests, H, D, segments=None):
    """The RWKV recurrence with data-dependent decay, unit norm per head, norm weight and silu gate; see
    recurrent.cu.  r, k, v, wraw, g float32 [n, H*D] (equal row strides); out activation type.
    segments: the step's TimeSegments (long portions are then worked through segment by segment, side
    by side) or None."""
    _need_cuda(r, k, v, wraw, g, w0, u, norm_w, state, h, out)
    n = out.shape[0]
    for name, t in (("r", r), ("k", k), ("v", v), ("wraw", wraw), ("g", g)):
        _rows2d(t, name)
        assert t.dtype == torch.float32 and t.shape == (n, H * D) and t.stride(0) == r.stride(0)
    _need_contig(out=out, h=h, w0=w0, u=u, norm_w=norm_w)
    assert out.shape == (n, H * D) and h.dtype == out.dtype and h.shape[0] == n
    assert w0.dtype == u.dtype == norm_w.dtype == torch.float32
    assert w0.numel() == u.numel() == norm_w.numel() == H * D
    if D > 256:
        raise KernelError(f"head size {D} exceeds the WKV kernel's limit of 256")
    st = _state2d(state)
    assert prev_off >= wkv_state_floats(H, D) and prev_off + h.shape[1] <= st.shape[1]
    sg = segments
    carry = decay = None
    if sg is not None:
        per_head = wkv_state_floats(1, D)
        carry = torch.empty((sg.n_items, H, per_head), dtype=torch.float32, device=out.device)
        decay = torch.empty((sg.n_items, H, int(per_head ** 0.5)), dtype=torch.float32, device=out.device)
    _check(_lib("recur").rllm_wkv(_ptr(r), _ptr(k), _ptr(v), _ptr(wraw), _ptr(g), c_longlong(r.stride(0)), _ptr(w0),
                                  _ptr(u), _ptr(norm_w), c_float(eps), _ptr(st), c_longlong(st.stride(0)),
                                  c_longlong(prev_off), _ptr(h), c_int(_code(h)), c_int(h.shape[1]), _ptr(cu_q),
                                  _ptr(slots), _ptr(out), c_int(n_requests), c_int(H), c_int(D),
                                  _ptr(sg.t0 if sg else None), _ptr(sg.t1 if sg else None), _ptr(sg.req if sg else None),
                                  _ptr(sg.flags if sg else None), _ptr(sg.item0 if sg else None),
                                  _ptr(sg.items if sg else None), c_int(sg.n_items if sg else 0), _ptr(carry),
                                  _ptr(decay), _stream()), "wkv")
    if sg is not None:
        global _launches
        _launches += 2                         # the local pass and the combine kernel
    return out


def retention_state_floats(H: int, dk: int, dv: int) -> int:
    """Floats of a request's retention state (each head's dk x dv state padded to the kernel's tile and in
    its threads' order; recurrent.cu).  No device needed."""
    dkmax = 32 if dk <= 32 else 64 if dk <= 64 else 128 if dk <= 128 else 256
    threads = ((dv + 1) // 2 * 8 + 31) // 32 * 32
    return H * dkmax * (threads // 8 * 2)


GATES = {None: 0, "none": 0, "silu": 1, "sigmoid": 2}


def retention(rows, q_off, k_off, v_off, g_off, cs_table, rot, pairs, key_scale, decay, eps, state, cu_q, slots, out,
              n_requests, H, dk, dv, gate="silu", segments=None):
    """Linear attention with a fixed decay per head over each request's tokens, its state in state[slot];
    see recurrent.cu.  rows: float32 [n, ...] holding q, k ([H*dk] each) and v, gate ([H*dv] each) at the
    given column offsets; decay float32 [H]; out activation type [n, H*dv].  segments: the step's
    TimeSegments or None."""
    _need_cuda(rows, cs_table, decay, state, cu_q, slots, out)
    _rows2d(rows, "rows")
    _need_contig(out=out, decay=decay)
    n = out.shape[0]
    assert rows.dtype == torch.float32 and rows.shape[0] == n and out.shape == (n, H * dv)
    assert decay.dtype == torch.float32 and decay.numel() == H
    assert max(q_off, k_off) + H * dk <= rows.shape[1] and v_off + H * dv <= rows.shape[1]
    assert gate in (None, "none") or g_off + H * dv <= rows.shape[1]
    assert rot == 0 or (cs_table.dtype == torch.float32 and cs_table.shape == (n, rot // 2, 2) and cs_table.is_contiguous())
    if dk > 256 or dv > 256:
        raise KernelError(f"head sizes {dk} x {dv} exceed the retention kernel's limit of 256")
    st = _state2d(state)
    per_head = retention_state_floats(1, dk, dv)
    assert H * per_head <= st.shape[1]
    sg = segments
    carry = torch.empty((sg.n_items, H, per_head), dtype=torch.float32, device=out.device) if sg is not None else None
    base = rows.data_ptr()
    col = lambda off: c_void_p(base + 4 * off)
    _ptr(rows)                                 # a traced launch keeps the rows alive
    _check(_lib("recur").rllm_retention(
        col(q_off), col(k_off), col(v_off), col(g_off) if GATES[gate] else c_void_p(0), c_longlong(rows.stride(0)),
        _ptr(cs_table if rot else None), c_int(rot), c_int(1 if pairs else 0), c_float(key_scale), _ptr(decay),
        c_float(eps), _ptr(st), c_longlong(st.stride(0)), _ptr(cu_q), _ptr(slots), _ptr(out), c_int(_code(out)),
        c_int(n_requests), c_int(H), c_int(dk), c_int(dv), c_int(GATES[gate]),
        _ptr(sg.t0 if sg else None), _ptr(sg.t1 if sg else None), _ptr(sg.req if sg else None),
        _ptr(sg.flags if sg else None), _ptr(sg.item0 if sg else None), _ptr(sg.items if sg else None),
        c_int(sg.n_items if sg else 0), _ptr(carry), _stream()), "retention")
    if sg is not None:
        global _launches
        _launches += 2                         # the local pass and the combine kernel
    return out


def mlstm_state_floats(H: int, dk: int, dv: int) -> int:
    """Floats of a request's matrix-memory state: per head the dk x (dv + 1) memory (the last column is the
    normaliser) padded to the kernel's tile and in its threads' order, then four floats of which the first
    is the running maximum (recurrent.cu).  Heads beyond the fast kernel's sizes (keys over 256 entries, values
    over 254) keep dk x (dv + 1) floats as they are.  No device needed."""
    if dk > 256 or dv > 254:
        return H * (dk * (dv + 1) + 4)
    dkmax = 32 if dk <= 32 else 64 if dk <= 64 else 128 if dk <= 128 else 256
    threads = ((dv + 2) // 2 * 8 + 31) // 32 * 32
    return H * (dkmax * (threads // 8 * 2) + 4)


def mlstm(rows, q_off, k_off, v_off, g_off, i_off, f_off, i_bias, f_bias, cap, q_scale, norm_w, eps, state, cu_q, slots,
          out, n_requests, H, dk, dv, gate="sigmoid", segments=None):
    """The matrix memory with exponential gates and a running maximum over each request's tokens, its
    state in state[slot]; see recurrent.cu.  rows: float32 [n, ...] holding q, k ([H*dk] each), v, gate
    ([H*dv] each) and the two gate pre-activations ([H] each) at the given column offsets; i_bias, f_bias
    float32 [H]; norm_w float32 [H*dv] or None; out activation type [n, H*dv].  cap 0: the gates are not
    capped."""
    _need_cuda(rows, i_bias, f_bias, norm_w, state, cu_q, slots, out)
    _rows2d(rows, "rows")
    _need_contig(out=out)
    n = out.shape[0]
    assert rows.dtype == torch.float32 and rows.shape[0] == n and out.shape == (n, H * dv)
    assert max(q_off, k_off) + H * dk <= rows.shape[1] and v_off + H * dv <= rows.shape[1]
    assert max(i_off, f_off) + H <= rows.shape[1]
    assert gate in (None, "none") or g_off + H * dv <= rows.shape[1]
    for b in (i_bias, f_bias):
        assert b is None or (b.dtype == torch.float32 and b.numel() == H and b.is_contiguous())
    assert norm_w is None or (norm_w.dtype == torch.float32 and norm_w.numel() == H * dv and norm_w.is_contiguous())
    if 2 * dk + dv + 1 > 12288:
        raise KernelError(f"head sizes {dk} x {dv} exceed the matrix-memory kernels' shared memory")
    st = _state2d(state)
    per_head = mlstm_state_floats(1, dk, dv)
    assert H * per_head <= st.shape[1]
    sg = segments if (dk <= 256 and dv <= 254) else None          # the kernel for larger heads is not cut along time
    carry = torch.empty((sg.n_items, H, per_head), dtype=torch.float32, device=out.device) if sg is not None else None
    base = rows.data_ptr()
    col = lambda off: c_void_p(base + 4 * off)
    _ptr(rows)                                 # a traced launch keeps the rows alive
    _check(_lib("recur").rllm_mlstm(
        col(q_off), col(k_off), col(v_off), col(g_off) if GATES[gate] else c_void_p(0), col(i_off), col(f_off),
        c_longlong(rows.stride(0)), _ptr(i_bias), _ptr(f_bias), c_float(cap), c_float(q_scale), _ptr(norm_w),
        c_float(eps), _ptr(st), c_longlong(st.stride(0)), _ptr(cu_q), _ptr(slots), _ptr(out), c_int(_code(out)),
        c_int(n_requests), c_int(H), c_int(dk), c_int(dv), c_int(GATES[gate]),
        _ptr(sg.t0 if sg else None), _ptr(sg.t1 if sg else None), _ptr(sg.req if sg else None),
        _ptr(sg.flags if sg else None), _ptr(sg.item0 if sg else None), _ptr(sg.items if sg else None),
        c_int(sg.n_items if sg else 0), _ptr(carry), _stream()), "mlstm")
    if sg is not None:
        global _launches
        _launches += 2                         # the local pass and the combine kernel
    return out


# ------------------------------------------------------------------ routed experts (moe.cu)

def moe_route(logits, correction, idx, weight, E, top_k, n_groups=1, keep_groups=1, group_best=2, score="sigmoid",
              normalize=True, weight_eps=0.0, route_scale=1.0, bias=None):
    """The router's choice per token from float32 logits (the first E columns of `logits`, plus `bias`
    float32 [E] if given): idx int32 [n, top_k], weight float32 [n, top_k]; see moe.cu."""
    _need_cuda(logits, correction, idx, weight, bias)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == E and bias.is_contiguous())
    _rows2d(logits, "logits")
    _need_contig(idx=idx, weight=weight, correction=correction)
    n = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.shape[1] >= E
    assert idx.dtype == torch.int32 and idx.shape == (n, top_k) and weight.dtype == torch.float32 and weight.shape == (n, top_k)
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == E)
    if score not in ("sigmoid", "softmax"):
        raise KernelError(f"moe_route: score {score!r} is not known")
    if E > 1024:
        raise KernelError(f"{E} experts exceed the router kernel's limit of 1024")
    _check(_lib("moe").rllm_moe_route(_ptr(logits), c_longlong(logits.stride(0)), _ptr(correction), _ptr(idx), _ptr(weight),
                                      c_int(n), c_int(E), c_int(top_k), c_int(n_groups), c_int(keep_groups),
                                      c_int(group_best), c_int(1 if score == "softmax" else 0), c_int(1 if normalize else 0),
                                      c_float(weight_eps), c_float(route_scale), _ptr(bias), _stream()), "moe_route")
    return idx, weight


MOE_EXPERT_ROWS = 1024        # rows of a step the per-expert kernels can list (MOE_LIST in moe.cu)


def _by_expert(x, n, k):
    """Whether the few-row products run expert by expert on the tensor cores (bfloat16, rows of a multiple
    of 8 entries), not pair by pair."""
    return x.dtype == torch.bfloat16 and n <= MOE_EXPERT_ROWS and k % 8 == 0


def moe_pairs_gate_up(h, w_gu, idx, act, glu=(0.0, 1.0, 0.0)):
    """act[t * top_k + j] = glu(Wg[e] h[t], Wu[e] h[t]) with e = idx[t, j]; w_gu [E, 2F, d] (gate rows, then up
    rows); h, w_gu, act of one type.  bfloat16 rows that fit run expert by expert (an expert's matrices are
    read once for eight of its tokens), the rest pair by pair; each way sums in its own fixed order, and which
    way runs depends on types and sizes only, never on the batch."""
    _need_cuda(h, w_gu, idx, act)
    _need_contig(h=h, w_gu=w_gu, idx=idx, act=act)
    n, d = h.shape
    top_k, F = idx.shape[1], act.shape[1]
    assert w_gu.shape[1:] == (2 * F, d) and act.shape == (n * top_k, F) and h.dtype == w_gu.dtype == act.dtype
    if _by_expert(h, n, d):
        _check(_lib("moe").rllm_moe_expert_gate_up(_ptr(h), _ptr(w_gu), _ptr(idx), _ptr(act), c_int(n), c_int(top_k),
                                                   c_int(w_gu.shape[0]), c_int(d), c_int(F), c_float(glu[0]),
                                                   c_float(glu[1]), c_float(glu[2]), _stream()), "moe_expert_gate_up")
        return act
    _check(_lib("moe").rllm_moe_pairs_gate_up(_ptr(h), _ptr(w_gu), c_int(_code(h)), _ptr(idx), _ptr(act), c_int(n),
                                              c_int(top_k), c_int(d), c_int(F), c_float(glu[0]), c_float(glu[1]),
                                              c_float(glu[2]), _stream()), "moe_pairs_gate_up")
    return act


def moe_pairs_down(act, w_down, idx, weight, out, shared=None, gate=None):
    """out[t] = sum_j weight[t, j] * Wd[idx[t, j]] act[t * top_k + j] (+ shared[t] * sigmoid(gate[t]));
    w_down [E, d, F]; out, shared float32 [n, d]; gate: float32 logits, one per token (a column)."""
    _need_cuda(act, w_down, idx, weight, out, shared, gate)
    _need_contig(act=act, w_down=w_down, idx=idx, weight=weight, out=out, shared=shared)
    n, d = out.shape
    top_k, F = idx.shape[1], act.shape[1]
    assert w_down.shape[1:] == (d, F) and act.shape == (n * top_k, F) and act.dtype == w_down.dtype
    assert out.dtype == torch.float32 and (shared is None or (shared.dtype == torch.float32 and shared.shape == (n, d)))
    assert gate is None or (gate.dtype == torch.float32 and gate.shape[0] == n)
    if _by_expert(act, n, F):
        y = torch.empty((n * top_k, d), dtype=torch.float32, device=out.device)
        _check(_lib("moe").rllm_moe_expert_down(_ptr(act), _ptr(w_down), _ptr(idx), _ptr(y), c_int(n), c_int(top_k),
                                                c_int(w_down.shape[0]), c_int(d), c_int(F), _stream()), "moe_expert_down")
        return moe_combine(y, None, weight, out, shared, gate)
    if top_k * F * 4 > 96 * 1024:
        raise KernelError("moe_pairs_down: top_k * expert size exceeds the kernel's shared memory")
    _check(_lib("moe").rllm_moe_pairs_down(_ptr(act), _ptr(w_down), c_int(_code(act)), _ptr(idx), _ptr(weight), _ptr(out),
                                           _ptr(shared), _ptr(gate), c_longlong(gate.stride(0) if gate is not None else 0),
                                           c_int(n), c_int(top_k), c_int(d), c_int(F), _stream()), "moe_pairs_down")
    return out


def moe_sort(idx, E):
    """(offsets int32 [E + 1], place int32 [pairs]): the pairs of idx [n, top_k] in expert order (stable)."""
    _need_cuda(idx)
    _need_contig(idx=idx)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=idx.device)
    place = torch.empty(idx.numel(), dtype=torch.int32, device=idx.device)
    _check(_lib("moe").rllm_moe_sort(_ptr(idx), c_int(idx.numel()), c_int(E), _ptr(offsets), _ptr(place), _stream()),
           "moe_sort")
    return offsets, place


def moe_gather_rows(h, place, rows, top_k):
    """rows[place[p]] = h[p // top_k] for every pair p."""
    _need_cuda(h, place, rows)
    _need_contig(h=h, place=place, rows=rows)
    assert rows.shape == (place.numel(), h.shape[1]) and rows.dtype == h.dtype
    _check(_lib("moe").rllm_moe_gather_rows(_ptr(h), c_int(_code(h)), _ptr(place), _ptr(rows), c_int(place.numel()),
                                            c_int(top_k), c_int(h.shape[1]), _stream()), "moe_gather_rows")
    return rows


def moe_combine(y, place, weight, out, shared=None, gate=None):
    """out[t] = sum_j weight[t, j] * y[place[t * top_k + j]] (+ shared[t] * sigmoid(gate[t])), float32;
    place None: y holds the pairs in their own order."""
    _need_cuda(y, place, weight, out, shared, gate)
    _need_contig(y=y, place=place, weight=weight, out=out, shared=shared)
    n, d = out.shape
    top_k = weight.shape[1]
    assert y.dtype == out.dtype == torch.float32 and y.shape == (n * top_k, d)
    assert shared is None or (shared.dtype == torch.float32 and shared.shape == (n, d))
    _check(_lib("moe").rllm_moe_combine(_ptr(y), _ptr(place), _ptr(weight), _ptr(out), _ptr(shared), _ptr(gate),
                                        c_longlong(gate.stride(0) if gate is not None else 0), c_int(n), c_int(top_k),
                                        c_int(d), _stream()), "moe_combine")
    return out


# ------------------------------------------------------------------ matrix products

def gemm_plain(a, w, out, accumulate=False):
    """out[m,n] (+)= a[m,k] . w[n,k]^T with float32 multiply-add on the CUDA cores."""
    _need_cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if accumulate and out.dtype != torch.float32:
        raise KernelError("accumulating product needs a float32 output")
    _check(core().rllm_gemm_plain(_ptr(a), c_int(_code(a)), _ptr(w), c_int(_code(w)), _ptr(out),
                                  c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
                                  c_int(w.stride(0)), c_int(out.stride(0)), c_int(1 if accumulate else 0),
                                  _stream()), "gemm_plain")
    return out


def head_linear(a, w, out):
    """One product per head: out[t, h, :] = w[h] . a[t, h, :] for a [n, H, k], w [H, m, k], out [n, H, m].
    `a` and `out` may be views into wider rows (a head's columns inside a token's row); their last
    axis is contiguous.  float32 operands take the plain product, bfloat16 the library's strided batch
    (float32 accumulation in both)."""
    _need_cuda(a, w, out)
    n, H, k = a.shape
    m = w.shape[1]
    assert w.shape == (H, m, k) and w.is_contiguous() and out.shape == (n, H, m)
    assert a.stride(2) == 1 and out.stride(2) == 1
    if n == 0:
        return out
    lib_ok = (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 8 == 0 and a.stride(0) % 8 == 0
              and a.stride(1) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
              and out.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0 and out.stride(1) % 8 == 0)
    if lib_ok:
        st = _lib("blas").rllm_gemm_lib_batched(
            _ptr(a), _ptr(w), _ptr(out), c_int(_code(out)), c_int(n), c_int(m), c_int(k), c_int(a.stride(0)), c_int(k),
            c_int(out.stride(0)), c_int(H), c_longlong(a.stride(1)), c_longlong(m * k), c_longlong(out.stride(1)),
            _stream())
        if st >= 10000:
            raise KernelError(f"head_linear: cuBLAS status {st - 10000} for {H} products of m={n} n={m} k={k}")
        _check(st, "gemm_lib_batched", own=False)
        return out
    if a.dtype != w.dtype:
        raise KernelError(f"head_linear: activation {a.dtype} and weight {w.dtype} differ")
    _check(core().rllm_gemm_plain_batched(
        _ptr(a), c_int(_code(a)), _ptr(w), c_int(_code(w)), _ptr(out), c_int(_code(out)), c_int(n), c_int(m), c_int(k),
        c_int(a.stride(0)), c_int(k), c_int(out.stride(0)), c_int(0), c_int(H), c_longlong(a.stride(1)),
        c_longlong(m * k), c_longlong(out.stride(1)), _stream()), "gemm_plain_batched")
    return out


# ------------------------------------------------------------------ sampling

def logit_adjust(logits, index, delta):
    """logits.view(-1)[index[i]] += delta[i] in place (float32 logits, int64 index, float32 delta on
    the device; the positions must be distinct)."""
    _need_cuda(logits, index, delta)
    assert logits.dtype == torch.float32 and index.dtype == torch.int64 and delta.dtype == torch.float32
    assert index.numel() == delta.numel() and index.is_contiguous() and delta.is_contiguous()
    _check(core().rllm_logit_adjust(_ptr(logits), _ptr(index), _ptr(delta), c_int(index.numel()), _stream()),
           "logit_adjust")
    return logits


def sample_rows(logits, out_ids, temperature=None, top_k=None, top_p=None, seed=None, counter=None):
    """One token id per row of float32 logits [rows, vocab]; all parameter arrays are per row
    (float32, int32, float32, int64, int64) or None (greedy)."""
    _need_cuda(logits, out_ids, temperature, top_k, top_p, seed, counter)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert out_ids.dtype == torch.int32 and out_ids.numel() == rows
    for t, dt in ((temperature, torch.float32), (top_k, torch.int32), (top_p, torch.float32),
                  (seed, torch.int64), (counter, torch.int64)):
        assert t is None or (t.dtype == dt and t.numel() == rows and t.is_contiguous())
    if vocab >= 1 << 24:
        raise KernelError(f"vocabulary {vocab} exceeds the sampler's limit of 2^24 - 1")
    _check(core().rllm_sample_rows(_ptr(logits), c_longlong(logits.stride(0)), c_int(rows), c_int(vocab),
                                   _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(seed), _ptr(counter),
                                   _ptr(out_ids), _stream()), "sample_rows")
    return out_ids


# ------------------------------------------------------------------ library product and dispatch

def gemm_lib(a, w, out, accumulate=False):
    """out[m,n] (+)= a[m,k] . w[n,k]^T through cuBLAS: bfloat16 operands, float32 accumulation."""
    _need_cuda(a, w, out)
    m, k = a.shape
    n = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert w.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    st = _lib("blas").rllm_gemm_lib(_ptr(a), _ptr(w), _ptr(out), c_int(_code(out)), c_int(m), c_int(n),
                                          c_int(k), c_int(a.stride(0)), c_int(w.stride(0)),
                                          c_int(out.stride(0)), c_int(1 if accumulate else 0), _stream())
    if st >= 10000:
        raise KernelError(f"gemm_lib: cuBLAS status {st - 10000} for m={m} n={n} k={k}")
    _check(st, "gemm_lib", own=False)
    return out


EPI_STORE, EPI_ACCUM, EPI_SWIGLU = 0, 1, 2
SKINNY_MAX_ROWS = 64


def _skinny_ok(a, w) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] <= SKINNY_MAX_ROWS
            and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_gemm(a, w, out, epilogue=EPI_STORE, up_row_offset=0, then_norm=None):
    """out (+)= a . w^T for at most 64 rows of a, streaming w once (tensor-core kernel for decode).
    epilogue EPI_SWIGLU: w holds gate rows then (from up_row_offset) up rows; out[b, j] =
    silu(gate_j) * up_j with out [m, n], n = number of gate rows.
    `a` as NormedRows and `then_norm`: as for gemv_stream."""
    scale = a if isinstance(a, NormedRows) else None
    if scale is not None:
        a = scale.xw
    _need_cuda(a, w, out)
    if not _skinny_ok(a, w):
        raise KernelError("skinny_gemm needs bfloat16 operands, at most 64 rows, k a multiple of 8 and "
                          "16-byte aligned rows")
    m, k = a.shape
    n = out.shape[1]
    assert out.shape[0] == m and out.stride(1) == 1
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] >= up_row_offset + n
    else:
        assert w.shape[0] == n
    xw, w_next, ssq_out, cols, eps_next = _norm_producer(then_norm, epilogue, scale, m, n, -(-n // 16),
                                                         16 if m <= 16 else 64, a.device, "skinny_gemm")
    _check(_lib("fast").rllm_skinny_gemm(
        _ptr(w), _ptr(a), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(w.stride(0)),
        c_int(a.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset),
        _ptr(xw), c_int(n), _ptr(w_next), _ptr(ssq_out), *_norm_consumer(scale, epilogue, m, "skinny_gemm"), _stream()),
        "skinny_gemm")
    if then_norm is not None:
        return NormedRows(xw, ssq_out, -(-n // 16), n, eps_next, cols=cols)
    return out


def _norm_producer(then_norm, epilogue, scale, m, n, n_parts, cols, device, who):
    """Buffers of the producing side of a deferred norm: (xw, norm weight, parts, columns of a part, eps)."""
    if then_norm is None:
        return None, None, None, cols, 0.0
    if epilogue != EPI_ACCUM or scale is not None:
        raise KernelError(f"{who}: then_norm goes with the accumulate epilogue")
    w_next, eps_next = then_norm
    assert w_next.dtype == torch.float32 and w_next.numel() == n and w_next.is_contiguous()
    xw = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    ssq_out = torch.empty((max(n_parts, 1), cols), dtype=torch.float32, device=device)
    return xw, w_next, ssq_out, cols, float(eps_next)


def _norm_consumer(scale, epilogue, m, who):
    """Arguments of the consuming side of a deferred norm: parts, their number and width, d, eps."""
    if scale is None:
        return _ptr(None), c_int(0), c_int(0), c_int(0), c_float(0.0)
    if epilogue == EPI_ACCUM:
        raise KernelError(f"{who}: rows with a deferred norm go with the store and SwiGLU epilogues")
    if scale.cols < m:
        raise KernelError(f"{who}: parts of {scale.cols} columns for {m} rows")
    return _ptr(scale.ssq), c_int(scale.n_parts), c_int(scale.cols), c_int(scale.d), c_float(scale.eps)


_error_words: dict = {}
ERROR_CODES_RANGE = {4: "a token id outside the vocabulary", 5: "a cache slot outside the pool",
                     6: "a page outside the pool"}


def error_word(device) -> torch.Tensor:
    """The device int into which kernels with bounded waits write a code when a wait runs out."""
    key = torch.device(device).index or 0
    if key not in _error_words:
        _error_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_words[key]


def check_device_errors(device="cuda:0") -> None:
    """Raises if a kernel reported a fault it caught itself: a bounded wait that ran out, or an
    index that its range check refused (reads one int from the device)."""
    code = int(error_word(device).item())
    if code:
        error_word(device).zero_()
        if code in ERROR_CODES_RANGE:
            raise KernelError(f"a kernel refused an index (code {code}: {ERROR_CODES_RANGE[code]}); the access was "
                              f"skipped, the step's results are not to be used")
        raise KernelError(f"a kernel's bounded wait ran out (code {code}: 1 operand tiles never arrived, "
                          f"2 a stage was never released, 3 the accumulator never completed)")


_WAIT_LIBRARIES = {"tc": "rllm_tc", "tc2": "rllm_tc2", "stream": "rllm_stream", "attn_tc": "rllm_attn_tc"}


def set_wait_cycles(cycles: int = 0, libraries=None) -> None:
    """Limit, in clock cycles, of every bounded wait (mbarrier polls) in the kernels of the TMA
    libraries; 0 restores the default of about a second."""
    for name in (libraries or _WAIT_LIBRARIES):
        fn = getattr(_lib(name), _WAIT_LIBRARIES[name] + "_set_wait_cycles")
        fn.argtypes = [c_longlong]
        _check(fn(c_longlong(int(cycles))), f"set_wait_cycles({name})", own=False)


def wait_probe(library: str, code: int, device="cuda:0") -> None:
    """Launches the library's probe kernel: one thread waits, with the library's limit, on an
    mbarrier at which nothing arrives, gives up, writes `code` to the error word and returns."""
    fn = getattr(_lib(library), _WAIT_LIBRARIES[library] + "_wait_probe")
    with torch.cuda.device(device):
        _check(fn(_ptr(error_word(device)), c_int(code), _stream()), f"wait_probe({library})")


def _tc_ok(a, w, _meta=False) -> bool:
    """_meta: `a` stands for a freshly allocated activation (contiguous, aligned)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and (_meta or a.data_ptr() % 16 == 0) and w.data_ptr() % 16 == 0)


def gemm_tc(a, w, out, epilogue=EPI_STORE, up_row_offset=0, glu=None):
    """out (+)= a . w^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory).
    epilogue as for skinny_gemm; glu = (limit, alpha, shift): the gated epilogue's constants (None:
    SwiGLU).  See gemm_tc.cu."""
    _need_cuda(a, w, out)
    if not _tc_ok(a, w):
        raise KernelError("gemm_tc needs bfloat16 operands, k a multiple of 8 and 16-byte aligned rows")
    m, k = a.shape
    n = out.shape[1]
    assert out.shape[0] == m and out.stride(1) == 1
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] >= up_row_offset + n
    else:
        assert w.shape[0] == n
    limit, alpha, shift = glu or (0.0, 1.0, 0.0)
    st = _lib("tc").rllm_gemm_tc_glu(
        _ptr(a), _ptr(w), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
        c_int(w.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset), c_float(limit),
        c_float(alpha), c_float(shift), _ptr(error_word(a.device)), _stream())
    if st >= 30000:
        raise KernelError(f"gemm_tc: tensor map encoding failed (CUresult {st - 30000}) for m={m} n={n} k={k}")
    _check(st, "gemm_tc")
    return out


def gemm_tc2(a, w, out, epilogue=EPI_STORE, up_row_offset=0, glu=None):
    """out (+)= a . w^T on the tcgen05 tensor cores with two SMs per 256 x 256 tile
    (tcgen05.mma.cta_group::2; each CTA of the pair stages half of the operands).  Arguments as
    gemm_tc.  See gemm_tc2.cu."""
    _need_cuda(a, w, out)
    if not _tc_ok(a, w):
        raise KernelError("gemm_tc2 needs bfloat16 operands, k a multiple of 8 and 16-byte aligned rows")
    m, k = a.shape
    n = out.shape[1]
    assert out.shape[0] == m and out.stride(1) == 1
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] >= up_row_offset + n
    else:
        assert w.shape[0] == n
    limit, alpha, shift = glu or (0.0, 1.0, 0.0)
    st = _lib("tc2").rllm_gemm_tc2_glu(
        _ptr(a), _ptr(w), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
        c_int(w.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset), c_float(limit),
        c_float(alpha), c_float(shift), _ptr(error_word(a.device)), _stream())
    if st >= 30000:
        raise KernelError(f"gemm_tc2: tensor map encoding failed (CUresult {st - 30000}) for m={m} n={n} k={k}")
    _check(st, "gemm_tc2")
    return out


# From this many rows on the fused projection is at least as fast as the library product followed by the q/k
# norm + rotary kernel (us, library + kernel / fused; 8B sizes: 1,024 rows 46.6 / 46.1, 1,536 rows 64.4 / 58.2,
# 2,048 rows 90.1 / 78.1; 0.6B sizes: 512 rows 10.9 / 12.5, 1,024 rows 20.8 / 19.0; 32B sizes: 2,048 rows 170 / 147)
QKV_FUSED_MIN_ROWS = 1024
USE_QKV_FUSED = os.environ.get("RLLM_B200_NO_QKV_FUSED", "0") in ("", "0")


def can_fuse_qkv(h, w_qkv, hd: int, q_out, k_cache) -> bool:
    """Whether qkv_norm_rope_store_fused takes this step: a prompt step of many rows, bfloat16
    throughout, head size 64 or 128."""
    return (USE_QKV_FUSED and isinstance(h, torch.Tensor) and h.shape[0] >= QKV_FUSED_MIN_ROWS and hd in (64, 128)
            and _tc_ok(h, w_qkv) and q_out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and q_out.is_contiguous() and q_out.data_ptr() % 16 == 0)


def qkv_norm_rope_store_fused(h, w_qkv, q_norm_w, k_norm_w, cs_table, slots, q_out, k_cache, v_cache, H, K, hd,
                              block_size, eps, write_kv=True):
    """q_out, caches <- norm / rotary / store of h . w_qkv^T, in one kernel: the two-SM tcgen05 product
    with qk_norm_rope_store's work in its epilogue (gemm_tc2.cu); the float32 projection is never
    written.  Arguments as qk_norm_rope_store with a table of angles (or None)."""
    _need_cuda(h, w_qkv, q_out, k_cache, v_cache, slots)
    n = h.shape[0]
    if not _tc_ok(h, w_qkv) or hd not in (64, 128) or w_qkv.shape[0] != (H + 2 * K) * hd:
        raise KernelError("qkv_norm_rope_store_fused needs bfloat16 operands with 16-byte aligned rows, head size 64 "
                          "or 128 and the stacked q, k, v projections")
    assert q_out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16
    assert q_out.shape == (n, H * hd) and q_out.is_contiguous() and slots.dtype == torch.int32 and slots.numel() >= n
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape[-1] == hd
    if cs_table is not None:
        assert cs_table.dtype == torch.float32 and cs_table.numel() >= n * hd and cs_table.is_contiguous()
    for nw in (q_norm_w, k_norm_w):
        assert nw is None or (nw.dtype == torch.float32 and nw.numel() == hd and nw.is_contiguous())
    n_slots = k_cache.numel() // (K * hd)
    st = _lib("tc2").rllm_qkv_tc2(
        _ptr(h), _ptr(w_qkv), c_int(n), c_int(h.shape[1]), c_int(h.stride(0)), c_int(w_qkv.stride(0)), _ptr(q_out),
        _ptr(k_cache), _ptr(v_cache), _ptr(slots), _ptr(cs_table), _ptr(q_norm_w), _ptr(k_norm_w), c_int(H), c_int(K),
        c_int(hd), c_int(block_size), c_float(eps), c_int(1 if write_kv else 0), c_longlong(n_slots),
        _ptr(error_word(h.device)), _stream())
    if st >= 30000:
        raise KernelError(f"qkv_norm_rope_store_fused: tensor map encoding failed (CUresult {st - 30000})")
    _check(st, "qkv_norm_rope_store_fused")
    return q_out


def tc_swap_splits(n_tiles: int, k: int, swiglu: bool = False, n_sm: int = 148) -> int:
    """Number of K splits (CTAs of a cluster) for the swapped tcgen05 product, a power of two up to
    8 (clusters of 3, 5, 6, 7 CTAs schedule badly) that leaves every CTA at least 4 blocks of 64
    along K.  Plain products: as many as keep the CTAs under 1.6 per SM: above one per SM two CTAs
    share an SM, one streaming while the other starts or ends, and the cluster's CTAs share the
    additions and the writes.  (Measured at 24 and 64 rows on the layer sizes of Qwen3-0.6B, 8B and
    32B: 48 tiles take 4 splits, 32 take 4, 40 take 4, 8 take 8.)  SwiGLU, where the cluster's
    leader adds and writes alone: at most one CTA per SM."""
    nkb = -(-k // 64)
    if swiglu:
        limit = min(n_sm // n_tiles, nkb // 8)
    else:
        limit = min(int(1.6 * n_sm) // n_tiles, nkb // 4)
    limit = max(1, min(limit, 8))
    splits = 1
    while splits * 2 <= limit:
        splits *= 2
    return splits


def skinny_gemm_tc(a, w, out, epilogue=EPI_STORE, up_row_offset=0, n_splits=None, then_norm=None):
    """out (+)= a . w^T for at most 64 rows of a on the tcgen05 tensor cores with the weights as
    the streamed M operand (TMA ring), the K range split over the CTAs of a cluster where the weight
    matrix has few rows.  `a` as NormedRows and `then_norm`: as for gemv_stream (parts of 64 columns)."""
    scale = a if isinstance(a, NormedRows) else None
    if scale is not None:
        a = scale.xw
    _need_cuda(a, w, out)
    if not _tc_ok(a, w) or a.shape[0] > 64:
        raise KernelError("skinny_gemm_tc needs bfloat16 operands, at most 64 rows, k a multiple of 8 and "
                          "16-byte aligned rows")
    m, k = a.shape
    n = out.shape[1]
    assert out.shape[0] == m and out.stride(1) == 1
    rows_out = 64 if epilogue == EPI_SWIGLU else 128
    n_tiles = -(-n // rows_out)
    if n_splits is None:
        n_splits = tc_swap_splits(n_tiles, k, epilogue == EPI_SWIGLU, sm_count(a.device))
    n_splits = max(1, min(int(n_splits), 8))
    xw, w_next, ssq_out, cols, eps_next = _norm_producer(then_norm, epilogue, scale, m, n, n_tiles * n_splits,
                                                         TC_SWAP_NORM_COLS, a.device, "skinny_gemm_tc")
    st = _lib("tc").rllm_gemm_tc_swap(
        _ptr(w), _ptr(a), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(w.stride(0)),
        c_int(a.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset), c_int(n_splits),
        _ptr(error_word(a.device)), _ptr(xw), c_int(n), _ptr(w_next), _ptr(ssq_out),
        *_norm_consumer(scale, epilogue, m, "skinny_gemm_tc"), _stream())
    if st >= 30000:
        raise KernelError(f"skinny_gemm_tc: tensor map encoding failed (CUresult {st - 30000})")
    _check(st, "skinny_gemm_tc")
    if then_norm is not None:
        return NormedRows(xw, ssq_out, n_tiles * n_splits, n, eps_next, cols=cols)
    return out


STREAM_MAX_ROWS = 16
TC_SWAP_NORM_COLS = 64            # columns of a part of sums of squares that skinny_gemm_tc writes and reads
# a norm between two products of at most 64 rows is deferred into them (RLLM_B200_NO_DEFER_NORMS=1: never)
DEFER_NORMS = os.environ.get("RLLM_B200_NO_DEFER_NORMS", "0") in ("", "0")
_n_sm: dict = {}


def sm_count(device=None) -> int:
    """Number of SMs of the device (148 on a B200), looked up once."""
    key = torch.device(device).index if device is not None else torch.cuda.current_device()
    key = key or 0
    if key not in _n_sm:
        _n_sm[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _n_sm[key]


def stream_plan(n: int, k: int, swiglu: bool = False, n_sm: int = 148):
    """(CTAs, ring stages) of gemv_stream for n output rows: three CTAs of three stages per SM when
    each still gets three and more boxes of 8 rows, else two (measured inside the decode step of
    the 8B layer sizes: 444 x 3 for gate/up and the LM head, 296 x 3 for QKV, O and down)."""
    boxes = -(-n // 8) * (2 if swiglu else 1)
    per_sm = 3 if boxes >= 3 * 3 * n_sm else 2
    return per_sm * n_sm, 3


class NormedRows:
    """Rows of the residual stream on their way through an RMSNorm whose division has not happened
    yet: `xw` = bfloat16(x * norm weight) [m, d] and, per row, `n_parts` partial sums of squares of x
    (`ssq` [n_parts, cols] float32, row b in column b).  The product that takes them as its input
    multiplies its result rows by 1 / sqrt(sum / d + eps):  (x w r) . W^T = r ((x w) . W^T).
    Made by an accumulating launch of one of the few-row kernels (`then_norm`; gemv_stream and
    skinny_gemm up to 16 rows write parts of 16 columns, skinny_gemm above that and skinny_gemm_tc
    parts of 64), taken by `linear` and `gate_up_swiglu` in place of a tensor; each of the three
    kernels reads parts of either width."""
    __slots__ = ("xw", "ssq", "n_parts", "d", "eps", "cols")

    def __init__(self, xw, ssq, n_parts, d, eps, cols=16):
        self.xw, self.ssq, self.n_parts, self.d, self.eps, self.cols = xw, ssq, n_parts, d, eps, cols

    @property
    def shape(self):
        return self.xw.shape

    @property
    def dtype(self):
        return self.xw.dtype

    @property
    def device(self):
        return self.xw.device


def gemv_stream(a, w, out, epilogue=EPI_STORE, up_row_offset=0, grid=None, stages=None, then_norm=None):
    """out (+)= a . w^T for at most 16 rows of `a`: persistent CTAs stream their shares of w's rows
    through TMA rings (mma.sync consumers).  Epilogues as skinny_gemm.  grid, stages: number of CTAs
    and ring depth (3, 5 or 10); by default from stream_plan.
    `a` may be NormedRows (store and SwiGLU epilogues): the result rows are divided by the rows' rms.
    then_norm = (norm weight [n] float32, eps), accumulate epilogue only: the launch also prepares
    the RMSNorm of the sums it writes and returns them as NormedRows (else it returns `out`)."""
    scale = a if isinstance(a, NormedRows) else None
    if scale is not None:
        a = scale.xw
    _need_cuda(a, w, out)
    m, k = a.shape
    n = out.shape[1]
    if m > STREAM_MAX_ROWS or k % 64 or not _tc_ok(a, w):
        raise KernelError("gemv_stream: needs at most 16 rows, k % 64 == 0, bfloat16 operands with 16-byte aligned rows")
    if epilogue == EPI_SWIGLU:
        assert w.shape[0] >= up_row_offset + n
    else:
        assert w.shape[0] == n
    assert out.stride(1) == 1 and w.shape[1] == k
    plan = stream_plan(n, k, epilogue == EPI_SWIGLU, sm_count(a.device))
    n_ctas = plan[0] if grid is None else grid
    n_parts = c_int(0)
    xw, w_next, ssq_out, cols, eps_next = _norm_producer(then_norm, epilogue, scale, m, n, n_ctas, 16, a.device,
                                                         "gemv_stream")
    st = _lib("stream").rllm_gemv_stream(
        _ptr(w), _ptr(a), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k), c_int(w.stride(0)),
        c_int(a.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_int(up_row_offset),
        c_int(n_ctas), c_int(plan[1] if stages is None else stages),
        _ptr(error_word(a.device)), _ptr(xw), c_int(n), _ptr(w_next), _ptr(ssq_out), ctypes.byref(n_parts),
        *_norm_consumer(scale, epilogue, 16, "gemv_stream"), _stream())
    _check(st, "gemv_stream")
    if then_norm is not None:
        return NormedRows(xw, ssq_out, n_parts.value, n, eps_next, cols=cols)
    return out


USE_STREAM = True
STREAM_MIN_WEIGHTS = 1 << 23      # below 16 MB of weights the short-lived CTAs of skinny_gemm start faster,
STREAM_MIN_WEIGHTS_4_ROWS = 1 << 21   # but with 4 to 8 rows the norm kernels that gemv_stream saves count for more
                                  # (decode step at the 0.6B layer sizes, all four products of 4 to 12 MB on
                                  # gemv_stream against skinny_gemm: batch 1 -0.5 %, 2 -1.4 %, 4 +2.5 %, 8 +6.8 %)


def _stream_ok(a, w, _meta=False) -> bool:
    return USE_STREAM and a.shape[0] <= 8 and a.shape[1] % 64 == 0 and _tc_ok(a, w, _meta)


def _prefer_stream(a, w, n: int, swiglu: bool = False, _meta=False) -> bool:
    """gemv_stream takes up to 8 rows always, and 9 to 16 rows for the layer's plain products; with
    9 to 16 rows the gate/up product and the LM head are faster on the tcgen05 kernel (measured
    inside the decode step at batch 9, 12 and 16: 3 to 7 % of the step)."""
    m, k = a.shape
    least = STREAM_MIN_WEIGHTS_4_ROWS if 4 <= m <= 8 else STREAM_MIN_WEIGHTS
    if not USE_STREAM or k % 64 or n * k < least or not _tc_ok(a, w, _meta):
        return False
    return m <= 8 or (m <= STREAM_MAX_ROWS and not swiglu and n * k < (1 << 27))


def _prefer_tc_swap(m: int, n: int, k: int, swiglu: bool = False) -> bool:
    """Measured crossover between the two few-row kernels (B200, Qwen3-8B shapes).  The mma.sync
    kernel wins on the small per-layer matrices up to 8 rows (1.5-3 us less fixed cost); the
    tcgen05 kernel wins wherever there are more rows to multiply: everything above 16 rows, and all
    but the smallest matrix between 9 and 16 rows."""
    if k < 512 or n < 512:
        return False                      # tiny models: the fixed cost of TMEM and TMA set-up dominates
    if m <= 8:
        return False                      # (gate/up alone is 2.5 us faster on tcgen05, but not inside a decode step)
    if m <= 16:
        return n * k > 4096 * 4096
    return True


class Preceding:
    """The product launched directly before another one: its activation, its weight matrix and
    whether it was the fused gate/up product.  Handed to `linear` as `follow`, so that the second
    product takes the kernel family of the first where the shape allows it."""
    __slots__ = ("a", "w", "swiglu")

    def __init__(self, a, w, swiglu=False):
        self.a, self.w, self.swiglu = a, w, swiglu

    def took_stream(self) -> bool:
        return (self.a.dtype == torch.bfloat16
                and _prefer_stream(self.a, self.w, self.w.shape[0], swiglu=self.swiglu))


def defers_norm(m: int, w_before, w_after, swiglu_after: bool = False, w_lead=None, swiglu_lead: bool = False) -> bool:
    """Whether the RMSNorm between the accumulating product with `w_before` and the product with
    `w_after` can do without a kernel of its own at `m` rows: both products then run on one of the
    few-row kernels (gemv_stream, skinny_gemm, skinny_gemm_tc; `linear` and `gate_up_swiglu` choose
    as always), the first preparing the norm (`then_norm`), the second dividing by the rms
    (NormedRows).  The three kernels write and read the same parts of sums of squares, so any of
    them may stand on either side.  (w_lead, swiglu_lead, swiglu_after: what the caller knows of the
    products around; the answer does not depend on them.)"""
    if not DEFER_NORMS or not 0 < m <= SKINNY_MAX_ROWS:
        return False
    return all(w.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[1] % 8 == 0 and w.stride(0) % 8 == 0
               and w.stride(1) == 1 and w.data_ptr() % 16 == 0 for w in (w_before, w_after))


def linear(a, w, out=None, out_dtype=None, accumulate=False, stream=None, follow=None, then_norm=None):
    """out (+)= a . w^T, choosing the kernel by element type and shape.

    float32 operands always take the plain CUDA-core product (the true 32-bit path).
    bfloat16 operands: up to 64 rows take the weight-streaming tensor-core kernel, more rows the
    library product; shapes neither can take (a row length that is not a multiple of 8
    elements) take the plain product with the same operand types."""
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        if accumulate:
            raise KernelError("linear: accumulate needs an output to add to")
        out = torch.empty((m, n), dtype=out_dtype or a.dtype, device=a.device)
    if m == 0:
        return out
    rows = a.xw if isinstance(a, NormedRows) else a          # what the rules below look at
    if rows.dtype == torch.float32 or w.dtype == torch.float32:
        if rows.dtype != w.dtype:
            raise KernelError(f"linear: activation {rows.dtype} and weight {w.dtype} differ")
        return gemm_plain(a, w, out, accumulate)
    if follow is not None and stream is None and follow.took_stream():
        stream = True
    if _skinny_ok(rows, w):
        # stream: the wish for the kernel family (a product that follows a gemv_stream launch directly
        # should be one too, whatever its size: a launch of short-lived CTAs right behind the persistent
        # ones is slow), where the shape allows it; `follow` describes the product before and decides it
        epilogue = EPI_ACCUM if accumulate else EPI_STORE
        want_stream = _prefer_stream(rows, w, n) if stream is None else (stream and _stream_ok(rows, w))
        if want_stream:
            return gemv_stream(a, w, out, epilogue, then_norm=then_norm)
        if _prefer_tc_swap(m, n, k) and out.data_ptr() % 16 == 0:
            return skinny_gemm_tc(a, w, out, epilogue, then_norm=then_norm)
        return skinny_gemm(a, w, out, epilogue, then_norm=then_norm)
    if isinstance(a, NormedRows) or then_norm is not None:
        raise KernelError("linear: a deferred norm needs a product that one of the few-row kernels takes "
                          "(ask defers_norm first)")
    aligned = (a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
               and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
               and out.stride(0) % (4 if out.dtype == torch.float32 else 8) == 0)
    if aligned:
        return gemm_lib(a, w, out, accumulate)
    return gemm_plain(a, w, out, accumulate)


def _prefer_tc2(m: int, n_col_tiles: int, n_sm: int = 148) -> bool:
    """Which of the two many-row kernels finishes the product in fewer waves: the one-CTA kernel
    walks 128-row tiles on n_sm CTAs, the two-SM kernel 256-row tiles on n_sm / 2 pairs, whose wave
    takes 0.93 of the other's (2,048 x 24,576 x 4,096: 270 us against 290 in 11 waves each).
    Measured at 12,288 x 4,096 with SwiGLU: 544 rows 116 us (two SMs) against 121, 672 rows 118
    against 128, 896 rows 160 against 141, 1,152 rows 185 against 171."""
    if not USE_TC2:
        return False
    tiles128 = -(-m // 128)
    waves_one = -(-(tiles128 * n_col_tiles) // n_sm)
    waves_two = -(-(-(-tiles128 // 2) * n_col_tiles) // (n_sm // 2))
    return 0.93 * waves_two < waves_one


USE_TC2 = True


def gate_up_swiglu(h, w_gate_up, out, glu=None):
    """out[m, F] = silu(h . Wg^T) * (h . Wu^T) with w_gate_up = [Wg; Wu] stacked ([2F, k]).
    bfloat16: one kernel (the weight-streaming kernel up to 64 rows, the tcgen05 kernel above);
    float32 and odd shapes: a product followed by the activation kernel.
    glu = (limit, alpha, shift): another gated form, g sigmoid(alpha g) (u + shift) with g = min(gate,
    limit), u = clamp(up, -limit, limit); the tcgen05 kernels take it in their epilogue, fewer rows and
    the other shapes a product followed by the activation kernel."""
    m = h.shape[0]
    F = out.shape[1]
    rows = h.xw if isinstance(h, NormedRows) else h
    if glu is not None:
        if not _skinny_ok(rows, w_gate_up) and _tc_ok(h, w_gate_up) and out.data_ptr() % 16 == 0:
            many = gemm_tc2 if _prefer_tc2(m, -(-F // 128), sm_count(h.device)) else gemm_tc
            return many(h, w_gate_up, out, EPI_SWIGLU, up_row_offset=F, glu=glu)
        return glu_clamped(linear(h, w_gate_up, out_dtype=torch.float32), out, *glu)
    if _skinny_ok(rows, w_gate_up):
        if _prefer_stream(rows, w_gate_up, 2 * F, swiglu=True):
            return gemv_stream(h, w_gate_up, out, EPI_SWIGLU, up_row_offset=F)
        if _prefer_tc_swap(m, 2 * F, h.shape[1], swiglu=True):
            return skinny_gemm_tc(h, w_gate_up, out, EPI_SWIGLU, up_row_offset=F)
        return skinny_gemm(h, w_gate_up, out, EPI_SWIGLU, up_row_offset=F)
    if isinstance(h, NormedRows):
        raise KernelError("gate_up_swiglu: a deferred norm needs a product that one of the few-row kernels takes")
    if _tc_ok(h, w_gate_up) and out.data_ptr() % 16 == 0:
        # tcgen05, activation in the epilogue; two SMs per tile where that takes fewer waves
        many = gemm_tc2 if _prefer_tc2(m, -(-F // 128), sm_count(h.device)) else gemm_tc
        return many(h, w_gate_up, out, EPI_SWIGLU, up_row_offset=F)
    gu = linear(h, w_gate_up, out_dtype=torch.float32)     # same rounding points as the fused kernels
    return silu_mul(gu, out)


FLASH_HEAD_DIMS = (64, 128)
USE_ATTENTION_TC = True        # prompt portions with head size 128 take the tcgen05 kernel where it applies
DECODE_SPLIT_KEYS = 128        # keys per split of the decode shape: a constant, so that a request's
                               # result never depends on the batch around it
DECODE_MAX_Q = 8               # requests with at most this many tokens in the step take the decode shape
DECODE_ROWS = 8                # (token, head) rows of a decode tile: 8 takes the kernel with the keys as the M side


class AttentionPlan:
    """Tiles of one step for one attention geometry (query heads per key/value head, window):
    which requests take the decode shape (16-row tiles, split keys) and which the prefill shape
    (64-row tiles).  Built once per step on the host and shared by every layer of that geometry."""

    def __init__(self, ctx, H, K, window, device, chunk=0):
        g = H // K
        self.GHd = min(g, DECODE_ROWS)
        self.chunks_d = -(-g // self.GHd)
        self.GHp = min(g, 64)
        self.chunks_p = -(-g // self.GHp)
        self.TTp = 64 // self.GHp
        dec = [r for r in range(ctx.n_requests) if ctx.q_lens[r] <= DECODE_MAX_Q]
        pre = [r for r in range(ctx.n_requests) if ctx.q_lens[r] > DECODE_MAX_Q]
        self.TTd = 1 if all(ctx.q_lens[r] == 1 for r in dec) else max(1, DECODE_ROWS // self.GHd)
        cu = [0]
        for ql in ctx.q_lens:
            cu.append(cu[-1] + ql)
        d_req, d_tok, p_req, p_tok = [], [], [], []
        n_splits = 1
        for r in dec:
            for t0 in range(0, ctx.q_lens[r], self.TTd):
                d_req.append(r)
                d_tok.append(cu[r] + t0)
                pos_first = ctx.start_pos[r] + t0
                pos_last = ctx.start_pos[r] + min(t0 + self.TTd, ctx.q_lens[r]) - 1
                # an upper bound of the keys the tile reads (the kernel rounds the window's start
                # down to a multiple of 32); a function of the padded shape only, so that a graph
                # captured for a padded context covers every real one
                span = pos_last + 1
                if window > 0:
                    span = min(span, window + self.TTd + 30)
                if chunk > 0:                    # the keys of a run, from its start rounded down likewise
                    span = min(span, chunk + self.TTd + 30)
                n_splits = max(n_splits, -(-span // DECODE_SPLIT_KEYS))
        for r in pre:
            for t0 in range(0, ctx.q_lens[r], self.TTp):
                p_req.append(r)
                p_tok.append(cu[r] + t0)
        # tiles of the tcgen05 kernel: 128 rows = (128 / g) tokens x g heads, when g divides 128
        t_req, t_tok = [], []
        self.TTt = 128 // g if g <= 128 and 128 % g == 0 else 0
        if self.TTt:
            for r in pre:
                for t0 in range(0, ctx.q_lens[r], self.TTt):
                    t_req.append(r)
                    t_tok.append(cu[r] + t0)
        self.n_dec, self.n_pre, self.n_tc, self.n_splits = len(d_req), len(p_req), len(t_req), n_splits
        flat = torch.tensor(d_req + d_tok + p_req + p_tok + t_req + t_tok + [0], dtype=torch.int32).to(device)
        nd, np_, nt = self.n_dec, self.n_pre, self.n_tc
        self.d_req, self.d_tok = flat[:nd], flat[nd:2 * nd]
        self.p_req, self.p_tok = flat[2 * nd:2 * nd + np_], flat[2 * nd + np_:2 * nd + 2 * np_]
        o = 2 * nd + 2 * np_
        self.t_req, self.t_tok = flat[o:o + nt], flat[o + nt:o + 2 * nt]


def paged_flash_attention(q, k_cache, v_cache, out, positions, cu_q, block_table, tile_req, tile_tok0,
                          n_tiles, H, K, hd, block_size, scale, window, mode, TT, GH, head_chunks,
                          split_keys=DECODE_SPLIT_KEYS, n_splits=1, keep_first=0, chunk=0, softcap=0.0, sink=None):
    """Tensor-core paged attention; mode 0: prefill shape, mode 1: decode shape with split keys
    (allocates the partials as scratch).  keep_first (with a window): the first keys of a request stay
    visible; in mode 1 one split more, the last, is theirs.  chunk: the chunked mask (runs of that many
    positions); softcap: capped scores; sink (float32 [H]): exp(sink[h]) joins the denominator of head
    h's softmax.  See attention_flash.cu."""
    if keep_first and window and mode == 1:
        n_splits += 1
    _need_cuda(q, k_cache, v_cache, out, positions, cu_q, block_table, tile_req, tile_tok0, sink)
    _need_contig(q=q, k_cache=k_cache, v_cache=v_cache, out=out)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H and sink.is_contiguous())
    if q.dtype != torch.bfloat16 or hd not in FLASH_HEAD_DIMS:
        raise KernelError(f"paged_flash_attention takes bfloat16 and a head size of 64 or 128, got {q.dtype}, {hd}")
    assert block_table.stride(1) == 1
    part_o = part_ml = None
    if mode == 1:
        rows = n_tiles * K * head_chunks * n_splits * TT * GH
        part_o = torch.empty(rows * hd, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(rows * 2, dtype=torch.float32, device=q.device)
    _check(_lib("attn").rllm_paged_flash_attention_sink(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(positions),
        _ptr(cu_q), _ptr(block_table), c_int(block_table.stride(0)), _ptr(tile_req), _ptr(tile_tok0),
        c_int(n_tiles), c_int(H), c_int(K), c_int(hd), c_int(block_size), c_float(scale), c_int(window),
        c_int(keep_first if window else 0), c_int(mode), c_int(TT), c_int(GH), c_int(head_chunks), c_int(split_keys),
        c_int(n_splits), c_longlong(k_cache.shape[0]), _ptr(error_word(q.device)), c_int(chunk), c_float(softcap),
        _ptr(sink), _stream()),
        "paged_flash_attention")
    global _launches
    if mode == 1:
        _launches += 1                         # the combine kernel
    return out


def attention_tc_ok(q, hd, block_size, H, K) -> bool:
    g = H // K
    return (q.dtype == torch.bfloat16 and hd == 128 and 8 <= block_size <= 128
            and block_size & (block_size - 1) == 0 and g <= 128 and 128 % g == 0)


def attention_tc(q, k_cache, v_cache, out, positions, cu_q, block_table, tile_req, tile_tok0, n_tiles, H, K, hd,
                 block_size, scale, window, chunk=0, softcap=0.0, sink=None):
    """Prefill attention on the tcgen05 tensor cores (S and O in tensor memory); see attention_tc.cu."""
    _need_cuda(q, k_cache, v_cache, out, positions, cu_q, block_table, tile_req, tile_tok0, sink)
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H and sink.is_contiguous())
    _need_contig(q=q, k_cache=k_cache, v_cache=v_cache, out=out)
    if not attention_tc_ok(q, hd, block_size, H, K):
        raise KernelError("attention_tc takes bfloat16, head size 128, a power-of-two page size from 8 to 128 and "
                          "a number of query heads per key/value head that divides 128")
    st = _lib("attn_tc").rllm_attention_tc_sink(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), c_int(q.shape[0]), c_longlong(k_cache.shape[0]),
        _ptr(positions), _ptr(cu_q), _ptr(block_table), c_int(block_table.stride(0)), _ptr(tile_req),
        _ptr(tile_tok0), c_int(n_tiles), c_int(H), c_int(K), c_int(hd), c_int(block_size), c_float(scale),
        c_int(window), c_int(chunk), c_float(softcap), _ptr(sink), _ptr(error_word(q.device)), _stream())
    if st >= 30000:
        raise KernelError(f"attention_tc: tensor map encoding failed (CUresult {st - 30000})")
    _check(st, "attention_tc")
    return out


PRODUCTS_MAX_SCORE_BYTES = 1 << 30      # score rows of one call of the attention written as two products
PRODUCTS_BLOCK_TOKENS = 512             # tokens of a portion whose score rows are one product


def gemm_lib_nn(a, b, out):
    """out[m,n] = a[m,k] . b[k,n], b row-major as it lies, through cuBLAS (bfloat16, float32 accumulation)."""
    _need_cuda(a, b, out)
    m, k = a.shape
    n = b.shape[1]
    assert a.dtype == b.dtype == torch.bfloat16 and b.shape[0] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1
    st = _lib("blas").rllm_gemm_lib_nn(_ptr(a), _ptr(b), _ptr(out), c_int(_code(out)), c_int(m), c_int(n), c_int(k),
                                       c_int(a.stride(0)), c_int(b.stride(0)), c_int(out.stride(0)), _stream())
    if st >= 10000:
        raise KernelError(f"gemm_lib_nn: cuBLAS status {st - 10000} for m={m} n={n} k={k}")
    _check(st, "gemm_lib_nn", own=False)
    return out


def masked_softmax_rows(scores, probs, H, pos0, n_cols, scale, softcap=0.0, chunk=0, window=0, col0=0):
    """scores [rows, >= n_cols] float32 (row = token * H + head, the token at position pos0 + token; column j
    the key at position col0 + j) -> probs [rows, >= n_cols] bfloat16: softmax over the visible keys (causal;
    inside the token's chunk; the last `window` keys), zero elsewhere.  See headwise.cu."""
    _need_cuda(scores, probs)
    _rows2d(scores, "scores"), _rows2d(probs, "probs")
    rows = scores.shape[0]
    assert scores.dtype == torch.float32 and probs.dtype == torch.bfloat16 and probs.shape[0] == rows
    assert scores.shape[1] >= n_cols and probs.shape[1] >= n_cols
    _check(core().rllm_masked_softmax_rows(_ptr(scores), c_longlong(scores.stride(0)), _ptr(probs),
                                           c_longlong(probs.stride(0)), c_int(rows), c_int(H), c_int(pos0),
                                           c_int(n_cols), c_float(scale), c_float(softcap), c_int(chunk), c_int(window),
                                           c_int(col0), _stream()),
           "masked_softmax_rows")
    return probs


LATENT_SPLIT_KEYS = 128        # keys per split of the latent decode kernel: a constant, as DECODE_SPLIT_KEYS


def latent_decode_ok(q, hd, hdv) -> bool:
    return q.dtype == torch.bfloat16 and hd % 16 == 0 and hdv % 64 == 0 and 0 < hdv <= 512 and hdv <= hd and hd <= 1152


def latent_decode_attention(q, cache, out, positions, seq_ids, block_table, H, hd, hdv, block_size, scale, softcap,
                            max_ctx_len, window=0):
    """The decode shape of attention over one shared key/value head on the tensor cores (split keys,
    partials as scratch, merged by a second kernel); see attention_latent.cu."""
    _need_cuda(q, cache, out, positions, seq_ids, block_table)
    _need_contig(q=q, cache=cache, out=out, positions=positions, seq_ids=seq_ids)
    n = q.shape[0]
    assert q.shape == (n, H * hd) and out.shape == (n, H * hdv) and cache.shape[1:] == (1, block_size, hd)
    assert q.dtype == cache.dtype == out.dtype == torch.bfloat16 and block_table.stride(1) == 1
    if not latent_decode_ok(q, hd, hdv):
        raise KernelError("latent_decode_attention takes bfloat16, key rows of a multiple of 16 entries up to 1152 and "
                          "values of a multiple of 64 entries up to 512")
    # with a window the splits start at the window's first key rounded down to a tile of 32 keys
    span = int(max_ctx_len) if window <= 0 else min(int(max_ctx_len), window + 31)
    n_splits = max(1, -(-span // LATENT_SPLIT_KEYS))
    rows = n * (-(-H // 32)) * n_splits * 32
    part_o = torch.empty(rows * hdv, dtype=torch.float32, device=q.device)
    part_ml = torch.empty(rows * 2, dtype=torch.float32, device=q.device)
    _check(_lib("attn_latent").rllm_latent_decode_attention(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(positions), _ptr(seq_ids), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(n), c_int(H), c_int(hd), c_int(hdv), c_int(block_size), c_float(scale),
        c_float(softcap), c_int(LATENT_SPLIT_KEYS), c_int(n_splits), c_longlong(cache.shape[0]),
        _ptr(error_word(q.device)), c_int(window), _stream()), "latent_decode_attention")
    global _launches
    _launches += 1                             # the merge kernel
    return out


def shared_kv_attention(q, cache, out, ctx, block_table, H, hd, hdv, block_size, scale, softcap=0.0, window=0):
    """Causal attention of H query heads over ONE key/value head whose values are the first hdv entries
    of the key rows (attention through a latent).  q [n, H * hd], cache [pages, 1, block_size, hd], out
    [n, H * hdv].  bfloat16 portions of more than DECODE_MAX_Q tokens are two library products around a
    softmax kernel per request: the request's pages gathered into one matrix C [keys, hd], scores =
    Q C^T for all its (token, head) rows at once (the heads share C, so the product has H times the rows
    of a head's own), probabilities, then P C[:, :hdv].  The other rows (decode steps, short portions)
    take the tensor-core decode kernel of attention_latent.cu where the sizes allow it; float32 and odd
    sizes take the plain kernel.  window > 0: a token sees its last `window` keys only (itself included);
    the products then start at the page that holds the first visible key of a block of tokens."""
    n = q.shape[0]
    runs = []            # (first row, rows) of the tokens that take the plain kernel, merged
    big = []
    lib_ok = (q.dtype == torch.bfloat16 and hd % 8 == 0 and hdv % 8 == 0 and (H * hd) % 8 == 0
              and block_size % 8 == 0)
    at = 0
    for r in range(ctx.n_requests):
        k = ctx.q_lens[r]
        if lib_ok and k > DECODE_MAX_Q:
            big.append((r, at, k))
        elif runs and runs[-1][0] + runs[-1][1] == at:
            runs[-1] = (runs[-1][0], runs[-1][1] + k)
        else:
            runs.append((at, k))
        at += k
    for a, k in runs:
        if latent_decode_ok(q, hd, hdv):
            latent_decode_attention(q[a:a + k], cache, out[a:a + k], ctx.positions[a:a + k], ctx.seq_ids[a:a + k],
                                    block_table, H, hd, hdv, block_size, scale, softcap, ctx.max_ctx_len, window)
        else:
            paged_attention_generic(q[a:a + k], cache, cache, out[a:a + k], ctx.positions[a:a + k],
                                    ctx.seq_ids[a:a + k], block_table, H, 1, hd, block_size, scale, window, 0, hdv, 0,
                                    softcap)
    for r, a, k in big:
        start, length = ctx.start_pos[r], ctx.start_pos[r] + k
        n_pages = -(-length // block_size)
        # with a window only the pages from the first visible key of the portion's first token on are read
        # (earlier ones may have gone back to the pool)
        page0 = max(0, start + 1 - window) // block_size if window > 0 else 0
        first = page0 * block_size
        keys = cache.index_select(0, block_table[r, page0:n_pages].long()).view((n_pages - page0) * block_size, hd)
        L = (n_pages - page0) * block_size
        # blocks of tokens: a block's products stop at its last token's key, so shorter blocks skip more of the
        # masked upper triangle (a third of the work at four blocks) for three more launches each
        step = max(1, min(k, PRODUCTS_BLOCK_TOKENS, PRODUCTS_MAX_SCORE_BYTES // (4 * H * L)))
        for t0 in range(0, k, step):
            t1 = min(k, t0 + step)
            rows = (t1 - t0) * H
            hi = min(L, -(-(start + t1 - first) // 8) * 8)        # keys beyond the last token of these rows are not needed
            lo = (max(0, start + t0 + 1 - window) - first) // 8 * 8 if window > 0 else 0    # nor those before the block's window
            scores = torch.empty((rows, hi - lo), dtype=torch.float32, device=q.device)
            gemm_lib(q[a + t0:a + t1].view(rows, hd), keys[lo:hi], scores)
            probs = torch.empty((rows, hi - lo), dtype=torch.bfloat16, device=q.device)
            masked_softmax_rows(scores, probs, H, start + t0, hi - lo, scale, softcap, window=window, col0=first + lo)
            gemm_lib_nn(probs, keys[lo:hi, :hdv], out[a + t0:a + t1].view(rows, hdv))
    return out


def paged_attention(q, k_cache, v_cache, out, ctx, block_table, H, K, hd, block_size, scale, window=0,
                    keep_first=0, v_head_dim=None, chunk=0, softcap=0.0, sink=None):
    """Attention of the step's tokens over the paged cache; chooses the kernel by element type,
    head size and the shape of the step (`ctx`: the step's StepContext).  float32, head sizes
    other than 64 and 128 and value heads of another size than the key heads take the plain kernel;
    windows that keep the first keys take the mma.sync kernels, not the tcgen05 one."""
    hdv = hd if not v_head_dim else int(v_head_dim)
    keep_first = keep_first if window else 0
    if q.dtype != torch.bfloat16 or hd not in FLASH_HEAD_DIMS or hdv != hd:
        return paged_attention_generic(q, k_cache, v_cache, out, ctx.positions, ctx.seq_ids, block_table,
                                       H, K, hd, block_size, scale, window, keep_first, hdv, chunk, softcap, sink)
    key = (H // K, window, chunk)
    plan = ctx.plans.get(key)
    if plan is None:
        plan = ctx.plans[key] = AttentionPlan(ctx, H, K, window, q.device, chunk)
    if plan.n_pre and plan.n_tc and USE_ATTENTION_TC and attention_tc_ok(q, hd, block_size, H, K) and not keep_first:
        attention_tc(q, k_cache, v_cache, out, ctx.positions, ctx.cu_q, block_table, plan.t_req, plan.t_tok,
                     plan.n_tc, H, K, hd, block_size, scale, window, chunk, softcap, sink)
    elif plan.n_pre:
        paged_flash_attention(q, k_cache, v_cache, out, ctx.positions, ctx.cu_q, block_table, plan.p_req,
                              plan.p_tok, plan.n_pre, H, K, hd, block_size, scale, window, 0, plan.TTp,
                              plan.GHp, plan.chunks_p, keep_first=keep_first, chunk=chunk, softcap=softcap, sink=sink)
    if plan.n_dec:
        paged_flash_attention(q, k_cache, v_cache, out, ctx.positions, ctx.cu_q, block_table, plan.d_req,
                              plan.d_tok, plan.n_dec, H, K, hd, block_size, scale, window, 1, plan.TTd,
                              plan.GHd, plan.chunks_d, DECODE_SPLIT_KEYS, plan.n_splits, keep_first=keep_first,
                              chunk=chunk, softcap=softcap, sink=sink)
    return out
