"""Grouped-query causal attention over the paged cache.

q/k/v projections without bias, optional per-head RMSNorm on queries and keys (one weight of
head_dim entries shared by all heads, applied before the rotation), position encoding on
queries and keys, keys and values written to the cache at the step's slots, softmax(q.k *
scale) over keys pos+1-window..pos (window 0: all), output projection
(AxiomOperator/rllm: crates/rllm-model/src/qwen3.rs:195-201; attention formula
crates/rllm-cpu/src/lib.rs:389-425; q/k norm crates/rllm-core/src/lib.rs:459-476).

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm, qk_norm_eps, window,
scale.  Tensors: <prefix>{q,k,v,o}_proj.weight and, with qk_norm, <prefix>{q,k}_norm.weight.
Load-time transform: q, k and v are stacked into one [(H + 2K) * head_dim, hidden] matrix.

Further parameters (each with the default that leaves the above as it is):
`v_head_dim`: value heads of their own size (the output projection then reads H * v_head_dim columns).
`sink`: a learned number per query head, <prefix>sink [H], whose exponential joins the softmax's
denominator: p_j = exp(s_j - m) / (sum_i exp(s_i - m) + exp(sink_h - m)); it has no key and no value
and is not scaled.
`own_kv` False: the layer has no key and value projections (nor a key norm); it reads the keys (as
cached: normed and rotated) and values that another layer wrote (the run entry's `cache_of`), with
queries, sinks and output projection of its own.
`names` "short": the tensors are <prefix>q, k, v, o, q.norm, k.norm, sink.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PagedKVNeed, PartError, register_part


@register_part("mixer", "attention")
class Attention(Mixer):
    CAPTURE_SAFE = True
    TRACEABLE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden_size = int(p["hidden_size"])
        self.H = int(p["num_heads"])
        self.K = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.window = int(p.get("window", 0) or 0)
        self.scale = float(p["scale"])
        if self.H % self.K:
            raise PartError(f"attention: {self.H} heads are not a multiple of {self.K} key/value heads")
        self.hdv = int(p.get("v_head_dim") or self.hd)
        self.has_sink = bool(p.get("sink", False))
        self.own_kv = bool(p.get("own_kv", True))
        short = p.get("names") == "short"
        self.plain = self.hdv == self.hd and not self.has_sink and self.own_kv
        if (self.hd % 16 and self.plain) or self.hd % 2 or self.hd > 256 or self.hdv > 256:
            raise PartError(f"attention: head_dim {self.hd} must be a multiple of 16 and at most 256")
        n = (lambda s: s) if short else (lambda s: {"q.norm": "q_norm.weight", "k.norm": "k_norm.weight",
                                                    "sink": "sink"}.get(s, s + "_proj.weight"))
        self._n = {s: self.prefix + n(s) for s in ("q", "k", "v", "o", "q.norm", "k.norm", "sink")}
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = self.sink = None

    def cache_need(self):
        return PagedKVNeed(self.K, self.hd, self.window, 0, self.hdv if self.hdv != self.hd else 0)

    def expected_tensors(self):
        d, H, K, hd, n = self.hidden_size, self.H, self.K, self.hd, self._n
        t = {n["q"]: ((H * hd, d), "matrix"), n["o"]: ((d, H * self.hdv), "matrix")}
        if self.own_kv:
            t[n["k"]] = ((K * hd, d), "matrix")
            t[n["v"]] = ((K * self.hdv, d), "matrix")
        if self.qk_norm:
            t[n["q.norm"]] = ((hd,), "norm")
            if self.own_kv:
                t[n["k.norm"]] = ((hd,), "norm")
        if self.has_sink:
            t[n["sink"]] = ((H,), "unit")
        return t

    def load(self, tensors):
        n, dt = self._n, self.runtime.dtype
        self.w_qkv = self._to_device(torch.cat([tensors[n[s]].to(dt) for s in ("qkv" if self.own_kv else "q")], 0))
        self.w_o = self._to_device(tensors[n["o"]])
        if self.qk_norm:
            self.q_norm_w = self._to_device(tensors[n["q.norm"]], torch.float32)
            if self.own_kv:
                self.k_norm_w = self._to_device(tensors[n["k.norm"]], torch.float32)
        if self.has_sink:
            self.sink = self._to_device(tensors[n["sink"]], torch.float32)

    # A norm between two products may go without a kernel of its own (ops.NormedRows): the block asks the
    # parts on both sides for the matrices of their last and first product.
    def first_product(self):
        return self.w_qkv, False

    def last_product(self):
        return self.w_o, None, False

    def forward(self, h, ctx, cache, position, residual=None, then_norm=None):
        """`h` may be ops.NormedRows; then_norm = (weight, eps): the output product also prepares the
        norm that follows and the rows come back as ops.NormedRows (needs `residual`)."""
        n = h.shape[0]
        dt = self.runtime.dtype
        q = torch.empty((n, self.H * self.hd), dtype=dt, device=self.w_qkv.device)
        if not self.plain:
            return self._forward_general(h, ctx, cache, position, q)
        whole = getattr(position, "project_and_store", None)
        if whole is not None and whole(h, self.w_qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, ctx, cache, q,
                                       self.H, self.K, self.hd):
            qkv = None                            # the position part did the projection too
        else:
            qkv = ops.linear(h, self.w_qkv, out_dtype=torch.float32)
        if qkv is None:
            pass
        elif position is not None and hasattr(position, "apply_and_store"):
            # the position part does it all: q/k norm, its own encoding, queries out, keys and values stored
            position.apply_and_store(qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, ctx, cache, q,
                                     self.H, self.K, self.hd)
        else:
            ops.qk_norm_rope_store(qkv, self.q_norm_w, self.k_norm_w,
                                   position.table() if position is not None else None, ctx.positions,
                                   cache.slots, q, cache.k, cache.v, self.H, self.K, self.hd,
                                   cache.block_size, self.qk_norm_eps, write_kv=cache.write)
        attn = torch.empty_like(q)
        ops.paged_attention(q, cache.k, cache.v, attn, ctx, cache.block_table, self.H, self.K, self.hd,
                            cache.block_size, self.scale, self.window)
        if residual is not None:
            if then_norm is not None:
                return ops.linear(attn, self.w_o, out=residual, accumulate=True, then_norm=then_norm)
            ops.linear(attn, self.w_o, out=residual, accumulate=True)
            return None
        return ops.linear(attn, self.w_o, out_dtype=torch.float32)

    def _forward_general(self, h, ctx, cache, position, q):
        """Value heads of their own size, sinks, or another layer's keys and values: the position part
        does norm, rotation and the cache write (`apply_and_store` with `v_head_dim` and `has_kv`)."""
        if cache.write != self.own_kv:
            raise PartError("attention: a layer with keys and values of its own writes its cache; one without "
                            "reads another entry's (cache_of)")
        qkv = ops.linear(h, self.w_qkv, out_dtype=torch.float32)              # [q (| k | v)]
        if position is not None:
            position.apply_and_store(qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, ctx, cache, q,
                                     self.H, self.K, self.hd, v_head_dim=self.hdv, has_kv=self.own_kv)
        else:
            ops.head_norm_rope_store(qkv, self.q_norm_w, self.k_norm_w, None, 0, False, cache.slots, q, cache.k,
                                     cache.v, self.H, self.K, self.hd, self.hdv, cache.block_size, self.qk_norm_eps,
                                     has_kv=self.own_kv)
        attn = torch.empty((q.shape[0], self.H * self.hdv), dtype=q.dtype, device=q.device)
        ops.paged_attention(q, cache.k, cache.v, attn, ctx, cache.block_table, self.H, self.K, self.hd,
                            cache.block_size, self.scale, self.window, v_head_dim=self.hdv, sink=self.sink)
        return ops.linear(attn, self.w_o, out_dtype=torch.float32)
