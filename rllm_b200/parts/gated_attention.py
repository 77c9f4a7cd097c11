"""Grouped-query attention with a sliding window that keeps the first tokens, biased projections,
an RMSNorm over the whole query and key rows, value heads of their own size and an output gate.

For normed input rows h [n, d] (H query heads, G key/value heads, key size dk, value size dv):

    q = h Wq^T + bq,  k = h Wk^T + bk,  v = h Wv^T + bv
    q <- q / rms(q) * nq,  k <- k / rms(k) * nk      (rms over the whole row of H*dk resp. G*dk
                                                      entries, eps inside the root; `qk_norm: "row"`)
    with a position part: the first rot.dims entries of every query and key head are rotated by the token's
        angles AFTER the norm (either pair layout); without one a score depends on the two rows only
    query at position i sees key j iff j <= i and (i - j < window or j < keep_first)
    p = softmax over the visible keys of (q_head . k_group) * scale;  a_head = sum_j p_j v_j
    out = ((a_1 | ... | a_H) * sigmoid(h Wg^T)) Wo^T                       (`gate: "sigmoid"`; with
                                                      `gate_per_head` Wg has one row per head and its
                                                      number multiplies the whole head)

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim, bias, qk_norm ("row" or
None), eps, window (0: all keys), keep_first, scale, gate ("sigmoid" or None), gate_per_head.  Tensors under
<prefix>: q, k, v, o, g and, by the options, q.b, k.b, v.b, q.norm, k.norm.  Load-time transform:
q, k, v and the gate are stacked into one projection [q | k | v | g] (the biases of q, k, v likewise; rows of
zeros up to a multiple of 8 rows).  Scores, softmax, norms and the
gate's sigmoid are float32 in every mode.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PagedKVNeed, PartError, register_part


@register_part("mixer", "gated_attention")
class GatedWindowAttention(Mixer):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden_size = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk = int(p["head_dim"])
        self.dv = int(p.get("v_head_dim") or self.dk)
        self.bias = bool(p.get("bias", False))
        self.qk_norm = p.get("qk_norm")
        self.eps = float(p.get("eps", 1e-6))
        self.window = int(p.get("window", 0) or 0)
        self.keep_first = int(p.get("keep_first", 0) or 0) if self.window else 0
        self.scale = float(p["scale"])
        self.gate = p.get("gate")
        self.gate_per_head = bool(p.get("gate_per_head", False)) and bool(self.gate)
        if self.H % self.G:
            raise PartError(f"gated_attention: {self.H} heads are not a multiple of {self.G} key/value heads")
        if self.qk_norm not in (None, "row"):
            raise PartError(f"gated_attention: qk_norm {self.qk_norm!r} is not supported ('row' or none)")
        if self.gate not in (None, "sigmoid", "silu"):
            raise PartError(f"gated_attention: gate {self.gate!r} is not supported")
        if max(self.dk, self.dv) > 512:
            raise PartError("gated_attention: head sizes up to 512")
        self.w_qkv = self.b_qkv = self.q_norm_w = self.k_norm_w = self.w_o = None

    def cache_need(self):
        return PagedKVNeed(self.G, self.dk, self.window, self.keep_first, self.dv if self.dv != self.dk else 0)

    def expected_tensors(self):
        d, p = self.hidden_size, self.prefix
        wq, wk, wv = self.H * self.dk, self.G * self.dk, self.G * self.dv
        t = {p + "q": ((wq, d), "matrix"), p + "k": ((wk, d), "matrix"), p + "v": ((wv, d), "matrix"),
             p + "o": ((d, self.H * self.dv), "matrix")}
        if self.bias:
            t.update({p + "q.b": ((wq,), "bias"), p + "k.b": ((wk,), "bias"), p + "v.b": ((wv,), "bias")})
        if self.qk_norm:
            t.update({p + "q.norm": ((wq,), "norm"), p + "k.norm": ((wk,), "norm")})
        if self.gate:
            t[p + "g"] = ((self.H if self.gate_per_head else self.H * self.dv, d), "matrix")
        return t

    def load(self, tensors):
        p, dt = self.prefix, self.runtime.dtype
        names = "qkvg" if self.gate else "qkv"
        stack = [tensors[p + n].to(dt) for n in names]
        rows = sum(t.shape[0] for t in stack)
        if rows % 8:                 # the projection's float32 rows stay aligned for every product kernel
            stack.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=dt, device=stack[0].device))
        self.w_qkv = self._to_device(torch.cat(stack, 0))
        if self.bias:
            self.b_qkv = self._to_device(torch.cat([tensors[p + n + ".b"].to(torch.float32) for n in "qkv"], 0),
                                         torch.float32)
        if self.qk_norm:
            self.q_norm_w = self._to_device(tensors[p + "q.norm"], torch.float32)
            self.k_norm_w = self._to_device(tensors[p + "k.norm"], torch.float32)
        self.w_o = self._to_device(tensors[p + "o"])

    def forward(self, h, ctx, cache, position=None, residual=None):
        n, dt, dev = h.shape[0], self.runtime.dtype, h.device
        wide = ops.linear(h, self.w_qkv, out_dtype=torch.float32)          # [q | k | v | gate]
        n_qkv = self.H * self.dk + self.G * (self.dk + self.dv)
        qkv = wide[:, :n_qkv]
        q = torch.empty((n, self.H * self.dk), dtype=dt, device=dev)
        rot = min(position.dims, self.dk) if position is not None else 0
        if rot and getattr(position, "mult", 1.0) != 1.0:
            raise PartError("gated_attention: cos and sin with a multiplier are not supported")
        ops.qkv_rownorm_store(qkv, self.b_qkv, self.q_norm_w, self.k_norm_w, cache.slots, q, cache.k, cache.v,
                              self.H, self.G, self.dk, self.dv, cache.block_size, self.eps, write_kv=cache.write,
                              cs_table=position.angles(ctx) if rot else None, rot=rot,
                              pairs=bool(rot) and position.layout == "pairs")
        attn = torch.empty((n, self.H * self.dv), dtype=dt, device=dev)
        ops.paged_attention(q, cache.k, cache.v, attn, ctx, cache.block_table, self.H, self.G, self.dk,
                            cache.block_size, self.scale, self.window, self.keep_first, self.dv)
        if self.gate:
            n_gate = self.H if self.gate_per_head else self.H * self.dv
            ops.rows_act(attn, attn, mul=wide[:, n_qkv:n_qkv + n_gate], mul_act=self.gate,
                         mul_group=self.dv if self.gate_per_head else 1)
        return ops.linear(attn, self.w_o, out_dtype=torch.float32)
