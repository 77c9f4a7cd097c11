"""The matrix memory of xLSTM (mLSTM): linear attention whose memory is fed and forgotten through
exponential gates, kept in range by a running maximum.

For input rows h [n, d] of one request in order, H heads with keys of dk and values of dv entries:

    q = h Wq^T * q_scale,  k = h Wk^T  ([H, dk]),  v = h Wv^T  ([H, dv])
    per head, from two more rows of the projection and their biases:
        i = cap * tanh((h . w_i + b_i) / cap),   f = logsigmoid(cap * tanh((h . w_f + b_f) / cap))
    per head, S [dk, dv], n [dk] and the running maximum m, all three zero before the first token:
        m_t = max(f + m_(t-1), i)
        S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T       n_t likewise with k alone
        o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
    out = ((o / rms(o) per head, eps inside the root) * norm_w * gate(h Wg^T)) Wo^T

State per request (float32): S and n of every head in the kernel's own order, and m, kept from step to
step (csrc/recurrent.cu).  Key heads up to 256 and value heads up to 254 entries take the fast kernel (cut
along time for long portions); larger heads a plain kernel that walks the tokens with the memory in the slot.  Parameters: hidden_size, num_heads, head_dim, v_head_dim, gate_cap (0: the
gates are not capped), q_scale, eps, gate ("sigmoid", "silu" or None).  Tensors under <prefix>: q, k
[H*dk, d]; v, g [H*dv, d]; i, f [H, d]; i.b, f.b [H]; norm [H*dv]; o [d, H*dv].  q, k, v, the gate and the
two gate rows are one stacked product (rows of zeros up to a multiple of 8) whose result stays float32;
the gates, their exponentials, the maximum, the memory, the unit norm and the gate's activation are
float32 in every mode.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PartError, StateNeed, register_part


@register_part("mixer", "mlstm")
class MatrixMemory(Mixer):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden_size = int(p["hidden_size"])
        self.H, self.dk = int(p["num_heads"]), int(p["head_dim"])
        self.dv = int(p.get("v_head_dim") or self.dk)
        self.cap = float(p.get("gate_cap", 0.0) or 0.0)
        self.q_scale = float(p.get("q_scale", self.dk ** -0.5))
        self.eps = float(p.get("eps", 1e-6))
        self.gate = p.get("gate", "sigmoid")
        if self.gate not in ops.GATES:
            raise PartError(f"mlstm: gate {self.gate!r} is not known")
        if 2 * self.dk + self.dv + 1 > 12288:
            raise PartError("mlstm: head sizes beyond the kernels' shared memory (2 dim + vdim up to 12,287)")
        if self.cap < 0:
            raise PartError("mlstm: gate_cap must not be negative")
        self.has_gate = bool(ops.GATES[self.gate])
        self.w_in = self.w_o = self.norm_w = self.i_bias = self.f_bias = None

    def cache_need(self):
        return StateNeed((ops.mlstm_state_floats(self.H, self.dk, self.dv),), torch.float32)

    def expected_tensors(self):
        d, p, H = self.hidden_size, self.prefix, self.H
        t = {p + "q": ((H * self.dk, d), "matrix"), p + "k": ((H * self.dk, d), "matrix"),
             p + "v": ((H * self.dv, d), "matrix"), p + "o": ((d, H * self.dv), "matrix"),
             p + "i": ((H, d), "matrix"), p + "f": ((H, d), "matrix"), p + "i.b": ((H,), "bias"),
             p + "f.b": ((H,), "bias"), p + "norm": ((H * self.dv,), "norm")}
        if self.has_gate:
            t[p + "g"] = ((H * self.dv, d), "matrix")
        return t

    def load(self, tensors):
        p, dt = self.prefix, self.runtime.dtype
        names = ["q", "k", "v"] + (["g"] if self.has_gate else []) + ["i", "f"]
        stack = [tensors[p + n].to(dt) for n in names]
        rows = sum(t.shape[0] for t in stack)
        if rows % 8:                 # the projection's float32 rows stay aligned for every product kernel
            stack.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=dt, device=stack[0].device))
        self.w_in = self._to_device(torch.cat(stack, 0))
        self.w_o = self._to_device(tensors[p + "o"])
        self.norm_w = self._to_device(tensors[p + "norm"], torch.float32)
        self.i_bias = self._to_device(tensors[p + "i.b"], torch.float32)
        self.f_bias = self._to_device(tensors[p + "f.b"], torch.float32)

    def forward(self, h, ctx, cache, position=None, residual=None):
        n, dev = h.shape[0], h.device
        rows = ops.linear(h, self.w_in, out_dtype=torch.float32)               # [q | k | v | gate | i | f]
        hk, hv = self.H * self.dk, self.H * self.dv
        g_off = 2 * hk + hv
        i_off = g_off + (hv if self.has_gate else 0)
        out = torch.empty((n, hv), dtype=self.runtime.dtype, device=dev)
        ops.mlstm(rows, 0, hk, 2 * hk, g_off, i_off, i_off + self.H, self.i_bias, self.f_bias, self.cap, self.q_scale,
                  self.norm_w, self.eps, cache.state, ctx.cu_q, cache.slots, out, ctx.n_requests, self.H, self.dk,
                  self.dv, gate=self.gate, segments=ops.time_segments(ctx, dev))
        return ops.linear(out, self.w_o, out_dtype=torch.float32)
