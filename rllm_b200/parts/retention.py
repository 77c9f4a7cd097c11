"""Retention: linear attention with a fixed decay per head, no softmax and no denominator.

For normed input rows h [n, d] of one request in order, H heads with keys of dk and values of dv
entries, c_h the head's decay:

    q = h Wq^T,  k = h Wk^T  ([H, dk]),  v = h Wv^T  ([H, dv])            no biases
    q, k <- rotary on their first rot.dims entries (the position part; rotate-half or pair layout)
    k <- k * key_scale                                                     after the rotation
    per head, S [dk, dv] starting at zero:   S_t = c_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
    out = ((o / rms(o) per head, eps inside the root, no weight) * gate(h Wg^T)) Wo^T

State per request (float32): S of every head, in the retention kernel's own order, kept from step to
step.  Parameters: hidden_size, num_heads, head_dim, v_head_dim, decay (one number per head),
key_scale, eps, gate ("silu", "sigmoid" or None: no gate and no tensor g).  Tensors under <prefix>:
q, k [H*dk, d]; v, g [H*dv, d]; o [d, H*dv].  q, k, v and the gate are one stacked product whose result
stays float32; angles, the rotation, the decay, the state, the unit norm and the gate's activation are
float32 in every mode.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PartError, StateNeed, register_part


@register_part("mixer", "retention")
class Retention(Mixer):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden_size = int(p["hidden_size"])
        self.H, self.dk = int(p["num_heads"]), int(p["head_dim"])
        self.dv = int(p.get("v_head_dim") or self.dk)
        self.decay_values = tuple(float(x) for x in p["decay"])
        self.key_scale = float(p.get("key_scale", 1.0))
        self.eps = float(p.get("eps", 1e-6))
        self.gate = p.get("gate", "silu")
        if len(self.decay_values) != self.H:
            raise PartError(f"retention: {len(self.decay_values)} decays for {self.H} heads")
        if self.gate not in ops.GATES:
            raise PartError(f"retention: gate {self.gate!r} is not known")
        if max(self.dk, self.dv) > 256:
            raise PartError("retention: head sizes up to 256")
        self.has_gate = bool(ops.GATES[self.gate])
        self.w_in = self.w_o = None
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def cache_need(self):
        return StateNeed((ops.retention_state_floats(self.H, self.dk, self.dv),), torch.float32)

    def expected_tensors(self):
        d, p = self.hidden_size, self.prefix
        t = {p + "q": ((self.H * self.dk, d), "matrix"), p + "k": ((self.H * self.dk, d), "matrix"),
             p + "v": ((self.H * self.dv, d), "matrix"), p + "o": ((d, self.H * self.dv), "matrix")}
        if self.has_gate:
            t[p + "g"] = ((self.H * self.dv, d), "matrix")
        return t

    def load(self, tensors):
        p, dt = self.prefix, self.runtime.dtype
        names = "qkvg" if self.has_gate else "qkv"
        self.w_in = self._to_device(torch.cat([tensors[p + n].to(dt) for n in names], 0))
        self.w_o = self._to_device(tensors[p + "o"])

    def forward(self, h, ctx, cache, position=None, residual=None):
        n, dev = h.shape[0], h.device
        rows = ops.linear(h, self.w_in, out_dtype=torch.float32)               # [q | k | v | gate]
        hk, hv = self.H * self.dk, self.H * self.dv
        rot = min(position.dims, self.dk) if position is not None else 0
        if rot and position.mult != 1.0:
            raise PartError("retention: scaled rotary frequencies are not supported")
        out = torch.empty((n, hv), dtype=self.runtime.dtype, device=dev)
        ops.retention(rows, 0, hk, 2 * hk, 2 * hk + hv, position.angles(ctx) if rot else None, rot,
                      rot and position.layout == "pairs", self.key_scale, self.decay, self.eps, cache.state, ctx.cu_q,
                      cache.slots, out, ctx.n_requests, self.H, self.dk, self.dv, gate=self.gate,
                      segments=ops.time_segments(ctx, dev))
        return ops.linear(out, self.w_o, out_dtype=torch.float32)
