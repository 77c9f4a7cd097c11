"""Feed-forwards.  ``dense_act``: out = act(h . Wup^T) . Wdown^T with one of the activations of
csrc/rowwise.cu (relu2: the square of relu), no gate, no biases; parameters hidden_size,
intermediate_size, activation; tensors <prefix>up, <prefix>down.

SwiGLU feed-forward: out = (silu(h . Wg^T) * (h . Wu^T)) . Wd^T, no biases
(AxiomOperator/rllm: crates/rllm-core/src/lib.rs:247-262, crates/rllm-cpu/src/lib.rs:292-298).
Parameters: hidden_size, intermediate_size.  Tensors: <prefix>{gate,up,down}_proj.weight.
Load-time transform: gate and up are stacked into one [2F, hidden] matrix so that one product
feeds the activation kernel.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, register_part


@register_part("ffn", "swiglu")
class SwiGLU(FeedForward):
    CAPTURE_SAFE = True
    TRACEABLE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def expected_tensors(self):
        F, d = self.intermediate_size, self.hidden_size
        return {self.prefix + "gate_proj.weight": ((F, d), "matrix"),
                self.prefix + "up_proj.weight": ((F, d), "matrix"),
                self.prefix + "down_proj.weight": ((d, F), "matrix")}

    def load(self, tensors):
        g = tensors[self.prefix + "gate_proj.weight"]
        u = tensors[self.prefix + "up_proj.weight"]
        self.w_gate_up = self._to_device(torch.cat([g.to(self.runtime.dtype), u.to(self.runtime.dtype)], 0))
        self.w_down = self._to_device(tensors[self.prefix + "down_proj.weight"])

    def first_product(self):
        return self.w_gate_up, True

    def last_product(self):
        return self.w_down, self.w_gate_up, True          # the down product follows the gate/up kernel

    def forward(self, h, ctx=None, residual=None, then_norm=None):
        """`h` may be ops.NormedRows; then_norm as for the attention part."""
        n = h.shape[0]
        act = torch.empty((n, self.intermediate_size), dtype=self.runtime.dtype, device=h.device)
        ops.gate_up_swiglu(h, self.w_gate_up, act)
        # the down product runs directly behind the gate/up product: ops is told so and keeps both on
        # one kernel family
        before = ops.Preceding(h.xw if isinstance(h, ops.NormedRows) else h, self.w_gate_up, swiglu=True)
        if residual is not None:
            if then_norm is not None:
                return ops.linear(act, self.w_down, out=residual, accumulate=True, then_norm=then_norm)
            ops.linear(act, self.w_down, out=residual, accumulate=True, follow=before)
            return None
        return ops.linear(act, self.w_down, out_dtype=torch.float32, follow=before)


@register_part("ffn", "dense_act")
class DenseAct(FeedForward):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.activation = params["activation"]
        if self.activation not in ops.ACT:
            raise ValueError(f"dense_act: unknown activation {self.activation!r}")
        self.w_up = self.w_down = None

    def expected_tensors(self):
        F, d = self.intermediate_size, self.hidden_size
        return {self.prefix + "up": ((F, d), "matrix"), self.prefix + "down": ((d, F), "matrix")}

    def load(self, tensors):
        self.w_up = self._to_device(tensors[self.prefix + "up"])
        self.w_down = self._to_device(tensors[self.prefix + "down"])

    def forward(self, h, ctx=None, residual=None):
        up = ops.linear(h, self.w_up, out_dtype=torch.float32)
        act = torch.empty(up.shape, dtype=self.runtime.dtype, device=h.device)
        ops.rows_act(up, act, act=self.activation)
        return ops.linear(act, self.w_down, out_dtype=torch.float32)


@register_part("ffn", "clamped_glu")
class ClampedGLU(FeedForward):
    """Gated feed-forward with clamped branches:

        g = min(h . Wg^T, limit),  u = clamp(h . Wu^T, -limit, limit)
        out = (g * sigmoid(alpha * g) * (u + shift)) . Wd^T

    With `activation` "gelu_tanh" the gate's factor g sigmoid(alpha g) is the tanh form of gelu instead,
    0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) (alpha is then not used).

    Parameters: hidden_size, intermediate_size, limit (0: no clamp), alpha, shift, activation.  Tensors
    <prefix>gate, <prefix>up, <prefix>down; gate and up are stacked into one [2F, hidden] matrix."""
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.limit = float(params.get("limit", 0.0) or 0.0)
        self.alpha = float(params.get("alpha", 1.0))
        self.shift = float(params.get("shift", 0.0))
        act = params.get("activation") or "sigmoid"
        if act not in ("sigmoid", "gelu_tanh"):
            raise ValueError(f"clamped_glu: activation {act!r} is not known ('sigmoid', 'gelu_tanh')")
        if act == "gelu_tanh":
            self.alpha = ops.GLU_GELU_TANH[1]           # the kernels' mark for the tanh form of gelu
        elif self.alpha == 0.0:
            raise ValueError("clamped_glu: alpha must not be 0")
        self.w_gate_up = self.w_down = None

    def expected_tensors(self):
        F, d, p = self.intermediate_size, self.hidden_size, self.prefix
        return {p + "gate": ((F, d), "matrix"), p + "up": ((F, d), "matrix"), p + "down": ((d, F), "matrix")}

    def load(self, tensors):
        p, dt = self.prefix, self.runtime.dtype
        self.w_gate_up = self._to_device(torch.cat([tensors[p + "gate"].to(dt), tensors[p + "up"].to(dt)], 0))
        self.w_down = self._to_device(tensors[p + "down"])

    def forward(self, h, ctx=None, residual=None):
        act = torch.empty((h.shape[0], self.intermediate_size), dtype=self.runtime.dtype, device=h.device)
        ops.gate_up_swiglu(h, self.w_gate_up, act, glu=(self.limit, self.alpha, self.shift))
        return ops.linear(act, self.w_down, out_dtype=torch.float32)
