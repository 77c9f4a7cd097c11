"""RMSNorm with the residual add fused in.

out = v * (1 / sqrt(mean(v^2) + eps)) * weight, v = x (+ delta); the weight multiplies
directly (no 1 + w), statistics in float32 (AxiomOperator/rllm:
crates/rllm-cpu/src/lib.rs:241-254; the fusion with the residual add is
crates/rllm-cuda/kernels/kernels.cu:794-820 and crates/rllm-model/src/qwen3.rs:202-208).
Parameters: size, eps, optionally `tensor` (the weight's full name) and `one_plus` (the stored
weight lies around zero and multiplies as 1 + w; the sum is formed once, in float32, at load).  Tensor: <prefix>weight
[size], kept in float32.  `delta_scale`: the delta joins the stream multiplied by it.  `join(x, y)`: the norm of a sublayer's
output, x += norm(y) * weight.  `sum_norm(x, y, alpha)`: the norm behind the sum, x = norm(alpha x + y) * weight.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, register_part


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    CAPTURE_SAFE = True
    TRACEABLE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = params.get("tensor") or self.prefix + "weight"
        self.one_plus = bool(params.get("one_plus", False))
        self.weight = None

    def expected_tensors(self):
        return {self.name: ((self.size,), "norm0" if self.one_plus else "norm")}

    def load(self, tensors):
        w = tensors[self.name].to(torch.float32)
        self.weight = self._to_device(1.0 + w if self.one_plus else w, torch.float32)

    def deferrable(self):
        """(weight, eps) for a product kernel that prepares this norm in its epilogue (the division by
        the rms then happens in the product after it: csrc/ops.NormedRows)."""
        return self.weight, self.eps

    def join(self, x, y, copy=None):
        """x += y / rms(y) * weight: the norm stands on a sublayer's OUTPUT `y` as it joins the float32
        stream `x` (in place).  `copy`, if given, also takes the new x in its own type (the operand of
        the next product).  Returns `copy`, or x."""
        return ops.norm_rows(y, self.weight, self.eps, x=x, add=True, low=copy)

    def sum_norm(self, x, y, alpha=1.0, copy=None):
        """x <- (alpha * x + y) / rms(alpha * x + y) * weight: the norm stands behind the residual sum and
        the normed rows are the float32 stream `x` (in place); `copy`, if given, also takes them in its own
        type (the operand of the next product)."""
        return ops.sum_norm_rows(x, y, alpha, self.weight, self.eps, low=copy)

    def join_then(self, x, y, nxt):
        """x += y / rms(y) * weight, and in the same kernel the rows of the norm `nxt` of the new x (in
        the runtime's type): a norm on a sublayer's output followed by the norm in front of the next
        sublayer."""
        w_next, eps_next = nxt.deferrable()
        out = torch.empty(x.shape, dtype=self.runtime.dtype, device=x.device)
        return ops.join_norm_rows(y, self.weight, self.eps, x, w_next, eps_next, out)

    def forward(self, x, delta=None, rows=None, write_x=True, delta_scale=1.0):
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=self.runtime.dtype, device=x.device)
        return ops.add_rms_norm(x, delta, self.weight, out, self.eps, rows=rows, write_x=write_x,
                                delta_scale=delta_scale)
