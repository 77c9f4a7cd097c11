"""Token embedding and LM head.

Embedding: x[t,:] = table[tokens[t],:] into the float32 residual stream, no scaling
(AxiomOperator/rllm: crates/rllm-model/src/qwen3.rs:191).  LM head: logits = rows . W^T in
float32, W its own tensor or, when `tied_to` names one, the embedding table
(crates/rllm-model/src/qwen3.rs:151-154, 232).

Options: the embedding may be followed by an RMSNorm of its own (`norm`: the weight's name,
`norm_eps`); the logits may be capped, logits <- softcap * tanh(logits / softcap) (`softcap`), or
multiplied by a constant (`scale`).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Part, register_part


@register_part("embedding", "embedding")
class Embedding(Part):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.name = params.get("tensor") or self.prefix + "weight"      # the table's name in the weight file
        self.norm_name = params.get("norm")                             # an RMSNorm on the looked-up rows, or None
        self.norm_eps = float(params.get("norm_eps", 1e-6))
        self.weight = self.norm_weight = None

    def expected_tensors(self):
        t = {self.name: ((self.vocab_size, self.hidden_size), "matrix")}
        if self.norm_name:
            t[self.norm_name] = ((self.hidden_size,), "norm")
        return t

    def load(self, tensors):
        self.weight = self._to_device(tensors[self.name])
        if self.norm_name:
            self.norm_weight = self._to_device(tensors[self.norm_name], torch.float32)

    def forward(self, tokens):
        out = torch.empty((tokens.numel(), self.hidden_size), dtype=torch.float32, device=tokens.device)
        ops.embed(self.weight, tokens, out, ops.error_word(tokens.device))
        if self.norm_weight is not None:
            ops.norm_rows(out, self.norm_weight, self.norm_eps, x=out)       # in place
        return out


@register_part("lm_head", "lm_head")
class LMHead(Part):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.name = params.get("tensor") or self.prefix + "weight"
        self.softcap = float(params.get("softcap", 0.0) or 0.0)
        self.scale = float(params.get("scale", 1.0))
        self.weight = None

    def expected_tensors(self):
        if self.tied_to:
            return {}
        return {self.name: ((self.vocab_size, self.hidden_size), "matrix")}

    def ignorable_tensors(self):
        """A tied model may still store the head; it is not read."""
        return {self.name} if self.tied_to else set()

    def load(self, tensors, shared=None):
        if self.tied_to:
            self.weight = shared[self.tied_to]
        else:
            self.weight = self._to_device(tensors[self.name])

    def forward(self, h):
        """h [m, hidden] normed rows -> float32 logits [m, vocab]."""
        logits = ops.linear(h, self.weight, out_dtype=torch.float32)
        if self.softcap > 0.0:
            ops.softcap_rows(logits, self.softcap)
        if self.scale != 1.0:
            ops.axpby(self.scale, logits, 0.0, logits, logits)
        return logits
