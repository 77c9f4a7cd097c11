"""Token embedding and LM head.

Embedding: x[t,:] = table[tokens[t],:] into the float32 residual stream, no scaling
(AxiomOperator/rllm: crates/rllm-model/src/qwen3.rs:191).  LM head: logits = rows . W^T in
float32, W its own tensor or, when `tied_to` names one, the embedding table
(crates/rllm-model/src/qwen3.rs:151-154, 232).

Options: the embedding may be followed by an RMSNorm of its own (`norm`: the weight's name,
`norm_eps`); the logits may be capped, logits <- softcap * tanh(logits / softcap) (`softcap`), or
multiplied by a constant (`scale`).

The embedding may be multiplied by a constant (`scale`) and joined by a second table looked up by the
pair (previous token, token) (`pair`: {tensor, buckets, mul_prev, mul_cur}):

    x = table[token] * scale + pair_table[(previous * mul_prev + token * mul_cur) mod buckets]

with the table's last row (number `buckets`) for the first token of a sequence.  The previous token of
the first token a request brings in a step is part of the request's state: the part then asks the cache
manager for one int32 per request (`cache_need`), which the model hands it as a view like a mixer's.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Part, PartError, StateNeed, register_part


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
        self.scale = float(params.get("scale", 1.0))
        self.pair = dict(params["pair"]) if params.get("pair") else None
        if self.pair is not None:
            self.buckets = int(self.pair["buckets"])
            self.mul_prev, self.mul_cur = int(self.pair["mul_prev"]), int(self.pair["mul_cur"])
            if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
                raise PartError("embedding: pair.buckets must be positive, the multipliers not negative")
        self.weight = self.norm_weight = self.pair_weight = None

    def cache_need(self):
        """One int32 per request (the last token it has brought) when there is a pair table, else None."""
        return StateNeed((1,), torch.int32) if self.pair is not None else None

    def expected_tensors(self):
        t = {self.name: ((self.vocab_size, self.hidden_size), "matrix")}
        if self.norm_name:
            t[self.norm_name] = ((self.hidden_size,), "norm")
        if self.pair is not None:
            t[self.pair["tensor"]] = ((self.buckets + 1, self.hidden_size), "matrix")
        return t

    def load(self, tensors):
        self.weight = self._to_device(tensors[self.name])
        if self.norm_name:
            self.norm_weight = self._to_device(tensors[self.norm_name], torch.float32)
        if self.pair is not None:
            self.pair_weight = self._to_device(tensors[self.pair["tensor"]])

    def forward(self, tokens, ctx=None, cache=None):
        out = torch.empty((tokens.numel(), self.hidden_size), dtype=torch.float32, device=tokens.device)
        if self.pair is not None:
            if ctx is None or cache is None:
                raise PartError("embedding: a pair table needs the step's context and the requests' state")
            last = cache.state.view(-1)
            ops.embed_pair(self.weight, self.pair_weight, tokens, ctx.positions, ctx.seq_ids, ctx.cu_q, cache.slots, last,
                           out, self.scale, self.buckets, self.mul_prev, self.mul_cur, ops.error_word(tokens.device))
            ops.keep_last_tokens(tokens, ctx.cu_q, cache.slots, last, ctx.n_requests)
            return out
        ops.embed(self.weight, tokens, out, ops.error_word(tokens.device))
        if self.scale != 1.0:
            ops.axpby(self.scale, out, 0.0, out, out)
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
