"""Routed experts: a feed-forward made of many small gated feed-forwards of which each token uses a few.

For normed input rows h [n, d], E experts of size F, each token using `top_k`:

    z = h Wr^T (+ a stored bias per expert: `router_bias`)  (float32);  s = sigmoid(z)  (or softmax over the
        experts: `score`; softmax scores of the chosen experts divided by their sum are the softmax over the
        chosen logits alone)
    choice scores c = s + correction                     (`correction`: a stored vector, else none)
    experts form `n_groups` equal groups of neighbours; a group's score is the sum of its `group_best`
        largest c; only experts of the `keep_groups` best groups can be chosen (the others count as
        minus infinity)
    the `top_k` experts with the largest c are chosen;  their weights are their s (without the
        correction), divided by their sum + `weight_eps` when `normalize`, times `route_scale`
    expert e:  y_e = Wd_e (silu(Wg_e h) * (Wu_e h))
    out = sum over the chosen e of weight_e * y_e
          + sigmoid(h . w_sg) * shared(h)                (`shared_size` > 0: one more expert of that size
                                                          for every token; `shared_gate`: its gate)

Parameters: hidden_size, intermediate_size, num_experts, top_k, n_groups, keep_groups, group_best, score,
correction, normalize, weight_eps, route_scale, shared_size, shared_gate, router_bias.  Tensors under <prefix>:
router [E, d], router.b [E], correction [E], e<i>.gate, e<i>.up [F, d], e<i>.down [d, F], shared.gate, shared.up,
shared.down, shared.sg [1, d].  Load-time transform: the experts' matrices are stacked ([E, 2F, d] gate
rows then up rows, [E, d, F]), and the shared expert's gate row is stacked under the router's so that
one product gives both (with rows of zeros up to a multiple of 8 rows).  The router's logits, scores, choice
and weights are float32 in every mode.

Steps of few rows run every (token, chosen expert) pair against its expert's matrices directly, with no
host involvement (so such steps can be captured into graphs).  Steps of many rows sort the pairs by
expert on the device, read the experts' counts back and run each expert's rows through the package's
products.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, PartError, register_part

PAIR_ROWS = 64           # up to this many rows a step takes the pair kernels


@register_part("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    CAPTURE_SAFE = True       # steps that are captured have few rows (see PAIR_ROWS and the engine's graph limits)

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden_size, self.F, self.E = int(p["hidden_size"]), int(p["intermediate_size"]), int(p["num_experts"])
        self.top_k = int(p["top_k"])
        self.n_groups, self.keep_groups = int(p.get("n_groups", 1)), int(p.get("keep_groups", 1))
        self.group_best = int(p.get("group_best", 2))
        self.score = p.get("score", "sigmoid")
        self.has_correction = bool(p.get("correction", False))
        self.has_bias = bool(p.get("router_bias", False))
        self.normalize = bool(p.get("normalize", True))
        self.weight_eps = float(p.get("weight_eps", 0.0))
        self.route_scale = float(p.get("route_scale", 1.0))
        self.shared_size = int(p.get("shared_size", 0) or 0)
        self.shared_gate = bool(p.get("shared_gate", False)) and self.shared_size > 0
        if self.E % self.n_groups or not 0 < self.keep_groups <= self.n_groups:
            raise PartError(f"routed_experts: {self.E} experts do not form {self.n_groups} equal groups "
                            f"of which {self.keep_groups} are kept")
        if not 0 < self.top_k <= self.keep_groups * (self.E // self.n_groups):
            raise PartError(f"routed_experts: top_k {self.top_k} exceeds the experts of the kept groups")
        self.router_bias = None
        self.w_router = self.correction = self.w_gu = self.w_down = self.w_shared_gu = self.w_shared_down = None

    def expected_tensors(self):
        d, F, p = self.hidden_size, self.F, self.prefix
        t = {p + "router": ((self.E, d), "matrix")}
        if self.has_correction:
            t[p + "correction"] = ((self.E,), "unit")
        if self.has_bias:
            t[p + "router.b"] = ((self.E,), "unit")
        for e in range(self.E):
            t.update({f"{p}e{e}.gate": ((F, d), "matrix"), f"{p}e{e}.up": ((F, d), "matrix"),
                      f"{p}e{e}.down": ((d, F), "matrix")})
        if self.shared_size:
            S = self.shared_size
            t.update({p + "shared.gate": ((S, d), "matrix"), p + "shared.up": ((S, d), "matrix"),
                      p + "shared.down": ((d, S), "matrix")})
            if self.shared_gate:
                t[p + "shared.sg"] = ((1, d), "matrix")
        return t

    def load(self, tensors):
        p, dt = self.prefix, self.runtime.dtype
        router = [tensors[p + "router"].to(dt)]
        if self.shared_gate:
            router.append(tensors[p + "shared.sg"].to(dt).reshape(1, -1))
        rows = sum(r.shape[0] for r in router)
        if rows % 8:                # rows of zeros up to a multiple of 8: the logits' rows are then aligned for every product kernel
            router.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=dt, device=router[0].device))
        self.w_router = self._to_device(torch.cat(router, 0))
        if self.has_correction:
            self.correction = self._to_device(tensors[p + "correction"], torch.float32)
        if self.has_bias:
            self.router_bias = self._to_device(tensors[p + "router.b"], torch.float32)
        self.w_gu = self._to_device(torch.stack(
            [torch.cat([tensors[f"{p}e{e}.gate"].to(dt), tensors[f"{p}e{e}.up"].to(dt)], 0) for e in range(self.E)], 0))
        self.w_down = self._to_device(torch.stack([tensors[f"{p}e{e}.down"].to(dt) for e in range(self.E)], 0))
        if self.shared_size:
            self.w_shared_gu = self._to_device(torch.cat([tensors[p + "shared.gate"].to(dt),
                                                          tensors[p + "shared.up"].to(dt)], 0))
            self.w_shared_down = self._to_device(tensors[p + "shared.down"])

    def route(self, h):
        """(idx int32 [n, top_k], weight float32 [n, top_k], logits float32 [n, E (+ 1), padded to a multiple of 8])."""
        n, dev = h.shape[0], h.device
        logits = ops.linear(h, self.w_router, out_dtype=torch.float32)
        idx = torch.empty((n, self.top_k), dtype=torch.int32, device=dev)
        weight = torch.empty((n, self.top_k), dtype=torch.float32, device=dev)
        ops.moe_route(logits, self.correction, idx, weight, self.E, self.top_k, self.n_groups, self.keep_groups,
                      self.group_best, self.score, self.normalize, self.weight_eps, self.route_scale, bias=self.router_bias)
        return idx, weight, logits

    def forward(self, h, ctx=None, residual=None):
        n, d, dev, dt = h.shape[0], self.hidden_size, h.device, self.runtime.dtype
        idx, weight, logits = self.route(h)
        shared = gate = None
        if self.shared_size:
            act = torch.empty((n, self.shared_size), dtype=dt, device=dev)
            ops.gate_up_swiglu(h, self.w_shared_gu, act)
            shared = ops.linear(act, self.w_shared_down, out_dtype=torch.float32)
            gate = logits[:, self.E:self.E + 1] if self.shared_gate else None
        out = torch.empty((n, d), dtype=torch.float32, device=dev)
        if n <= PAIR_ROWS or torch.cuda.is_current_stream_capturing():
            act = torch.empty((n * self.top_k, self.F), dtype=dt, device=dev)
            ops.moe_pairs_gate_up(h, self.w_gu, idx, act)
            return ops.moe_pairs_down(act, self.w_down, idx, weight, out, shared, gate)
        # many rows: the pairs in expert order, each expert's rows through the package's products
        offsets, place = ops.moe_sort(idx, self.E)
        rows = torch.empty((n * self.top_k, d), dtype=dt, device=dev)
        ops.moe_gather_rows(h, place, rows, self.top_k)
        bounds = offsets.tolist()                          # the host learns how many rows each expert has
        act = torch.empty((n * self.top_k, self.F), dtype=dt, device=dev)
        y = torch.empty((n * self.top_k, d), dtype=torch.float32, device=dev)
        for e in range(self.E):
            a, b = bounds[e], bounds[e + 1]
            if b > a:
                ops.gate_up_swiglu(rows[a:b], self.w_gu[e], act[a:b])
                ops.linear(act[a:b], self.w_down[e], out=y[a:b])
        return ops.moe_combine(y, place, weight, out, shared, gate)
