"""Rotate-half (NeoX) rotary position encoding over the whole head.

inv_freq[i] = 1 / theta^(2i / head_dim) for i < head_dim/2; the angle of pair (i, i + head_dim/2)
at position p is p * inv_freq[i], computed in float32 (AxiomOperator/rllm:
crates/rllm-cpu/src/lib.rs:256-290).  The part owns the inv_freq table; the rotation itself
is applied inside the mixer's fused kernel, which receives the table.
Parameters: head_dim, theta.  No tensors.

A position part's interface, either of:

``apply_and_store(qkv, q_norm_w, k_norm_w, eps, ctx, cache, q_out, H, K, head_dim)``: the
part itself turns the fused projection rows ``qkv`` [n, (H + 2K) * head_dim] (float32) into the
queries ``q_out`` [n, H * head_dim] and writes keys and values to ``cache`` (a PagedKVView: ``k``,
``v``, ``slots``, ``block_size``, ``write``) at the step's slots, applying the per-head q/k norm
(if the weights are given) before its own encoding; ``ctx`` is the step's StepContext (positions in
``ctx.positions``; ``ctx.scratch`` is a dictionary that lives for one forward pass, for what the
layers of the pass can share).  Any scheme can be written this way, with
kernels of its own or on top of ``ops.qk_norm_rope_store`` (which, without a table, norms and
stores without rotating).

``project_and_store(h, w_qkv, ...same arguments...) -> bool`` (optional): as apply_and_store, but the
part is given the rows before the fused projection and the projection's matrix, and may do the
projection too (one kernel with the norm, the encoding and the cache write in its epilogue); it
returns False when it does not take the step.

``table()``: for schemes of the form "rotate pairs (i, i + head_dim/2) by position * table[i]":
the float32 vector of head_dim/2 entries that the fused kernel takes; the mixer then calls the
kernel itself.  This part offers both.
"""
from __future__ import annotations

import torch

from .base import Part, PartError, register_part


@register_part("position", "rotary_neox")
class RotaryNeox(Part):
    CAPTURE_SAFE = True
    TRACEABLE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        if self.head_dim % 2:
            raise PartError(f"rotary_neox: head_dim {self.head_dim} must be even")
        i = torch.arange(0, self.head_dim, 2, dtype=torch.float32)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), i / self.head_dim)
        self.inv_freq = inv.to(runtime.device)

    def table(self):
        return self.inv_freq

    def _angles(self, ctx):
        """(cos, sin) of the step's tokens: the same in every layer with this table, so once per pass."""
        from ..csrc import ops
        key = ("rotary_neox", self.head_dim, self.theta)
        table = ctx.scratch.get(key)
        if table is None:
            with ops.untraced():                  # once per pass, not once per layer that replays this one
                table = ctx.scratch[key] = ops.rope_table(ctx.positions, self.inv_freq)
        return table

    def apply_and_store(self, qkv, q_norm_w, k_norm_w, eps, ctx, cache, q_out, H, K, head_dim):
        from ..csrc import ops
        return ops.qk_norm_rope_store(qkv, q_norm_w, k_norm_w, None, ctx.positions, cache.slots, q_out,
                                      cache.k, cache.v, H, K, head_dim, cache.block_size, eps, write_kv=cache.write,
                                      cs_table=self._angles(ctx))

    def project_and_store(self, h, w_qkv, q_norm_w, k_norm_w, eps, ctx, cache, q_out, H, K, head_dim) -> bool:
        """Optional third form of a position part's interface: the part also does the q/k/v projection
        h . w_qkv^T itself, so that it can be one kernel with what follows it.  Returns False when it
        does not take the step (the mixer then projects and calls apply_and_store)."""
        from ..csrc import ops
        if not ops.can_fuse_qkv(h, w_qkv, head_dim, q_out, cache.k):
            return False
        ops.qkv_norm_rope_store_fused(h, w_qkv, q_norm_w, k_norm_w, self._angles(ctx), cache.slots, q_out, cache.k,
                                      cache.v, H, K, head_dim, cache.block_size, eps, write_kv=cache.write)
        return True


@register_part("position", "rotary_scaled")
class RotaryScaled(Part):
    """Rotary encoding over the first `dims` entries of a head (the rest pass), with optional
    YaRN-style frequency scaling.  `layout` "half" (default): entry i turns with entry i + dims/2;
    "pairs": entry 2i turns with entry 2i + 1.  In both, the pair (u, v) at position p becomes
    (u cos a - v sin a, v cos a + u sin a) with a = p * f_i.

    f_i = base^(-2i / dims) for i < dims/2.  With `scaling` = {factor, original, fast, slow}: let
    dim(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(dim(fast)), 0),
    hi = min(ceil(dim(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); pair
    i then turns with f_i / factor * ramp_i + f_i * (1 - ramp_i), and cos and sin are multiplied by
    `mult` = 0.1 ln(factor) + 1.  With `scaling` = {factor, low, high, original} (the long-context rule
    of Llama 3.1) a pair's wavelength l = 2 pi / f_i decides: l < original / high keeps f_i; l >
    original / low turns with f_i / factor; between the two, with s = (original / l - low) / (high - low),
    with (1 - s) f_i / factor + s f_i; cos and sin are not multiplied.  Frequencies are worked out in
    double precision on the host and rounded once; angles (position * frequency), cos and sin are float32
    on the device.

    Parameters: dims, base, scaling (or None), layout.  No tensors.  The part offers `table()` (the
    frequencies), `mult` and `angles(ctx)` (cos, sin per token and pair, once per pass) to mixers whose
    own kernel applies them, and `apply_and_store` to the attention part: RMS norm per head with a
    weight, then the rotation, queries out, keys and values (heads of `v_head_dim` entries) into the
    pages; `has_kv` False: the rows hold queries only."""
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        import math
        self.dims = int(params["dims"])
        self.base = float(params["base"])
        if self.dims <= 0 or self.dims % 2:
            raise PartError(f"rotary_scaled: dims {self.dims} must be positive and even")
        half = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        self.mult = 1.0
        sc = params.get("scaling")
        if sc and "low" in sc:
            factor, original, low, high = (float(sc[k]) for k in ("factor", "original", "low", "high"))
            if not high > low > 0 or not factor > 0 or not original > 0:
                raise PartError("rotary_scaled: scaling needs factor > 0, original > 0 and high > low > 0")
            for i in range(half):
                wave = 2.0 * math.pi / f[i]
                if wave > original / low:
                    f[i] = f[i] / factor
                elif wave >= original / high:
                    s = (original / wave - low) / (high - low)
                    f[i] = (1.0 - s) * f[i] / factor + s * f[i]
        elif sc:
            factor, original = float(sc["factor"]), float(sc["original"])

            def dim_of(turns):
                return self.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
            lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
            hi = min(math.ceil(dim_of(float(sc["slow"]))), self.dims - 1)
            for i in range(half):
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
            self.mult = 0.1 * math.log(factor) + 1.0
        self.layout = params.get("layout") or "half"
        if self.layout not in ("half", "pairs"):
            raise PartError(f"rotary_scaled: layout {self.layout!r} is not known ('half', 'pairs')")
        self._key = ("rotary_scaled", self.dims, tuple(f))
        self.freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def table(self):
        return self.freq

    def angles(self, ctx):
        """(cos, sin) [n, dims/2, 2] of the step's tokens, shared by the layers with these frequencies."""
        from ..csrc import ops
        table = ctx.scratch.get(self._key)
        if table is None:
            with ops.untraced():
                table = ctx.scratch[self._key] = ops.rope_table(ctx.positions, self.freq)
        return table

    def apply_and_store(self, qkv, q_norm_w, k_norm_w, eps, ctx, cache, q_out, H, K, head_dim, v_head_dim=None,
                        has_kv=True):
        from ..csrc import ops
        if self.mult != 1.0:
            raise PartError("rotary_scaled: apply_and_store does not take scaled frequencies")
        return ops.head_norm_rope_store(qkv, q_norm_w, k_norm_w, self.angles(ctx), min(self.dims, head_dim),
                                        self.layout == "pairs", cache.slots, q_out, cache.k, cache.v, H, K, head_dim,
                                        v_head_dim or head_dim, cache.block_size, eps, has_kv=has_kv,
                                        write_kv=cache.write)
