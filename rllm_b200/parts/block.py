"""How a layer's parts are arranged.  ``pre_norm``:

    x += pending;  a = mixer(norm_mixer(x));  x += a;  f = ffn(norm_ffn(x));  pending = f

A mixer or feed-forward is handed the float32 residual stream as `residual`; it may add its
output into it itself (its last product accumulates into x) and return None, or ignore it and
return its output, which the next norm then adds in the same kernel that normalizes
(AxiomOperator/rllm fuses the next layer's norm into the residual add:
crates/rllm-model/src/qwen3.rs:192-208).

With the block parameter ``residual_mult`` = m (a constant of the model, the same for all its
layers) a sublayer's output joins the stream multiplied by m: x += m * mixer(norm(x)), x += m *
ffn(norm(x)); the multiplication happens inside the norm kernel that adds the output (and in the
model's final norm, or a junction, for the last one).  A layer whose spec has no feed-forward
has the mixer sublayer only.  Such blocks take the plain path below (no deferred norms, no
accumulation into the stream by the products).

``post_norm`` (further down) puts the norms on the sublayers' outputs instead, ``sandwich_norm`` on both
sides of each sublayer, and ``sum_norm`` (at the end of this file) behind the residual sums, so that the
normed rows are the stream.

A block's interface: ``__init__(layer_spec, runtime)`` builds its parts from the registries;
``parts()`` lists them; ``forward(x, pending, ctx, cache) -> pending``.

Optional, for blocks that set ``DEFERS_NORM``: ``entry()`` returns the block's first norm and the
part behind it, and ``forward`` takes ``next_entry`` (the same pair of the block that runs next).
A norm that stands between two weight-streaming products of a decode step then needs no kernel of
its own: the product before it prepares it (``then_norm``) and hands the rows on as
``ops.NormedRows``, which the product after it divides by the rms.  ``pending`` is then that
object: the residual stream is complete and the next block's first norm is under way.  Whether
this happens is decided per step from the parts on both sides (``first_product`` / ``last_product``,
``deferrable``) and the number of rows; parts or norms without these methods get the plain path.
"""
from __future__ import annotations

from ..csrc import ops
from .base import build_part, register_part


def deferral(before, norm, after, m: int):
    """(weight, eps) if `norm`, between the parts `before` and `after`, can be deferred at m rows."""
    last, first, able = (getattr(before, "last_product", None), getattr(after, "first_product", None),
                         getattr(norm, "deferrable", None))
    if last is None or first is None or able is None or before.runtime.is_f32:
        return None
    w_before, w_lead, swiglu_lead = last()
    w_after, swiglu_after = first()
    if not ops.defers_norm(m, w_before, w_after, swiglu_after, w_lead, swiglu_lead):
        return None
    return able()


@register_part("block", "pre_norm")
class PreNormBlock:
    def __init__(self, layer_spec, runtime):
        self.residual_mult = float(dict(getattr(layer_spec, "block_params", None) or {}).get("residual_mult", 1.0))
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime)
        self.ffn = build_part("ffn", layer_spec.ffn, runtime) if layer_spec.ffn is not None else None
        self.norm_ffn = build_part("norm", layer_spec.norms["ffn"], runtime) if self.ffn is not None else None
        self.position = (build_part("position", layer_spec.position, runtime)
                         if layer_spec.position is not None else None)
        # the fused arrangements (products that add into the stream, norms without a kernel, recorded
        # layers) are those of the unscaled two-sublayer block
        self.scaled = self.residual_mult != 1.0 or self.ffn is None
        if self.scaled:
            self.DEFERS_NORM = self.TRACEABLE = False
        self.CAPTURE_SAFE = all(getattr(p, "CAPTURE_SAFE", False) for p in self.parts())

    def parts(self):
        ps = [self.norm_mixer, self.mixer]
        if self.ffn is not None:
            ps += [self.norm_ffn, self.ffn]
        if self.position is not None:
            ps.append(self.position)
        return ps

    DEFERS_NORM = True
    CAPTURE_SAFE = True
    TRACEABLE = True

    def entry(self):
        return self.norm_mixer, self.mixer

    def _forward_scaled(self, x, pending, ctx, cache):
        s = self.residual_mult
        h = self.norm_mixer.forward(x, pending, delta_scale=s)
        a = self.mixer.forward(h, ctx, cache, self.position)
        if self.ffn is None:
            return a
        h = self.norm_ffn.forward(x, a, delta_scale=s)
        return self.ffn.forward(h, ctx)

    def forward(self, x, pending, ctx, cache, next_entry=None):
        if self.scaled:
            return self._forward_scaled(x, pending, ctx, cache)
        m = x.shape[0]
        h = pending if isinstance(pending, ops.NormedRows) else self.norm_mixer.forward(x, pending)
        later = deferral(self.mixer, self.norm_ffn, self.ffn, m)
        if later is not None:
            h = self.mixer.forward(h, ctx, cache, self.position, residual=x, then_norm=later)
        else:
            a = self.mixer.forward(h, ctx, cache, self.position, residual=x)
            h = self.norm_ffn.forward(x, a)
        later = deferral(self.ffn, next_entry[0], next_entry[1], m) if next_entry is not None else None
        if later is not None:
            return self.ffn.forward(h, ctx, residual=x, then_norm=later)
        return self.ffn.forward(h, ctx, residual=x)


@register_part("block", "post_norm")
class OutputNormBlock:
    """The norms stand on the sublayers' outputs and the sublayers read the stream itself:

        x += norm_mixer(mixer(x));  x += norm_ffn(ffn(x))        (a spec without a feed-forward: the first only)

    The stream is float32; a product's operand is the stream rounded to the activation type.  The
    kernel that joins a sublayer's normed output to the stream also writes that rounded copy for the
    sublayer after it, and leaves it in the pass's scratch for the block that follows; only the
    first block of a pass makes its own.  Nothing is owed to the stream when the block returns
    (`pending` is None on both sides)."""

    CAPTURE_SAFE = True
    TRACEABLE = False
    DEFERS_NORM = False

    def __init__(self, layer_spec, runtime):
        self.runtime = runtime
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime)
        self.ffn = build_part("ffn", layer_spec.ffn, runtime) if layer_spec.ffn is not None else None
        self.norm_ffn = build_part("norm", layer_spec.norms["ffn"], runtime) if self.ffn is not None else None
        self.position = (build_part("position", layer_spec.position, runtime)
                         if layer_spec.position is not None else None)
        self.CAPTURE_SAFE = all(getattr(p, "CAPTURE_SAFE", False) for p in self.parts())

    def parts(self):
        ps = [self.norm_mixer, self.mixer]
        if self.ffn is not None:
            ps += [self.norm_ffn, self.ffn]
        if self.position is not None:
            ps.append(self.position)
        return ps

    def _operand(self, x, ctx):
        """The stream as a product's operand: itself in float32, else its rounded copy."""
        import torch
        if self.runtime.is_f32:
            return x, None
        key = ("stream_copy", x.data_ptr())
        h = ctx.scratch.get(key)
        if h is None:
            h = ctx.scratch[key] = torch.empty(x.shape, dtype=self.runtime.dtype, device=x.device)
            ops.rows_act(x, h)                     # a plain conversion
        return h, h

    def forward(self, x, pending, ctx, cache):
        if pending is not None:
            raise ValueError("post_norm: the block before still owes the stream something; it joins its outputs itself")
        h, copy = self._operand(x, ctx)
        a = self.mixer.forward(h, ctx, cache, self.position)
        self.norm_mixer.join(x, a, copy)           # x and its copy are the new stream
        if self.ffn is not None:
            f = self.ffn.forward(h, ctx)
            self.norm_ffn.join(x, f, copy)
        return None


class PreparedRows:
    """What a ``sandwich_norm`` block hands the block after it: the stream is complete and `h` holds the
    rows of the next block's first norm already (made by the kernel that joined the last output)."""
    __slots__ = ("h",)

    def __init__(self, h):
        self.h = h


@register_part("block", "sandwich_norm")
class SandwichNormBlock:
    """A norm before AND after each sublayer:

        x += norm_mixer_out(mixer(norm_mixer(x)));  x += norm_ffn_out(ffn(norm_ffn(x)))

    (a spec without a feed-forward: the first only).  The stream is float32.  The kernel that joins a
    sublayer's normed output to the stream also makes the rows of the norm that reads the stream next
    (`Norm.join_then`): the feed-forward's first norm, and the first norm of the block that follows
    when that block is one of this kind (`next_entry`), which then gets them as `PreparedRows`.
    Nothing is owed to the stream when the block returns."""

    CAPTURE_SAFE = True
    TRACEABLE = False
    DEFERS_NORM = True            # the model hands `next_entry` to blocks that say so

    def __init__(self, layer_spec, runtime):
        self.runtime = runtime
        norms = layer_spec.norms
        self.norm_mixer = build_part("norm", norms["mixer"], runtime)
        self.norm_mixer_out = build_part("norm", norms["mixer_out"], runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime)
        self.ffn = build_part("ffn", layer_spec.ffn, runtime) if layer_spec.ffn is not None else None
        self.norm_ffn = build_part("norm", norms["ffn"], runtime) if self.ffn is not None else None
        self.norm_ffn_out = build_part("norm", norms["ffn_out"], runtime) if self.ffn is not None else None
        self.position = (build_part("position", layer_spec.position, runtime)
                         if layer_spec.position is not None else None)
        self.CAPTURE_SAFE = all(getattr(p, "CAPTURE_SAFE", False) for p in self.parts())

    def parts(self):
        ps = [self.norm_mixer, self.norm_mixer_out, self.mixer]
        if self.ffn is not None:
            ps += [self.norm_ffn, self.norm_ffn_out, self.ffn]
        if self.position is not None:
            ps.append(self.position)
        return ps

    def entry(self):
        return self.norm_mixer, self.mixer

    @staticmethod
    def _join(norm_out, x, y, norm_next):
        """x += norm_out(y); the rows of norm_next(x) if that norm can be made in the same kernel."""
        if norm_next is not None and hasattr(norm_out, "join_then") and hasattr(norm_next, "deferrable"):
            return norm_out.join_then(x, y, norm_next)
        norm_out.join(x, y)
        return None

    def forward(self, x, pending, ctx, cache, next_entry=None):
        if isinstance(pending, PreparedRows):
            h = pending.h
        elif pending is not None:
            raise ValueError("sandwich_norm: the block before still owes the stream something; "
                             "blocks of this kind join their outputs themselves")
        else:
            h = self.norm_mixer.forward(x)
        a = self.mixer.forward(h, ctx, cache, self.position)
        nxt = next_entry[0] if next_entry is not None else None
        if self.ffn is None:
            h = self._join(self.norm_mixer_out, x, a, nxt)
            return PreparedRows(h) if h is not None else None
        h = self._join(self.norm_mixer_out, x, a, self.norm_ffn)
        if h is None:
            h = self.norm_ffn.forward(x)
        f = self.ffn.forward(h, ctx)
        h = self._join(self.norm_ffn_out, x, f, nxt)
        return PreparedRows(h) if h is not None else None


@register_part("block", "sum_norm")
class SumNormBlock:
    """The norm stands AFTER the residual sum and its result is the stream:

        x <- norm_mixer(alpha * x + mixer(x));  x <- norm_ffn(alpha * x + ffn(x))     (no feed-forward: the first only)

    with `alpha` a constant of the model (block parameter, default 1).  The sublayers read the stream
    itself; the stream, the sum and the norm are float32, and a product's operand is the stream rounded to
    the activation type, which the kernel that norms a sum writes beside the stream (the first block of a
    pass makes its own copy).  Nothing is owed to the stream when the block returns."""

    CAPTURE_SAFE = True
    TRACEABLE = False
    DEFERS_NORM = False

    def __init__(self, layer_spec, runtime):
        self.runtime = runtime
        self.alpha = float(dict(getattr(layer_spec, "block_params", None) or {}).get("alpha", 1.0))
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime)
        self.ffn = build_part("ffn", layer_spec.ffn, runtime) if layer_spec.ffn is not None else None
        self.norm_ffn = build_part("norm", layer_spec.norms["ffn"], runtime) if self.ffn is not None else None
        self.position = (build_part("position", layer_spec.position, runtime)
                         if layer_spec.position is not None else None)
        for nm in (self.norm_mixer, self.norm_ffn):
            if nm is not None and not hasattr(nm, "sum_norm"):
                raise ValueError("sum_norm: the norm part must offer sum_norm(x, y, alpha, copy)")
        self.CAPTURE_SAFE = all(getattr(p, "CAPTURE_SAFE", False) for p in self.parts())

    parts = OutputNormBlock.parts
    _operand = OutputNormBlock._operand

    def forward(self, x, pending, ctx, cache):
        if pending is not None:
            raise ValueError("sum_norm: the block before still owes the stream something; it joins its outputs itself")
        h, copy = self._operand(x, ctx)
        a = self.mixer.forward(h, ctx, cache, self.position)
        self.norm_mixer.sum_norm(x, a, self.alpha, copy)        # x and its copy are the new stream
        if self.ffn is not None:
            f = self.ffn.forward(h, ctx)
            self.norm_ffn.sum_norm(x, f, self.alpha, copy)
        return None
