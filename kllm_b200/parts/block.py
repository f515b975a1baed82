"""Arrangements of a layer's parts.

``pre_norm``: x += mixer(norm1(x)); x += ff(norm2(x)), with the feed-forward's
output handed on as ``pending`` and added inside the next norm (the next layer's
first norm, or the model's final norm), as the reference does
(backend/model.cu:1068-1072, 1083-1089, 1105, 1117).

``output_norm``: x += norm1(mixer(x)); x += norm2(ff(x)), the sublayers reading the stream itself, with an
optional third sublayer that reads the step's token ids (``OutputNormBlock``).

Interface of a block: ``forward(x, pending, ctx, cache) -> pending'``.  x is the
float32 residual stream, updated in place; ``pending`` (float32 or model dtype, or
None) is what is still to be added to x.

A mixer or feed-forward may offer ``forward_residual`` (the part applies the norm and
adds its result into x itself, in whichever kernels fit the step's size); the block
uses it whenever nothing is pending.  The built-in attention and gated feed-forward
both offer it and always accept, so a Llama layer never hands anything on as
``pending``.  A part without it, or one that returns False, gets norm -> ``forward``
-> pending.  Both routes compute the same sums.

Two more optional methods let a part's kernels warm L2 for the kernels after them:
``streamed_weights()`` (the matrices a part streams in a small step, in kernel order)
and ``set_prefetch_targets(weights)`` (what runs right after the part).  The block
wires mixer -> feed-forward when it is bound, the model wires feed-forward -> the next
block's mixer through ``set_successor``.  A part without them is left alone.
"""
from __future__ import annotations

from .spec import BlockSpec, BuildEnv, part_factory, register_part


class PreNormBlock:
    def __init__(self, spec: BlockSpec, env: BuildEnv):
        self.mixer = part_factory("mixer", spec.mixer.kind)(spec.mixer, env)
        self.mixer_norm = part_factory("norm", spec.mixer_norm.kind)(spec.mixer_norm, env)
        self.feed_forward = self.ff_norm = None            # a layer may be its mixer alone
        if spec.feed_forward is not None:
            self.feed_forward = part_factory("feed_forward", spec.feed_forward.kind)(spec.feed_forward, env)
            self.ff_norm = part_factory("norm", spec.ff_norm.kind)(spec.ff_norm, env)

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    def tensor_specs(self):
        return [s for p in self.parts() for s in p.tensor_specs()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def bind(self, tensors):
        for p in self.parts():
            p.bind(tensors)
        self._wire(self.mixer, self.feed_forward)

    @staticmethod
    def _wire(part, following):
        """Tell ``part`` which weights the part after it streams, if both take part in
        that (optional methods ``set_prefetch_targets`` / ``streamed_weights``)."""
        tell, ask = getattr(part, "set_prefetch_targets", None), getattr(following, "streamed_weights", None)
        if tell is not None and ask is not None:
            tell(ask())

    def set_successor(self, block):
        """The block that runs after this one in the model's schedule."""
        self._wire(self.feed_forward, getattr(block, "mixer", None))

    def forward(self, x, pending, ctx, cache):
        fused = getattr(self.mixer, "forward_residual", None)
        if pending is None and fused is not None and fused(x, self.mixer_norm, ctx, cache):
            pending = None
        else:
            xn = self.mixer_norm.forward(x, pending)
            pending = self.mixer.forward(xn, ctx, cache)
        if self.feed_forward is None:
            return pending
        fused = getattr(self.feed_forward, "forward_residual", None)
        if pending is None and fused is not None and fused(x, self.ff_norm, ctx):
            return None
        xn = self.ff_norm.forward(x, pending)
        return self.feed_forward.forward(xn, ctx)


class DeferredNorm:
    """What a block still owes the residual stream: ``x += norm(y)``.  Whoever runs next may fold
    it into its own first norm (``norm.add_normed(x, y, then=...)``) or ``settle`` it."""

    accepted_by = "accepts_deferred_norm"      # the attribute by which a block says that it takes this hand-over

    def __init__(self, norm, y):
        self.norm, self.y = norm, y

    def settle(self, x):
        self.norm.add_normed(x, self.y)


class SandwichNormBlock:
    """``sandwich_norm``: a norm before AND after each sublayer,

        x += post1(mixer(pre1(x)));  x += post2(ff(pre2(x)))

    ``BlockSpec.mixer_norm`` / ``ff_norm`` are the norms in front; ``params`` holds
    ``mixer_post_norm`` and ``ff_post_norm`` (PartSpecs of the norm family whose parts offer
    ``add_normed``).  ``feed_forward`` may be None: the layer is its mixer alone.  The
    sublayers' outputs are float32; the norm behind the mixer and the norm in front of the
    feed-forward are one kernel, and so are the norm behind the layer's last sublayer and the
    first norm of the next block of this kind: the block hands on a ``DeferredNorm`` as its
    ``pending`` (``accepts_deferred_norm``; the model settles it before a block that does not take
    one, before its final norm, and for a debugging tap)."""

    accepts_deferred_norm = True

    def __init__(self, spec: BlockSpec, env: BuildEnv):
        def norm(ps):
            return part_factory("norm", ps.kind)(ps, env)
        self.mixer = part_factory("mixer", spec.mixer.kind)(spec.mixer, env)
        self.mixer_norm = norm(spec.mixer_norm)
        self.mixer_post = norm(spec.params["mixer_post_norm"])
        self.feed_forward = self.ff_norm = self.ff_post = None
        if spec.feed_forward is not None:
            self.feed_forward = part_factory("feed_forward", spec.feed_forward.kind)(spec.feed_forward, env)
            self.ff_norm = norm(spec.ff_norm)
            self.ff_post = norm(spec.params["ff_post_norm"])

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_post, self.ff_norm, self.feed_forward, self.ff_post)
                if p is not None]

    def tensor_specs(self):
        return [s for p in self.parts() for s in p.tensor_specs()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def bind(self, tensors):
        for p in self.parts():
            p.bind(tensors)

    def forward(self, x, pending, ctx, cache):
        if isinstance(pending, DeferredNorm):
            xn = pending.norm.add_normed(x, pending.y, then=self.mixer_norm)
        else:
            xn = self.mixer_norm.forward(x, pending)
        y = self.mixer.forward(xn, ctx, cache)
        if self.feed_forward is None:
            return DeferredNorm(self.mixer_post, y)
        xn = self.mixer_post.add_normed(x, y, then=self.ff_norm)
        return DeferredNorm(self.ff_post, self.feed_forward.forward(xn, ctx))


class ReadyRows:
    """Nothing is owed to the residual stream; the block before only hands on the stream's rows in the model
    dtype, which it formed in its last kernel, for a block that would otherwise form them again."""

    accepted_by = "accepts_ready_rows"

    def __init__(self, rows):
        self.rows = rows

    def settle(self, x):
        return None

    def peek(self, x):
        return x


class OutputNormBlock:
    """``output_norm``: a norm on each sublayer's OUTPUT only,

        x += norm1(mixer(x));  x += norm2(ff(x));  x += side_norm(side(x, token))

    The sublayers read the stream x itself (in the model dtype: for bfloat16 the rows rounded once, for
    float32 the stream).  ``BlockSpec.mixer_norm`` / ``ff_norm`` are the norms behind the mixer and the
    feed-forward (parts that offer ``add_normed``); ``feed_forward`` may be None.  ``params``: optional
    ``side`` (a PartSpec of the side_input family: a third sublayer that also reads the step's token ids,
    ``forward(h, ctx) -> float32 [n, hidden]``) with ``side_norm`` (its norm).  Every norm's kernel also
    stores the updated rows in the model dtype, the next sublayer's input, also across blocks (``ReadyRows``)."""

    accepts_ready_rows = True

    def __init__(self, spec: BlockSpec, env: BuildEnv):
        def norm(ps):
            return part_factory("norm", ps.kind)(ps, env)
        self.dtype = env.dtype
        self.mixer = part_factory("mixer", spec.mixer.kind)(spec.mixer, env)
        self.mixer_norm = norm(spec.mixer_norm)
        self.feed_forward = self.ff_norm = self.side = self.side_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = part_factory("feed_forward", spec.feed_forward.kind)(spec.feed_forward, env)
            self.ff_norm = norm(spec.ff_norm)
        side = spec.params.get("side")
        if side is not None:
            self.side = part_factory("side_input", side.kind)(side, env)
            self.side_norm = norm(spec.params["side_norm"])

    def parts(self):
        return [p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.ff_norm, self.side, self.side_norm)
                if p is not None]

    def tensor_specs(self):
        return [s for p in self.parts() for s in p.tensor_specs()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def bind(self, tensors):
        for p in self.parts():
            p.bind(tensors)

    def _rows(self, x):
        from .. import kernels
        import torch
        return x if self.dtype == torch.float32 else kernels.unary(x, "copy", self.dtype)

    def _join(self, norm, x, y):
        """x += norm(y); the updated rows in the model dtype (x itself when that is float32)."""
        import torch
        if self.dtype == torch.float32:
            norm.add_normed(x, y)
            return x
        return norm.add_normed(x, y, then="rows")

    def forward(self, x, pending, ctx, cache):
        if isinstance(pending, ReadyRows):
            h = pending.rows
        else:
            if hasattr(pending, "settle"):
                pending = pending.settle(x)
            if pending is not None:
                x.add_(pending.float())
            h = self._rows(x)
        h = self._join(self.mixer_norm, x, self._f32(self.mixer.forward(h, ctx, cache)))
        if self.feed_forward is not None:
            h = self._join(self.ff_norm, x, self._f32(self.feed_forward.forward(h, ctx)))
        if self.side is not None:
            h = self._join(self.side_norm, x, self._f32(self.side.forward(h, ctx)))
        return ReadyRows(h)

    @staticmethod
    def _f32(y):
        import torch
        return y if y.dtype == torch.float32 and y.is_contiguous() else y.float().contiguous()


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "output_norm", OutputNormBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
