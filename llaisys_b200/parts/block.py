from __future__ import annotations

from .base import Block, register_part


@register_part("block", "pre_norm_residual")
class PreNormResidual(Block):
    """x -> norm -> part -> + for every sub-layer in turn; with a mixer and a feed-forward that is
    x -> norm -> mixer -> +x -> norm -> feed-forward -> +   (xsmccc/llaisys
    src/models/qwen2/layer.hpp:47-84).  A part that can add its result to the residual stream in its
    own last kernel does so (forward_into); otherwise the add is done by the norm that follows, so
    the block hands its last delta on to the next block (or to the final norm).  A sub-layer
    without a norm of its own gets the residual stream as it is (the pending delta added)."""
    capturable = True

    def forward(self, residual, pending, ctx, users):
        from .. import kernels
        if isinstance(pending, PendingNormed):
            pending = settle(residual, pending)
        mixers = iter(users)
        for sub in self.sublayers:
            if sub.norm is not None:
                h = sub.norm.forward(residual, pending)
            else:
                if pending is not None:
                    kernels.residual_add(residual, pending)
                h = residual.to(self.env.dtype)
            if sub.category == "mixer":
                call = next(mixers)
                pending = None if sub.part.forward_into(h, ctx, call, residual) else sub.part.forward(h, ctx, call)
            else:
                pending = None if sub.part.forward_into(h, ctx, residual) else sub.part.forward(h, ctx)
        return residual, pending


@register_part("block", "parallel_residual")
class ParallelResidual(Block):
    """x -> x + sum over the sub-layers of part(norm(x)): every sub-layer reads the same stream, each through a norm
    of its own.  The norms are computed first, all from one root mean square per row (they differ in their weights
    only) in one pass over the stream; after that the parts may add into the stream in any order, each in its own
    last kernel where it can.  Needs norms that are RMS norms with one eps."""
    capturable = True

    def forward(self, residual, pending, ctx, users):
        from .. import kernels
        if isinstance(pending, PendingNormed):
            pending = settle(residual, pending)
        if pending is not None:
            kernels.residual_add(residual, pending)
        norms = [sub.norm for sub in self.sublayers]
        if any(n is None or n.kind != "rms_norm" or n.eps != norms[0].eps for n in norms):
            raise ValueError("a parallel layer needs an RMS norm with the same eps ahead of every sub-layer")
        hs = []
        for i in range(0, len(norms), 2):
            hs += kernels.rmsnorm_multi(residual, [n.weight for n in norms[i:i + 2]], norms[0].eps, self.env.dtype)
        mixers = iter(users)
        for sub, h in zip(self.sublayers, hs):
            if sub.category == "mixer":
                call = next(mixers)
                if not sub.part.forward_into(h, ctx, call, residual):
                    kernels.residual_add(residual, sub.part.forward(h, ctx, call))
            elif not sub.part.forward_into(h, ctx, residual):
                kernels.residual_add(residual, sub.part.forward(h, ctx))
        return residual, None


@register_part("block", "sandwich_residual")
class SandwichResidual(Block):
    """x -> x + mult * post_norm(part(norm(x))) for every sub-layer in turn: each part sits between a norm of its input
    and a norm of its output, and the normed output is scaled by the layer's constant `mult` before it joins the float32
    stream.  Output norm, add and the next sub-layer's input norm are one pass over the row (Norm.forward_scaled_add);
    the layer's last part leaves its output pending with its norm, and the block after it (or the final norm) runs
    that pass, so a layer costs one norm launch per part.  params: mult."""
    capturable = True

    def __init__(self, sublayers, env, params=None):
        super().__init__(sublayers, env, params)
        self.mult = float(self.params.get("mult", 1.0))
        for sub in self.sublayers:
            if sub.norm is None or sub.post_norm is None:
                raise ValueError("every sub-layer of this arrangement has a norm before and a norm after its part")

    def forward(self, residual, pending, ctx, users):
        mixers = iter(users)
        h = None
        for i, sub in enumerate(self.sublayers):
            if i == 0:
                h = settle(residual, pending, sub.norm)
            if sub.category == "mixer":
                delta = sub.part.forward(h, ctx, next(mixers))
            else:
                delta = sub.part.forward(h, ctx)
            if i + 1 < len(self.sublayers):
                h = sub.post_norm.forward_scaled_add(residual, delta, self.mult, then=self.sublayers[i + 1].norm)
            else:
                pending = PendingNormed(delta, sub.post_norm, self.mult)
        return residual, pending


class PendingNormed:
    """A part's output that has not joined the stream yet: it is to be normed by `norm`, scaled by `mult` and added."""

    def __init__(self, delta, norm, mult):
        self.delta, self.norm, self.mult = delta, norm, mult


def settle(residual, pending, norm=None, rows=None):
    """Adds whatever the block before left pending to the float32 stream and returns `norm` of the result (None without
    a norm).  With `rows` only those rows are returned (the stream itself is still brought up to date)."""
    from .. import kernels
    if isinstance(pending, PendingNormed):
        if rows is None:
            try:
                return pending.norm.forward_scaled_add(residual, pending.delta, pending.mult, then=norm)
            except ValueError:
                pass                                    # norms of different kinds: two passes
        pending.norm.forward_scaled_add(residual, pending.delta, pending.mult)
        pending = None
    if norm is None:
        if pending is not None:
            kernels.residual_add(residual, pending)
        return None
    return norm.forward(residual, pending, rows=rows)
