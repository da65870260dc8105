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
