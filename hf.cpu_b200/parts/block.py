"""Residual arrangements.  Pre-norm: ``x += mixer(norm1(x)); x += ffn(norm2(x))`` (src/model.c:580-623).
Norm on both sides of each sublayer: ``x += post1(mixer(norm1(x))); x += post2(ffn(norm2(x)))``, where a layer may
have no feed-forward at all."""
from __future__ import annotations

import torch

from .base import Block, register_part


class PreNormResidual(Block):
    graph_safe = True

    def __init__(self, **_):
        pass

    def forward(self, ctx, x, norm1, mixer, norm2, ffn, cache, state, write_cache, xn_ready=None, next_norm=None):
        if xn_ready is None:
            xn = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            norm1.forward(x, xn)
        else:
            xn = xn_ready
        if ffn is None:
            # a layer that is a mixer only: the norm behind its product is the next block's first
            fused = getattr(mixer, "forward_then_norm", None) if next_norm is not None else None
            if not fused:
                mixer.forward(ctx, xn, x, cache, state, write_cache)
                return None
            nxt = ctx.buf("block_xn", x.shape, ctx.run_dtype)       # (xn may live there: the mixer has read it by then)
            if not fused(ctx, xn, x, cache, state, write_cache, next_norm, nxt):
                next_norm.forward(x, nxt)
            return nxt
        xn2 = ctx.buf("block_xn2", x.shape, ctx.run_dtype)
        fused = getattr(mixer, "forward_then_norm", None)
        if not (fused and fused(ctx, xn, x, cache, state, write_cache, norm2, xn2)):
            if not fused:
                mixer.forward(ctx, xn, x, cache, state, write_cache)
            norm2.forward(x, xn2)
        fused = getattr(ffn, "forward_then_norm", None) if next_norm is not None else None
        if fused:
            nxt = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            if not fused(ctx, xn2, x, next_norm, nxt):
                next_norm.forward(x, nxt)
            return nxt
        ffn.forward(ctx, xn2, x)
        return None


class SandwichResidual(Block):
    """``x += post1(mixer(norm1(x)))``, then, if the layer has a feed-forward, ``x += post2(ffn(norm2(x)))``.  The
    sublayers write their output to a float32 buffer (``accumulate=False``) instead of adding it to the stream; the
    post-norm adds it, and where it can it hands back the following norm of the new stream from the same pass."""
    graph_safe = True

    def __init__(self, **_):
        pass

    def forward(self, ctx, x, norm1, mixer, norm2, ffn, cache, state, write_cache, xn_ready=None, next_norm=None,
                post1=None, post2=None):
        if post1 is None or (ffn is not None and post2 is None):
            raise ValueError("this block needs a norm behind each sublayer")
        if xn_ready is None:
            xn = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            norm1.forward(x, xn)
        else:
            xn = xn_ready
        y = ctx.buf("block_y", x.shape, torch.float32)
        # A part whose output is a product may hand that product to the norm behind it (``forward_into_norm``), which
        # then sums the product's partial sums in its own pass; else the part stores its output in y and the norm adds it.
        # Either way the norm returns whether the following norm of the new stream came out of the same pass.
        fused_norms = hasattr(post1, "add_product_into")

        def mix(following, out):
            into = getattr(mixer, "forward_into_norm", None) if fused_norms else None
            if into is not None:
                return into(ctx, xn, cache, state, write_cache, y, x, post1, following, out)
            mixer.forward(ctx, xn, y, cache, state, write_cache, accumulate=False)
            return post1.add_into(y, x, following, out)

        def feed_forward(xin, following, out):
            into = getattr(ffn, "forward_into_norm", None) if fused_norms else None
            if into is not None:
                return into(ctx, xin, y, x, post2, following, out)
            ffn.forward(ctx, xin, y, accumulate=False)
            return post2.add_into(y, x, following, out)

        nxt = ctx.buf("block_xn", x.shape, ctx.run_dtype) if next_norm is not None else None
        if ffn is None:
            return nxt if mix(next_norm, nxt) else None
        xn2 = ctx.buf("block_xn2", x.shape, ctx.run_dtype)
        if not mix(norm2, xn2):
            norm2.forward(x, xn2)
        return nxt if feed_forward(xn2, next_norm, nxt) else None


register_part("block", "prenorm_residual", PreNormResidual)
register_part("block", "sandwich_residual", SandwichResidual)
