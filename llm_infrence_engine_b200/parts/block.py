"""One layer: how norms, mixer and feed-forward are arranged around the residual stream."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .base import INIT_NORM, VECTOR, FeedForward, Mixer, Norm, ParamSpec, Part, Source


class PreNormBlock(Part):
    """``x += mixer(norm1(x)); x += ff(norm2(x))`` (src/miniserve/model.py:184-185).

    The residual stream ``x`` is 32-bit and is updated in place: the mixer and the feed-forward are handed
    ``x`` and add their result into it themselves, which lets their last matrix product do the addition
    in its own epilogue instead of a kernel of its own.

    With a layer scale (``scale1`` / ``scale2`` name vectors of ``dim`` entries): ``x += scale1 * mixer(norm1(x))`` and
    ``x += scale2 * ff(norm2(x))``, element by element. The sublayer then adds its result into a zeroed tensor as it would into the
    stream, and the scaled addition is put off until the next norm of the stream, whose kernel adds and normalises in one pass.
    """

    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm] = None, ff: Optional[FeedForward] = None,
                 scale1: Optional[str] = None, scale2: Optional[str] = None, dim: int = 0):
        if (norm2 is None) != (ff is None):
            raise ValueError("a feed-forward comes with its norm, or neither is there")
        if (scale1 or scale2) and dim <= 0:
            raise ValueError("a layer scale needs the width of the stream")
        if scale2 and ff is None:
            raise ValueError("a layer scale of the feed-forward needs a feed-forward")
        self.norm1, self.mixer, self.norm2, self.ff = norm1, mixer, norm2, ff
        self.scale1_name, self.scale2_name, self.dim = scale1, scale2, int(dim)
        self.scale1: Optional[torch.Tensor] = None
        self.scale2: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        out = {}
        if self.scale1_name:
            out["scale1"] = ParamSpec((Source(self.scale1_name, (self.dim,), INIT_NORM),), VECTOR)
        if self.scale2_name:
            out["scale2"] = ParamSpec((Source(self.scale2_name, (self.dim,), INIT_NORM),), VECTOR)
        return out

    def children(self) -> Sequence[Part]:
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.ff) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, residual: torch.Tensor, cache) -> None:
        K = ctx.K
        h = self.norm1.norm(ctx, residual)
        if self.scale1 is None:
            self.mixer.forward(ctx, h, cache, residual)
        else:
            y = K.zeros_like_rows(residual)
            self.mixer.forward(ctx, h, cache, y)
            K.scaled_add(residual, y, self.scale1)
        if self.ff is not None:   # a layer may be a mixer alone
            h = self.norm2.norm(ctx, residual)
            if self.scale2 is None:
                self.ff.forward(ctx, h, residual)
            else:
                y = K.zeros_like_rows(residual)
                self.ff.forward(ctx, h, y)
                K.scaled_add(residual, y, self.scale2)


class SandwichBlock(Part):
    """``x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x)))``: a norm before every sublayer and another on its result.

    A sublayer adds its result into a zeroed tensor exactly as it would add into the residual stream (so any mixer or
    feed-forward of the package fits); the closing norm then adds the normed result into the stream. The closing norms have
    ``add_normed(ctx, residual, y)``.
    """

    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm1b: Norm, norm2: Optional[Norm] = None, ff: Optional[FeedForward] = None,
                 norm2b: Optional[Norm] = None):
        if (norm2 is None) != (ff is None) or (norm2b is None) != (ff is None):
            raise ValueError("a feed-forward comes with its two norms, or none of the three is there")
        self.norm1, self.mixer, self.norm1b, self.norm2, self.ff, self.norm2b = norm1, mixer, norm1b, norm2, ff, norm2b

    def children(self) -> Sequence[Part]:
        return tuple(p for p in (self.norm1, self.mixer, self.norm1b, self.norm2, self.ff, self.norm2b) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, residual: torch.Tensor, cache) -> None:
        K = ctx.K
        h = self.norm1.norm(ctx, residual)
        y = K.zeros_like_rows(residual)
        self.mixer.forward(ctx, h, cache, y)
        self.norm1b.add_normed(ctx, residual, y)
        if self.ff is not None:
            h = self.norm2.norm(ctx, residual)
            y = K.zeros_like_rows(residual)
            self.ff.forward(ctx, h, y)
            self.norm2b.add_normed(ctx, residual, y)


class ParallelBlock(Part):
    """``h = norm(x); x += mixer(h) + ff(h)``: one norm, and both sublayers read its output. Each sublayer adds its result into
    the 32-bit stream itself, so the sum of the two is never a tensor of its own; a layer may be a mixer alone."""

    graph_safe = True

    def __init__(self, norm: Norm, mixer: Mixer, ff: Optional[FeedForward] = None):
        self.norm, self.mixer, self.ff = norm, mixer, ff

    def children(self) -> Sequence[Part]:
        return tuple(p for p in (self.norm, self.mixer, self.ff) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, residual: torch.Tensor, cache) -> None:
        h = self.norm.norm(ctx, residual)   # (the stream is read here, before either sublayer adds into it)
        self.mixer.forward(ctx, h, cache, residual)
        if self.ff is not None:
            self.ff.forward(ctx, h, residual)
