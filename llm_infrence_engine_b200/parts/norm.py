"""Normalisation of rows of the 32-bit residual stream: root mean square, and layer norm with a weight."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import INIT_NORM, INIT_SMALL, VECTOR, Norm, ParamSpec, Source


class RMSNorm(Norm):
    """``y = weight * cast(x * rsqrt(mean(x^2) + eps))`` with the mean and the scaling in 32-bit.

    The reference reduces in 32-bit, casts to the model's dtype and multiplies by the weight there
    (src/miniserve/model.py:69-73). ``eps`` sits inside the square root, added to the mean.

    ``offset``: what is added to the stored weight before it is used. A checkpoint that keeps its norm weights around zero
    (the scaling is ``1 + w``) has ``offset = 1``; the sum is made once, in 32-bit, when the weights are bound.

    ``norm_streams``: the norm of a weighted sum of several residual streams ``[N, streams, dim]``, everything in 32-bit up
    to the one rounding of the result (the kernel also carries out a stream update that was put off until now).
    """

    graph_safe = True

    def __init__(self, dim: int, eps: float, weight_name: str, offset: float = 0.0):
        self.dim = dim
        self.eps = float(eps)
        self.weight_name = weight_name
        self.offset = float(offset)
        self.weight: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        init = INIT_NORM if self.offset == 0.0 else INIT_SMALL
        return {"weight": ParamSpec((Source(self.weight_name, (self.dim,), init),), VECTOR)}

    def bind(self, tensors) -> None:
        self.weight = tensors["weight"] + self.offset if self.offset else tensors["weight"]

    def norm_streams(self, ctx, streams, coef, rows=None):
        return ctx.K.streams_norm(streams, coef, self.weight, self.eps, ctx.dtype, rows)

    def norm(self, ctx, residual):
        return ctx.K.add_rmsnorm(residual, None, self.weight, self.eps, ctx.dtype)

    def norm_rows(self, ctx, residual, rows):
        return ctx.K.rmsnorm_rows(residual, None, self.weight, self.eps, rows, ctx.dtype)


class LayerNorm(Norm):
    """``y = (x - mean) / sqrt(var + eps) * weight`` (``+ bias`` where ``bias_name`` names one), the variance being the mean
    squared deviation; mean, variance and scaling in 32-bit, one rounding of the result.

    The same norm also closes a sublayer: ``add_normed(ctx, residual, y)`` is ``residual += norm(y)``. That addition is put
    off until the next norm of the stream, whose kernel adds and normalises in one pass.
    """

    graph_safe = True

    def __init__(self, dim: int, eps: float, weight_name: str, bias_name: Optional[str] = None):
        self.dim, self.eps, self.weight_name, self.bias_name = dim, float(eps), weight_name, bias_name
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        out = {"weight": ParamSpec((Source(self.weight_name, (self.dim,), INIT_NORM),), VECTOR)}
        if self.bias_name is not None:
            out["bias"] = ParamSpec((Source(self.bias_name, (self.dim,), INIT_SMALL),), VECTOR)
        return out

    def norm(self, ctx, residual):
        if self.bias is None:
            return ctx.K.layernorm(residual, self.weight, self.eps, ctx.dtype)
        return ctx.K.layernorm(residual, self.weight, self.eps, ctx.dtype, bias=self.bias)

    def norm_rows(self, ctx, residual, rows):
        if self.bias is None:
            return ctx.K.layernorm(residual, self.weight, self.eps, ctx.dtype, rows)
        return ctx.K.layernorm(residual, self.weight, self.eps, ctx.dtype, rows, bias=self.bias)

    def add_normed(self, ctx, residual, y) -> None:
        if self.bias is not None:
            raise ValueError("a layer norm with a bias does not close a sublayer here")
        ctx.K.post_norm_add(residual, y, self.weight, self.eps)
