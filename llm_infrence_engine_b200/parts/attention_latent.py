"""Attention whose keys and values are rebuilt from one small latent vector per token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import PagedKVSpec
from .base import INIT_NORM, INIT_SMALL, MATRIX, VECTOR, Mixer, ParamSpec, PositionEncoding, Source


class LatentAttention(Mixer):
    """Per token the cache holds one row ``[c | r]``: the normed latent ``c`` (``kv_rank``) and one rotated key part ``r``
    (``rot_dim``) that all heads share. Head ``h`` has the key ``[Uk_h c | r]`` and the value ``Uv_h c``; a query is
    ``[q_h | rot(q'_h)]`` with ``q = Uq norm(Dq x)``.

    Nothing per head is ever made for a cached token. Because ``q_h . (Uk_h c) = (Uk_h^T q_h) . c``, the query is carried
    into the latent space (``latent_absorb``), the attention runs over the cache rows as they lie, with ONE key/value
    head whose values are the first ``kv_rank`` entries of its keys, and ``Uv_h`` is applied to the attention's result
    (``latent_expand``, which also multiplies by the output gate ``sigmoid(g x)``, one number per element).

    * rotation: neighbouring pairs ``(2i, 2i + 1)`` of the first ``position.head_dim`` rotated entries;
    * ``window``: a position sees itself and the ``window - 1`` before it;
    * ``sink``: one learned number per head whose exponential joins the softmax's denominator (no key, no value).

    The three projections of the input (query latent, key/value latent with the rotated part, gate) are one matrix; both
    latent norms, the rotation of ``r`` and the cache write are one kernel.

    ``q_rank = 0``: the queries come straight from the input, ``q = W_q x`` (``{prefix}.q``), with no latent and no norm of their own.
    ``gate``: ``"element"`` (one number per entry of the result), ``"head"`` (``{prefix}.g`` has one row per head; the attention over
    the latents applies it, which is the same since the step back out of the latent space is linear) or None.
    """

    graph_safe = True

    def __init__(self, hidden: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, q_rank: int, kv_rank: int,
                 scale: float, eps: float, position: Optional[PositionEncoding], prefix: str, window: Optional[int] = None,
                 sink: bool = True, gate: Optional[str] = "element"):
        if gate not in ("element", "head", None):
            raise ValueError(f"a latent attention's gate is per 'element', per 'head' or None, got {gate!r}")
        self.hidden, self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim = hidden, num_heads, head_dim, rot_dim, v_head_dim
        self.q_rank, self.kv_rank, self.scale, self.eps = q_rank, kv_rank, float(scale), float(eps)
        self.position, self.prefix, self.window, self.has_sink = position, prefix, window, sink
        self.rot_dims = position.head_dim if position is not None else 0
        if self.rot_dims > rot_dim:
            raise ValueError(f"{self.rot_dims} rotated dimensions do not fit the rotated part of {rot_dim}")
        self.gate = gate
        self.g_col = q_rank + kv_rank + rot_dim
        self.g_rows = {"element": num_heads * v_head_dim, "head": num_heads, None: 0}[gate]
        for name in ("w_in", "w_q", "w_uq", "w_uk", "w_uv", "w_o", "q_norm", "kv_norm", "sink"):
            setattr(self, name, None)

    def params(self) -> Dict[str, ParamSpec]:
        p, h, H = self.prefix, self.hidden, self.num_heads
        joined = (Source(f"{p}.dkv", (self.kv_rank + self.rot_dim, h)),)
        if self.q_rank:
            joined = (Source(f"{p}.dq", (self.q_rank, h)),) + joined
        if self.gate:
            joined += (Source(f"{p}.g", (self.g_rows, h)),)
        out = {"w_in": ParamSpec(joined, MATRIX)}
        if self.q_rank:
            out["q_norm"] = ParamSpec((Source(f"{p}.dq.norm", (self.q_rank,), INIT_NORM),), VECTOR)
            out["w_uq"] = ParamSpec((Source(f"{p}.uq", (H * (self.head_dim + self.rot_dim), self.q_rank)),), MATRIX)
        else:
            out["w_q"] = ParamSpec((Source(f"{p}.q", (H * (self.head_dim + self.rot_dim), h)),), MATRIX)
        out.update({
            "kv_norm": ParamSpec((Source(f"{p}.dkv.norm", (self.kv_rank,), INIT_NORM),), VECTOR),
            "w_uk": ParamSpec((Source(f"{p}.uk", (H * self.head_dim, self.kv_rank)),), MATRIX),
            "w_uv": ParamSpec((Source(f"{p}.uv", (H * self.v_head_dim, self.kv_rank)),), MATRIX),
            "w_o": ParamSpec((Source(f"{p}.o", (h, H * self.v_head_dim)),), MATRIX),
        })
        if self.has_sink:
            out["sink"] = ParamSpec((Source(f"{p}.sink", (H,), INIT_SMALL),), VECTOR)
        return out

    def bind(self, tensors) -> None:
        super().bind(tensors)
        # per head [kv_rank, v_head_dim]: the layout in which ``latent_expand`` reads it (as ``w_uk`` is [head_dim, kv_rank] per head)
        self.w_uv = tensors["w_uv"].view(self.num_heads, self.v_head_dim, self.kv_rank).transpose(1, 2).contiguous()
        pad = -self.w_in.shape[0] % 8 if not self.q_rank else 0   # (rows of the product that start on a 16-byte boundary)
        if pad:
            self.w_in = torch.cat([self.w_in, self.w_in.new_zeros((pad, self.w_in.shape[1]))]).contiguous()

    def cache_spec(self):
        return PagedKVSpec(1, self.kv_rank + self.rot_dim, self.window, 0)

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        cos, sin = ctx.position_tables(self.position) if self.position is not None else (None, None)
        z = K.linear(h, self.w_in, out_dtype=ctx.dtype)      # [query latent | key/value latent, rotated part | gate]
        cq = K.latent_prepare(z, self.q_rank, self.kv_rank, self.rot_dim, self.rot_dims, self.q_norm, self.kv_norm, self.eps, cos, sin,
                              ctx.slot_mapping[cache.group], cache.k, ctx.page_size, cache.write)
        q = K.linear(cq, self.w_uq, out_dtype=ctx.dtype) if self.q_rank else K.linear(h, self.w_q, out_dtype=ctx.dtype)
        q_lat = K.latent_absorb(q, self.w_uk, cos, sin, self.num_heads, self.head_dim, self.rot_dim, self.rot_dims, self.kv_rank)
        per_head = self.gate == "head"
        o_lat = K.attention_ext(q_lat, 0, self.num_heads, 1, self.kv_rank + self.rot_dim, self.kv_rank, cache.k, None,
                                ctx.block_tables[cache.group], ctx.token_seq, ctx.positions, ctx.page_size, self.scale,
                                self.window or 0, ctx.max_context, sink=self.sink, batch=ctx, gate=z if per_head else None,
                                gate_col=self.g_col, gate_per_head=per_head)
        o = K.latent_expand(o_lat, self.w_uv, z if self.gate == "element" else None, self.g_col, self.num_heads, self.kv_rank, self.v_head_dim)
        K.linear(o, self.w_o, add_to=residual)
