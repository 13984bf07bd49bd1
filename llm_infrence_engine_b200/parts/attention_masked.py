"""Grouped-query attention with partly rotated heads and a mask that is more than causal."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import FixedStateSpec, PagedKVSpec
from .base import INIT_EYE, INIT_NORM, INIT_PROJ, INIT_SMALL, INIT_TAPS, MATRIX, VECTOR, Mixer, ParamSpec, PositionEncoding, Source


class MaskedAttention(Mixer):
    """``o(softmax(cap(scale * q k^T) + mask) v)`` over a paged cache, ``num_heads`` query heads sharing ``num_kv_heads``
    key/value heads (query head ``h`` reads key/value head ``h // (num_heads // num_kv_heads)``), no biases. Options, each off
    unless asked for:

    * ``conv_taps``: a short causal convolution per channel on q, k and v right after their projection (no bias, no
      activation); a request's last ``conv_taps - 1`` projected rows are part of its state;
    * ``qk_norm``: RMS norm of every query and key head with a weight of ``head_dim`` entries shared by the heads, before rotation;
    * ``position``: a rotary encoding with ``dims`` and ``tables`` (cos, sin of ``[N, dims / 2]``); the first ``dims`` entries of a
      head turn, the rest pass; pairs are ``(i, i + dims/2)``, or neighbours ``(2i, 2i+1)`` when ``interleaved``;
    * ``window`` with ``keep_first``: position i sees ``j <= i`` with ``i - j < window`` or ``j < keep_first``;
    * ``chunk``: position i sees ``j <= i`` with ``floor(i / chunk) == floor(j / chunk)``;
    * ``softcap``: the scaled score s becomes ``softcap * tanh(s / softcap)``;
    * keys and values may differ in size (``head_dim``, ``v_head_dim``);
    * ``talking_heads``: the heads' scaled and capped scores at one (query, key) pair are mixed before mask and softmax,
      ``score'_h = sum_g talk[h, g] score_g`` with ``talk [heads, heads]`` (``{prefix}.talk``);
    * ``sink``: a learned number per head (``{prefix}.sink``) whose exponential joins the softmax's denominator once: it has no key and
      no value and is neither scaled nor capped nor mixed;
    * ``head_gate``: head h's result is multiplied by ``sigmoid(W_g x)_h`` (``{prefix}.g``, one row per head, read from the mixer's input).

    The three projections are one matrix; norm, rotation and the cache write are one kernel; the mask is never a tensor.
    Pages that neither window nor chunk can reach any more go back to the pool as a request moves on.
    """

    graph_safe = True

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, scale: float, prefix: str,
                 position: Optional[PositionEncoding] = None, interleaved: bool = False, window: Optional[int] = None, keep_first: int = 0,
                 chunk: Optional[int] = None, softcap: Optional[float] = None, conv_taps: int = 0, qk_norm: bool = False, eps: float = 1e-6,
                 talking_heads: bool = False, sink: bool = False, head_gate: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        if keep_first and not window:
            raise ValueError("first tokens can only be kept where a window would pass them")
        if position is not None and position.dims > head_dim:
            raise ValueError(f"{position.dims} rotated dimensions do not fit heads of {head_dim}")
        if conv_taps and not 1 <= conv_taps <= 8:
            raise ValueError(f"a short convolution has 1 to 8 taps, got {conv_taps}")
        self.hidden, self.num_heads, self.num_kv_heads = hidden, num_heads, num_kv_heads
        self.head_dim, self.v_head_dim, self.scale, self.prefix = head_dim, v_head_dim, float(scale), prefix
        self.position, self.interleaved = position, bool(interleaved)
        self.window, self.keep_first, self.chunk = window, int(keep_first), chunk
        self.softcap = float(softcap) if softcap else 0.0
        self.conv_taps, self.qk_norm, self.eps = int(conv_taps), bool(qk_norm), float(eps)
        self.channels = (num_heads + num_kv_heads) * head_dim + num_kv_heads * v_head_dim
        self.talking_heads, self.has_sink, self.head_gate = bool(talking_heads), bool(sink), bool(head_gate)
        self.talk: Optional[torch.Tensor] = None
        self.sink: Optional[torch.Tensor] = None
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.conv_w: Optional[torch.Tensor] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.k_norm: Optional[torch.Tensor] = None

    def _rows(self):
        return (("q", self.num_heads * self.head_dim), ("k", self.num_kv_heads * self.head_dim), ("v", self.num_kv_heads * self.v_head_dim))

    def params(self) -> Dict[str, ParamSpec]:
        p, h = self.prefix, self.hidden
        joined = tuple(Source(f"{p}.{n}", (r, h), INIT_PROJ) for n, r in self._rows())
        if self.head_gate:   # the gate's rows ride behind q, k and v in the joined projection
            joined += (Source(f"{p}.g", (self.num_heads, h), INIT_PROJ),)
        out = {"w_qkv": ParamSpec(joined, MATRIX),
               "w_o": ParamSpec((Source(f"{p}.o", (h, self.num_heads * self.v_head_dim), INIT_PROJ),), MATRIX)}
        if self.talking_heads:
            out["talk"] = ParamSpec((Source(f"{p}.talk", (self.num_heads, self.num_heads), INIT_EYE),), VECTOR)
        if self.has_sink:
            out["sink"] = ParamSpec((Source(f"{p}.sink", (self.num_heads,), INIT_SMALL),), VECTOR)
        if self.conv_taps:
            out["conv_w"] = ParamSpec(tuple(Source(f"{p}.{n}.conv", (r, self.conv_taps), INIT_TAPS) for n, r in self._rows()), VECTOR)
        if self.qk_norm:
            out["q_norm"] = ParamSpec((Source(f"{p}.q.norm", (self.head_dim,), INIT_NORM),), VECTOR)
            out["k_norm"] = ParamSpec((Source(f"{p}.k.norm", (self.head_dim,), INIT_NORM),), VECTOR)
        return out

    def bind(self, tensors) -> None:
        super().bind(tensors)
        pad = -self.w_qkv.shape[0] % 8   # (rows of the product that start on a 16-byte boundary)
        if pad:
            self.w_qkv = torch.cat([self.w_qkv, self.w_qkv.new_zeros((pad, self.w_qkv.shape[1]))]).contiguous()

    def cache_spec(self):
        pages = PagedKVSpec(self.num_kv_heads, self.head_dim, self.window, self.v_head_dim, self.keep_first, self.chunk)
        if self.conv_taps:
            return (pages, FixedStateSpec((self.conv_taps - 1, self.channels)))
        return pages

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        kv, conv_state = cache if self.conv_taps else (cache, None)
        z = K.linear(h, self.w_qkv, out_dtype=ctx.dtype)
        gate = z if self.head_gate else None   # (its columns lie behind the heads, from ``channels`` on)
        if self.conv_taps:
            z = K.causal_conv(z, 0, self.channels, self.conv_w, None, conv_state.state, ctx)
        cos = sin = None
        dims = 0
        if self.position is not None:
            cos, sin = ctx.position_tables(self.position)
            dims = self.position.dims
        q = K.qk_norm_rope_store(z, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim, self.q_norm, self.k_norm, self.eps, cos, sin,
                                 dims, self.interleaved, ctx.slot_mapping[kv.group], kv.k, kv.v, ctx.page_size, write_kv=kv.write)
        attn = K.attention_ext(q, 0, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim, kv.k, kv.v, ctx.block_tables[kv.group],
                               ctx.token_seq, ctx.positions, ctx.page_size, self.scale, self.window or 0, ctx.max_context, batch=ctx,
                               keep_first=self.keep_first, chunk=self.chunk or 0, softcap=self.softcap, sink=self.sink, gate=gate,
                               gate_col=self.channels, gate_per_head=True, talk=self.talk)
        K.linear(attn, self.w_o, add_to=residual)
