"""Mixers that carry a state of fixed size from token to token, and two mixers side by side."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from ..cache.spec import FixedStateSpec
from .base import ANY, INIT_LOG_RATE, INIT_NORM, INIT_PROJ, INIT_SMALL, INIT_STEP_BIAS, INIT_TAPS, MATRIX, VECTOR, Mixer, ParamSpec, Part, Source


def _padded(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """Rows added so that every row of the product starts on a 16-byte boundary."""
    pad = -w.shape[0] % multiple
    return torch.cat([w, w.new_zeros((pad, w.shape[1]))]).contiguous() if pad else w


class GatedDeltaMixer(Mixer):
    """The gated delta rule with one decay per head AND key channel. With q, k of ``num_kv_heads x head_dim`` and v of
    ``num_heads x v_head_dim`` (head ``h`` uses q/k head ``h // (num_heads // num_kv_heads)``), each through a short causal
    convolution and SiLU, q and k then made unit vectors per head (``x / sqrt(sum x^2 + 1e-6)``, q also times ``head_dim^-1/2``):

        beta = sigmoid(W_b x)                                                  one per head
        g    = exp(-exp(A_log[h]) * softplus(W_a2 (W_a1 x) + dt_bias))         heads x head_dim
        S <- g (.) S (row d by g[d]);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q

    per head, ``S [head_dim, v_head_dim]`` starting at zero. Each head's ``o`` is divided by its root mean square, multiplied by
    a weight shared by the heads and by ``sigmoid(W_g2 (W_g1 x))``; then the output projection. The ranks of the two low-rank
    projections are read off the checkpoint. Decays, gates, unit norms and the state are 32-bit; a request's state is ``S`` and
    the convolution's last ``conv_taps - 1`` inputs.
    """

    graph_safe = True

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, conv_taps: int, eps: float, prefix: str,
                 random_rank: int = 16):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} query/key heads")
        if not 1 <= conv_taps <= 8:
            raise ValueError(f"a short convolution has 1 to 8 taps, got {conv_taps}")
        if head_dim > 256:
            raise ValueError(f"the delta rule's kernel keeps a column of the state in registers: head_dim {head_dim} is more than 256")
        self.hidden, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim = hidden, num_heads, num_kv_heads, head_dim, v_head_dim
        self.conv_taps, self.eps, self.prefix, self.random_rank = int(conv_taps), float(eps), prefix, random_rank
        self.qk = num_kv_heads * head_dim
        self.channels = 2 * self.qk + num_heads * v_head_dim      # what the convolution sees: q | k | v
        self.b_col = self.a1_col = self.g1_col = 0      # columns of the joined projection's sections: set when the weights are bound
        self.w_in = self.w_a2 = self.w_g2 = self.w_low2 = self.w_o = self.conv_w = self.A_log = self.dt_bias = self.norm_w = None

    def params(self) -> Dict[str, ParamSpec]:
        p, h, H, D, DV = self.prefix, self.hidden, self.num_heads, self.head_dim, self.v_head_dim
        rows = (("q", self.qk), ("k", self.qk), ("v", H * DV))
        r = self.random_rank
        return {
            "w_in": ParamSpec(tuple(Source(f"{p}.{n}", (c, h), INIT_PROJ) for n, c in rows)
                              + (Source(f"{p}.b", (H, h), INIT_PROJ), Source(f"{p}.a1", (ANY, h), INIT_PROJ, free=r),
                                 Source(f"{p}.g1", (ANY, h), INIT_PROJ, free=r)), MATRIX),
            "w_a2": ParamSpec((Source(f"{p}.a2", (H * D, ANY), INIT_PROJ, free=r),), MATRIX),
            "w_g2": ParamSpec((Source(f"{p}.g2", (H * DV, ANY), INIT_PROJ, free=r),), MATRIX),
            "w_o": ParamSpec((Source(f"{p}.o", (h, H * DV), INIT_PROJ),), MATRIX),
            "conv_w": ParamSpec(tuple(Source(f"{p}.{n}.conv", (c, self.conv_taps), INIT_TAPS) for n, c in rows), VECTOR),
            "A_log": ParamSpec((Source(f"{p}.A_log", (H,), INIT_LOG_RATE),), VECTOR),
            "dt_bias": ParamSpec((Source(f"{p}.dt_bias", (H * D,), INIT_STEP_BIAS),), VECTOR),
            "norm_w": ParamSpec((Source(f"{p}.norm", (DV,), INIT_NORM),), VECTOR),
        }

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_low2, self.w_o, self.conv_w, self.A_log, self.dt_bias, self.norm_w)
                   if t is not None)

    def bind(self, tensors) -> None:
        super().bind(tensors)
        self.rank_a, self.rank_g = self.w_a2.shape[1], self.w_g2.shape[1]
        rows = (self.channels, self.num_heads, self.rank_a, self.rank_g)
        if self.w_in.shape[0] != sum(rows):
            raise ValueError(f"{self.prefix}: the two halves of a low-rank projection do not agree on its rank")
        # every section of the joined projection starts on a multiple of 8 rows: its columns of the product then start on a
        # 16-byte boundary, and the second halves of the low-rank projections can read them where they lie
        pieces, starts, at = [], [], 0
        for part in torch.split(self.w_in, rows):
            starts.append(at)
            pieces.append(_padded(part))
            at += pieces[-1].shape[0]
        _, self.b_col, self.a1_col, self.g1_col = starts
        self.w_in = torch.cat(pieces).contiguous()
        # the second halves of the two low-rank projections as ONE product: [a2 0; 0 g2] over the columns of both first halves
        HD, HV = self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        self.low_cols = at - self.a1_col
        w2 = self.w_a2.new_zeros((HD + HV, self.low_cols))
        w2[:HD, :self.rank_a] = self.w_a2
        w2[HD:, self.g1_col - self.a1_col:self.g1_col - self.a1_col + self.rank_g] = self.w_g2
        self.w_low2 = w2.contiguous()
        self.w_a2 = self.w_g2 = None

    def cache_spec(self):
        return (FixedStateSpec((self.num_heads, self.v_head_dim, self.head_dim)), FixedStateSpec((self.conv_taps - 1, self.channels)))   # S column by column

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        state, conv_state = cache
        H, G, D, DV = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        z = K.linear(h, self.w_in, out_dtype=ctx.dtype)
        qkv = K.causal_conv(z, 0, self.channels, self.conv_w, None, conv_state.state, ctx, activation="silu")
        ag = K.linear(z[:, self.a1_col:self.a1_col + self.low_cols], self.w_low2, out_dtype=ctx.dtype)    # [decay logits | gate logits]
        o = K.delta_rule(qkv, H, G, D, DV, ag[:, :H * D], z, self.b_col, self.A_log, self.dt_bias, state.state, ctx)
        y = K.group_rmsnorm_gate(o, ag, H * D, self.norm_w, DV, self.eps, gate_first=False, out_dtype=ctx.dtype)
        K.linear(y, self.w_o, add_to=residual)


class StateSpaceMixer(Mixer):
    """A selective state-space mixer with one decay per head (the recurrence of Mamba-2). ``W_in x`` is laid out as
    ``[z: inner | x: inner | B: groups * state | C: groups * state | dt: heads]`` with ``inner = heads * v_head_dim``; x, B and C
    together pass a short causal convolution with a bias and SiLU; ``dt <- softplus(dt + dt_bias)`` without a clamp; per head
    (head ``h`` uses group ``h // (heads // groups)``), ``S [state, v_head_dim]`` starting at zero:

        S <- exp(-exp(A_log[h]) dt) S + dt B x^T;   y = S^T C + D[h] x

    ``y`` is multiplied by ``silu(z)`` and THEN normed by its root mean square in ``norm_groups`` equal parts, times a weight per
    channel; then the output projection. Step sizes, decays and the state are 32-bit; a request's state is ``S`` and the
    convolution's last ``conv_taps - 1`` inputs.
    """

    graph_safe = True

    def __init__(self, hidden: int, num_heads: int, v_head_dim: int, state_size: int, groups: int, norm_groups: int, conv_taps: int,
                 eps: float, prefix: str):
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads cannot share {groups} groups")
        inner = num_heads * v_head_dim
        if inner % norm_groups:
            raise ValueError(f"{inner} channels cannot be normed in {norm_groups} equal parts")
        if not 1 <= conv_taps <= 8:
            raise ValueError(f"a short convolution has 1 to 8 taps, got {conv_taps}")
        if state_size > 256:
            raise ValueError(f"the recurrence's kernel keeps a column of the state in registers: state size {state_size} is more than 256")
        self.hidden, self.num_heads, self.v_head_dim, self.state_size, self.groups = hidden, num_heads, v_head_dim, state_size, groups
        self.norm_groups, self.conv_taps, self.eps, self.prefix = norm_groups, int(conv_taps), float(eps), prefix
        self.inner = inner
        self.channels = inner + 2 * groups * state_size            # what the convolution sees: x | B | C
        self.dt_col = inner + self.channels
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.A_log = self.skip = self.norm_w = None

    def params(self) -> Dict[str, ParamSpec]:
        p, h, H = self.prefix, self.hidden, self.num_heads
        return {
            "w_in": ParamSpec((Source(f"{p}.in", (self.dt_col + H, h), INIT_PROJ),), MATRIX),
            "w_o": ParamSpec((Source(f"{p}.o", (h, self.inner), INIT_PROJ),), MATRIX),
            "conv_w": ParamSpec((Source(f"{p}.conv", (self.channels, self.conv_taps), INIT_TAPS),), VECTOR),
            "conv_b": ParamSpec((Source(f"{p}.conv.b", (self.channels,), INIT_SMALL),), VECTOR),
            "dt_bias": ParamSpec((Source(f"{p}.dt_bias", (H,), INIT_STEP_BIAS),), VECTOR),
            "A_log": ParamSpec((Source(f"{p}.A_log", (H,), INIT_LOG_RATE),), VECTOR),
            "skip": ParamSpec((Source(f"{p}.D", (H,), INIT_NORM),), VECTOR),
            "norm_w": ParamSpec((Source(f"{p}.norm", (self.inner,), INIT_NORM),), VECTOR),
        }

    def bind(self, tensors) -> None:
        super().bind(tensors)
        self.w_in = _padded(self.w_in)

    def cache_spec(self):
        return (FixedStateSpec((self.num_heads, self.v_head_dim, self.state_size)), FixedStateSpec((self.conv_taps - 1, self.channels)))   # S column by column

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        state, conv_state = cache
        z = K.linear(h, self.w_in, out_dtype=ctx.dtype)
        xbc = K.causal_conv(z, self.inner, self.channels, self.conv_w, self.conv_b, conv_state.state, ctx, activation="silu")
        y = K.ssm_scan(xbc, self.num_heads, self.groups, self.state_size, self.v_head_dim, z, self.dt_col, self.A_log, self.dt_bias, self.skip,
                       state.state, ctx)
        y = K.group_rmsnorm_gate(y, z, 0, self.norm_w, self.inner // self.norm_groups, self.eps, gate_first=True, out_dtype=ctx.dtype)
        K.linear(y, self.w_o, add_to=residual)


class HeadDecayDeltaMixer(Mixer):
    """The gated delta rule with ONE decay per head. With q, k of ``num_kv_heads x head_dim`` and v of ``num_heads x v_head_dim``
    (head ``h`` uses q/k head ``h // (num_heads // num_kv_heads)``), each through a short causal convolution and SiLU, q and k then
    made unit vectors per head (``x / sqrt(sum x^2 + 1e-6)``, q also times ``head_dim^-1/2``):

        beta = sigmoid(W_b x)                                           one per head
        g    = exp(-exp(A_log[h]) * softplus(W_a x + dt_bias[h]))       one per head
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q

    per head, ``S [head_dim, v_head_dim]`` starting at zero. Each head's ``o`` is divided by its root mean square, multiplied by a
    weight shared by the heads and by ``silu(W_g x)``; then the output projection. All six projections of the input are one
    matrix. Decays, gates, unit norms and the state are 32-bit; a request's state is ``S`` and the convolution's last
    ``conv_taps - 1`` inputs. Checkpoint names: ``{prefix}.q / k / v`` (+ ``.conv``), ``.b``, ``.a``, ``.g``, ``.o``, ``.A_log``,
    ``.dt_bias``, ``.norm``."""

    graph_safe = True

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, conv_taps: int, eps: float, prefix: str):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} query/key heads")
        if not 1 <= conv_taps <= 8:
            raise ValueError(f"a short convolution has 1 to 8 taps, got {conv_taps}")
        if head_dim > 256:
            raise ValueError(f"the delta rule's kernel keeps a column of the state in registers: head_dim {head_dim} is more than 256")
        self.hidden, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim = hidden, num_heads, num_kv_heads, head_dim, v_head_dim
        self.conv_taps, self.eps, self.prefix = int(conv_taps), float(eps), prefix
        self.qk = num_kv_heads * head_dim
        self.channels = 2 * self.qk + num_heads * v_head_dim      # what the convolution sees: q | k | v
        self.b_col = self.a_col = self.g_col = 0      # columns of the joined projection's sections: set when the weights are bound
        self.w_in = self.w_o = self.conv_w = self.A_log = self.dt_bias = self.norm_w = None

    def params(self) -> Dict[str, ParamSpec]:
        p, h, H, DV = self.prefix, self.hidden, self.num_heads, self.v_head_dim
        rows = (("q", self.qk), ("k", self.qk), ("v", H * DV))
        return {
            "w_in": ParamSpec(tuple(Source(f"{p}.{n}", (c, h), INIT_PROJ) for n, c in rows)
                              + (Source(f"{p}.b", (H, h), INIT_PROJ), Source(f"{p}.a", (H, h), INIT_PROJ), Source(f"{p}.g", (H * DV, h), INIT_PROJ)), MATRIX),
            "w_o": ParamSpec((Source(f"{p}.o", (h, H * DV), INIT_PROJ),), MATRIX),
            "conv_w": ParamSpec(tuple(Source(f"{p}.{n}.conv", (c, self.conv_taps), INIT_TAPS) for n, c in rows), VECTOR),
            "A_log": ParamSpec((Source(f"{p}.A_log", (H,), INIT_LOG_RATE),), VECTOR),
            "dt_bias": ParamSpec((Source(f"{p}.dt_bias", (H,), INIT_STEP_BIAS),), VECTOR),
            "norm_w": ParamSpec((Source(f"{p}.norm", (DV,), INIT_NORM),), VECTOR),
        }

    def bind(self, tensors) -> None:
        super().bind(tensors)
        H = self.num_heads
        # every section of the joined projection starts on a multiple of 8 rows: its columns of the product then start on a
        # 16-byte boundary
        pieces, starts, at = [], [], 0
        for part in torch.split(self.w_in, (self.channels, H, H, H * self.v_head_dim)):
            starts.append(at)
            pieces.append(_padded(part))
            at += pieces[-1].shape[0]
        _, self.b_col, self.a_col, self.g_col = starts
        self.w_in = torch.cat(pieces).contiguous()

    def cache_spec(self):
        return (FixedStateSpec((self.num_heads, self.v_head_dim, self.head_dim)), FixedStateSpec((self.conv_taps - 1, self.channels)))   # S column by column

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        state, conv_state = cache
        H, G, D, DV = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        z = K.linear(h, self.w_in, out_dtype=ctx.dtype)
        qkv = K.causal_conv(z, 0, self.channels, self.conv_w, None, conv_state.state, ctx, activation="silu")
        o = K.delta_rule(qkv, H, G, D, DV, z[:, self.a_col:self.a_col + H], z, self.b_col, self.A_log, self.dt_bias, state.state, ctx, decay_per_head=True)
        y = K.group_rmsnorm_gate(o, z, self.g_col, self.norm_w, DV, self.eps, gate_first=False, out_dtype=ctx.dtype, gate_act="silu")
        K.linear(y, self.w_o, add_to=residual)


class SelectiveScanMixer(Mixer):
    """A selective scan with a state per channel and state index (the recurrence of Mamba). ``W_in x`` is ``[x: inner | z: inner]``;
    x passes a short causal convolution with a bias and SiLU; ``W_x x`` is ``[dt: dt_rank | B: state | C: state]``;
    ``dt <- softplus(W_dt dt + dt_bias)``, one per channel; ``A = -exp(A_log)`` ``[inner, state]``; per channel c and state index n:

        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c

    then ``y * silu(z)`` and the output projection. Step sizes, decays and the state are 32-bit; a request's state is ``S``
    (starting at zero) and the convolution's last ``conv_taps - 1`` inputs. Checkpoint names: ``{prefix}.in``, ``.conv`` (+ ``.b``),
    ``.x``, ``.dt`` (+ ``.b``), ``.A_log``, ``.D``, ``.o``."""

    graph_safe = True

    def __init__(self, hidden: int, inner: int, state_size: int, dt_rank: int, conv_taps: int, prefix: str):
        if not 1 <= conv_taps <= 8:
            raise ValueError(f"a short convolution has 1 to 8 taps, got {conv_taps}")
        if state_size > 256:
            raise ValueError(f"the recurrence's kernel keeps a channel's state in registers: state size {state_size} is more than 256")
        self.hidden, self.inner, self.state_size, self.dt_rank, self.conv_taps, self.prefix = hidden, inner, state_size, dt_rank, int(conv_taps), prefix
        self.w_in = self.w_x = self.w_dt = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.A_log = self.skip = None

    def params(self) -> Dict[str, ParamSpec]:
        p, h, C, NS, R = self.prefix, self.hidden, self.inner, self.state_size, self.dt_rank
        return {
            "w_in": ParamSpec((Source(f"{p}.in", (2 * C, h), INIT_PROJ),), MATRIX),
            "w_x": ParamSpec((Source(f"{p}.x", (R + 2 * NS, C), INIT_PROJ),), MATRIX),
            "w_dt": ParamSpec((Source(f"{p}.dt", (C, R), INIT_PROJ),), MATRIX),
            "w_o": ParamSpec((Source(f"{p}.o", (h, C), INIT_PROJ),), MATRIX),
            "conv_w": ParamSpec((Source(f"{p}.conv", (C, self.conv_taps), INIT_TAPS),), VECTOR),
            "conv_b": ParamSpec((Source(f"{p}.conv.b", (C,), INIT_SMALL),), VECTOR),
            "dt_bias": ParamSpec((Source(f"{p}.dt.b", (C,), INIT_STEP_BIAS),), VECTOR),
            "A_log": ParamSpec((Source(f"{p}.A_log", (C, NS), INIT_LOG_RATE),), VECTOR),
            "skip": ParamSpec((Source(f"{p}.D", (C,), INIT_NORM),), VECTOR),
        }

    def bind(self, tensors) -> None:
        super().bind(tensors)
        # ``W_x``'s rows are padded to a multiple of 8 (16-byte rows of the product), and ``W_dt`` gets zero columns for B, C and
        # the padding, so that the step sizes are a product over the whole row of ``W_x x`` as it lies
        self.w_x = _padded(self.w_x)
        wide = self.w_dt.new_zeros((self.inner, self.w_x.shape[0]))
        wide[:, :self.dt_rank] = self.w_dt
        self.w_dt = wide.contiguous()

    def cache_spec(self):
        return (FixedStateSpec((self.inner, self.state_size)), FixedStateSpec((self.conv_taps - 1, self.inner)))

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        state, conv_state = cache
        C, NS, R = self.inner, self.state_size, self.dt_rank
        xz = K.linear(h, self.w_in, out_dtype=ctx.dtype)
        x = K.causal_conv(xz, 0, C, self.conv_w, self.conv_b, conv_state.state, ctx, activation="silu")
        dbc = K.linear(x, self.w_x, out_dtype=ctx.dtype)
        dt = K.linear(dbc, self.w_dt, out_dtype=ctx.dtype)
        y = K.selective_scan(x, dt, dbc, R, R + NS, xz, C, self.A_log, self.dt_bias, self.skip, state.state, ctx)
        K.linear(y, self.w_o, add_to=residual)


class MatrixMemoryMixer(Mixer):
    """A matrix memory with exponential gates (the mLSTM cell of xLSTM). Per head, with ``q = W_q x * head_dim^-1/2``, ``k = W_k x``
    (``head_dim`` entries) and ``v = W_v x`` (``v_head_dim``), a log input gate ``i = cap tanh((W_i x + b_i) / cap)`` and a log forget
    gate ``f = ln sigmoid(cap tanh((W_f x + b_f) / cap))`` (``gate_cap`` None: no cap), and a running maximum ``m`` that starts at 0:

        m' = max(f + m, i);   S <- exp(f + m - m') S + exp(i - m') k v^T;   n <- the same with k alone;
        o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)

    Every head's ``o`` is divided by its root mean square; the heads side by side are multiplied by a weight of ``heads * v_head_dim``
    entries and by ``sigmoid(W_g x)``; then the output projection. ``S``, ``n`` and ``m`` start at zero and are a request's state (32-bit:
    the memory column by column with the normaliser as one more column, and ``m``); gates, their logarithms and exponentials are
    32-bit, made from 32-bit pre-activations (a small product of its own beside the joined projection ``q | k | v | g``).
    Checkpoint names: ``{prefix}.q / k / v / g / o``, ``.i`` and ``.f`` (+ ``.b``), ``.norm``."""

    graph_safe = True

    def __init__(self, hidden: int, num_heads: int, head_dim: int, v_head_dim: int, gate_cap: Optional[float], eps: float, prefix: str):
        if head_dim > 256:
            raise ValueError(f"the memory's kernel keeps a column in registers: head_dim {head_dim} is more than 256")
        self.hidden, self.num_heads, self.head_dim, self.v_head_dim = hidden, num_heads, head_dim, v_head_dim
        self.gate_cap = float(gate_cap) if gate_cap else None
        self.eps, self.prefix = float(eps), prefix
        self.q_col = self.k_col = self.v_col = self.g_col = 0     # columns of the joined projection's sections: set when the weights are bound
        self.w_in = self.w_gates = self.w_o = self.bias_i = self.bias_f = self.norm_w = None

    def params(self) -> Dict[str, ParamSpec]:
        p, h, H, D, DV = self.prefix, self.hidden, self.num_heads, self.head_dim, self.v_head_dim
        return {
            "w_in": ParamSpec((Source(f"{p}.q", (H * D, h), INIT_PROJ), Source(f"{p}.k", (H * D, h), INIT_PROJ), Source(f"{p}.v", (H * DV, h), INIT_PROJ),
                               Source(f"{p}.g", (H * DV, h), INIT_PROJ)), MATRIX),
            "w_gates": ParamSpec((Source(f"{p}.i", (H, h), INIT_PROJ), Source(f"{p}.f", (H, h), INIT_PROJ)), MATRIX),
            "w_o": ParamSpec((Source(f"{p}.o", (h, H * DV), INIT_PROJ),), MATRIX),
            "bias_i": ParamSpec((Source(f"{p}.i.b", (H,), INIT_SMALL),), VECTOR),
            "bias_f": ParamSpec((Source(f"{p}.f.b", (H,), INIT_NORM),), VECTOR),
            "norm_w": ParamSpec((Source(f"{p}.norm", (H * DV,), INIT_NORM),), VECTOR),
        }

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_gates, self.w_o, self.bias_i, self.bias_f, self.norm_w) if t is not None)

    def bind(self, tensors) -> None:
        super().bind(tensors)
        H, D, DV = self.num_heads, self.head_dim, self.v_head_dim
        # every section of the joined projection starts on a multiple of 8 rows: its columns of the product then start on a 16-byte boundary
        pieces, starts, at = [], [], 0
        for part in torch.split(self.w_in, (H * D, H * D, H * DV, H * DV)):
            starts.append(at)
            pieces.append(_padded(part))
            at += pieces[-1].shape[0]
        self.q_col, self.k_col, self.v_col, self.g_col = starts
        self.w_in = torch.cat(pieces).contiguous()
        self.w_gates = _padded(self.w_gates)   # [i | f], then zero rows

    def cache_spec(self):
        return (FixedStateSpec((self.num_heads, self.v_head_dim + 1, self.head_dim)), FixedStateSpec((self.num_heads,)))   # S and n column by column; m

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        memory, maximum = cache
        H, D, DV = self.num_heads, self.head_dim, self.v_head_dim
        z = K.linear(h, self.w_in, out_dtype=ctx.dtype)
        gates = K.linear(h, self.w_gates, out_dtype=torch.float32)
        num, m = K.mlstm(z, self.q_col, self.k_col, self.v_col, gates, self.bias_i, self.bias_f, self.gate_cap, H, D, DV, memory.state, maximum.state, ctx)
        y = K.mlstm_finish(num, m, z, self.g_col, self.norm_w, self.eps, ctx.dtype)
        K.linear(y, self.w_o, add_to=residual)


class ParallelMixer(Mixer):
    """Two mixers side by side on the same input, each with its own cache or state. Two ways of joining their outputs:

    * normed mean (``left_weight``, ``right_weight`` name two vectors of the checkpoint): half the sum of the outputs, each first
      divided by its root mean square over the model width and multiplied by its vector;
    * ``scales = (a, b)``: ``a * left + b * right``, nothing else."""

    graph_safe = True

    def __init__(self, hidden: int, left: Mixer, right: Mixer, eps: float, left_weight: Optional[str] = None, right_weight: Optional[str] = None,
                 scales: Optional[tuple] = None):
        if (scales is None) == (left_weight is None) or (left_weight is None) != (right_weight is None):
            raise ValueError("two mixers side by side are joined by two named weight vectors or by two scales, not both")
        self.hidden, self.left, self.right, self.eps = hidden, left, right, float(eps)
        self.left_weight, self.right_weight = left_weight, right_weight
        self.scales = None if scales is None else (float(scales[0]), float(scales[1]))
        self.w_left: Optional[torch.Tensor] = None
        self.w_right: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        if self.scales is not None:
            return {}
        return {"w_left": ParamSpec((Source(self.left_weight, (self.hidden,), INIT_NORM),), VECTOR),
                "w_right": ParamSpec((Source(self.right_weight, (self.hidden,), INIT_NORM),), VECTOR)}

    def children(self) -> Sequence[Part]:
        return (self.left, self.right)

    def cache_spec(self):
        return (self.left.cache_spec(), self.right.cache_spec())

    def forward(self, ctx, h, cache, residual):
        K = ctx.K
        a = K.zeros_like_rows(residual, 1)
        self.left.forward(ctx, h, cache[0], a)
        a = K.take_result(a)
        b = K.zeros_like_rows(residual, 2)
        self.right.forward(ctx, h, cache[1], b)
        b = K.take_result(b)
        if self.scales is not None:
            K.weighted_pair(a, b, self.scales[0], self.scales[1], add_to=residual)
        else:
            K.dual_rmsnorm_mix(a, b, self.w_left, self.w_right, self.eps, 0.5, add_to=residual)
