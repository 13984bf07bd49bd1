"""Dense gated feed-forward."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import INIT_PROJ, INIT_SMALL, MATRIX, VECTOR, FeedForward, ParamSpec, Source

ACTIVATIONS = ("silu",)


class GatedMLP(FeedForward):
    """``down(act(gate(x)) * up(x))`` without biases (src/miniserve/model.py:164-165).

    ``gate`` and ``up`` are kept as one matrix ``[2 * intermediate, hidden]`` (gate rows first) so a
    step multiplies once; the activation and the product of the two halves are the epilogue of that product
    (prompt portions) or one kernel over its float32 sums (decode steps): ``gate_up_act`` of the kernels object decides.
    """

    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, prefix: str, activation: str = "silu"):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not one of {ACTIVATIONS}")
        self.hidden, self.intermediate, self.prefix, self.activation = hidden, intermediate, prefix, activation
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        p, h, i = self.prefix, self.hidden, self.intermediate
        return {
            "w_gate_up": ParamSpec((Source(f"{p}.gate_proj.weight", (i, h)), Source(f"{p}.up_proj.weight", (i, h))), MATRIX),
            "w_down": ParamSpec((Source(f"{p}.down_proj.weight", (h, i)),), MATRIX),
        }

    def forward(self, ctx, h, residual):
        K = ctx.K
        K.linear(K.gate_up_act(h, self.w_gate_up, ctx.dtype), self.w_down, add_to=residual)


class DenseMLP(FeedForward):
    """``down(act(up(x)))`` without biases; ``act`` is the tanh form of GELU,
    ``0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))``, computed in 32-bit on the product's sums."""

    graph_safe = True
    ACTIVATIONS = ("gelu_tanh",)

    def __init__(self, hidden: int, intermediate: int, up_name: str, down_name: str, activation: str = "gelu_tanh"):
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not one of {self.ACTIVATIONS}")
        self.hidden, self.intermediate, self.up_name, self.down_name, self.activation = hidden, intermediate, up_name, down_name, activation
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        return {"w_up": ParamSpec((Source(self.up_name, (self.intermediate, self.hidden)),), MATRIX),
                "w_down": ParamSpec((Source(self.down_name, (self.hidden, self.intermediate)),), MATRIX)}

    def forward(self, ctx, h, residual):
        K = ctx.K
        K.linear(K.linear_act(h, self.w_up, self.activation, ctx.dtype), self.w_down, add_to=residual)


class ClampedGLU(FeedForward):
    """``down(g * sigmoid(alpha g) * (u + shift))`` with ``g = min(gate(x), limit)`` and ``u = clamp(up(x), -limit, limit)``, no
    biases. ``gate`` and ``up`` are one matrix ``[2 * intermediate, hidden]`` (gate rows first); the gated unit is the epilogue of
    that product (prompt portions) or one kernel over its float32 sums (decode steps): ``gate_up_act`` of the kernels object decides."""

    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, gate_name: str, up_name: str, down_name: str, limit: float, alpha: float = 1.702,
                 shift: float = 1.0):
        if not limit > 0:
            raise ValueError(f"the limit of a clamped gated unit must be positive, got {limit}")
        self.hidden, self.intermediate = hidden, intermediate
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        h, i = self.hidden, self.intermediate
        return {"w_gate_up": ParamSpec((Source(self.gate_name, (i, h)), Source(self.up_name, (i, h))), MATRIX),
                "w_down": ParamSpec((Source(self.down_name, (h, i)),), MATRIX)}

    def forward(self, ctx, h, residual):
        K = ctx.K
        K.linear(K.gate_up_act(h, self.w_gate_up, ctx.dtype, glu=(self.limit, self.alpha, self.shift)), self.w_down, add_to=residual)


class GatedUnit(FeedForward):
    """``down(act(gate(x)) * up(x))`` without biases, under checkpoint names of the caller's choice; ``act`` is ``silu`` or the
    tanh form of GELU, ``0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))``. ``gate`` and ``up`` are one matrix (gate rows first);
    the activation is the epilogue of that product (prompt portions) or one kernel over its float32 sums (decode steps)."""

    graph_safe = True
    ACTIVATIONS = ("silu", "gelu_tanh")

    def __init__(self, hidden: int, intermediate: int, gate_name: str, up_name: str, down_name: str, activation: str = "silu"):
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not one of {self.ACTIVATIONS}")
        self.hidden, self.intermediate, self.activation = hidden, intermediate, activation
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def params(self) -> Dict[str, ParamSpec]:
        h, i = self.hidden, self.intermediate
        return {"w_gate_up": ParamSpec((Source(self.gate_name, (i, h), INIT_PROJ), Source(self.up_name, (i, h), INIT_PROJ)), MATRIX),
                "w_down": ParamSpec((Source(self.down_name, (h, i), INIT_PROJ),), MATRIX)}

    def forward(self, ctx, h, residual):
        K = ctx.K
        K.linear(K.gate_up_act(h, self.w_gate_up, ctx.dtype, activation=self.activation), self.w_down, add_to=residual)


class RoutedExperts(FeedForward):
    """``num_experts`` gated units (``down(silu(gate x) * (up x))``, no biases) of which every token uses ``top``, chosen by a router:

        s = softmax(W_router x) over all router outputs, in 32-bit;   choice = s + correction;
        the ``top`` outputs with the largest choice are taken; their weights are ``s / (sum of the taken s + 1e-20)``.

    The router has ``num_identity`` outputs more than there are experts with matrices: a token that takes one of them gets its own
    input back from it (times the weight). ``shared`` (a feed-forward of its own, or None) runs for every token and is added.
    Checkpoint names: ``{prefix}.router``, ``{prefix}.correction``, ``{prefix}.e<i>.gate / up / down``. The experts' matrices are
    kept stacked (``[E, 2 ff, hidden]`` and ``[E, hidden, ff]``); tokens are sorted by expert on the device and every expert's
    rows pass its matrices in one grouped product, so the part only launches kernels.

    Other routers and experts, each a constructor argument:

    * ``scoring="sigmoid"``: ``s = sigmoid(W_router x)``, every output by itself, and the weights are the chosen ``s`` as they are;
    * ``correction=False``: no correction vector in the checkpoint;
    * ``weight_inputs``: the weight multiplies the expert's INPUT, the output is ``sum_k expert(w_k x)``;
    * ``expert_glu=(limit, alpha, shift)``: the experts are clamped units, ``down(g sigmoid(alpha g) (u + shift))`` with
      ``g = min(gate x, limit)`` and ``u = clamp(up x, -limit, limit)``."""

    graph_safe = True

    def __init__(self, hidden: int, intermediate: int, num_experts: int, num_identity: int, top: int, prefix: str,
                 shared: Optional[FeedForward] = None, scoring: str = "softmax", correction: bool = True, weight_inputs: bool = False,
                 expert_glu: Optional[tuple] = None):
        if not 1 <= top <= num_experts + num_identity:
            raise ValueError(f"{top} of {num_experts + num_identity} router outputs cannot be chosen")
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"a router scores by 'softmax' or 'sigmoid', got {scoring!r}")
        if weight_inputs and num_identity:
            raise ValueError("weights on the experts' inputs are not built together with identity experts")
        self.hidden, self.intermediate, self.num_experts, self.num_identity, self.top = hidden, intermediate, num_experts, num_identity, top
        self.prefix, self.shared = prefix, shared
        self.scoring, self.has_correction, self.weight_inputs = scoring, bool(correction), bool(weight_inputs)
        self.expert_glu = None if expert_glu is None else tuple(float(v) for v in expert_glu)
        self.w_router = self.correction = self.w_gate_up = self.w_down = None

    def children(self):
        return (self.shared,) if self.shared is not None else ()

    def params(self) -> Dict[str, ParamSpec]:
        p, h, i, E = self.prefix, self.hidden, self.intermediate, self.num_experts
        total = E + self.num_identity
        gate_up = tuple(Source(f"{p}.e{e}.{n}", (i, h), INIT_PROJ) for e in range(E) for n in ("gate", "up"))
        out = {"w_router": ParamSpec((Source(f"{p}.router", (total, h), INIT_PROJ),), MATRIX),
               "w_gate_up": ParamSpec(gate_up, MATRIX),
               "w_down": ParamSpec(tuple(Source(f"{p}.e{e}.down", (h, i), INIT_PROJ) for e in range(E)), MATRIX)}
        if self.has_correction:
            out["correction"] = ParamSpec((Source(f"{p}.correction", (total,), INIT_SMALL),), VECTOR)
        return out

    def bind(self, tensors) -> None:
        super().bind(tensors)
        E, h, i = self.num_experts, self.hidden, self.intermediate
        self.w_gate_up = self.w_gate_up.view(E, 2 * i, h)
        self.w_down = self.w_down.view(E, h, i)

    def forward(self, ctx, h, residual):
        K = ctx.K
        if self.scoring == "softmax" and not self.weight_inputs and self.expert_glu is None:
            ids, weights = K.moe_router(h, self.w_router, self.correction, self.top)
            K.moe_experts(h, ids, weights, self.w_gate_up, self.w_down, add_to=residual)
        else:
            ids, weights = K.moe_router(h, self.w_router, self.correction, self.top, scoring=self.scoring)
            K.moe_experts(h, ids, weights, self.w_gate_up, self.w_down, add_to=residual, glu=self.expert_glu, weight_inputs=self.weight_inputs)
        if self.shared is not None:
            self.shared.forward(ctx, h, residual)
