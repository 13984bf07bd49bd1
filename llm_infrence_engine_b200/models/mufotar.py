"""Mufotar: a decoder whose layers are listed one by one in config.json.

Every layer has ONE norm (a layer norm with weight and bias) whose output both sublayers read: ``h = norm1(x)``,
``x += mixer(h) + ff(h)``. The mixer is one of

* ``delta``: the gated delta rule with one decay per head (a recurrent state of fixed size);
* ``parallel``: causal softmax attention (query/key norm per head, the first ``rot.dims`` entries of a head turned in pairs half
  that span apart) beside a selective scan with a state per channel and state index; the result is
  ``left_scale * left + right_scale * right``.

The feed-forward is a dense gated unit with the tanh form of GELU, or routed experts (SiLU units; the router also has outputs
that stand for identity experts; a shared unit runs for every token), or absent. A layer with ``weights_of: j`` has no tensors:
it is layer j's part run once more, with a cache entry of its own, which the running order expresses directly. The output head
is the embedding table itself; the logits are bounded by ``logit_softcap * tanh(logits / logit_softcap)``.
Tensor names: ``embed``, ``l<i>.norm1`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm`` (+ ``.b``).
"""
from __future__ import annotations

from ..config.model_config import MufotarConfig, RoutedExpertsConfig
from ..parts import OutputHead, TokenEmbedding
from ..parts.attention_masked import MaskedAttention
from ..parts.block import ParallelBlock
from ..parts.mlp import GatedUnit, RoutedExperts
from ..parts.norm import LayerNorm
from ..parts.recurrent import HeadDecayDeltaMixer, ParallelMixer, SelectiveScanMixer
from ..parts.rotary import RampedRotary
from .registry import register_architecture
from .spec import LayerCall, ModelSpec


def build_mufotar(cfg: MufotarConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.eps
    rotary = {}

    def feed_forward(mlp, p: str):
        if mlp is None:
            return None
        if isinstance(mlp, RoutedExpertsConfig):
            shared = GatedUnit(W, mlp.shared_ff, f"{p}.shared.gate", f"{p}.shared.up", f"{p}.shared.down", "silu") if mlp.shared_ff else None
            return RoutedExperts(W, mlp.ff, mlp.experts, mlp.identity, mlp.top, p, shared)
        return GatedUnit(W, int(mlp), f"{p}.gate", f"{p}.up", f"{p}.down", "gelu_tanh")

    layers, part_of = [], {}
    for i, lc in enumerate(cfg.layers):
        if lc.weights_of is not None:      # no part of its own: the running order below names the other layer's part once more
            continue
        p, m = f"l{i}", lc.mixer
        if lc.kind == "delta":
            mixer = HeadDecayDeltaMixer(W, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, eps, f"{p}.mix")
        else:
            a = m.left
            position = None
            if a.rot is not None:
                position = rotary.setdefault(a.rot, RampedRotary(a.rot.dims, a.rot.base))
            left = MaskedAttention(W, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, f"{p}.mix.left", position=position, qk_norm=True, eps=eps)
            right = SelectiveScanMixer(W, m.right.inner, m.right.state, m.right.dt_rank, m.right.conv, f"{p}.mix.right")
            mixer = ParallelMixer(W, left, right, eps, scales=(m.left_scale, m.right_scale))
        part_of[i] = len(layers)
        layers.append(ParallelBlock(LayerNorm(W, eps, f"{p}.norm1", f"{p}.norm1.b"), mixer, feed_forward(lc.mlp, f"{p}.mlp")))
    # layer i runs its own part, or the part of the layer whose weights it runs on, always with cache entry i
    schedule = [LayerCall(part_of[i if lc.weights_of is None else lc.weights_of], i) for i, lc in enumerate(cfg.layers)]
    embedding = TokenEmbedding(cfg.vocab, W, "embed")
    return ModelSpec(
        config=cfg,
        embedding=embedding,
        layers=layers,
        schedule=schedule,
        final_norm=LayerNorm(W, eps, "final.norm", "final.norm.b"),
        head=OutputHead(cfg.vocab, W, "head", tied_to=embedding, softcap=cfg.logit_softcap),
    )


register_architecture("Mufotar", MufotarConfig, build_mufotar)
