"""Memilorn: a decoder whose layers are listed one by one in config.json.

Every layer is pre-norm with layer norms that have a weight and no bias, and each sublayer's result passes a layer scale (a vector
of the model's width) before it joins the stream: ``x += ls1 * mixer(norm1(x))``, ``x += ls2 * ff(norm2(x))``. The mixer is one of

* ``mlstm``: a matrix memory with exponential gates and a running maximum (a recurrent state of fixed size);
* ``latent_attention``: causal softmax attention without positions whose keys and values are rebuilt from a small normed latent
  per token (only the latent is cached), with a gate per head;
* ``attention``: grouped causal softmax attention, the first ``rot.dims`` entries of a head turned in neighbouring pairs, scores
  bounded by ``softcap`` and mixed between the heads before the softmax, a sink per head in the denominator, a gate per head.

The feed-forward (where a layer has one) is a mixture of clamped gated units: the router's sigmoid scores choose ``top`` experts
and multiply the experts' INPUTS (not renormalised); a shared unit runs for every token. ``loop``: the layers ``start .. stop - 1``
run ``times`` times in a row on the same weights, every pass with cache entries of its own, and before every pass but the first the
tokens' embedding is added to the stream again; the running order expresses both directly. The output head is the embedding table.
Tensor names: ``embed``, ``l<i>.norm1 / norm2 / ls1 / ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.model_config import MemilornConfig
from ..parts import OutputHead, TokenEmbedding
from ..parts.attention_latent import LatentAttention
from ..parts.attention_masked import MaskedAttention
from ..parts.block import PreNormBlock
from ..parts.mlp import ClampedGLU, RoutedExperts
from ..parts.norm import LayerNorm
from ..parts.recurrent import MatrixMemoryMixer
from ..parts.rotary import RampedRotary
from .registry import register_architecture
from .spec import LayerCall, ModelSpec

GLU_ALPHA, GLU_SHIFT = 1.702, 1.0   # the clamped unit of this architecture: g sigmoid(1.702 g) (u + 1)


def build_memilorn(cfg: MemilornConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.eps
    rotary = {}

    def feed_forward(mlp, p: str):
        shared = None
        if mlp.shared_ff:
            shared = ClampedGLU(W, mlp.shared_ff, f"{p}.shared.gate", f"{p}.shared.up", f"{p}.shared.down", mlp.shared_limit, GLU_ALPHA, GLU_SHIFT)
        return RoutedExperts(W, mlp.ff, mlp.experts, 0, mlp.top, p, shared, scoring="sigmoid", correction=False, weight_inputs=True,
                             expert_glu=(mlp.limit, GLU_ALPHA, GLU_SHIFT))

    layers = []
    for i, lc in enumerate(cfg.layers):
        p, m = f"l{i}", lc.mixer
        if lc.kind == "mlstm":
            mixer = MatrixMemoryMixer(W, m.heads, m.dim, m.vdim, m.gate_cap, eps, f"{p}.mix")
        elif lc.kind == "latent_attention":
            mixer = LatentAttention(W, m.heads, m.dim, 0, m.vdim, 0, m.kv_rank, m.scale, eps, None, f"{p}.mix", sink=False, gate="head")
        else:
            position = None
            if m.rot is not None:
                position = rotary.setdefault(m.rot, RampedRotary(m.rot.dims, m.rot.base))
            mixer = MaskedAttention(W, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, f"{p}.mix", position=position, interleaved=True,
                                    softcap=m.softcap, talking_heads=True, sink=True, head_gate=True)
        ff = feed_forward(lc.mlp, f"{p}.mlp") if lc.mlp is not None else None
        layers.append(PreNormBlock(LayerNorm(W, eps, f"{p}.norm1"), mixer, LayerNorm(W, eps, f"{p}.norm2") if ff is not None else None, ff,
                                   scale1=f"{p}.ls1", scale2=f"{p}.ls2" if ff is not None else None, dim=W))
    # every run of a layer has a cache entry of its own; a further pass over the looped layers opens with the embedding added again
    schedule = [LayerCall(i, entry, add_embedding=again) for entry, (i, _, again) in enumerate(cfg.running_order())]
    embedding = TokenEmbedding(cfg.vocab, W, "embed")
    return ModelSpec(
        config=cfg,
        embedding=embedding,
        layers=layers,
        schedule=schedule,
        final_norm=LayerNorm(W, eps, "final.norm"),
        head=OutputHead(cfg.vocab, W, "head", tied_to=embedding),
    )


register_architecture("Memilorn", MemilornConfig, build_memilorn)
