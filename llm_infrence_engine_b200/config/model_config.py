"""Typed model configurations, read from the architecture's own ``config.json`` keys.

A configuration class knows the keys of one architecture, their defaults and the combinations that
make no sense. It holds every size and constant of the model; code below it takes them as
parameters and never writes one down itself.

The reference reads nine keys into ``ModelConfig`` (src/miniserve/model.py:26-58) and derives
``head_dim``; the class here reads the same keys with the same defaults and adds the ones the
checkpoint format carries but the reference ignores (explicit ``head_dim``, the sliding window
triple, ``attention_bias``, ``hidden_act``, ``max_position_embeddings``).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, fields
from pathlib import Path
from typing import Any, Mapping, Optional


class ConfigError(ValueError):
    """config.json is missing a key, has a value of the wrong kind, or asks for an impossible model."""


def _need(d: Mapping[str, Any], key: str, kind):
    if key not in d:
        raise ConfigError(f"config.json has no '{key}'")
    v = d[key]
    if kind is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if (isinstance(v, bool) and kind is not bool) or not isinstance(v, kind):
        raise ConfigError(f"config.json: '{key}' must be {kind.__name__}, got {v!r}")
    return v


def _refuse_unread_arithmetic(d: Mapping[str, Any]) -> None:
    """Keys that change the model's arithmetic and that this engine does not carry out: a checkpoint that sets one of
    them would give wrong logits without a word (the reference reads none of them, src/miniserve/model.py:42-58, and
    is silent). A key that is absent, null or at its neutral value is fine."""
    nested = d.get("rope_parameters") if isinstance(d.get("rope_parameters"), Mapping) else {}
    scaling = d.get("rope_scaling")
    if scaling is None and nested.get("rope_type") not in (None, "default"):
        scaling = {k: v for k, v in nested.items() if k != "rope_theta"}
    if isinstance(scaling, Mapping) and (scaling.get("rope_type") or scaling.get("type")) == "default":
        scaling = None
    if scaling is not None:
        raise ConfigError(f"config.json: 'rope_scaling' is {scaling!r}; scaled rotary positions are not built here "
                          "(only plain rotary positions with 'rope_theta')")
    prf = d.get("partial_rotary_factor", nested.get("partial_rotary_factor"))
    if prf is not None and float(prf) != 1.0:
        raise ConfigError(f"config.json: 'partial_rotary_factor' is {prf!r}; only whole heads are rotated here (1.0)")
    drop = d.get("attention_dropout")
    if drop is not None and float(drop) != 0.0:
        raise ConfigError(f"config.json: 'attention_dropout' is {drop!r}; an inference engine has none (0.0)")
    if d.get("mlp_bias"):
        raise ConfigError("config.json: 'mlp_bias' is true; the feed-forward of Qwen2 has no biases")


@dataclass(frozen=True)
class Qwen2Config:
    """The dense Qwen2 decoder: GQA attention with QKV bias, rotary positions, RMSNorm, SwiGLU."""

    architecture = "Qwen2ForCausalLM"

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    attention_bias: bool = True
    hidden_act: str = "silu"
    max_position_embeddings: int = 32768
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    torch_dtype: str = "bfloat16"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen2Config":
        _refuse_unread_arithmetic(d)
        heads = _need(d, "num_attention_heads", int)
        hidden = _need(d, "hidden_size", int)
        rope = d.get("rope_theta")
        if rope is None:  # newer checkpoints nest it (src/miniserve/model.py:45-47)
            rope = (d.get("rope_parameters") or {}).get("rope_theta", 10000.0)
        head_dim = d.get("head_dim")
        if head_dim is None:
            if heads <= 0 or hidden % heads:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads  # src/miniserve/model.py:38-40
        cfg = cls(
            vocab_size=_need(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_need(d, "intermediate_size", int),
            num_hidden_layers=_need(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=_need(d, "num_key_value_heads", int),
            head_dim=int(head_dim),
            rms_norm_eps=_need(d, "rms_norm_eps", float),
            rope_theta=float(rope),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", True)),
            hidden_act=str(d.get("hidden_act", "silu")),
            max_position_embeddings=int(d.get("max_position_embeddings", 32768)),
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            sliding_window=d.get("sliding_window"),
            max_window_layers=int(d.get("max_window_layers", 0) or 0),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act '{self.hidden_act}' is not known to Qwen2 (only 'silu')")
        if self.use_sliding_window and (not isinstance(self.sliding_window, int) or self.sliding_window <= 0):
            raise ConfigError("use_sliding_window is true but sliding_window is not a positive integer")

    # ------------------------------------------------------------------ derived
    def layer_window(self, layer: int) -> Optional[int]:
        """Keys a layer may look back over (itself included), or None for all of them."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return int(self.sliding_window)
        return None

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen2"
        return d


def read_config_json(folder: str | Path) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d


def architecture_name(d: Mapping[str, Any]) -> str:
    """The model class a config.json names: the first entry of ``architectures``, or a plain ``architecture`` string."""
    if isinstance(d.get("architecture"), str) and "architectures" not in d:
        return d["architecture"]
    arch = d.get("architectures")
    if not isinstance(arch, (list, tuple)) or not arch or not isinstance(arch[0], str):
        raise ConfigError("config.json has no 'architectures' list naming the model class")
    return arch[0]


def config_field_names(cls) -> list[str]:
    return [f.name for f in fields(cls)]


# ---------------------------------------------------------------------------------------------------------------------
# Luvutar: a decoder whose config.json lists its layers one by one.

def _sub(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be a positive integer, got {v!r}")
    return v


def _number(d: Mapping[str, Any], key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class BiasedAttentionConfig:
    """Mixer ``attention``: grouped heads without rotation; the position enters through a query temperature and a learned
    bias by bucketed distance."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: Optional[float] = None       # distance from which the bias table's last row is used; None: no bias table
    temp_coef: float = 0.0                 # query temperature 1 + coef * ln(floor((p + 1) / every) + 1); 0 / 0: none
    temp_every: int = 0
    kv_from: Optional[int] = None          # the layer whose keys and values this one reads instead of making its own

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "BiasedAttentionConfig":
        qt = m.get("q_temp")
        if qt is not None and not isinstance(qt, Mapping):
            raise ConfigError(f"config.json: {where}'q_temp' must be an object")
        kv_from = m.get("kv_from")
        if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or kv_from < 0):
            raise ConfigError(f"config.json: {where}'kv_from' must be a layer index, got {kv_from!r}")
        heads, kv_heads = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}{heads} heads cannot share {kv_heads} kv_heads")
        dim = _pos_int(m, "dim", where)
        return cls(heads, kv_heads, dim, _pos_int(m, "vdim", where) if "vdim" in m else dim, _number(m, "scale", where),
                   _number(m, "bias_max", where) if m.get("bias_max") is not None else None,
                   _number(qt, "coef", where + "q_temp.") if qt else 0.0, _pos_int(qt, "every", where + "q_temp.") if qt else 0, kv_from)


@dataclass(frozen=True)
class LatentAttentionConfig:
    """Mixer ``latent_attention``: queries and keys/values through low-rank latents, one rotated key part for all heads."""

    heads: int
    dim: int          # unrotated query/key dimensions per head
    rot_dim: int      # rotated ones
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float = 10000.0
    rot_dims: int = 0                # how many of the rot_dim entries turn (0: none)
    window: Optional[int] = None     # keys a position sees, itself included; None: all
    sink: bool = True

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "LatentAttentionConfig":
        rot, mask = m.get("rot"), m.get("mask")
        for name, v in (("rot", rot), ("mask", mask)):
            if v is not None and not isinstance(v, Mapping):
                raise ConfigError(f"config.json: {where}'{name}' must be an object")
        rot_dim = _pos_int(m, "rot_dim", where)
        rot_dims = _pos_int(rot, "dims", where + "rot.") if rot else 0
        if rot_dims % 2 or rot_dims > rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims {rot_dims} must be even and at most rot_dim {rot_dim}")
        return cls(_pos_int(m, "heads", where), _pos_int(m, "dim", where), rot_dim, _pos_int(m, "vdim", where), _pos_int(m, "q_rank", where),
                   _pos_int(m, "kv_rank", where), _number(m, "scale", where), _number(rot, "base", where + "rot.") if rot else 10000.0, rot_dims,
                   _pos_int(mask, "size", where + "mask.") if mask else None)


@dataclass(frozen=True)
class LuvutarLayerConfig:
    kind: str                  # "attention" or "latent_attention"
    mixer: Any
    ff: Optional[int]          # width of the dense feed-forward, None: the layer has none


@dataclass(frozen=True)
class LuvutarConfig:
    """The whole of a Luvutar config.json: vocabulary, width, norm epsilon, residual streams and the list of layers."""

    architecture = "Luvutar"
    MIXERS = {"attention": BiasedAttentionConfig, "latent_attention": LatentAttentionConfig}

    vocab: int
    width: int
    eps: float
    streams: Optional[int]     # None: one residual stream with plain additions; n: hyper-connections over n streams
    layers: tuple

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LuvutarConfig":
        if not isinstance(d.get("layers"), (list, tuple)) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, layer in enumerate(d["layers"]):
            where = f"layers[{i}]."
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is not one of {sorted(cls.MIXERS)}")
            mixer = cls.MIXERS[kind].from_dict(_sub(layer, "mixer", where), where + "mixer.")
            mlp = layer.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}mlp must be null or an object of kind 'dense'")
                ff = _pos_int(mlp, "ff", where + "mlp.")
            layers.append(LuvutarLayerConfig(kind, mixer, ff))
        streams = d.get("streams")
        cfg = cls(_pos_int(d, "vocab", ""), _pos_int(d, "width", ""), _number(_sub(d, "norm", ""), "eps", "norm."),
                  _pos_int(d, "streams", "") if streams is not None else None, tuple(layers))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        if self.streams is not None and self.streams > 16:
            raise ConfigError(f"streams {self.streams}: at most 16 residual streams are built")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            src = getattr(m, "kv_from", None)
            if src is None:
                continue
            if src >= i or self.layers[src].kind != layer.kind or self.layers[src].mixer.kv_from is not None:
                raise ConfigError(f"layers[{i}].mixer.kv_from {src} must name an earlier layer of the same type with keys and values of its own")
            o = self.layers[src].mixer
            if (o.kv_heads, o.dim, o.vdim) != (m.kv_heads, m.dim, m.vdim):
                raise ConfigError(f"layers[{i}] reads the keys and values of layer {src}, whose head sizes differ")


# ---------------------------------------------------------------------------------------------------------------------
# Zepalorn: a decoder whose config.json lists its layers one by one; a layer has one of three mixers and a gated
# feed-forward, and may run on the weights of an earlier layer.

def _opt_sub(d: Mapping[str, Any], key: str, where: str) -> Optional[Mapping[str, Any]]:
    v = d.get(key)
    if v is not None and not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


@dataclass(frozen=True)
class RotationConfig:
    """``rot``: how many entries of a head turn, the base of the frequencies, and (under ``scaling``) how they are stretched."""

    dims: int
    base: float
    factor: Optional[float] = None   # None: plain frequencies
    original: float = 0.0
    fast: float = 32.0
    slow: float = 1.0

    @classmethod
    def from_dict(cls, r: Mapping[str, Any], where: str) -> "RotationConfig":
        dims = _pos_int(r, "dims", where)
        if dims % 2:
            raise ConfigError(f"config.json: {where}'dims' must be even, got {dims}")
        base = _number(r, "base", where)
        if not base > 1:
            raise ConfigError(f"config.json: {where}'base' must be more than 1, got {base}")
        sc = _opt_sub(r, "scaling", where)
        if not sc:
            return cls(dims, base)
        w = where + "scaling."
        factor, original = _number(sc, "factor", w), _number(sc, "original", w)
        if not factor > 0 or not original > 0:
            raise ConfigError(f"config.json: {w}'factor' and 'original' must be positive")
        return cls(dims, base, factor, original, _number(sc, "fast", w), _number(sc, "slow", w))


@dataclass(frozen=True)
class MaskedAttentionConfig:
    """Softmax attention over grouped heads. As the mixer ``attention``: plain projections, pairs ``(i, i + dims/2)`` turn, a
    sliding window that keeps the first tokens. As the left half of ``parallel``: short convolutions, query/key norm,
    neighbouring pairs turn, a soft cap on the scores, chunks."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig] = None
    mask_size: Optional[int] = None    # the window, or the chunk
    keep_first: int = 0
    chunked: bool = False
    softcap: Optional[float] = None
    conv: int = 0
    qk_norm: bool = False
    interleaved: bool = False

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str, side_by_side: bool = False) -> "MaskedAttentionConfig":
        heads, kv_heads = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}{heads} heads cannot share {kv_heads} kv_heads")
        dim = _pos_int(m, "dim", where)
        rot = _opt_sub(m, "rot", where)
        rot = RotationConfig.from_dict(rot, where + "rot.") if rot else None
        if rot is not None and rot.dims > dim:
            raise ConfigError(f"config.json: {where}rot.dims {rot.dims} is more than dim {dim}")
        mask = _opt_sub(m, "mask", where)
        size = _pos_int(mask, "size", where + "mask.") if mask else None
        keep = 0
        if mask and mask.get("keep_first") is not None:
            keep = mask["keep_first"]
            if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
                raise ConfigError(f"config.json: {where}mask.keep_first must be a count, got {keep!r}")
            if side_by_side:
                raise ConfigError(f"config.json: {where}mask.keep_first belongs to a window, not to chunks")
        cap = _number(m, "softcap", where) if m.get("softcap") is not None else None
        if cap is not None and not cap > 0:
            raise ConfigError(f"config.json: {where}'softcap' must be positive, got {cap}")
        conv = _pos_int(m, "conv", where) if m.get("conv") is not None else 0
        if conv > 8:
            raise ConfigError(f"config.json: {where}'conv' must be 1 to 8 taps, got {conv}")
        if side_by_side and not conv:
            raise ConfigError(f"config.json: {where}'conv' is missing")
        return cls(heads, kv_heads, dim, _pos_int(m, "vdim", where) if "vdim" in m else dim, _number(m, "scale", where), rot, size, keep,
                   chunked=side_by_side, softcap=cap, conv=conv, qk_norm=side_by_side, interleaved=side_by_side)


@dataclass(frozen=True)
class DeltaConfig:
    """Mixer ``channel_delta``: the gated delta rule with a decay per head and key channel."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "DeltaConfig":
        heads, kv_heads = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}{heads} heads cannot share {kv_heads} kv_heads")
        dim, conv = _pos_int(m, "dim", where), _pos_int(m, "conv", where)
        if dim > 256:
            raise ConfigError(f"config.json: {where}'dim' {dim}: the delta rule is built for key sizes up to 256")
        if conv > 8:
            raise ConfigError(f"config.json: {where}'conv' must be 1 to 8 taps, got {conv}")
        return cls(heads, kv_heads, dim, _pos_int(m, "vdim", where), conv)


@dataclass(frozen=True)
class StateSpaceConfig:
    """The right half of ``parallel``: a state-space mixer with one decay per head."""

    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "StateSpaceConfig":
        c = cls(_pos_int(m, "heads", where), _pos_int(m, "vdim", where), _pos_int(m, "state", where), _pos_int(m, "groups", where),
                _pos_int(m, "norm_groups", where), _pos_int(m, "conv", where))
        if c.heads % c.groups:
            raise ConfigError(f"config.json: {where}{c.heads} heads cannot share {c.groups} groups")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"config.json: {where}{c.heads * c.vdim} channels cannot be normed in {c.norm_groups} equal parts")
        if c.state > 256:
            raise ConfigError(f"config.json: {where}'state' {c.state}: the recurrence is built for state sizes up to 256")
        if c.conv > 8:
            raise ConfigError(f"config.json: {where}'conv' must be 1 to 8 taps, got {c.conv}")
        return c


@dataclass(frozen=True)
class ParallelConfig:
    """Mixer ``parallel``: attention on the left, a state-space mixer on the right, both reading the same input."""

    left: MaskedAttentionConfig
    right: StateSpaceConfig

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "ParallelConfig":
        return cls(MaskedAttentionConfig.from_dict(_sub(m, "left", where), where + "left.", side_by_side=True),
                   StateSpaceConfig.from_dict(_sub(m, "right", where), where + "right."))


@dataclass(frozen=True)
class ZepalornLayerConfig:
    kind: str                       # "channel_delta", "attention" or "parallel"
    mixer: Any
    ff: Optional[int]               # width of the gated feed-forward, None: the layer has none
    ff_limit: float = 0.0
    weights_of: Optional[int] = None  # the layer whose tensors this one runs on (with a cache and state of its own)


@dataclass(frozen=True)
class ZepalornConfig:
    """The whole of a Zepalorn config.json: vocabulary, width, norm epsilon, the embedding's scale and the list of layers."""

    architecture = "Zepalorn"

    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple

    @staticmethod
    def _mixer(kind: str, m: Mapping[str, Any], where: str):
        if kind == "channel_delta":
            return DeltaConfig.from_dict(m, where)
        if kind == "attention":
            return MaskedAttentionConfig.from_dict(m, where)
        if kind == "parallel":
            return ParallelConfig.from_dict(m, where)
        raise ConfigError(f"config.json: {where[:-6]}type {kind!r} is not one of ['attention', 'channel_delta', 'parallel']")

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ZepalornConfig":
        if not isinstance(d.get("layers"), (list, tuple)) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, layer in enumerate(d["layers"]):
            where = f"layers[{i}]."
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            mixer = cls._mixer(kind, _sub(layer, "mixer", where), where + "mixer.")
            mlp = layer.get("mlp")
            ff, limit = None, 0.0
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}mlp must be null or an object of kind 'dense'")
                ff, limit = _pos_int(mlp, "ff", where + "mlp."), _number(mlp, "limit", where + "mlp.")
                if not limit > 0:
                    raise ConfigError(f"config.json: {where}mlp.limit must be positive, got {limit}")
            src = layer.get("weights_of")
            if src is not None and (isinstance(src, bool) or not isinstance(src, int) or src < 0):
                raise ConfigError(f"config.json: {where}'weights_of' must be a layer index, got {src!r}")
            layers.append(ZepalornLayerConfig(kind, mixer, ff, limit, src))
        emb = _opt_sub(d, "embedding", "")
        cfg = cls(_pos_int(d, "vocab", ""), _pos_int(d, "width", ""), _number(_sub(d, "norm", ""), "eps", "norm."),
                  _number(emb, "scale", "embedding.") if emb and emb.get("scale") is not None else 1.0, tuple(layers))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        for i, layer in enumerate(self.layers):
            src = layer.weights_of
            if src is None:
                continue
            if src == i or src >= len(self.layers) or self.layers[src].weights_of is not None:
                raise ConfigError(f"layers[{i}].weights_of {src} must name another layer, one with tensors of its own")
            o = self.layers[src]
            if (o.kind, o.mixer, o.ff, o.ff_limit) != (layer.kind, layer.mixer, layer.ff, layer.ff_limit):
                raise ConfigError(f"layers[{i}] runs on the weights of layer {src}, but the rest of its entry differs from that layer's")


# ---------------------------------------------------------------------------------------------------------------------
# Mufotar: a decoder whose config.json lists its layers one by one; in every layer the mixer and the feed-forward read the
# same normed input and their sum is added to the stream. Mixers: the gated delta rule with a decay per head, or softmax
# attention beside a selective scan; feed-forwards: a dense gated unit, or routed experts with identity experts and a shared one.

@dataclass(frozen=True)
class SelectiveScanConfig:
    """The right half of Mufotar's ``parallel`` mixer: a selective scan with a state per channel and state index."""

    inner: int
    state: int
    dt_rank: int
    conv: int

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "SelectiveScanConfig":
        c = cls(_pos_int(m, "inner", where), _pos_int(m, "state", where), _pos_int(m, "dt_rank", where), _pos_int(m, "conv", where))
        if c.state > 256:
            raise ConfigError(f"config.json: {where}'state' {c.state}: the recurrence is built for state sizes up to 256")
        if c.conv > 8:
            raise ConfigError(f"config.json: {where}'conv' must be 1 to 8 taps, got {c.conv}")
        return c


@dataclass(frozen=True)
class WeightedPairConfig:
    """Mixer ``parallel`` of Mufotar: attention on the left, a selective scan on the right, summed with a factor each."""

    left: MaskedAttentionConfig
    right: SelectiveScanConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "WeightedPairConfig":
        from dataclasses import replace

        left = MaskedAttentionConfig.from_dict(_sub(m, "left", where), where + "left.")
        if left.mask_size is not None or left.softcap is not None or left.conv:
            raise ConfigError(f"config.json: {where}left: this attention is causal, without mask, soft cap or convolution")
        return cls(replace(left, qk_norm=True), SelectiveScanConfig.from_dict(_sub(m, "right", where), where + "right."),
                   _number(m, "left_scale", where), _number(m, "right_scale", where))


@dataclass(frozen=True)
class RoutedExpertsConfig:
    """``mlp.kind = "moe"``: ``experts`` gated units of width ``ff`` of which a token uses ``top``; the router has ``identity`` more
    outputs, which stand for experts that return their input; ``shared_ff`` (or None) is the width of a unit that every token uses."""

    experts: int
    identity: int
    top: int
    ff: int
    shared_ff: Optional[int]

    @classmethod
    def from_dict(cls, mlp: Mapping[str, Any], where: str) -> "RoutedExpertsConfig":
        r = _sub(mlp, "router", where)
        identity = r.get("identity", 0) or 0
        if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
            raise ConfigError(f"config.json: {where}router.identity must be a count, got {identity!r}")
        shared = _opt_sub(mlp, "shared", where)
        c = cls(_pos_int(r, "experts", where + "router."), identity, _pos_int(r, "top", where + "router."),
                _pos_int(_sub(mlp, "expert", where), "ff", where + "expert."), _pos_int(shared, "ff", where + "shared.") if shared else None)
        if c.top > c.experts + c.identity:
            raise ConfigError(f"config.json: {where}router.top {c.top} is more than the router has outputs")
        if c.experts + c.identity > 512:
            raise ConfigError(f"config.json: {where}router: at most 512 outputs are built")
        return c


@dataclass(frozen=True)
class MufotarLayerConfig:
    kind: str                       # "delta" or "parallel"
    mixer: Any
    mlp: Any                        # None, the width of a dense gated unit, or a RoutedExpertsConfig
    weights_of: Optional[int] = None  # the layer whose tensors this one runs on (with a cache and state of its own)


@dataclass(frozen=True)
class MufotarConfig:
    """The whole of a Mufotar config.json: vocabulary, width, norm epsilon, the soft cap on the logits and the list of layers."""

    architecture = "Mufotar"

    vocab: int
    width: int
    eps: float
    logit_softcap: Optional[float]
    layers: tuple

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MufotarConfig":
        if not isinstance(d.get("layers"), (list, tuple)) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, layer in enumerate(d["layers"]):
            where = f"layers[{i}]."
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            m = _sub(layer, "mixer", where)
            if kind == "delta":
                mixer = DeltaConfig.from_dict(m, where + "mixer.")
            elif kind == "parallel":
                mixer = WeightedPairConfig.from_dict(m, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not one of ['delta', 'parallel']")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind", "dense") not in ("dense", "moe"):
                    raise ConfigError(f"config.json: {where}mlp must be null or an object of kind 'dense' or 'moe'")
                mlp = _pos_int(mlp, "ff", where + "mlp.") if mlp.get("kind", "dense") == "dense" else RoutedExpertsConfig.from_dict(mlp, where + "mlp.")
            src = layer.get("weights_of")
            if src is not None and (isinstance(src, bool) or not isinstance(src, int) or src < 0):
                raise ConfigError(f"config.json: {where}'weights_of' must be a layer index, got {src!r}")
            layers.append(MufotarLayerConfig(kind, mixer, mlp, src))
        cap = d.get("logit_softcap")
        cfg = cls(_pos_int(d, "vocab", ""), _pos_int(d, "width", ""), _number(_sub(d, "norm", ""), "eps", "norm."),
                  _number(d, "logit_softcap", "") if cap is not None else None, tuple(layers))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError(f"logit_softcap must be positive, got {self.logit_softcap}")
        for i, layer in enumerate(self.layers):
            src = layer.weights_of
            if src is None:
                continue
            if src == i or src >= len(self.layers) or self.layers[src].weights_of is not None:
                raise ConfigError(f"layers[{i}].weights_of {src} must name another layer, one with tensors of its own")
            o = self.layers[src]
            if (o.kind, o.mixer, o.mlp) != (layer.kind, layer.mixer, layer.mlp):
                raise ConfigError(f"layers[{i}] runs on the weights of layer {src}, but the rest of its entry differs from that layer's")


# ---------------------------------------------------------------------------------------------------------------------
# Memilorn: a decoder whose config.json lists its layers one by one; pre-norm layers (layer norms with a weight) whose sublayer
# results pass a layer scale; a run of layers may loop on the same weights, the embedding added again before every further pass.
# Mixers: a matrix memory with exponential gates (mLSTM), latent attention without positions, grouped attention whose heads'
# scores are mixed before the softmax. Feed-forward: routed experts with sigmoid scores on the experts' inputs, and a shared one.

@dataclass(frozen=True)
class MatrixMemoryConfig:
    """``mlstm``: ``heads`` heads with query/key size ``dim`` and value size ``vdim``; both gates' pre-activations are bounded by
    ``gate_cap * tanh(x / gate_cap)`` (None: not bounded)."""

    heads: int
    dim: int
    vdim: int
    gate_cap: Optional[float]

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "MatrixMemoryConfig":
        cap = _number(m, "gate_cap", where) if m.get("gate_cap") is not None else None
        if cap is not None and not cap > 0:
            raise ConfigError(f"config.json: {where}'gate_cap' must be positive, got {cap}")
        dim = _pos_int(m, "dim", where)
        if dim > 256:
            raise ConfigError(f"config.json: {where}'dim' {dim} is more than the 256 entries of a memory column that are built")
        return cls(_pos_int(m, "heads", where), dim, _pos_int(m, "vdim", where) if "vdim" in m else dim, cap)


@dataclass(frozen=True)
class PlainLatentConfig:
    """``latent_attention`` without positions: queries straight from the input, keys and values rebuilt from a normed latent of
    ``kv_rank`` entries per token."""

    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "PlainLatentConfig":
        dim = _pos_int(m, "dim", where)
        return cls(_pos_int(m, "heads", where), dim, _pos_int(m, "vdim", where) if "vdim" in m else dim, _pos_int(m, "kv_rank", where),
                   _number(m, "scale", where))


@dataclass(frozen=True)
class TalkingAttentionConfig:
    """``attention``: grouped heads, the first ``rot.dims`` entries of a head turned in neighbouring pairs, scores bounded by
    ``softcap`` and mixed between the heads before the softmax, a sink and a gate per head."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig]
    softcap: Optional[float]

    @classmethod
    def from_dict(cls, m: Mapping[str, Any], where: str) -> "TalkingAttentionConfig":
        heads, kv_heads = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}{heads} heads cannot share {kv_heads} kv_heads")
        dim = _pos_int(m, "dim", where)
        rot = _opt_sub(m, "rot", where)
        rot = RotationConfig.from_dict(rot, where + "rot.") if rot else None
        if rot is not None and rot.dims > dim:
            raise ConfigError(f"config.json: {where}rot.dims {rot.dims} is more than dim {dim}")
        if rot is not None and rot.factor is not None:
            raise ConfigError(f"config.json: {where}rot.scaling is not part of this architecture")
        cap = _number(m, "softcap", where) if m.get("softcap") is not None else None
        if cap is not None and not cap > 0:
            raise ConfigError(f"config.json: {where}'softcap' must be positive, got {cap}")
        return cls(heads, kv_heads, dim, _pos_int(m, "vdim", where) if "vdim" in m else dim, _number(m, "scale", where), rot, cap)


@dataclass(frozen=True)
class SigmoidExpertsConfig:
    """``mlp.kind = "moe"``: ``experts`` clamped gated units of width ``ff`` (bound ``limit``) of which a token uses ``top``, chosen
    and weighted by the sigmoid of the router's outputs; ``shared_ff`` / ``shared_limit``: a unit that every token uses (None: none)."""

    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: Optional[int]
    shared_limit: float

    @classmethod
    def from_dict(cls, mlp: Mapping[str, Any], where: str) -> "SigmoidExpertsConfig":
        r, e = _sub(mlp, "router", where), _sub(mlp, "expert", where)
        shared = _opt_sub(mlp, "shared", where)
        c = cls(_pos_int(r, "experts", where + "router."), _pos_int(r, "top", where + "router."), _pos_int(e, "ff", where + "expert."),
                _number(e, "limit", where + "expert."), _pos_int(shared, "ff", where + "shared.") if shared else None,
                _number(shared, "limit", where + "shared.") if shared else 0.0)
        if c.top > c.experts:
            raise ConfigError(f"config.json: {where}router.top {c.top} is more than the {c.experts} experts")
        if c.experts > 512:
            raise ConfigError(f"config.json: {where}router: at most 512 experts are built")
        if not c.limit > 0 or (shared and not c.shared_limit > 0):
            raise ConfigError(f"config.json: {where}the limit of a clamped unit must be positive")
        return c


@dataclass(frozen=True)
class MemilornLayerConfig:
    kind: str                       # "mlstm", "latent_attention" or "attention"
    mixer: Any
    mlp: Optional[SigmoidExpertsConfig]   # None: the layer is a mixer alone


@dataclass(frozen=True)
class MemilornConfig:
    """The whole of a Memilorn config.json: vocabulary, width, norm epsilon, the list of layers and the loop (layers
    ``loop_start .. loop_stop - 1`` run ``loop_times`` times in a row on the same weights; no ``loop``: every layer once)."""

    architecture = "Memilorn"

    vocab: int
    width: int
    eps: float
    layers: tuple
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1

    _MIXERS = {"mlstm": MatrixMemoryConfig, "latent_attention": PlainLatentConfig, "attention": TalkingAttentionConfig}

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MemilornConfig":
        if not isinstance(d.get("layers"), (list, tuple)) or not d["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, layer in enumerate(d["layers"]):
            where = f"layers[{i}]."
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            if kind not in cls._MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is not one of {sorted(cls._MIXERS)}")
            mixer = cls._MIXERS[kind].from_dict(_sub(layer, "mixer", where), where + "mixer.")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {where}mlp must be null or an object of kind 'moe'")
                mlp = SigmoidExpertsConfig.from_dict(mlp, where + "mlp.")
            layers.append(MemilornLayerConfig(kind, mixer, mlp))
        loop = _opt_sub(d, "loop", "")
        start = stop = 0
        times = 1
        if loop:
            for key in ("start", "stop", "times"):
                v = loop.get(key)
                if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                    raise ConfigError(f"config.json: loop.{key} must be a count, got {v!r}")
            start, stop, times = loop["start"], loop["stop"], loop["times"]
        cfg = cls(_pos_int(d, "vocab", ""), _pos_int(d, "width", ""), _number(_sub(d, "norm", ""), "eps", "norm."), tuple(layers), start, stop, times)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.eps}")
        if not 0 <= self.loop_start <= self.loop_stop <= len(self.layers):
            raise ConfigError(f"loop: layers {self.loop_start} .. {self.loop_stop} - 1 are not a run of the {len(self.layers)} layers")
        if self.loop_times < 1:
            raise ConfigError(f"loop.times must be at least 1, got {self.loop_times}")

    def running_order(self) -> list:
        """``(layer, pass, first of a further pass)`` in the order the layers run: the layers before the loop, the looped run
        ``loop_times`` times, the rest."""
        order = [(i, 0, False) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            order += [(i, t, t > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, 0, False) for i in range(self.loop_stop, len(self.layers))]
