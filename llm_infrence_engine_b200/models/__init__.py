from . import luvutar, memilorn, mufotar, qwen2, zepalorn  # noqa: F401  (each registers its architecture)
from .registry import build_model_spec, known_architectures, lookup, parse_config, register_architecture
from .spec import LayerCall, ModelSpec, sequential

__all__ = ["build_model_spec", "known_architectures", "lookup", "parse_config", "register_architecture",
           "LayerCall", "ModelSpec", "sequential"]
