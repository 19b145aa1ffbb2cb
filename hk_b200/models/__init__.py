from . import kedanex, mifolorn, padodra, qwen3, zazulix  # noqa: F401  (register the architectures)
from .spec import LayerCall, ModelSpec

__all__ = ["LayerCall", "ModelSpec"]
