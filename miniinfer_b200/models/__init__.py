from . import qwen3  # noqa: F401  (registers the architecture)
from .spec import LayerRun, ModelSpec

__all__ = ["LayerRun", "ModelSpec"]
