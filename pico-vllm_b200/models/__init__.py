from .decoder import DecoderModel, LayerCall, Binding
from .qwen2 import build_qwen2
from .zapipel import build_zapipel

__all__ = ["DecoderModel", "LayerCall", "Binding", "build_qwen2", "build_zapipel"]
