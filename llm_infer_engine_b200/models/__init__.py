from . import llama, zemivik  # noqa: F401  (register LlamaForCausalLM and Zemivik)
from .decoder import DecoderModel

__all__ = ["DecoderModel"]
