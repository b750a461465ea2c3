from . import dofipel, llama, zemivik  # noqa: F401  (register LlamaForCausalLM, Zemivik and Dofipel)
from .decoder import DecoderModel

__all__ = ["DecoderModel"]
