from . import koronex, qwen2  # noqa: F401  (register Koronex and Qwen2ForCausalLM)
from .decoder import DecoderModel
