from . import dotivik, koronex, qwen2  # noqa: F401  (register Dotivik, Koronex and Qwen2ForCausalLM)
from .decoder import DecoderModel
