from .decoder import DecoderModel
from . import opt  # noqa: F401  registers OPTForCausalLM; another built-in architecture is one more line here
