"""A one-GPU inference engine for the OPT decoder on NVIDIA B200 (sm_100a): typed configuration,
weights by name, layers put together from parts, a paged cache, one step function, a scheduler,
sampling, and hand-written CUDA kernels.  Capabilities follow aws-neuron/transformers-neuronx's OPT
support; the design does not."""
__version__ = "0.1.0"

from .config.generation_config import (BlkSparseAttnConfig, ContinuousBatchingConfig, GenerationConfig, NeuronConfig,
                                       SlidingWindowAttnConfig, SparseAttnConfig)      # as `from transformers_neuronx import ...`

_LAZY = {"OPTForSampling": ".opt.model", "OPTForGreedySearch": ".opt.model",
         "NeuronAutoModelForCausalLM": ".modeling_auto", "HuggingFaceGenerationModelAdapter": ".generation_utils"}


def __getattr__(name):
    """The entry-point classes under the package's own name, as `from transformers_neuronx import OPTForSampling`
    (src/transformers_neuronx/__init__.py); imported when first asked for."""
    if name in _LAZY:
        import importlib
        return getattr(importlib.import_module(_LAZY[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
