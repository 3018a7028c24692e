"""A one-GPU inference engine for the OPT decoder on NVIDIA B200 (sm_100a): typed configuration,
weights by name, layers put together from parts, a paged cache, one step function, a scheduler,
sampling, and hand-written CUDA kernels.  Capabilities follow aws-neuron/transformers-neuronx's OPT
support; the design does not."""
__version__ = "0.1.0"

from .config.generation_config import ContinuousBatchingConfig, GenerationConfig, NeuronConfig      # as `from transformers_neuronx import ...`
