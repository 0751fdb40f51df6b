"""tgo_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

From a model folder (config.json + safetensors) to next-token logits and generated
tokens: typed configuration and registries, weights by tensor name, layers put
together from parts, a paged cache with block tables, one step function for mixed
batches, a scheduler, samplers, and hand-written CUDA kernels. There is no CPU path.
"""
from .api import LoadedModel, open, open_random  # noqa: A004,F401

__version__ = "0.1.0"
