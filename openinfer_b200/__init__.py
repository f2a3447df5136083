"""openinfer_b200: a small, whole inference engine for one GPU (B200, sm_100a).

From a model folder (config.json + safetensors, or a configuration and a seed) to
generated tokens: typed config and architecture registry, weights by tensor name, layers
assembled from parts, a paged cache manager, one step function for mixed batches, a
continuous-batching scheduler, sampling, and hand-written CUDA kernels.
"""
__version__ = "0.1.0"
