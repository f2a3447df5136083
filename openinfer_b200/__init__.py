"""openinfer_b200: a small, whole inference engine for one GPU (B200, sm_100a).

From a model folder (config.json + safetensors, or a configuration and a seed) to
generated tokens: typed config and architecture registry, weights by tensor name, layers
assembled from parts, a paged cache manager, one step function for mixed batches, a
continuous-batching scheduler, sampling, and hand-written CUDA kernels.

    from openinfer_b200 import LLM, SamplingParams
    llm = LLM("/path/to/model")
    tokens = llm.generate([[1, 2, 3]], SamplingParams(temperature=0.8, seed=1), max_tokens=16)
"""
__version__ = "0.1.0"

_LAZY = {
    "LLM": ("openinfer_b200.engine.engine", "LLM"),
    "generate": ("openinfer_b200.engine.engine", "generate"),
    "SamplingParams": ("openinfer_b200.sampling.params", "SamplingParams"),
    "TokenLogprob": ("openinfer_b200.sampling.params", "TokenLogprob"),
    "ModelRunner": ("openinfer_b200.engine.runner", "ModelRunner"),
    "StepEntry": ("openinfer_b200.engine.runner", "StepEntry"),
    "load_config": ("openinfer_b200.config.base", "load_config"),
    "write_random_model": ("openinfer_b200.weights.random", "write_random_model"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module 'openinfer_b200' has no attribute {name!r}")
