"""agave_b200: a small Gemma 3 generation library for one B200.

Everything between a request's token ids and its next token: typed
configuration and architecture registry, safetensors weights by name, layers
assembled from parts, a paged slot cache, one batched step function, a
generation loop with sampling, and hand-written sm_100a kernels under it.
"""
__version__ = "0.1.0"

from . import models as _models      # registers the architectures


def __getattr__(name):
    # the engine needs torch with CUDA; keep `import agave_b200` light
    if name == "Engine":
        from .engine.api import Engine
        return Engine
    if name == "SamplingParams":
        from .sampling import SamplingParams
        return SamplingParams
    raise AttributeError(name)
