"""shiso-llm for one B200: an inference engine for LFM2 built from parameterised parts.

Layers, top to bottom: the entry point and command line (``shiso_llm_b200.api``,
``python -m shiso_llm_b200``), the scheduler, the step function (``engine``), the cache
manager (``cache``), the model assembled from parts (``parts``) chosen by a typed
configuration (``config``) with weights loaded by name (``weights``), and hand-written
CUDA kernels for sm_100a (``csrc`` through ``kernels``).
"""

__version__ = "0.1.0"


def __getattr__(name):
    # Imported lazily so that `import shiso_llm_b200` stays light (no torch import).
    if name in ("LLM", "Output"):
        from . import api

        return getattr(api, name)
    if name == "SamplingParams":
        from .sampling.params import SamplingParams

        return SamplingParams
    if name in ("Engine", "EngineOptions", "StepEntry"):
        from . import engine

        return getattr(engine, name)
    raise AttributeError(name)
