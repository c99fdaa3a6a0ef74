"""shiso-llm for one B200: an inference engine for LFM2 built from parameterised parts.

Layers, top to bottom: the entry point and command line (``shiso_llm_b200.api``,
``python -m shiso_llm_b200``), the scheduler, the step function (``engine``), the cache
manager (``cache``), the model assembled from parts (``parts``) chosen by a typed
configuration (``config``) with weights loaded by name (``weights``), and hand-written
CUDA kernels for sm_100a (``csrc`` through ``kernels``).
"""

__version__ = "0.1.0"
