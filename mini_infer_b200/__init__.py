"""mini_infer_b200: a small, whole inference engine for one GPU (B200, sm_100a).

From a model folder (``config.json`` + safetensors) or seeded random weights to
generated tokens: typed configuration and registries (``config``), checkpoint
reading (``weights``), layers put together from parts (``parts``, ``models``),
a paged cache manager (``cache``), the step function, scheduler and entry
points (``engine``), sampling (``sampling``) and hand-written CUDA kernels
(``csrc``, bound in ``ops``).
"""

__version__ = "0.1.0"
