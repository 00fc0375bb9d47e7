"""archkit: bring-up tooling for a new model package.

* ``adapt``: a Hugging Face ``config.json`` -> package description (per-layer kind table, needed capabilities, the
  capability gate's verdict) with the checks that a scaffolded config must pass before any kernel sees it: every
  layer has a kind, the kinds add up to the layer count, the id is a legal identifier.
* ``gates``: geometry and parallelism gates (head widths the kernels have, kv heads and weight columns divisible by
  the tensor-parallel world, nvfp4 scale tiles).
* ``matrix``: per-GPU budget table -- which weight formats fit, and the context each KV tier reaches beside them
  (the KV budget mirror of the bit-budget planner's tier widths).

Reference: tools/archkit (target scaffolder from a spec, geometry / parameter gates, GPU matrix, KV budget mirrors).
"""
from .adapt import adapt_config, fold_identifier            # noqa: F401
from .gates import geometry_gates                           # noqa: F401
from .matrix import GPUS, budget_matrix                     # noqa: F401
