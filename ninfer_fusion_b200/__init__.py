"""B200-native (sm_100a) LLM inference engine for Qwen3.x hybrid decoders.

Layers (bottom to top): ``csrc`` (hand-written CUDA kernels and the native
runtime), ``ops`` (checked Python entry points + fp32 torch oracles),
``models`` (hybrid GDN/GQA decoders, dense and MoE, MTP draft head),
``parallel`` (rank runtime, shard plan, fused collectives), ``runtime``
(paged KV pool, state pools, CUDA-graph families, engine/scheduler),
``kv`` (codec policy: bit budget, block descent, tiers; speculative
decoding lives in ``runtime.speculative``), ``artifact`` (.ninfer v2 container), ``serve`` /
``cli`` (gateways).
"""

__version__ = "0.1.0"

from ._lib import load_native, native_available  # noqa: F401
