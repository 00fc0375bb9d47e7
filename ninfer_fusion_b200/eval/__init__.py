"""Capability evaluation coordinator: YAML suites of jobs run against model targets (this server, any OpenAI-compatible
endpoint, or a deterministic mock), with bounded concurrency, JSONL events, resume and rule-based scoring.

Counterpart of the reference's `eval/ninfer_eval` coordinator (configuration / events / progress / result contracts,
mock backend); the EvalScope backend is gated on that package being importable.
"""
from .coordinator import Coordinator, load_config, run_suite  # noqa: F401
