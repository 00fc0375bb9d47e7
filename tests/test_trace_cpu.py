"""Phase tracing: off by default, span log lines with the fixed vocabulary when switched on."""
import json

import pytest

from ninfer_fusion_b200.utils import trace


def test_spans_are_free_when_off_and_logged_when_on(tmp_path):
    trace.configure(nvtx=False, log_path="")
    assert not trace.enabled()
    with trace.span("engine", "no-such-name"):            # not even validated when tracing is off: zero cost
        pass
    log = tmp_path / "spans.jsonl"
    trace.configure(log_path=str(log))
    try:
        with trace.span("engine", "decode_round", lanes=3):
            pass
        with pytest.raises(ValueError, match="vocabulary"):
            with trace.span("engine", "no-such-name"):
                pass
        rows = [json.loads(l) for l in log.read_text().splitlines()]
        assert len(rows) == 1 and rows[0]["cat"] == "engine" and rows[0]["name"] == "decode_round" and rows[0]["lanes"] == 3
        assert rows[0]["ms"] >= 0
    finally:
        trace.configure(log_path="")


def test_engine_emits_prefill_and_decode_spans(tmp_path):
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.engine import Engine, RequestOptions
    from ninfer_fusion_b200.runtime.program import ReferenceProgram
    log = tmp_path / "engine.jsonl"
    trace.configure(log_path=str(log))
    w = random_weights(TINY_DENSE, "cpu", seed=1, std=0.05)
    eng = Engine(lambda: ReferenceProgram(TINY_DENSE, w, max_lanes=2, max_context=128), prefill_chunk=16)
    try:
        eng.generate(list(range(5, 45)), RequestOptions(max_tokens=3))
    finally:
        eng.shutdown()
        trace.configure(log_path="")
    names = [json.loads(l)["name"] for l in log.read_text().splitlines()]
    assert names.count("prefill_chunk") == 3 and names.count("decode_round") >= 2


def test_progress_bar_is_silent_off_a_terminal_and_draws_on_one():
    import io
    from ninfer_fusion_b200.utils.progress import Progress
    quiet = io.StringIO()
    p = Progress(100, "loading", stream=quiet)
    p.advance(50, "a"); p.advance(50, "b"); p.close()
    assert quiet.getvalue() == "" and p.done == 100
    loud = io.StringIO()
    p = Progress(4 << 20, "loading", stream=loud, force=True)
    p.advance(1 << 20, "text/embed"); p.advance(10 << 20, "text/lm_head"); p.close()
    out = loud.getvalue()
    assert "100.0%" in out and "text/lm_head" in out and out.endswith("\n") and p.done == 4 << 20
