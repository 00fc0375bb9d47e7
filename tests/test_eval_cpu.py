"""Evaluation coordinator: mock suite, resume, scorers, and an OpenAI-compatible target served by this package."""
import json
import os
import threading

import pytest

from ninfer_fusion_b200.eval import Coordinator, load_config, run_suite
from ninfer_fusion_b200.eval import tasks as T


def test_scorers():
    assert T.score_exact(" Paris ", {"answer": "paris"}) == 1.0
    assert T.score_contains("the code is 123456.", {"answer": "123456"}) == 1.0
    assert T.score_choice("I think the answer is B", {"answer": "b"}) == 1.0
    assert T.score_choice("A or maybe C", {"answer": "A"}) == 0.0
    assert T.score_number("so we get 1,234.0", {"answer": "1234"}) == 1.0
    s = list(T.needle_samples({"lengths": [50], "depths": [0.5], "seed": 1}))
    assert len(s) == 1 and s[0]["answer"] in s[0]["prompt"]
    msgs = T.build_messages({"task": "multiple_choice", "system": "be brief"}, {"question": "Pick", "choices": ["x", "y"]})
    assert msgs[0]["role"] == "system" and "B. y" in msgs[1]["content"]


def test_mock_suite_and_resume(tmp_path):
    here = os.path.dirname(os.path.abspath(T.__file__))
    out = str(tmp_path / "run")
    res = run_suite(os.path.join(here, "mock-suite.yaml"), out)
    jobs = {j["job"]: j for j in res["jobs"]}
    assert jobs["arithmetic"]["samples"] == 4 and jobs["needle"]["samples"] == 6
    assert 0.0 <= jobs["arithmetic"]["score"] <= 1.0 and jobs["needle"]["errors"] == 0
    events = [json.loads(l) for l in open(os.path.join(out, "events.jsonl"))]
    assert events[0]["event"] == "suite_start" and events[-1]["event"] == "suite_done"
    assert sum(e["event"] == "sample_done" for e in events) == 10
    # second run resumes: nothing left to do, same scores
    res2 = run_suite(os.path.join(here, "mock-suite.yaml"), out)
    assert [j["score"] for j in res2["jobs"]] == [j["score"] for j in res["jobs"]]
    events2 = [json.loads(l) for l in open(os.path.join(out, "events.jsonl"))]
    assert sum(e["event"] == "sample_done" for e in events2) == 10
    with pytest.raises(ValueError):
        load_config_from({"targets": {}, "jobs": [{"name": "x", "target": "nope"}]}, tmp_path)


def load_config_from(cfg, tmp_path):
    import yaml
    p = str(tmp_path / "bad.yaml")
    with open(p, "w") as f:
        yaml.safe_dump(cfg, f)
    return load_config(p)


def test_openai_target_against_local_server(tmp_path):
    import torch
    from ninfer_fusion_b200 import cli
    from ninfer_fusion_b200.frontend.tokenizer import Tokenizer
    from ninfer_fusion_b200.models.config import TINY_DENSE
    from ninfer_fusion_b200.models.weights import random_weights
    from ninfer_fusion_b200.runtime.engine import Engine
    from ninfer_fusion_b200.runtime.program import ReferenceProgram
    from ninfer_fusion_b200.serve.server import serve
    from ninfer_fusion_b200.serve.service import GenerationService

    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=3, std=0.05)
    tok = Tokenizer.train_toy(cli.DEFAULT_CORPUS, 200, cli.SPECIAL_TOKENS)
    engine = Engine(lambda: ReferenceProgram(cfg, w, max_lanes=2, max_context=256), prefill_chunk=64)
    svc = GenerationService(engine, tok, "tiny", max_concurrent=2)
    httpd = serve(svc, "127.0.0.1", 0, api_key="k")
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        suite = {"targets": {"local": {"protocol": "openai_chat", "base_url": f"http://127.0.0.1:{httpd.server_address[1]}/v1",
                                       "model": "tiny", "api_key": "k", "max_concurrency": 2,
                                       "request": {"timeout_seconds": 60, "retries": 0}}},
                 "jobs": [{"name": "smoke", "target": "local", "scorer": "contains", "generation": {"max_tokens": 4, "temperature": 0},
                           "samples": [{"prompt": "hello", "answer": "x"}, {"prompt": "bye", "answer": "y"}]}]}
        res = Coordinator(suite, str(tmp_path / "o")).run()
        j = res["jobs"][0]
        assert j["samples"] == 2 and j["errors"] == 0 and j["completion_tokens"] > 0
    finally:
        httpd.shutdown()
        httpd.server_close()
        engine.shutdown()
