"""`ninfer-serve` over the CPU oracle program: OpenAI chat / responses, Anthropic messages, SSE, auth, logs, CLI."""
import http.client
import json
import os
import threading
import time

import pytest
import torch

from ninfer_fusion_b200 import cli
from ninfer_fusion_b200.frontend.tokenizer import Tokenizer
from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.weights import random_weights
from ninfer_fusion_b200.runtime.engine import Engine
from ninfer_fusion_b200.runtime.program import ReferenceProgram
from ninfer_fusion_b200.serve.server import serve
from ninfer_fusion_b200.serve.service import GenerationService, GenRequest


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=3, std=0.05)
    tok = Tokenizer.train_toy(cli.DEFAULT_CORPUS, 200, cli.SPECIAL_TOKENS)
    engine = Engine(lambda: ReferenceProgram(cfg, w, max_lanes=4, max_context=512), prefill_chunk=64)
    svc = GenerationService(engine, tok, "tiny-dense:test", max_concurrent=4, queue_timeout_s=20.0)
    log = str(tmp_path_factory.mktemp("log") / "requests.jsonl")
    httpd = serve(svc, "127.0.0.1", 0, api_key="sekret", log_path=log)
    t = threading.Thread(target=httpd.serve_forever, daemon=True)
    t.start()
    yield httpd.server_address[1], svc, log
    httpd.shutdown()
    httpd.server_close()
    engine.shutdown()


def call(port, method, path, body=None, key="sekret", header="Authorization"):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
    headers = {"Content-Type": "application/json"}
    if key:
        headers[header] = f"Bearer {key}" if header == "Authorization" else key
    c.request(method, path, json.dumps(body) if body is not None else None, headers)
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, r.getheader("Content-Type", ""), data


def sse_events(data: bytes):
    out = []
    for block in data.decode("utf-8").split("\n\n"):
        ev, payload = None, None
        for line in block.split("\n"):
            if line.startswith("event: "):
                ev = line[7:]
            elif line.startswith("data: "):
                payload = line[6:]
        if payload is not None:
            out.append((ev, payload if payload == "[DONE]" else json.loads(payload)))
    return out


def test_response_store_is_bounded_and_bad_content_length_is_a_400(server):
    port, svc, _ = server
    import socket as _socket

    from ninfer_fusion_b200.serve import server as S
    # the store drops its least recently used entry once it is full
    st = S.ServeState(svc, None, None, max_stored_responses=2)
    handler = S.make_handler(st)
    assert handler is not None
    for i in range(3):
        with st.lock:
            st.responses[f"r{i}"] = {"id": f"r{i}"}
            st.responses.move_to_end(f"r{i}")
            while len(st.responses) > st.max_stored_responses:
                st.responses.popitem(last=False)
    assert list(st.responses) == ["r1", "r2"]
    # a Content-Length that is not a number is the client's mistake, not a server error
    c = _socket.create_connection(("127.0.0.1", port), timeout=30)
    c.sendall(b"POST /v1/chat/completions HTTP/1.1\r\nHost: x\r\nAuthorization: Bearer sekret\r\n"
              b"Content-Type: application/json\r\nContent-Length: banana\r\nConnection: close\r\n\r\n{}")
    head = c.recv(4096).decode("latin1")
    c.close()
    assert head.startswith("HTTP/1.1 400"), head[:200]


def test_health_models_auth(server):
    port, svc, _ = server
    st, _, data = call(port, "GET", "/health", key=None)
    assert st == 200 and json.loads(data)["status"] == "ok"
    assert call(port, "GET", "/v1/models", key=None)[0] == 401
    assert call(port, "GET", "/v1/models", key="wrong")[0] == 401
    st, _, data = call(port, "GET", "/v1/models", key="sekret", header="x-api-key")
    assert st == 200 and json.loads(data)["data"][0]["id"] == "tiny-dense:test"
    assert call(port, "GET", "/v1/models/tiny-dense:test")[0] == 200
    assert call(port, "GET", "/v1/models/other")[0] == 404
    assert call(port, "GET", "/nope")[0] == 404


def test_openai_chat_blocking_and_streaming_agree(server):
    port, svc, _ = server
    body = {"model": "x", "messages": [{"role": "user", "content": "Hello there"}], "max_tokens": 12, "temperature": 0}
    st, ct, data = call(port, "POST", "/v1/chat/completions", body)
    assert st == 200 and ct.startswith("application/json")
    obj = json.loads(data)
    assert obj["object"] == "chat.completion" and obj["choices"][0]["finish_reason"] in ("stop", "length")
    assert obj["usage"]["completion_tokens"] <= 12 and obj["usage"]["prompt_tokens"] > 3
    text = obj["choices"][0]["message"]["content"] or ""
    st, ct, data = call(port, "POST", "/v1/chat/completions", dict(body, stream=True, stream_options={"include_usage": True}))
    assert st == 200 and ct.startswith("text/event-stream")
    evs = sse_events(data)
    assert evs[-1][1] == "[DONE]"
    chunks = [e for _, e in evs[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    streamed = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert streamed == text  # greedy: same tokens
    assert any(c.get("usage") for c in chunks)
    assert [c for c in chunks if c["choices"] and c["choices"][0]["finish_reason"]]


def test_openai_chat_rejects_bad_requests(server):
    port, _, _ = server
    assert call(port, "POST", "/v1/chat/completions", {"messages": []})[0] == 400
    assert call(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "n": 2})[0] == 400
    st, _, data = call(port, "POST", "/v1/chat/completions",
                       {"messages": [{"role": "user", "content": "x"}], "response_format": {"type": "json_schema"}})
    assert st == 400 and json.loads(data)["error"]["code"] == "unsupported_parameter"
    st, _, data = call(port, "POST", "/v1/chat/completions",
                       {"messages": [{"role": "user", "content": "x"}], "max_tokens": 100000})
    assert st == 400 and "context window" in json.loads(data)["error"]["message"]
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=10)
    c.request("POST", "/v1/chat/completions", "{not json", {"Authorization": "Bearer sekret", "Content-Type": "application/json"})
    assert c.getresponse().status == 400


def test_openai_responses_store_and_continuation(server):
    port, _, _ = server
    st, _, data = call(port, "POST", "/v1/responses", {"input": "Say hi", "max_output_tokens": 8, "temperature": 0})
    assert st == 200
    obj = json.loads(data)
    assert obj["object"] == "response" and obj["status"] in ("completed", "incomplete")
    assert obj["usage"]["output_tokens"] <= 8 and obj["output"][-1]["type"] in ("message", "function_call")
    rid = obj["id"]
    st, _, data = call(port, "GET", f"/v1/responses/{rid}")
    assert st == 200 and json.loads(data)["id"] == rid
    st, _, data = call(port, "GET", f"/v1/responses/{rid}/input_items")
    assert st == 200 and json.loads(data)["data"][0]["content"] == "Say hi"
    st, _, data = call(port, "POST", "/v1/responses", {"input": "And again", "previous_response_id": rid,
                                                       "max_output_tokens": 4, "temperature": 0, "stream": True})
    evs = sse_events(data)
    names = [e for e, _ in evs]
    assert names[0] == "response.created" and names[-1] in ("response.completed", "response.incomplete")
    st, _, data = call(port, "POST", "/v1/responses/input_tokens", {"input": "count me"})
    assert st == 200 and json.loads(data)["input_tokens"] > 2
    st, _, data = call(port, "POST", "/v1/responses/compact", {"input": [{"type": "message", "role": "user", "content": "a " * 50},
                                                                        {"type": "message", "role": "user", "content": "b"}],
                                                              "max_input_tokens": 12})
    assert st == 200 and json.loads(data)["output"][-1]["content"] == "b" and len(json.loads(data)["output"]) == 1
    assert call(port, "DELETE", f"/v1/responses/{rid}")[0] == 200
    assert call(port, "GET", f"/v1/responses/{rid}")[0] == 404
    assert call(port, "POST", "/v1/responses", {"input": "x", "previous_response_id": "resp_missing"})[0] == 404


def test_anthropic_messages(server):
    port, _, _ = server
    body = {"model": "x", "max_tokens": 10, "temperature": 0, "system": "Be brief.",
            "messages": [{"role": "user", "content": [{"type": "text", "text": "Hello"}]}]}
    st, _, data = call(port, "POST", "/v1/messages", body, header="x-api-key")
    assert st == 200
    obj = json.loads(data)
    assert obj["type"] == "message" and obj["role"] == "assistant" and obj["stop_reason"] in ("end_turn", "max_tokens")
    assert obj["usage"]["output_tokens"] <= 10 and obj["content"][-1]["type"] == "text"
    st, ct, data = call(port, "POST", "/v1/messages", dict(body, stream=True), header="x-api-key")
    names = [e for e, _ in sse_events(data)]
    assert names[0] == "message_start" and names[-1] == "message_stop" and "message_delta" in names
    st, _, data = call(port, "POST", "/v1/messages/count_tokens", {"messages": body["messages"]}, header="x-api-key")
    assert st == 200 and json.loads(data)["input_tokens"] > 2
    st, _, data = call(port, "POST", "/v1/messages", {"messages": body["messages"]}, header="x-api-key")
    assert st == 400 and json.loads(data)["type"] == "error"


def test_request_log_lines(server):
    port, _, log = server
    call(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "log me"}], "max_tokens": 3})
    recs = [json.loads(line) for line in open(log, encoding="utf-8")]
    kinds = {r["event"] for r in recs}
    assert {"server_start", "request_start", "request_done"} <= kinds and "request_rejected" in kinds
    done = [r for r in recs if r["event"] == "request_done"][-1]
    # the reference's measurement-log contract: schema name and version, ids on every line, raw counts and seconds
    assert done["schema"] == "ninfer_serve_request_log" and done["schema_version"] == 18
    assert all("timestamp_unix_ms" in r and r["server_instance_id"] == done["server_instance_id"] for r in recs)
    assert done["protocol"] == "openai_chat" and done["tokens"]["completion"] <= 3
    assert done["tokens"]["prompt"] == done["tokens"]["cached"] + done["tokens"]["computed_prefill"]
    assert done["reuse_path"] in ("root", "private_endpoint", "private_turn_closure", "private_response_replay",
                                  "private_long_anchor", "shared_stable_prefix")
    t = done["timings_seconds"]
    assert set(t) == {"prepare", "ttft", "vision", "prefill", "decode", "total"} and t["total"] >= t["ttft"] > 0
    assert done["engine_timing"]["queue_wait_seconds"] >= 0 and done["engine_timing"]["units"]["prefill"] >= 1
    et = done["engine_timing"]
    # exposure accounting: the units this request took part in, split into device wait (none on the CPU program) and
    # host-active time; the five host phases of the reference's schema are present, only their total is measured
    assert et["device_wait_exposed_seconds"] == 0.0 and et["host_exposed_seconds"]["total"] > 0
    assert set(et["host_exposed_seconds"]) == {"engine_boundary", "program_submit", "program_post", "engine_commit_output",
                                               "engine_maintenance", "total"}
    assert et["decode"]["rounds"] >= 1 and 0 < et["decode"]["host_exposed_seconds"] <= et["host_exposed_seconds"]["total"]
    assert et["host_exposed_seconds"]["total"] <= t["total"] + 1e-6
    assert set(done["speculative"]) == {"backend", "draft_window", "rounds", "drafted_tokens", "accepted_tokens",
                                        "fallback_steps", "accepted_per_position"}
    start = [r for r in recs if r["event"] == "server_start"][-1]
    assert "sekret" not in json.dumps(start) and "argv" in start
    rs = [r for r in recs if r["event"] == "request_start"][-1]
    assert rs["output_budget"] == 3 and "sampler" in rs


def test_overload_is_429(server):
    port, svc, _ = server
    held = [svc._permits.acquire(blocking=False) for _ in range(svc.max_concurrent)]
    try:
        st, _, data = call(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}]})
        assert st == 429 and json.loads(data)["error"]["code"] == "server_overloaded"
    finally:
        for h in held:
            if h:
                svc._permits.release()


def test_cli_artifact_roundtrip(tmp_path, capsys):
    art = str(tmp_path / "tiny.ninfer")
    assert cli.main(["make-artifact", "--model", "tiny-dense", "--out", art]) == 0
    assert cli.main(["inspect", art]) == 0
    listing = json.loads(capsys.readouterr().out)
    names = {o["name"] for o in listing["objects"]}
    assert {"tokenizer.json", "chat_template.jinja", "text/embed"} <= names
    assert cli.main(["generate", "--artifact", art, "--device", "cpu", "--prompt", "Hello", "--max-tokens", "5",
                     "--temperature", "0"]) == 0
    out = capsys.readouterr()
    stats = json.loads(out.err.strip().splitlines()[-1])
    assert stats["completion_tokens"] <= 5 and stats["model"].startswith("tiny-dense")
    corpus = tmp_path / "c.txt"
    corpus.write_text("the quick brown fox jumps over the lazy dog " * 4)
    assert cli.main(["perplexity", "--artifact", art, "--corpus", str(corpus), "--max-tokens", "40"]) == 0
    ppl = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert ppl["perplexity"] > 1.0


def test_loadgen_against_the_server(server):
    from ninfer_fusion_b200.serve.loadgen import run_level
    port, _, _ = server
    res = run_level(f"http://127.0.0.1:{port}/v1", "tiny-dense:test", ["hello there", "count to three"], concurrency=2,
                    n_requests=4, max_tokens=5, api_key="sekret")
    assert res["ok"] == 4 and res["errors"] == 0
    assert res["output_tokens"] >= 4 and res["ttft_ms_p50"] is not None and res["output_tok_s"] > 0
    bad = run_level(f"http://127.0.0.1:{port}/v1", "tiny-dense:test", ["x"], 1, 1, 2, api_key="wrong")
    assert bad["ok"] == 0 and bad["errors"] == 1


def test_first_token_campaign_reports_cold_and_warm_runs(server):
    from ninfer_fusion_b200.serve.loadgen import FILLER, sized_prompt, ttft_campaign
    port, svc, _ = server
    assert sized_prompt(300, "a", 100.0).count(FILLER) == 3 and sized_prompt(300, "a", 100.0).startswith("[a] ")
    per = len(svc.tok.encode(FILLER))
    recs = ttft_campaign(f"http://127.0.0.1:{port}/v1", "tiny-dense:test", [per, 2 * per], repeats=2, api_key="sekret")
    assert [r["target_tokens"] for r in recs] == [per, 2 * per]
    for r in recs:
        assert r["ok"] == 2 and r["errors"] == 0 and r["ttft_cold_ms_p50"] > 0 and r["prefill_tok_s"] > 0
        assert r["cold_cached_tokens_max"] == 0 and r["ttft_warm_ms"] > 0       # unique heads: nothing to reuse when cold
        assert r["warm_cached_tokens"] > 0                                     # the repeat starts from the kept frontier
    assert recs[1]["prompt_tokens"] > recs[0]["prompt_tokens"] >= per


def test_service_finds_the_shared_system_prefix(server):
    _, svc, _ = server
    long_system = "You are a careful assistant. " * 12
    req = GenRequest(messages=[{"role": "system", "content": long_system}, {"role": "user", "content": "hi"}], max_tokens=2)
    ids = svc.prepare(req)
    n = svc.shared_prefix_tokens(req, ids)
    assert 32 <= n < len(ids)
    assert svc.tok.decode(ids[:n]).endswith("<|im_end|>\n") or svc.tok.decode(ids[:n], skip_special=False).endswith("<|im_end|>\n")
    short = GenRequest(messages=[{"role": "system", "content": "Be brief."}, {"role": "user", "content": "hi"}], max_tokens=2)
    assert svc.shared_prefix_tokens(short, svc.prepare(short)) == 0
    none = GenRequest(messages=[{"role": "user", "content": "hi"}], max_tokens=2)
    assert svc.shared_prefix_tokens(none, svc.prepare(none)) == 0
    before = svc.engine.program.shared_stats["published"]
    a = svc.generate(GenRequest(messages=req.messages, max_tokens=3, temperature=0.0, session="u1"))
    b = svc.generate(GenRequest(messages=[req.messages[0], {"role": "user", "content": "other question"}], max_tokens=3,
                                temperature=0.0, session="u2"))
    assert a.error == "" and b.error == ""
    assert svc.engine.program.shared_stats["published"] == before + 1 and svc.engine.program.shared_stats["hits"] >= 1


def test_browser_console_is_served_without_a_key_and_uses_public_routes(server):
    port, _, _ = server
    for path in ("/", "/console"):
        status, ctype, data = call(port, "GET", path, key=None)
        assert status == 200 and ctype.startswith("text/html")
        page = data.decode("utf-8")
        assert "<title>ninfer-fusion-b200 console</title>" in page
        # it only ever calls routes any client can call, and sends the typed key as a bearer header
        assert "/v1/chat/completions" in page and "/v1/models" in page and "/health" in page and "Bearer" in page
    assert call(port, "GET", "/v1/models", key=None)[0] == 401          # the API itself still wants the key
    # what the page sends is accepted by the chat route
    body = {"model": "tiny-dense:test", "messages": [{"role": "user", "content": "hi"}], "stream": True, "max_tokens": 4,
            "temperature": 0.7, "enable_thinking": False}
    status, ctype, data = call(port, "POST", "/v1/chat/completions", body)
    assert status == 200 and ctype.startswith("text/event-stream") and sse_events(data)[-1][1] == "[DONE]"


def test_response_replay_frontier(server):
    """A chat request of a session leaves a frontier before the generation opener; asking for the same response again
    (same history, thinking switched the other way, so another opener) starts from it."""
    port, svc, _ = server
    msgs = [{"role": "user", "content": "tell me about pages and frontiers " * 3}]
    body = {"model": "tiny-dense:test", "messages": msgs, "max_tokens": 4, "user": "replay-session", "enable_thinking": True}
    assert call(port, "POST", "/v1/chat/completions", body)[0] == 200
    prog = svc.engine.program
    kinds = {c.kind for c in prog.checkpoints if c.session == "replay-session"}
    assert "replay" in kinds and "turn" in kinds
    replay = next(c for c in prog.checkpoints if c.session == "replay-session" and c.kind == "replay")
    turn = next(c for c in prog.checkpoints if c.session == "replay-session" and c.kind == "turn")
    assert 0 < len(replay.tokens) < len(turn.tokens) and turn.tokens[:len(replay.tokens)] == replay.tokens
    hits = svc.engine.stats.prefix_hits
    assert call(port, "POST", "/v1/chat/completions", dict(body, enable_thinking=False))[0] == 200
    assert svc.engine.stats.prefix_hits == hits + 1


def test_dead_peer_timeout_is_set_on_accepted_connections(server):
    import socket
    from ninfer_fusion_b200.serve import server as S
    if not hasattr(socket, "TCP_USER_TIMEOUT"):
        pytest.skip("no TCP_USER_TIMEOUT on this platform")
    port, _, _ = server
    seen = {}
    orig = S.BaseHTTPRequestHandler.finish

    def spy(self):                                    # runs on the server thread while the connection is still open
        seen["ms"] = self.connection.getsockopt(socket.IPPROTO_TCP, socket.TCP_USER_TIMEOUT)
        orig(self)
    S.BaseHTTPRequestHandler.finish = spy
    try:
        assert call(port, "GET", "/health", key=None)[0] == 200
        for _ in range(100):
            if "ms" in seen:
                break
            time.sleep(0.01)
    finally:
        S.BaseHTTPRequestHandler.finish = orig
    assert seen.get("ms") == S.DEAD_PEER_MS == 15000


def test_artifact_diff(tmp_path, capsys):
    a, b, c = (str(tmp_path / n) for n in ("a.ninfer", "b.ninfer", "c.ninfer"))
    assert cli.main(["make-artifact", "--model", "tiny-dense", "--out", a]) == 0
    assert cli.main(["make-artifact", "--model", "tiny-dense", "--out", b]) == 0
    assert cli.main(["make-artifact", "--model", "tiny-dense", "--format", "W8G32_F16S", "--out", c]) == 0
    capsys.readouterr()
    assert cli.main(["diff", a, b]) == 0                                   # same seed, same bytes
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert summary["reported"] == 0 and summary["worst_relative_diff"] == 0
    assert cli.main(["diff", a, c]) == 1                                   # quantised copy: values differ, beyond tolerance 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    changed = [l for l in lines[:-1] if l["status"] == "format_differs"]
    assert changed and all(l["formats"] == ["BF16", "W8G32_F16S"] and 0 < l["relative"] < 0.02 for l in changed)
    assert cli.main(["diff", a, c, "--tolerance", "0.02"]) == 0            # within the int8 envelope
    capsys.readouterr()


def test_prompt_cache_hints_are_validated_and_become_write_candidates():
    from ninfer_fusion_b200.serve import protocols as P
    msgs = [{"role": "system", "content": "s" * 10},
            {"role": "user", "content": [{"type": "text", "text": "doc", "prompt_cache_breakpoint": {"mode": "explicit"}}]},
            {"role": "assistant", "content": "ok"},
            {"role": "user", "content": "q", "prompt_cache_breakpoint": {"mode": "explicit"}}]
    req, _ = P.parse_openai_chat({"messages": msgs, "prompt_cache_options": {"mode": "explicit"},
                                  "prompt_cache_key": "tenant-7", "prompt_cache_retention": "24h"})
    assert req.cache_implicit is False and list(req.cache_breakpoints) == [1, 3]
    assert req.cache_key == "tenant-7" and req.cache_retention == "24h" and req.session is None   # the key is not a session
    req, _ = P.parse_openai_chat({"messages": msgs[:1] + [{"role": "user", "content": "q"}]})
    assert req.cache_implicit is True and list(req.cache_breakpoints) == []
    for bad in ({"prompt_cache_options": {"mode": "always"}}, {"prompt_cache_options": "implicit"},
                {"prompt_cache_retention": "7d"}, {"prompt_cache_key": 5}):
        with pytest.raises(P.BadRequest):
            P.parse_openai_chat(dict({"messages": msgs}, **bad))
    with pytest.raises(P.BadRequest):
        P.parse_openai_chat({"messages": [{"role": "user", "content": "q", "prompt_cache_breakpoint": {"mode": "implicit"}}]})
    # Anthropic cache_control marks the same kind of boundary
    areq, _ = P.parse_anthropic_messages({
        "max_tokens": 8, "system": [{"type": "text", "text": "be brief", "cache_control": {"type": "ephemeral"}}],
        "messages": [{"role": "user", "content": [{"type": "text", "text": "long doc", "cache_control": {"type": "ephemeral", "ttl": "1h"}}]},
                     {"role": "assistant", "content": "ok"}, {"role": "user", "content": "q"}]})
    assert list(areq.cache_breakpoints) == [0, 1]
    with pytest.raises(P.BadRequest):
        P.parse_anthropic_messages({"max_tokens": 8, "messages": [{"role": "user", "content": [
            {"type": "text", "text": "x", "cache_control": {"type": "persistent"}}]}]})


def test_explicit_breakpoints_publish_shared_prefixes_and_usage_reports_cached_tokens(server):
    port, svc, _ = server
    doc = "The quarterly report lists seventeen regional offices and their budgets. " * 6
    base = [{"role": "user", "content": [{"type": "text", "text": doc, "prompt_cache_breakpoint": {"mode": "explicit"}}]},
            {"role": "assistant", "content": "Noted."}]
    st, _, data = call(port, "POST", "/v1/chat/completions",
                       {"messages": base + [{"role": "user", "content": "How many offices?"}], "max_tokens": 2,
                        "prompt_cache_options": {"mode": "explicit"}})
    assert st == 200 and json.loads(data)["usage"]["prompt_tokens_details"]["cached_tokens"] == 0
    published = svc.engine.program.shared_stats["published"] if hasattr(svc.engine.program, "shared_stats") else None
    # another client, another question, same document: the explicit boundary after the document message is a read hit
    st, _, data = call(port, "POST", "/v1/chat/completions",
                       {"messages": base + [{"role": "user", "content": "Which office is largest?"}], "max_tokens": 2})
    usage = json.loads(data)["usage"]
    assert st == 200 and usage["prompt_tokens_details"]["cached_tokens"] >= 32 and usage["prompt_tokens"] > usage["prompt_tokens_details"]["cached_tokens"]
    assert published is None or svc.engine.program.shared_stats["hits"] >= 1


def test_server_option_table_process_settings(tmp_path):
    """The process-level settings of the server's option table: sampler defaults and forced arg-max, default output
    budget and thinking mode, prefix reuse off, CORS, body-size limit, the response store's record and byte bounds,
    catalogue capacities applied to every Program the engine builds."""
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=3, std=0.05)
    tok = Tokenizer.train_toy(cli.DEFAULT_CORPUS, 200, cli.SPECIAL_TOKENS)
    engine = Engine(lambda: ReferenceProgram(cfg, w, max_lanes=2, max_context=256), prefill_chunk=64)
    svc = GenerationService(engine, tok, "tiny-dense:test", max_concurrent=2, queue_timeout_s=20.0)
    from ninfer_fusion_b200.serve.service import GenRequest
    # sampler: registered default < process override < the request's own value; --greedy beats all
    svc.sampling_overrides = {"temperature": 0.3, "top_k": 7}
    sp = svc._options(GenRequest(prompt="x")).sampling
    assert sp.temperature == 0.3 and sp.top_k == 7
    assert svc._options(GenRequest(prompt="x", temperature=0.9)).sampling.temperature == 0.9
    svc.fixed_seed = 1234
    assert svc._options(GenRequest(prompt="x")).sampling.seed == 1234 and svc._options(GenRequest(prompt="x", seed=5)).sampling.seed == 5
    svc.force_greedy = True
    sp = svc._options(GenRequest(prompt="x", temperature=0.9)).sampling
    assert sp.temperature == 0.0 and sp.top_k == 1
    svc.prefix_reuse = False
    assert svc._options(GenRequest(prompt="x", session="s")).session is None
    # catalogue capacities survive a recover()
    import argparse
    cli.apply_retention_options(engine, argparse.Namespace(max_private_continuations=3, max_shared_prefixes=2,
                                                           max_long_anchors_per_continuation=1, host_kv_mib=1.5))
    for _ in range(2):
        p = engine.program
        assert (p.max_checkpoints, p.max_shared_prefixes, p.max_anchors, p.host_budget_bytes) == (3, 2, 1, int(1.5 * (1 << 20)))
        engine.program = engine._factory()
    httpd = serve(svc, "127.0.0.1", 0, api_key=None, log_path=None, max_stored_responses=100, max_stored_bytes=2500,
                  max_body_bytes=4096, cors=True, log_interval_s=0, default_max_tokens=2, default_thinking=False)
    t = threading.Thread(target=httpd.serve_forever, daemon=True)
    t.start()
    port = httpd.server_address[1]
    try:
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
        c.request("OPTIONS", "/v1/chat/completions", None, {"Origin": "http://localhost:3000"})
        r = c.getresponse()
        r.read()
        assert r.status == 204 and r.getheader("Access-Control-Allow-Origin") == "*"
        c.request("GET", "/health")
        r = c.getresponse()
        r.read()
        assert r.status == 200 and r.getheader("Access-Control-Allow-Origin") == "*"
        c.close()
        st, _, data = call(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}]}, key=None)
        assert st == 200 and json.loads(data)["usage"]["completion_tokens"] <= 2           # --default-max-tokens 2
        st, _, data = call(port, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x" * 5000}]}, key=None)
        assert st == 413 or (st == 400 and b"large" in data.lower())                          # --max-request-mib
        ids = []
        for i in range(4):
            st, _, data = call(port, "POST", "/v1/responses", {"input": f"question number {i} " + "pad " * 40, "max_output_tokens": 1}, key=None)
            assert st == 200
            ids.append(json.loads(data)["id"])
        state = httpd.state
        assert 1 <= len(state.responses) < 4 and state.stored_bytes <= max(2500, max(r["_bytes"] for r in state.responses.values()))
        assert call(port, "GET", f"/v1/responses/{ids[-1]}", key=None)[0] == 200 and call(port, "GET", f"/v1/responses/{ids[0]}", key=None)[0] == 404
        assert call(port, "DELETE", f"/v1/responses/{ids[-1]}", key=None)[0] == 200 and state.stored_bytes == sum(r["_bytes"] for r in state.responses.values())
    finally:
        httpd.shutdown()
        httpd.server_close()
        engine.shutdown()


def test_thinking_budget_reaches_the_engine_from_every_protocol(server):
    from ninfer_fusion_b200.serve import protocols as P
    from ninfer_fusion_b200.serve.service import GenRequest
    _, svc, _ = server
    req, _ = P.parse_anthropic_messages({"max_tokens": 64, "thinking": {"type": "enabled", "budget_tokens": 20},
                                         "messages": [{"role": "user", "content": "q"}]})
    assert req.enable_thinking and req.thinking_budget == 20
    req2, _ = P.parse_openai_chat({"messages": [{"role": "user", "content": "q"}], "thinking_budget": 9})
    assert req2.thinking_budget == 9
    for bad in ({"thinking_budget": 0}, {"thinking_budget": "many"}, {"chat_template_kwargs": {"thinking_budget": -1}}):
        with pytest.raises(P.BadRequest):
            P.parse_openai_chat(dict({"messages": [{"role": "user", "content": "q"}]}, **bad))
    with pytest.raises(P.BadRequest):
        P.parse_anthropic_messages({"max_tokens": 8, "thinking": {"type": "enabled", "budget_tokens": 0},
                                    "messages": [{"role": "user", "content": "q"}]})
    o = svc._options(req)
    close = svc.tok.token_id("</think>")
    assert o.thinking_budget == 20 and o.think_close_id == close and close in o.think_close_ids
    assert o.think_open_id == svc.tok.token_id("<think>")
    assert svc._options(GenRequest(prompt="x")).thinking_budget is None
    svc.default_thinking_budget = 50
    try:
        assert svc._options(GenRequest(prompt="x")).thinking_budget == 50
        assert svc._options(GenRequest(prompt="x", enable_thinking=False)).thinking_budget is None   # nothing to cap
    finally:
        svc.default_thinking_budget = None


def test_rag_store_chunks_indexes_and_retrieves():
    from ninfer_fusion_b200.serve import rag
    assert rag.tokenize("Hello, World_1! 東京") == ["hello", "world_1", "東", "京"]
    text = "\n\n".join(f"Paragraph {i} talks about topic{i}. " + "filler words here. " * 20 for i in range(6))
    parts = rag.chunk_text(text, 500)
    assert len(parts) >= 6 and all(len(p) <= 500 for p in parts) and "topic3" in "".join(parts)
    assert all(len(p) <= 80 for p in rag.chunk_text("x" * 300, 80))              # a sentence longer than the limit is cut
    store = rag.DocumentStore(max_documents=3, max_bytes=10_000, chunk_chars=300)
    a = store.add("fruit", "Apples are red or green. They grow on trees.\n\nBananas are yellow and grow in bunches.")
    b = store.add("metal", "Iron rusts in wet air. Copper turns green over the years.\n\nGold does not tarnish.")
    hits = store.retrieve("what colour are bananas", top_k=2)
    assert hits and hits[0][1].document == a["id"] and "Bananas" in hits[0][1].text
    assert store.retrieve("zebra quantum", 3) == [] and store.retrieve("", 3) == []
    msgs, sources = store.build_messages("Does gold tarnish?", store.retrieve("gold tarnish", 2))
    assert msgs[0]["role"] == "system" and "[1] metal" in msgs[0]["content"] and sources[0]["document"] == b["id"]
    assert store.remove(a["id"]) and not store.remove(a["id"]) and store.retrieve("bananas", 2) == []
    assert "banana" not in store.df and "bananas" not in store.df
    for i in range(4):                                                            # bounded: the oldest document goes first
        store.add(f"d{i}", f"document number {i} about widgets")
    assert len(store.list()) == 3 and b["id"] not in [d["id"] for d in store.list()]
    with pytest.raises(ValueError):
        store.add("empty", "   ")
    with pytest.raises(ValueError):
        store.add("huge", "x" * 20_000)


def test_rag_routes_answer_with_sources(server):
    port, _, _ = server
    st, _, data = call(port, "POST", "/v1/rag/documents", {"title": "handbook", "text": "The office opens at nine.\n\nLunch is at noon."})
    doc = json.loads(data)
    assert st == 200 and doc["chunks"] >= 1
    st, _, data = call(port, "GET", "/v1/rag/documents")
    assert st == 200 and doc["id"] in [d["id"] for d in json.loads(data)["data"]]
    st, _, data = call(port, "POST", "/v1/rag/query", {"query": "When does the office open?", "top_k": 2, "max_tokens": 3})
    ans = json.loads(data)
    assert st == 200 and ans["object"] == "rag.answer" and ans["sources"] and ans["sources"][0]["title"] == "handbook"
    assert ans["usage"]["completion_tokens"] <= 3 and "office" in ans["sources"][0]["text"]
    assert call(port, "POST", "/v1/rag/query", {"query": ""})[0] == 400
    assert call(port, "POST", "/v1/rag/documents", {"title": "x", "text": ""})[0] == 400
    assert call(port, "GET", "/v1/rag/documents", key=None)[0] == 401                 # the data routes need the key
    st, ctype, page = call(port, "GET", "/rag", key=None)
    assert st == 200 and "text/html" in ctype and b"/v1/rag/query" in page            # the page itself holds no data
    assert call(port, "DELETE", f"/v1/rag/documents/{doc['id']}")[0] == 200
    assert call(port, "DELETE", f"/v1/rag/documents/{doc['id']}")[0] == 404


def test_soft_limit_over_http_carries_the_notice_and_logs_it(server):
    port, _, log = server
    body = {"model": "tiny-dense:test", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "soft_max_tokens": 6,
            "temperature": 0.0}
    status, _, data = call(port, "POST", "/v1/chat/completions", body)
    out = json.loads(data)
    assert status == 200 and out["choices"][0]["finish_reason"] in ("length", "stop")
    if out["choices"][0]["finish_reason"] == "length":
        assert out["stop_boundary"]["state"] in ("stopped", "deferred") and out["stop_boundary"]["emits_tokens"] is False
    status, _, err = call(port, "POST", "/v1/chat/completions", {**body, "soft_max_tokens": 7})
    assert status == 400 and b"soft_max_tokens" in err
    with open(log, encoding="utf-8") as f:
        done = [json.loads(l) for l in f if '"request_done"' in l]
    assert "stop_boundary" in done[-1]
