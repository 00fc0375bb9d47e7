"""Serving load generator: C concurrent streaming chat requests against an OpenAI-compatible endpoint.

Measures, per request, time to first token, completion tokens and total time; reports p50 / p90 TTFT, aggregate
output tokens per second and per-request decode speed.  Counterpart of the reference's `tools/bench/
run_serve_concurrency.py` and `run_serve_corpus.py` (prompts from a text corpus, fixed concurrency levels).

    python -m ninfer_fusion_b200.serve.loadgen --base-url http://127.0.0.1:8080/v1 --model m --concurrency 1,2,4,8 \
        --requests 16 --max-tokens 128 [--corpus prompts.txt] [--api-key K]

First-token campaign (the reference's TTFT campaign): `--ttft-lengths 256,2048,16384 [--ttft-repeats 3]` sends, per
length, prompts of about that many tokens with one output token, each with a unique head (so no cached frontier can
serve it: the cold first-token time and the prefill rate it implies), then one of them again (the warm first-token
time and how many prompt tokens the server reports as cached).
"""
from __future__ import annotations

import argparse
import http.client
import json
import statistics
import sys
import threading
import time
from typing import List, Optional
from urllib.parse import urlparse

DEFAULT_PROMPTS = ["Explain how a paged key-value cache works.", "Write a haiku about memory bandwidth.",
                   "What is speculative decoding?", "Summarise the delta rule in two sentences."]


def one_request(base_url: str, model: str, prompt: str, max_tokens: int, api_key: str = "", timeout: float = 600.0,
                temperature: float = 0.0, user: str = "") -> dict:
    u = urlparse(base_url)
    cls = http.client.HTTPSConnection if u.scheme == "https" else http.client.HTTPConnection
    c = cls(u.hostname, u.port or (443 if u.scheme == "https" else 80), timeout=timeout)
    body = {"model": model, "messages": [{"role": "user", "content": prompt}], "max_tokens": max_tokens, "stream": True,
            "temperature": temperature, "stream_options": {"include_usage": True}}
    if user:
        body["user"] = user          # the server's continuation key: a repeated request may start from a kept frontier
    headers = {"Content-Type": "application/json", "Accept": "text/event-stream"}
    if api_key:
        headers["Authorization"] = f"Bearer {api_key}"
    t0 = time.perf_counter()
    rec = {"ok": False, "ttft_s": None, "total_s": 0.0, "completion_tokens": 0, "chunks": 0, "error": ""}
    try:
        c.request("POST", u.path.rstrip("/") + "/chat/completions", json.dumps(body), headers)
        r = c.getresponse()
        if r.status != 200:
            rec["error"] = f"HTTP {r.status}"
            r.read()
            return rec
        while True:
            line = r.readline()
            if not line:
                break
            line = line.strip()
            if not line.startswith(b"data: "):
                continue
            payload = line[6:]
            if payload == b"[DONE]":
                break
            ev = json.loads(payload)
            ch = ev.get("choices") or []
            if ch and (ch[0].get("delta", {}).get("content") or ch[0].get("delta", {}).get("reasoning_content")):
                rec["chunks"] += 1
                if rec["ttft_s"] is None:
                    rec["ttft_s"] = time.perf_counter() - t0
            if ev.get("usage"):
                rec["completion_tokens"] = int(ev["usage"].get("completion_tokens", 0))
                rec["prompt_tokens"] = int(ev["usage"].get("prompt_tokens", 0))
                rec["cached_tokens"] = int((ev["usage"].get("prompt_tokens_details") or {}).get("cached_tokens", 0))
        rec["ok"] = True
    except (OSError, http.client.HTTPException, json.JSONDecodeError) as e:
        rec["error"] = f"{type(e).__name__}: {e}"
    finally:
        rec["total_s"] = time.perf_counter() - t0
        c.close()
    if rec["completion_tokens"] == 0:
        rec["completion_tokens"] = rec["chunks"]
    return rec


def run_level(base_url: str, model: str, prompts: List[str], concurrency: int, n_requests: int, max_tokens: int,
              api_key: str = "") -> dict:
    results: List[dict] = []
    lock = threading.Lock()
    nxt = [0]

    def worker():
        while True:
            with lock:
                i = nxt[0]
                if i >= n_requests:
                    return
                nxt[0] += 1
            r = one_request(base_url, model, prompts[i % len(prompts)], max_tokens, api_key)
            with lock:
                results.append(r)

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker) for _ in range(concurrency)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    ok = [r for r in results if r["ok"]]
    ttft = sorted(r["ttft_s"] for r in ok if r["ttft_s"] is not None)
    toks = sum(r["completion_tokens"] for r in ok)

    def pct(v, q):
        return round(v[min(len(v) - 1, int(q * len(v)))] * 1e3, 2) if v else None

    dec = [(r["completion_tokens"] - 1) / (r["total_s"] - r["ttft_s"]) for r in ok
           if r["ttft_s"] is not None and r["completion_tokens"] > 1 and r["total_s"] > r["ttft_s"]]
    return {"concurrency": concurrency, "requests": len(results), "ok": len(ok), "errors": len(results) - len(ok),
            "wall_s": round(wall, 3), "output_tokens": toks, "output_tok_s": round(toks / wall, 2) if wall > 0 else 0.0,
            "ttft_ms_p50": pct(ttft, 0.5), "ttft_ms_p90": pct(ttft, 0.9),
            "decode_tok_s_per_request_median": round(statistics.median(dec), 2) if dec else None}


FILLER = ("The scheduler admits requests in arrival order and gives each one a lane, a page reservation and a slot for its "
          "recurrent state; prefill runs in units, decode in rounds, and the two alternate while both kinds are runnable. ")


def sized_prompt(target_tokens: int, tag: str, tokens_per_filler: float) -> str:
    """A prompt of about `target_tokens` tokens whose first characters are unique to `tag`."""
    n = max(1, int(round(target_tokens / max(tokens_per_filler, 1e-6))))
    return f"[{tag}] " + FILLER * n + "Reply with one word."


def ttft_campaign(base_url: str, model: str, lengths: List[int], repeats: int = 3, api_key: str = "") -> List[dict]:
    """One record per prompt length: cold and warm first-token time, the prefill rate the cold one implies."""
    probe = one_request(base_url, model, sized_prompt(0, "probe", 1.0).replace(FILLER, FILLER * 2, 1), 1, api_key)
    base = one_request(base_url, model, sized_prompt(0, "probe", 1.0), 1, api_key)
    if not (probe["ok"] and base["ok"] and probe.get("prompt_tokens", 0) > base.get("prompt_tokens", 0)):
        raise RuntimeError(f"calibration requests failed: {probe.get('error') or base.get('error') or 'no usage block in the stream'}")
    per_filler = float(probe["prompt_tokens"] - base["prompt_tokens"])       # tokens one FILLER adds under this tokenizer
    out = []
    for n in lengths:
        cold, last_prompt = [], ""
        user = ""
        for r in range(repeats):
            user = f"ttft-{n}-{r}-{time.time_ns():x}"
            last_prompt = sized_prompt(n, user, per_filler)
            cold.append(one_request(base_url, model, last_prompt, 1, api_key, user=user))
        warm = one_request(base_url, model, last_prompt, 1, api_key, user=user)   # a regeneration: served from the replay frontier
        for c in cold + [warm]:
            if c["ok"] and c["ttft_s"] is None:
                c["ttft_s"] = c["total_s"]      # one token that decodes to no text: the stream's end is the first token
        ok = [c for c in cold if c["ok"]]
        ttft = sorted(c["ttft_s"] for c in ok)
        p50 = ttft[len(ttft) // 2] if ttft else None
        toks = ok[0].get("prompt_tokens", 0) if ok else 0
        out.append({"target_tokens": n, "prompt_tokens": toks, "ok": len(ok), "errors": len(cold) - len(ok),
                    "ttft_cold_ms_p50": round(p50 * 1e3, 2) if p50 else None,
                    "prefill_tok_s": round(toks / p50, 1) if p50 and toks else None,
                    "ttft_warm_ms": round(warm["ttft_s"] * 1e3, 2) if warm.get("ttft_s") else None,
                    "warm_cached_tokens": warm.get("cached_tokens", 0),
                    "cold_cached_tokens_max": max([c.get("cached_tokens", 0) for c in ok], default=0)})
    return out


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="ninfer_fusion_b200.serve.loadgen")
    ap.add_argument("--base-url", required=True)
    ap.add_argument("--model", default="")
    ap.add_argument("--api-key", default="")
    ap.add_argument("--concurrency", default="1,2,4,8")
    ap.add_argument("--requests", type=int, default=16, help="requests per concurrency level")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--corpus", help="text file, one prompt per line")
    ap.add_argument("--ttft-lengths", default="", help="comma-separated prompt lengths in tokens: run the first-token campaign instead")
    ap.add_argument("--ttft-repeats", type=int, default=3)
    a = ap.parse_args(argv)
    if a.ttft_lengths:
        for rec in ttft_campaign(a.base_url, a.model, [int(v) for v in a.ttft_lengths.split(",")], a.ttft_repeats, a.api_key):
            print(json.dumps(rec), flush=True)
        return 0
    prompts = DEFAULT_PROMPTS
    if a.corpus:
        with open(a.corpus, encoding="utf-8") as f:
            prompts = [l.strip() for l in f if l.strip()] or DEFAULT_PROMPTS
    for c in [int(v) for v in a.concurrency.split(",")]:
        print(json.dumps(run_level(a.base_url, a.model, prompts, c, a.requests, a.max_tokens, a.api_key)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
