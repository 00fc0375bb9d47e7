"""Serving load generator: C concurrent streaming chat requests against an OpenAI-compatible endpoint.

Measures, per request, time to first token, completion tokens and total time; reports p50 / p90 TTFT, aggregate
output tokens per second and per-request decode speed.  Counterpart of the reference's `tools/bench/
run_serve_concurrency.py` and `run_serve_corpus.py` (prompts from a text corpus, fixed concurrency levels).

    python -m ninfer_fusion_b200.serve.loadgen --base-url http://127.0.0.1:8080/v1 --model m --concurrency 1,2,4,8 \
        --requests 16 --max-tokens 128 [--corpus prompts.txt] [--api-key K]
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
                temperature: float = 0.0) -> dict:
    u = urlparse(base_url)
    cls = http.client.HTTPSConnection if u.scheme == "https" else http.client.HTTPConnection
    c = cls(u.hostname, u.port or (443 if u.scheme == "https" else 80), timeout=timeout)
    body = {"model": model, "messages": [{"role": "user", "content": prompt}], "max_tokens": max_tokens, "stream": True,
            "temperature": temperature, "stream_options": {"include_usage": True}}
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


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="ninfer_fusion_b200.serve.loadgen")
    ap.add_argument("--base-url", required=True)
    ap.add_argument("--model", default="")
    ap.add_argument("--api-key", default="")
    ap.add_argument("--concurrency", default="1,2,4,8")
    ap.add_argument("--requests", type=int, default=16, help="requests per concurrency level")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--corpus", help="text file, one prompt per line")
    a = ap.parse_args(argv)
    prompts = DEFAULT_PROMPTS
    if a.corpus:
        with open(a.corpus, encoding="utf-8") as f:
            prompts = [l.strip() for l in f if l.strip()] or DEFAULT_PROMPTS
    for c in [int(v) for v in a.concurrency.split(",")]:
        print(json.dumps(run_level(a.base_url, a.model, prompts, c, a.requests, a.max_tokens, a.api_key)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
