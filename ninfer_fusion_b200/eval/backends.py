"""Model targets of the evaluation coordinator."""
from __future__ import annotations

import hashlib
import http.client
import json
import os
import time
from typing import Dict, List, Optional
from urllib.parse import urlparse


class TargetError(Exception):
    pass


class MockTarget:
    """Deterministic stand-in: answers with the sample's reference for a configurable fraction of the samples (chosen by
    a hash of the prompt), so that coordinator, scoring and resume logic can be exercised without a model."""

    def __init__(self, spec: dict):
        self.accuracy = float(spec.get("accuracy", 1.0))
        self.latency_s = float(spec.get("latency_seconds", 0.0))
        self.max_concurrency = int(spec.get("max_concurrency", 4))

    def complete(self, messages: List[dict], params: dict, sample: dict) -> dict:
        if self.latency_s:
            time.sleep(self.latency_s)
        h = int(hashlib.sha256(json.dumps(messages, sort_keys=True).encode()).hexdigest()[:8], 16) / 0xFFFFFFFF
        text = str(sample.get("answer", "")) if h < self.accuracy else "I do not know."
        return {"text": text, "prompt_tokens": sum(len(str(m.get("content", "")).split()) for m in messages),
                "completion_tokens": len(text.split())}


class OpenAIChatTarget:
    """POST {base_url}/chat/completions (non-streaming) with retries."""

    def __init__(self, spec: dict):
        u = urlparse(spec["base_url"])
        if u.scheme not in ("http", "https"):
            raise TargetError(f"unsupported base_url {spec['base_url']}")
        self.scheme, self.host, self.port = u.scheme, u.hostname, u.port or (443 if u.scheme == "https" else 80)
        self.path = u.path.rstrip("/") + "/chat/completions"
        self.model = spec.get("model", "")
        env = spec.get("api_key_env")
        self.api_key = os.environ.get(env, "") if env else spec.get("api_key", "")
        req = spec.get("request", {})
        self.timeout = float(req.get("timeout_seconds", 600))
        self.retries = int(req.get("retries", 1))
        self.max_concurrency = int(spec.get("max_concurrency", 1))

    def complete(self, messages: List[dict], params: dict, sample: dict) -> dict:
        body = {"model": self.model, "messages": messages, "stream": False}
        body.update({k: v for k, v in params.items() if v is not None})
        headers = {"Content-Type": "application/json"}
        if self.api_key:
            headers["Authorization"] = f"Bearer {self.api_key}"
        last = ""
        for attempt in range(self.retries + 1):
            try:
                cls = http.client.HTTPSConnection if self.scheme == "https" else http.client.HTTPConnection
                c = cls(self.host, self.port, timeout=self.timeout)
                c.request("POST", self.path, json.dumps(body), headers)
                r = c.getresponse()
                data = r.read()
                c.close()
                if r.status == 200:
                    out = json.loads(data)
                    msg = out["choices"][0]["message"]
                    usage = out.get("usage", {})
                    return {"text": msg.get("content") or "", "reasoning": msg.get("reasoning_content") or "",
                            "prompt_tokens": usage.get("prompt_tokens", 0),
                            "completion_tokens": usage.get("completion_tokens", 0),
                            "finish_reason": out["choices"][0].get("finish_reason", "")}
                last = f"HTTP {r.status}: {data[:200]!r}"
                if r.status not in (429, 500, 502, 503, 504):
                    break
            except (OSError, http.client.HTTPException, json.JSONDecodeError, KeyError) as e:
                last = f"{type(e).__name__}: {e}"
            time.sleep(min(2.0 ** attempt, 10.0) * 0.1)
        raise TargetError(last)


def make_target(spec: dict):
    proto = spec.get("protocol", "mock")
    if proto == "mock":
        return MockTarget(spec)
    if proto == "openai_chat":
        return OpenAIChatTarget(spec)
    if proto == "evalscope":
        try:
            import evalscope  # noqa: F401
        except ImportError as e:
            raise TargetError("the evalscope backend needs the evalscope package, which is not installed here") from e
        raise TargetError("evalscope backend: hand the suite to evalscope's own runner with this target's base_url")
    raise TargetError(f"unknown target protocol '{proto}'")
