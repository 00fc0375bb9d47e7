"""Runs the jobs of a suite against their targets: bounded concurrency per target, JSONL events, resume, summary."""
from __future__ import annotations

import json
import os
import threading
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from typing import Dict, List, Optional

from .backends import TargetError, make_target
from .tasks import SCORERS, build_messages, load_samples


def load_config(path: str) -> dict:
    import yaml
    with open(path, encoding="utf-8") as f:
        cfg = yaml.safe_load(f)
    if not isinstance(cfg, dict) or "targets" not in cfg or "jobs" not in cfg:
        raise ValueError("an evaluation suite needs `targets` and `jobs`")
    for j in cfg["jobs"]:
        if j.get("target") not in cfg["targets"]:
            raise ValueError(f"job '{j.get('name')}' names an unknown target '{j.get('target')}'")
        scorer = j.get("scorer", j.get("task", "exact_match"))
        if scorer not in SCORERS:
            raise ValueError(f"job '{j.get('name')}': unknown scorer '{scorer}'")
    return cfg


class Coordinator:
    def __init__(self, cfg: dict, out_dir: str, events: Optional[callable] = None):
        self.cfg, self.out_dir = cfg, out_dir
        os.makedirs(out_dir, exist_ok=True)
        self._lock = threading.Lock()
        self._events_path = os.path.join(out_dir, "events.jsonl")
        self._listener = events

    def _emit(self, kind: str, **kw) -> None:
        rec = {"ts": round(time.time(), 3), "event": kind, **kw}
        with self._lock:
            with open(self._events_path, "a", encoding="utf-8") as f:
                f.write(json.dumps(rec) + "\n")
        if self._listener:
            self._listener(rec)

    def _done_ids(self, path: str) -> Dict[str, dict]:
        done: Dict[str, dict] = {}
        if os.path.exists(path):
            with open(path, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        r = json.loads(line)
                        if not r.get("error"):
                            done[r["id"]] = r
        return done

    def run_job(self, job: dict) -> dict:
        name = job["name"]
        target = make_target(self.cfg["targets"][job["target"]])
        scorer = SCORERS[job.get("scorer", job.get("task", "exact_match"))]
        samples = load_samples(job)
        res_path = os.path.join(self.out_dir, f"{name}.samples.jsonl")
        done = self._done_ids(res_path) if job.get("resume", True) else {}
        todo = [s for s in samples if s["id"] not in done]
        params = dict(job.get("generation", {}))
        conc = max(1, min(int(job.get("concurrency", target.max_concurrency)), target.max_concurrency))
        self._emit("job_start", job=name, samples=len(samples), resumed=len(done), concurrency=conc)
        t0 = time.perf_counter()
        records: List[dict] = list(done.values())

        def one(sample: dict) -> dict:
            t = time.perf_counter()
            try:
                out = target.complete(build_messages(job, sample), params, sample)
                rec = {"id": sample["id"], "score": scorer(out["text"], sample), "text": out["text"],
                       "prompt_tokens": out.get("prompt_tokens", 0), "completion_tokens": out.get("completion_tokens", 0),
                       "seconds": round(time.perf_counter() - t, 4)}
            except TargetError as e:
                rec = {"id": sample["id"], "score": 0.0, "error": str(e), "seconds": round(time.perf_counter() - t, 4)}
            with self._lock:
                with open(res_path, "a", encoding="utf-8") as f:
                    f.write(json.dumps(rec) + "\n")
            self._emit("sample_done", job=name, id=sample["id"], score=rec["score"], error=rec.get("error", ""))
            return rec

        with ThreadPoolExecutor(max_workers=conc) as pool:
            for fut in as_completed([pool.submit(one, s) for s in todo]):
                records.append(fut.result())
        n = len(records)
        errors = sum(1 for r in records if r.get("error"))
        summary = {"job": name, "target": job["target"], "samples": n, "errors": errors,
                   "score": round(sum(r["score"] for r in records) / max(1, n), 6),
                   "completion_tokens": sum(r.get("completion_tokens", 0) for r in records),
                   "seconds": round(time.perf_counter() - t0, 3)}
        self._emit("job_done", **summary)
        return summary

    def run(self) -> dict:
        self._emit("suite_start", jobs=[j["name"] for j in self.cfg["jobs"]])
        out = {"jobs": [self.run_job(j) for j in self.cfg["jobs"]]}
        with open(os.path.join(self.out_dir, "summary.json"), "w", encoding="utf-8") as f:
            json.dump(out, f, indent=1)
        self._emit("suite_done", jobs=len(out["jobs"]))
        return out


def run_suite(config_path: str, out_dir: str) -> dict:
    return Coordinator(load_config(config_path), out_dir).run()
