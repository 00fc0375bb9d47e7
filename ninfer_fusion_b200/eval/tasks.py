"""Datasets and rule-based scorers."""
from __future__ import annotations

import json
import random
import re
from typing import Callable, Dict, Iterator, List


def load_samples(job: dict) -> List[dict]:
    """Samples of a job: inline `samples`, a JSONL `dataset` file, or the built-in needle generator."""
    if job.get("task") == "needle":
        return list(needle_samples(job))
    if "samples" in job:
        out = [dict(s) for s in job["samples"]]
    elif "dataset" in job:
        with open(job["dataset"], encoding="utf-8") as f:
            out = [json.loads(line) for line in f if line.strip()]
    else:
        raise ValueError(f"job '{job.get('name')}' has neither samples nor dataset")
    for i, s in enumerate(out):
        s.setdefault("id", str(i))
    limit = job.get("limit")
    return out[: int(limit)] if limit else out


def needle_samples(job: dict) -> Iterator[dict]:
    """Needle-in-a-haystack: a fact hidden at a given depth of filler text of a given length (in words)."""
    rng = random.Random(int(job.get("seed", 0)))
    filler = job.get("filler", "The quick brown fox jumps over the lazy dog. ")
    for length in job.get("lengths", [200, 1000]):
        for depth in job.get("depths", [0.0, 0.5, 1.0]):
            code = str(rng.randrange(100000, 999999))
            needle = f"The secret access code is {code}. "
            words = (filler * (length // max(1, len(filler.split())) + 1)).split()[:length]
            at = int(len(words) * float(depth))
            text = " ".join(words[:at]) + " " + needle + " ".join(words[at:])
            yield {"id": f"len{length}-depth{depth}", "prompt": text + "\n\nWhat is the secret access code? Answer with the number only.",
                   "answer": code}


def build_messages(job: dict, sample: dict) -> List[dict]:
    if "messages" in sample:
        return sample["messages"]
    prompt = sample.get("prompt", sample.get("question", ""))
    if job.get("task") == "multiple_choice" and "choices" in sample:
        letters = "ABCDEFGHIJ"
        prompt += "\n" + "\n".join(f"{letters[i]}. {c}" for i, c in enumerate(sample["choices"]))
        prompt += "\nAnswer with the letter of the correct choice."
    msgs = []
    if job.get("system"):
        msgs.append({"role": "system", "content": job["system"]})
    msgs.append({"role": "user", "content": prompt})
    return msgs


def _norm(s: str) -> str:
    return re.sub(r"\s+", " ", s.strip().lower())


def score_exact(text: str, sample: dict) -> float:
    return float(_norm(text) == _norm(str(sample.get("answer", ""))))


def score_contains(text: str, sample: dict) -> float:
    return float(_norm(str(sample.get("answer", ""))) in _norm(text))


def score_choice(text: str, sample: dict) -> float:
    m = re.findall(r"\b([A-J])\b", text.strip().upper())
    want = str(sample.get("answer", "")).strip().upper()
    return float(bool(m) and m[-1] == want)


def score_number(text: str, sample: dict) -> float:
    nums = re.findall(r"-?\d+(?:\.\d+)?", text.replace(",", ""))
    try:
        return float(bool(nums) and abs(float(nums[-1]) - float(sample.get("answer"))) < 1e-6)
    except (TypeError, ValueError):
        return 0.0


SCORERS: Dict[str, Callable[[str, dict], float]] = {"exact_match": score_exact, "contains": score_contains,
                                                   "multiple_choice": score_choice, "number": score_number,
                                                   "needle": score_contains}
