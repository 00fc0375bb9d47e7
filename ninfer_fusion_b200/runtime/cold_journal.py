"""A persistent journal of the disk tier: which file holds which frontier, so that cold copies survive a restart.

The disk tier (`ProgramBase._trim_cold`) writes one file per frontier that is pushed out of pinned host memory.  The
map frontier -> file used to live in memory only: after a restart the files were orphans and every session started
from token zero.  The journal is that map on disk.

* **Append only.**  A record is written when a frontier goes to disk (`spill`) and when its file is given up
  (`release`: promoted back to the device, dropped for budget, or found damaged).  The live set is what replaying the
  file leaves.
* **Framed and checked.**  `magic | payload length | crc32(payload) | payload`.  A crash can only tear the LAST
  record; a reader stops at the first frame that is short, has the wrong magic or fails its checksum, reports how many
  bytes it ignored, and the next writer truncates the file there.
* **A mirror, never the only replica.**  Losing the last record costs a re-prefill, never correctness, which is why
  the default flush policy does not fsync.
* **A digest is a shortlist, not an identity.**  A record carries the exact token ids (and their digest for quick
  look-ups); a frontier adopted from the journal is reusable only for a prompt that starts with exactly those tokens,
  which is the comparison the Program makes for every frontier.  The journal is bound to one `fingerprint` (program
  class, model geometry, KV storage, weights identity): a journal of anything else is refused as a whole.
* **A hole is a refusal.**  A record whose file is missing or has another size is not adopted and is released.

Reading back is not always a win: `RecallCost` compares reading `nbytes` at the disk's rate with prefilling the same
tokens again.  On a GPU that prefills tens of thousands of tokens per second the margin over an NVMe read is a small
factor, not orders of magnitude, so the comparison is made per frontier with the rates the caller measured.

Reference: src/spec/turn_recall_journal.h (persistent page -> file-slot log with checksummed records, mirror-not-tier,
digest-as-shortlist, hole = refusal, read vs re-prefill cost verdict), src/product/cold_spill_writeback.h.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
import zlib
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

MAGIC = 0x314A4C43            # "CLJ1"
_FRAME = struct.Struct("<III")  # magic, payload bytes, crc32 of the payload
MAX_PAYLOAD = 64 << 20
FLUSH_POLICIES = ("none", "flush", "fsync")


def token_digest(tokens: Sequence[int]) -> str:
    """128-bit content digest of a token history (a shortlist key; equality of tokens stays authoritative)."""
    h = hashlib.blake2b(digest_size=16)
    h.update(struct.pack(f"<{len(tokens)}i", *[int(t) for t in tokens]))
    return h.hexdigest()


@dataclass
class LoadReport:
    records: int = 0
    live: int = 0
    released: int = 0
    ignored_tail_bytes: int = 0
    refused: str = ""            # the whole journal was refused (other fingerprint / not a journal)
    valid_bytes: int = 0


@dataclass
class SpillRecord:
    file: str                    # file name inside the cold directory
    nbytes: int                  # size of the frontier's cold copy as the Program accounts it
    file_bytes: int              # size of the file on disk (what adoption checks)
    session: str
    kind: str
    tokens: List[int]
    digest: str = ""

    def to_payload(self) -> Dict:
        return {"op": "spill", "file": self.file, "nbytes": self.nbytes, "file_bytes": self.file_bytes,
                "session": self.session, "kind": self.kind, "tokens": self.tokens, "digest": self.digest or token_digest(self.tokens)}


def _frame(payload: Dict) -> bytes:
    body = json.dumps(payload, separators=(",", ":")).encode()
    return _FRAME.pack(MAGIC, len(body), zlib.crc32(body) & 0xFFFFFFFF) + body


def read_frames(path: str) -> Tuple[List[Dict], int, int]:
    """(payloads, bytes of valid frames, bytes ignored after them).  Never raises on a damaged file."""
    out: List[Dict] = []
    try:
        data = open(path, "rb").read()
    except OSError:
        return out, 0, 0
    pos = 0
    while pos + _FRAME.size <= len(data):
        magic, n, crc = _FRAME.unpack_from(data, pos)
        end = pos + _FRAME.size + n
        if magic != MAGIC or n > MAX_PAYLOAD or end > len(data):
            break
        body = data[pos + _FRAME.size:end]
        if zlib.crc32(body) & 0xFFFFFFFF != crc:
            break
        try:
            payload = json.loads(body)
        except ValueError:
            break
        if not isinstance(payload, dict):
            break
        out.append(payload)
        pos = end
    return out, pos, len(data) - pos


class ColdJournal:
    FILE = "journal.clj"

    def __init__(self, directory: str, fingerprint: str, flush: str = "none"):
        if flush not in FLUSH_POLICIES:
            raise ValueError(f"flush policy must be one of {FLUSH_POLICIES}")
        self.directory, self.fingerprint, self.flush = directory, fingerprint, flush
        self.path = os.path.join(directory, self.FILE)
        self.live: Dict[str, SpillRecord] = {}
        self.report = LoadReport()
        self.write_failures = 0
        self._fh = None
        self._load()

    # ------------------------------------------------------------------ load
    def _load(self) -> None:
        rep = self.report
        frames, valid, ignored = read_frames(self.path)
        rep.valid_bytes, rep.ignored_tail_bytes = valid, ignored
        if frames:
            head = frames[0]
            if head.get("op") != "open" or head.get("fingerprint") != self.fingerprint:
                rep.refused = "journal belongs to another program, model, KV storage or set of weights"
                return
        for p in frames[1:]:
            rep.records += 1
            if p.get("op") == "spill":
                try:
                    r = SpillRecord(str(p["file"]), int(p["nbytes"]), int(p["file_bytes"]), str(p["session"]), str(p["kind"]),
                                    [int(t) for t in p["tokens"]], str(p.get("digest", "")))
                except (KeyError, TypeError, ValueError):
                    continue
                if os.path.basename(r.file) != r.file:       # a record never points outside the cold directory
                    continue
                self.live[r.file] = r
            elif p.get("op") == "release":
                if self.live.pop(str(p.get("file")), None) is not None:
                    rep.released += 1
        rep.live = len(self.live)

    # ------------------------------------------------------------------ append
    def _writer(self):
        if self._fh is None:
            os.makedirs(self.directory, exist_ok=True)
            fresh = self.report.refused or self.report.valid_bytes == 0
            if fresh:
                # a refused journal is replaced: its files belong to another model and can never be adopted here
                self._fh = open(self.path, "wb")
                self._fh.write(_frame({"op": "open", "fingerprint": self.fingerprint}))
                self.live.clear()
            else:
                self._fh = open(self.path, "r+b")
                self._fh.truncate(self.report.valid_bytes)   # drop a torn tail before appending after it
                self._fh.seek(self.report.valid_bytes)
        return self._fh

    def _append(self, payload: Dict) -> bool:
        try:
            fh = self._writer()
            fh.write(_frame(payload))
            if self.flush != "none":
                fh.flush()
            if self.flush == "fsync":
                os.fsync(fh.fileno())
            return True
        except OSError:
            self.write_failures += 1     # the journal is a mirror: a write that fails costs a future re-prefill only
            return False

    def spill(self, rec: SpillRecord) -> bool:
        rec.digest = rec.digest or token_digest(rec.tokens)
        ok = self._append(rec.to_payload())      # first: opening the writer over a refused journal empties the live set
        self.live[rec.file] = rec
        return ok

    def release(self, file: str, reason: str = "") -> bool:
        if self.live.pop(file, None) is None:
            return False
        return self._append({"op": "release", "file": file, "reason": reason})

    def close(self) -> None:
        if self._fh is not None:
            try:
                self._fh.flush()
                self._fh.close()
            except OSError:
                pass
            self._fh = None
            # a later append re-opens the file: it continues after what was written, it does not start over
            try:
                self.report.valid_bytes, self.report.refused, self.report.ignored_tail_bytes = os.path.getsize(self.path), "", 0
            except OSError:
                self.report.valid_bytes = 0

    # ------------------------------------------------------------------ adoption
    def adoptable(self) -> Tuple[List[SpillRecord], List[Tuple[str, str]]]:
        """Live records whose file is there with the recorded size and whose tokens match their digest; the others
        come back as (file, why) and are released."""
        good: List[SpillRecord] = []
        holes: List[Tuple[str, str]] = []
        for name, r in list(self.live.items()):
            path = os.path.join(self.directory, name)
            try:
                size = os.path.getsize(path)
            except OSError:
                holes.append((name, "file missing"))
                continue
            if size != r.file_bytes:
                holes.append((name, f"file has {size} bytes, the record says {r.file_bytes}"))
            elif r.digest and token_digest(r.tokens) != r.digest:
                holes.append((name, "token history does not match its digest"))
            elif not r.tokens:
                holes.append((name, "empty token history"))
            else:
                good.append(r)
        for name, why in holes:
            self.release(name, why)
        return good, holes

    def orphans(self) -> List[str]:
        """Cold files in the directory that no live record names (left by a crash between write and record)."""
        try:
            names = os.listdir(self.directory)
        except OSError:
            return []
        return sorted(n for n in names if n.startswith("ckpt_") and n not in self.live)

    def compact(self) -> int:
        """Rewrites the journal as `open` + the live records; returns the bytes saved."""
        self.close()
        before = os.path.getsize(self.path) if os.path.exists(self.path) else 0
        tmp = self.path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(_frame({"op": "open", "fingerprint": self.fingerprint}))
            for r in self.live.values():
                f.write(_frame(r.to_payload()))
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, self.path)
        after = os.path.getsize(self.path)
        self.report = LoadReport(records=len(self.live), live=len(self.live), valid_bytes=after)
        return before - after


@dataclass
class RecallCost:
    """Read the cold copy or prefill the tokens again?  Rates are the caller's measurements."""
    read_gbs: float = 3.0                # sequential read of the cold directory's device
    prefill_tok_s: float = 30000.0       # the program's prefill rate at this prompt length
    decode_overhead_ms: float = 1.0      # decoding the entropy stage / staging copy, per frontier
    margin: float = 1.25                 # reading must beat prefilling by this factor to be chosen
    decisions: Dict[str, int] = field(default_factory=lambda: {"read": 0, "prefill": 0})

    def read_ms(self, nbytes: int) -> float:
        return nbytes / (self.read_gbs * 1e9) * 1e3 + self.decode_overhead_ms

    def prefill_ms(self, n_tokens: int) -> float:
        return n_tokens / self.prefill_tok_s * 1e3

    def worthwhile(self, nbytes: int, n_tokens: int) -> bool:
        ok = self.read_ms(nbytes) * self.margin <= self.prefill_ms(n_tokens)
        self.decisions["read" if ok else "prefill"] += 1
        return ok

    def line(self, nbytes: int, n_tokens: int) -> str:
        r, p = self.read_ms(nbytes), self.prefill_ms(n_tokens)
        return (f"recall {n_tokens} tokens / {nbytes} bytes: read {r:.2f} ms vs prefill {p:.2f} ms -> "
                f"{'read' if r * self.margin <= p else 'prefill'} ({p / max(r, 1e-9):.1f}x)")
