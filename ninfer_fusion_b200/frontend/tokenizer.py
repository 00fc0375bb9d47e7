"""Byte-level BPE tokenizer reading the `tokenizer.json` resource embedded in an artifact.

Pipeline (the Qwen / GPT-2 family): split out added (special) tokens by longest literal match -> Unicode
regex pre-tokeniser -> bytes mapped onto the printable byte alphabet -> BPE merges by rank -> ids.  The merge
loop runs in native code (csrc/text/bpe.cpp, reached through ctypes) with a pure-Python twin that is used
when the library is not built and as the test oracle.  Every token id also carries a *frame class* so that the
output session can recognise control frames without string compares.

Reference: src/targets/qwen3_6/impl/frontend/tokenizer.cpp (BPE with added tokens and the frame-class
column), docs/maintainer/qwen3.8-27b-artifact.md:181-190 (embedded frontend resources).
"""
from __future__ import annotations

import ctypes
import json
import os
import unicodedata
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

try:  # `regex` understands \\p{L} / \\p{N}; the stdlib module does not
    import regex as _re
except ImportError:  # pragma: no cover
    import re as _re

# Pre-tokeniser of the Qwen2/3 family (tokenizer.json -> pre_tokenizer.pretokenizers[0].pattern.Regex).
QWEN_SPLIT = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*"
              r"|\s*[\r\n]+|\s+(?!\S)|\s+")

FRAME_TEXT, FRAME_CONTROL, FRAME_THINK, FRAME_TOOL = 0, 1, 2, 3
_THINK = ("<think>", "</think>")
_TOOL = ("<tool_call>", "</tool_call>", "<tool_response>", "</tool_response>")


def bytes_to_unicode() -> Dict[int, str]:
    """The reversible byte -> printable character table of byte-level BPE."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


_B2U = bytes_to_unicode()
_U2B = {c: b for b, c in _B2U.items()}


def _load_native():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")
    if not os.path.exists(path):
        return None
    try:
        lib = ctypes.CDLL(path)
        lib.nfb200_bpe_create.restype = ctypes.c_void_p
        lib.nfb200_bpe_create.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32]
        lib.nfb200_bpe_destroy.argtypes = [ctypes.c_void_p]
        lib.nfb200_bpe_encode.restype = ctypes.c_int32
        lib.nfb200_bpe_encode.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
        return lib
    except (OSError, AttributeError):
        return None


# where a prompt token came from (see Tokenizer.encode_framed)
ORIGIN_TEMPLATE, ORIGIN_LITERAL, ORIGIN_MIXED = 0, 1, 2


class Tokenizer:
    def __init__(self, vocab: Dict[str, int], merges: Sequence[Tuple[str, str]], added_tokens: Sequence[dict] = (),
                 split_pattern: str = QWEN_SPLIT, use_native: bool = True, normalizer: str = ""):
        if normalizer not in ("", "NFC", "NFKC", "NFD", "NFKD"):
            raise ValueError(f"unsupported normalizer '{normalizer}'")
        # Unicode normal form applied to ordinary text before it is split (added tokens pass through untouched);
        # the Qwen tokenizer declares NFC, so that 'e' + combining acute and the precomposed letter give the same ids
        self.normalizer = normalizer
        self.vocab = dict(vocab)
        self.added: Dict[str, int] = {}
        self.special_ids = set()
        for t in added_tokens:
            self.added[t["content"]] = int(t["id"])
            if t.get("special", False):
                self.special_ids.add(int(t["id"]))
        size = max(list(self.vocab.values()) + list(self.added.values()) + [-1]) + 1
        self.id_to_bytes: List[bytes] = [b""] * size
        for s, i in self.vocab.items():
            self.id_to_bytes[i] = bytes(_U2B[c] for c in s) if all(c in _U2B for c in s) else s.encode("utf-8")
        for s, i in self.added.items():
            self.id_to_bytes[i] = s.encode("utf-8")
        self.byte_ids = [self.vocab.get(_B2U[b], -1) for b in range(256)]
        self.ranks: Dict[Tuple[int, int], Tuple[int, int]] = {}
        left, right, merged = [], [], []
        for rank, (a, b) in enumerate(merges):
            ia, ib, im = self.vocab.get(a), self.vocab.get(b), self.vocab.get(a + b)
            if ia is None or ib is None or im is None:
                continue
            if (ia, ib) not in self.ranks:
                self.ranks[(ia, ib)] = (len(left), im)
                left.append(ia); right.append(ib); merged.append(im)
        self._split = _re.compile(split_pattern)
        self._added_re = None
        if self.added:
            alts = sorted(self.added, key=len, reverse=True)
            self._added_re = _re.compile("(" + "|".join(_re.escape(a) for a in alts) + ")")
        self.frame_class = [FRAME_TEXT] * size
        for s, i in self.added.items():
            self.frame_class[i] = FRAME_THINK if s in _THINK else FRAME_TOOL if s in _TOOL else \
                (FRAME_CONTROL if i in self.special_ids else FRAME_TEXT)
        self._cache: Dict[str, List[int]] = {}
        self._lib = _load_native() if use_native else None
        self._handle = None
        if self._lib is not None and left:
            arr = ctypes.c_int32 * len(left)
            self._handle = self._lib.nfb200_bpe_create(arr(*left), arr(*right), arr(*merged), len(left))

    def __del__(self):
        if getattr(self, "_handle", None) and self._lib is not None:
            self._lib.nfb200_bpe_destroy(self._handle)
            self._handle = None

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_json(cls, text: str | bytes, **kw) -> "Tokenizer":
        cfg = json.loads(text)
        model = cfg["model"]
        if model.get("type", "BPE") != "BPE":
            raise ValueError(f"unsupported tokenizer model '{model.get('type')}'")
        merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else (m[0], m[1]) for m in model.get("merges", [])]
        pattern = QWEN_SPLIT
        pre = cfg.get("pre_tokenizer") or {}
        for p in ([pre] if pre.get("type") != "Sequence" else pre.get("pretokenizers", [])):
            if p.get("type") == "Split" and isinstance(p.get("pattern"), dict) and "Regex" in p["pattern"]:
                pattern = p["pattern"]["Regex"]
        norm = cfg.get("normalizer") or {}
        forms = [n.get("type", "") for n in ([norm] if norm.get("type") != "Sequence" else norm.get("normalizers", []))]
        form = next((f for f in forms if f in ("NFC", "NFKC", "NFD", "NFKD")), "")
        kw.setdefault("normalizer", form)
        return cls(model["vocab"], merges, cfg.get("added_tokens", []), split_pattern=pattern, **kw)

    @classmethod
    def from_file(cls, path: str, **kw) -> "Tokenizer":
        with open(path, "rb") as f:
            return cls.from_json(f.read(), **kw)

    @classmethod
    def train_toy(cls, corpus: str, n_merges: int = 200, added_tokens: Sequence[str] = (), **kw) -> "Tokenizer":
        """A small byte-level BPE learnt from `corpus` (tests, demos, synthetic artifacts)."""
        vocab = {_B2U[b]: b for b in range(256)}
        words: Dict[Tuple[str, ...], int] = {}
        for piece in _re.findall(QWEN_SPLIT, corpus):
            w = tuple(_B2U[b] for b in piece.encode("utf-8"))
            words[w] = words.get(w, 0) + 1
        merges: List[Tuple[str, str]] = []
        for _ in range(n_merges):
            counts: Dict[Tuple[str, str], int] = {}
            for w, c in words.items():
                for a, b in zip(w, w[1:]):
                    counts[(a, b)] = counts.get((a, b), 0) + c
            if not counts:
                break
            (a, b), c = max(counts.items(), key=lambda kv: (kv[1], kv[0]))
            if c < 2:
                break
            merges.append((a, b))
            vocab.setdefault(a + b, len(vocab))
            new_words: Dict[Tuple[str, ...], int] = {}
            for w, cnt in words.items():
                out, i = [], 0
                while i < len(w):
                    if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                        out.append(a + b); i += 2
                    else:
                        out.append(w[i]); i += 1
                new_words[tuple(out)] = new_words.get(tuple(out), 0) + cnt
            words = new_words
        added = [{"id": len(vocab) + i, "content": s, "special": True} for i, s in enumerate(added_tokens)]
        return cls(vocab, merges, added, **kw)

    def to_json(self) -> str:
        inv = sorted(self.ranks.items(), key=lambda kv: kv[1][0])
        id_to_str = {i: s for s, i in self.vocab.items()}
        merges = [f"{id_to_str[a]} {id_to_str[b]}" for (a, b), _ in inv]
        added = [{"id": i, "content": s, "special": i in self.special_ids} for s, i in self.added.items()]
        return json.dumps({"version": "1.0", "added_tokens": added,
                           "normalizer": {"type": self.normalizer} if self.normalizer else None,
                           "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
                               {"type": "Split", "pattern": {"Regex": self._split.pattern}, "behavior": "Isolated"},
                               {"type": "ByteLevel", "add_prefix_space": False, "use_regex": False}]},
                           "decoder": {"type": "ByteLevel"},
                           "model": {"type": "BPE", "vocab": self.vocab, "merges": merges}}, ensure_ascii=False)

    # ------------------------------------------------------------------ encode / decode
    @property
    def vocab_size(self) -> int:
        return len(self.id_to_bytes)

    def token_id(self, literal: str) -> Optional[int]:
        return self.added.get(literal, self.vocab.get(literal))

    def _bpe_python(self, symbols: List[int]) -> List[int]:
        sym = list(symbols)
        while len(sym) > 1:
            best, best_i = None, -1
            for i in range(len(sym) - 1):
                r = self.ranks.get((sym[i], sym[i + 1]))
                if r is not None and (best is None or r[0] < best[0]):
                    best, best_i = r, i
            if best is None:
                break
            sym[best_i:best_i + 2] = [best[1]]
        return sym

    def _bpe(self, piece: str) -> List[int]:
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        symbols = [self.byte_ids[b] for b in piece.encode("utf-8")]
        if any(s < 0 for s in symbols):
            raise ValueError("tokenizer vocabulary lacks a byte symbol")
        if self._handle is not None:
            n = len(symbols)
            arr = (ctypes.c_int32 * n)(*symbols)
            out = (ctypes.c_int32 * n)()
            m = self._lib.nfb200_bpe_encode(self._handle, arr, n, out)
            ids = list(out[:m])
        else:
            ids = self._bpe_python(symbols)
        if len(self._cache) < 200000:
            self._cache[piece] = ids
        return ids

    def encode(self, text: str, allow_special: bool = True) -> List[int]:
        ids: List[int] = []
        parts: Iterable[str] = [text]
        if self._added_re is not None and allow_special:
            parts = [p for p in self._added_re.split(text) if p]
        for part in parts:
            if allow_special and part in self.added:
                ids.append(self.added[part])
                continue
            if self.normalizer:
                part = unicodedata.normalize(self.normalizer, part)
            for piece in self._split.findall(part):
                ids.extend(self._bpe(piece))
        return ids

    def encode_framed(self, text: str, literal_spans: Sequence[Tuple[int, int]]) -> Tuple[List[int], List[int]]:
        """Token ids of a rendered prompt whose character spans `literal_spans` came from the caller, and per token
        where it came from (ORIGIN_TEMPLATE / ORIGIN_LITERAL / ORIGIN_MIXED).  Inside a literal span a control
        (special) token's spelling is ordinary text: only the template can produce control tokens, so a message
        that spells an end-of-turn marker cannot close its own frame.  Added tokens that are not special (reasoning
        and tool tags) are matched everywhere, as the stock tokenizer does.  For a prompt without such spellings the
        ids are exactly those of `encode(text)`: ordinary text is still split and merged across span edges.
        Reference: src/spec/frame_axis.h (the origin column), src/targets/qwen3_6/impl/frontend/tokenizer.cpp
        (encode_with_frame_classes; literal spans never yield control tokens)."""
        n = len(text)
        spans = sorted((max(0, int(a)), min(n, int(b))) for a, b in literal_spans if int(b) > int(a))
        # segments: alternating template / literal pieces that cover the text
        segs: List[Tuple[int, int, bool]] = []
        at = 0
        for a, b in spans:
            a = max(a, at)
            if b <= a:
                continue
            if a > at:
                segs.append((at, a, False))
            segs.append((a, b, True))
            at = b
        if at < n:
            segs.append((at, n, False))
        # added-token matches, found inside one segment at a time (a control token never straddles an edge)
        kept: List[Tuple[int, int, int]] = []
        if self._added_re is not None:
            for a, b, lit in segs:
                for m in self._added_re.finditer(text, a, b):
                    tid = self.added[m.group()]
                    if lit and tid in self.special_ids:
                        continue
                    kept.append((m.start(), m.end(), tid))
        ids: List[int] = []
        origin: List[int] = []

        def is_literal(pos: int) -> bool:
            for a, b, lit in segs:
                if a <= pos < b:
                    return lit
            return False

        def ordinary(a: int, b: int) -> None:
            if b <= a:
                return
            # the run's text, normalised piece by piece so that byte offsets can be mapped back to their origin
            pieces: List[Tuple[str, bool]] = []
            for sa, sb, lit in segs:
                lo, hi = max(a, sa), min(b, sb)
                if lo < hi:
                    t = text[lo:hi]
                    pieces.append((unicodedata.normalize(self.normalizer, t) if self.normalizer else t, lit))
            joined = "".join(t for t, _ in pieces)
            whole = unicodedata.normalize(self.normalizer, text[a:b]) if self.normalizer else text[a:b]
            exact = joined == whole       # false when normalisation composes characters across an edge
            edges: List[Tuple[int, int, bool]] = []
            off = 0
            for t, lit in pieces:
                nb = len(t.encode("utf-8"))
                edges.append((off, off + nb, lit))
                off += nb
            if not exact or len(edges) == 1:
                # one origin for the whole run (or no byte map to trust): no per-token bookkeeping
                cls = ORIGIN_MIXED if not exact else (ORIGIN_LITERAL if edges[0][2] else ORIGIN_TEMPLATE)
                first = len(ids)
                for piece in self._split.findall(whole):
                    ids.extend(self._bpe(piece))
                origin.extend([cls] * (len(ids) - first))
                return
            pos, e, last = 0, 0, len(edges) - 1
            nbytes = self.id_to_bytes
            for piece in self._split.findall(whole):
                for tid in self._bpe(piece):
                    nb = len(nbytes[tid])
                    while e < last and pos >= edges[e][1]:
                        e += 1
                    # inside one piece: that piece's origin; across an edge: mixed, unless both sides agree
                    if pos + nb <= edges[e][1]:
                        cls = ORIGIN_LITERAL if edges[e][2] else ORIGIN_TEMPLATE
                    else:
                        kinds = {lit for ea, eb, lit in edges[e:] if ea < pos + nb}
                        cls = ORIGIN_MIXED if len(kinds) != 1 else (ORIGIN_LITERAL if kinds.pop() else ORIGIN_TEMPLATE)
                    ids.append(tid)
                    origin.append(cls)
                    pos += nb
        at = 0
        for a, b, tid in sorted(kept):
            if a < at:
                continue                  # overlapping match (cannot happen within one alternation; kept for safety)
            ordinary(at, a)
            ids.append(tid)
            origin.append(ORIGIN_LITERAL if is_literal(a) else ORIGIN_TEMPLATE)
            at = b
        ordinary(at, n)
        return ids, origin

    def spells_control(self, text: str, literal_spans: Sequence[Tuple[int, int]]) -> bool:
        """Does any literal span spell a control (special) token?"""
        if self._added_re is None:
            return False
        for a, b in literal_spans:
            for m in self._added_re.finditer(text, max(0, int(a)), min(len(text), int(b))):
                if self.added[m.group()] in self.special_ids:
                    return True
        return False

    def decode_bytes(self, ids: Sequence[int], skip_special: bool = False) -> bytes:
        return b"".join(self.id_to_bytes[i] for i in ids
                        if 0 <= i < len(self.id_to_bytes) and not (skip_special and i in self.special_ids))

    def decode(self, ids: Sequence[int], skip_special: bool = False) -> str:
        return self.decode_bytes(ids, skip_special).decode("utf-8", errors="replace")


class StreamDecoder:
    """Incremental detokeniser: emits only complete UTF-8 characters, holds back a split multi-byte tail."""

    def __init__(self, tok: Tokenizer, skip_special: bool = True):
        self.tok, self.skip_special = tok, skip_special
        self._buf = b""

    def feed(self, token_id: int) -> str:
        self._buf += self.tok.decode_bytes([token_id], self.skip_special)
        cut = len(self._buf)
        # back off over an incomplete trailing sequence (at most 3 continuation bytes + 1 lead byte)
        for back in range(1, min(4, len(self._buf)) + 1):
            b = self._buf[-back]
            if b & 0xC0 == 0x80:
                continue
            need = 1 if b < 0x80 else 2 if b >> 5 == 0b110 else 3 if b >> 4 == 0b1110 else 4 if b >> 3 == 0b11110 else 1
            if need > back:
                cut = len(self._buf) - back
            break
        out, self._buf = self._buf[:cut], self._buf[cut:]
        return out.decode("utf-8", errors="replace")

    def flush(self) -> str:
        out, self._buf = self._buf, b""
        return out.decode("utf-8", errors="replace")
