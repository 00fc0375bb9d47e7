"""Retrieval-augmented answering over documents held by the server: a bounded in-memory store with a BM25 index,
prompt assembly with numbered sources, and the routes that expose it.

    POST   /v1/rag/documents          {"title": "...", "text": "..."}        -> {"id", "chunks"}
    GET    /v1/rag/documents                                                  -> list (ids, titles, sizes; no text)
    DELETE /v1/rag/documents/{id}
    POST   /v1/rag/query              {"query": "...", "top_k": 4, "max_tokens": 256, ...sampler fields}
                                      -> {"answer", "sources": [{"n", "document", "title", "chunk", "score", "text"}], "usage"}

Documents are split into chunks on paragraph boundaries (long paragraphs on sentence boundaries) of at most
`chunk_chars` characters; retrieval is Okapi BM25 over lower-cased word tokens (CJK characters count as words of
their own); the answer is one ordinary chat generation whose system message carries the retrieved chunks as numbered
sources and asks for citations like [1].  The store is bounded in documents and bytes (oldest first out) and lives in
the server process only.

Reference: tools/gui/rag_gui.py (the reference's document question-answering console over its own server).
"""
from __future__ import annotations

import math
import re
import threading
import uuid
from collections import Counter, OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

_WORD = re.compile(r"[A-Za-z0-9_]+|[぀-ヿ㐀-鿿가-힯]")
_SENT = re.compile(r"(?<=[.!?。！？])\s+")

SYSTEM = ("Answer the question using only the numbered sources below. Cite the sources you use like [1]. "
          "If the sources do not contain the answer, say so.\n\n{sources}")


def tokenize(text: str) -> List[str]:
    return [m.group(0).lower() for m in _WORD.finditer(text)]


def chunk_text(text: str, chunk_chars: int = 1200) -> List[str]:
    """Paragraphs packed into chunks of at most `chunk_chars`; a longer paragraph is cut at sentence ends, a longer
    sentence at the limit."""
    out: List[str] = []
    cur = ""
    for para in (p.strip() for p in re.split(r"\n\s*\n", text) if p.strip()):
        pieces = [para]
        if len(para) > chunk_chars:
            pieces, buf = [], ""
            for sent in _SENT.split(para):
                while len(sent) > chunk_chars:
                    pieces.append(sent[:chunk_chars])
                    sent = sent[chunk_chars:]
                if len(buf) + len(sent) + 1 > chunk_chars and buf:
                    pieces.append(buf)
                    buf = sent
                else:
                    buf = (buf + " " + sent).strip()
            if buf:
                pieces.append(buf)
        for piece in pieces:
            if len(cur) + len(piece) + 2 > chunk_chars and cur:
                out.append(cur)
                cur = piece
            else:
                cur = (cur + "\n\n" + piece).strip()
    if cur:
        out.append(cur)
    return out


@dataclass
class Chunk:
    document: str
    index: int
    text: str
    tf: Counter = field(default_factory=Counter)
    length: int = 0


class DocumentStore:
    def __init__(self, max_documents: int = 256, max_bytes: int = 64 << 20, chunk_chars: int = 1200,
                 k1: float = 1.5, b: float = 0.75):
        self.max_documents, self.max_bytes, self.chunk_chars = max_documents, max_bytes, chunk_chars
        self.k1, self.b = k1, b
        self.docs: "OrderedDict[str, dict]" = OrderedDict()
        self.chunks: List[Chunk] = []
        self.df: Counter = Counter()
        self.bytes = 0
        self.lock = threading.Lock()

    def add(self, title: str, text: str) -> dict:
        if not isinstance(text, str) or not text.strip():
            raise ValueError("document text is empty")
        size = len(text.encode("utf-8"))
        if size > self.max_bytes:
            raise ValueError("document exceeds the store's byte limit")
        doc_id = "doc_" + uuid.uuid4().hex[:16]
        parts = chunk_text(text, self.chunk_chars)
        with self.lock:
            while self.docs and (len(self.docs) >= self.max_documents or self.bytes + size > self.max_bytes):
                self._remove(next(iter(self.docs)))
            for i, t in enumerate(parts):
                toks = tokenize(t)
                c = Chunk(doc_id, i, t, Counter(toks), len(toks))
                self.chunks.append(c)
                self.df.update(c.tf.keys())
            self.docs[doc_id] = {"id": doc_id, "title": str(title or "untitled")[:200], "bytes": size, "chunks": len(parts)}
            self.bytes += size
        return dict(self.docs[doc_id])

    def _remove(self, doc_id: str) -> bool:
        meta = self.docs.pop(doc_id, None)
        if meta is None:
            return False
        keep = []
        for c in self.chunks:
            if c.document == doc_id:
                self.df.subtract(c.tf.keys())
            else:
                keep.append(c)
        self.chunks = keep
        self.df = +self.df          # drop zero counts
        self.bytes -= meta["bytes"]
        return True

    def remove(self, doc_id: str) -> bool:
        with self.lock:
            return self._remove(doc_id)

    def list(self) -> List[dict]:
        with self.lock:
            return [dict(d) for d in self.docs.values()]

    def retrieve(self, query: str, top_k: int = 4) -> List[Tuple[float, Chunk]]:
        """Okapi BM25; chunks that share no term with the query are not returned."""
        q = tokenize(query)
        with self.lock:
            n = len(self.chunks)
            if not q or n == 0:
                return []
            avg = sum(c.length for c in self.chunks) / n or 1.0
            scored = []
            for c in self.chunks:
                s = 0.0
                for term in set(q):
                    f = c.tf.get(term, 0)
                    if not f:
                        continue
                    idf = math.log(1.0 + (n - self.df[term] + 0.5) / (self.df[term] + 0.5))
                    s += idf * f * (self.k1 + 1) / (f + self.k1 * (1 - self.b + self.b * c.length / avg))
                if s > 0:
                    scored.append((s, c))
        scored.sort(key=lambda sc: (-sc[0], sc[1].document, sc[1].index))
        return scored[: max(1, int(top_k))]

    def build_messages(self, query: str, hits: List[Tuple[float, Chunk]]) -> Tuple[List[dict], List[dict]]:
        sources, blocks = [], []
        for n, (score, c) in enumerate(hits, 1):
            title = self.docs.get(c.document, {}).get("title", "")
            blocks.append(f"[{n}] {title}\n{c.text}")
            sources.append({"n": n, "document": c.document, "title": title, "chunk": c.index, "score": round(score, 4),
                            "text": c.text})
        system = SYSTEM.format(sources="\n\n".join(blocks) if blocks else "(no source matched the question)")
        return [{"role": "system", "content": system}, {"role": "user", "content": query}], sources


PAGE = """<!doctype html><html lang="en"><head><meta charset="utf-8"><title>documents</title>
<style>body{font:14px/1.45 system-ui,sans-serif;margin:0;background:#111;color:#ddd;padding:16px;max-width:920px}
input,textarea{background:#222;color:#ddd;border:1px solid #444;border-radius:4px;padding:6px;width:100%;box-sizing:border-box}
textarea{min-height:120px}button{background:#2d5fa8;color:#fff;border:0;border-radius:4px;padding:6px 14px;margin:6px 0;cursor:pointer}
pre{white-space:pre-wrap;background:#1b1b1b;padding:10px;border-radius:6px}.src{color:#9ab}</style></head><body>
<h3>Documents</h3><input id="key" type="password" placeholder="API key"><input id="title" placeholder="title">
<textarea id="text" placeholder="paste a document"></textarea><button id="add">add document</button><pre id="docs"></pre>
<h3>Question</h3><input id="q" placeholder="question"><button id="ask">ask</button><pre id="ans"></pre><pre id="srcs" class="src"></pre>
<script>
const $=id=>document.getElementById(id);const H=()=>{const h={'Content-Type':'application/json'};if($('key').value)h['Authorization']='Bearer '+$('key').value;return h};
async function list(){const r=await fetch('/v1/rag/documents',{headers:H()});$('docs').textContent=r.ok?JSON.stringify((await r.json()).data,null,1):'('+r.status+')'}
$('add').onclick=async()=>{await fetch('/v1/rag/documents',{method:'POST',headers:H(),body:JSON.stringify({title:$('title').value,text:$('text').value})});$('text').value='';list()};
$('ask').onclick=async()=>{$('ans').textContent='...';const r=await fetch('/v1/rag/query',{method:'POST',headers:H(),body:JSON.stringify({query:$('q').value,top_k:4,max_tokens:256})});
const j=await r.json();$('ans').textContent=j.answer||JSON.stringify(j);$('srcs').textContent=(j.sources||[]).map(s=>'['+s.n+'] '+s.title+' (score '+s.score+')\\n'+s.text).join('\\n\\n')};
list();
</script></body></html>"""


def page_bytes() -> bytes:
    return PAGE.encode("utf-8")
