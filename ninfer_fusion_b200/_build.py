"""In-tree build of the native library (``ninfer_fusion_b200/_C.so``).

Every ``.cu`` under ``csrc/`` is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``) by calling nvcc
directly; the torch binding translation unit is compiled with g++ against the
torch headers; everything is linked into one shared object that
``torch.ops.load_library`` loads.  Objects are cached under ``build/`` keyed
by a hash of the source, its local headers and the flags, so a rebuild only
recompiles what changed.  nvcc cross-compiles, so this runs without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
ROOT = PKG.parent
BUILD = ROOT / "build" / "obj"
LIB = PKG / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-DNDEBUG",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-DNDEBUG", "-Wno-deprecated-declarations"]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".h", ".cuh", ".hpp"):
            h.update(p.read_bytes())
    return h.hexdigest()


def _sources():
    cu = sorted(CSRC.rglob("*.cu"))
    cpp = sorted(p for p in CSRC.rglob("*.cpp"))
    return cu, cpp


def _compile(src: Path, cmd_prefix: list[str], tag: str, hdr: str, verbose: bool) -> tuple[Path, bool]:
    key = hashlib.sha256()
    key.update(src.read_bytes())
    key.update(hdr.encode())
    key.update(" ".join(cmd_prefix).encode())
    rel = src.relative_to(CSRC).as_posix().replace("/", "__")
    obj = BUILD / f"{rel}.{key.hexdigest()[:16]}.o"
    if obj.exists():
        return obj, False
    for stale in BUILD.glob(f"{rel}.*.o"):
        stale.unlink()
    cmd = cmd_prefix + ["-c", str(src), "-o", str(obj)]
    if verbose:
        print(f"[build] {tag} {src.relative_to(ROOT)}", flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr.strip():
        print(r.stderr, flush=True)
    return obj, True


def build(verbose: bool = True, ptxas_info: bool = False) -> Path:
    """Compile (if needed) and link ``_C.so``; returns its path."""
    import torch
    from torch.utils import cpp_extension as ce

    BUILD.mkdir(parents=True, exist_ok=True)
    cuda = _cuda_home()
    nvcc = os.path.join(cuda, "bin", "nvcc")
    hdr = _headers_digest()
    inc = [f"-I{CSRC}", f"-I{cuda}/include"]
    torch_inc = [f"-I{p}" for p in ce.include_paths()]
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    cu, cpp = _sources()
    jobs = []
    nv = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + inc
    for s in cu:
        jobs.append((s, nv, "nvcc"))
    for s in cpp:
        uses_torch = "torch/" in s.read_text() or "ATen/" in s.read_text()
        cx = ["g++"] + CXX_FLAGS + inc + ([abi] + torch_inc if uses_torch else [])
        jobs.append((s, cx, "g++ "))
    workers = max(1, min(len(jobs), os.cpu_count() or 4))
    with ThreadPoolExecutor(workers) as ex:
        res = list(ex.map(lambda j: _compile(j[0], j[1], j[2], hdr, verbose), jobs))
    objs = [r[0] for r in res]
    changed = any(r[1] for r in res)
    # (objects may also have been compiled by an earlier, link-less pass: compare against the library's age)
    stale = LIB.exists() and any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs)
    if changed or stale or not LIB.exists():
        tl = ce.library_paths()
        # link beside the final name and rename: a reader (a process that loads the library, a copy of the tree) never
        # sees a half-written file
        tmp = LIB.with_suffix(".so.tmp")
        link = ["g++", "-shared", "-o", str(tmp)] + [str(o) for o in objs]
        for p in tl:
            link += [f"-L{p}", f"-Wl,-rpath,{p}"]
        link += [f"-L{cuda}/lib64", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
        if verbose:
            print(f"[build] link {LIB.relative_to(ROOT)}", flush=True)
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(link)}\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    build(verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    print(LIB)
