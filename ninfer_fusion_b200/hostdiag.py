"""Two front doors that need no GPU, no CUDA library and no torch import:

    python ninfer_fusion_b200/hostdiag.py cufree
    python ninfer_fusion_b200/hostdiag.py hostpath ARTIFACT.ninfer [MORE.ninfer ...]

`cufree` reports what the loader and the file system can answer without calling a single CUDA function: which
accelerator device nodes exist, whether the driver and runtime libraries are findable, whether the native library
of this package has been built.  Every row names the exact path that was tested, so "absent" means "this path was
tested and does not exist", never "the probe found nothing".

`hostpath` opens real artifacts with the container's own rules (prefix, JSON directory, closed member sets, known
formats and layouts, ordered aligned non-overlapping payloads) and asks the engine's own registry gate about the
model they name.  It runs no model arithmetic and emits no tokens, and says so in its verdict.
Exit code: 0 = every artifact was opened and every gate answered, 3 = at least one artifact was refused, 2 = usage.

Counterparts of the reference's ninfer-cufree and ninfer-hostpath (apps/cufree/main.cpp, apps/hostpath/main.cpp).
This file is run as a script on purpose: importing the package would import torch.
"""
import glob
import importlib.util
import json
import os
import struct
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
MAGIC = b"NINFER\x00\x02"
TENSOR_KEYS = {"name", "kind", "shape", "format", "layout", "offset", "bytes"}
RESOURCE_KEYS = {"name", "kind", "encoding", "offset", "bytes"}
KNOWN_FORMATS = {"BF16", "FP32", "I32", "Q4G64_F16S", "Q5G64_F16S", "Q6G64_F16S", "W8G32_F16S", "NVFP4",
                 "FP8_E4M3FN_ROW_BF16S", "FP8_E4M3FN_BLOCK128_F32S"}
TENSOR_ALIGNMENT = 256
LIB_DIRS = ("/usr/lib/x86_64-linux-gnu", "/usr/lib64", "/usr/local/cuda/lib64", "/usr/local/cuda/targets/x86_64-linux/lib",
            "/usr/lib/wsl/lib")


def _row(what, path, present):
    print(f"  {'present' if present else 'absent ':8s} {what}: {path}")


def cufree() -> int:
    print("ninfer-fusion host report (no CUDA function is called, no device is opened)")
    print("accelerator kernel interfaces, as paths:")
    for pattern in ("/dev/nvidiactl", "/dev/nvidia-uvm", "/dev/nvidia[0-9]*", "/proc/driver/nvidia/version", "/dev/kfd", "/dev/dri/renderD*"):
        hits = sorted(glob.glob(pattern))
        _row("device interface", pattern + (f" -> {len(hits)} entries" if len(hits) > 1 else ""), bool(hits))
    print("libraries the native path needs, as files:")
    for soname in ("libcuda.so.1", "libcudart.so.12", "libcudart.so"):
        found = [os.path.join(d, soname) for d in LIB_DIRS if os.path.exists(os.path.join(d, soname))]
        _row("library", found[0] if found else f"{soname} in {', '.join(LIB_DIRS)}", bool(found))
    lib = os.path.join(HERE, "_C.so")
    _row("native kernels of this package (sm_100a only)", lib, os.path.exists(lib))
    for dist in ("torch", "numpy"):
        spec = importlib.util.find_spec(dist)
        _row(f"python package {dist} (not imported)", spec.origin if spec and spec.origin else dist, spec is not None)
    print("architectures and what this package's kernels find on them (capability table, no device is asked):")
    spec = importlib.util.spec_from_file_location("_nfb_archcaps", os.path.join(HERE, "archcaps.py"))
    caps = importlib.util.module_from_spec(spec)
    sys.modules["_nfb_archcaps"] = caps
    spec.loader.exec_module(caps)
    for rung in caps.ARCH_LADDER:
        print("  " + caps.device_report(rung.sm))
    print("verdict: this program cannot tell whether a GPU works; it reports which of the things a GPU run needs exist as files")
    return 0


def _registry():
    """models/config.py and models/packages.py loaded by path under stand-in packages, so that the real package
    __init__ (which imports torch) never runs."""
    for name, path in (("ninfer_fusion_b200", HERE), ("ninfer_fusion_b200.models", os.path.join(HERE, "models"))):
        if name not in sys.modules:
            pkg = types.ModuleType(name)
            pkg.__path__ = [path]
            sys.modules[name] = pkg
    mods = {}
    for leaf in ("config", "packages"):
        full = f"ninfer_fusion_b200.models.{leaf}"
        spec = importlib.util.spec_from_file_location(full, os.path.join(HERE, "models", f"{leaf}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[full] = mod
        spec.loader.exec_module(mod)
        mods[leaf] = mod
    return mods["packages"]


def read_directory(path):
    """(identity, objects, payload start) of a .ninfer file, or raises ValueError naming the rule that failed."""
    with open(path, "rb") as f:
        prefix = f.read(16)
        if len(prefix) != 16 or prefix[:8] != MAGIC:
            raise ValueError("not a version-2 .ninfer file (prefix magic)")
        (n_json,) = struct.unpack("<Q", prefix[8:])
        size = os.path.getsize(path)
        if n_json == 0 or 16 + n_json > size:
            raise ValueError("JSON directory length exceeds the file")
        root = json.loads(f.read(n_json).decode("utf-8"))
    if set(root) != {"identity", "objects"} or set(root["identity"]) != {"model_id", "weights_id"}:
        raise ValueError("JSON root must hold exactly identity{model_id, weights_id} and objects")
    start = (16 + n_json + 4095) // 4096 * 4096
    end_prev = 0
    for o in root["objects"]:
        want = TENSOR_KEYS if o.get("kind") == "tensor" else RESOURCE_KEYS if o.get("kind") == "resource" else None
        if want is None or set(o) != want:
            raise ValueError(f"object '{o.get('name')}': member set is not the closed set of its kind")
        if o["kind"] == "tensor" and o["format"] not in KNOWN_FORMATS:
            raise ValueError(f"object '{o['name']}': unknown format '{o['format']}'")
        if o["offset"] < end_prev or (o["kind"] == "tensor" and o["offset"] % TENSOR_ALIGNMENT):
            raise ValueError(f"object '{o['name']}': payloads must be ordered and non-overlapping, tensors "
                             f"{TENSOR_ALIGNMENT}-byte aligned")
        end_prev = o["offset"] + o["bytes"]
    if start + end_prev > size:
        raise ValueError("payloads run past the end of the file")
    return root["identity"], root["objects"], start


def hostpath(paths) -> int:
    packages = _registry()
    refused = 0
    for path in paths:
        print(f"artifact: {path}")
        try:
            identity, objects, start = read_directory(path)
        except (OSError, ValueError, KeyError, json.JSONDecodeError) as e:
            print(f"  refused: {e}")
            refused += 1
            continue
        tensors = [o for o in objects if o["kind"] == "tensor"]
        by_format = {}
        for o in tensors:
            by_format[o["format"]] = by_format.get(o["format"], 0) + o["bytes"]
        print(f"  identity: model_id={identity['model_id']} weights_id={identity['weights_id']}")
        print(f"  objects: {len(tensors)} tensors, {len(objects) - len(tensors)} resources, payloads start at byte {start}")
        for fmt, n in sorted(by_format.items()):
            print(f"  format {fmt}: {n / 2**20:.1f} MiB")
        try:
            cfg = packages.construct(identity["model_id"])
            print(f"  registry gate: accepted ({cfg.n_layers} layers, hidden {cfg.hidden}, "
                  f"{len(cfg.attn_layers)} full-attention / {len(cfg.gdn_layers)} linear-attention layers)")
        except (KeyError, ValueError) as e:
            print(f"  registry gate: refused: {e}")
            refused += 1
    print("verdict: content_tokens_emitted: 0 (this program runs no model arithmetic; it read directories and asked gates)")
    return 3 if refused else 0


def main(argv) -> int:
    if len(argv) >= 2 and argv[1] == "cufree" and len(argv) == 2:
        return cufree()
    if len(argv) >= 3 and argv[1] == "hostpath":
        return hostpath(argv[2:])
    print(__doc__.strip().split("\n\n")[0], file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main(sys.argv))
