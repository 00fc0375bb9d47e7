"""GGUF import: container reader, block-quant decoders and the tensor-name map of the GDN-hybrid family.

A GGUF file is `GGUF` magic, version, tensor count, metadata count, typed key/value metadata, tensor infos (name,
dims with the fastest-varying first, ggml type, offset) and, aligned to `general.alignment`, the tensor data.  The
decoders cover the types the published hybrid checkpoints use (F32 / F16 / BF16 / Q8_0 / Q4_0 / Q4_K / Q6_K); every
tensor is decoded to fp32 in ggml element order and reshaped to the Hugging Face (outermost-first) shape.

`GgufSource` presents the file under Hugging Face tensor names, so the same `convert.hf.hf_to_weights` mapping
builds the engine inventory.  Three value conventions of the llama.cpp exporter are undone on the way (each can be
switched off): `ssm_a` holds -exp(A_log); RMSNorm weights other than the GDN head norm are stored as 1 + w; the
conv kernel is stored [kernel, channels] without the unit middle axis.

Reference: tools/convert/gguf_names.py (rule set per architecture, block_count includes the nextn block),
tools/convert/gguf_kquant.py (Q4_K 144-byte / Q6_K 210-byte blocks), tools/convert/unit_offset_norms.py.
"""
from __future__ import annotations

import re
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from ..models.config import ModelConfig, MoEConfig

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q6_K, GGML_BF16 = 0, 1, 2, 8, 12, 14, 30
QK_K = 256
_BLOCK = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_BF16: (1, 2), GGML_Q4_0: (32, 18), GGML_Q8_0: (32, 34),
          GGML_Q4_K: (QK_K, 144), GGML_Q6_K: (QK_K, 210)}
_TYPE_NAMES = {0: "F32", 1: "F16", 2: "Q4_0", 8: "Q8_0", 12: "Q4_K", 14: "Q6_K", 30: "BF16"}


# ---------------------------------------------------------------------------------------- decoders
def _f16(b: np.ndarray) -> np.ndarray:
    return b.copy().view(np.float16).astype(np.float32)


def dequant_q8_0(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw.reshape(-1, 34)
    d = _f16(blk[:, :2]).reshape(-1, 1)
    return (d * blk[:, 2:].copy().view(np.int8).astype(np.float32)).reshape(-1)[:n]


def dequant_q4_0(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw.reshape(-1, 18)
    d = _f16(blk[:, :2]).reshape(-1, 1)
    q = blk[:, 2:]
    lo = (q & 0xF).astype(np.float32) - 8.0
    hi = (q >> 4).astype(np.float32) - 8.0
    return (d * np.concatenate([lo, hi], axis=1)).reshape(-1)[:n]


def dequant_q4_k(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw.reshape(-1, 144)
    d = _f16(blk[:, 0:2]).reshape(-1, 1)
    dmin = _f16(blk[:, 2:4]).reshape(-1, 1)
    s = blk[:, 4:16].astype(np.int32)
    qs = blk[:, 16:144]
    sc = np.empty((blk.shape[0], 8), dtype=np.float32)
    mn = np.empty((blk.shape[0], 8), dtype=np.float32)
    for j in range(8):
        if j < 4:
            sc[:, j] = s[:, j] & 63
            mn[:, j] = s[:, j + 4] & 63
        else:
            sc[:, j] = (s[:, j + 4] & 0xF) | ((s[:, j - 4] >> 6) << 4)
            mn[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
    out = np.empty((blk.shape[0], 8, 32), dtype=np.float32)
    for pair in range(4):
        q = qs[:, 32 * pair:32 * pair + 32]
        out[:, 2 * pair] = d * sc[:, 2 * pair:2 * pair + 1] * (q & 0xF) - dmin * mn[:, 2 * pair:2 * pair + 1]
        out[:, 2 * pair + 1] = d * sc[:, 2 * pair + 1:2 * pair + 2] * (q >> 4) - dmin * mn[:, 2 * pair + 1:2 * pair + 2]
    return out.reshape(-1)[:n]


def dequant_q6_k(raw: np.ndarray, n: int) -> np.ndarray:
    blk = raw.reshape(-1, 210)
    ql, qh = blk[:, :128].astype(np.int32), blk[:, 128:192].astype(np.int32)
    sc = blk[:, 192:208].copy().view(np.int8).astype(np.float32)
    d = _f16(blk[:, 208:210]).reshape(-1, 1)
    out = np.empty((blk.shape[0], 256), dtype=np.float32)
    for half in range(2):
        l, h, s = ql[:, 64 * half:64 * half + 64], qh[:, 32 * half:32 * half + 32], sc[:, 8 * half:8 * half + 8]
        idx = np.arange(32) // 16
        q1 = ((l[:, :32] & 0xF) | (((h >> 0) & 3) << 4)) - 32
        q2 = ((l[:, 32:] & 0xF) | (((h >> 2) & 3) << 4)) - 32
        q3 = ((l[:, :32] >> 4) | (((h >> 4) & 3) << 4)) - 32
        q4 = ((l[:, 32:] >> 4) | (((h >> 6) & 3) << 4)) - 32
        base = 128 * half
        out[:, base:base + 32] = d * s[:, idx] * q1
        out[:, base + 32:base + 64] = d * s[:, idx + 2] * q2
        out[:, base + 64:base + 96] = d * s[:, idx + 4] * q3
        out[:, base + 96:base + 128] = d * s[:, idx + 6] * q4
    return out.reshape(-1)[:n]


def to_fp32(ggml_type: int, raw: np.ndarray, n: int) -> np.ndarray:
    if ggml_type == GGML_F32:
        return raw.copy().view(np.float32)[:n]
    if ggml_type == GGML_F16:
        return _f16(raw)[:n]
    if ggml_type == GGML_BF16:
        return (raw.copy().view(np.uint16).astype(np.uint32) << 16).view(np.float32)[:n]
    fn = {GGML_Q8_0: dequant_q8_0, GGML_Q4_0: dequant_q4_0, GGML_Q4_K: dequant_q4_k, GGML_Q6_K: dequant_q6_k}.get(ggml_type)
    if fn is None:
        raise ValueError(f"ggml tensor type {ggml_type} is not supported by this importer")
    return fn(raw, n)


def tensor_nbytes(ggml_type: int, n: int) -> int:
    if ggml_type not in _BLOCK:
        raise ValueError(f"ggml tensor type {ggml_type} is not supported by this importer")
    per, size = _BLOCK[ggml_type]
    if n % per:
        raise ValueError(f"{_TYPE_NAMES[ggml_type]} needs a multiple of {per} values, got {n}")
    return n // per * size


# ---------------------------------------------------------------------------------------- container
class GgufFile:
    def __init__(self, path: str):
        self.path = path
        self.data = np.memmap(path, dtype=np.uint8, mode="r")
        self._pos = 0
        if bytes(self._take(4)) != b"GGUF":
            raise ValueError(f"{path}: not a GGUF file")
        self.version = self._u32()
        if self.version not in (2, 3):
            raise ValueError(f"{path}: GGUF version {self.version} is not supported")
        n_tensors, n_kv = self._u64(), self._u64()
        self.kv: Dict[str, object] = {}
        for _ in range(n_kv):
            key = self._string()
            self.kv[key] = self._value(self._u32())
        self.tensors: Dict[str, Tuple[Tuple[int, ...], int, int]] = {}   # name -> (ne, type, offset)
        for _ in range(n_tensors):
            name = self._string()
            nd = self._u32()
            ne = tuple(self._u64() for _ in range(nd))
            t = self._u32()
            self.tensors[name] = (ne, t, self._u64())
        align = int(self.kv.get("general.alignment", 32))
        self.data_start = (self._pos + align - 1) // align * align

    def _take(self, n: int) -> np.ndarray:
        out = self.data[self._pos:self._pos + n]
        if out.shape[0] != n:
            raise ValueError(f"{self.path}: truncated file")
        self._pos += n
        return out

    def _u32(self) -> int:
        return struct.unpack("<I", bytes(self._take(4)))[0]

    def _u64(self) -> int:
        return struct.unpack("<Q", bytes(self._take(8)))[0]

    def _string(self) -> str:
        return bytes(self._take(self._u64())).decode("utf-8", errors="replace")

    def _value(self, t: int):
        fmt = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
        if t in fmt:
            return struct.unpack(fmt[t], bytes(self._take(struct.calcsize(fmt[t]))))[0]
        if t == 8:
            return self._string()
        if t == 9:
            et, n = self._u32(), self._u64()
            return [self._value(et) for _ in range(n)]
        raise ValueError(f"{self.path}: unknown metadata type {t}")

    def names(self) -> List[str]:
        return list(self.tensors)

    def hf_shape(self, name: str) -> Tuple[int, ...]:
        return tuple(reversed(self.tensors[name][0]))

    def tensor(self, name: str) -> torch.Tensor:
        """fp32 tensor in the Hugging Face (outermost-first) shape."""
        ne, t, off = self.tensors[name]
        n = int(np.prod(ne)) if ne else 1
        raw = np.asarray(self.data[self.data_start + off:self.data_start + off + tensor_nbytes(t, n)])
        return torch.from_numpy(to_fp32(t, raw, n).astype(np.float32, copy=True)).reshape(tuple(reversed(ne)))


# ---------------------------------------------------------------------------------------- names
_RULES = [
    (r"^token_embd\.weight$", "model.language_model.embed_tokens.weight"),
    (r"^output_norm\.weight$", "model.language_model.norm.weight"),
    (r"^output\.weight$", "lm_head.weight"),
    (r"^blk\.\d+\.nextn\.eh_proj\.weight$", "mtp.fc.weight"),
    (r"^blk\.\d+\.nextn\.enorm\.weight$", "mtp.pre_fc_norm_embedding.weight"),
    (r"^blk\.\d+\.nextn\.hnorm\.weight$", "mtp.pre_fc_norm_hidden.weight"),
    (r"^blk\.\d+\.nextn\.shared_head_norm\.weight$", "mtp.norm.weight"),
    (r"^blk\.(\d+)\.attn_norm\.weight$", "{p}input_layernorm.weight"),
    (r"^blk\.(\d+)\.post_attention_norm\.weight$", "{p}post_attention_layernorm.weight"),
    (r"^blk\.(\d+)\.ffn_gate\.weight$", "{p}mlp.gate_proj.weight"),
    (r"^blk\.(\d+)\.ffn_up\.weight$", "{p}mlp.up_proj.weight"),
    (r"^blk\.(\d+)\.ffn_down\.weight$", "{p}mlp.down_proj.weight"),
    (r"^blk\.(\d+)\.attn_q\.weight$", "{p}self_attn.q_proj.weight"),
    (r"^blk\.(\d+)\.attn_k\.weight$", "{p}self_attn.k_proj.weight"),
    (r"^blk\.(\d+)\.attn_v\.weight$", "{p}self_attn.v_proj.weight"),
    (r"^blk\.(\d+)\.attn_output\.weight$", "{p}self_attn.o_proj.weight"),
    (r"^blk\.(\d+)\.attn_q_norm\.weight$", "{p}self_attn.q_norm.weight"),
    (r"^blk\.(\d+)\.attn_k_norm\.weight$", "{p}self_attn.k_norm.weight"),
    (r"^blk\.(\d+)\.attn_qkv\.weight$", "{p}linear_attn.in_proj_qkv.weight"),
    (r"^blk\.(\d+)\.attn_gate\.weight$", "{p}linear_attn.in_proj_z.weight"),
    (r"^blk\.(\d+)\.ssm_alpha\.weight$", "{p}linear_attn.in_proj_a.weight"),
    (r"^blk\.(\d+)\.ssm_beta\.weight$", "{p}linear_attn.in_proj_b.weight"),
    (r"^blk\.(\d+)\.ssm_conv1d\.weight$", "{p}linear_attn.conv1d.weight"),
    (r"^blk\.(\d+)\.ssm_dt\.bias$", "{p}linear_attn.dt_bias"),
    (r"^blk\.(\d+)\.ssm_a$", "{p}linear_attn.A_log"),
    (r"^blk\.(\d+)\.ssm_norm\.weight$", "{p}linear_attn.norm.weight"),
    (r"^blk\.(\d+)\.ssm_out\.weight$", "{p}linear_attn.out_proj.weight"),
]
_COMPILED = [(re.compile(a), b) for a, b in _RULES]


def layer_split(kv: Dict[str, object], arch: str) -> Tuple[int, int]:
    """(main layers, nextn / draft layers): `block_count` counts the draft blocks too."""
    blocks = int(kv[f"{arch}.block_count"])
    nextn = int(kv.get(f"{arch}.nextn_predict_layers", 0) or 0)
    if nextn > blocks:
        raise ValueError(f"{arch}.nextn_predict_layers={nextn} exceeds block_count={blocks}")
    return blocks - nextn, nextn


def hf_name(gguf_name: str, main_layers: int) -> Optional[str]:
    for rx, target in _COMPILED:
        m = rx.match(gguf_name)
        if m is None:
            continue
        if "{p}" not in target:
            return target
        i = int(m.group(1))
        prefix = f"model.language_model.layers.{i}." if i < main_layers else f"mtp.layers.{i - main_layers}."
        return target.replace("{p}", prefix)
    return None


class GgufSource:
    """A GGUF file under Hugging Face tensor names (`in`, `.tensor(name)`, `.names()`), values in HF conventions."""

    def __init__(self, path: str, undo_norm_offset: bool = True, undo_a_exp: bool = True):
        self.file = GgufFile(path)
        self.arch = str(self.file.kv.get("general.architecture", "qwen35"))
        self.main_layers, self.nextn = layer_split(self.file.kv, self.arch)
        self.undo_norm_offset, self.undo_a_exp = undo_norm_offset, undo_a_exp
        self.map: Dict[str, str] = {}
        self.unmapped: List[str] = []
        for n in self.file.names():
            h = hf_name(n, self.main_layers)
            if h is None:
                self.unmapped.append(n)
            else:
                self.map[h] = n

    def __contains__(self, name: str) -> bool:
        return name in self.map

    def names(self) -> List[str]:
        return list(self.map)

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self.map:
            raise KeyError(f"GGUF file has no tensor for '{name}'")
        t = self.file.tensor(self.map[name])
        if name.endswith("linear_attn.conv1d.weight"):
            return t.t().contiguous()[:, None, :] if t.dim() == 2 and t.shape[0] < t.shape[1] else t.reshape(t.shape[0], 1, -1)
        if name.endswith(".A_log") and self.undo_a_exp and bool((t < 0).all()):
            return torch.log(-t)
        if self.undo_norm_offset and name.endswith("norm.weight") and not name.endswith("linear_attn.norm.weight"):
            return t - 1.0
        return t

    def close(self) -> None:
        del self.file


def config_from_gguf(kv: Dict[str, object], name: str = "gguf-import") -> ModelConfig:
    arch = str(kv.get("general.architecture", "qwen35"))
    g = lambda k, d=None: kv.get(f"{arch}.{k}", d)   # noqa: E731
    main, _ = layer_split(kv, arch)
    moe = None
    if int(g("expert_count", 0) or 0) > 0:
        moe = MoEConfig(n_experts=int(g("expert_count")), top_k=int(g("expert_used_count")),
                        expert_inter=int(g("expert_feed_forward_length")),
                        shared_inter=int(g("expert_shared_feed_forward_length", g("expert_feed_forward_length"))))
    vocab = len(kv.get("tokenizer.ggml.tokens", [])) or int(g("vocab_size", 0))
    return ModelConfig(
        name=name, n_layers=main, hidden=int(g("embedding_length")), vocab=vocab,
        n_q_heads=int(g("attention.head_count")), n_kv_heads=int(g("attention.head_count_kv")),
        head_dim=int(g("attention.key_length", 256)), rot_dim=int(g("rope.dimension_count", 64)),
        rope_theta=float(g("rope.freq_base", 1e7)), gdn_qk_heads=int(g("ssm.group_count", 16)),
        gdn_v_heads=int(g("ssm.time_step_rank", 32)), gdn_head_dim=int(g("ssm.state_size", 128)),
        conv_kernel=int(g("ssm.conv_kernel", 4)), ffn_inter=0 if moe else int(g("feed_forward_length")), moe=moe,
        rms_eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)),
        full_attn_interval=int(g("full_attention_interval", 4)), max_context=int(g("context_length", 262144)))


# ---------------------------------------------------------------------------------------- writer (tests, export)
def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    b = x.astype(np.float32).reshape(-1, 32)
    d = np.abs(b).max(axis=1, keepdims=True) / 127.0
    q = np.where(d > 0, np.rint(b / np.where(d > 0, d, 1.0)), 0).astype(np.int8)
    out = np.empty((b.shape[0], 34), dtype=np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def write_gguf(path: str, kv: Dict[str, object], tensors: Dict[str, Tuple[torch.Tensor, int]], alignment: int = 32) -> None:
    """`tensors`: gguf name -> (tensor in HF shape, ggml type among F32 / F16 / BF16 / Q8_0)."""
    def s(v: str) -> bytes:
        b = v.encode("utf-8")
        return struct.pack("<Q", len(b)) + b

    def val(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<I?", 7, v)
        if isinstance(v, int):
            return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v) if v < (1 << 32) else struct.pack("<IQ", 10, v)
        if isinstance(v, float):
            return struct.pack("<If", 6, v)
        if isinstance(v, str):
            return struct.pack("<I", 8) + s(v)
        if isinstance(v, (list, tuple)):
            body = b"".join(val(e)[4:] for e in v)
            et = struct.unpack("<I", val(v[0])[:4])[0] if v else 4
            return struct.pack("<IIQ", 9, et, len(v)) + body
        raise TypeError(f"metadata value {v!r}")

    kv = dict(kv)
    kv.setdefault("general.alignment", alignment)
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv))
    for k, v in kv.items():
        head += s(k) + val(v)
    blobs, infos, off = [], b"", 0
    for name, (t, gt) in tensors.items():
        a = t.detach().float().cpu().numpy()
        if gt == GGML_F32:
            raw = a.astype(np.float32).tobytes()
        elif gt == GGML_F16:
            raw = a.astype(np.float16).tobytes()
        elif gt == GGML_BF16:
            raw = t.detach().to(torch.bfloat16).cpu().view(torch.int16).numpy().tobytes()
        elif gt == GGML_Q8_0:
            raw = quantize_q8_0(a).tobytes()
        else:
            raise ValueError(f"cannot write ggml type {gt}")
        ne = tuple(reversed(a.shape))
        infos += s(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne) + struct.pack("<IQ", gt, off)
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    pre = head + infos
    pre += b"\0" * ((-len(pre)) % alignment)
    with open(path, "wb") as f:
        f.write(pre)
        for b in blobs:
            f.write(b)
