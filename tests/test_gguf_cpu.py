"""GGUF import: block-quant decoders against scalar re-statements of the ggml structs, container round trip, and the
full path GGUF -> engine inventory for the tiny hybrid geometry."""
import struct

import numpy as np
import pytest
import torch

from ninfer_fusion_b200 import cli
from ninfer_fusion_b200.artifact.container import ArtifactReader
from ninfer_fusion_b200.convert import gguf as G
from ninfer_fusion_b200.convert import hf
from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.weights import random_weights


def _half(x):
    return np.array([x], dtype=np.float16).view(np.uint8)


def test_q4_k_decoder_matches_scalar_definition():
    rng = np.random.default_rng(0)
    blk = rng.integers(0, 256, 144, dtype=np.uint8)
    blk[0:2], blk[2:4] = _half(0.0123), _half(0.0071)
    d, dmin = float(np.float16(0.0123)), float(np.float16(0.0071))
    s, qs = blk[4:16].astype(int), blk[16:144].astype(int)

    def scale_min(j):
        if j < 4:
            return s[j] & 63, s[j + 4] & 63
        return (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4), (s[j + 4] >> 4) | ((s[j] >> 6) << 4)

    want, q, is_ = [], 0, 0
    for _ in range(4):
        sc1, m1 = scale_min(is_)
        sc2, m2 = scale_min(is_ + 1)
        want += [d * sc1 * (qs[q + l] & 0xF) - dmin * m1 for l in range(32)]
        want += [d * sc2 * (qs[q + l] >> 4) - dmin * m2 for l in range(32)]
        q += 32
        is_ += 2
    got = G.dequant_q4_k(np.concatenate([blk, blk]), 512)
    assert np.allclose(got[:256], np.array(want, dtype=np.float32), rtol=1e-6, atol=1e-7)
    assert np.array_equal(got[:256], got[256:])


def test_q6_k_decoder_matches_scalar_definition():
    rng = np.random.default_rng(1)
    blk = rng.integers(0, 256, 210, dtype=np.uint8)
    blk[208:210] = _half(0.0031)
    d = float(np.float16(0.0031))
    ql, qh = blk[:128].astype(int), blk[128:192].astype(int)
    sc = blk[192:208].view(np.int8).astype(int)
    want = np.zeros(256, dtype=np.float64)
    y = 0
    for half in range(2):
        L, H, S = ql[64 * half:], qh[32 * half:], sc[8 * half:]
        for l in range(32):
            i = l // 16
            q1 = ((L[l] & 0xF) | (((H[l] >> 0) & 3) << 4)) - 32
            q2 = ((L[l + 32] & 0xF) | (((H[l] >> 2) & 3) << 4)) - 32
            q3 = ((L[l] >> 4) | (((H[l] >> 4) & 3) << 4)) - 32
            q4 = ((L[l + 32] >> 4) | (((H[l] >> 6) & 3) << 4)) - 32
            want[y + l], want[y + l + 32] = d * S[i] * q1, d * S[i + 2] * q2
            want[y + l + 64], want[y + l + 96] = d * S[i + 4] * q3, d * S[i + 6] * q4
        y += 128
    got = G.dequant_q6_k(blk.copy(), 256)
    assert np.allclose(got, want.astype(np.float32), rtol=1e-6, atol=1e-7)


def test_q8_0_and_q4_0_roundtrip():
    rng = np.random.default_rng(2)
    x = rng.standard_normal(320).astype(np.float32)
    deq = G.dequant_q8_0(G.quantize_q8_0(x), 320)
    assert np.abs(deq - x).max() <= np.abs(x).max() / 127 * 0.51 + 1e-3
    blk = np.zeros(18, dtype=np.uint8)
    blk[0:2] = _half(0.5)
    blk[2:] = np.arange(16, dtype=np.uint8) | ((15 - np.arange(16, dtype=np.uint8)) << 4)
    got = G.dequant_q4_0(blk, 32)
    assert np.allclose(got[:16], (np.arange(16) - 8) * 0.5) and np.allclose(got[16:], (15 - np.arange(16) - 8) * 0.5)
    assert G.tensor_nbytes(G.GGML_Q4_K, 512) == 288 and G.tensor_nbytes(G.GGML_Q6_K, 256) == 210
    with pytest.raises(ValueError):
        G.tensor_nbytes(G.GGML_Q4_K, 100)


def _export_tiny(path, cfg, w):
    """The tiny model as a llama.cpp-style GGUF: reversed dims, -exp(A_log), 1 + w norms, [kernel, channels] conv."""
    t = hf.weights_to_hf(cfg, w)
    main = cfg.n_layers
    rev = {}
    for rx, target in G._RULES:
        rev[target] = rx
    tensors = {}
    for name, ten in t.items():
        if name.startswith("model.language_model.layers.") or name.startswith("mtp.layers."):
            parts = name.split(".")
            if name.startswith("mtp.layers."):
                i, rest = main + int(parts[2]), ".".join(parts[3:])
            else:
                i, rest = int(parts[3]), ".".join(parts[4:])
            pat = rev["{p}" + rest]
            gname = pat.strip("^$").replace("\\.", ".").replace("(\\d+)", str(i))
        else:
            pat = rev[name]
            gname = pat.strip("^$").replace("\\.", ".").replace("\\d+", str(main))
        v = ten.float()
        if name.endswith(".A_log"):
            v = -torch.exp(v)
        elif name.endswith("norm.weight") and not name.endswith("linear_attn.norm.weight"):
            v = v + 1.0
        elif name.endswith("conv1d.weight"):
            v = v[:, 0, :]
        gt = G.GGML_F32 if v.dim() == 1 else (G.GGML_Q8_0 if "ffn_" in gname else G.GGML_BF16)
        tensors[gname] = (v, gt)
    kv = {"general.architecture": "qwen35", "qwen35.block_count": main + 1, "qwen35.nextn_predict_layers": 1,
          "qwen35.embedding_length": cfg.hidden, "qwen35.feed_forward_length": cfg.ffn_inter,
          "qwen35.attention.head_count": cfg.n_q_heads, "qwen35.attention.head_count_kv": cfg.n_kv_heads,
          "qwen35.attention.key_length": cfg.head_dim, "qwen35.rope.dimension_count": cfg.rot_dim,
          "qwen35.rope.freq_base": float(cfg.rope_theta), "qwen35.ssm.group_count": cfg.gdn_qk_heads,
          "qwen35.ssm.time_step_rank": cfg.gdn_v_heads, "qwen35.ssm.state_size": cfg.gdn_head_dim,
          "qwen35.ssm.conv_kernel": cfg.conv_kernel, "qwen35.full_attention_interval": cfg.full_attn_interval,
          "qwen35.context_length": 4096, "qwen35.vocab_size": cfg.vocab, "general.name": "tiny"}
    G.write_gguf(path, kv, tensors)


def test_gguf_to_engine_inventory(tmp_path):
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=9, std=0.05, with_mtp=True)
    path = str(tmp_path / "tiny.gguf")
    _export_tiny(path, cfg, w)
    src = G.GgufSource(path)
    assert (src.main_layers, src.nextn) == (cfg.n_layers, 1) and not src.unmapped
    derived = G.config_from_gguf(src.file.kv)
    assert (derived.n_layers, derived.hidden, derived.ffn_inter, derived.gdn_v_heads, derived.rot_dim) == \
        (cfg.n_layers, cfg.hidden, cfg.ffn_inter, cfg.gdn_v_heads, cfg.rot_dim)
    back = dict(hf.hf_to_weights(cfg, src, with_mtp=True))
    assert set(back) == set(w)
    for k, t in w.items():
        if "mlp/" in k:                                   # Q8_0 payloads: close, not exact
            err = (back[k].float() - t.float()).abs().max().item()
            assert err <= t.float().abs().max().item() / 127 + 2e-3, k
        elif k.endswith("A_log"):
            assert torch.allclose(back[k], t, atol=1e-5), k
        elif "norm" in k and not k.endswith("gdn/norm"):
            assert (back[k].float() - t.float()).abs().max().item() < 1e-2, k   # 1 + w went through fp32 and back to bf16
        else:
            assert torch.equal(back[k], t), k
    art = str(tmp_path / "tiny.ninfer")
    assert cli.main(["convert", path, "--model", "tiny-dense", "--out", art]) == 0
    with ArtifactReader(art) as rd:
        assert torch.equal(rd.tensor("text/embed").to(torch.bfloat16), w["text/embed"])
        assert "mtp/fc" in rd.tensors()
