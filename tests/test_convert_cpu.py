"""Hugging Face <-> engine weight mapping: exact round trip through safetensors files and the convert CLI."""
import json
import os

import torch

from ninfer_fusion_b200 import cli
from ninfer_fusion_b200.artifact.container import ArtifactReader
from ninfer_fusion_b200.convert import hf
from ninfer_fusion_b200.convert.safetensors_io import SafetensorsSource, write_safetensors
from ninfer_fusion_b200.models import vision as V
from ninfer_fusion_b200.models.config import TINY_DENSE, TINY_MOE
from ninfer_fusion_b200.models.weights import random_weights


def _roundtrip(cfg, tmp_path, with_mtp, vcfg=None):
    w = random_weights(cfg, "cpu", seed=1, std=0.05, with_mtp=with_mtp)
    if vcfg is not None:
        w.update(V.random_vision_weights(vcfg, seed=2))
    hf_tensors = hf.weights_to_hf(cfg, w, vcfg)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, hf_tensors, {"format": "pt"})
    src = SafetensorsSource(path)
    back = dict(hf.hf_to_weights(cfg, src, with_mtp=with_mtp, vision=vcfg))
    src.close()
    assert set(back) == set(w)
    for k in w:
        assert back[k].dtype == w[k].dtype and torch.equal(back[k], w[k]), k
    return hf_tensors


def test_dense_roundtrip_with_draft_and_vision(tmp_path):
    cfg = TINY_DENSE
    vcfg = V.VisionConfig().scaled(1, cfg.hidden)
    t = _roundtrip(cfg, tmp_path, True, vcfg)
    D, H = cfg.head_dim, cfg.n_q_heads
    q = t["model.language_model.layers.3.self_attn.q_proj.weight"]
    assert q.shape == (2 * H * D, cfg.hidden)                       # head-interleaved [query | gate]
    assert t["model.language_model.layers.0.linear_attn.conv1d.weight"].shape == (cfg.gdn_conv_dim, 1, 4)
    assert t["model.visual.patch_embed.proj.weight"].shape == (1152, 3, 2, 16, 16)
    assert "mtp.layers.0.self_attn.q_proj.weight" in t


def test_moe_roundtrip(tmp_path):
    t = _roundtrip(TINY_MOE, tmp_path, False)
    m = TINY_MOE.moe
    assert t["model.language_model.layers.0.mlp.experts.gate_up_proj"].shape == (m.n_experts, 2 * m.expert_inter, TINY_MOE.hidden)
    assert t["model.language_model.layers.0.mlp.shared_expert_gate.weight"].shape == (1, TINY_MOE.hidden)


def test_q_gate_split_is_per_head():
    H, D, hid = 3, 4, 5
    q_proj = torch.arange(H * 2 * D * hid, dtype=torch.float32).view(H * 2 * D, hid)
    q, g = hf._split_q_gate(q_proj, H, D)
    for h in range(H):
        assert torch.equal(q[h * D:(h + 1) * D], q_proj[h * 2 * D:h * 2 * D + D])
        assert torch.equal(g[h * D:(h + 1) * D], q_proj[h * 2 * D + D:(h + 1) * 2 * D])
    assert torch.equal(hf._join_q_gate(q, g, H, D), q_proj)


def test_convert_cli_checkpoint_dir_to_artifact_and_back(tmp_path):
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=4, std=0.05, with_mtp=True)
    ckpt = tmp_path / "ckpt"
    os.makedirs(ckpt)
    tensors = hf.weights_to_hf(cfg, w)
    names = sorted(tensors)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fn, ns in shards.items():
        write_safetensors(str(ckpt / fn), {n: tensors[n] for n in ns})
    with open(ckpt / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": {n: fn for fn, ns in shards.items() for n in ns}}, f)
    with open(ckpt / "config.json", "w") as f:
        json.dump({"text_config": {"num_hidden_layers": cfg.n_layers, "hidden_size": cfg.hidden, "vocab_size": cfg.vocab,
                                   "num_attention_heads": cfg.n_q_heads, "num_key_value_heads": cfg.n_kv_heads,
                                   "head_dim": cfg.head_dim, "partial_rotary_factor": 0.25, "rope_theta": cfg.rope_theta,
                                   "linear_num_key_heads": cfg.gdn_qk_heads, "linear_num_value_heads": cfg.gdn_v_heads,
                                   "intermediate_size": cfg.ffn_inter}}, f)
    derived = hf.config_from_hf(json.load(open(ckpt / "config.json")))
    assert (derived.n_layers, derived.hidden, derived.rot_dim, derived.ffn_inter) == (cfg.n_layers, cfg.hidden, cfg.rot_dim, cfg.ffn_inter)
    art = str(tmp_path / "m.ninfer")
    assert cli.main(["convert", str(ckpt), "--model", "tiny-dense", "--out", art]) == 0
    with ArtifactReader(art) as rd:
        assert rd.identity[0] == "tiny-dense"
        for k, t in w.items():
            assert torch.equal(rd.tensor(k).to(t.dtype), t), k
    back = str(tmp_path / "back.safetensors")
    assert cli.main(["convert", art, "--to-hf", "--out", back]) == 0
    src = SafetensorsSource(back)
    for n in names:
        assert torch.equal(src.tensor(n), tensors[n]), n
    src.close()
