"""K row-scale loop on the CPU: solver, side-file format and refusals, oracle invariance of the attention scores."""
import struct

import pytest
import torch

from ninfer_fusion_b200.kv import rowscale as RS
from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.reference_model import ReferenceModel, ReferenceSequence
from ninfer_fusion_b200.models.weights import random_weights
from ninfer_fusion_b200.ops import reference as R


def _loud_rows(n=512, D=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((n, D), generator=g)
    x[:, 5] *= 12.0
    x[:, 77] *= 5.0
    x[:, 130] *= 0.05
    return x


def test_solver_respects_bounds_and_flattens_rows():
    x = _loud_rows()
    s = RS.solve_row_scale(x)
    assert s.shape == (256,) and float(s.min()) >= 0.5 and float(s.max()) <= 2.0
    assert s[5] == 0.5 and s[77] == 0.5 and s[130] == 2.0         # loud channels pushed down, the quiet one up
    free = (s > 0.5) & (s < 2.0)
    assert free.sum() > 240
    rms = (x * s).pow(2).mean(0).sqrt()
    assert float(rms[free].max() / rms[free].min()) < 1.02        # free channels are equalised (bf16 rounding of s)
    assert RS.balance_gain(x, s) > 3.5
    # already balanced rows: nothing to do
    flat = torch.randn((2048, 64), generator=torch.Generator().manual_seed(1))
    s2 = RS.solve_row_scale(flat)
    assert float((s2 - 1).abs().max()) < 0.1


def test_table_roundtrip_and_refusals(tmp_path):
    path = str(tmp_path / "t.kvrowscale.bin")
    scales = torch.stack([RS.solve_row_scale(_loud_rows(seed=i)) for i in range(6)]).reshape(3, 2, 256)
    RS.write_table(path, scales, tag="unit", model_hash=0x1234)
    t = RS.read_table(path)
    assert t.geometry == (3, 2, 256) and not t.identity and t.tag == "unit" and t.model_hash == 0x1234
    assert torch.equal(t.scales.float(), scales)
    RS.validate(t, 3, 2, 256, model_hash=0x1234)
    for args, field in (((4, 2, 256), "layers"), ((3, 4, 256), "kv_heads"), ((3, 2, 128), "head_dim")):
        with pytest.raises(RS.RowScaleError, match=field):
            RS.validate(t, *args)
    with pytest.raises(RS.RowScaleError, match="model_hash"):
        RS.validate(t, 3, 2, 256, model_hash=0x9999)
    raw = bytearray(open(path, "rb").read())
    bad = bytearray(raw); bad[RS.HEADER_BYTES + 3] ^= 0x01
    open(path, "wb").write(bad)
    with pytest.raises(RS.RowScaleError, match="crc32"):
        RS.read_table(path)
    bad = bytearray(raw); bad[0] = ord("X")
    open(path, "wb").write(bad)
    with pytest.raises(RS.RowScaleError, match="magic"):
        RS.read_table(path)
    open(path, "wb").write(raw[:-2])
    with pytest.raises(RS.RowScaleError, match="payload"):
        RS.read_table(path)
    with pytest.raises(RS.RowScaleError, match=r"\[0.5, 2.0\]"):
        RS.write_table(path, torch.full((1, 1, 16), 3.0))


def test_identity_tables(tmp_path):
    path = str(tmp_path / "id.bin")
    RS.write_table(path, torch.ones((2, 1, 256)), identity=True)
    t = RS.read_table(path)
    assert t.identity
    RS.validate(t, 16, 1, 256)                                   # an identity table may cover fewer layers
    with pytest.raises(RS.RowScaleError, match="layers"):
        RS.validate(t, 1, 1, 256)

    class M:
        k_row_scale = {}
        device = "cpu"
    assert RS.load_into(M, t, [3, 7]) == 0 and M.k_row_scale == {}
    with pytest.raises(RS.RowScaleError, match="identity flag"):
        RS.write_table(path, torch.full((1, 1, 16), 1.5), identity=True)
    # flag says identity, payload does not
    raw = bytearray(open(path, "rb").read())
    raw[RS.HEADER_BYTES:RS.HEADER_BYTES + 2] = struct.pack("<H", 0x3FC0)
    import zlib
    raw[36:40] = struct.pack("<I", zlib.crc32(bytes(raw[RS.HEADER_BYTES:])) & 0xFFFFFFFF)
    open(path, "wb").write(raw)
    with pytest.raises(RS.RowScaleError, match="identity table"):
        RS.read_table(path)


def test_oracle_scores_are_preserved_and_nvfp4_error_drops():
    """With bf16 KV the row scale changes nothing but rounding; with nvfp4 KV and loud K channels it lowers the
    attention-output error against the bf16-KV run."""
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=3, std=0.05)
    # make a few K channels loud through the k_norm weight (the norm's (1 + w) factor)
    kn = [k for k in w if k.endswith("attn/k_norm")]
    for name in kn:
        w[name] = w[name].clone()
        w[name][[4, 9, 100]] = 15.0
    model = ReferenceModel(cfg, w)
    toks = torch.randint(0, cfg.vocab, (48,), generator=torch.Generator().manual_seed(0))

    def run(fmt, scales):
        seq = ReferenceSequence(cfg, fmt)
        seq.k_row_scale = scales
        return model.logits(model.forward(seq, toks)[-4:])

    # sample K of every attention layer from a bf16 run to solve the tables
    seq = ReferenceSequence(cfg, R.KV_BF16)
    model.forward(seq, toks)
    tables = {ai: torch.stack([RS.solve_row_scale(seq.k[ai][:, h]) for h in range(cfg.n_kv_heads)])
              for ai in range(len(cfg.attn_layers))}
    assert all(float(t.min()) == 0.5 for t in tables.values())
    base = run(R.KV_BF16, {})
    same = run(R.KV_BF16, tables)
    assert (same - base).abs().max() < 0.03 * base.abs().max()
    err_plain = (run(R.KV_NVFP4, {}) - base).pow(2).mean().sqrt()
    err_scaled = (run(R.KV_NVFP4, tables) - base).pow(2).mean().sqrt()
    assert err_scaled < err_plain
