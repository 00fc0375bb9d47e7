"""`.ninfer` v2 container: layout byte rules, round trips and schema refusals (CPU)."""
import json
import struct

import numpy as np
import pytest
import torch

from ninfer_fusion_b200.artifact import layouts as L
from ninfer_fusion_b200.artifact.container import (MAGIC, ArtifactError, ArtifactReader, ArtifactWriter,
                                                   parse_directory, rank_artifact_name)


def test_encoded_sizes_match_the_documented_examples():
    # Q5 [2,130]: K_pad 256, 4 groups/row, base 256, high 64, scale 16 -> 528
    assert L.encoded_size("Q5G64_F16S", "row-split-k128-v1", [2, 130]) == 528
    assert L.encoded_size("NVFP4", "blockscale-k16-m128x4-v1", [128, 64]) == 4096 + 512 + 4
    assert L.encoded_size("FP8_E4M3FN_ROW_BF16S", "row-scale-v1", [3, 100]) == 512 + 6
    assert L.encoded_size("BF16", "contiguous-le-v1", [4, 5]) == 40
    with pytest.raises(ValueError):
        L.encoded_size("NVFP4", "blockscale-k16-m128x4-v1", [100, 64])
    with pytest.raises(ValueError):
        L.encoded_size("BF16", "row-scale-v1", [4, 4])


def test_nvfp4_scale_swizzle_is_a_permutation_and_matches_formula():
    N, K = 256, 128
    n, g = np.meshgrid(np.arange(N), np.arange(K // 16), indexing="ij")
    off = L.nvfp4_scale_offset(n, g, K)
    assert sorted(off.flatten().tolist()) == list(range(N * K // 16))
    # row 33 (tile 0, inner 33), group 5 -> scale tile 1, lane 1
    assert L.nvfp4_scale_offset(np.array(33), np.array(5), K) == (0 * 2 + 1) * 512 + (33 % 32) * 16 + (33 // 32) * 4 + 1


@pytest.mark.parametrize("fmt", ["Q4G64_F16S", "Q5G64_F16S", "Q6G64_F16S", "W8G32_F16S"])
def test_row_split_round_trip(fmt):
    rng = np.random.default_rng(0)
    w = rng.standard_normal((5, 200)).astype(np.float32)
    codes, scale = L.quantize_group_int(w, fmt)
    payload = L.encode_row_split(codes, scale, fmt, 200)
    assert len(payload) == L.encoded_size(fmt, "row-split-k128-v1", [5, 200])
    c2, s2 = L.decode_row_split(payload, fmt, [5, 200])
    assert np.array_equal(c2, codes.astype(np.int16)) and np.array_equal(s2, scale)
    deq = L.dequant_row_split(c2, s2, fmt, 200)
    qmax = L.GROUP_FORMATS[fmt][4]
    assert np.abs(deq - w).max() <= np.abs(w).max() / qmax * 0.51 + 1e-3
    # physical padding decodes to zero and wholly physical groups have a zero scale
    assert (c2[:, 200:] == 0).all()


def test_q5_high_plane_bit_order():
    codes = np.zeros((1, 128), dtype=np.int8)
    codes[0, 0] = -16   # u = 0b10000 -> high bit set, low nibble 0
    codes[0, 9] = 15    # high bit clear
    codes[0, 10] = -1   # u = 0b11111
    scale = np.ones((1, 2), dtype=np.float16)
    p = L.encode_row_split(codes, scale, "Q5G64_F16S", 128)
    high_off = L.align_up(1 * 2 * 32, 256)
    assert p[high_off] == 0b00000001 and p[high_off + 1] == 0b00000100
    assert p[4] == 0xF0 and p[5] == 0x0F  # byte 4 = lanes 8 (low nibble, 0) and 9; byte 5 = lanes 10 and 11


def test_nvfp4_fp8_round_trips():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((128, 192)).astype(np.float32) * 0.05
    codes, sw, d_w = L.quantize_nvfp4(w)
    payload = L.encode_nvfp4(codes, sw, d_w)
    c2, s2, d2 = L.decode_nvfp4(payload, [128, 192])
    assert np.array_equal(c2, codes) and np.array_equal(s2, sw) and d2 == d_w
    deq = L.dequant_nvfp4(c2, s2, d2)
    assert np.abs(deq - w).mean() < 0.1 * np.abs(w).mean() + 1e-4
    cw, sc = L.quantize_fp8_row(w)
    c3, s3 = L.decode_fp8_row(L.encode_fp8_row(cw, sc), [128, 192])
    assert np.array_equal(c3, cw) and np.array_equal(s3, sc)
    assert np.abs(L.dequant_fp8_row(c3, s3) - w).max() < 0.07 * np.abs(w).max()
    cb, sb = L.quantize_fp8_block128(w)
    c4, s4 = L.decode_fp8_block128(L.encode_fp8_block128(cb, sb), [128, 192])
    assert np.array_equal(c4, cb) and np.array_equal(s4, sb) and s4.shape == (1, 2)
    assert np.abs(L.dequant_fp8_block128(c4, s4) - w).max() < 0.07 * np.abs(w).max()


def test_container_round_trip_and_framing(tmp_path):
    torch.manual_seed(0)
    path = str(tmp_path / "m.ninfer")
    w = ArtifactWriter("tiny-dense", "bf16")
    t1 = torch.randn(7, 33).to(torch.bfloat16)
    t2 = torch.randn(128, 128) * 0.1
    w.add_resource("frontend/tokenizer.json", b'{"model": {}}')
    w.add_tensor("text/a", t1, "BF16")
    w.add_tensor("text/b", t2, "NVFP4")
    w.add_tensor("text/c", t2, "Q4G64_F16S")
    w.add_tensor("text/idx", torch.arange(5, dtype=torch.int32), "I32")
    w.write(path)
    raw = open(path, "rb").read()
    assert raw[:8] == MAGIC
    (jb,) = struct.unpack("<Q", raw[8:16])
    doc = json.loads(raw[16:16 + jb])
    assert set(doc) == {"identity", "objects"} and doc["objects"][1]["offset"] % 256 == 0
    with ArtifactReader(path) as r:
        assert r.identity == ("tiny-dense", "bf16") and r.payload_offset % 4096 == 0
        assert torch.equal(r.tensor("text/a"), t1)
        assert r.resource("frontend/tokenizer.json") == b'{"model": {}}'
        assert (r.tensor("text/b") - t2).abs().mean() < 0.02
        assert (r.tensor("text/c") - t2).abs().max() < 0.05
        assert r.tensor("text/idx").tolist() == [0, 1, 2, 3, 4]


def test_schema_refusals():
    good = {"identity": {"model_id": "m", "weights_id": "w"},
            "objects": [{"name": "t", "kind": "tensor", "shape": [2, 2], "format": "BF16",
                         "layout": "contiguous-le-v1", "offset": 0, "bytes": 8}]}
    parse_directory(good)

    def broken(mut):
        d = json.loads(json.dumps(good))
        mut(d)
        with pytest.raises(ArtifactError):
            parse_directory(d)

    broken(lambda d: d.update(extra=1))
    broken(lambda d: d["identity"].update(model_id=""))
    broken(lambda d: d["objects"][0].update(bytes=9))
    broken(lambda d: d["objects"][0].update(offset=8))
    broken(lambda d: d["objects"][0].update(format="FP16"))
    broken(lambda d: d["objects"][0].update(shape=[2, True]))
    broken(lambda d: d["objects"][0].update(note="x"))
    broken(lambda d: d["objects"].append(dict(d["objects"][0])))
    broken(lambda d: d.update(objects=[]))
    assert rank_artifact_name("a/b.ninfer", 1, 4) == "a/b.tp1of4.ninfer"
