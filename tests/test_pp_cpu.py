"""Pipeline stage plans, the checksummed file hand-off and the same-process stage walk on the oracle model."""
import os

import pytest
import torch

from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.reference_model import ReferenceModel, ReferenceSequence
from ninfer_fusion_b200.models.weights import random_weights
from ninfer_fusion_b200.ops import reference as R
from ninfer_fusion_b200.parallel.pp import (StagePlan, StagePlanError, fnv1a64, read_handoff, stage_walk_reference,
                                            write_handoff)


def test_stage_plan_grammar():
    p = StagePlan.parse("0-31,32-63", 64)
    assert p.stages == ((0, 32), (32, 64)) and p.world == 2 and p.uniform and not p.is_identity
    assert p.spec() == "0-31,32-63"
    assert StagePlan.parse("0-63", 64).is_identity
    assert not StagePlan.parse("0-9,10-63", 64).uniform
    for bad in ("", "0-31;32-63", "0-31,33-63", "0-31,32-62", "5-3,6-63", "a-b", "0-31,31-63", "0-31,32-64"):
        with pytest.raises(StagePlanError):
            StagePlan.parse(bad, 64)
    b = StagePlan.balanced(64, 4, interval=4)
    assert b.stages == ((0, 16), (16, 32), (32, 48), (48, 64))
    b3 = StagePlan.balanced(64, 3, interval=4)
    assert b3.stages[0][0] == 0 and b3.stages[-1][1] == 64 and all(a % 4 == 0 for a, _ in b3.stages)
    with pytest.raises(StagePlanError):
        StagePlan.balanced(4, 5)


def test_handoff_file_roundtrip_and_checks(tmp_path):
    d = str(tmp_path)
    x = torch.randn(7, 256)
    write_handoff(d, 0, x)
    y = read_handoff(d, 0, 7, 256)
    assert torch.equal(y, x.to(torch.bfloat16))
    with pytest.raises(StagePlanError):
        read_handoff(d, 0, 8, 256)                      # wrong shape
    with pytest.raises(StagePlanError):
        read_handoff(d, 1, 7, 256)                      # missing boundary
    path = os.path.join(d, "stage_0.bin")
    blob = bytearray(open(path, "rb").read())
    blob[40] ^= 0xFF
    open(path, "wb").write(bytes(blob))
    with pytest.raises(StagePlanError):
        read_handoff(d, 0, 7, 256)                      # corrupted payload
    assert fnv1a64(b"") == 0xCBF29CE484222325 and fnv1a64(b"a") == 0xAF63DC4C8601EC8C


def test_stage_walk_matches_the_plain_forward(tmp_path):
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=5, std=0.05)
    model = ReferenceModel(cfg, w)
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (19,))
    nxt = torch.randint(0, cfg.vocab, (1,))
    full_seq = ReferenceSequence(cfg, R.KV_BF16)
    h_full = model.forward(full_seq, ids)
    h_full2 = model.forward(full_seq, nxt)
    for spec, use_files in (("0-3", False), ("0-1,2-3", False), ("0-0,1-2,3-3", True)):
        plan = StagePlan.parse(spec, cfg.n_layers)
        seq = ReferenceSequence(cfg, R.KV_BF16)
        d = str(tmp_path / spec.replace(",", "_")) if use_files else None
        h = stage_walk_reference(model, seq, ids, plan, d)
        assert torch.equal(h, h_full), spec
        assert seq.n_tokens == 19
        assert torch.equal(stage_walk_reference(model, seq, nxt, plan, d), h_full2)   # caches continue across stages
    # negative control: with the writes cut, the next stage has nothing valid to read
    plan = StagePlan.parse("0-1,2-3", cfg.n_layers)
    with pytest.raises(StagePlanError):
        stage_walk_reference(model, ReferenceSequence(cfg, R.KV_BF16), ids, plan, str(tmp_path / "cut"), cut=True)
