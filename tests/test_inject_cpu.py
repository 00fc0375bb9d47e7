"""The tensor ingress: an injected embed(t) reproduces the token prompt bit for bit; other rows change the output;
malformed payloads are refused."""
import base64

import pytest
import torch

from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.weights import random_weights
from ninfer_fusion_b200.runtime import inject as I
from ninfer_fusion_b200.runtime.engine import Engine, RequestError, RequestOptions
from ninfer_fusion_b200.runtime.program import ReferenceProgram


def _payload(rows, cols, dtype="bf16", scale=1.0):
    return {"dtype": dtype, "scale": scale, "columns": list(cols), "data": base64.b64encode(I.encode_rows(rows, dtype)).decode()}


def test_wire_round_trip_and_refusals():
    rows = (torch.randn(3, 8) * 2).to(torch.bfloat16)
    got = I.decode_rows("bf16", I.encode_rows(rows), 3, 8)
    assert torch.equal(got.view(torch.int16), rows.view(torch.int16))              # the identity: same 16-bit words
    f32 = I.decode_rows("f32", I.encode_rows(rows, "f32"), 3, 8, scale=0.5)
    assert torch.equal(f32, (rows.float() * 0.5).to(torch.bfloat16))
    f16 = I.decode_rows("f16", I.encode_rows(rows, "f16"), 3, 8)
    assert torch.allclose(f16.float(), rows.float(), rtol=1e-2)
    ids = list(range(10, 20))
    ok = I.parse_injection(_payload(rows, [1, 4, 9]), ids, 8)
    assert ok.embed_rows.tolist() == [1, 4, 9] and ok.positions.shape == (10, 3) and ok.rope_delta == 0 and not ok.items
    bad_nan = rows.clone()
    bad_nan[0, 0] = float("nan")
    for payload, why in ((_payload(rows, [4, 1, 9]), "ascending"), (_payload(rows, [1, 4, 10]), "inside"),
                         (_payload(rows, [1, 4]), "bytes"), (_payload(bad_nan, [1, 4, 9]), "NaN"),
                         (_payload(rows, [1, 4, 9], scale=0.0), "scale"), (_payload(rows, [1, 4, 9], scale=float("inf")), "scale"),
                         ({**_payload(rows, [1, 4, 9]), "dtype": "fp8"}, "dtype"), ({**_payload(rows, [1, 4, 9]), "extra": 1}, "unknown"),
                         ({**_payload(rows, [1, 4, 9]), "data": "@@"}, "base64"), ({**_payload(rows, [1, 4, 9]), "columns": [1, 4, True]}, "integers"),
                         (_payload(rows.float() * 1e36, [1, 4, 9], dtype="f32", scale=1e3), "overflow")):
        with pytest.raises(I.InjectRefused, match=why):
            I.parse_injection(payload, ids, 8)


def test_injecting_the_gathered_rows_reproduces_the_token_prompt_and_other_rows_do_not():
    cfg = TINY_DENSE.shrink(2)
    w = random_weights(cfg, "cpu", seed=7, std=0.05)
    eng = Engine(lambda: ReferenceProgram(cfg, w, max_lanes=2, max_context=256), prefill_chunk=8)   # several prefill chunks
    try:
        ids = list(range(30, 60))
        plain = eng.submit(ids, RequestOptions(max_tokens=8)).wait(timeout=120)
        cols = [0, 7, 8, 15, 29]                                    # across chunk edges, first and last column
        embed = eng.program.model.w["text/embed"]
        rows = embed[torch.tensor([ids[c] for c in cols])].to(torch.bfloat16)
        scrambled = list(ids)
        for c in cols:
            scrambled[c] = 5                                         # the token under an injected column does not matter
        same = I.parse_injection(_payload(rows, cols), scrambled, cfg.hidden)
        assert eng.submit(scrambled, RequestOptions(max_tokens=8, media=same)).wait(timeout=120) == plain
        assert eng.submit(scrambled, RequestOptions(max_tokens=8)).wait(timeout=120) != plain
        other = I.parse_injection(_payload(torch.flip(rows, dims=[0]) * 3, cols), scrambled, cfg.hidden)
        assert eng.submit(scrambled, RequestOptions(max_tokens=8, media=other)).wait(timeout=120) != plain
        with pytest.raises(RequestError, match="does not match"):
            eng.submit(ids, RequestOptions(max_tokens=4, media=same))
    finally:
        eng.shutdown()


def test_the_service_takes_a_payload_with_prompt_ids_and_programs_without_the_channel_refuse():
    from ninfer_fusion_b200 import cli
    from ninfer_fusion_b200.frontend.tokenizer import Tokenizer
    from ninfer_fusion_b200.models import packages
    from ninfer_fusion_b200.models.all_attention import random_package_weights
    from ninfer_fusion_b200.runtime.program import PackageProgram
    from ninfer_fusion_b200.serve.service import GenerationService, GenRequest
    from ninfer_fusion_b200.serve.service import RequestError as ServiceRequestError
    tok = Tokenizer.train_toy(cli.DEFAULT_CORPUS, 200, cli.SPECIAL_TOKENS)
    cfg = TINY_DENSE.shrink(2)
    w = random_weights(cfg, "cpu", seed=7, std=0.05)
    eng = Engine(lambda: ReferenceProgram(cfg, w, max_lanes=2, max_context=256), prefill_chunk=16)
    svc = GenerationService(eng, tok, "m", max_concurrent=2, queue_timeout_s=20.0)
    try:
        ids = list(range(30, 50))
        rows = eng.program.model.w["text/embed"][torch.tensor([ids[3], ids[4]])].to(torch.bfloat16)
        plain = svc.generate(GenRequest(prompt_ids=ids, max_tokens=6, temperature=0.0))
        inj = svc.generate(GenRequest(prompt_ids=ids, max_tokens=6, temperature=0.0, inject=_payload(rows, [3, 4])))
        assert inj.token_ids == plain.token_ids and inj.finish_reason == plain.finish_reason
        for bad in (GenRequest(prompt="text", inject=_payload(rows, [3, 4])), GenRequest(prompt_ids=ids, inject=_payload(rows, [3]))):
            with pytest.raises(ServiceRequestError):
                svc.prepare_full(bad)
    finally:
        eng.shutdown()
    pkg = packages.construct_oracle("spark-x2.5-4b", layers=2, vocab=256, hidden_div=8)
    eng2 = Engine(lambda: PackageProgram(pkg, random_package_weights(pkg, seed=1), max_lanes=2, max_context=128), prefill_chunk=16)
    try:
        rows2 = torch.zeros(1, pkg.hidden, dtype=torch.bfloat16)
        with pytest.raises(RequestError, match="does not accept"):
            eng2.submit([1, 2, 3], RequestOptions(max_tokens=2, media=I.build_injected_prompt([1, 2, 3], [1], rows2, pkg.hidden)))
    finally:
        eng2.shutdown()
