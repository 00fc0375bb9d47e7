"""Attention-only packages on their fp32 oracle runtime: schedule traits, cache consistency, window, soft cap, Engine."""
from dataclasses import replace

import pytest
import torch

from ninfer_fusion_b200.models import all_attention as AA
from ninfer_fusion_b200.models.packages import FULL, SLIDING, PACKAGES, PackageRefused, construct, construct_oracle, describe
from ninfer_fusion_b200.runtime.engine import Engine, RequestOptions
from ninfer_fusion_b200.runtime.program import PackageProgram


def _small(name, layers):
    return construct_oracle(name, layers=layers, vocab=512, hidden_div=8)


@pytest.mark.parametrize("name,layers", [("spark-x2.5-4b", 4), ("muse-glimmer-30b", 4), ("gemma4-31b", 6)])
def test_incremental_decode_equals_one_pass_and_traits_follow_the_description(name, layers):
    pkg = _small(name, layers)
    w = AA.random_package_weights(pkg, seed=1)
    model = AA.PackageReference(pkg, w)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, pkg.vocab, (24,), generator=g)
    one = model.logits(model.forward(AA.PackageSequence(pkg), ids)[-1:])[0]
    seq = AA.PackageSequence(pkg)
    model.forward(seq, ids[:17])
    for t in ids[17:-1]:
        model.forward(seq, t[None])
    inc = model.logits(model.forward(seq, ids[-1:]))[0]
    assert torch.allclose(one, inc, atol=6e-2, rtol=0) and one[int(inc.argmax())] >= one.max() - 6e-2
    assert seq.n_tokens == 24 and all(k.shape[0] == 24 for k in seq.k)
    kinds = [l.kind for l in pkg.layers]
    assert FULL in kinds and SLIDING in kinds                       # every shrink keeps both kinds of layer
    t = AA.package_traits(pkg)
    if name == "spark-x2.5-4b":
        assert t["headwise_gate"] and t["geglu"] and not t["qk_norm"] and pkg.tie_word_embeddings and "text/lm_head" not in w
        assert w["text/layers/0/attn/gate"].shape == (pkg.layers[0].q_heads, pkg.hidden)
    if name == "muse-glimmer-30b":
        assert t["post_branch_norms"] and t["qk_norm"] and pkg.layers[3].rotary_dim == 0            # a layer without rotation
        assert one.abs().max() < pkg.final_logit_softcap and t["output_multiplier"] == pytest.approx(0.19611613513818404)
    if name == "gemma4-31b":
        full = [i for i, l in enumerate(pkg.layers) if l.kind == FULL][0]
        assert pkg.layers[full].head_dim == 512 and pkg.layers[0].head_dim == 256                    # two head widths
        rot = pkg.layers[full].rotary_dim
        # K shared with V: no value projection; the cached V is the key projection before its rotation
        assert f"text/layers/{full}/attn/v_proj" not in w and torch.equal(seq.k[full][..., rot:], seq.v[full][..., rot:])
        assert not torch.equal(seq.k[full][..., :rot], seq.v[full][..., :rot])
        assert "text/layers/0/attn/v_proj" in w and one.abs().max() < pkg.final_logit_softcap


def test_sliding_window_bounds_what_a_token_can_see_and_rope_is_relative():
    base = construct_oracle("spark-x2.5-4b", layers=3, vocab=256, hidden_div=8)         # three sliding layers
    pkg = replace(base, layers=tuple(replace(l, window=4) for l in base.layers))
    model = AA.PackageReference(pkg, AA.random_package_weights(pkg, seed=2))
    ids = torch.arange(40) % pkg.vocab

    def last(v):
        return model.logits(model.forward(AA.PackageSequence(pkg), v)[-1:])[0]
    ref = last(ids)
    far = ids.clone()
    far[5] = 99                         # 34 positions back: outside 3 layers x (window - 1)
    near = ids.clone()
    near[37] = 99
    assert torch.equal(last(far), ref) and not torch.equal(last(near), ref)
    # rotation encodes distances only: the same tokens at shifted positions give the same logits
    shifted = model.logits(model.forward(AA.PackageSequence(pkg), ids, positions=torch.arange(40) + 1000)[-1:])[0]
    assert torch.allclose(shifted, ref, atol=1e-1, rtol=0) and torch.corrcoef(torch.stack([shifted, ref]))[0, 1] > 0.999


def test_gate_refuses_on_the_gpu_route_and_serves_on_the_oracle_route():
    for name in ("spark-x2.5-4b", "muse-glimmer-30b", "gemma4-31b"):
        with pytest.raises(PackageRefused, match="lacks"):
            construct(name)
        d = describe(name)
        assert not d["servable"] and d["oracle_runtime"] and d["missing"]
        assert construct_oracle(name).n_layers == PACKAGES[name].n_layers
    with pytest.raises(PackageRefused, match="hybrid"):
        construct_oracle("qwen3.6-27b")
    assert construct_oracle("muse-glimmer-30b@8").n_layers == 8


def test_engine_serves_an_attention_only_package_like_its_oracle():
    pkg = _small("muse-glimmer-30b", 4)
    w = AA.random_package_weights(pkg, seed=3)
    prompts = [[5, 9, 2, 7, 11], list(range(20, 50)), [77, 3, 5]]
    want = [AA.PackageReference(pkg, w).generate_greedy(torch.tensor(p), 6) for p in prompts]
    eng = Engine(lambda: PackageProgram(pkg, w, max_lanes=2, max_context=128), prefill_chunk=16)
    try:
        hs = [eng.submit(p, RequestOptions(max_tokens=6, session=f"s{i}")) for i, p in enumerate(prompts)]
        assert [h.wait(timeout=120) for h in hs] == want
        # a second turn of a session continues from the retained frontier
        turn2 = prompts[1] + want[1] + [8, 8]
        h = eng.submit(turn2, RequestOptions(max_tokens=3, session="s1"))
        out = h.wait(timeout=120)
        assert h.cached_tokens > 0 and out == AA.PackageReference(pkg, w).generate_greedy(torch.tensor(turn2), 3)
        assert eng.health()["status"] == "ok"
    finally:
        eng.shutdown()


def test_cli_generates_with_an_attention_only_package_on_the_cpu(capsys):
    from ninfer_fusion_b200 import cli
    assert cli.main(["generate", "--random-init", "--model", "gemma4-31b@6", "--device", "cpu", "--prompt", "hi", "--max-tokens", "3",
                     "--greedy"]) == 0
    err = capsys.readouterr().err
    assert '"completion_tokens": 3' in err and "gemma4-31b@6:random-init" in err
    with pytest.raises(SystemExit, match="GPU runtime lacks"):
        cli.main(["generate", "--random-init", "--model", "spark-x2.5-4b", "--device", "cuda", "--prompt", "hi"])
