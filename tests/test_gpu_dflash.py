"""DFlash drafter on the GPU: the native context append + one-pass block proposal against the dense fp32 oracle fed
with the same tapped features, and draft-verify generation with it against plain greedy decoding."""
import pytest
import torch

from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.dflash import DFlashConfig, DFlashReference, random_dflash_weights
from ninfer_fusion_b200.models.weights import random_weights

pytestmark = pytest.mark.gpu


def _build(dc, K, B=2, ctx=160):
    from ninfer_fusion_b200.runtime.speculative import SpeculativeGenerator
    cfg, dev = TINY_DENSE, torch.device("cuda")
    w = random_weights(cfg, dev, seed=0, std=0.05)
    w.update(random_dflash_weights(cfg, dc, w, dev, seed=5, std=0.05))
    spec = SpeculativeGenerator(cfg, w, dev, max_batch=B, max_context=ctx, draft_tokens=K, drafter="dflash",
                                kv_format="bf16", page_size=16, prefill_chunk=64, dflash_config=dc)
    return cfg, w, spec


@pytest.mark.parametrize("dc", [DFlashConfig(n_layers=2, window=0, mask_token=3),
                                DFlashConfig(n_layers=2, local_layers=1, window=16, mask_token=3)])
def test_proposal_pass_matches_the_oracle_on_the_same_features(dc):
    K = 4
    cfg, w, spec = _build(dc, K)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (70, 37)]   # 70 > one prefill chunk
    seen = {0: [], 1: []}
    inner = spec.dflash.append_context

    def record(features, table_row, positions, row_ends):
        f, r = features.float().cpu(), table_row.cpu().tolist()
        for i, row in enumerate(r):
            seen[row].append(f[i])
        inner(features, table_row, positions, row_ends)
    spec.dflash.append_context = record
    first = spec.prefill(prompts)
    assert [len(seen[b]) for b in (0, 1)] == [70, 37]                 # every prompt position became draft context
    lg = spec.dflash.logits(spec.rows, first, spec.lengths).float().cpu()
    for b in (0, 1):
        ref = DFlashReference(cfg, dc, w)
        ref.append_context(torch.stack(seen[b]))
        want = ref.logits(first[b], K)
        scale = want.abs().max().item()
        err = (lg[b] - want).abs().max().item()
        assert err < 0.03 * max(1.0, scale), f"sequence {b}: {err} of {scale}"


def test_generation_with_the_drafter_equals_plain_greedy_decoding():
    from ninfer_fusion_b200.runtime.generator import Generator
    dc, K = DFlashConfig(n_layers=2, local_layers=1, window=32, mask_token=3), 3
    cfg, w, spec = _build(dc, K, B=3, ctx=200)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (25, 64, 9)]
    plain = Generator(cfg, w, torch.device("cuda"), max_batch=3, max_context=200, kv_format="bf16", page_size=16,
                      prefill_chunk=64, use_graph=False)
    want = plain.generate(prompts, 24)
    got = spec.generate(prompts, 24)
    assert got == want
    assert spec.rounds > 0 and spec.dflash.proposals == spec.rounds and 1.0 <= spec.tokens_per_round <= K + 1
    # the draft context follows the committed tokens: one context row per cache position of every sequence
    assert spec.lengths == [len(p) + len(o) - 1 for p, o in zip(prompts, [spec.history[b][len(prompts[b]):] for b in range(3)])]
