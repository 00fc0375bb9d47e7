"""DFlash draft model, CPU side: weight set, the dense oracle's block semantics (one pass, bidirectional inside the
block, sliding window on the local layers) and the feature plumbing."""
import torch

from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.dflash import (DFlashConfig, DFlashReference, draft_model_config, random_dflash_weights,
                                              reference_features)
from ninfer_fusion_b200.models.weights import random_weights


def _setup(dc, seed=0):
    cfg = TINY_DENSE
    w = random_weights(cfg, "cpu", seed=seed, std=0.05)
    w.update(random_dflash_weights(cfg, dc, w, "cpu", seed=seed + 3, std=0.05))
    return cfg, w


def _features(cfg, dc, n, seed):
    g = torch.Generator().manual_seed(seed)
    F = len(dc.resolved(cfg).feature_layers)
    return reference_features([torch.randn(n, cfg.hidden, generator=g) for _ in range(F)])


def test_weight_set_shares_the_targets_embedding_and_head():
    dc = DFlashConfig(n_layers=2, window=0)
    cfg, w = _setup(dc)
    d = draft_model_config(cfg, dc.resolved(cfg))
    assert d.n_layers == 2 and d.gdn_layers == [] and d.attn_layers == [0, 1]
    assert w["dflash/embed"] is w["text/embed"] and w["dflash/lm_head"] is w["text/lm_head"]
    F = len(dc.resolved(cfg).feature_layers)
    assert w["dflash/feature_proj"].shape == (cfg.hidden, F * cfg.hidden)
    assert w["dflash/layers/1/ctx_kv"].shape == (2 * cfg.kv_dim, cfg.hidden)
    assert "dflash/layers/0/attn/in_proj" in w and "dflash/final_norm" in w


def test_block_is_proposed_in_one_pass_and_is_bidirectional():
    dc = DFlashConfig(n_layers=2, window=0, mask_token=5)
    cfg, w = _setup(dc)
    ref = DFlashReference(cfg, dc, w)
    ref.append_context(_features(cfg, dc, 40, 1))
    a = ref.logits(anchor=17, K=4)
    assert a.shape == (4, cfg.vocab) and ref.n_context == 40          # proposing does not touch the context
    assert ref.propose(17, 4) == [int(t) for t in a.argmax(-1)]
    # not causal inside the block: a different token at the LAST position changes the FIRST position's logits
    other = DFlashReference(cfg, DFlashConfig(n_layers=2, window=0, mask_token=9), w)
    other.k, other.v = [k.clone() for k in ref.k], [v.clone() for v in ref.v]
    b = other.logits(anchor=17, K=4)
    assert (a[0] - b[0]).abs().max().item() > 1e-3
    # and the anchor matters to every row
    c = ref.logits(anchor=18, K=4)
    assert all((a[i] - c[i]).abs().max().item() > 1e-3 for i in range(4))


def test_local_layers_forget_context_beyond_their_window():
    dc = DFlashConfig(n_layers=1, local_layers=1, window=16)
    cfg, w = _setup(dc)
    long, short = DFlashReference(cfg, dc, w), DFlashReference(cfg, dc, w)
    f = _features(cfg, dc, 60, 2)
    long.append_context(f)
    # the same last 16 context rows at the same positions, everything older replaced
    g = f.clone()
    g[:40] = _features(cfg, dc, 40, 3)
    short.append_context(g)
    K = 4
    assert torch.equal(long.logits(3, K), short.logits(3, K))        # keys before 60 + 4 - 16 = 48 are invisible
    full = DFlashReference(cfg, DFlashConfig(n_layers=1, window=0), w)
    full2 = DFlashReference(cfg, DFlashConfig(n_layers=1, window=0), w)
    full.append_context(f)
    full2.append_context(g)
    assert not torch.equal(full.logits(3, K), full2.logits(3, K))     # a full-context layer does see them
