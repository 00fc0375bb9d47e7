"""Speculative options: spellings, width domains, which option needs which backend, resolution against the weights."""
import pytest

from ninfer_fusion_b200.runtime.spec_options import (ADAPTIVE_MAX_WIDTH, SpeculativeOptions, from_strings, parse_backend,
                                                     parse_tree)


def test_backend_spellings():
    assert parse_backend("off") == "none" and parse_backend("NONE") == "none"
    assert parse_backend("dspark") == "dflash" and parse_backend("mtp") == "mtp" and parse_backend("auto") == "auto"
    with pytest.raises(ValueError):
        parse_backend("medusa")


def test_width_domains_and_backend_requirements():
    assert from_strings("mtp", 0).adaptive and from_strings("mtp", 0).width == ADAPTIVE_MAX_WIDTH
    assert not from_strings("mtp", 9).adaptive and from_strings("mtp", 9).width == 9
    for bad in (("mtp", 16), ("dflash", 0), ("dflash", 16), ("none", 3), ("auto", 3)):
        with pytest.raises(ValueError):
            from_strings(*bad)
    with pytest.raises(ValueError):
        from_strings("none", 0, "shortlist")
    with pytest.raises(ValueError):
        from_strings("mtp", 4, "shortlist", "3,4")          # a tree ranks over the full distribution
    with pytest.raises(ValueError):
        from_strings("mtp", 3, "shortlist", None, True)     # sampled drafts export q over the full vocabulary
    with pytest.raises(ValueError):
        from_strings("dflash", 4, "auto", "2,2")
    t = from_strings("mtp", 4, "auto", "3,4")
    assert (t.tree_ranks, t.tree_depths, t.width) == (3, 4, 4)


def test_tree_shape():
    assert parse_tree(None) == (1, 0) and parse_tree("3,4") == (3, 4)
    for bad in ("3", "3,4,5", "a,b", "0,4", "8,8"):          # 1 + 8 * 8 = 65 nodes: one more than the window holds
        with pytest.raises(ValueError):
            parse_tree(bad)


def test_resolution_against_the_weights():
    auto = from_strings("auto")
    assert auto.resolve(True, False, False).backend == "mtp" and auto.resolve(True, False, False).adaptive
    assert auto.resolve(False, False, False).backend == "none"
    with pytest.raises(ValueError):
        from_strings("mtp", 3).resolve(False, False, False)
    with pytest.raises(ValueError):
        from_strings("dflash", 4).resolve(True, False, False)
    assert from_strings("mtp", 3).resolve(True, False, True).proposal_head == "shortlist"      # auto head: use what the artifact has
    assert from_strings("mtp", 3).resolve(True, False, False).proposal_head == "full"
    assert from_strings("mtp", 4, "auto", "3,4").resolve(True, False, True).proposal_head == "full"
    with pytest.raises(ValueError):
        from_strings("mtp", 3, "shortlist").resolve(True, False, False)
    assert SpeculativeOptions().validate().backend == "none"
