"""History look-up drafts: match definition and scan bound, chain policy with copied-from positions, width controller."""
import pytest

from ninfer_fusion_b200.runtime.lookup_fuse import (VerifyWidthController, fuse_chain, lookup_drafter, scan_limit,
                                                    suffix_best)


def test_match_prefers_the_latest_earlier_window_and_never_overlaps_the_query():
    ids = [1, 2, 3, 4, 9, 1, 2, 3, 4, 7, 7, 1, 2, 3, 4]
    # query = the last four tokens; two earlier full occurrences (offsets 0 and 5): the later one wins
    assert suffix_best(ids, len(ids) - 4, 4, 2, continuation_tokens=1) == (4, 5)
    # the continuation must fit inside the history: with K = 6 only offset 0 leaves room... and even that needs 0+4+6 < 15
    assert suffix_best(ids, len(ids) - 4, 4, 2, continuation_tokens=6) == (4, 0)
    assert scan_limit(11, 15, 4, 6) == 5 and scan_limit(11, 15, 4, 1) == 7
    # a window that overlaps the query is not a candidate: [5, 5, 5, 5, 5] has no earlier non-overlapping tail of length 3
    assert suffix_best([5, 5, 5, 5, 5], 2, 3, 2) == (0, 0)
    # partial match: only the last two tokens occur earlier
    assert suffix_best([8, 3, 4, 6, 0, 0, 2, 3, 4], 6, 3, 2, 1) == (2, 0)


def test_chain_policy_full_partial_and_no_match():
    ids = [1, 2, 3, 4, 9, 8, 7, 6, 5, 1, 2, 3, 4]
    toks, src, length = fuse_chain(ids, query_len=4, min_len=2, k=3)
    assert (toks, src, length) == ([9, 8, 7], [4, 5, 6], 4)                 # full match: K tokens straight from history
    part = [8, 3, 4, 6, 0, 0, 2, 3, 4]
    assert fuse_chain(part, 3, 2, 3) == ([6], [3], 2)                        # partial: one probe, the token after the match
    assert fuse_chain([1, 2, 3, 4, 5, 6], 3, 2, 3) == ([], [], 0)           # nothing: the neural drafter proposes
    assert fuse_chain([1, 2], 4, 2, 3)[0] == [] and fuse_chain(ids, 4, 2, 0)[0] == []
    # as a drafter hook the probe is padded from the history after it
    assert lookup_drafter(part, 3, query_len=3) == [6, 0, 0]
    assert lookup_drafter(ids, 3, query_len=4) == [9, 8, 7] and lookup_drafter([1, 2, 3, 4, 5, 6], 3) is None
    # page of the copied-from positions (64-token pages): what a source-keyed retention policy would count
    assert [p // 64 for p in src] == [0, 0, 0]


def test_width_controller_earns_the_wide_rung_and_loses_it():
    c = VerifyWidthController()
    assert c.width == 8 and c.lookup_slots == 8
    assert c.observe(1, 1, match_len=8, continuation=8) == 8        # one strong round is not a streak
    assert c.observe(1, 1, 8, 8) == 16                               # the second consecutive one is
    assert c.observe(1, 1, 3, 8) == 16 and c.observe(1, 1, 3, 8) == 16 and c.observe(1, 1, 3, 8) == 16   # a lone request coasts 3 rounds
    assert c.observe(1, 1, 3, 8) == 8 and c.refusals["miss"] == 1    # ... and no further
    c.observe(1, 1, 8, 8)
    assert c.observe(1, 1, 8, 8) == 16
    assert c.observe(1, 1, 0, 0) == 8                                # a plain miss drops at once, even alone
    c.observe(1, 1, 8, 8)
    c.observe(1, 1, 8, 8)
    assert c.observe(1, 1, 8, 5) == 8 and c.refusals["short_continuation"] == 1   # every extra slot filled, or no wide round
    c.observe(1, 2, 8, 8)
    assert c.observe(1, 2, 8, 8) == 16
    assert c.observe(1, 2, 3, 8) == 8                                # several requests decoding: no coasting
    c.observe(1, 1, 8, 8)
    assert c.observe(1, 1, 8, 8) == 16
    assert c.observe(2, 1, 8, 8) == 8 and c.refusals["other_request"] == 1        # another request does not inherit the latch
    assert c.observe(2, 1, 8, 8) == 16                               # it earns its own
    assert c.observe(2, 1, 8, 8, accepted_all=False) == 16 and c.observe(2, 1, 0, 8) == 8
    with pytest.raises(ValueError):
        VerifyWidthController(narrow=8, wide=8)
