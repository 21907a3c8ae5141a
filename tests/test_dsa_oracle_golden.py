"""The DSA top-k indexer's oracle against outputs of the reference's own (pure torch) entry point."""
import os

import pytest
import torch


@pytest.mark.parametrize("name", ["dsa_small", "dsa_cut", "dsa_long"])
def test_oracle_matches_reference_entry_point(name, golden_dir):
    from oracle import dsa_oracle
    g = torch.load(os.path.join(golden_dir, name + ".pt"))
    q, cache, w, sl, table = dsa_oracle.make_inputs(**g["make_inputs"])
    out, scores = dsa_oracle.topk_indexer(q, cache, w, sl, table)
    # same operations on the same host: identical tokens in identical order
    assert torch.equal(out, g["topk_indices"])
    ok, stats = dsa_oracle.check_topk(out, g["topk_indices"], scores, sl, table)
    assert ok, stats


def test_selection_check_rejects_wrong_answers():
    from oracle import dsa_oracle
    q, cache, w, sl, table = dsa_oracle.make_inputs([3000], seed=7)
    out, scores = dsa_oracle.topk_indexer(q, cache, w, sl, table)
    worst = int(torch.argmin(scores[0]))
    bad = out.clone()
    bad[0, 5] = table[0, worst // 64] * 64 + worst % 64       # the worst token of the sequence smuggled in
    ok, _ = dsa_oracle.check_topk(bad, out, scores, sl, table)
    assert not ok
    swapped = out.clone()
    swapped[0, 0], swapped[0, 2047] = out[0, 2047], out[0, 0]  # right set, wrong order
    ok, _ = dsa_oracle.check_topk(swapped, out, scores, sl, table)
    assert not ok
