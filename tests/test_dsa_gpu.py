"""Parity of the DSA top-k indexer's CUDA path (through the C ABI) against its oracle.  Needs a B200."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _run(pkg, inputs):
    q, cache, w, sl, table = (t.to(DEV) for t in inputs)
    out = torch.full((q.shape[0], 2048), -7, dtype=torch.int32, device=DEV)
    pkg.run_dsa_topk_indexer(q, cache, w, sl, table, out)
    pkg.dsa_check()
    return out


@pytest.mark.parametrize("name", ["dsa_small", "dsa_cut", "dsa_long"])
def test_indexer_matches_reference_entry_point_vectors(name, pkg, golden_dir):
    """Against the stored outputs of the reference's own entry point: the same tokens, best first; tokens whose
    scores differ by less than 2e-5 of the largest score may swap places (the tensor core sums the 128 products of a
    head in another order than the host's matrix product, the sum over the heads likewise)."""
    from oracle import dsa_oracle
    g = torch.load(os.path.join(golden_dir, name + ".pt"))
    inputs = dsa_oracle.make_inputs(**g["make_inputs"])
    _, scores = dsa_oracle.topk_indexer(*inputs)
    out = _run(pkg, inputs)
    ok, stats = dsa_oracle.check_topk(out, g["topk_indices"], scores, inputs[3], inputs[4])
    assert ok, stats
    # sequences no longer than 2048 keep every token: exactly the same set as the reference
    for b, n in enumerate(g["make_inputs"]["seq_lens"]):
        if 0 < n <= 2048:
            assert set(out[b, :n].tolist()) == set(g["topk_indices"][b, :n].tolist())
        if n == 0:
            assert bool((out[b] == -1).all())


@pytest.mark.parametrize("seq_lens,seed", [([40000, 3, 17000, 2048, 70000], 11), ([128] * 40, 12)])
def test_indexer_matches_oracle(seq_lens, seed, pkg):
    """Long sequences (several radix passes with many candidates per byte) and a wide batch, against the oracle
    evaluated with torch on the GPU."""
    from oracle import dsa_oracle
    inputs = tuple(t.to(DEV) for t in dsa_oracle.make_inputs(seq_lens, seed=seed))
    want, scores = dsa_oracle.topk_indexer(*inputs)
    out = _run(pkg, inputs)
    ok, stats = dsa_oracle.check_topk(out, want, scores, inputs[3].cpu(), inputs[4].cpu())
    assert ok, stats
    assert stats["most_tokens_swapped_at_the_cut"] <= 4


def test_indexer_ties_and_determinism(pkg):
    """All keys equal: every score is the same, so the cut is one big tie; the lowest positions win, in position
    order, run after run."""
    from oracle import dsa_oracle
    q, cache, w, sl, table = dsa_oracle.make_inputs([5000], seed=13)
    cache = cache.view(torch.uint8).reshape(cache.shape[0], -1).clone()
    cache[:] = cache[0, :132].repeat(64)[: cache.shape[1]] * 0 + cache[0:1]      # every page a copy of page 0
    row0 = cache[:, :128].clone()
    cache[:, : 64 * 128] = row0.repeat(1, 64)                                   # every token a copy of token 0
    cache[:, 64 * 128:] = cache[:, 64 * 128: 64 * 128 + 4].repeat(1, 64)        # ... with token 0's scale
    cache = cache.view(torch.int8).view(-1, 64, 1, 132)
    a = _run(pkg, (q, cache, w, sl, table))
    b = _run(pkg, (q, cache, w, sl, table))
    assert torch.equal(a, b)
    want = (table[0, torch.arange(2048) // 64].to(torch.int64) * 64 + torch.arange(2048) % 64).to(torch.int32)
    assert torch.equal(a[0].cpu(), want)


def test_indexer_argument_validation(pkg):
    from oracle import dsa_oracle
    q, cache, w, sl, table = (t.to(DEV) for t in dsa_oracle.make_inputs([100], seed=1))
    out = torch.empty(1, 2048, dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError, match="topk_indices"):
        pkg.run_dsa_topk_indexer(q, cache, w, sl, table, out[:, :100])
    with pytest.raises(ValueError, match="weights"):
        pkg.run_dsa_topk_indexer(q, cache, w.double(), sl, table, out)
    with pytest.raises(ValueError, match="no CPU path"):
        pkg.run_dsa_topk_indexer(q.cpu(), cache, w, sl, table, out)
    pkg.run_dsa_topk_indexer(q, cache, w, sl, table, out)
    pkg.dsa_check()
