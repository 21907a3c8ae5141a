"""CPU oracle for the DSA top-k indexer (definition ``dsa_topk_indexer_fp8_h64_d128_topk2048_ps64``).

TEST INFRASTRUCTURE ONLY: the checker of the sibling operator's parity tests.  The product never imports it.

It restates the reference's shipped entry point for this definition, which is pure torch
(dsa_indexer/solution/python/dsa_topk_indexer.py: cache dequantisation :38-58, scoring and selection :84-108):

* the index cache holds pages of 64 tokens, 8448 bytes each: 64 x 128 e4m3 bytes, then 64 f32 scales;
* a token's key is its 128 e4m3 values times its scale; a query has 64 heads of 128 e4m3 values (no scale);
* score[t] = sum_h weights[h] * relu(q[h] . key[t]);
* the 2048 best tokens of the sequence (all of them when it is shorter), best first, as
  page_id * 64 + offset in the cache; -1 beyond.

Pinning: ``tests/golden/make_golden_dsa.py`` imports the reference's entry point itself and stores its output for
seeded cases; ``tests/test_dsa_oracle_golden.py`` checks this module against those files.
"""
from __future__ import annotations

import torch

HEADS = 64
DIM = 128
PAGE = 64
PAGE_BYTES = PAGE * (DIM + 4)
TOPK = 2048


def dequant_cache(k_index_cache_fp8):
    """[pages, 64, 1, 132] int8 -> f32 [pages, 64, 128] (dsa_topk_indexer.py:38-58)."""
    u8 = k_index_cache_fp8.view(torch.uint8)
    pages = u8.shape[0]
    flat = u8.reshape(pages, PAGE_BYTES)
    data = flat[:, : PAGE * DIM].contiguous().view(pages, PAGE, DIM).view(torch.float8_e4m3fn).to(torch.float32)
    scale = flat[:, PAGE * DIM:].contiguous().view(pages, PAGE, 4).view(torch.float32)
    return data * scale


@torch.no_grad()
def topk_indexer(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk=TOPK):
    """Returns (indices int32 [B, topk], list of f32 score vectors, one per sequence)
    (dsa_topk_indexer.py:84-108)."""
    B = q_index_fp8.shape[0]
    q = q_index_fp8.to(torch.float32)
    K_all = dequant_cache(k_index_cache_fp8)
    out = torch.full((B, topk), -1, dtype=torch.int32, device=q.device)
    all_scores = []
    for b in range(B):
        n = int(seq_lens[b])
        if n == 0:
            all_scores.append(torch.empty(0, dtype=torch.float32, device=q.device))
            continue
        pages = block_table[b, : (n + PAGE - 1) // PAGE].to(torch.long)
        K = K_all[pages].reshape(-1, DIM)[:n]
        s = torch.relu(q[b] @ K.T)
        final = (s * weights[b][:, None]).sum(dim=0)
        k = min(topk, n)
        _, idx = torch.topk(final, k)
        out[b, :k] = (pages[idx // PAGE] * PAGE + idx % PAGE).to(torch.int32)
        all_scores.append(final)
    return out, all_scores


def make_inputs(seq_lens, num_pages=None, seed=0, device="cpu", weight_sign="mixed"):
    """Seeded synthetic inputs with the definition's shapes: queries and keys ~N(0,1) rounded to e4m3 (keys with
    a per-token scale amax/448 like the activations of the serving stack), head weights ~N(0,1)/8 (both signs:
    the reference applies them after the relu), pages of every sequence scattered over the cache."""
    g = torch.Generator().manual_seed(seed)
    B = len(seq_lens)
    need = [(n + PAGE - 1) // PAGE for n in seq_lens]
    max_pages = max(max(need), 1)
    if num_pages is None:
        num_pages = sum(need) + 3
    q = torch.randn(B, HEADS, DIM, generator=g).to(torch.float8_e4m3fn)
    keys = torch.randn(num_pages, PAGE, DIM, generator=g) * (0.5 + torch.rand(num_pages, PAGE, 1, generator=g))
    scale = keys.abs().amax(-1, keepdim=True).clamp_min(1e-6) / 448.0
    k8 = (keys / scale).to(torch.float8_e4m3fn)
    cache = torch.empty(num_pages, PAGE_BYTES, dtype=torch.uint8)
    cache[:, : PAGE * DIM] = k8.view(torch.uint8).reshape(num_pages, PAGE * DIM)
    cache[:, PAGE * DIM:] = scale.to(torch.float32).reshape(num_pages, PAGE).contiguous().view(torch.uint8).reshape(num_pages, PAGE * 4)
    cache = cache.view(torch.int8).view(num_pages, PAGE, 1, DIM + 4)
    w = torch.randn(B, HEADS, generator=g) / 8.0
    if weight_sign == "positive":
        w = w.abs()
    perm = torch.randperm(num_pages, generator=g)
    table = torch.zeros(B, max_pages, dtype=torch.int32)
    at = 0
    for b in range(B):
        table[b, : need[b]] = perm[at: at + need[b]].to(torch.int32)
        at += need[b]
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    return tuple(t.to(device) for t in (q, cache, w, sl, table))


def check_topk(got, want, scores, seq_lens, block_table, rtol=2e-5):
    """Selection parity: per sequence the same SET of tokens, except that tokens whose oracle score lies within
    `rtol` (relative to the largest score) of the score of the last kept token may be swapped (two summation orders of
    the same products differ in the last bits), and the order returned must be best-first by the oracle's scores to
    the same tolerance.  Returns (ok, stats)."""
    B = want.shape[0]
    worst_swaps, bad = 0, []
    for b in range(B):
        n = int(seq_lens[b])
        k = min(want.shape[1], n)
        g, w = got[b].cpu().to(torch.int64), want[b].cpu().to(torch.int64)
        if not bool((g[k:] == -1).all()):
            bad.append((b, "tail not -1"))
            continue
        if k == 0:
            continue
        pages = block_table[b, : (n + PAGE - 1) // PAGE].cpu().to(torch.int64)
        pos = {int(p): i for i, p in enumerate(pages.tolist())}
        sc = scores[b].cpu()

        def local(tok):     # cache token id -> position in the sequence, or -1
            p, o = int(tok) // PAGE, int(tok) % PAGE
            i = pos.get(p, -1)
            return i * PAGE + o if i >= 0 and i * PAGE + o < n else -1
        gl = [local(t) for t in g[:k].tolist()]
        if min(gl) < 0 or len(set(gl)) != k:
            bad.append((b, "token outside the sequence or repeated"))
            continue
        tol = rtol * float(sc.abs().max())
        kth = float(torch.topk(sc, k).values[-1])
        gs = sc[torch.tensor(gl)]
        if float(gs.min()) < kth - tol:
            bad.append((b, f"kept a token {kth - float(gs.min()):.3g} below the last place"))
            continue
        if bool((gs[1:] - gs[:-1] > tol).any()):
            bad.append((b, "not best-first"))
            continue
        worst_swaps = max(worst_swaps, len(set(g[:k].tolist()) ^ set(w[:k].tolist())) // 2)
    return len(bad) == 0, {"sequences": B, "failed": bad[:4], "most_tokens_swapped_at_the_cut": worst_swaps}
