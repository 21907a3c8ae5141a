"""Parity of the CUDA path (called through the C ABI) against the oracle.  All tests need a B200."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _run(pkg, inp, dtype=torch.bfloat16):
    out = torch.full((inp.num_tokens, 7168), float("nan"), dtype=dtype, device=inp.gemm1_weights.device)
    pkg.run_moe(*inp.args(), out)
    stats = pkg.get_context(0).check()
    return out, stats


# ------------------------------------------------------------------ routing
@pytest.mark.parametrize("T", [1, 7, 16, 64, 1024, 8192])
def test_routing_bit_exact(T, pkg, oracle):
    inp = pkg.make_inputs(num_tokens=T, seed=0, e_local=1, device="cpu")
    idx, w = pkg.route(inp.routing_logits.to(DEV), inp.routing_bias.to(DEV), 0, 2.5)
    ridx, rw = oracle.route(inp.routing_logits, inp.routing_bias, 2.5)
    ok, stats = oracle.check_routing(idx, w, ridx, rw)
    assert ok, stats
    # best-first order: weights follow the biased score, so just check indices are a permutation of the set
    assert idx.dtype == torch.int32 and w.dtype == torch.float32


@pytest.mark.parametrize("T", [1024, 8192])
def test_routing_matches_published_reference_vectors(T, pkg, oracle, golden_dir):
    g = torch.load(os.path.join(golden_dir, f"route_t{T}.pt"))
    inp = pkg.make_inputs(num_tokens=T, seed=0, e_local=1, device="cpu")
    idx, w = pkg.route(inp.routing_logits.to(DEV), inp.routing_bias.to(DEV), 0, 2.5)
    a = torch.sort(idx.cpu().long(), dim=1).values
    b = torch.sort(g["topk_idx"].long(), dim=1).values
    assert torch.equal(a, b)
    ok, stats = oracle.check_routing(idx[:256], w[:256], g["topk_idx"][:256].long(), g["topk_w_first256"])
    assert ok, stats


def test_routing_with_skewed_logits(pkg, oracle):
    inp = pkg.make_inputs(num_tokens=4096, seed=0, e_local=1, hot_experts=16, device="cpu")
    idx, w = pkg.route(inp.routing_logits.to(DEV), inp.routing_bias.to(DEV), 64, 1.0, num_local_experts=32)
    ridx, rw = oracle.route(inp.routing_logits, inp.routing_bias, 1.0)
    ok, stats = oracle.check_routing(idx, w, ridx, rw)
    assert ok, stats


# -------------------------------------------------------------- permutation
@pytest.mark.parametrize("T,E,off", [(64, 32, 0), (300, 8, 0), (129, 4, 36), (5000, 32, 0), (8200, 5, 16)])
def test_row_lists(T, E, off, pkg):
    inp = pkg.make_inputs(num_tokens=T, seed=1, e_local=E, local_expert_offset=off, device=DEV)
    _, stats = _run(pkg, inp)
    ctx = pkg.get_context(0)
    idx, _ = ctx.last_routing(T)
    row_token, cap = ctx.debug_read("row_token", torch.int32)
    route_row, _ = ctx.debug_read("route_row", torch.int32)
    counts, _ = ctx.debug_read("counts", torch.int32)
    route_row = route_row[: T * 8].view(T, 8)
    local = (idx >= off) & (idx < off + E)
    assert stats["routes"] == int(local.sum())
    assert stats["active_experts"] == int(torch.unique(idx[local]).numel())
    exp_counts = torch.bincount((idx[local] - off).long(), minlength=32)[:E]
    assert torch.equal(counts[:E].long(), exp_counts)
    pad = (exp_counts + 15) // 16 * 16
    assert stats["padded_rows"] == int(pad.sum())
    # rows of an expert are its tokens in increasing order, then -1 padding
    start = 0
    for e in range(E):
        c, cp = int(exp_counts[e]), int(pad[e])
        toks = torch.nonzero((idx == e + off).any(1)).squeeze(1).int()
        assert torch.equal(row_token[start:start + c], toks)
        assert bool((row_token[start + c:start + cp] == -1).all())
        start += cp
    # route_row inverts row_token for local routes and is -1 elsewhere
    assert bool((route_row[~local] == -1).all())
    rows = route_row[local].long()
    assert torch.equal(row_token[rows].long(), torch.nonzero(local)[:, 0])
    # per-expert work table: row ranges tile the padded row space, token tiles are counted consistently
    work, _ = ctx.debug_read("expert_work", torch.int32)
    work = work.view(32, 4)[:E]
    tile = 32 if T <= 1024 else 64 if T < 6144 else 128     # from 4096 tokens on, four CTAs share an expert's tokens
    bounds = torch.cumsum(torch.cat([torch.zeros(1, dtype=torch.long), pad]), 0)
    tile_off = 0
    for e, (row_off, rows_pad, t_off, tiles) in enumerate(work.tolist()):
        assert row_off == int(bounds[e]) and rows_pad == int(pad[e])
        assert tiles == (rows_pad + tile - 1) // tile and t_off == tile_off
        tile_off += tiles
    assert stats["token_tiles"] == tile_off


# ------------------------------------------------------------ whole layer
@pytest.mark.parametrize("T,E,off,seed", [
    (16, 32, 0, 0),      # the CPU-runnable configuration
    (64, 32, 0, 0),      # decode batch
    (1, 32, 0, 3), (2, 32, 0, 4), (7, 8, 0, 5),
    (127, 8, 8, 6), (128, 8, 8, 6), (129, 8, 8, 6),
    (300, 4, 36, 7),
])
def test_layer_matches_oracle(T, E, off, seed, pkg, oracle):
    inp = pkg.make_inputs(num_tokens=T, seed=seed, e_local=E, local_expert_offset=off, device=DEV)
    out, stats = _run(pkg, inp)
    ref, ridx, rw = oracle.moe_forward(*inp.to("cpu").args())
    idx, w = pkg.get_context(0).last_routing(T)
    ok, rstats = oracle.check_routing(idx, w, ridx, rw)
    assert ok, rstats
    ok, ostats = oracle.check_output(out, ref)
    assert ok, (ostats, stats)


def test_prefill_chunk_matches_oracle(pkg, oracle):
    """T = 1024, 32 local experts; the oracle runs with torch on the GPU to keep the test short."""
    inp = pkg.make_inputs(num_tokens=1024, seed=0, e_local=32, device=DEV)
    out, stats = _run(pkg, inp)
    ref, ridx, rw = oracle.moe_forward(*inp.args())
    cidx, cw = oracle.route(inp.routing_logits.cpu(), inp.routing_bias.cpu(), 2.5)
    idx, w = pkg.get_context(0).last_routing(1024)
    ok, rstats = oracle.check_routing(idx, w, cidx, cw)
    assert ok, rstats
    ok, ostats = oracle.check_output(out, ref)
    assert ok, (ostats, stats)


@pytest.mark.parametrize("T,E,off,seed", [(1000, 32, 224, 3), (513, 31, 1, 7), (4096, 2, 100, 2), (8192, 1, 0, 6)])
def test_odd_shapes_match_oracle(T, E, off, seed, pkg, oracle):
    """The last experts of the global range, an odd expert count, and very few experts with many rows each
    (several token tiles per expert); the oracle runs with torch on the GPU."""
    inp = pkg.make_inputs(num_tokens=T, seed=seed, e_local=E, local_expert_offset=off, device=DEV)
    out, stats = _run(pkg, inp)
    ref, _, _ = oracle.moe_forward(*inp.args())
    ok, ostats = oracle.check_output(out, ref)
    assert ok, (ostats, stats)


def _check_against_gpu_oracle(pkg, oracle, inp):
    """Whole layer against the oracle executed with torch on the GPU (large cases), routing against the
    oracle's CPU route (the one the golden vectors pin)."""
    T = inp.num_tokens
    out, stats = _run(pkg, inp)
    ref, _, _ = oracle.moe_forward(*inp.args())
    cidx, cw = oracle.route(inp.routing_logits.cpu(), inp.routing_bias.cpu(), inp.routed_scaling_factor)
    idx, w = pkg.get_context(0).last_routing(T)
    ok, rstats = oracle.check_routing(idx, w, cidx, cw)
    assert ok, rstats
    ok, ostats = oracle.check_output(out, ref)
    assert ok, (ostats, stats)
    return out, stats


def test_twice_the_largest_configuration_matches_oracle(pkg, oracle):
    """16384 tokens, 32 local experts: twice the largest configuration (experts with up to ~2600 rows,
    ~18000 routed rows), against the oracle run with torch on the GPU."""
    inp = pkg.make_inputs(num_tokens=16384, seed=0, e_local=32, device=DEV)
    _, stats = _check_against_gpu_oracle(pkg, oracle, inp)
    assert stats["routes"] > 16384 and stats["active_experts"] >= 30
    del inp
    torch.cuda.empty_cache()


def test_full_prefill_configuration_matches_oracle(pkg, oracle):
    """The largest single-GPU configuration: T = 8192 tokens, all 32 local experts, seed 0, offset 0
    (8951 routed rows over 30 active experts, 0 .. 1316 rows per expert).  Runs the CTA-pair kernels."""
    inp = pkg.make_inputs(num_tokens=8192, seed=0, e_local=32, device=DEV)
    _, stats = _check_against_gpu_oracle(pkg, oracle, inp)
    assert stats["routes"] == 8951 and stats["active_experts"] == 30


@pytest.mark.parametrize("rank", [0, 5])
def test_skewed_full_layer_rank_matches_oracle(rank, pkg, oracle):
    """One rank of the 256-expert, 8-rank configuration with load imbalance: T = 4096 tokens shared by all
    ranks, logits of 16 hot experts raised by 1.5 (chosen with seed 1), this rank's 32 experts drawn from
    weight seed = rank, offset 32 * rank."""
    inp = pkg.make_inputs(num_tokens=4096, seed=0, e_local=32, local_expert_offset=32 * rank, device=DEV,
                          hot_experts=16, weight_seed=rank)
    _, stats = _check_against_gpu_oracle(pkg, oracle, inp)
    assert stats["routes"] > 2000


@pytest.mark.parametrize("T,E,off,tile", [(300, 8, 0, None), (129, 4, 36, None), (1500, 4, 8, 256)])
def test_intermediate_stages_match_oracle(T, E, off, tile, pkg, oracle, monkeypatch):
    """Stage by stage through the workspace: the gathered activation bytes and scales are exact copies of the
    routed tokens' rows; the two-term e4m3 SwiGLU output s * (hi + lo / 28) reproduces the oracle's f32
    silu(X2) * X1 to ~8 bits (a single e4m3 term would be ~4: this is what the second term buys); the per-route
    GEMM2 rows match the oracle's C W2^T."""
    if tile is not None:
        monkeypatch.setenv("SYFI_MOE_TOKEN_TILE", str(tile))
    inp = pkg.make_inputs(num_tokens=T, seed=5, e_local=E, local_expert_offset=off, device=DEV)
    _run(pkg, inp)
    ctx = pkg.get_context(0)
    meta, cap = ctx.debug_read("meta", torch.int32)
    R = int(meta[1])
    row_token, _ = ctx.debug_read("row_token", torch.int32)
    row_token = row_token[:R].long()
    valid = row_token >= 0
    a_perm, _ = ctx.debug_read("a_perm", torch.uint8, max_bytes=R * 7168)
    a_scale, _ = ctx.debug_read("a_scale", torch.float32)
    hs = inp.hidden_states.cpu().view(torch.uint8)
    assert torch.equal(a_perm.view(R, 7168)[valid], hs[row_token[valid]])
    assert bool((a_perm.view(R, 7168)[~valid] == 0).all())
    assert torch.equal(a_scale.view(56, cap)[:, :R][:, valid], inp.hidden_states_scale.cpu()[:, row_token[valid]])
    c_hi, _ = ctx.debug_read("c_hi", torch.uint8, max_bytes=R * 2048)
    c_lo, _ = ctx.debug_read("c_lo", torch.uint8, max_bytes=R * 2048)
    c_scale, _ = ctx.debug_read("c_scale", torch.float32)
    o_rows, _ = ctx.debug_read("o_rows", torch.float32, max_bytes=R * 7168 * 4)
    c_scale = c_scale.view(16, cap)[:, :R].t().contiguous()
    hi = c_hi.view(R, 2048).view(torch.float8_e4m3fn).float().view(R, 16, 128)
    lo = c_lo.view(R, 2048).view(torch.float8_e4m3fn).float().view(R, 16, 128)
    c_two = ((hi + lo / 28.0) * c_scale.unsqueeze(-1)).view(R, 2048).to(DEV)
    c_one = (hi * c_scale.unsqueeze(-1)).view(R, 2048).to(DEV)
    o_rows = o_rows.view(R, 7168).to(DEV)
    counts, _ = ctx.debug_read("counts", torch.int32)
    A = oracle.dequant_act(inp.hidden_states, inp.hidden_states_scale)
    start, worst_two, worst_one, worst_o = 0, 0.0, 0.0, 0.0
    for e in range(E):
        c = int(counts[e])
        if c:
            tok = row_token[start:start + c].to(DEV)
            W13 = oracle.dequant_weight(inp.gemm1_weights[e], inp.gemm1_weights_scale[e])
            W2 = oracle.dequant_weight(inp.gemm2_weights[e], inp.gemm2_weights_scale[e])
            G1 = A[tok] @ W13.t()
            C = (G1[:, 2048:] / (1.0 + torch.exp(-G1[:, 2048:]))) * G1[:, :2048]
            # per 1x128 block, relative to the block's amax (the quantity the block scale is made from)
            amax = C.view(c, 16, 128).abs().amax(-1, keepdim=True).clamp_min(1e-30)
            worst_two = max(worst_two, float(((c_two[start:start + c] - C).view(c, 16, 128).abs() / amax).max()))
            worst_one = max(worst_one, float(((c_one[start:start + c] - C).view(c, 16, 128).abs() / amax).max()))
            O = C @ W2.t()
            worst_o = max(worst_o, float((o_rows[start:start + c] - O).abs().max() / O.abs().max()))
        start += (c + 15) // 16 * 16
    assert worst_two <= 2.0 ** -8, worst_two      # two terms: error below 2^-8 of the block's amax
    assert worst_one >= 2.0 ** -6, worst_one      # one term alone is an order of magnitude coarser
    assert worst_o <= 4e-3, worst_o


@pytest.mark.parametrize("T,E,off,seed", [(600, 8, 16, 11), (3000, 4, 100, 12)])
def test_every_token_tile_gives_the_same_bits(T, E, off, seed, pkg, oracle, monkeypatch):
    """The GEMM kernels exist for token tiles of 32, 64 and 128 rows and as the CTA-pair configuration
    (256: token-major GEMM1 on 256-row tiles, GEMM2 on 128-row tiles); the library picks by batch size, the
    environment variable forces one.  The tile changes the work split and the operand orientation, never
    the arithmetic of an output element (same products, same K-block order, same promotion), so all four
    must agree bit for bit, and with the oracle within tolerance.  600 tokens over 8 experts give every
    expert several small tiles and a ragged last one; 3000 tokens over 4 experts give the pair kernels
    experts with more than 256 rows (several 256-row tiles, the second CTA of a pair partly filled)."""
    inp = pkg.make_inputs(num_tokens=T, seed=seed, e_local=E, local_expert_offset=off, device=DEV)
    ref, _, _ = oracle.moe_forward(*inp.args())
    outs = []
    for tile in (32, 64, 128, 256):
        monkeypatch.setenv("SYFI_MOE_TOKEN_TILE", str(tile))
        out, stats = _run(pkg, inp)
        ok, ostats = oracle.check_output(out, ref)
        assert ok, (tile, ostats, stats)
        outs.append(out)
    for o in outs[1:]:
        assert torch.equal(outs[0], o)


def _swizzled_tiles(x):
    """x: [..., 128 rows, 8 chunks, 16 bytes] -> chunk c of row r moved to chunk c ^ (r & 7)."""
    r = torch.arange(128, device=x.device)[:, None]
    c = torch.arange(8, device=x.device)[None, :]
    return x[..., r, c ^ (r & 7), :]


def test_prepacked_weight_layout(pkg):
    """Every byte of the packed buffers is where the header says: tiles of 128 rows x 128 bytes in
    (expert, feature tile, K block[, up/gate]) order with the 128-byte swizzle inside a tile."""
    E = 2
    g = torch.Generator(device=DEV).manual_seed(5)
    w13 = torch.randint(0, 256, (E, 4096, 7168), dtype=torch.uint8, device=DEV, generator=g)
    w2 = torch.randint(0, 256, (E, 7168, 2048), dtype=torch.uint8, device=DEV, generator=g)
    packed = pkg.prepack_weights(w13.view(torch.float8_e4m3fn), w2.view(torch.float8_e4m3fn))
    torch.cuda.synchronize()
    # [e, half, ft, r, kb, chunk, byte] -> [e, ft, kb, half, r, chunk, byte]
    want13 = _swizzled_tiles(w13.view(E, 2, 16, 128, 56, 8, 16).permute(0, 2, 4, 1, 3, 5, 6)).reshape(-1)
    # [e, ft, r, kb, chunk, byte] -> [e, ft, kb, r, chunk, byte]
    want2 = _swizzled_tiles(w2.view(E, 56, 128, 16, 8, 16).permute(0, 1, 3, 2, 4, 5)).reshape(-1)
    assert torch.equal(packed.gemm1, want13)
    assert torch.equal(packed.gemm2, want2)


@pytest.mark.parametrize("T,E,off,tile", [(1, 8, 0, None), (64, 32, 0, None), (333, 8, 24, None), (333, 8, 24, 128),
                                          (1500, 8, 8, None)])
def test_prepacked_forward_is_bit_identical(T, E, off, tile, pkg, monkeypatch):
    """The packed path changes how weight tiles reach shared memory, not one arithmetic operation."""
    if tile is not None:
        monkeypatch.setenv("SYFI_MOE_TOKEN_TILE", str(tile))
    inp = pkg.make_inputs(num_tokens=T, seed=21, e_local=E, local_expert_offset=off, device=DEV)
    out, _ = _run(pkg, inp)
    packed = pkg.prepack_weights(inp.gemm1_weights, inp.gemm2_weights)
    out_p = torch.full_like(out, float("nan"))
    pkg.run_moe_prepacked(inp.routing_logits, inp.routing_bias, inp.hidden_states, inp.hidden_states_scale, packed,
                          inp.gemm1_weights_scale, inp.gemm2_weights_scale, off, inp.routed_scaling_factor, out_p)
    pkg.get_context(0).check()
    assert torch.isfinite(out_p.float()).all()
    assert torch.equal(out, out_p)
    # and back on the plain path with the same context (the cached tensor maps must be rebuilt)
    out2, _ = _run(pkg, inp)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("name", ["e4_off36", "e8_t16"])
def test_layer_matches_published_reference_vectors(name, pkg, oracle, golden_dir):
    """CPU-generated inputs, output compared with what the definition's published reference produced."""
    g = torch.load(os.path.join(golden_dir, name + ".pt"))
    inp = pkg.make_inputs(device="cpu", **g["make_inputs"]).to(DEV)
    out, _ = _run(pkg, inp)
    ok, ostats = oracle.check_output(out, g["output_bf16_bits"].view(torch.bfloat16))
    assert ok, ostats
    idx, w = pkg.get_context(0).last_routing(inp.num_tokens)
    ok, rstats = oracle.check_routing(idx, w, g["topk_idx"].long(), g["topk_w"])
    assert ok, rstats


def test_tokens_without_local_route_get_zero(pkg):
    inp = pkg.make_inputs(num_tokens=33, seed=9, e_local=1, local_expert_offset=200, device=DEV)
    out, stats = _run(pkg, inp)
    idx, _ = pkg.get_context(0).last_routing(33)
    hit = (idx == 200).any(1)
    assert bool((out[~hit.to(DEV)] == 0).all())
    assert stats["routes"] == int(hit.sum())


def test_deterministic_and_workspace_reuse(pkg):
    inp = pkg.make_inputs(num_tokens=200, seed=11, e_local=8, device=DEV)
    a, _ = _run(pkg, inp)
    small = pkg.make_inputs(num_tokens=5, seed=12, e_local=8, device=DEV)
    _run(pkg, small)                     # a different shape in between, same workspace
    b, _ = _run(pkg, inp)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("T,E", [(64, 32), (700, 16)])
def test_back_to_back_calls_are_bit_identical(T, E, pkg):
    """GEMM2 starts while GEMM1 is still running and is released expert by expert through counters in
    global memory; the row counters are re-zeroed by the chain itself.  Two hundred calls in a row without a
    host synchronisation in between must each reproduce the first one bit for bit."""
    inp = pkg.make_inputs(num_tokens=T, seed=3, e_local=E, device=DEV)
    ref, _ = _run(pkg, inp)
    outs = [torch.empty_like(ref) for _ in range(4)]
    for i in range(200):
        outs[i % 4].fill_(float("nan"))
        pkg.run_moe(*inp.args(), outs[i % 4])
        if i % 4 == 3:
            for o in outs:
                assert torch.equal(o, ref), i
    pkg.get_context(0).check()


def test_cuda_graph_replay(pkg):
    """The call enqueues only stream work (no host synchronisation, no per-call device state passed by
    value), so it can be captured once and replayed; replays reproduce the eager result bit for bit."""
    inp = pkg.make_inputs(num_tokens=48, seed=17, e_local=16, device=DEV)
    eager, _ = _run(pkg, inp)
    out = torch.empty_like(eager)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pkg.run_moe(*inp.args(), out)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), eager.view(torch.int16))
    pkg.get_context(0).check()


def test_scaling_factor_is_linear_exactly(pkg):
    """Doubling routed_scaling_factor doubles every f32 partial exactly (power-of-two scaling
    commutes with every rounding on the path), a size-independent property checked at T = 2048."""
    inp = pkg.make_inputs(num_tokens=2048, seed=13, e_local=16, device=DEV)
    a, _ = _run(pkg, inp, torch.float32)
    inp.routed_scaling_factor = 5.0
    b, _ = _run(pkg, inp, torch.float32)
    assert torch.equal(b, 2.0 * a)
    assert float(a.abs().max()) > 0


def test_f32_partial_rounds_to_bf16_output(pkg):
    inp = pkg.make_inputs(num_tokens=96, seed=14, e_local=8, device=DEV)
    a, _ = _run(pkg, inp)
    p, _ = _run(pkg, inp, torch.float32)
    assert torch.equal(a.view(torch.int16), p.to(torch.bfloat16).view(torch.int16))


def test_expert_slices_sum_to_full_layer(pkg, oracle):
    """Four ranks' worth of 8-expert slices (partials summed in f32) equal one 32-expert call."""
    inp = pkg.make_inputs(num_tokens=256, seed=15, e_local=32, device=DEV)
    full, _ = _run(pkg, inp, torch.float32)
    acc = torch.zeros_like(full)
    for r in range(4):
        sl = slice(8 * r, 8 * r + 8)
        part = pkg.MoeInputs(inp.routing_logits, inp.routing_bias, inp.hidden_states, inp.hidden_states_scale,
                             inp.gemm1_weights[sl].contiguous(), inp.gemm1_weights_scale[sl].contiguous(),
                             inp.gemm2_weights[sl].contiguous(), inp.gemm2_weights_scale[sl].contiguous(),
                             8 * r, 2.5)
        p, _ = _run(pkg, part, torch.float32)
        acc += p
    # the K split of a work item depends on how many items a call has, so f32 sums are reordered
    err = float((acc - full).abs().max())
    assert err <= 1e-4 * float(full.abs().max()), err


@pytest.mark.parametrize("pinned", [True, False])
def test_host_entry_point_matches_device_entry_point(pinned, pkg):
    """Pinned buffers are read and written by the kernels directly, pageable ones go through the staging
    area; a second call with other buffers of the other kind must not reuse a remembered mapping."""
    inp = pkg.make_inputs(num_tokens=64, seed=16, e_local=8, device=DEV)
    dev_out, _ = _run(pkg, inp)
    place = (lambda t: t.pin_memory()) if pinned else (lambda t: t.clone())
    host = [place(t.cpu()) for t in (inp.routing_logits, inp.routing_bias, inp.hidden_states,
                                     inp.hidden_states_scale)]
    for _ in range(2):
        out = place(torch.zeros(64, 7168, dtype=torch.bfloat16))
        pkg.run_moe_host(*host, inp.gemm1_weights, inp.gemm1_weights_scale, inp.gemm2_weights,
                         inp.gemm2_weights_scale, 0, 2.5, out)
        pkg.get_context(0).check()
        assert torch.equal(out.view(torch.int16), dev_out.cpu().view(torch.int16))


@pytest.mark.parametrize("pinned", [True, False])
def test_host_entry_point_in_slices_matches_device_entry_point(pinned, pkg):
    """From 2048 tokens on the host entry point works in slices of 1024 tokens (copy in, compute and copy out
    overlap); 2500 tokens make two full slices and a ragged one.  Bit-identical to the device entry point on the
    whole batch, twice in a row on the same staging area."""
    T = 2500
    inp = pkg.make_inputs(num_tokens=T, seed=17, e_local=8, device=DEV)
    dev_out, _ = _run(pkg, inp)
    place = (lambda t: t.pin_memory()) if pinned else (lambda t: t.clone())
    host = [place(t.cpu()) for t in (inp.routing_logits, inp.routing_bias, inp.hidden_states,
                                     inp.hidden_states_scale)]
    for _ in range(2):
        out = place(torch.full((T, 7168), float("nan"), dtype=torch.bfloat16))
        pkg.run_moe_host(*host, inp.gemm1_weights, inp.gemm1_weights_scale, inp.gemm2_weights,
                         inp.gemm2_weights_scale, 0, 2.5, out)
        pkg.get_context(0).check()
        assert torch.equal(out.view(torch.int16), dev_out.cpu().view(torch.int16))


def test_torch_operator_gives_the_same_bits(pkg):
    """The layer through the torch dispatcher (`torch.ops.syfi_moe.run_moe`) against the plain function."""
    inp = pkg.make_inputs(num_tokens=48, seed=19, e_local=8, device=DEV)
    want, _ = _run(pkg, inp)
    got = torch.full((48, 7168), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert torch.ops.syfi_moe.run_moe(*inp.args(), got) is None
    pkg.get_context(0).check()
    assert torch.equal(got, want)


def test_zero_tokens_is_a_no_op(pkg):
    inp = pkg.make_inputs(num_tokens=0, seed=0, e_local=2, device=DEV)
    out = torch.empty(0, 7168, dtype=torch.bfloat16, device=DEV)
    assert pkg.run_moe(*inp.args(), out) is out


def test_argument_validation(pkg):
    inp = pkg.make_inputs(num_tokens=4, seed=0, e_local=2, device=DEV)
    out = torch.empty(4, 7168, dtype=torch.bfloat16, device=DEV)
    args = list(inp.args())
    with pytest.raises(ValueError, match="output"):
        pkg.run_moe(*args, out[:3])
    with pytest.raises(ValueError, match="dtype"):
        pkg.run_moe(args[0].double(), *args[1:], out)
    with pytest.raises(ValueError, match="contiguous"):
        pkg.run_moe(args[0], args[1], args[2], inp.hidden_states_scale.t().contiguous().t(), *args[4:], out)
    with pytest.raises(ValueError, match="outside"):
        pkg.run_moe(*args[:8], 255, 2.5, out)
    with pytest.raises(ValueError, match="host tensor|must be on"):
        pkg.run_moe(args[0].cpu(), *args[1:], out)
    pkg.run_moe(*args, out)              # the context is still usable afterwards
    pkg.get_context(0).check()


@pytest.mark.parametrize("T,E,seed", [(8, 2, 3), (77, 8, 4), (1500, 32, 5), (6200, 6, 9)])
def test_token_dispatch_on_one_rank_equals_the_plain_layer(T, E, seed, pkg):
    """The token-dispatch entry point with a world of one rank: route, publish, pull the routed rows from
    the rank's own region, the layer from the row lists on, push and final sum.  Everything but the link is
    exercised, and the result must equal the plain layer bit for bit — over several steps on different
    tokens (alternating buffer sets) and interleaved with the all-gather layout on the same region.  The
    largest case runs the CTA-pair kernels, whose GEMM2 epilogue then stores through the row targets."""
    nbytes = pkg.ep_region_bytes(1, T)
    region = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    desc = pkg.EpDesc()
    desc.world_size, desc.rank, desc.tokens_per_rank = 1, 0, T
    desc.region[0] = region.data_ptr()
    desc.wait_limit_cycles = 1 << 27
    base = pkg.make_inputs(num_tokens=T, seed=seed, e_local=E, local_expert_offset=32 if E < 32 else 0, device=DEV)
    w = base.args()[4:8]
    for step in range(1, 6):
        tok = pkg.make_inputs(num_tokens=T, seed=100 * seed + step, e_local=1, device="cpu")
        lg, hs, sc = (t.to(DEV) for t in (tok.routing_logits, tok.hidden_states, tok.hidden_states_scale))
        want = torch.empty(T, 7168, dtype=torch.bfloat16, device=DEV)
        pkg.run_moe(lg, base.routing_bias, hs, sc, *w, base.local_expert_offset, 2.5, want)
        got = torch.full((T, 7168), float("nan"), dtype=torch.bfloat16, device=DEV)
        pkg.run_moe_ep(desc, step, lg, base.routing_bias, hs, sc, *w, base.local_expert_offset, 2.5, got,
                       dispatch=(step != 3))
        stats = pkg.get_context(0).check()
        assert torch.equal(got, want), (step, float((got.float() - want.float()).abs().max()))
    assert stats["routes"] > 0      # the cases route rows to the local experts


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_walked_through_a_step_on_one_gpu_sum_to_the_plain_layer(world, pkg):
    """Several ranks of the replicated-token layout on ONE GPU, one after the other: every rank runs its expert
    slice up to its flags (GEMM2 storing each row into the region of the token's owner), then every owner sums
    what arrived.  No kernel waits for a kernel launched later.  Three steps on different tokens (alternating
    buffer sets); every owner's rows must equal the plain layer with all 32 experts bit for bit."""
    T, per = 256, 256 // world
    full = pkg.make_inputs(num_tokens=T, seed=41, e_local=32, device=DEV)
    regions = [torch.zeros(pkg.ep_region_bytes(world, per), dtype=torch.uint8, device=DEV) for _ in range(world)]
    descs = []
    for r in range(world):
        d = pkg.EpDesc()
        d.world_size, d.rank, d.tokens_per_rank = world, r, per
        for q in range(world):
            d.region[q] = regions[q].data_ptr()
        d.wait_limit_cycles = 1 << 27
        descs.append(d)
    ctx = pkg.get_context(0)
    e_per = 32 // world
    for step in range(1, 4):
        tok = pkg.make_inputs(num_tokens=T, seed=500 + step, e_local=1, device="cpu")
        lg, hs, sc = (t.to(DEV) for t in (tok.routing_logits, tok.hidden_states, tok.hidden_states_scale))
        want = torch.empty(T, 7168, dtype=torch.bfloat16, device=DEV)
        pkg.run_moe(lg, full.routing_bias, hs, sc, *full.args()[4:8], 0, 2.5, want)
        outs = [torch.full((per, 7168), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]

        def call(r):
            sl = slice(r * e_per, (r + 1) * e_per)
            pkg.run_moe_ep_replicated(descs[r], step, lg, full.routing_bias, hs, sc, full.gemm1_weights[sl],
                                      full.gemm1_weights_scale[sl], full.gemm2_weights[sl],
                                      full.gemm2_weights_scale[sl], r * e_per, 2.5, outs[r])
        for r in range(world):          # every rank up to its flags
            ctx.debug_fault(16, 0)
            call(r)
        for r in range(world):          # every owner's sum
            ctx.debug_fault(32, 0)
            call(r)
        ctx.check()
        got = torch.cat(outs, 0)
        assert torch.equal(got, want), (step, float((got.float() - want.float()).abs().max()))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ranks_walked_through_a_dispatch_step_on_one_gpu(world, pkg):
    """Token dispatch between several ranks on ONE GPU, in three sweeps over the ranks: every rank routes and
    publishes its own tokens; every rank pulls the rows routed to its experts out of the OTHER ranks' regions,
    runs its experts and stores the rows into the owners' regions; every owner sums.  Different tokens on every
    rank and in every step; each rank's output must equal the plain layer with all 32 experts on its tokens."""
    per, e_per = 96, 32 // world
    full = pkg.make_inputs(num_tokens=8, seed=43, e_local=32, device=DEV)
    regions = [torch.zeros(pkg.ep_region_bytes(world, per), dtype=torch.uint8, device=DEV) for _ in range(world)]
    descs = []
    for r in range(world):
        d = pkg.EpDesc()
        d.world_size, d.rank, d.tokens_per_rank = world, r, per
        for q in range(world):
            d.region[q] = regions[q].data_ptr()
        d.wait_limit_cycles = 1 << 27
        descs.append(d)
    ctx = pkg.get_context(0)
    for step in range(1, 4):
        toks, wants = [], []
        for r in range(world):
            tk = pkg.make_inputs(num_tokens=per, seed=600 + 10 * step + r, e_local=1, device="cpu")
            lg, hs, sc = (t.to(DEV) for t in (tk.routing_logits, tk.hidden_states, tk.hidden_states_scale))
            toks.append((lg, hs, sc))
            w = torch.empty(per, 7168, dtype=torch.bfloat16, device=DEV)
            pkg.run_moe(lg, full.routing_bias, hs, sc, *full.args()[4:8], 0, 2.5, w)
            wants.append(w)
        outs = [torch.full((per, 7168), float("nan"), dtype=torch.bfloat16, device=DEV) for _ in range(world)]

        def call(r):
            sl = slice(r * e_per, (r + 1) * e_per)
            lg, hs, sc = toks[r]
            pkg.run_moe_ep(descs[r], step, lg, full.routing_bias, hs, sc, full.gemm1_weights[sl],
                           full.gemm1_weights_scale[sl], full.gemm2_weights[sl], full.gemm2_weights_scale[sl],
                           r * e_per, 2.5, outs[r], dispatch=True)
        for mask in (64, 128 | 16, 128 | 32):     # publish; pull + experts + flags; owners' sums
            for r in range(world):
                ctx.debug_fault(mask, 0)
                call(r)
        ctx.check()
        for r in range(world):
            assert torch.equal(outs[r], wants[r]), (step, r, float((outs[r].float() - wants[r].float()).abs().max()))


def test_peer_wait_runs_out_without_hanging(pkg):
    """Failure detection without a GPU fault: an expert-parallel step whose 'peer' never publishes
    (a second local buffer stands in for rank 1).  The flag waits give up after their limit (set short
    here), the kernels return, the status word reports it, the output rows are NaN rather than sums over
    stale data, and the context keeps working."""
    import ctypes
    moe = __import__("importlib").import_module(pkg.__name__ + ".moe")
    T = 8
    inp = pkg.make_inputs(num_tokens=T, seed=31, e_local=2, device=DEV)
    nbytes = pkg.ep_region_bytes(2, T)
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    silent_peer = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    desc = pkg.EpDesc()
    desc.world_size, desc.rank, desc.tokens_per_rank = 2, 0, T
    desc.region[0], desc.region[1] = mine.data_ptr(), silent_peer.data_ptr()
    desc.wait_limit_cycles = 1 << 27          # ~70 ms per wait instead of the serving default of many seconds
    out = torch.zeros(T, 7168, dtype=torch.bfloat16, device=DEV)
    for step, dispatch in ((1, False), (2, True)):     # the all-gather layout, then token dispatch
        out.zero_()
        pkg.run_moe_ep(desc, step, *inp.args()[:8], 0, 2.5, out, dispatch=dispatch)
        with pytest.raises(pkg.MoeError, match="105"):
            pkg.get_context(0).check()
        # a step whose peer never answered must not leave plausible numbers behind: every row is NaN
        assert bool(torch.isnan(out.float()).all())
    # the context is usable afterwards
    good = torch.empty(T, 7168, dtype=torch.bfloat16, device=DEV)
    pkg.run_moe(*inp.args(), good)
    pkg.get_context(0).check()
    assert bool(torch.isfinite(good.float()).all())


def test_tvm_ffi_entry_point(pkg, oracle):
    """Calls the layer the way the reference's harness does: through tvm-ffi, `run_moe(*inputs, output)`
    (moe/scripts/debug_correctness.py:49-55)."""
    tvm_ffi = pytest.importorskip("tvm_ffi")
    build = __import__("importlib").import_module(pkg.__name__ + ".build")
    pkg.load_library()
    path = build.build_tvm_ffi_binding()
    mod = tvm_ffi.load_module(path)
    inp = pkg.make_inputs(num_tokens=40, seed=23, e_local=8, device=DEV)
    out = torch.zeros(40, 7168, dtype=torch.bfloat16, device=DEV)
    u8 = lambda t: t.view(torch.uint8)       # the binding only takes addresses; fp8 travels as bytes
    mod.run_moe(inp.routing_logits, inp.routing_bias, u8(inp.hidden_states), inp.hidden_states_scale,
                u8(inp.gemm1_weights), inp.gemm1_weights_scale, u8(inp.gemm2_weights), inp.gemm2_weights_scale,
                0, 2.5, out)
    torch.cuda.synchronize()
    ref, _, _ = oracle.moe_forward(*inp.to("cpu").args())
    ok, stats = oracle.check_output(out, ref)
    assert ok, stats


def test_tvm_ffi_entry_point_rejects_mismatched_tensors(pkg):
    """The symbol the reference's harness loads validates dtype, rank, every dimension, device and
    contiguity of all nine tensors (the reference checks nothing, moe.cu:3045-3053): a hidden-state tensor one
    row short would make the gather read out of bounds, so it must raise instead, and name the argument."""
    tvm_ffi = pytest.importorskip("tvm_ffi")
    build = __import__("importlib").import_module(pkg.__name__ + ".build")
    pkg.load_library()
    mod = tvm_ffi.load_module(build.build_tvm_ffi_binding())
    T = 24
    inp = pkg.make_inputs(num_tokens=T, seed=29, e_local=4, device=DEV)
    out = torch.zeros(T, 7168, dtype=torch.bfloat16, device=DEV)
    u8 = lambda t: t.view(torch.uint8)
    good = [inp.routing_logits, inp.routing_bias, u8(inp.hidden_states), inp.hidden_states_scale,
            u8(inp.gemm1_weights), inp.gemm1_weights_scale, u8(inp.gemm2_weights), inp.gemm2_weights_scale, 0, 2.5, out]

    def expect_error(pos, value, word):
        args = list(good)
        args[pos] = value
        with pytest.raises(Exception, match=word):
            mod.run_moe(*args)

    expect_error(2, u8(inp.hidden_states)[:T - 1], "hidden_states")                 # one row short
    expect_error(3, inp.hidden_states_scale[:, :T - 1].contiguous(), "hidden_states_scale")
    expect_error(0, inp.routing_logits.double(), "routing_logits")                  # wrong dtype
    expect_error(3, inp.hidden_states_scale.t().contiguous().t(), "contiguous")     # right shape, wrong strides
    expect_error(5, inp.gemm1_weights_scale[:3].contiguous(), "gemm1_weights_scale")  # expert count mismatch
    expect_error(10, out[:T - 1], "output")
    expect_error(8, 254, "outside")                                                 # expert range
    mod.run_moe(*good)                                                              # still works afterwards
    torch.cuda.synchronize()
    assert bool(torch.isfinite(out.float()).all())


@pytest.mark.parametrize("T,E,tile", [(200, 8, None), (700, 4, 256)])
@pytest.mark.parametrize("mask,expected", [(1 | 4, {102, 103}), (2, {106}), (8, {102, 103})])
def test_bounded_waits_run_out_and_the_context_recovers(T, E, tile, mask, expected, pkg, monkeypatch):
    """Failure detection without a GPU fault: one forward is made with a short wait limit (2^22 clocks, about
    two milliseconds) and a role or kernel left out, so that a bounded wait inside the GEMM kernels runs
    out — a silent TMA producer starves the MMA and epilogue roles (status 102 / 103), a GEMM1 that never ran
    starves GEMM2's wait for its experts (106).  The roles give up, the kernels free tensor memory and return,
    the status word names the wait, and the next normal call reproduces the earlier result bit for bit.
    Both kernel families: the single-CTA GEMMs and (tile 256) the CTA-pair GEMMs."""
    if tile is not None:
        monkeypatch.setenv("SYFI_MOE_TOKEN_TILE", str(tile))
    inp = pkg.make_inputs(num_tokens=T, seed=41, e_local=E, device=DEV)
    before, _ = _run(pkg, inp)
    ctx = pkg.get_context(0)
    ctx.debug_fault(mask, 1 << 22)
    junk = torch.empty_like(before)
    pkg.run_moe(*inp.args(), junk)
    with pytest.raises(pkg.MoeError) as err:
        ctx.check()
    assert any(f"status {c}" in str(err.value) for c in expected), str(err.value)
    after, _ = _run(pkg, inp)                    # the hook was one-shot; the context works as before
    assert torch.equal(before, after)


def test_row_capacity_overflow_is_reported_not_written(pkg):
    """The workspace holds 3 rows per token beyond 2048 tokens (a token sends about one of its 8 routes to 32 of
    256 experts).  Every local expert made hot sends far more: the row-list kernel refuses to write past the
    capacity and the call reports status 104; after reserving the worst case the same call succeeds."""
    T = 2304
    inp = pkg.make_inputs(num_tokens=T, seed=43, e_local=32, device=DEV)
    # raise the logits of the 32 local experts so that most of every token's 8 routes stay local
    logits = inp.routing_logits.clone()
    logits[:, :32] += 6.0
    hot = pkg.MoeInputs(logits, *inp.args()[1:])
    ctx = pkg.get_context(0, T)
    ctx.reserve(T, 3 * T)                       # the default rule, made explicit
    out = torch.empty(T, 7168, dtype=torch.bfloat16, device=DEV)
    pkg.run_moe(*hot.args(), out)
    with pytest.raises(pkg.MoeError, match="status 104"):
        ctx.check()
    ctx.reserve(T, 0)                           # worst case: 8 rows per token
    out2, stats = _run(pkg, hot)
    assert stats["routes"] > 3 * T
    assert bool(torch.isfinite(out2.float()).all())
    ctx.reserve(64, 0)                          # back to a small workspace for whatever runs next
