"""The oracle against the golden vectors of the published definition reference (CPU only)."""
import os

import pytest
import torch


def _load(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name + ".pt"))


@pytest.mark.parametrize("name", ["e4_off36", "e8_t16", "cfg0"])
def test_layer_matches_published_reference(name, golden_dir, pkg, oracle):
    g = _load(golden_dir, name)
    inp = pkg.make_inputs(device="cpu", **g["make_inputs"])
    out, idx, w = oracle.moe_forward(*inp.args())
    # routing: identical index sets, identical weights (same operations on the same host)
    ok, stats = oracle.check_routing(idx, w, g["topk_idx"].to(torch.int64), g["topk_w"], w_rtol=0, w_atol=0)
    assert ok, stats
    ref = g["output_bf16_bits"].view(torch.bfloat16)
    # same math, same operation order: at most the last bf16 bit may differ through matmul blocking
    ok, stats = oracle.check_output(out, ref)
    assert ok, stats
    d = (out.float() - ref.float()).abs()
    assert float(d.max()) <= 2 ** -6, float(d.max())
    assert float((d == 0).float().mean()) > 0.99


@pytest.mark.parametrize("T", [1024, 8192])
def test_routing_matches_published_reference(T, golden_dir, pkg, oracle):
    g = _load(golden_dir, f"route_t{T}")
    inp = pkg.make_inputs(num_tokens=T, seed=0, e_local=1, device="cpu")
    idx, w = oracle.route(inp.routing_logits, inp.routing_bias, inp.routed_scaling_factor)
    a = torch.sort(idx, dim=1).values
    b = torch.sort(g["topk_idx"].to(torch.int64), dim=1).values
    assert torch.equal(a, b)
    ok, stats = oracle.check_routing(idx[:256], w[:256], g["topk_idx"][:256].to(torch.int64), g["topk_w_first256"],
                                     w_rtol=0, w_atol=0)
    assert ok, stats


def test_routing_properties(pkg, oracle):
    inp = pkg.make_inputs(num_tokens=257, seed=5, e_local=1, device="cpu")
    idx, w = oracle.route(inp.routing_logits, inp.routing_bias, 2.5)
    assert idx.shape == (257, 8) and w.shape == (257, 8)
    assert int(idx.min()) >= 0 and int(idx.max()) < 256
    assert all(len(set(r.tolist())) == 8 for r in idx)            # eight distinct experts
    assert bool(((idx // 32).unsqueeze(2) == (idx // 32).unsqueeze(1)).sum(2).max() <= 8)
    assert all(len(set((r // 32).tolist())) <= 4 for r in idx)    # at most four groups
    assert torch.allclose(w.sum(1), torch.full((257,), 2.5), atol=1e-5)


def test_tolerance_rule(oracle):
    ref = torch.randn(64, 128)
    assert oracle.check_output(ref.clone(), ref)[0]
    bad = ref.clone()
    bad[0, 0] += 1.0
    assert not oracle.check_output(bad, ref)[0]          # max-abs rule
    noisy = ref + 0.05 * torch.randn_like(ref)
    assert not oracle.check_output(noisy, ref)[0]        # 99.9 % rule
    nan = ref.clone()
    nan[3, 3] = float("nan")
    assert not oracle.check_output(nan, ref)[0]
