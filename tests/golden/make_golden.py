"""Generate the golden vectors that pin the oracle (run once, offline; commit the outputs).

Runs the PUBLISHED PyTorch reference of the definition
``moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048`` — the function
``_trtllm_fp8_block_scale_moe_ds_routing_reference`` of flashinfer-python
0.6.11.post2 (flashinfer/trace/templates/moe.py:109-183) — on seeded inputs from
this repository's workload generator, and stores what it returned.  Routing is
captured by wrapping the helper the reference hands its routing result to
(templates/moe.py:170-183), so nothing about routing is restated here.

    python tests/golden/make_golden.py            # writes tests/golden/*.pt

Cases (all CPU-generated inputs, so they reproduce on any host with this torch build):
  e8_t16     T=16, 8 local experts, offset 0, seed 0      routing + bf16 output
  cfg0       T=16, 32 local experts, offset 0, seed 0     routing + bf16 output (the CPU-runnable config)
  e4_off36   T=24, 4 local experts, offset 36, seed 3     routing + bf16 output (non-zero expert offset)
  route_t1024 / route_t8192   routing only at the prefill sizes
"""
import importlib
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
pkg = importlib.import_module("mlsys-contest-syfi-agent-assisted_b200.workloads")

import flashinfer.trace.templates.moe as fi_moe  # noqa: E402


def run_reference(inp, experts=True):
    captured = {}
    orig = fi_moe._fp8_moe_run_experts

    def capture(hs, hss, w1, w1s, w2, w2s, weights, topk_idx, off, e_global):
        captured["topk_w"] = weights.clone()
        captured["topk_idx"] = topk_idx.clone()
        if not experts:
            return torch.zeros(1)
        return orig(hs, hss, w1, w1s, w2, w2s, weights, topk_idx, off, e_global)

    fi_moe._fp8_moe_run_experts = capture
    try:
        out = fi_moe._trtllm_fp8_block_scale_moe_ds_routing_reference(
            inp.routing_logits, inp.routing_bias, inp.hidden_states, inp.hidden_states_scale,
            inp.gemm1_weights, inp.gemm1_weights_scale, inp.gemm2_weights, inp.gemm2_weights_scale,
            8, 8, 4, inp.local_expert_offset, inp.routed_scaling_factor)
    finally:
        fi_moe._fp8_moe_run_experts = orig
    return out, captured["topk_idx"], captured["topk_w"]


def main():
    cases = [
        ("e8_t16", dict(num_tokens=16, seed=0, e_local=8, local_expert_offset=0), True),
        ("e4_off36", dict(num_tokens=24, seed=3, e_local=4, local_expert_offset=36), True),
        ("cfg0", dict(num_tokens=16, seed=0, e_local=32, local_expert_offset=0), True),
    ]
    for name, kw, experts in cases:
        t0 = time.time()
        inp = pkg.make_inputs(device="cpu", **kw)
        t1 = time.time()
        out, idx, w = run_reference(inp, experts)
        t2 = time.time()
        torch.save({"make_inputs": kw, "topk_idx": idx.to(torch.int16), "topk_w": w,
                    "output_bf16_bits": out.view(torch.int16),
                    "flashinfer": "0.6.11.post2", "torch": str(torch.__version__)},
                   os.path.join(HERE, name + ".pt"))
        print(f"{name}: gen {t1 - t0:.1f}s ref {t2 - t1:.1f}s max|out|={out.float().abs().max():.4f}", flush=True)
    for T in (1024, 8192):
        # routing only: one local expert keeps weight generation negligible
        inp = pkg.make_inputs(num_tokens=T, seed=0, e_local=1, device="cpu")
        _, idx, w = run_reference(inp, experts=False)
        torch.save({"make_inputs": dict(num_tokens=T, seed=0), "topk_idx": idx.to(torch.uint8),
                    "topk_w_first256": w[:256].clone()},
                   os.path.join(HERE, f"route_t{T}.pt"))
        print(f"route_t{T}: done", flush=True)


if __name__ == "__main__":
    main()
