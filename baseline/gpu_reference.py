"""Times the reference's own CUDA implementation of the layer on this GPU, for a same-box comparison.

    python baseline/gpu_reference.py [--tokens 64,1024,8192] [--iters 100]

Loads ``baseline/_ref/libref_moe.so`` — the reference's ``moe/solution/cuda/moe.cu`` compiled UNMODIFIED
for sm_100a by ``build.build_reference_gpu()`` — through tvm-ffi, the way the reference's harness does
(``moe/scripts/debug_correctness.py:49-55``), and calls ``run_moe(*inputs, output)`` on the same seeded
workloads the benchmark uses.  Protocol of the reference's own runs (``moe/scripts/run_modal.py:41-46``):
3 warm-up calls, then ``--iters`` timed calls between two CUDA events on the stream the reference
launches on (stream 0).  Prints one JSON object: per token count the time per call, tokens/s and the
agreement with the oracle under the tolerance this repository's tests use and under the contest's rule.

This file never touches this repository's kernels; it is the measured baseline, not the product.
The reference's device-side waits are unbounded (``moe.cu:1298-1305``), so callers run this script as
a child process with a time limit.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
PKG = "mlsys-contest-syfi-agent-assisted_b200"
LIB = os.path.join(ROOT, "baseline", "_ref", "libref_moe.so")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="64,1024,8192")
    ap.add_argument("--iters", type=int, default=100)
    args = ap.parse_args()
    if not os.path.exists(LIB):
        print(json.dumps({"unavailable": "baseline/_ref/libref_moe.so has not been built"}))
        return 0
    import torch
    import tvm_ffi
    workloads = importlib.import_module(PKG + ".workloads")
    oracle = importlib.import_module("oracle.moe_oracle")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    mod = tvm_ffi.load_module(LIB)
    u8 = lambda t: t.view(torch.uint8)
    weights = workloads.make_inputs(num_tokens=1, seed=0, e_local=32, device=dev)
    res = {}
    for T in [int(x) for x in args.tokens.split(",")]:
        tk = workloads.make_inputs(num_tokens=T, seed=0, e_local=1, device="cpu")
        inp = workloads.MoeInputs(tk.routing_logits.to(dev), tk.routing_bias.to(dev), tk.hidden_states.to(dev),
                                  tk.hidden_states_scale.to(dev), weights.gemm1_weights, weights.gemm1_weights_scale,
                                  weights.gemm2_weights, weights.gemm2_weights_scale, 0, 2.5)
        out = torch.zeros(T, 7168, dtype=torch.bfloat16, device=dev)

        def call():
            mod.run_moe(inp.routing_logits, inp.routing_bias, u8(inp.hidden_states), inp.hidden_states_scale,
                        u8(inp.gemm1_weights), inp.gemm1_weights_scale, u8(inp.gemm2_weights),
                        inp.gemm2_weights_scale, 0, 2.5, out)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.iters
        ref, _, _ = oracle.moe_forward(*inp.args())
        ok, st = oracle.check_output(out, ref)
        d = (out.float() - ref.float()).abs()
        contest = float(((d <= 1.0) | (d <= 0.3 * ref.float().abs())).float().mean())
        res[f"T{T}"] = {"tokens": T, "ms_per_step": ms, "tokens_per_s": T / (ms / 1e3), "iters": args.iters,
                        "passes_repo_tolerance": bool(ok), "max_abs_vs_oracle": st["max_abs"], "limit": st["limit"],
                        "frac_within": st["frac_within"], "contest_match_ratio": contest}
        del ref
    print(json.dumps({"impl": "reference CUDA kernel (moe/solution/cuda/moe.cu, unmodified, sm_100a)", "results": res}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
