"""Benchmark of the fused FP8 block-scale DeepSeek-V3 MoE layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens T]

One "step" is one call of the layer on one batch of synthetic tokens.

N = 1 (default): the decode-batch configuration — T = 64 tokens, 32 local experts of 256
(offset 0), seed 0, weights generated on the device.  ``value`` is tokens/s with every
input already resident in HBM; ``e2e`` is the same call made through ``run_moe_host``
with the per-step tensors in pinned host memory (H2D of logits / bias / hidden states /
scales and D2H of the bf16 output inside the timed region; the weights are resident
parameters).  ``roofline`` is for the dominant kernel (GEMM1 with fused SwiGLU), timed
with CUDA events recorded by the library around that kernel on the launching stream.
``cpu_baseline`` times the oracle on the host cores.

N > 1 (launched by torchrun, one rank per GPU): expert parallelism with weak scaling.
Every rank brings its own batch of T tokens and owns experts [32 r, 32 r + 32); per step
the token-side tensors are all-gathered, each rank runs the layer for its experts over
the N*T gathered tokens (f32 partial sums), and a reduce-scatter sums the partials and
returns each rank its own T rows, which are rounded to bf16 once.  ``value`` counts the
N*T tokens of the job.

``--impl reference`` times the CPU restatement of the definition's reference (the oracle)
on the host cores, on a bounded sample of the same workload, and prints the same line.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
PKG = "mlsys-contest-syfi-agent-assisted_b200"

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
H, I = 7168, 2048

# DRAM bytes (read + write) of one GEMM1 launch at the N = 1 workload, from the ncu capture
# summarised in profiles/gemm_decode_T64.md (dram__bytes_read.sum + dram__bytes_write.sum).
GEMM1_NCU_TRAFFIC_BYTES = 476318208


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception as e:  # NVML missing: report that no clocks were sampled
            self.err = repr(e)

    def sample(self):
        if not self.ok:
            return
        nv = self.nv
        try:
            self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
            get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
            bits = int(get(self.h))
            names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                     0x4: "sw_power_cap", 0x80: "hw_power_brake", 0x2: "applications_clocks_setting"}
            for bit, name in names.items():
                if bits & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def run(self):
        while not self._halt.is_set():
            self.sample()
            time.sleep(self.period)

    def finish(self):
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


# --------------------------------------------------------------------------- CPU arm
class CpuArm:
    """The oracle on the host cores.  Its cost is per active expert, so when one call on the
    full workload would exceed the budget it runs on the first n active local experts only and
    the time is scaled by active_experts(full) / n."""

    def __init__(self, torch, oracle, inp_cpu, budget_s: float):
        self.torch, self.oracle, self.inp = torch, oracle, inp_cpu
        self.T = inp_cpu.routing_logits.shape[0]
        idx, _ = oracle.route(inp_cpu.routing_logits, inp_cpu.routing_bias, inp_cpu.routed_scaling_factor)
        off, E = inp_cpu.local_expert_offset, inp_cpu.gemm1_weights.shape[0]
        self.active = [e for e in range(E) if bool((idx == off + e).any())] or [0]
        t1 = self._run(1)                       # calibration: one active expert
        self.n = max(1, min(len(self.active), int(budget_s / max(t1, 1e-3))))

    def _run(self, n):
        i, e_hi = self.inp, self.active[n - 1] + 1
        t0 = time.perf_counter()
        self.oracle.moe_forward(i.routing_logits, i.routing_bias, i.hidden_states, i.hidden_states_scale,
                                i.gemm1_weights[:e_hi], i.gemm1_weights_scale[:e_hi], i.gemm2_weights[:e_hi],
                                i.gemm2_weights_scale[:e_hi], i.local_expert_offset, i.routed_scaling_factor)
        return time.perf_counter() - t0

    def step(self):
        """One timed call; returns the time of the full workload in seconds (scaled if sampled)."""
        self.last = self._run(self.n)
        return self.last * len(self.active) / self.n

    def describe(self, full_s):
        n, a = self.n, len(self.active)
        sample = (f"oracle (CPU restatement of the definition's reference) on T={self.T} tokens and the first {n} of "
                  f"{a} active local experts, {self.last:.2f} s per call"
                  + ("" if n == a else f", scaled by {a}/{n} to the full workload"))
        return {"value": self.T / full_s, "unit": UNIT, "cores": int(self.torch.get_num_threads()), "kind": "port",
                "sample": sample}


def run_reference_arm(args):
    import torch
    rank, local_rank, world = dist_env()
    if rank != 0:
        return 0
    pkg = importlib.import_module(PKG)
    oracle = importlib.import_module("oracle.moe_oracle")
    T = args.tokens
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"   # the device only draws the weights faster
    inp = pkg.make_inputs(num_tokens=T, seed=0, e_local=32, device=dev).to("cpu")
    W, K = max(args.warmup, 0), max(args.steps, 1)
    per_call_budget = max(2.0, min(30.0, 150.0 / (W + K)))
    arm = CpuArm(torch, oracle, inp, per_call_budget)
    times = []
    for i in range(W + K):
        fs = arm.step()
        if i >= W:
            times.append(fs)
    ms = 1e3 * sum(times) / len(times)
    value = T / (ms / 1e3)
    base = arm.describe(ms / 1e3)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"decode batch T={T}, 32 local experts of 256, offset 0, seed 0 (CPU oracle)",
                       "tokens": T, "local_experts": 32},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


# --------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE layer has no CPU path")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if world > 8:
        raise SystemExit("at most 8 ranks (8 x 32 experts = the 256 global experts)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pkg = importlib.import_module(PKG)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    T = args.tokens
    W, K = max(args.warmup, 3), max(args.steps, 1)
    # token-side tensors: this rank's own batch; weights: this rank's 32 experts
    inp = pkg.make_inputs(num_tokens=T, seed=rank, e_local=32, local_expert_offset=32 * rank if world > 1 else 0,
                          device=dev, weight_seed=rank)
    ctx = pkg.get_context(local_rank, T * world)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

    peer_ok = False
    if world == 1:
        def step():
            pkg.run_moe(*inp.args(), out)
        n_tok_layer = T
    else:
        ep = pkg.ExpertParallelMoe(inp.gemm1_weights, inp.gemm1_weights_scale, inp.gemm2_weights,
                                   inp.gemm2_weights_scale, inp.local_expert_offset, inp.routed_scaling_factor)
        # token all-gather and reduce-scatter through the library's own peer-memory kernels when the
        # ranks can map each other's memory, NCCL collectives otherwise
        peer_ok = ep.enable_peer_exchange(T, dev)
        flag = torch.tensor([1 if peer_ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            ep._peer = None
            peer_ok = False

        def step():
            ep.forward_sharded(inp.routing_logits, inp.routing_bias, inp.hidden_states, inp.hidden_states_scale, out)
        n_tok_layer = T * world

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        step()
    barrier()
    stats = ctx.check()

    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(K):
        step()
    e1.record()
    sampler.sample()
    barrier()
    clocks = sampler.finish()
    ms = e0.elapsed_time(e1) / K
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    stats = ctx.check()
    launches = ctx.launch_count() * K
    value = world * T / (ms / 1e3)

    # ---- per-kernel pass (same steps, events around every kernel) -> roofline of GEMM1
    ctx.set_stage_timing(True)
    Ks = min(K, 200)
    acc = {}
    for _ in range(Ks):
        step()
        for k, v in ctx.last_stage_ms().items():
            acc[k] = acc.get(k, 0.0) + v
    ctx.set_stage_timing(False)
    stage_ms = {k: v / Ks for k, v in acc.items()}
    rows, active = stats["routes"], stats["active_experts"]
    gemm1_bytes = active * (2 * I * H + 4 * (2 * I // 128) * (H // 128)) + rows * (H + 4 * (H // 128)) \
        + rows * (2 * I + 4 * (I // 128))
    peak, peak_src = measured_peaks()
    achieved = gemm1_bytes / (stage_ms["gemm1"] * 1e-3) / 1e9
    roofline = {"kernel": "grouped_gemm_kernel<1> (GEMM1 + SwiGLU + requantisation)", "bound": "hbm",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": (GEMM1_NCU_TRAFFIC_BYTES if (world == 1 and T == 64) else None), "algorithmic_bytes": gemm1_bytes,
                "launch_ms": stage_ms["gemm1"], "peak_source": peak_src, "timed_steps": Ks,
                "stage_ms": stage_ms}
    flops, layer_bytes = pkg.algorithmic_work(rows, active, n_tok_layer)

    # ---- end to end: per-step tensors in pinned host memory
    h_in = [t.cpu().pin_memory() for t in (inp.routing_logits, inp.routing_bias, inp.hidden_states,
                                            inp.hidden_states_scale)]
    h_out = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in h_in)
    d2h = h_out.numel() * h_out.element_size()
    if world == 1:
        def e2e_step():
            pkg.run_moe_host(*h_in, inp.gemm1_weights, inp.gemm1_weights_scale, inp.gemm2_weights,
                             inp.gemm2_weights_scale, inp.local_expert_offset, inp.routed_scaling_factor, h_out)
    else:
        d_in = [inp.routing_logits, inp.routing_bias, inp.hidden_states, inp.hidden_states_scale]

        def e2e_step():
            for d, h in zip(d_in, h_in):
                d.copy_(h, non_blocking=True)
            step()
            h_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
    Ke = min(K, 300)
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(Ke):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / Ke
    if dist is not None:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    ctx.check()

    # ---- the same steps on weights re-laid out once by prepack_weights (1 GPU only; an extra, not the headline)
    prepacked = None
    if world == 1:
        packed = pkg.prepack_weights(inp.gemm1_weights, inp.gemm2_weights)
        out_p = torch.empty_like(out)

        def packed_step():
            pkg.run_moe_prepacked(inp.routing_logits, inp.routing_bias, inp.hidden_states, inp.hidden_states_scale,
                                  packed, inp.gemm1_weights_scale, inp.gemm2_weights_scale, inp.local_expert_offset,
                                  inp.routed_scaling_factor, out_p)
        for _ in range(max(W, 3)):
            packed_step()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(K):
            packed_step()
        p1.record()
        torch.cuda.synchronize(dev)
        pms = p0.elapsed_time(p1) / K
        step()
        torch.cuda.synchronize(dev)
        prepacked = {"ms_per_step": pms, "value": T / (pms / 1e3), "unit": UNIT,
                     "bit_identical_to_unpacked": bool(torch.equal(out, out_p)),
                     "note": "weights re-laid out once into consumption-order swizzled tiles, fetched with untiled bulk copies"}
        ctx.check()
        del packed

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f8e4m3",
            "data": "synthetic",
            "config": {"workload": (f"decode batch T={T} per rank, 32 local experts per rank of 256 global, seed = rank"
                                    + ("" if world == 1 else f"; expert parallel over {world} ranks: all-gather tokens, "
                                       "reduce-scatter f32 partials ("
                                       + ("own kernels over peer memory" if peer_ok else "NCCL") + ")")),
                       "tokens_per_rank": T, "local_experts": 32, "routes": rows, "active_experts": active,
                       "l2": f"inputs larger than L2: {active * 44050944 / 1e6:.0f} MB of active-expert weights per step",
                       "layer_algorithmic_bytes": layer_bytes, "layer_flops": flops,
                       "layer_gbs": layer_bytes / (ms * 1e-3) / 1e9, "layer_tflops": flops / (ms * 1e-3) / 1e12},
            "clocks": clocks,
            "e2e": {"value": world * T / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": Ke},
            "gpu_launches": launches, "roofline": roofline}
    if prepacked is not None:
        line["prepacked"] = prepacked

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        oracle = importlib.import_module("oracle.moe_oracle")
        arm = CpuArm(torch, oracle, inp.to("cpu"), budget_s=25.0)
        line["cpu_baseline"] = arm.describe(arm.step())
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
