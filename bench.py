"""Benchmark of the fused FP8 block-scale DeepSeek-V3 MoE layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config 3|4] [--tokens T] [--no-cpu-baseline] [--no-decode] [--no-parity]
                    [--operator moe|dsa-indexer]

One "step" is one call of the layer on one batch of synthetic tokens.

Workloads (seeded synthetic tensors with the definition's shapes and value distributions):

* config 3 (default), the largest single-GPU configuration: T = 8192 tokens, the 32 local experts
  [0, 32) of 256, seed 0.  On N > 1 GPUs (launched by torchrun, one rank per GPU) the SAME layer is
  sharded by expert: rank r owns experts [32 r / N, 32 (r + 1) / N) (slices of the same seed-0
  weights), every rank holds all T tokens and computes the f32 partial of its experts; the partial rows
  are summed over the ranks and each rank ends with the bf16 rows of its own T / N tokens (a
  reduce-scatter by rows, fused into GEMM2 over NVLink peer memory: its epilogue stores every expert row into
  the memory of the token's owner, which sums them; NCCL's reduce-scatter when the ranks cannot map each other).  Total work is fixed as N grows: "strong"
  scaling.
* config 4 (``--config 4``), the full 256-expert layer with load imbalance: T = 4096 tokens shared by
  all ranks, logits of 16 hot experts raised by 1.5, rank r owns experts [32 r, 32 r + 32) drawn from
  weight seed r; meant for N = 8 (fewer ranks compute the first 32 N experts only).
* ``--tokens T`` replaces the token count of config 3 (sweeps; T = 64 is the decode batch).

``value`` is tokens/s with every input already resident in HBM, timed with CUDA events on the
launching stream (max over ranks).  ``e2e`` is the same call made through ``run_moe_host`` with the
per-step tensors in pinned host memory (H2D of logits / bias / hidden states / scales and D2H of the
bf16 output inside the timed region; the weights are resident parameters).  ``roofline`` is for the
dominant kernel (GEMM1 with fused SwiGLU and requantisation), timed with CUDA events the library
records around that kernel: tensor-bound (TFLOP/s) from 4096 tokens on, HBM-bound (GB/s) below.
``decode`` repeats the measurement for the decode batch (T = 64) and adds T = 16 and T = 1024: the
metric is quoted against T.  ``parity`` compares one step's output with the oracle (executed with torch
on the GPU, summed over ranks in f32) outside the timed region.  ``cpu_baseline`` times the oracle on the
host cores on a bounded sample of the workload.

``gpu_reference`` is the reference's own CUDA kernel (``moe/solution/cuda/moe.cu`` compiled unmodified for
sm_100a into ``baseline/_ref``), timed on the same GPU and workloads by ``baseline/gpu_reference.py``.

``--impl reference`` times the CPU restatement of the definition's reference (the oracle) on the host
cores, on a bounded sample of the same workload, and prints the same line.

At N > 1 the line also carries ``return_leg`` (the step with GEMM2 storing its rows into the owners' memory against
the step with the combine-and-push kernel), ``sharded`` (the serving layout, every rank bringing its own T / N tokens:
token dispatch against the all-gather, and whether its output equals the replicated step's bit for bit) and an ``e2e``
measured on the serving layout.  ``--operator dsa-indexer`` times the sibling operator (the DSA top-k indexer) on one
GPU instead and prints a line of the same shape.
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
GEMM1_FLOP_PER_ROW = 2 * H * 2 * I          # 58,720,256
NOMINAL_FP8_TFLOPS = 4500.0                 # dense FP8, NVIDIA's B200 figure


def workload_name(config: int, T: int) -> str:
    if config == 4:
        return (f"config 4: T={T} tokens shared by all ranks, 256 experts in 8 x 32 (rank r: experts [32r, 32r+32), "
                "weight seed r), 16 hot experts (logits +1.5, hot seed 1), token seed 0")
    return f"config 3: T={T} tokens, 32 local experts [0, 32) of 256 global, seed 0, routed_scaling_factor 2.5"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback (earlier measurement on this pool)"}


def ncu_traffic(kernel_key: str):
    """DRAM bytes per launch from the committed ncu summary (profiles/ncu_traffic.json), or None."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            return json.load(f).get(kernel_key)
    except Exception:
        return None


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.005):
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


def build_inputs(pkg, args, rank, world, dev):
    """This rank's inputs: (MoeInputs with the rank's expert slice, experts per rank)."""
    T = args.tokens
    if args.config == 4:
        inp = pkg.make_inputs(num_tokens=T, seed=0, e_local=32, local_expert_offset=32 * rank, device=dev,
                              hot_experts=16, weight_seed=rank)
        return inp, 32
    inp = pkg.make_inputs(num_tokens=T, seed=0, e_local=args.experts if world == 1 else 32, local_expert_offset=0, device=dev)
    if world == 1:
        return inp, args.experts
    per = 32 // world
    sl = slice(rank * per, (rank + 1) * per)
    part = pkg.MoeInputs(inp.routing_logits, inp.routing_bias, inp.hidden_states, inp.hidden_states_scale,
                         inp.gemm1_weights[sl].clone(), inp.gemm1_weights_scale[sl].clone(),
                         inp.gemm2_weights[sl].clone(), inp.gemm2_weights_scale[sl].clone(), rank * per,
                         inp.routed_scaling_factor)
    del inp
    return part, per


def run_reference_arm(args):
    import torch
    rank, local_rank, world = dist_env()
    if rank != 0:
        return 0
    pkg = importlib.import_module(PKG)
    oracle = importlib.import_module("oracle.moe_oracle")
    T = args.tokens
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"   # the device only draws the weights faster
    inp, _ = build_inputs(pkg, args, 0, 1, dev)
    inp = inp.to("cpu")
    W, K = max(args.warmup, 0), max(args.steps, 1)
    W, K = min(W, 1), min(K, 3)               # bounded: every step is tens of seconds of host work
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
            "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if args.config == 3 else "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args.config, T), "tokens": T, "local_experts": 32,
                       "note": "the reference arm is the CPU oracle on rank 0's experts (single-GPU workload)"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


def run_gpu_reference(T: int):
    """The reference's own sm_100a kernel (moe/solution/cuda/moe.cu, compiled unmodified) timed on this GPU
    on the same workloads, by baseline/gpu_reference.py in a child process."""
    import subprocess
    lib = os.path.join(ROOT, "baseline", "_ref", "libref_moe.so")
    if not os.path.exists(lib):
        return {"unavailable": "baseline/_ref/libref_moe.so has not been built (the reference source was not at hand)"}
    tokens = sorted({64, 1024, T})
    try:
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "gpu_reference.py"), "--tokens",
                               ",".join(str(t) for t in tokens), "--iters", "50"], capture_output=True, text=True,
                              timeout=240)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference kernel did not finish within 240 s"}
    for ln in reversed(proc.stdout.strip().splitlines()):
        if ln.startswith("{"):
            try:
                return json.loads(ln)
            except ValueError:
                break
    return {"unavailable": "no result line", "stderr_tail": proc.stderr[-300:]}


def time_layer(torch, step, K, barrier, dist, dev):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(K):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / K
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def stage_pass(ctx, step, n):
    ctx.set_stage_timing(True)
    acc = {}
    for _ in range(n):
        step()
        for k, v in ctx.last_stage_ms().items():
            acc[k] = acc.get(k, 0.0) + v
    ctx.set_stage_timing(False)
    return {k: v / n for k, v in acc.items()}


def gemm1_roofline(T, rows, active, stage_ms, peaks, world):
    """Roofline entry of the dominant kernel for one workload."""
    t = stage_ms["gemm1"] * 1e-3
    if T >= 4096:
        flops = rows * GEMM1_FLOP_PER_ROW
        achieved = flops / t / 1e12
        peak = 2.0 * peaks["bf16_tflops_sustained"]
        key = "pair_gemm_kernel<1>@T8192_E32" if (T == 8192 and world == 1 and active >= 24) else None
        return {"kernel": "pair_gemm_kernel<1> (GEMM1 + SwiGLU + two-term requantisation, CTA pairs, tcgen05 cta_group::2)",
                "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_note": "no FP8 figure in MEASURED_PEAKS.json: 2 x bf16_tflops_sustained as the measured proxy "
                             "(kernel timed inside a long step)",
                "frac_of_nominal_fp8": achieved / NOMINAL_FP8_TFLOPS, "nominal_fp8_tflops": NOMINAL_FP8_TFLOPS,
                "traffic": ncu_traffic(key) if key else None, "algorithmic_flops": flops,
                "launch_ms": stage_ms["gemm1"], "peak_source": peaks["source"]}
    gemm1_bytes = active * (2 * I * H + 4 * (2 * I // 128) * (H // 128)) + rows * (H + 4 * (H // 128)) \
        + rows * (2 * I + 4 * (I // 128))
    achieved = gemm1_bytes / t / 1e9
    key = "grouped_gemm_kernel<1,32>@T64_E32" if (T == 64 and world == 1) else None
    return {"kernel": "grouped_gemm_kernel<1> (GEMM1 + SwiGLU + two-term requantisation)", "bound": "hbm",
            "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "traffic": ncu_traffic(key) if key else None, "algorithmic_bytes": gemm1_bytes,
            "launch_ms": stage_ms["gemm1"], "peak_source": peaks["source"]}


# --------------------------------------------------------------------------- GPU arm
def run_dsa_indexer(args):
    """The sibling operator on one GPU: 32 sequences of 65536 tokens (2 M tokens, 277 MB of index cache: larger than
    L2), scored and cut to the best 2048 each.  One JSON line: scored tokens per second, the HBM roofline of the
    operator as a whole (algorithmic bytes = the cache bytes of the sequences' tokens + queries + output), the
    reference's own entry point (pure torch, dsa_indexer/solution/python/dsa_topk_indexer.py, restated by the oracle)
    evaluated on the same GPU and on the host cores, and one parity step."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the indexer has no CPU path")
    pkg = importlib.import_module(PKG)
    dsa_oracle = importlib.import_module("oracle.dsa_oracle")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    seq_lens = [65536] * 32
    W, K = max(args.warmup, 3), max(min(args.steps, 100), 1)
    inputs = tuple(t.to(dev) for t in dsa_oracle.make_inputs(seq_lens, seed=0))
    q, cache, w, sl, table = inputs
    out = torch.empty(len(seq_lens), dsa_oracle.TOPK, dtype=torch.int32, device=dev)

    def step():
        pkg.run_dsa_topk_indexer(q, cache, w, sl, table, out)
    for _ in range(W):
        step()
    pkg.dsa_check()
    peaks = measured_peaks()
    sampler = ClockSampler(0)
    sampler.start()
    ms = time_layer(torch, step, K, torch.cuda.synchronize, None, dev)
    sampler.sample()
    clocks = sampler.finish()
    pkg.dsa_check()
    tokens = sum(seq_lens)
    nbytes = tokens * 132 + q.numel() + w.numel() * 4 + out.numel() * 4
    want, scores = dsa_oracle.topk_indexer(*inputs)           # the reference's torch code on this GPU: parity ...
    ok, pstats = dsa_oracle.check_topk(out, want, scores, sl.cpu(), table.cpu())
    ref_ms = time_layer(torch, lambda: dsa_oracle.topk_indexer(*inputs), 3, torch.cuda.synchronize, None, dev)   # ... and time
    line = {"metric": "dsa_indexer_scored_tokens_per_s", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1,
            "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f8e4m3", "data": "synthetic",
            "config": {"workload": "dsa_topk_indexer_fp8_h64_d128_topk2048_ps64: 32 sequences of 65536 tokens, pages "
                                   "scattered over a 277 MB cache, seed 0", "l2": "inputs larger than L2"},
            "clocks": clocks, "gpu_launches": 2 * K,
            "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                         "peak_source": peaks.get("source", "MEASURED_PEAKS.json"), "kernel": "dsa_score_kernel + dsa_select_kernel"},
            "parity": {"ok": bool(ok), "selection": pstats,
                       "against": "the reference's torch entry point restated by the oracle, evaluated on this GPU"},
            "gpu_reference": {"impl": "the definition's configured entry point (pure torch) on the same GPU",
                              "ms_per_step": ref_ms, "times_slower": ref_ms / ms}}
    if not args.no_cpu_baseline:
        small = dsa_oracle.make_inputs([65536] * 2, seed=0)
        t0 = time.perf_counter()
        dsa_oracle.topk_indexer(*small)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 2 * 65536 / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "the oracle on 2 of the 32 sequences, %.2f s" % dt}
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=3, choices=[3, 4])
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--experts", type=int, default=32, help="1 GPU, config 3: only the first E local experts (profiling on a small case)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-gpu-reference", action="store_true")
    ap.add_argument("--operator", default="moe", choices=["moe", "dsa-indexer"],
                    help="dsa-indexer: the sibling operator (DSA top-k indexer) on one GPU instead of the MoE layer")
    args = ap.parse_args()
    if args.tokens is None:
        args.tokens = 8192 if args.config == 3 else 4096
    if args.operator == "dsa-indexer":
        return run_dsa_indexer(args)
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE layer has no CPU path")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    if world > 8 or 32 % world != 0 or args.tokens % world != 0:
        raise SystemExit("1, 2, 4 or 8 ranks, and a token count they divide")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pkg = importlib.import_module(PKG)
    oracle = importlib.import_module("oracle.moe_oracle")
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    T = args.tokens
    W, K = max(args.warmup, 3), max(args.steps, 1)
    inp, e_per_rank = build_inputs(pkg, args, rank, world, dev)
    ctx = pkg.get_context(local_rank, T)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    peaks = measured_peaks()
    peer_ok = False

    if world == 1:
        def step():
            pkg.run_moe(*inp.args(), out)
    else:
        ep = pkg.ExpertParallelMoe(inp.gemm1_weights, inp.gemm1_weights_scale, inp.gemm2_weights,
                                   inp.gemm2_weights_scale, inp.local_expert_offset, inp.routed_scaling_factor)

        # every rank ends with the rows of its own T / N tokens (reduce-scatter by rows): fused into the
        # layer's combine kernel over peer memory when the ranks can map each other, NCCL otherwise
        peer_ok = ep.enable_peer_exchange(T // world, dev)
        flag = torch.tensor([1 if peer_ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            ep._peer = None
            peer_ok = False
        out = torch.empty(T // world, H, dtype=torch.bfloat16, device=dev)

        def step():
            ep.forward_replicated(inp.routing_logits, inp.routing_bias, inp.hidden_states, inp.hidden_states_scale, out,
                                  scatter_rows=True)

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
    ms = time_layer(torch, step, K, barrier, dist, dev)
    sampler.sample()
    clocks = sampler.finish()
    stats = ctx.check()
    launches = ctx.launch_count() * K
    value = T / (ms / 1e3)

    # ---- parity of one step against the oracle (torch on the GPU, f32 partials summed over ranks); untimed
    parity = None
    if not args.no_parity:
        out.fill_(float("nan"))
        step()
        barrier()
        ref32, ridx, rw = oracle.moe_forward(*inp.args(), return_f32=True)
        if dist is not None:
            dist.all_reduce(ref32)
        mine = slice(rank * (T // world), (rank + 1) * (T // world))
        ok, ostats = oracle.check_output(out, ref32[mine].to(torch.bfloat16))
        idx, w = ctx.last_routing(T)
        golden = os.path.join(ROOT, "tests", "golden", f"route_t{T}.pt")
        if args.config == 3 and os.path.exists(golden):
            # this workload's routing as the published reference computed it (stored expert ids of every token,
            # weights of the first 256): no host arithmetic in the check
            g = torch.load(golden)
            mine_sets = torch.sort(idx.cpu().to(torch.int64), dim=1).values
            their_sets = torch.sort(g["topk_idx"].to(torch.int64), dim=1).values
            wok, wstats = oracle.check_routing(idx[:256], w[:256], g["topk_idx"][:256].to(torch.int64), g["topk_w_first256"])
            rstats = {"idx_equal": bool(torch.equal(mine_sets, their_sets)), "weights_close": wstats["weights_close"],
                      "tokens_differing": int((mine_sets != their_sets).any(dim=1).sum())}
            rok = rstats["idx_equal"] and wok
            routing_against = "stored routing of the published reference for this workload (tests/golden)"
        else:
            cidx, cw = oracle.route(inp.routing_logits.cpu(), inp.routing_bias.cpu(), inp.routed_scaling_factor)
            rok, rstats = oracle.check_routing(idx, w, cidx, cw)
            routing_against = "the oracle's CPU route"

        flag = torch.tensor([1 if (ok and rok) else 0], device=dev)
        if dist is not None:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        parity = {"ok": bool(int(flag.item())), "output": ostats, "routing": rstats,
                  "against": "oracle with torch on the GPU, f32 partials summed over ranks, one rounding to bf16; "
                             "routing against " + routing_against}
        del ref32

    # ---- the return leg both ways: GEMM2 storing its rows straight into the owners' memory (the default, timed
    # above) against rows kept local + a combine kernel that pushes partial rows after GEMM2
    return_leg = None
    if world > 1 and peer_ok:
        barrier()
        os.environ["SYFI_MOE_EP_RETURN"] = "push"
        for _ in range(3):
            step()
        ms_push = time_layer(torch, step, K, barrier, dist, dev)
        del os.environ["SYFI_MOE_EP_RETURN"]
        barrier()
        step()
        barrier()
        ctx.check()
        return_leg = {"rows_stored_by_gemm2_into_owner_memory_ms": ms, "combine_kernel_pushes_partial_rows_ms": ms_push}

    # ---- the serving layout on the same tokens: every rank brings only its own T/N tokens (token dispatch: routed
    # rows pulled over NVLink; beside it the all-gather of every token).  Same rows in the same order reach every
    # expert as with replicated tokens, so the outputs must equal the replicated step's bit for bit.
    sharded = None
    if world > 1 and peer_ok:
        mine = slice(rank * (T // world), (rank + 1) * (T // world))
        s_in = (inp.routing_logits[mine].contiguous(), inp.hidden_states[mine].contiguous(),
                inp.hidden_states_scale[:, mine].contiguous())
        o_d, o_g = torch.empty_like(out), torch.empty_like(out)

        def dstep():
            ep.forward_sharded(s_in[0], inp.routing_bias, s_in[1], s_in[2], o_d, dispatch=True)

        def gstep():
            ep.forward_sharded(s_in[0], inp.routing_bias, s_in[1], s_in[2], o_g, dispatch=False)
        for _ in range(3):
            dstep()
            gstep()
        barrier()
        ms_d = time_layer(torch, dstep, K, barrier, dist, dev)
        ms_g = time_layer(torch, gstep, K, barrier, dist, dev)
        step()
        barrier()
        same = torch.tensor([1 if (torch.equal(o_d, out) and torch.equal(o_g, out)) else 0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        ctx.check()
        sharded = {"tokens_per_rank": T // world, "unit": UNIT,
                   "token_dispatch": {"ms_per_step": ms_d, "value": T / (ms_d / 1e3)},
                   "all_gather": {"ms_per_step": ms_g, "value": T / (ms_g / 1e3)},
                   "bit_identical_to_replicated_step": bool(int(same.item())),
                   "note": "each rank passes its own T/N tokens; dispatch = route own tokens, peers pull only the rows "
                           "routed to their experts; all_gather = every token to every rank; both return partial rows "
                           "to the owners through the fused combine + push"}

    # ---- per-kernel pass (same steps, events around every kernel) -> roofline of GEMM1
    Ks = min(K, 100)
    stage_ms = stage_pass(ctx, step, Ks)
    rows, active = stats["routes"], stats["active_experts"]
    roofline = gemm1_roofline(T, rows, active, stage_ms, peaks, world)
    roofline["stage_ms"] = stage_ms
    roofline["timed_steps"] = Ks
    flops, layer_bytes = pkg.algorithmic_work(rows, active, T)
    if dist is not None:
        tot = torch.tensor([float(rows), float(flops)], device=dev, dtype=torch.float64)
        dist.all_reduce(tot)
        rows_all, flops_all = int(tot[0].item()), float(tot[1].item())
    else:
        rows_all, flops_all = rows, flops

    # ---- end to end: per-step tensors in pinned host memory
    h_in = [t.cpu().pin_memory() for t in (inp.routing_logits, inp.routing_bias, inp.hidden_states,
                                            inp.hidden_states_scale)]
    h_out = torch.empty(out.shape[0], H, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in h_in)
    d2h = h_out.numel() * h_out.element_size()
    if world == 1:
        def e2e_step():
            pkg.run_moe_host(*h_in, inp.gemm1_weights, inp.gemm1_weights_scale, inp.gemm2_weights,
                             inp.gemm2_weights_scale, inp.local_expert_offset, inp.routed_scaling_factor, h_out)
    elif peer_ok:
        # N GPUs end to end: every rank's host holds its own T/N tokens (the serving layout); they travel in, the
        # ranks exchange the routed rows (token dispatch), and every rank's own output rows travel back
        mine = slice(rank * (T // world), (rank + 1) * (T // world))
        d_in = [inp.routing_logits[mine].contiguous(), inp.routing_bias, inp.hidden_states[mine].contiguous(),
                inp.hidden_states_scale[:, mine].contiguous()]
        h_in = [t.cpu().pin_memory() for t in d_in]
        h2d = sum(t.numel() * t.element_size() for t in h_in) * world
        d2h = h_out.numel() * h_out.element_size() * world

        def e2e_step():
            for d, h in zip(d_in, h_in):
                d.copy_(h, non_blocking=True)
            ep.forward_sharded(d_in[0], d_in[1], d_in[2], d_in[3], out, dispatch=True)
            h_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
    else:
        d_in = [inp.routing_logits, inp.routing_bias, inp.hidden_states, inp.hidden_states_scale]

        def e2e_step():
            for d, h in zip(d_in, h_in):
                d.copy_(h, non_blocking=True)
            step()
            h_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
    Ke = min(K, 50)
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

    # ---- the decode batch and two more sizes on the same weights (1 GPU, config 3 only): the metric is quoted vs T
    decode = None
    if world == 1 and args.config == 3 and not args.no_decode and T != 64 and args.experts == 32:
        decode = {}
        for Td in (16, 64, 1024):
            tk = pkg.make_inputs(num_tokens=Td, seed=0, e_local=1, device="cpu")
            small = pkg.MoeInputs(tk.routing_logits.to(dev), tk.routing_bias.to(dev), tk.hidden_states.to(dev),
                                  tk.hidden_states_scale.to(dev), inp.gemm1_weights, inp.gemm1_weights_scale,
                                  inp.gemm2_weights, inp.gemm2_weights_scale, 0, inp.routed_scaling_factor)
            o = torch.empty(Td, H, dtype=torch.bfloat16, device=dev)

            def dstep():
                pkg.run_moe(*small.args(), o)
            for _ in range(5):
                dstep()
            torch.cuda.synchronize()
            dms = time_layer(torch, dstep, 300, torch.cuda.synchronize, None, dev)
            dstats = ctx.check()
            dstage = stage_pass(ctx, dstep, 50)
            fl, by = pkg.algorithmic_work(dstats["routes"], dstats["active_experts"], Td)
            entry = {"tokens": Td, "ms_per_step": dms, "value": Td / (dms / 1e3), "unit": UNIT,
                     "routes": dstats["routes"], "active_experts": dstats["active_experts"],
                     "layer_gbs": by / (dms * 1e-3) / 1e9, "layer_frac_of_hbm_peak": by / (dms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "layer_tflops": fl / (dms * 1e-3) / 1e12,
                     "roofline": gemm1_roofline(Td, dstats["routes"], dstats["active_experts"], dstage, peaks, 1),
                     "stage_ms": dstage}
            if Td == 64:
                hd = [t.cpu().pin_memory() for t in (small.routing_logits, small.routing_bias, small.hidden_states,
                                                     small.hidden_states_scale)]
                ho = torch.empty(Td, H, dtype=torch.bfloat16).pin_memory()

                def de2e():
                    pkg.run_moe_host(*hd, inp.gemm1_weights, inp.gemm1_weights_scale, inp.gemm2_weights,
                                     inp.gemm2_weights_scale, 0, inp.routed_scaling_factor, ho)
                for _ in range(5):
                    de2e()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(300):
                    de2e()
                torch.cuda.synchronize()
                dems = (time.perf_counter() - t0) * 1e3 / 300
                entry["e2e"] = {"value": Td / (dems / 1e3), "unit": UNIT, "ms_per_step": dems,
                                "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in hd),
                                "d2h_bytes_per_step": ho.numel() * ho.element_size()}
            decode[f"T{Td}"] = entry
            ctx.check()

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if args.config == 3 else "weak",
            "vs_baseline": None, "dtype": "f8e4m3", "data": "synthetic",
            "config": {"workload": workload_name(args.config, T), "tokens": T, "local_experts_per_rank": e_per_rank,
                       "parallelism": ("1 GPU" if world == 1 else
                                       f"expert parallel over {world} ranks, tokens replicated, every rank ends with its T/{world} rows: "
                                       + ("reduce-scatter fused into GEMM2: its epilogue stores every expert row into the token owner's memory over NVLink, the owner sums in route order" if peer_ok
                                          else "f32 partials reduce-scattered by NCCL")),
                       "routes": rows_all, "routes_rank0": rows, "active_experts_rank0": active,
                       "l2": f"inputs larger than L2: {active * 44050944 / 1e6:.0f} MB of active-expert weights per step on rank 0",
                       "layer_flops": flops_all, "layer_tflops": flops_all / (ms * 1e-3) / 1e12,
                       "layer_frac_of_nominal_fp8": flops_all / (ms * 1e-3) / 1e12 / (NOMINAL_FP8_TFLOPS * world),
                       "layer_algorithmic_bytes_rank0": layer_bytes,
                       "workspace_bytes": ctx.workspace_bytes() if hasattr(ctx, "workspace_bytes") else None},
            "clocks": clocks,
            "e2e": {"value": T / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": Ke,
                    "path": ("syfi_moe_forward_host: pinned host buffers, slices of 1024 tokens pipelined over three streams"
                             if world == 1 else
                             ("every rank's own T/N tokens from pinned host memory, token dispatch between the ranks, own "
                              "output rows back; bytes are totals over the ranks" if peer_ok else
                              "all tokens to every rank, NCCL reduce-scatter, own rows back"))},
            "gpu_launches": launches, "roofline": roofline}
    if parity is not None:
        line["parity"] = parity
    if decode is not None:
        line["decode"] = decode
    if sharded is not None:
        line["sharded"] = sharded
    if return_leg is not None:
        line["return_leg"] = return_leg
    if args.experts != 32:
        line["config"]["workload"] += f" (first {args.experts} experts only: a profiling case, not the headline)"

    # ---- the reference's own CUDA kernel on this GPU (compiled unmodified into baseline/_ref), as a child process
    # with a time limit: its device-side waits are unbounded
    if rank == 0 and world == 1 and args.config == 3 and not args.no_gpu_reference:
        line["gpu_reference"] = run_gpu_reference(T)

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        arm = CpuArm(torch, oracle, inp.to("cpu"), budget_s=20.0)
        line["cpu_baseline"] = arm.describe(arm.step())
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
