"""Seeded synthetic workloads for the fused FP8 block-scale DeepSeek-V3 MoE layer.

The contest dataset the reference was graded on is not available, so every
input here is drawn from a seeded generator with the shapes, dtypes and value
distributions of the definition
``moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048``:

* ``routing_logits``  f32  [T, 256]        ~ N(0, 1)
* ``routing_bias``    bf16 [256]           ~ N(0, 0.1)
* ``hidden_states``   e4m3 [T, 7168]       bf16 N(0, 1) quantised per 1x128 block, scale = amax / 448
* ``hidden_states_scale`` f32 [56, T]      (stored transposed, as the reference expects,
                                            moe/solution/cuda/moe.cu:2991)
* ``gemm1_weights``   e4m3 [E, 4096, 7168] N(0, 0.02) quantised per 128x128 block
* ``gemm1_weights_scale`` f32 [E, 32, 56]
* ``gemm2_weights``   e4m3 [E, 7168, 2048]
* ``gemm2_weights_scale`` f32 [E, 56, 16]

Draw order is fixed: logits, bias, hidden states, then per expert W13 and W2.
The small tensors always come from a CPU generator so routing is the same on
every machine; the weights come from a generator on ``device`` (a CUDA
generator is far faster but draws a different, equally valid, stream).
"""
from __future__ import annotations

import dataclasses

import torch

HIDDEN = 7168
INTER = 2048
BLOCK = 128
E_GLOBAL = 256
N_GROUP = 8
TOPK_GROUP = 4
TOP_K = 8
FP8_MAX = 448.0


@dataclasses.dataclass
class MoeInputs:
    routing_logits: torch.Tensor
    routing_bias: torch.Tensor
    hidden_states: torch.Tensor
    hidden_states_scale: torch.Tensor
    gemm1_weights: torch.Tensor
    gemm1_weights_scale: torch.Tensor
    gemm2_weights: torch.Tensor
    gemm2_weights_scale: torch.Tensor
    local_expert_offset: int
    routed_scaling_factor: float

    def to(self, device) -> "MoeInputs":
        kw = {}
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            kw[f.name] = v.to(device) if isinstance(v, torch.Tensor) else v
        return MoeInputs(**kw)

    def args(self):
        """Positional arguments in the reference entry point's order
        (moe/solution/cuda/moe.cu:2987-2998), without the output tensor."""
        return (self.routing_logits, self.routing_bias, self.hidden_states,
                self.hidden_states_scale, self.gemm1_weights, self.gemm1_weights_scale,
                self.gemm2_weights, self.gemm2_weights_scale,
                self.local_expert_offset, self.routed_scaling_factor)

    @property
    def num_tokens(self) -> int:
        return int(self.routing_logits.shape[0])


def quantize_act_1x128(x: torch.Tensor):
    """[T, K] -> (e4m3 [T, K], scale f32 [K/128, T]); scale = amax / 448 per 1x128 block."""
    T, K = x.shape
    xb = x.float().view(T, K // BLOCK, BLOCK)
    amax = xb.abs().amax(-1).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (xb / scale.unsqueeze(-1)).view(T, K).to(torch.float8_e4m3fn)
    return q, scale.t().contiguous()


def quantize_weight_128x128(w: torch.Tensor):
    """[N, K] -> (e4m3 [N, K], scale f32 [N/128, K/128]); scale = amax / 448 per 128x128 block."""
    N, K = w.shape
    wb = w.view(N // BLOCK, BLOCK, K // BLOCK, BLOCK)
    amax = wb.abs().amax((1, 3)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (wb / scale[:, None, :, None]).view(N, K).to(torch.float8_e4m3fn)
    return q, scale


def make_inputs(num_tokens: int, seed: int = 0, e_local: int = 32, local_expert_offset: int = 0,
                device="cpu", routed_scaling_factor: float = 2.5, hot_experts: int = 0,
                hot_seed: int = 1, hot_skew: float = 1.5, hidden: int = HIDDEN,
                inter: int = INTER, weight_seed: int | None = None) -> MoeInputs:
    """Build one workload.

    ``hot_experts`` > 0 adds ``hot_skew`` to the logits of that many experts chosen
    with ``hot_seed`` (the load-imbalance configuration).  ``weight_seed`` lets a
    rank of an expert-parallel job draw its own weights while sharing the
    token-side tensors with the other ranks.
    """
    device = torch.device(device)
    T = int(num_tokens)
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    logits = torch.randn(T, E_GLOBAL, generator=g, dtype=torch.float32)
    if hot_experts > 0:
        gh = torch.Generator(device="cpu")
        gh.manual_seed(hot_seed)
        hot = torch.randperm(E_GLOBAL, generator=gh)[:hot_experts]
        logits[:, hot] += hot_skew
    bias = (torch.randn(E_GLOBAL, generator=g, dtype=torch.float32) * 0.1).to(torch.bfloat16)
    hs = torch.randn(T, hidden, generator=g, dtype=torch.float32).to(torch.bfloat16)
    hs_q, hs_scale = quantize_act_1x128(hs)

    gw = torch.Generator(device=device)
    gw.manual_seed(seed if weight_seed is None else weight_seed)
    w13 = torch.empty(e_local, 2 * inter, hidden, dtype=torch.float8_e4m3fn, device=device)
    w13_s = torch.empty(e_local, 2 * inter // BLOCK, hidden // BLOCK, dtype=torch.float32, device=device)
    w2 = torch.empty(e_local, hidden, inter, dtype=torch.float8_e4m3fn, device=device)
    w2_s = torch.empty(e_local, hidden // BLOCK, inter // BLOCK, dtype=torch.float32, device=device)
    for e in range(e_local):
        w = torch.randn(2 * inter, hidden, generator=gw, dtype=torch.float32, device=device) * 0.02
        w13[e], w13_s[e] = quantize_weight_128x128(w)
        w = torch.randn(hidden, inter, generator=gw, dtype=torch.float32, device=device) * 0.02
        w2[e], w2_s[e] = quantize_weight_128x128(w)
    del w
    return MoeInputs(logits.to(device), bias.to(device), hs_q.to(device), hs_scale.to(device),
                     w13, w13_s, w2, w2_s, int(local_expert_offset), float(routed_scaling_factor))


def algorithmic_work(num_routes: int, active_experts: int, num_tokens: int):
    """Flops and bytes one layer call must do (intermediates excluded).

    Per (token, local expert) route: GEMM1 2*7168*4096 + GEMM2 2*2048*7168 flop.
    Per active expert: W13 + W2 fp8 bytes plus their block scales.
    Per token: logits, fp8 hidden row, its scales, and the bf16 output row.
    """
    flops = num_routes * (2 * HIDDEN * 2 * INTER + 2 * INTER * HIDDEN)
    w_bytes = active_experts * (2 * INTER * HIDDEN + HIDDEN * INTER
                                + 4 * (2 * INTER // BLOCK) * (HIDDEN // BLOCK)
                                + 4 * (HIDDEN // BLOCK) * (INTER // BLOCK))
    t_bytes = num_tokens * (4 * E_GLOBAL + HIDDEN + 4 * (HIDDEN // BLOCK) + 2 * HIDDEN) + 2 * E_GLOBAL
    return flops, w_bytes + t_bytes
