"""Expert parallelism over ``torch.distributed`` (one process per GPU, NCCL over NVLink).

The reference has no multi-GPU code; its only hook is ``local_expert_offset``
(moe/solution/cuda/moe.cu:182-185, 250-256): a call computes the contribution of
experts [offset, offset + E_local) and nothing else.  The layer therefore shards by
expert with one exchange step, the sum of the ranks' partial outputs:

* ``forward_replicated`` — every rank holds the same T tokens (the large-prefill
  configuration): each rank computes an f32 partial [T, 7168] for its experts, the
  partials are all-reduced (or reduce-scattered by rows) and rounded to bf16 once.
* ``forward_sharded`` — every rank brings its own T tokens (the serving layout:
  data-parallel attention, expert-parallel MoE).  Peer-memory path: token dispatch (each rank
  routes its own tokens, every rank pulls only the rows routed to its experts); GEMM2 stores
  every expert row straight into the memory of the token's owner, which sums them in route order.  NCCL path: token-side tensors are all-gathered,
  each rank runs its experts over the W*T gathered tokens, and a reduce-scatter returns
  to each rank the summed rows of its own tokens.

``layer_fn`` computes one rank's f32 partial and defaults to the CUDA operator; tests of
the plumbing on CPU ranks (gloo) pass a stand-in.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

class _coalesced:
    """Batches the collectives issued inside the block into one NCCL group; a plain pass-through
    on backends without coalescing (gloo)."""

    def __init__(self, group, device):
        self.cm = None
        if dist.get_backend(group) == "nccl":
            try:
                from torch.distributed.distributed_c10d import _coalescing_manager
                self.cm = _coalescing_manager(group=group, device=device, async_ops=False)
            except Exception:
                self.cm = None

    def __enter__(self):
        if self.cm is not None:
            self.cm.__enter__()
        return self

    def __exit__(self, *exc):
        if self.cm is not None:
            return self.cm.__exit__(*exc)
        return False


def _reduce_scatter_rows(out, inp, group):
    """Sum ``inp`` [W*R, H] over ranks and leave this rank's R rows in ``out``.  NCCL does it in one
    collective; backends without reduce-scatter (gloo, used by the CPU tests) all-reduce and slice."""
    if dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(out, inp, group=group)
        return
    dist.all_reduce(inp, group=group)
    r = dist.get_rank(group)
    out.copy_(inp[r * out.shape[0]:(r + 1) * out.shape[0]])


def expert_slice(rank: int, world: int, num_experts: int = 32, base_offset: int = 0):
    """Contiguous slice of ``num_experts`` owned by ``rank``: (global offset, count).
    ``num_experts`` must divide evenly (32 experts over 2/4/8 ranks -> 16/8/4 each)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if num_experts % world != 0:
        raise ValueError(f"{num_experts} experts do not split evenly over {world} ranks")
    per = num_experts // world
    return base_offset + rank * per, per


def _cuda_layer(logits, bias, hs, hs_scale, w13, w13_s, w2, w2_s, offset, scaling, out_f32):
    from .moe import run_moe
    return run_moe(logits, bias, hs, hs_scale, w13, w13_s, w2, w2_s, offset, scaling, out_f32)


class ExpertParallelMoe:
    """One rank's experts plus the collectives that combine the ranks."""

    def __init__(self, gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale,
                 local_expert_offset: int, routed_scaling_factor: float, group=None, layer_fn=None):
        self.w13, self.w13_s = gemm1_weights, gemm1_weights_scale
        self.w2, self.w2_s = gemm2_weights, gemm2_weights_scale
        self.offset = int(local_expert_offset)
        self.scaling = float(routed_scaling_factor)
        self.group = group
        self.layer_fn = layer_fn or _cuda_layer
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._buf = {}

    def _buffer(self, name, shape, dtype, device):
        key = (name, tuple(shape), dtype, str(device))
        b = self._buf.get(key)
        if b is None:
            b = torch.empty(shape, dtype=dtype, device=device)
            self._buf[key] = b
        return b

    def partial(self, logits, bias, hs, hs_scale, out_f32=None):
        """This rank's un-rounded contribution, f32 [T, 7168]."""
        T, H = hs.shape
        if out_f32 is None:
            out_f32 = self._buffer("partial", (T, H), torch.float32, logits.device)
        self.layer_fn(logits, bias, hs, hs_scale, self.w13, self.w13_s, self.w2, self.w2_s, self.offset,
                      self.scaling, out_f32)
        return out_f32

    def forward_replicated(self, logits, bias, hs, hs_scale, out_bf16=None, scatter_rows: bool = False):
        """Tokens replicated on every rank.  Returns bf16 [T, 7168] on every rank, or with
        ``scatter_rows`` this rank's T/W rows of it (T must divide by the world size).  With
        ``scatter_rows`` and the peer-memory path enabled for T/W tokens per rank
        (:meth:`enable_peer_exchange`), the reduce-scatter is fused into GEMM2 (rows stored into the owners' memory)
        (``syfi_moe_ep_forward_replicated``); otherwise NCCL sums the f32 partials."""
        T = logits.shape[0]
        peer = getattr(self, "_peer", None)
        if (scatter_rows and self.world > 1 and peer is not None and T % self.world == 0
                and peer[2].tokens_per_rank == T // self.world):
            from . import moe as _moe
            if out_bf16 is None:
                out_bf16 = torch.empty(T // self.world, hs.shape[1], dtype=torch.bfloat16, device=logits.device)
            self._peer_step += 1
            return _moe.run_moe_ep_replicated(peer[2], self._peer_step, logits, bias, hs, hs_scale, self.w13,
                                              self.w13_s, self.w2, self.w2_s, self.offset, self.scaling, out_bf16)
        part = self.partial(logits, bias, hs, hs_scale)
        if self.world == 1:
            res = part
        elif scatter_rows:
            if T % self.world != 0:
                raise ValueError(f"{T} tokens do not split evenly over {self.world} ranks")
            res = self._buffer("rows", (T // self.world, part.shape[1]), torch.float32, part.device)
            _reduce_scatter_rows(res, part, self.group)
        else:
            dist.all_reduce(part, group=self.group)
            res = part
        if out_bf16 is None:
            return res.to(torch.bfloat16)
        out_bf16.copy_(res)
        return out_bf16

    def enable_peer_exchange(self, tokens_per_rank: int, device, wait_limit_cycles: int = 0) -> bool:
        """Set up the peer-memory path for ``forward_sharded``: a symmetric region on every rank, mapped
        into every other rank (torch's symmetric memory does the allocation and the exchange of
        mappings; the data path is this library's own kernels).  Returns False when symmetric memory is
        not available (then ``forward_sharded`` keeps using NCCL)."""
        from . import moe as _moe
        if self.world < 2 or self.world > _moe.EP_MAX_RANKS:
            return False
        try:
            import torch.distributed._symmetric_memory as symm
            nbytes = _moe.ep_region_bytes(self.world, tokens_per_rank)
            region = symm.empty(nbytes, dtype=torch.uint8, device=device)
            handle = symm.rendezvous(region, self.group if self.group is not None else dist.group.WORLD)
            region.zero_()
            torch.cuda.synchronize(device)
            handle.barrier()
            torch.cuda.synchronize(device)
            desc = _moe.EpDesc()
            desc.world_size, desc.rank, desc.tokens_per_rank = self.world, self.rank, int(tokens_per_rank)
            desc.wait_limit_cycles = int(wait_limit_cycles)      # 0: the library's serving default
            for r, ptr in enumerate(handle.buffer_ptrs):
                desc.region[r] = ptr
            # allocate the workspace and the gathered-token buffers now, then meet the other ranks: no rank
            # may stall in an allocation inside its first step while its peers are already waiting for it
            _moe.ep_prepare(desc, device.index if isinstance(device, torch.device) else torch.device(device).index)
            torch.cuda.synchronize(device)
            handle.barrier()
        except Exception as exc:  # no symmetric memory on this system / backend
            self._peer_error = repr(exc)
            return False
        self._peer = (region, handle, desc)
        self._peer_step = 0
        return True

    def forward_sharded(self, logits, bias, hs, hs_scale, out_bf16=None, dispatch: bool = True):
        """Each rank passes its OWN T tokens (same T on every rank); returns their bf16 outputs
        summed over all ranks' experts.  On the peer-memory path ``dispatch`` (default) sends only the
        rows a rank's experts were selected for (token dispatch); ``dispatch=False`` all-gathers every
        token to every rank.  Both give the same bits."""
        T = logits.shape[0]
        W = self.world
        if W == 1:
            return self.forward_replicated(logits, bias, hs, hs_scale, out_bf16)
        dev = logits.device
        peer = getattr(self, "_peer", None)
        if peer is not None and peer[2].tokens_per_rank == T:
            from . import moe as _moe
            if out_bf16 is None:
                out_bf16 = torch.empty(T, hs.shape[1], dtype=torch.bfloat16, device=dev)
            self._peer_step += 1
            return _moe.run_moe_ep(peer[2], self._peer_step, logits, bias, hs, hs_scale, self.w13, self.w13_s,
                                   self.w2, self.w2_s, self.offset, self.scaling, out_bf16, dispatch=dispatch)
        g_logits = self._buffer("g_logits", (W * T, logits.shape[1]), logits.dtype, dev)
        g_hs = self._buffer("g_hs", (W * T, hs.shape[1]), torch.uint8, dev)
        g_sc = self._buffer("g_sc", (W * hs_scale.shape[0], T), hs_scale.dtype, dev)
        # one NCCL group launch for the three gathers (each costs a launch latency on its own)
        with _coalesced(self.group, dev):
            dist.all_gather_into_tensor(g_logits, logits.contiguous(), group=self.group)
            dist.all_gather_into_tensor(g_hs, hs.view(torch.uint8).contiguous(), group=self.group)
            dist.all_gather_into_tensor(g_sc, hs_scale.contiguous(), group=self.group)
        # scales are stored [K/128, tokens]: put the gathered ranks side by side along the token axis
        sc = g_sc.view(W, hs_scale.shape[0], T).permute(1, 0, 2).reshape(hs_scale.shape[0], W * T).contiguous()
        part = self.partial(g_logits, bias, g_hs.view(hs.dtype), sc)
        mine = self._buffer("mine", (T, part.shape[1]), torch.float32, dev)
        _reduce_scatter_rows(mine, part, self.group)
        if out_bf16 is None:
            return mine.to(torch.bfloat16)
        out_bf16.copy_(mine)
        return out_bf16
