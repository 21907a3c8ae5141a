"""Expert-parallel plumbing on CPU ranks (gloo, world size 2): partitioning, gather of the token-side
tensors, and the sum of the ranks' partial outputs.  The per-rank layer is a stand-in (the oracle's
f32 partial) because the CUDA operator cannot run here; the GPU test of the real path is
tests/test_expert_parallel_gpu.py."""
import importlib
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = "mlsys-contest-syfi-agent-assisted_b200"
H, I = 256, 128


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_partial(oracle):
    def fn(logits, bias, hs, hs_scale, w13, w13_s, w2, w2_s, offset, scaling, out_f32):
        acc, _, _ = oracle.moe_forward(logits, bias, hs, hs_scale, w13, w13_s, w2, w2_s, offset, scaling,
                                       return_f32=True)
        out_f32.copy_(acc)
        return out_f32
    return fn


def _worker(rank, world, port, mode, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module(PKG)
        oracle = importlib.import_module("oracle.moe_oracle")
        torch.set_num_threads(2)
        e_total = 8
        off, per = pkg.expert_slice(rank, world, e_total)
        full = pkg.make_inputs(num_tokens=12, seed=0, e_local=e_total, hidden=H, inter=I)
        ep = pkg.ExpertParallelMoe(full.gemm1_weights[off:off + per], full.gemm1_weights_scale[off:off + per],
                                   full.gemm2_weights[off:off + per], full.gemm2_weights_scale[off:off + per],
                                   off, 2.5, layer_fn=_oracle_partial(oracle))
        if mode == "replicated":
            out = ep.forward_replicated(full.routing_logits, full.routing_bias, full.hidden_states,
                                        full.hidden_states_scale)
            ref, _, _ = oracle.moe_forward(*full.args())
            q.put((rank, bool(torch.equal(out.view(torch.int16), ref.view(torch.int16))) or
                   bool(oracle.check_output(out, ref)[0])))
        elif mode == "scatter":
            out = ep.forward_replicated(full.routing_logits, full.routing_bias, full.hidden_states,
                                        full.hidden_states_scale, scatter_rows=True)
            ref, _, _ = oracle.moe_forward(*full.args())
            rows = 12 // world
            q.put((rank, out.shape == (rows, H) and bool(oracle.check_output(out, ref[rank * rows:(rank + 1) * rows])[0])))
        else:  # sharded: every rank brings its own tokens
            mine = pkg.make_inputs(num_tokens=6, seed=10 + rank, e_local=1, hidden=H, inter=I)
            out = ep.forward_sharded(mine.routing_logits, full.routing_bias, mine.hidden_states,
                                     mine.hidden_states_scale)
            ref, _, _ = oracle.moe_forward(mine.routing_logits, full.routing_bias, mine.hidden_states,
                                           mine.hidden_states_scale, full.gemm1_weights, full.gemm1_weights_scale,
                                           full.gemm2_weights, full.gemm2_weights_scale, 0, 2.5)
            q.put((rank, out.shape == (6, H) and bool(oracle.check_output(out, ref)[0])))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["replicated", "scatter", "sharded"])
def test_two_ranks(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=90) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def test_expert_slice():
    pkg = importlib.import_module(PKG)
    assert pkg.expert_slice(0, 1) == (0, 32)
    assert [pkg.expert_slice(r, 4) for r in range(4)] == [(0, 8), (8, 8), (16, 8), (24, 8)]
    assert pkg.expert_slice(3, 8, 32, base_offset=64) == (76, 4)
    with pytest.raises(ValueError):
        pkg.expert_slice(0, 3)
    with pytest.raises(ValueError):
        pkg.expert_slice(2, 2)
