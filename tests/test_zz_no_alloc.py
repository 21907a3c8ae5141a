"""The allocation-free router entry point, called through the C ABI.

`syfi_moe_route_noalloc` exists for hosts that may not allocate device memory where they run the
router (a process whose pool already owns the GPU, a framework callback that forbids allocation,
code running next to a CUDA-graph capture).  It keeps its scratch in a fixed array inside the
library, so it needs no context.  This file is collected last on purpose: it must pass both on its
own in a fresh process and after every other test has used the library.
"""
import ctypes
import re
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _max_tokens():
    text = open(os.path.join(ROOT, "include", "syfi_moe.h")).read()
    return int(re.search(r"#define\s+SYFI_MOE_NOALLOC_MAX_TOKENS\s+(\d+)", text).group(1))


def _route_noalloc(lib, logits, bias, e_local, offset, scaling):
    T = logits.shape[0]
    idx = torch.full((T, 8), -7, dtype=torch.int32, device=logits.device)
    w = torch.full((T, 8), float("nan"), dtype=torch.float32, device=logits.device)
    rc = lib.syfi_moe_route_noalloc(logits.data_ptr(), bias.data_ptr(), T, e_local, offset, scaling,
                                    idx.data_ptr(), w.data_ptr(),
                                    torch.cuda.current_stream(logits.device).cuda_stream)
    return rc, idx, w


def test_matches_context_router_on_two_calls_in_a_row(pkg, oracle):
    torch.cuda.set_device(0)
    lib = pkg.load_library()
    # two different batches back to back: the second must not see anything the first left behind
    for T, seed, e_local, offset, scaling in [(300, 21, 32, 0, 2.5), (64, 22, 8, 40, 1.0)]:
        inp = pkg.make_inputs(num_tokens=T, seed=seed, e_local=1, device="cpu")
        logits, bias = inp.routing_logits.to(DEV), inp.routing_bias.to(DEV)
        rc, idx, w = _route_noalloc(lib, logits, bias, e_local, offset, scaling)
        assert rc == 0, lib.syfi_moe_last_error()
        ref_idx, ref_w = pkg.route(logits, bias, offset, scaling, num_local_experts=e_local)
        torch.cuda.synchronize()
        # same kernel, same inputs: identical indices and identical weight bits
        assert torch.equal(idx, ref_idx)
        assert torch.equal(w.view(torch.int32), ref_w.view(torch.int32))
        # and both agree with the oracle (bit-exact expert sets)
        oidx, ow = oracle.route(inp.routing_logits, inp.routing_bias, scaling)
        ok, stats = oracle.check_routing(idx, w, oidx, ow)
        assert ok, stats


def test_rejects_batches_beyond_its_fixed_scratch(pkg):
    torch.cuda.set_device(0)
    lib = pkg.load_library()
    limit = _max_tokens()
    T = limit + 1
    logits = torch.zeros(T, 256, dtype=torch.float32, device=DEV)
    bias = torch.zeros(256, dtype=torch.bfloat16, device=DEV)
    rc, _, _ = _route_noalloc(lib, logits, bias, 32, 0, 2.5)
    assert rc == 1
    msg = lib.syfi_moe_last_error().decode()
    assert "at most" in msg and str(limit) in msg
    # the limit itself is accepted
    rc, idx, w = _route_noalloc(lib, logits[:limit], bias, 32, 0, 2.5)
    assert rc == 0, lib.syfi_moe_last_error()
    torch.cuda.synchronize()
    assert int(idx.min()) >= 0 and bool(torch.isfinite(w).all())


def test_warmed_calls_leave_device_memory_untouched(pkg):
    """The point of the entry point: once the first call on the device has looked up the scratch array, a call
    allocates nothing — the free device memory reported by the driver is the same before and after two calls
    (torch's caching allocator is kept out of the picture: the output tensors exist before the measurement)."""
    torch.cuda.set_device(0)
    lib = pkg.load_library()
    T = 257
    inp = pkg.make_inputs(num_tokens=T, seed=23, e_local=1, device="cpu")
    logits, bias = inp.routing_logits.to(DEV), inp.routing_bias.to(DEV)
    idx = torch.empty(T, 8, dtype=torch.int32, device=DEV)
    w = torch.empty(T, 8, dtype=torch.float32, device=DEV)
    stream = torch.cuda.current_stream(logits.device).cuda_stream

    def call():
        return lib.syfi_moe_route_noalloc(logits.data_ptr(), bias.data_ptr(), T, 32, 0, 2.5, idx.data_ptr(),
                                          w.data_ptr(), stream)
    assert call() == 0, lib.syfi_moe_last_error()        # first call: set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    assert call() == 0 and call() == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before
    ref_idx, ref_w = pkg.route(logits, bias, 0, 2.5)
    assert torch.equal(idx, ref_idx) and torch.equal(w.view(torch.int32), ref_w.view(torch.int32))
