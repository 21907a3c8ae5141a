"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol the
header declares, the Python mirror validates its arguments, and the workload generator and
work model are what the documentation states."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "syfi_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(syfi_moe_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(pkg):
    names = _declared_symbols()
    assert "syfi_moe_forward" in names and len(names) >= 10
    lib = ctypes.CDLL(pkg.library_path())
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/syfi_moe.h but not exported"
    assert sorted(pkg.ABI.keys()) == names


def test_library_is_built_for_sm100a_only(pkg):
    from importlib import import_module
    build = import_module(pkg.__name__ + ".build")
    flags = " ".join(build.NVCC_FLAGS)
    assert "arch=compute_100a,code=sm_100a" in flags
    assert flags.count("-gencode") == 1


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_no_cpu_fallback(pkg):
    with pytest.raises(pkg.MoeError, match="no CUDA device"):
        pkg.MoeContext(0)
    inp = pkg.make_inputs(num_tokens=2, e_local=1, hidden=256, inter=128, device="cpu")
    out = torch.empty(2, 7168, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        pkg.run_moe(*inp.args(), out)


def test_prepacking_refuses_host_tensors_and_foreign_objects(pkg):
    """The packed-weights path has no CPU side either, and run_moe_prepacked only takes what
    prepack_weights returned."""
    f8 = torch.float8_e4m3fn
    w13 = torch.zeros(1, 4096, 7168, dtype=torch.uint8).view(f8)
    w2 = torch.zeros(1, 7168, 2048, dtype=torch.uint8).view(f8)
    with pytest.raises(ValueError, match="CUDA tensor"):
        pkg.prepack_weights(w13, w2)
    with pytest.raises(ValueError, match="prepack_weights"):
        pkg.run_moe_prepacked(None, None, None, None, (w13, w2), None, None, 0, 2.5, None)
    lib = ctypes.CDLL(pkg.library_path())
    lib.syfi_moe_prepack_weights.restype = ctypes.c_int
    assert lib.syfi_moe_prepack_weights(None, None, None, 1, None, None, None) == 1   # SYFI_MOE_ERR_INVALID
    lib.syfi_moe_last_error.restype = ctypes.c_char_p
    assert b"context is null" in lib.syfi_moe_last_error()


def test_last_error_is_empty_string_initially(pkg):
    lib = pkg.load_library()
    assert isinstance(lib.syfi_moe_last_error(), bytes)


def test_null_context_is_rejected(pkg):
    lib = pkg.load_library()
    rc = lib.syfi_moe_forward(None, *([None] * 8), 4, 32, 0, 2.5, None, None)
    assert rc == 1
    assert b"context" in lib.syfi_moe_last_error()
    assert lib.syfi_moe_destroy(None) == 0
    assert lib.syfi_moe_last_launch_count(None) == 0
    assert lib.syfi_moe_workspace_bytes(None) == 0


def test_workload_shapes_and_quantisation(pkg):
    inp = pkg.make_inputs(num_tokens=5, seed=1, e_local=2, hidden=256, inter=128, device="cpu")
    assert inp.routing_logits.shape == (5, 256) and inp.routing_logits.dtype == torch.float32
    assert inp.routing_bias.shape == (256,) and inp.routing_bias.dtype == torch.bfloat16
    assert inp.hidden_states.shape == (5, 256) and inp.hidden_states.dtype == torch.float8_e4m3fn
    assert inp.hidden_states_scale.shape == (2, 5)
    assert inp.gemm1_weights.shape == (2, 256, 256) and inp.gemm1_weights_scale.shape == (2, 2, 2)
    assert inp.gemm2_weights.shape == (2, 256, 128) and inp.gemm2_weights_scale.shape == (2, 2, 1)
    # block amax maps to +-448 exactly
    assert float(inp.hidden_states.float().abs().view(5, 2, 128).amax(-1).min()) == 448.0
    again = pkg.make_inputs(num_tokens=5, seed=1, e_local=2, hidden=256, inter=128, device="cpu")
    assert torch.equal(again.gemm1_weights.view(torch.uint8), inp.gemm1_weights.view(torch.uint8))
    assert torch.equal(again.routing_logits, inp.routing_logits)


def test_token_side_tensors_do_not_depend_on_expert_count(pkg):
    a = pkg.make_inputs(num_tokens=9, seed=2, e_local=1, hidden=256, inter=128)
    b = pkg.make_inputs(num_tokens=9, seed=2, e_local=3, hidden=256, inter=128)
    assert torch.equal(a.routing_logits, b.routing_logits)
    assert torch.equal(a.hidden_states.view(torch.uint8), b.hidden_states.view(torch.uint8))


def test_work_model(pkg):
    flops, nbytes = pkg.algorithmic_work(1, 1, 0)
    assert flops == 88_080_384
    assert nbytes == 44_050_944 + 512
    flops, nbytes = pkg.algorithmic_work(89, 16, 64)
    assert nbytes == 16 * 44_050_944 + 64 * 22_752 + 512


def test_tvm_ffi_binding_exports_the_reference_symbol(pkg):
    """The optional tvm-ffi shared object exports `__tvm_ffi_run_moe`, the symbol the reference's
    `TVM_FFI_DLL_EXPORT_TYPED_FUNC(run_moe, ...)` produces (moe/solution/cuda/moe.cu:3260)."""
    from importlib import import_module
    build = import_module(pkg.__name__ + ".build")
    pytest.importorskip("tvm_ffi")
    pkg.load_library()
    path = build.build_tvm_ffi_binding()
    assert path and os.path.exists(path)
    lib = ctypes.CDLL(path)
    assert hasattr(lib, "__tvm_ffi_run_moe")


def test_layer_is_registered_as_a_torch_operator(pkg):
    """`torch.ops.syfi_moe.run_moe` exists after importing the package: eleven arguments in the order of the
    reference's run_moe, mutating the last one."""
    import torch
    op = torch.ops.syfi_moe.run_moe
    schema = str(op.default._schema)
    assert "Tensor(a10!) output" in schema and schema.rstrip().endswith("-> ()"), schema
    assert schema.count("Tensor") == 9


def test_indexer_header_symbols_are_exported_and_bound(pkg):
    """Every function include/syfi_dsa.h declares is exported by the shared library and bound by the Python mirror."""
    from importlib import import_module
    text = open(os.path.join(ROOT, "include", "syfi_dsa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = sorted(set(re.findall(r"\b(syfi_dsa_[a-z0-9_]+)\s*\(", text)))
    assert names == ["syfi_dsa_check", "syfi_dsa_topk_indexer"]
    lib = ctypes.CDLL(pkg.library_path())
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/syfi_dsa.h but not exported"
    assert sorted(import_module(pkg.__name__ + ".dsa").ABI.keys()) == names
