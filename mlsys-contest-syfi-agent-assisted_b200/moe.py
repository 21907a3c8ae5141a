"""Host-side mirror of the reference's operator interface for the fused MoE layer.

``run_moe`` has the argument order and destination-passing convention of the
reference's exported ``run_moe`` (moe/solution/cuda/moe.cu:2987-2998, :3260;
moe/config.toml:10).  It validates its tensors and hands raw device pointers to
the C ABI declared in ``include/syfi_moe.h``; torch is used only for memory and
the current stream.  There is no CPU path and no fallback: without the compiled
library or without a CUDA device every call raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

from . import build as _build

HIDDEN = 7168
INTER = 2048
E_GLOBAL = 256
TOP_K = 8
MAX_LOCAL_EXPERTS = 32

_lib = None
_lib_lock = threading.Lock()
_contexts: dict[int, "MoeContext"] = {}

_vp, _i64, _i32, _f64 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_double

# name -> (restype, argtypes); must list every symbol include/syfi_moe.h declares
ABI = {
    "syfi_moe_create": (ctypes.c_int, [ctypes.c_int, _i64, ctypes.POINTER(_vp)]),
    "syfi_moe_destroy": (ctypes.c_int, [_vp]),
    "syfi_moe_forward": (ctypes.c_int, [_vp] + [_vp] * 8 + [_i64, _i32, _i64, _f64, _vp, _vp]),
    "syfi_moe_forward_partial_f32": (ctypes.c_int, [_vp] + [_vp] * 8 + [_i64, _i32, _i64, _f64, _vp, _vp]),
    "syfi_moe_prepack_weights": (ctypes.c_int, [_vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "syfi_moe_forward_prepacked": (ctypes.c_int, [_vp] + [_vp] * 8 + [_i64, _i32, _i64, _f64, _vp, _vp]),
    "syfi_moe_forward_host": (ctypes.c_int, [_vp] + [_vp] * 8 + [_i64, _i32, _i64, _f64, _vp, _vp]),
    "syfi_moe_route": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i32, _i64, _f64, _vp, _vp, _vp]),
    "syfi_moe_ep_region_bytes": (_i64, [_i32, _i64]),
    "syfi_moe_ep_forward": (ctypes.c_int, [_vp, _vp, _i64] + [_vp] * 8 + [_i32, _i64, _f64, _vp, _vp]),
    "syfi_moe_ep_forward_dispatch": (ctypes.c_int, [_vp, _vp, _i64] + [_vp] * 8 + [_i32, _i64, _f64, _vp, _vp]),
    "syfi_moe_ep_forward_replicated": (ctypes.c_int, [_vp, _vp, _i64] + [_vp] * 8 + [_i32, _i64, _f64, _vp, _vp]),
    "syfi_moe_ep_prepare": (ctypes.c_int, [_vp, _vp]),
    "syfi_moe_debug_fault": (ctypes.c_int, [_vp, _i32, _i64]),
    "syfi_moe_reserve": (ctypes.c_int, [_vp, _i64, _i64]),
    "syfi_moe_route_noalloc": (ctypes.c_int, [_vp, _vp, _i64, _i32, _i64, _f64, _vp, _vp, _vp]),
    "syfi_moe_last_routing": (ctypes.c_int, [_vp, _i64, _vp, _vp, _vp]),
    "syfi_moe_check": (ctypes.c_int, [_vp, ctypes.POINTER(_i32), _vp]),
    "syfi_moe_debug_read": (ctypes.c_int, [_vp, ctypes.c_char_p, _vp, _i64, ctypes.POINTER(_i64),
                                           ctypes.POINTER(_i32)]),
    "syfi_moe_set_stage_timing": (ctypes.c_int, [_vp, _i32]),
    "syfi_moe_last_stage_ms": (ctypes.c_int, [_vp, ctypes.POINTER(ctypes.c_float)]),
    "syfi_moe_last_launch_count": (ctypes.c_int, [_vp]),
    "syfi_moe_workspace_bytes": (_i64, [_vp]),
    "syfi_moe_last_error": (ctypes.c_char_p, []),
}


class MoeError(RuntimeError):
    pass


EP_MAX_RANKS = 8


class EpDesc(ctypes.Structure):
    """Mirror of ``syfi_moe_ep_desc`` (include/syfi_moe.h)."""
    _fields_ = [("world_size", _i32), ("rank", _i32), ("tokens_per_rank", _i64), ("region", _vp * EP_MAX_RANKS),
                ("wait_limit_cycles", _i64)]


def library_path() -> str:
    return _build.LIB


def load_library():
    """dlopen the in-tree CUDA library (building it with nvcc first if it is missing or stale)."""
    global _lib
    with _lib_lock:
        if _lib is None:
            # SYFI_MOE_LIBRARY points at an alternative build of the same sources (e.g. a tracing build)
            path = os.environ.get("SYFI_MOE_LIBRARY") or (
                _build.build_library() if _build.needs_build() else _build.LIB)
            lib = ctypes.CDLL(path)
            for name, (res, args) in ABI.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def _check(rc: int):
    if rc != 0:
        msg = load_library().syfi_moe_last_error().decode()
        if rc == 1:
            raise ValueError(msg)
        raise MoeError(f"syfi_moe error {rc}: {msg}")


class MoeContext:
    """Per-device workspace handle (counterpart of the reference's static g_ws, moe.cu:2832-2926)."""

    def __init__(self, device: int, max_tokens: int = 64):
        self.lib = load_library()
        self.device = int(device)
        h = _vp()
        _check(self.lib.syfi_moe_create(self.device, int(max_tokens), ctypes.byref(h)))
        self.handle = h

    def close(self):
        if getattr(self, "handle", None):
            self.lib.syfi_moe_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, stream=None):
        """Synchronise and raise if a kernel reported a failure; returns the work counters
        {'token_tiles', 'padded_rows', 'routes', 'active_experts'} of the last forward."""
        stats = (_i32 * 4)()
        _check(self.lib.syfi_moe_check(self.handle, stats, _stream_ptr(stream, self.device)))
        return {"token_tiles": stats[0], "padded_rows": stats[1], "routes": stats[2], "active_experts": stats[3]}

    def last_routing(self, num_tokens: int, stream=None):
        idx = torch.empty(num_tokens, TOP_K, dtype=torch.int32)
        w = torch.empty(num_tokens, TOP_K, dtype=torch.float32)
        _check(self.lib.syfi_moe_last_routing(self.handle, num_tokens, idx.data_ptr(), w.data_ptr(),
                                              _stream_ptr(stream, self.device)))
        return idx, w

    STAGES = ("router", "row_lists", "gather", "gemm1", "gemm2", "combine")

    def set_stage_timing(self, enable: bool):
        _check(self.lib.syfi_moe_set_stage_timing(self.handle, 1 if enable else 0))

    def last_stage_ms(self) -> dict:
        """Durations in ms of the six kernels of the last forward (stage timing must be on)."""
        ms = (ctypes.c_float * 6)()
        _check(self.lib.syfi_moe_last_stage_ms(self.handle, ms))
        return dict(zip(self.STAGES, [float(x) for x in ms]))

    def reserve(self, max_tokens: int, max_rows: int = 0):
        """Size the workspace for ``max_tokens`` tokens routing up to ``max_rows`` rows to this rank's experts
        (0 = the worst case of 8 per token); see ``syfi_moe_reserve``."""
        _check(self.lib.syfi_moe_reserve(self.handle, int(max_tokens), int(max_rows)))

    def debug_fault(self, mask: int, wait_limit_cycles: int):
        """Test hook (``syfi_moe_debug_fault``): the next forward runs with a short wait limit and the given
        roles / kernels left out, so that its bounded waits run out."""
        _check(self.lib.syfi_moe_debug_fault(self.handle, int(mask), int(wait_limit_cycles)))

    def launch_count(self) -> int:
        return int(self.lib.syfi_moe_last_launch_count(self.handle))

    def workspace_bytes(self) -> int:
        return int(self.lib.syfi_moe_workspace_bytes(self.handle))

    def debug_read(self, name: str, dtype: torch.dtype, max_bytes: int | None = None) -> tuple[torch.Tensor, int]:
        """Host copy of a workspace buffer as a flat tensor of ``dtype`` plus the row capacity (test hook)."""
        nbytes, cap = _i64(), _i32()
        _check(self.lib.syfi_moe_debug_read(self.handle, name.encode(), None, 0, ctypes.byref(nbytes),
                                            ctypes.byref(cap)))
        n = nbytes.value if max_bytes is None else min(nbytes.value, int(max_bytes))
        out = torch.empty(n, dtype=torch.uint8)
        _check(self.lib.syfi_moe_debug_read(self.handle, name.encode(), out.data_ptr(), n, ctypes.byref(nbytes),
                                            ctypes.byref(cap)))
        return out.view(dtype), cap.value


def get_context(device: int, min_tokens: int = 64) -> MoeContext:
    ctx = _contexts.get(device)
    if ctx is None:
        ctx = MoeContext(device, max_tokens=max(64, min_tokens))
        _contexts[device] = ctx
    return ctx


def release_contexts():
    for ctx in list(_contexts.values()):
        ctx.close()
    _contexts.clear()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(stream, device: int) -> int:
    if stream is None:
        if _raw_stream is not None:      # the handle of torch's current stream without building a Stream object
            return int(_raw_stream(device))
        stream = torch.cuda.current_stream(device)
    return int(stream.cuda_stream)


def _expect(t, name, dtype, shape, device=None):
    # fast path: one expression when everything is as it should be (this runs ten times per call)
    try:
        if (t.dtype is dtype and t.shape == shape and t.is_contiguous()
                and (device is None or (t.device.type == "cpu" if device == "cpu" else t.device == device))):
            return
    except AttributeError:
        pass
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name} must be a torch.Tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if device is not None:
        if device == "cpu":
            if t.device.type != "cpu":
                raise ValueError(f"{name} must be a host tensor")
        elif t.device != device:
            raise ValueError(f"{name} must be on {device}, got {t.device}")


def _validate(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
              gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset, output,
              out_dtype, token_device):
    if not isinstance(gemm1_weights, torch.Tensor) or gemm1_weights.dim() != 3:
        raise ValueError("gemm1_weights must be a 3-D tensor [E_local, 4096, 7168]")
    if gemm1_weights.device.type != "cuda":
        raise ValueError("weights must be CUDA tensors: this operator has no CPU path")
    wdev = gemm1_weights.device
    tdev = wdev if token_device is None else token_device
    if not isinstance(routing_logits, torch.Tensor) or routing_logits.dim() != 2:
        raise ValueError("routing_logits must be a 2-D tensor [T, 256]")
    T = routing_logits.shape[0]
    E = gemm1_weights.shape[0]
    if E < 1 or E > MAX_LOCAL_EXPERTS:
        raise ValueError(f"number of local experts must be in [1, {MAX_LOCAL_EXPERTS}], got {E}")
    off = int(local_expert_offset)
    if off < 0 or off + E > E_GLOBAL:
        raise ValueError(f"local experts [{off}, {off + E}) outside [0, {E_GLOBAL})")
    f8 = torch.float8_e4m3fn
    _expect(routing_logits, "routing_logits", torch.float32, (T, E_GLOBAL), tdev)
    _expect(routing_bias, "routing_bias", torch.bfloat16, (E_GLOBAL,), tdev)
    _expect(hidden_states, "hidden_states", f8, (T, HIDDEN), tdev)
    _expect(hidden_states_scale, "hidden_states_scale", torch.float32, (HIDDEN // 128, T), tdev)
    _expect(gemm1_weights, "gemm1_weights", f8, (E, 2 * INTER, HIDDEN), wdev)
    _expect(gemm1_weights_scale, "gemm1_weights_scale", torch.float32, (E, 2 * INTER // 128, HIDDEN // 128), wdev)
    _expect(gemm2_weights, "gemm2_weights", f8, (E, HIDDEN, INTER), wdev)
    _expect(gemm2_weights_scale, "gemm2_weights_scale", torch.float32, (E, HIDDEN // 128, INTER // 128), wdev)
    if output is not None:
        _expect(output, "output", out_dtype, (T, HIDDEN), tdev)
    return T, E, off, wdev


def run_moe(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
            gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
            routed_scaling_factor, output, *, stream=None):
    """Fused FP8 block-scale DeepSeek-V3 MoE layer; writes bf16 ``output`` [T, 7168] in place.

    Same positional arguments as the reference's ``run_moe`` (moe/solution/cuda/moe.cu:2987-2998);
    the number of local experts is taken from ``gemm1_weights.shape[0]`` (1..32).  Work is enqueued
    on the current CUDA stream and the call does not synchronise.  An ``output`` of dtype float32
    receives this rank's un-rounded partial sum instead (expert-parallel use).
    """
    out_dtype = output.dtype if isinstance(output, torch.Tensor) and output.dtype == torch.float32 else torch.bfloat16
    T, E, off, dev = _validate(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                               gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                               output, out_dtype, None)
    if T == 0:
        return output
    ctx = get_context(dev.index if dev.index is not None else torch.cuda.current_device(), T)
    fn = ctx.lib.syfi_moe_forward_partial_f32 if out_dtype == torch.float32 else ctx.lib.syfi_moe_forward
    _check(fn(ctx.handle, routing_logits.data_ptr(), routing_bias.data_ptr(), hidden_states.data_ptr(),
              hidden_states_scale.data_ptr(), gemm1_weights.data_ptr(), gemm1_weights_scale.data_ptr(),
              gemm2_weights.data_ptr(), gemm2_weights_scale.data_ptr(), T, E, off, float(routed_scaling_factor),
              output.data_ptr(), _stream_ptr(stream, ctx.device)))
    return output


def _register_torch_op():
    """Expose the layer as a torch operator, ``torch.ops.syfi_moe.run_moe`` (destination-passing like the
    reference's entry point: it mutates ``output`` and returns nothing), so that code built on the dispatcher
    — torch.compile graphs, operator registries of serving stacks — can call it like any other op.  The
    operator is a thin layer over :func:`run_moe`; the C ABI underneath stays the boundary other languages
    bind."""
    try:
        @torch.library.custom_op("syfi_moe::run_moe", mutates_args=("output",), device_types="cuda")
        def _op(routing_logits: torch.Tensor, routing_bias: torch.Tensor, hidden_states: torch.Tensor,
                hidden_states_scale: torch.Tensor, gemm1_weights: torch.Tensor, gemm1_weights_scale: torch.Tensor,
                gemm2_weights: torch.Tensor, gemm2_weights_scale: torch.Tensor, local_expert_offset: int,
                routed_scaling_factor: float, output: torch.Tensor) -> None:
            run_moe(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                    gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                    routed_scaling_factor, output)
        return _op
    except Exception:      # an older torch without custom_op: the plain function remains
        return None


torch_op = _register_torch_op()


class PackedWeights:
    """Weights rewritten by :func:`prepack_weights`: the two packed byte tensors (same sizes as the
    originals) and the expert count.  Pass ``packed.gemm1`` / ``packed.gemm2`` to :func:`run_moe_prepacked`
    in place of the weight tensors."""

    def __init__(self, gemm1, gemm2, num_local_experts):
        self.gemm1, self.gemm2, self.num_local_experts = gemm1, gemm2, int(num_local_experts)


def prepack_weights(gemm1_weights, gemm2_weights, *, stream=None) -> PackedWeights:
    """One-off re-layout of the expert weights for :func:`run_moe_prepacked` (see ``syfi_moe_prepack_weights``
    in the C header for the layout).  The originals are left untouched and may be freed afterwards."""
    f8 = torch.float8_e4m3fn
    if not isinstance(gemm1_weights, torch.Tensor) or gemm1_weights.dim() != 3 or gemm1_weights.device.type != "cuda":
        raise ValueError("gemm1_weights must be a 3-D CUDA tensor [E_local, 4096, 7168]")
    E, dev = gemm1_weights.shape[0], gemm1_weights.device
    if E < 1 or E > MAX_LOCAL_EXPERTS:
        raise ValueError(f"number of local experts must be in [1, {MAX_LOCAL_EXPERTS}], got {E}")
    _expect(gemm1_weights, "gemm1_weights", f8, (E, 2 * INTER, HIDDEN), dev)
    _expect(gemm2_weights, "gemm2_weights", f8, (E, HIDDEN, INTER), dev)
    p1 = torch.empty(E * 2 * INTER * HIDDEN, dtype=torch.uint8, device=dev)
    p2 = torch.empty(E * HIDDEN * INTER, dtype=torch.uint8, device=dev)
    ctx = get_context(dev.index if dev.index is not None else torch.cuda.current_device(), 1)
    _check(ctx.lib.syfi_moe_prepack_weights(ctx.handle, gemm1_weights.data_ptr(), gemm2_weights.data_ptr(), E,
                                            p1.data_ptr(), p2.data_ptr(), _stream_ptr(stream, ctx.device)))
    return PackedWeights(p1, p2, E)


def run_moe_prepacked(routing_logits, routing_bias, hidden_states, hidden_states_scale, packed: PackedWeights,
                      gemm1_weights_scale, gemm2_weights_scale, local_expert_offset, routed_scaling_factor, output,
                      *, stream=None):
    """:func:`run_moe` on weights packed once by :func:`prepack_weights`; bit-identical results."""
    if not isinstance(packed, PackedWeights):
        raise ValueError("packed must come from prepack_weights()")
    E, dev = packed.num_local_experts, packed.gemm1.device
    if not isinstance(routing_logits, torch.Tensor) or routing_logits.dim() != 2:
        raise ValueError("routing_logits must be a 2-D tensor [T, 256]")
    T = routing_logits.shape[0]
    off = int(local_expert_offset)
    if off < 0 or off + E > E_GLOBAL:
        raise ValueError(f"local experts [{off}, {off + E}) outside [0, {E_GLOBAL})")
    f8 = torch.float8_e4m3fn
    _expect(routing_logits, "routing_logits", torch.float32, (T, E_GLOBAL), dev)
    _expect(routing_bias, "routing_bias", torch.bfloat16, (E_GLOBAL,), dev)
    _expect(hidden_states, "hidden_states", f8, (T, HIDDEN), dev)
    _expect(hidden_states_scale, "hidden_states_scale", torch.float32, (HIDDEN // 128, T), dev)
    _expect(gemm1_weights_scale, "gemm1_weights_scale", torch.float32, (E, 2 * INTER // 128, HIDDEN // 128), dev)
    _expect(gemm2_weights_scale, "gemm2_weights_scale", torch.float32, (E, HIDDEN // 128, INTER // 128), dev)
    _expect(output, "output", torch.bfloat16, (T, HIDDEN), dev)
    if T == 0:
        return output
    ctx = get_context(dev.index if dev.index is not None else torch.cuda.current_device(), T)
    _check(ctx.lib.syfi_moe_forward_prepacked(
        ctx.handle, routing_logits.data_ptr(), routing_bias.data_ptr(), hidden_states.data_ptr(),
        hidden_states_scale.data_ptr(), packed.gemm1.data_ptr(), gemm1_weights_scale.data_ptr(),
        packed.gemm2.data_ptr(), gemm2_weights_scale.data_ptr(), T, E, off, float(routed_scaling_factor),
        output.data_ptr(), _stream_ptr(stream, ctx.device)))
    return output


def run_moe_host(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                 gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                 routed_scaling_factor, output, *, stream=None):
    """``run_moe`` for callers whose per-call tensors live in host memory (pinned for speed):
    logits, bias, hidden states and scales are copied to the device, the layer runs, and the
    bf16 result is copied back into the host tensor ``output`` before the call returns.  The
    weights stay resident on the device."""
    T, E, off, dev = _validate(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                               gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                               output, torch.bfloat16, "cpu")
    if T == 0:
        return output
    ctx = get_context(dev.index if dev.index is not None else torch.cuda.current_device(), T)
    _check(ctx.lib.syfi_moe_forward_host(
        ctx.handle, routing_logits.data_ptr(), routing_bias.data_ptr(), hidden_states.data_ptr(),
        hidden_states_scale.data_ptr(), gemm1_weights.data_ptr(), gemm1_weights_scale.data_ptr(),
        gemm2_weights.data_ptr(), gemm2_weights_scale.data_ptr(), T, E, off, float(routed_scaling_factor),
        output.data_ptr(), _stream_ptr(stream, ctx.device)))
    return output


def ep_region_bytes(world_size: int, tokens_per_rank: int) -> int:
    """Bytes every rank must allocate (symmetrically) for the peer-memory expert-parallel path."""
    n = int(load_library().syfi_moe_ep_region_bytes(int(world_size), int(tokens_per_rank)))
    if n <= 0:
        raise ValueError("world_size must be in [1, 8] and tokens_per_rank positive")
    return n


def run_moe_ep(desc: EpDesc, step: int, routing_logits, routing_bias, hidden_states, hidden_states_scale,
               gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
               routed_scaling_factor, output, *, stream=None, dispatch: bool = False):
    """One expert-parallel step through peer memory (see ``syfi_moe_ep_forward``): this rank's own
    tokens in, their bf16 outputs summed over all ranks' experts out.  ``step`` counts 1, 2, 3, ...
    identically on every rank.  ``dispatch`` selects token dispatch (``syfi_moe_ep_forward_dispatch``: only
    routed rows travel, each rank routes only its own tokens) instead of the all-gather of every token;
    the results are bit-identical."""
    T, E, off, dev = _validate(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                               gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                               output, torch.bfloat16, None)
    if T != desc.tokens_per_rank:
        raise ValueError(f"descriptor is for {desc.tokens_per_rank} tokens per rank, got {T}")
    ctx = get_context(dev.index, T * desc.world_size)
    fn = ctx.lib.syfi_moe_ep_forward_dispatch if dispatch else ctx.lib.syfi_moe_ep_forward
    _check(fn(
        ctx.handle, ctypes.byref(desc), int(step), routing_logits.data_ptr(), routing_bias.data_ptr(),
        hidden_states.data_ptr(), hidden_states_scale.data_ptr(), gemm1_weights.data_ptr(),
        gemm1_weights_scale.data_ptr(), gemm2_weights.data_ptr(), gemm2_weights_scale.data_ptr(), E, off,
        float(routed_scaling_factor), output.data_ptr(), _stream_ptr(stream, ctx.device)))
    return output


def ep_prepare(desc: EpDesc, device: int):
    """Allocate everything the expert-parallel steps for ``desc`` need (see ``syfi_moe_ep_prepare``); put a
    barrier of your own behind it on every rank before step 1."""
    ctx = get_context(device, int(desc.tokens_per_rank) * int(desc.world_size))
    _check(ctx.lib.syfi_moe_ep_prepare(ctx.handle, ctypes.byref(desc)))


def run_moe_ep_replicated(desc: EpDesc, step: int, routing_logits, routing_bias, hidden_states, hidden_states_scale,
                          gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                          routed_scaling_factor, output, *, stream=None):
    """One expert-parallel step with REPLICATED tokens through peer memory (``syfi_moe_ep_forward_replicated``):
    every rank passes all ``world_size * tokens_per_rank`` tokens and its expert slice; ``output`` receives the
    bf16 rows of this rank's tokens [rank * tokens_per_rank, ...) summed over all ranks, rounded once."""
    T_all = int(desc.tokens_per_rank) * int(desc.world_size)
    if not isinstance(output, torch.Tensor) or tuple(output.shape) != (int(desc.tokens_per_rank), HIDDEN):
        raise ValueError(f"output must have shape ({int(desc.tokens_per_rank)}, {HIDDEN})")
    T, E, off, dev = _validate(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                               gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                               None, torch.bfloat16, None)
    if T != T_all:
        raise ValueError(f"descriptor is for {T_all} tokens in all, got {T}")
    _expect(output, "output", torch.bfloat16, (int(desc.tokens_per_rank), HIDDEN), dev)
    ctx = get_context(dev.index, T_all)
    _check(ctx.lib.syfi_moe_ep_forward_replicated(
        ctx.handle, ctypes.byref(desc), int(step), routing_logits.data_ptr(), routing_bias.data_ptr(),
        hidden_states.data_ptr(), hidden_states_scale.data_ptr(), gemm1_weights.data_ptr(),
        gemm1_weights_scale.data_ptr(), gemm2_weights.data_ptr(), gemm2_weights_scale.data_ptr(), E, off,
        float(routed_scaling_factor), output.data_ptr(), _stream_ptr(stream, ctx.device)))
    return output


def route(routing_logits, routing_bias, local_expert_offset, routed_scaling_factor, num_local_experts=32):
    """Router only: returns (topk_idx int32 [T, 8], topk_weights f32 [T, 8]) on the device."""
    if not isinstance(routing_logits, torch.Tensor) or routing_logits.dim() != 2 or routing_logits.device.type != "cuda":
        raise ValueError("routing_logits must be a 2-D CUDA tensor [T, 256]")
    dev = routing_logits.device
    T = routing_logits.shape[0]
    _expect(routing_logits, "routing_logits", torch.float32, (T, E_GLOBAL), dev)
    _expect(routing_bias, "routing_bias", torch.bfloat16, (E_GLOBAL,), dev)
    idx = torch.empty(T, TOP_K, dtype=torch.int32, device=dev)
    w = torch.empty(T, TOP_K, dtype=torch.float32, device=dev)
    if T == 0:
        return idx, w
    ctx = get_context(dev.index, T)
    _check(ctx.lib.syfi_moe_route(ctx.handle, routing_logits.data_ptr(), routing_bias.data_ptr(), T,
                                  int(num_local_experts), int(local_expert_offset), float(routed_scaling_factor),
                                  idx.data_ptr(), w.data_ptr(), _stream_ptr(None, ctx.device)))
    return idx, w
