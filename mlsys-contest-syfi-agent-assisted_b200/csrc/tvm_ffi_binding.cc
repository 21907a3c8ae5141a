// Optional tvm-ffi export of the layer under the reference's own symbol.
//
// The reference is loaded by its harness through tvm-ffi: `binding = "tvm-ffi"`, entry point
// `moe.cu::run_moe` (moe/config.toml:7-11), exported with
// TVM_FFI_DLL_EXPORT_TYPED_FUNC(run_moe, run_impl) (moe/solution/cuda/moe.cu:3260).  This file exports
// the same symbol (`__tvm_ffi_run_moe`) with the same typed signature (moe.cu:2987-2998) and forwards
// to the C ABI of include/syfi_moe.h, so a harness that dlopens the reference's library can dlopen
// this one instead.  It is built into a separate shared object (libsyfi_moe_tvmffi.so) because it is
// the only translation unit that needs the tvm-ffi headers and runtime.
#include <tvm/ffi/container/tensor.h>
#include <tvm/ffi/error.h>
#include <tvm/ffi/extra/c_env_api.h>
#include <tvm/ffi/function.h>

#include <cstdint>
#include <initializer_list>
#include <mutex>

#include "../../include/syfi_moe.h"

namespace {

using tvm::ffi::TensorView;

std::mutex g_mu;
syfi_moe_ctx* g_ctx[64] = {nullptr};

enum class Kind { kF32, kBF16, kE4M3 };

// One argument of the entry point: dtype, rank, every dimension, device and contiguity.  The reference
// checks none of this (moe.cu:3045-3053 takes the data pointers as they are); a harness that hands over a
// tensor of another shape would make the kernels read out of bounds, so everything is checked here and
// the error names the argument.
void expect(const TensorView& t, const char* name, Kind kind, std::initializer_list<int64_t> shape, DLDevice dev) {
  const DLDataType dt = t.dtype();
  bool dtype_ok = dt.lanes == 1;
  if (kind == Kind::kF32) dtype_ok = dtype_ok && dt.code == kDLFloat && dt.bits == 32;
  if (kind == Kind::kBF16) dtype_ok = dtype_ok && dt.code == kDLBfloat && dt.bits == 16;
  // e4m3 tensors arrive as float8_e4m3fn, or as plain bytes from frameworks whose DLPack export has no fp8
  if (kind == Kind::kE4M3) dtype_ok = dtype_ok && dt.bits == 8 && (dt.code == kDLFloat8_e4m3fn || dt.code == kDLUInt);
  TVM_FFI_ICHECK(dtype_ok) << "run_moe: " << name << " has the wrong dtype (code " << int(dt.code) << ", " << int(dt.bits)
                           << " bits)";
  TVM_FFI_ICHECK(t.ndim() == static_cast<int32_t>(shape.size()))
      << "run_moe: " << name << " must have " << shape.size() << " dimensions, got " << t.ndim();
  int i = 0;
  int64_t expect_stride = 1;
  for (int64_t want : shape) {
    TVM_FFI_ICHECK(t.size(i) == want) << "run_moe: " << name << " dimension " << i << " must be " << want << ", got "
                                      << t.size(i);
    ++i;
  }
  for (int d = t.ndim() - 1; d >= 0; --d) {   // row-major, dense
    TVM_FFI_ICHECK(t.size(d) == 1 || t.stride(d) == expect_stride) << "run_moe: " << name << " must be contiguous";
    expect_stride *= t.size(d);
  }
  const DLDevice d = t.device();
  TVM_FFI_ICHECK(d.device_type == dev.device_type && d.device_id == dev.device_id)
      << "run_moe: " << name << " is on another device than routing_logits";
  TVM_FFI_ICHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0) << "run_moe: " << name << " is not 16-byte aligned";
}

void run_impl(TensorView routing_logits, TensorView routing_bias, TensorView hidden_states,
              TensorView hidden_states_scale, TensorView gemm1_weights, TensorView gemm1_weights_scale,
              TensorView gemm2_weights, TensorView gemm2_weights_scale, int64_t local_expert_offset,
              double routed_scaling_factor, TensorView output) {
  TVM_FFI_ICHECK(routing_logits.ndim() == 2) << "run_moe: routing_logits must be [T, 256]";
  const int64_t T = routing_logits.shape()[0];
  if (T == 0) return;                                   // as the reference (moe.cu:3001)
  const DLDevice dev = routing_logits.device();
  TVM_FFI_ICHECK(dev.device_type == kDLCUDA) << "run_moe needs CUDA tensors";
  TVM_FFI_ICHECK(dev.device_id >= 0 && dev.device_id < 64);
  TVM_FFI_ICHECK(gemm1_weights.ndim() == 3) << "run_moe: gemm1_weights must be [E_local, 4096, 7168]";
  const int64_t E = gemm1_weights.shape()[0];
  TVM_FFI_ICHECK(E >= 1 && E <= 32) << "run_moe: 1 to 32 local experts, got " << E;
  TVM_FFI_ICHECK(local_expert_offset >= 0 && local_expert_offset + E <= 256)
      << "run_moe: local experts [" << local_expert_offset << ", " << local_expert_offset + E << ") outside [0, 256)";
  expect(routing_logits, "routing_logits", Kind::kF32, {T, 256}, dev);
  expect(routing_bias, "routing_bias", Kind::kBF16, {256}, dev);
  expect(hidden_states, "hidden_states", Kind::kE4M3, {T, 7168}, dev);
  expect(hidden_states_scale, "hidden_states_scale", Kind::kF32, {56, T}, dev);
  expect(gemm1_weights, "gemm1_weights", Kind::kE4M3, {E, 4096, 7168}, dev);
  expect(gemm1_weights_scale, "gemm1_weights_scale", Kind::kF32, {E, 32, 56}, dev);
  expect(gemm2_weights, "gemm2_weights", Kind::kE4M3, {E, 7168, 2048}, dev);
  expect(gemm2_weights_scale, "gemm2_weights_scale", Kind::kF32, {E, 56, 16}, dev);
  expect(output, "output", Kind::kBF16, {T, 7168}, dev);
  syfi_moe_ctx* ctx;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_ctx[dev.device_id] == nullptr && syfi_moe_create(dev.device_id, T, &g_ctx[dev.device_id]) != 0)
      TVM_FFI_THROW(RuntimeError) << syfi_moe_last_error();
    ctx = g_ctx[dev.device_id];
  }
  // the stream the caller made current for tvm-ffi (the reference ignores it and uses stream 0)
  void* stream = TVMFFIEnvGetStream(dev.device_type, dev.device_id);
  const int rc = syfi_moe_forward(ctx, routing_logits.data_ptr(), routing_bias.data_ptr(), hidden_states.data_ptr(),
                                  hidden_states_scale.data_ptr(), gemm1_weights.data_ptr(),
                                  gemm1_weights_scale.data_ptr(), gemm2_weights.data_ptr(),
                                  gemm2_weights_scale.data_ptr(), T, static_cast<int32_t>(gemm1_weights.shape()[0]),
                                  local_expert_offset, routed_scaling_factor, output.data_ptr(), stream);
  if (rc != 0) TVM_FFI_THROW(RuntimeError) << syfi_moe_last_error();
}

}  // namespace

TVM_FFI_DLL_EXPORT_TYPED_FUNC(run_moe, run_impl);
