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

#include <mutex>

#include "../../include/syfi_moe.h"

namespace {

using tvm::ffi::TensorView;

std::mutex g_mu;
syfi_moe_ctx* g_ctx[64] = {nullptr};

void run_impl(TensorView routing_logits, TensorView routing_bias, TensorView hidden_states,
              TensorView hidden_states_scale, TensorView gemm1_weights, TensorView gemm1_weights_scale,
              TensorView gemm2_weights, TensorView gemm2_weights_scale, int64_t local_expert_offset,
              double routed_scaling_factor, TensorView output) {
  const int64_t T = routing_logits.shape()[0];
  if (T == 0) return;                                   // as the reference (moe.cu:3001)
  const DLDevice dev = routing_logits.device();
  TVM_FFI_ICHECK(dev.device_type == kDLCUDA) << "run_moe needs CUDA tensors";
  TVM_FFI_ICHECK(dev.device_id >= 0 && dev.device_id < 64);
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
