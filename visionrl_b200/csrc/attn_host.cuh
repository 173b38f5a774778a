// Host-side helpers shared by the attention forward and backward: the driver's tensor-map encoder,
// 4-D maps over [B, H, S, D] bf16 views and the per-device status word.
#pragma once

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cudaTypedefs.h>
#include <torch/extension.h>

#include <map>
#include <mutex>

namespace vrl {
namespace attn {

using EncodeFn = PFN_cuTensorMapEncodeTiled_v12000;

inline EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    C10_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q));
    TORCH_CHECK(ptr != nullptr && q == cudaDriverEntryPointSuccess,
                "cuTensorMapEncodeTiled is not available from this driver");
    return reinterpret_cast<EncodeFn>(ptr);
  }();
  return fn;
}

// A [B, H, S, D] bf16 view with unit stride in D: dims {D, S, H, B}; box = 64 columns x `box_rows`
// rows of one (batch, head), 128-byte swizzle.  Rows past S read as zeros.
inline CUtensorMap make_map4(const torch::Tensor& t, int box_rows) {
  CUtensorMap map;
  cuuint64_t dims[4] = {(cuuint64_t)t.size(3), (cuuint64_t)t.size(2), (cuuint64_t)t.size(1),
                        (cuuint64_t)t.size(0)};
  cuuint64_t strides[3] = {(cuuint64_t)t.stride(2) * 2, (cuuint64_t)t.stride(1) * 2,
                           (cuuint64_t)t.stride(0) * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult rc = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.data_ptr(), dims, strides, box,
                            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(rc == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)rc);
  return map;
}

// A tensor the 4-D map can describe as is: unit stride in D, other strides multiples of 16 bytes.
inline torch::Tensor mappable(torch::Tensor t) {
  const bool ok = t.stride(3) == 1 && t.stride(0) % 8 == 0 && t.stride(1) % 8 == 0 && t.stride(2) % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0;
  return ok ? t : t.contiguous();
}

// One status word per device, shared by the forward and the backward kernels.
int* status_word(int device);

// The tensor-map encoder is a driver entry point: make sure this thread has a current context.
inline void bind_context() {
  static thread_local bool bound = false;
  if (!bound) {
    C10_CUDA_CHECK(cudaFree(nullptr));
    bound = true;
  }
}

}  // namespace attn
}  // namespace vrl
