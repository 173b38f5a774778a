// One block of kernel status words per device.
//
// Every kernel with bounded waits (bf16 GEMM, flash attention, int4 GEMM) records where it gave
// up in its own word of this block.  Keeping the words side by side lets a training step poll all
// of them with a single 16-byte device-to-host copy.
#include <c10/cuda/CUDAException.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>

#include "ops.h"

namespace vrl {

int* kernel_status_block(int device) {
  static std::map<int, int*> blocks;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  auto it = blocks.find(device);
  if (it != blocks.end()) return it->second;
  int* w = nullptr;
  C10_CUDA_CHECK(cudaMalloc(&w, kStatusWords * sizeof(int)));
  C10_CUDA_CHECK(cudaMemset(w, 0, kStatusWords * sizeof(int)));
  blocks[device] = w;
  return w;
}

static int64_t read_and_clear(int index) {
  int device = 0;
  C10_CUDA_CHECK(cudaGetDevice(&device));
  int* word = kernel_status_block(device) + index;
  int host = 0;
  C10_CUDA_CHECK(cudaMemcpy(&host, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (host != 0) C10_CUDA_CHECK(cudaMemset(word, 0, sizeof(int)));
  return host;
}

int64_t gemm_last_status() { return read_and_clear(kStatusGemm); }
int64_t flash_attn_last_status() { return read_and_clear(kStatusAttention); }
int64_t int4_gemm_last_status() { return read_and_clear(kStatusInt4Gemm); }

std::vector<int64_t> kernel_status_all() {
  int device = 0;
  C10_CUDA_CHECK(cudaGetDevice(&device));
  int* block = kernel_status_block(device);
  int host[kStatusWords] = {0, 0, 0, 0};
  C10_CUDA_CHECK(cudaMemcpy(host, block, sizeof(host), cudaMemcpyDeviceToHost));
  bool any = false;
  for (int v : host) any = any || v != 0;
  if (any) C10_CUDA_CHECK(cudaMemset(block, 0, sizeof(host)));
  return {host[kStatusGemm], host[kStatusAttention], host[kStatusInt4Gemm]};
}

}  // namespace vrl
