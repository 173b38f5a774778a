// Issue-cost probe for the tensor-core path: one thread of one CTA issues groups of tcgen05.mma
// (M = 128, K = 16, bf16, operands all zero) and optionally a tcgen05.commit and an already
// complete mbarrier wait (try_wait loop = 1, single test_wait = 2) after every group, and reports cycles per group as seen by that thread
// and until the last product has completed.  The attention and GEMM kernels size their steps by
// these numbers: what one issuing thread can sustain bounds a CTA that uses small tiles.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "ops.h"
#include "sm100_ptx.cuh"

namespace vrl {
namespace probe {

using namespace ptx;

constexpr int kSmemBytes = 64 * 1024;

// GROUP and TMEM_A are compile-time so that the group unrolls and every operand is set up ahead of
// the loop: a loop the compiler cannot unroll costs the issuing thread about 140 cycles per product
// (each step of the address arithmetic is a dependent instruction feeding a uniform register).
template <int N, int GROUP, bool TMEM_A>
__global__ void __launch_bounds__(128, 1)
mma_issue_kernel(long long* out, int iters, int commit_each, int wait_each) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t done, ring[4], ready;
  __shared__ uint32_t slot;
  __shared__ int abort_flag;
  for (int i = threadIdx.x; i < kSmemBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    mbar_init(&done, 1);
    mbar_init(&ready, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&ring[i], 1);
    abort_flag = 0;
    mbar_fence_init();
    fence_async_smem();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) tmem_alloc(&slot, 512);
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tm = slot;
  if (warp == 1 && lane == 0) {
    constexpr uint32_t idesc = make_idesc(128, N, 0, 0);
    constexpr uint32_t hi = desc_hi(1024);
    // A: 128 rows x 64 columns at offset 0; B: N rows x 64 columns at 16 KB (N <= 256 -> 32 KB)
    const uint32_t a_lo = desc_lo(smem_u32(smem), 16), b_lo = desc_lo(smem_u32(smem + 16384), 16);
    bool ok = true;
    const long long t0 = clock64();
    for (int i = 0; i < iters && ok; ++i) {
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
        const uint32_t kk = (uint32_t)(g & 3) * 2;          // 32 bytes along K, in 16-byte units
        const uint32_t acc = tm + (uint32_t)(g & 1) * 256;  // two accumulators, alternating
        if (TMEM_A) umma_bf16_tmem_a(acc, tm + 248, b_lo + kk, hi, idesc, 1u);   // A: columns 248..255
        else umma_bf16_split(acc, a_lo + kk, hi, b_lo + kk, hi, idesc, 1u);
      }
      if (commit_each) umma_commit(&ring[i & 3]);
      // parity 1 of a barrier that never completed a phase: the wait succeeds at once
      if (wait_each == 1) ok = mbar_wait(&ready, 1, &abort_flag);
      if (wait_each == 2) ok = mbar_test(&ready, 1);          // the non-blocking form
    }
    umma_commit(&done);
    const long long t1 = clock64();
    ok = mbar_wait(&done, 0, &abort_flag) && ok;
    const long long t2 = clock64();
    out[0] = t1 - t0;
    out[1] = t2 - t0;
    out[2] = ok ? 1 : 0;
  }
  tmem_fence_before();
  __syncthreads();
  if (warp == 0) {
    tmem_fence_after();
    tmem_dealloc(tm, 512);
  }
}

template <int N, int GROUP, bool TMEM_A>
static void launch(long long* out, int iters, int commit_each, int wait_each, cudaStream_t stream) {
  C10_CUDA_CHECK(cudaFuncSetAttribute(mma_issue_kernel<N, GROUP, TMEM_A>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  mma_issue_kernel<N, GROUP, TMEM_A><<<1, 128, kSmemBytes, stream>>>(out, iters, commit_each, wait_each);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <int N>
static void dispatch(long long* out, int iters, int group, int commit_each, int wait_each, bool tmem_a,
                     cudaStream_t stream) {
  if (tmem_a) {
    if (group == 4) launch<N, 4, true>(out, iters, commit_each, wait_each, stream);
    else launch<N, 8, true>(out, iters, commit_each, wait_each, stream);
  } else {
    if (group == 4) launch<N, 4, false>(out, iters, commit_each, wait_each, stream);
    else launch<N, 8, false>(out, iters, commit_each, wait_each, stream);
  }
}

}  // namespace probe

// Returns [issue cycles, cycles until complete, ok] for `iters` groups of `group` products of width n.
torch::Tensor mma_issue_probe(int64_t n, int64_t iters, int64_t group, bool commit_each, int64_t wait_each,
                              bool tmem_a) {
  TORCH_CHECK(n == 64 || n == 128 || n == 256, "mma_issue_probe: n in {64, 128, 256}");
  TORCH_CHECK(iters > 0 && iters <= 4096 && (group == 4 || group == 8), "mma_issue_probe: groups of 4 or 8");
  TORCH_CHECK(n != 256 || (!tmem_a && group == 8), "mma_issue_probe: n = 256 runs groups of 8 from shared memory only");
  auto out = torch::zeros({3}, torch::dtype(torch::kInt64).device(torch::kCUDA));
  auto stream = at::cuda::getCurrentCUDAStream();
  auto* ptr = reinterpret_cast<long long*>(out.data_ptr<int64_t>());
  if (n == 64) probe::dispatch<64>(ptr, (int)iters, (int)group, commit_each, (int)wait_each, tmem_a, stream);
  else if (n == 128) probe::dispatch<128>(ptr, (int)iters, (int)group, commit_each, (int)wait_each, tmem_a, stream);
  else probe::launch<256, 8, false>(ptr, (int)iters, commit_each, (int)wait_each, stream);
  return out.cpu();
}

}  // namespace vrl
