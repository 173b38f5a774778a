// Weight-only int4 skinny GEMM for decode on the sm_100a tensor cores:
//   y[M, N] = x[M, K] . dequant(Wq)[N, K]^T      (M <= 64 activation rows)
// computed transposed, y^T = W x^T, so the 128-row UMMA dimension runs over output features and
// the small activation batch is the UMMA N dimension (32 or 64).
//
// One CTA owns 128 output features and a slice of K (split-K fills the machine when N / 128 is
// small; every split writes its own fp32 slice and the slices are summed afterwards, so the result
// does not depend on the order in which CTAs finish).
//   warp 0       TMA producer: packed int4 weights [128 x 32 bytes] and the activation tile
//                [32|64 rows x 64 k] per 64-wide k-block, 4-stage ring
//   warp 1       MMA issuer and TMEM owner
//   warps 2..9   dequantise: two threads per weight row turn the 4-bit codes into bf16
//                ((code - 8) * scale, scale per row and group of 128 k) and write them as the
//                128-byte-swizzled K-major A operand; warps 2..5 also run the epilogue
// Weights are read from HBM exactly once, as 4-bit codes.  All waits are bounded.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cudaTypedefs.h>

#include <map>
#include <mutex>

#include "common.cuh"
#include "ops.h"
#include "sm100_ptx.cuh"

namespace vrl {
namespace i4 {

using namespace ptx;

constexpr int kRows = 128;                 // output features per CTA
constexpr int kBK = 64;                    // k per stage
constexpr int kStages = 3;                 // 3 x 28 KiB: two CTAs fit on one SM
constexpr int kThreads = 320;
constexpr uint32_t kRawBytes = kRows * 32;         // packed codes of one k-block
constexpr uint32_t kABytes = kRows * 128;          // dequantised bf16 A tile
constexpr uint32_t kXBytesMax = 64 * 128;          // activation tile (up to 64 rows)
constexpr uint32_t kStageBytes = kABytes + kXBytesMax + kRawBytes;      // 28 KiB
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024 + 256;
constexpr uint32_t kTmemCols = 64;

enum Status : int { kOk = 0, kTimeoutProducer = 21, kTimeoutMma = 22, kTimeoutDequant = 23 };

struct Params {
  const __nv_bfloat16* scales;     // [N, K / group]
  const __nv_bfloat16* bias;       // [N] or null
  float* acc;                      // [ksplit, M, N] fp32 partial results, one slice per K split
  int* status;
  int m, n, k, group;
  int nmma;                        // 32 or 64: UMMA N (activation rows, zero padded)
  int ksplit;
};

__global__ void __launch_bounds__(kThreads, 2)
int4_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* raw_full = bars;                   // [kStages] TMA landed
  uint64_t* a_full = bars + kStages;           // [kStages] dequantised (8 warps arrive)
  uint64_t* empty = bars + 2 * kStages;        // [kStages] MMAs have read the stage
  uint64_t* acc_full = bars + 3 * kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * kStages + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kRows;
  const int k_blocks = p.k / kBK;
  const int per_split = (k_blocks + p.ksplit - 1) / p.ksplit;
  const int kb_begin = blockIdx.y * per_split;
  const int kb_end = min(k_blocks, kb_begin + per_split);
  const int my_blocks = max(0, kb_end - kb_begin);
  const uint32_t x_bytes = (uint32_t)p.nmma * 128u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&a_full[s], 8);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (my_blocks > 0) {
    if (warp == 0 && lane == 0) {
      // --------------------------------------------------------------------- TMA producer
      bool ok = true;
      for (int it = 0; it < my_blocks; ++it) {
        const int s = it % kStages;
        if (!mbar_wait(&empty[s], ((it / kStages) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        uint8_t* stage = smem + s * kStageBytes;
        const int kb = kb_begin + it;
        mbar_expect_tx(&raw_full[s], kRawBytes + x_bytes);
        tma_load_2d(stage + kABytes + kXBytesMax, &map_w, &raw_full[s], kb * 8, n0);
        tma_load_2d(stage + kABytes, &map_x, &raw_full[s], kb * kBK, 0);
      }
      if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutProducer);
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------------------- MMA issuer
      const uint32_t idesc = make_idesc(kRows, p.nmma, 0, 0);
      bool ok = true;
      for (int it = 0; it < my_blocks; ++it) {
        const int s = it % kStages;
        if (!mbar_wait(&a_full[s], (it / kStages) & 1u, abort_flag)) { ok = false; break; }
        tmem_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * kStageBytes), x_addr = a_addr + kABytes;
#pragma unroll
        for (int kk = 0; kk < kBK / 16; ++kk)
          umma_bf16(tmem_base, make_desc(a_addr + kk * 32, 16, 1024), make_desc(x_addr + kk * 32, 16, 1024),
                    idesc, (it | kk) ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(acc_full);
      else if (atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutMma);
    } else if (warp >= 2) {
      // ------------------------------------------------------------------------ dequantise
      const int t = threadIdx.x - 64;              // 0..255
      const int row = t >> 1, half = t & 1;        // two threads per weight row, 4 words each
      const int n = n0 + row;
      const int groups_per_row = p.k / p.group;
      bool ok = true;
      // the group scale of the NEXT k-block is requested before this one's barrier wait: a global
      // load in front of every dequantisation would otherwise sit on the critical path of the stage
      const __nv_bfloat16* srow = p.scales + (int64_t)min(n, p.n - 1) * groups_per_row;
      float sc_next = n < p.n ? __bfloat162float(srow[(kb_begin * kBK) / p.group]) : 0.f;
      for (int it = 0; it < my_blocks; ++it) {
        const int s = it % kStages;
        const float sc = sc_next;
        if (it + 1 < my_blocks && n < p.n) sc_next = __bfloat162float(srow[((kb_begin + it + 1) * kBK) / p.group]);
        ok = __all_sync(0xffffffffu, mbar_wait(&raw_full[s], (it / kStages) & 1u, abort_flag));
        if (!ok) break;
        uint8_t* stage = smem + s * kStageBytes;
        const uint4 words = *reinterpret_cast<const uint4*>(stage + kABytes + kXBytesMax + row * 32 + half * 16);
        const uint32_t w[4] = {words.x, words.y, words.z, words.w};
        const uint32_t a_row = smem_u32(stage) + row * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = (float)((int)((w[j] >> (4 * e)) & 15u) - 8) * sc;
          const bf16x8 o = pack8(f);
          const uint32_t chunk = (uint32_t)(half * 4 + j);           // 8 k per 16-byte chunk
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                           a_row + ((chunk ^ (uint32_t)(row & 7)) << 4)),
                       "r"(o.u.x), "r"(o.u.y), "r"(o.u.z), "r"(o.u.w)
                       : "memory");
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[s]);
      }
      // ------------------------------------------------------------------------- epilogue
      if (ok && warp < 6) {
        ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, abort_flag));
        if (ok) {
          tmem_fence_after();
          const int quarter = warp & 3;
          const int col = n0 + quarter * 32 + lane;
          const float b = (p.bias != nullptr && blockIdx.y == 0 && col < p.n) ? __bfloat162float(p.bias[col]) : 0.f;
          for (int c = 0; c < p.nmma / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c * 32, r);
            tmem_ld_wait();
            if (col < p.n) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int mrow = c * 32 + i;
                if (mrow < p.m)
                  p.acc[((int64_t)blockIdx.y * p.m + mrow) * p.n + col] = __uint_as_float(r[i]) + b;
              }
            }
          }
        }
      }
      if (!ok && lane == 0 && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0)
        atomicExch(p.status, kTimeoutDequant);
    }
  }

  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------------------- host side
using EncodeFn = PFN_cuTensorMapEncodeTiled_v12000;

static EncodeFn encode_fn() {
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

static CUtensorMap make_map(const void* base, CUtensorMapDataType type, uint64_t elem_bytes, uint64_t inner,
                            uint64_t outer, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
  CUtensorMap map;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * elem_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem[2] = {1, 1};
  CUresult rc = encode_fn()(&map, type, 2, const_cast<void*>(base), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(rc == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)rc);
  return map;
}

static int* status_word(int device) { return kernel_status_block(device) + kStatusInt4Gemm; }

// Sum of the split-K partial products, rounded to bf16 once: out[i] = sum_s acc[s, i].
__global__ void splitk_sum_bf16_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out,
                                       int splits, int64_t elems) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= elems) return;
  if (i + 3 < elems) {
    float4 t = *reinterpret_cast<const float4*>(acc + i);
    for (int sp = 1; sp < splits; ++sp) {
      const float4 u = *reinterpret_cast<const float4*>(acc + (int64_t)sp * elems + i);
      t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(t.x, t.y), hi = __floats2bfloat162_rn(t.z, t.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + i) = packed;
  } else {
    for (int64_t j = i; j < elems; ++j) {
      float t = 0.f;
      for (int sp = 0; sp < splits; ++sp) t += acc[(int64_t)sp * elems + j];
      out[j] = __float2bfloat16_rn(t);
    }
  }
}

}  // namespace i4

torch::Tensor int4_gemm(torch::Tensor x, torch::Tensor qweight, torch::Tensor scales,
                        c10::optional<torch::Tensor> bias, int64_t group) {
  using namespace i4;
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.is_contiguous());
  TORCH_CHECK(qweight.scalar_type() == torch::kInt32 && qweight.dim() == 2 && qweight.is_contiguous());
  TORCH_CHECK(scales.scalar_type() == torch::kBFloat16 && scales.is_contiguous());
  const int64_t m = x.size(0), k = x.size(1), n = qweight.size(0);
  TORCH_CHECK(m >= 1 && m <= 64, "int4_gemm: 1..64 activation rows");
  VRL_CHECK_OPERAND(qweight, x);
  VRL_CHECK_OPERAND(scales, x);
  VRL_CHECK_OPERAND(bias, x);
  TORCH_CHECK(k % kBK == 0 && qweight.size(1) * 8 == k, "int4_gemm: K must be a multiple of 64");
  TORCH_CHECK(group % kBK == 0 && k % group == 0 && scales.numel() == n * (k / group),
              "int4_gemm: scales must be [N, K / group] with group a multiple of 64");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(qweight.data_ptr()) % 16 == 0, "int4_gemm: 16-byte alignment");
  const c10::cuda::CUDAGuard guard(x.device());
  static thread_local bool context_bound = false;   // the encoder is a driver entry point
  if (!context_bound) {
    C10_CUDA_CHECK(cudaFree(nullptr));
    context_bound = true;
  }
  const __nv_bfloat16* bias_p = nullptr;
  torch::Tensor bias_c;
  if (bias.has_value()) {
    bias_c = bias->to(torch::kBFloat16).contiguous();
    TORCH_CHECK(bias_c.numel() == n);
    bias_p = reinterpret_cast<const __nv_bfloat16*>(bias_c.data_ptr());
  }
  Params p{};
  p.scales = reinterpret_cast<const __nv_bfloat16*>(scales.data_ptr());
  p.bias = bias_p;
  p.status = status_word(x.get_device());
  p.m = (int)m; p.n = (int)n; p.k = (int)k; p.group = (int)group;
  p.nmma = m <= 32 ? 32 : 64;
  if (m != p.nmma) {        // the activation tile is a full 32/64-row TMA box: pad with zero rows
    auto padded = torch::zeros({(int64_t)p.nmma, k}, x.options());
    padded.narrow(0, 0, m).copy_(x);
    x = padded;
  }
  const int n_tiles = (int)((n + kRows - 1) / kRows);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int k_blocks = (int)(k / kBK);
  // Split K so that the whole grid is resident at once (two CTAs per SM): a second, partly filled
  // wave would double the time of a kernel whose CTAs all take the same few microseconds.
  const int want = std::max(1, std::min((2 * sms) / n_tiles, std::max(1, k_blocks / 4)));
  const int per_split = (k_blocks + want - 1) / want;
  p.ksplit = (k_blocks + per_split - 1) / per_split;       // no empty split: every slice is written
  auto acc = torch::empty({(int64_t)p.ksplit, m, n}, x.options().dtype(torch::kFloat32));
  p.acc = acc.data_ptr<float>();
  const CUtensorMap map_w = make_map(qweight.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_INT32, 4, k / 8, n, 8, kRows,
                                     CU_TENSOR_MAP_SWIZZLE_NONE);
  const CUtensorMap map_x = make_map(x.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k, p.nmma, kBK, p.nmma,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
  static const bool attr_set = [] {
    C10_CUDA_CHECK(cudaFuncSetAttribute(int4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        kSmemBytes));
    return true;
  }();
  (void)attr_set;
  int4_gemm_kernel<<<dim3(n_tiles, p.ksplit), kThreads, kSmemBytes, at::cuda::getCurrentCUDAStream()>>>(
      map_w, map_x, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  auto y = torch::empty({m, n}, x.options());
  const int64_t elems = m * n;                 // m * n * 4 bytes per slice: slices stay 16-byte aligned when elems % 4 == 0
  if (elems % 4 != 0) return (p.ksplit == 1 ? acc.select(0, 0) : acc.sum(0)).to(torch::kBFloat16);
  splitk_sum_bf16_kernel<<<(unsigned)((elems / 4 + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      acc.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), p.ksplit, elems);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

}  // namespace vrl
