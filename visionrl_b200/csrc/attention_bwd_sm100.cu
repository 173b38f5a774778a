// Bidirectional flash attention backward for sm_100a on tcgen05.mma with every accumulator in
// tensor memory.
//
// Two launches of one kernel template, so that no gradient needs atomics and the result is
// deterministic:
//   dK/dV pass  a CTA owns 128 keys of one (batch, head) and streams the queries in tiles of 64
//   dQ pass     a CTA owns 128 queries and streams the keys in tiles of 64
// Both recompute the probabilities from the saved log-sum-exp.  With "own" the CTA's resident tile
// pair and "str" the streamed pair, one step is
//   S'  = own1 . str1^T            (K Q^T   |  Q K^T)        128 x 64, TMEM
//   dP' = own2 . str2^T            (V dO^T  |  dO V^T)       128 x 64, TMEM
//   P   = exp2(S' * scale * log2e - LSE * log2e),  dS = P * (dP' - delta)   in registers, bf16 to smem
//   acc1 += P  . str2              (dV += P^T dO)            dK/dV pass only
//   acc2 += dS . str1              (dK += dS^T Q  |  dQ += dS K)
// where delta = rowsum(dO * O) per query comes from a small pre-pass.  The streamed tiles are read
// twice from the same shared-memory copy: K-major for the first two products, MN-major for the
// accumulating ones.
//
//   warp 0      producer: own tiles once, then streamed tiles (and, in the dK/dV pass, the
//               queries' LSE and delta) through a ring
//   warp 1      MMA issuer and TMEM owner; S'/dP' are double-buffered so that the tensor core
//               works on step j+1 while the other warps handle step j
//   warps 2..9  elementwise: two threads per owned row, 32 of the 64 columns each; no reductions
//               across threads are needed in the backward
// TMEM columns: [S'0 dP'0 S'1 dP'1] (64 each), acc1 (D), acc2 (D).  Every wait is bounded; on
// expiry the role records a status code, raises the CTA's abort flag and all roles fall through to
// the common exit where the TMEM is released.
#include "attn_host.cuh"
#include "common.cuh"
#include "ops.h"
#include "sm100_ptx.cuh"

namespace vrl {
namespace attn_bwd {

using namespace ptx;

constexpr int kOwn = 128;                  // rows the CTA owns
constexpr int kStr = 64;                   // streamed rows per step
constexpr int kThreads = 320;
constexpr uint32_t kOwnBlock = kOwn * 128;       // one 64-column swizzle block of an owned tile
constexpr uint32_t kStrBlock = kStr * 128;       // the same for a streamed tile
constexpr uint32_t kPBytes = kOwn * kStr * 2;    // one P or dS tile (bf16, one swizzle block wide)

enum Status : int { kOk = 0, kTimeoutProducer = 21, kTimeoutMma = 22, kTimeoutElementwise = 23,
                    kMisalignedSmem = 24 };

template <int D>
struct Cfg {
  static constexpr int kDBlocks = D / 64;
  static constexpr int kStages = D == 64 ? 4 : 3;
  static constexpr uint32_t kOwnBytes = kDBlocks * kOwnBlock;
  static constexpr uint32_t kStrBytes = kDBlocks * kStrBlock;
  static constexpr uint32_t kVecBytes = kStages * kStr * 4;          // LSE or delta of the staged queries
  static constexpr uint32_t kSmemBytes =
      2 * kOwnBytes + 2 * kStages * kStrBytes + 4 * kPBytes + 2 * kVecBytes + 256;
  static constexpr uint32_t kAcc1Col = 4 * kStr;
  static constexpr uint32_t kAcc2Col = 4 * kStr + D;
  static constexpr uint32_t kTmemCols = 512;
};

struct Params {
  __nv_bfloat16* out1;    // dV, token-major [B, S_own, H, D] (dK/dV pass only)
  __nv_bfloat16* out2;    // dK (dK/dV pass) or dQ (dQ pass), token-major [B, S_own, H, D]
  const float* lse;       // [B, H, Sq] natural log
  const float* delta;     // [B, H, Sq]
  int heads;
  int s_own, s_str, sq;
  float scale_log2;       // softmax scale times log2(e)
  float scale;
  int* status;
};

template <int D, bool kDQ>
__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap map_own1, const __grid_constant__ CUtensorMap map_own2,
                 const __grid_constant__ CUtensorMap map_str1, const __grid_constant__ CUtensorMap map_str2,
                 const Params p) {
  using C = Cfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {          // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(p.status, kMisalignedSmem);
    return;
  }
  uint8_t* so1 = smem;
  uint8_t* so2 = so1 + C::kOwnBytes;
  uint8_t* ss1 = so2 + C::kOwnBytes;                       // [kStages]
  uint8_t* ss2 = ss1 + C::kStages * C::kStrBytes;          // [kStages]
  uint8_t* sp = ss2 + C::kStages * C::kStrBytes;           // P [2]
  uint8_t* sds = sp + 2 * kPBytes;                         // dS [2]
  float* lse_s = reinterpret_cast<float*>(sds + 2 * kPBytes);      // [kStages][kStr], times log2(e)
  float* del_s = lse_s + C::kStages * kStr;                        // [kStages][kStr]
  uint64_t* bars = reinterpret_cast<uint64_t*>(del_s + C::kStages * kStr);
  uint64_t* own_full = bars;
  uint64_t* str_full = bars + 1;                   // [kStages]
  uint64_t* str_empty = str_full + C::kStages;     // [kStages]
  uint64_t* s_full = str_empty + C::kStages;       // [2]
  uint64_t* p_full = s_full + 2;                   // [2]
  uint64_t* p_empty = p_full + 2;                  // [2]
  uint64_t* acc_full = p_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* skip_flag = abort_flag + 1;

  // a CTA of this or an earlier launch already gave up: the results are void, do not add more waits
  if (threadIdx.x == 0) *skip_flag = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (*skip_flag != 0) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, r0 = blockIdx.x * kOwn;
  const int bi = bh / p.heads, hi = bh % p.heads;
  const int n_tiles = (p.s_str + kStr - 1) / kStr;

  if (threadIdx.x == 0) {
    mbar_init(own_full, 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&str_full[s], 1);
      mbar_init(&str_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 8);
      mbar_init(&p_empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // --------------------------------------------------------------------------- producer
    bool ok = true;
    if (lane == 0) {
      mbar_expect_tx(own_full, 2 * C::kOwnBytes);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c) {
        tma_load_4d(so1 + c * kOwnBlock, &map_own1, own_full, c * 64, r0, hi, bi);
        tma_load_4d(so2 + c * kOwnBlock, &map_own2, own_full, c * 64, r0, hi, bi);
      }
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % C::kStages;
      const uint32_t ph = ((j / C::kStages) & 1u) ^ 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&str_empty[s], ph, abort_flag));
      if (!ok) break;
      if (!kDQ) {
        // the streamed rows are queries: stage their LSE (in log2 units) and delta next to the tiles
#pragma unroll
        for (int i = 0; i < kStr / 32; ++i) {
          const int col = i * 32 + lane;
          const int qi = j * kStr + col;
          const bool in = qi < p.sq;
          lse_s[s * kStr + col] = in ? p.lse[(int64_t)bh * p.sq + qi] * 1.4426950408889634f : INFINITY;
          del_s[s * kStr + col] = in ? p.delta[(int64_t)bh * p.sq + qi] : 0.f;
        }
        __syncwarp();
      }
      if (lane == 0) {
        mbar_expect_tx(&str_full[s], 2 * C::kStrBytes);
#pragma unroll
        for (int c = 0; c < C::kDBlocks; ++c) {
          tma_load_4d(ss1 + s * C::kStrBytes + c * kStrBlock, &map_str1, &str_full[s], c * 64, j * kStr, hi, bi);
          tma_load_4d(ss2 + s * C::kStrBytes + c * kStrBlock, &map_str2, &str_full[s], c * 64, j * kStr, hi, bi);
        }
      }
    }
    if (lane == 0) {
      if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutProducer);
      if (*abort_flag) {
        // copies already issued write into this CTA's shared memory: give them time to land
        for (uint32_t spin = 0; spin < (1u << 20); ++spin)
          if (mbar_try(own_full, 0)) break;
        for (int s = 0; s < C::kStages; ++s)
          for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
            if (mbar_try(&str_full[s], 0) || mbar_try(&str_full[s], 1)) break;
          }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = make_idesc(kOwn, kStr, 0, 0);
    constexpr uint32_t idesc_acc = make_idesc(kOwn, D, 0, 1);
    bool ok = mbar_wait(own_full, 0, abort_flag);
    tmem_fence_after();
    auto issue_s = [&](int j) -> bool {
      const int s = j % C::kStages;
      if (!mbar_wait(&str_full[s], (j / C::kStages) & 1u, abort_flag)) return false;
      tmem_fence_after();
      const uint32_t a1 = smem_u32(so1), a2 = smem_u32(so2);
      const uint32_t b1 = smem_u32(ss1 + s * C::kStrBytes), b2 = smem_u32(ss2 + s * C::kStrBytes);
      const uint32_t col = tmem_base + (uint32_t)(j & 1) * 2 * kStr;
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(col, make_desc(a1 + c * kOwnBlock + kk * 32, 16, 1024),
                    make_desc(b1 + c * kStrBlock + kk * 32, 16, 1024), idesc_s, (c | kk) ? 1u : 0u);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(col + kStr, make_desc(a2 + c * kOwnBlock + kk * 32, 16, 1024),
                    make_desc(b2 + c * kStrBlock + kk * 32, 16, 1024), idesc_s, (c | kk) ? 1u : 0u);
      umma_commit(&s_full[j & 1]);
      return true;
    };
    if (ok) ok = issue_s(0);
    if (ok && n_tiles > 1) ok = issue_s(1);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % C::kStages, b = j & 1;
      if (!mbar_wait(&p_full[b], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      tmem_fence_after();
      const uint32_t pa = smem_u32(sp + b * kPBytes), da = smem_u32(sds + b * kPBytes);
      const uint32_t b1 = smem_u32(ss1 + s * C::kStrBytes), b2 = smem_u32(ss2 + s * C::kStrBytes);
      if (!kDQ) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16(tmem_base + C::kAcc1Col, make_desc(pa + kk * 32, 16, 1024),
                    make_desc(b2 + kk * 2048, kStrBlock, 1024), idesc_acc, (j | kk) ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base + C::kAcc2Col, make_desc(da + kk * 32, 16, 1024),
                  make_desc(b1 + kk * 2048, kStrBlock, 1024), idesc_acc, (j | kk) ? 1u : 0u);
      umma_commit(&str_empty[s]);
      umma_commit(&p_empty[b]);
      // the elementwise warps have drained S'/dP' buffer b (they said so with p_full)
      if (j + 2 < n_tiles && !issue_s(j + 2)) { ok = false; break; }
    }
    if (ok) umma_commit(acc_full);
    if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutMma);
  } else if (warp >= 2) {
    // ----------------------------------------------------------------------- elementwise
    // Warp w may read TMEM lanes 32 (w % 4) .. +31, so two warps share every block of 32 owned
    // rows; they split the step's 64 columns in halves.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_local = quarter * 32 + lane;
    const int row = r0 + row_local;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t row_off = row_local * 128;
    const uint32_t swz = row_local & 7;
    float lse_row = INFINITY, del_row = 0.f;
    if (kDQ && row < p.sq) {
      lse_row = p.lse[(int64_t)bh * p.sq + row] * 1.4426950408889634f;
      del_row = p.delta[(int64_t)bh * p.sq + row];
    }
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1, s = j % C::kStages;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[b], (j >> 1) & 1u, abort_flag));
      if (!ok) break;
      if (!kDQ) {
        // acquire the producer's LSE / delta writes of this stage directly (already complete here)
        ok = __all_sync(0xffffffffu, mbar_wait(&str_full[s], (j / C::kStages) & 1u, abort_flag));
        if (!ok) break;
      }
      tmem_fence_after();
      uint32_t rs[32], rp[32];
      tmem_ld32(lane_base + b * 2 * kStr + half * 32, rs);
      tmem_ld32(lane_base + b * 2 * kStr + kStr + half * 32, rp);
      tmem_ld_wait();
      // the accumulating products of step j-2 must have finished reading P/dS buffer b
      ok = __all_sync(0xffffffffu, mbar_wait(&p_empty[b], ((j >> 1) & 1u) ^ 1u, abort_flag));
      if (!ok) break;
      const float4* lse_t = reinterpret_cast<const float4*>(lse_s + s * kStr + half * 32);
      const float4* del_t = reinterpret_cast<const float4*>(del_s + s * kStr + half * 32);
      // dQ pass: keys past the end read as zero rows, their probabilities must not count
      const int valid = kDQ ? min(kStr, p.s_str - j * kStr) - half * 32 : 32;
      const uint32_t p_row = smem_u32(sp + b * kPBytes) + row_off;
      const uint32_t d_row = smem_u32(sds + b * kPBytes) + row_off;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float pv[8], dv[8], lv[8], dl[8];
        if (kDQ) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { lv[i] = lse_row; dl[i] = del_row; }
        } else {
          const float4 l0 = lse_t[2 * g], l1 = lse_t[2 * g + 1], d0 = del_t[2 * g], d1 = del_t[2 * g + 1];
          lv[0] = l0.x; lv[1] = l0.y; lv[2] = l0.z; lv[3] = l0.w; lv[4] = l1.x; lv[5] = l1.y; lv[6] = l1.z; lv[7] = l1.w;
          dl[0] = d0.x; dl[1] = d0.y; dl[2] = d0.z; dl[3] = d0.w; dl[4] = d1.x; dl[5] = d1.y; dl[6] = d1.z; dl[7] = d1.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = g * 8 + i;
          pv[i] = exp2f(fmaf(__uint_as_float(rs[c]), p.scale_log2, -lv[i]));
          if (kDQ && c >= valid) pv[i] = 0.f;
          dv[i] = pv[i] * (__uint_as_float(rp[c]) - dl[i]);
        }
        const uint32_t chunk = (((uint32_t)(half * 4 + g)) ^ swz) << 4;
        if (!kDQ) {
          const bf16x8 pk = pack8(pv);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + chunk), "r"(pk.u.x),
                       "r"(pk.u.y), "r"(pk.u.z), "r"(pk.u.w)
                       : "memory");
        }
        const bf16x8 dk = pack8(dv);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d_row + chunk), "r"(dk.u.x),
                     "r"(dk.u.y), "r"(dk.u.z), "r"(dk.u.w)
                     : "memory");
      }
      fence_async_smem();
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, abort_flag));
    if (ok) {
      tmem_fence_after();
      constexpr int DH = D / 2;                    // output columns owned by this thread
      const int64_t dst_off = (((int64_t)bi * p.s_own + row) * p.heads + hi) * D + half * DH;
      if (!kDQ) {
        uint32_t q[DH];
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) tmem_ld32(lane_base + C::kAcc1Col + half * DH + c * 32, q + c * 32);
        tmem_ld_wait();
        if (row < p.s_own) {
#pragma unroll
          for (int g = 0; g < DH / 8; ++g) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(q[g * 8 + i]);
            *reinterpret_cast<bf16x8*>(p.out1 + dst_off + g * 8) = pack8(o);
          }
        }
      }
      {
        uint32_t q[DH];
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) tmem_ld32(lane_base + C::kAcc2Col + half * DH + c * 32, q + c * 32);
        tmem_ld_wait();
        if (row < p.s_own) {
#pragma unroll
          for (int g = 0; g < DH / 8; ++g) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(q[g * 8 + i]) * p.scale;
            *reinterpret_cast<bf16x8*>(p.out2 + dst_off + g * 8) = pack8(o);
          }
        }
      }
    }
    if (!ok && lane == 0) {
      if (atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutElementwise);
    }
  }

  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// delta[b, h, s] = sum_d dO[b, h, s, d] * O[b, h, s, d]; D / 8 lanes per row, 16-byte loads.
template <int D>
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                             float* __restrict__ delta, int64_t rows, int heads, int sq, int64_t do_sb,
                             int64_t do_sh, int64_t do_ss, int64_t o_sb, int64_t o_sh, int64_t o_ss) {
  constexpr int kLanes = D / 8;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r = gid / kLanes;
  const int part = (int)(gid % kLanes);
  float acc = 0.f;
  if (r < rows) {
    const int s = (int)(r % sq);
    const int64_t bhh = r / sq;
    const int h = (int)(bhh % heads);
    const int64_t b = bhh / heads;
    const bf16x8 a = *reinterpret_cast<const bf16x8*>(dout + b * do_sb + h * do_sh + s * do_ss + part * 8);
    const bf16x8 o = *reinterpret_cast<const bf16x8*>(out + b * o_sb + h * o_sh + s * o_ss + part * 8);
    float fa[8], fo[8];
    unpack8(a, fa);
    unpack8(o, fo);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(fa[i], fo[i], acc);
  }
#pragma unroll
  for (int off = kLanes / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (r < rows && part == 0) delta[r] = acc;
}

template <int D, bool kDQ>
static void launch(const CUtensorMap& o1, const CUtensorMap& o2, const CUtensorMap& s1, const CUtensorMap& s2,
                   const Params& p, int own_tiles, int bh, cudaStream_t stream) {
  static const bool attr_set = [] {
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_kernel<D, kDQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg<D>::kSmemBytes));
    return true;
  }();
  (void)attr_set;
  flash_bwd_kernel<D, kDQ><<<dim3(own_tiles, bh), kThreads, Cfg<D>::kSmemBytes, stream>>>(o1, o2, s1, s2, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <int D>
static void run(const torch::Tensor& dout, const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v,
                const torch::Tensor& out, const torch::Tensor& lse, torch::Tensor& delta, torch::Tensor& dq,
                torch::Tensor& dk, torch::Tensor& dv, double scale, cudaStream_t stream) {
  const int64_t b = q.size(0), h = q.size(1), sq = q.size(2), skv = k.size(2);
  {
    const int64_t rows = b * h * sq;
    const int64_t threads = rows * (D / 8);
    delta_kernel<D><<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()),
        reinterpret_cast<const __nv_bfloat16*>(out.data_ptr()), delta.data_ptr<float>(), rows, (int)h, (int)sq,
        dout.stride(0), dout.stride(1), dout.stride(2), out.stride(0), out.stride(1), out.stride(2));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  using attn::make_map4;
  Params p{};
  p.lse = lse.data_ptr<float>();
  p.delta = delta.data_ptr<float>();
  p.heads = (int)h;
  p.sq = (int)sq;
  p.scale = (float)scale;
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.status = attn::status_word(q.get_device());
  {
    // dK/dV: own K, V; stream Q, dO
    p.out1 = reinterpret_cast<__nv_bfloat16*>(dv.data_ptr());
    p.out2 = reinterpret_cast<__nv_bfloat16*>(dk.data_ptr());
    p.s_own = (int)skv;
    p.s_str = (int)sq;
    launch<D, false>(make_map4(k, kOwn), make_map4(v, kOwn), make_map4(q, kStr), make_map4(dout, kStr), p,
                     (int)((skv + kOwn - 1) / kOwn), (int)(b * h), stream);
  }
  {
    // dQ: own Q, dO; stream K, V
    p.out1 = nullptr;
    p.out2 = reinterpret_cast<__nv_bfloat16*>(dq.data_ptr());
    p.s_own = (int)sq;
    p.s_str = (int)skv;
    launch<D, true>(make_map4(q, kOwn), make_map4(dout, kOwn), make_map4(k, kStr), make_map4(v, kStr), p,
                    (int)((sq + kOwn - 1) / kOwn), (int)(b * h), stream);
  }
}

}  // namespace attn_bwd

// Gradients of softmax(scale * Q K^T) V for [B, H, S, D] bf16 views (any strides the 4-D tensor map
// can describe, unit stride in D).  `out` and `lse` are what flash_attn_fwd returned.  The three
// gradients are token-major [B, S, H, D] buffers returned as [B, H, S, D] views.
std::vector<torch::Tensor> flash_attn_bwd(torch::Tensor dout, torch::Tensor q, torch::Tensor k, torch::Tensor v,
                                          torch::Tensor out, torch::Tensor lse, double scale) {
  using namespace attn;
  TORCH_CHECK(q.is_cuda() && q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && dout.dim() == 4 && out.dim() == 4,
              "flash_attn_bwd: [B, H, S, D]");
  for (const auto& t : {dout, q, k, v, out}) TORCH_CHECK(t.scalar_type() == torch::kBFloat16, "flash_attn_bwd: bf16");
  const int64_t b = q.size(0), h = q.size(1), sq = q.size(2), d = q.size(3), skv = k.size(2);
  TORCH_CHECK(d == 64 || d == 128, "flash_attn_bwd: head dimension 64 or 128");
  TORCH_CHECK(k.size(0) == b && k.size(1) == h && k.size(3) == d && v.sizes() == k.sizes());
  TORCH_CHECK(dout.sizes() == q.sizes() && out.sizes() == q.sizes());
  TORCH_CHECK(lse.scalar_type() == torch::kFloat32 && lse.is_contiguous() && lse.numel() == b * h * sq);
  TORCH_CHECK(b * h <= 65535, "flash_attn_bwd: batch * heads exceeds the grid limit");
  q = mappable(q);
  k = mappable(k);
  v = mappable(v);
  dout = mappable(dout);
  out = mappable(out);
  const c10::cuda::CUDAGuard guard(q.device());
  bind_context();
  auto dq_tm = torch::empty({b, sq, h, d}, q.options());
  auto dk_tm = torch::empty({b, skv, h, d}, q.options());
  auto dv_tm = torch::empty({b, skv, h, d}, q.options());
  std::vector<torch::Tensor> grads = {dq_tm.transpose(1, 2), dk_tm.transpose(1, 2), dv_tm.transpose(1, 2)};
  if (b * h == 0 || sq == 0 || skv == 0) {
    for (auto& g : grads) g.zero_();
    return grads;
  }
  auto delta = torch::empty({b, h, sq}, lse.options());
  auto stream = at::cuda::getCurrentCUDAStream();
  if (d == 64) attn_bwd::run<64>(dout, q, k, v, out, lse, delta, dq_tm, dk_tm, dv_tm, scale, stream);
  else attn_bwd::run<128>(dout, q, k, v, out, lse, delta, dq_tm, dk_tm, dv_tm, scale, stream);
  return grads;
}

}  // namespace vrl
