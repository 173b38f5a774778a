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
//   P   = exp2(S' * scale * log2e - LSE * log2e),  dS = P * (dP' - delta)   in registers, then as
//                                  bf16 pairs back into TMEM over the columns S' and dP' came from
//   acc1 += P  . str2              (dV += P^T dO)            dK/dV pass only, A operand from TMEM
//   acc2 += dS . str1              (dK += dS^T Q  |  dQ += dS K)           A operand from TMEM
// where delta = rowsum(dO * O) per query comes from a small pre-pass.  The streamed tiles are read
// twice from the same shared-memory copy: K-major for the first two products, MN-major for the
// accumulating ones.  Keeping P and dS out of shared memory matters: every tcgen05.mma with a
// shared-memory A operand re-reads 4 KB of it, and that traffic, not the math, bounds small tiles.
//
//   warp 0      producer: own tiles once, then streamed tiles (and, in the dK/dV pass, the
//               queries' LSE and delta) through a ring
//   warp 1      MMA issuer A (S', dP') and TMEM owner; S'/dP' are double-buffered so that the
//               tensor core works on step j+1 while the other warps handle step j
//   warp 2      MMA issuer B (the accumulating products); warp 3 idles
//   warps 4..11 elementwise: two threads per owned row, 32 of the step's 64 columns each; no
//               reductions across threads are needed in the backward
// TMEM columns: [S'0 dP'0 S'1 dP'1] (64 each), acc1 (D), acc2 (D), and for D = 64 [P0 dS0 P1 dS1]
// (32 each).  Every wait is bounded; on
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
constexpr int kEwWarps = 8;                // elementwise warps: two threads per owned row
constexpr int kFirstEw = 4;                // warps 0..3: producer, two MMA issuers, one idle
constexpr int kThreads = 32 * (kFirstEw + kEwWarps);
constexpr uint32_t kOwnBlock = kOwn * 128;       // one 64-column swizzle block of an owned tile
constexpr uint32_t kStrBlock = kStr * 128;       // the same for a streamed tile

enum Status : int { kOk = 0, kTimeoutProducer = 21, kTimeoutMma = 22, kTimeoutElementwise = 23,
                    kMisalignedSmem = 24 };

template <int D>
struct Cfg {
  static constexpr int kDBlocks = D / 64;
  static constexpr int kStages = D == 64 ? 8 : 5;      // streamed-tile ring (fills the shared memory)
  static constexpr uint32_t kOwnBytes = kDBlocks * kOwnBlock;
  static constexpr uint32_t kStrBytes = kDBlocks * kStrBlock;
  static constexpr uint32_t kVecBytes = kStages * kStr * 4;          // LSE or delta of the staged queries
  static constexpr uint32_t kSmemBytes =
      2 * kOwnBytes + 2 * kStages * kStrBytes + 2 * kVecBytes + 256;
  static constexpr uint32_t kAcc1Col = 4 * kStr;
  static constexpr uint32_t kAcc2Col = 4 * kStr + D;
  static constexpr uint32_t kTmemCols = 512;
  // Where P and dS (bf16 pairs, 32 columns each per buffer) live in TMEM.  D = 64 leaves 128 spare
  // columns for two separate buffers; D = 128 does not, so there they overwrite the S'/dP' columns
  // they were computed from (each thread its own 32), and S' of step j+2 has to wait for the
  // accumulating products of step j.
  static constexpr bool kAliasP = 2 * D + 6 * kStr > 512;
  static constexpr uint32_t kPCol = 4 * kStr + 2 * D;
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
  unsigned long long* timing;   // optional [16] phase cycle counters (see flash_attn_bwd_timing), or null
  int causal;             // query row r attends keys 0 .. r + causal_off
  int causal_off;         // Skv - Sq
};

// Adds the cycles since `t0` to counter `slot` and restarts the interval.
__device__ __forceinline__ void lap(const Params& p, int slot, long long& t0) {
  if (p.timing != nullptr) {
    const long long t1 = clock64();
    atomicAdd(p.timing + slot, (unsigned long long)(t1 - t0));
    t0 = clock64();
  }
}

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
  float* lse_s = reinterpret_cast<float*>(ss2 + C::kStages * C::kStrBytes);   // [kStages][kStr], times log2(e)
  float* del_s = lse_s + C::kStages * kStr;                        // [kStages][kStr]
  uint64_t* bars = reinterpret_cast<uint64_t*>(del_s + C::kStages * kStr);
  uint64_t* own_full = bars;
  uint64_t* str_full = bars + 1;                   // [kStages]
  uint64_t* str_empty = str_full + C::kStages;     // [kStages]
  uint64_t* s_full = str_empty + C::kStages;       // [2] S' of a step is in TMEM
  uint64_t* d_full = s_full + 2;                   // [2] dP' of a step is in TMEM
  uint64_t* p_full = d_full + 2;                   // [2]
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
  // Streamed steps this CTA has to visit.  Causal attention skips the steps that lie entirely above
  // the diagonal: the dQ pass (owned queries, streamed keys) stops after the last key its rows can
  // see; the dK/dV pass (owned keys, streamed queries) starts at the first query that sees its keys.
  // `j_lo` is the first streamed step; loop counters keep running from 0 so stage / parity
  // arithmetic is unchanged.
  int n_tiles = (p.s_str + kStr - 1) / kStr;
  int j_lo = 0;
  if (p.causal) {
    if (kDQ) {
      const int last_key = min(r0 + kOwn, p.s_own) - 1 + p.causal_off;
      n_tiles = max(1, min(n_tiles, last_key / kStr + 1));
    } else {
      j_lo = min(max(0, (r0 - p.causal_off) / kStr), n_tiles - 1);
      n_tiles -= j_lo;
    }
  }

  if (threadIdx.x == 0) {
    mbar_init(own_full, 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&str_full[s], 1);
      mbar_init(&str_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&d_full[s], 1);
      mbar_init(&p_full[s], kEwWarps);
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
    long long t0 = clock64();
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
      // the streamed rows are queries: fetch their LSE (to log2 units) and delta while waiting for
      // the stage, then put them next to the tiles
      float vl[kStr / 32], vd[kStr / 32];
      if (!kDQ) {
#pragma unroll
        for (int i = 0; i < kStr / 32; ++i) {
          const int qi = (j + j_lo) * kStr + i * 32 + lane;
          const bool in = qi < p.sq;
          vl[i] = in ? p.lse[(int64_t)bh * p.sq + qi] * 1.4426950408889634f : INFINITY;
          vd[i] = in ? p.delta[(int64_t)bh * p.sq + qi] : 0.f;
        }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(&str_empty[s], ph, abort_flag));
      if (!ok) break;
      if (lane == 0) lap(p, 12, t0);
      if (!kDQ) {
#pragma unroll
        for (int i = 0; i < kStr / 32; ++i) {
          lse_s[s * kStr + i * 32 + lane] = vl[i];
          del_s[s * kStr + i * 32 + lane] = vd[i];
        }
        __syncwarp();
      }
      if (lane == 0) lap(p, 13, t0);
      if (lane == 0) {
        mbar_expect_tx(&str_full[s], 2 * C::kStrBytes);
#pragma unroll
        for (int c = 0; c < C::kDBlocks; ++c) {
          tma_load_4d(ss1 + s * C::kStrBytes + c * kStrBlock, &map_str1, &str_full[s], c * 64, (j + j_lo) * kStr, hi, bi);
          tma_load_4d(ss2 + s * C::kStrBytes + c * kStrBlock, &map_str2, &str_full[s], c * 64, (j + j_lo) * kStr, hi, bi);
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
    // ------------------------------------------------- MMA issuer A: S' and dP' of every step
    // One tcgen05.mma costs its issuing thread about 48 cycles, a commit about 100 and an mbarrier
    // wait 100 or more even when it is already complete, so a single thread issuing all four
    // products of a step is the bottleneck of the CTA.  Two threads share the work: this one the
    // products that feed the elementwise warps, warp 2 the accumulating ones.
    constexpr uint32_t idesc_s = make_idesc(kOwn, kStr, 0, 0);
    constexpr uint32_t hi = desc_hi(1024);
    long long t0 = clock64();
    const long long t_begin = t0;
    bool ok = mbar_wait(own_full, 0, abort_flag);
    lap(p, 2, t0);
    const uint32_t a1_lo = desc_lo(smem_u32(so1), 16), a2_lo = desc_lo(smem_u32(so2), 16);
    const uint32_t b1_lo = desc_lo(smem_u32(ss1), 16), b2_lo = desc_lo(smem_u32(ss2), 16);
    auto issue_s = [&](int j) -> bool {
      const int s = j % C::kStages;
      lap(p, 15, t0);
      if (!mbar_wait(&str_full[s], (j / C::kStages) & 1u, abort_flag)) return false;
      lap(p, 3, t0);
      const uint32_t stage = (uint32_t)s * (C::kStrBytes >> 4);
      const uint32_t col = tmem_base + (uint32_t)(j & 1) * 2 * kStr;
      // S' first and signalled on its own: the elementwise warps start on the exponentials while
      // the tensor core still works on dP'
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_split(col, a1_lo + ((c * kOwnBlock + kk * 32) >> 4), hi,
                          b1_lo + stage + ((c * kStrBlock + kk * 32) >> 4), hi, idesc_s, (c | kk) ? 1u : 0u);
      umma_commit(&s_full[j & 1]);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_split(col + kStr, a2_lo + ((c * kOwnBlock + kk * 32) >> 4), hi,
                          b2_lo + stage + ((c * kStrBlock + kk * 32) >> 4), hi, idesc_s, (c | kk) ? 1u : 0u);
      umma_commit(&d_full[j & 1]);
      return true;
    };
    if (ok) ok = issue_s(0);
    if (ok && n_tiles > 1) ok = issue_s(1);
    for (int j = 0; j + 2 < n_tiles && ok; ++j) {
      const int b = j & 1;
      lap(p, 15, t0);
      // S'/dP' buffer b is free once the elementwise warps have read step j out of it ...
      if (!mbar_wait(&p_full[b], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      // ... and, where P and dS were written back over it, once step j's accumulating products
      // have consumed them
      if (C::kAliasP && !mbar_wait(&p_empty[b], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      lap(p, 4, t0);
      tmem_fence_after();
      if (!issue_s(j + 2)) { ok = false; break; }
    }
    if (p.timing != nullptr) {
      atomicAdd(p.timing + 0, 1ull);
      atomicAdd(p.timing + 1, (unsigned long long)(clock64() - t_begin));
      atomicAdd(p.timing + 14, (unsigned long long)n_tiles);
    }
    if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutMma);
  } else if (warp == 2 && lane == 0) {
    // ------------------------------------------ MMA issuer B: the accumulating products
    constexpr uint32_t idesc_acc = make_idesc(kOwn, D, 0, 1);
    constexpr uint32_t hi = desc_hi(1024);
    const uint32_t b1_mn = desc_lo(smem_u32(ss1), kStrBlock), b2_mn = desc_lo(smem_u32(ss2), kStrBlock);
    long long t0 = clock64();
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % C::kStages, b = j & 1;
      if (!mbar_wait(&p_full[b], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      // the streamed tiles of this step landed long ago; this acquires them for this thread
      if (!mbar_wait(&str_full[s], (j / C::kStages) & 1u, abort_flag)) { ok = false; break; }
      lap(p, 7, t0);
      tmem_fence_after();
      const uint32_t stage = (uint32_t)s * (C::kStrBytes >> 4);
      const uint32_t first = j ? 1u : 0u;
      // 16 values of k-step kk = 8 packed columns
      const uint32_t pcol = C::kAliasP ? tmem_base + (uint32_t)b * 2 * kStr : tmem_base + C::kPCol + (uint32_t)b * kStr;
      const uint32_t dcol = C::kAliasP ? pcol + kStr : pcol + kStr / 2;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint32_t koff = C::kAliasP ? (kk >> 1) * 32 + (kk & 1) * 8 : kk * 8;
        if (!kDQ)
          umma_bf16_tmem_a(tmem_base + C::kAcc1Col, pcol + koff, b2_mn + stage + ((kk * 2048) >> 4), hi, idesc_acc,
                           kk ? 1u : first);
        umma_bf16_tmem_a(tmem_base + C::kAcc2Col, dcol + koff, b1_mn + stage + ((kk * 2048) >> 4), hi, idesc_acc,
                         kk ? 1u : first);
      }
      umma_commit(&str_empty[s]);
      umma_commit(&p_empty[b]);
      lap(p, 10, t0);
    }
    if (ok) umma_commit(acc_full);
    if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutMma);
  } else if (warp >= kFirstEw) {
    // ----------------------------------------------------------------------- elementwise
    // Warp w may read TMEM lanes 32 (w % 4) .. +31, so two warps share every block of 32 owned
    // rows; they split the step's 64 columns (and the output columns) evenly.
    constexpr int kParts = kEwWarps / 4;
    static_assert(kStr / kParts == 32, "the TMEM store below moves 16 packed columns per thread");
    constexpr int CPT = kStr / kParts;            // columns of a step per thread
    const int quarter = warp & 3;
    const int half = (warp - kFirstEw) >> 2;      // which part of the columns
    const int row_local = quarter * 32 + lane;
    const int row = r0 + row_local;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float lse_row = INFINITY, del_row = 0.f;
    if (kDQ && row < p.sq) {
      lse_row = p.lse[(int64_t)bh * p.sq + row] * 1.4426950408889634f;
      del_row = p.delta[(int64_t)bh * p.sq + row];
    }
    bool ok = true;
    const bool timed = warp == kFirstEw && lane == 0;
    long long t0 = clock64();
    for (int j = 0; j < n_tiles; ++j) {
      const int b = j & 1, s = j % C::kStages;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[b], (j >> 1) & 1u, abort_flag));
      if (!ok) break;
      if (timed) lap(p, 5, t0);
      if (!kDQ) {
        // acquire the producer's LSE / delta writes of this stage directly (already complete here)
        ok = __all_sync(0xffffffffu, mbar_wait(&str_full[s], (j / C::kStages) & 1u, abort_flag));
        if (!ok) break;
      }
      tmem_fence_after();
      uint32_t rs[CPT];
      tmem_ld_cols<CPT>(lane_base + b * 2 * kStr + half * CPT, rs);
      tmem_ld_wait();
      if (timed) lap(p, 6, t0);
      const float4* lse_t = reinterpret_cast<const float4*>(lse_s + s * kStr + half * CPT);
      const float4* del_t = reinterpret_cast<const float4*>(del_s + s * kStr + half * CPT);
      // dQ pass: keys past the end read as zero rows, their probabilities must not count
      const int valid = kDQ ? min(kStr, p.s_str - j * kStr) - half * CPT : CPT;
      float pv[CPT];
      uint32_t pk[CPT / 2], dk[CPT / 2];             // bf16 pairs
#pragma unroll
      for (int g = 0; g < CPT / 4; ++g) {
        float4 l4 = make_float4(lse_row, lse_row, lse_row, lse_row);
        if (!kDQ) l4 = lse_t[g];
        pv[4 * g + 0] = exp2f(fmaf(__uint_as_float(rs[4 * g + 0]), p.scale_log2, -l4.x));
        pv[4 * g + 1] = exp2f(fmaf(__uint_as_float(rs[4 * g + 1]), p.scale_log2, -l4.y));
        pv[4 * g + 2] = exp2f(fmaf(__uint_as_float(rs[4 * g + 2]), p.scale_log2, -l4.z));
        pv[4 * g + 3] = exp2f(fmaf(__uint_as_float(rs[4 * g + 3]), p.scale_log2, -l4.w));
      }
      if (kDQ && valid < CPT) {                    // only the last step of a ragged sequence
#pragma unroll
        for (int c = 0; c < CPT; ++c)
          if (c >= valid) pv[c] = 0.f;
      }
      if (p.causal) {
        // column c of this thread is streamed index s0 + c; the pair (query, key) is masked when
        // key > query + causal_off
        const int s0 = (j + j_lo) * kStr + half * CPT;
        if (kDQ) {
          const int seen = row + p.causal_off - s0 + 1;          // keys s0 .. s0 + seen - 1 are visible
          if (seen < CPT) {
#pragma unroll
            for (int c = 0; c < CPT; ++c)
              if (c >= seen) pv[c] = 0.f;
          }
        } else {
          const int hidden = row - p.causal_off - s0;            // queries s0 .. s0 + hidden - 1 cannot see key `row`
          if (hidden > 0) {
#pragma unroll
            for (int c = 0; c < CPT; ++c)
              if (c < hidden) pv[c] = 0.f;
          }
        }
      }
      if (!kDQ) {
#pragma unroll
        for (int c = 0; c < CPT / 2; ++c) pk[c] = float2_to_bf16pair(pv[2 * c], pv[2 * c + 1]);
      }
      // now dP' (the tensor core produced it while the exponentials ran)
      ok = __all_sync(0xffffffffu, mbar_wait(&d_full[b], (j >> 1) & 1u, abort_flag));
      if (!ok) break;
      tmem_fence_after();
      tmem_ld_cols<CPT>(lane_base + b * 2 * kStr + kStr + half * CPT, rs);
      tmem_ld_wait();
#pragma unroll
      for (int g = 0; g < CPT / 4; ++g) {
        float4 d4 = make_float4(del_row, del_row, del_row, del_row);
        if (!kDQ) d4 = del_t[g];
        const float d0 = pv[4 * g + 0] * (__uint_as_float(rs[4 * g + 0]) - d4.x);
        const float d1 = pv[4 * g + 1] * (__uint_as_float(rs[4 * g + 1]) - d4.y);
        const float d2 = pv[4 * g + 2] * (__uint_as_float(rs[4 * g + 2]) - d4.z);
        const float d3 = pv[4 * g + 3] * (__uint_as_float(rs[4 * g + 3]) - d4.w);
        dk[2 * g] = float2_to_bf16pair(d0, d1);
        dk[2 * g + 1] = float2_to_bf16pair(d2, d3);
      }
      if (C::kAliasP) {
        // over this thread's own, already consumed, S' and dP' columns
        if (!kDQ) tmem_st16(lane_base + b * 2 * kStr + half * CPT, pk);
        tmem_st16(lane_base + b * 2 * kStr + kStr + half * CPT, dk);
      } else {
        // separate P/dS buffer b: the accumulating products of step j-2 must be done with it
        ok = __all_sync(0xffffffffu, mbar_wait(&p_empty[b], ((j >> 1) & 1u) ^ 1u, abort_flag));
        if (!ok) break;
        if (!kDQ) tmem_st16(lane_base + C::kPCol + b * kStr + half * (CPT / 2), pk);
        tmem_st16(lane_base + C::kPCol + b * kStr + kStr / 2 + half * (CPT / 2), dk);
      }
      tmem_st_wait();
      if (timed) lap(p, 8, t0);
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
      if (timed) lap(p, 9, t0);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, abort_flag));
    if (ok) {
      tmem_fence_after();
      constexpr int DH = D / kParts;               // output columns owned by this thread
      const int64_t dst_off = (((int64_t)bi * p.s_own + row) * p.heads + hi) * D + half * DH;
      if (!kDQ) {
        uint32_t q[DH];
        tmem_ld_cols<DH>(lane_base + C::kAcc1Col + half * DH, q);
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
        tmem_ld_cols<DH>(lane_base + C::kAcc2Col + half * DH, q);
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
    if (timed) lap(p, 11, t0);
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

// Phase counters of the next backward calls on this device ([2 passes][16] cycles), or null when off.
static unsigned long long* g_timing = nullptr;

template <int D>
static void run(const torch::Tensor& dout, const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v,
                const torch::Tensor& out, const torch::Tensor& lse, torch::Tensor& delta, torch::Tensor& dq,
                torch::Tensor& dk, torch::Tensor& dv, double scale, bool causal, cudaStream_t stream) {
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
  p.timing = g_timing;
  p.causal = causal ? 1 : 0;
  p.causal_off = (int)(skv - sq);
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
    if (g_timing != nullptr) p.timing = g_timing + 16;
    launch<D, true>(make_map4(q, kOwn), make_map4(dout, kOwn), make_map4(k, kStr), make_map4(v, kStr), p,
                    (int)((sq + kOwn - 1) / kOwn), (int)(b * h), stream);
  }
}

}  // namespace attn_bwd

// Developer aid: switch per-phase cycle counters of the backward kernels on (zeroing them) or off, and
// read them back as a [2, 16] int64 tensor (row 0 the dK/dV pass, row 1 the dQ pass).  Slots: 0 CTAs,
// 1 CTA cycles, 2 MMA wait own tiles, 3 MMA wait streamed tiles, 4 MMA wait P/dS, 5 elementwise wait
// S'/dP', 6 TMEM load, 7 issuer B waits, 8 compute + TMEM stores, 9 fence + arrive, 10 issuer B issue (and elementwise wait for the
// accumulators), 11 epilogue, 12 producer wait free stage, 13 producer LSE/delta staging, 14 steps,
// 15 MMA issue.  Elementwise slots are measured on one thread per CTA.
torch::Tensor flash_attn_bwd_timing(bool enable) {
  using attn_bwd::g_timing;
  auto out = torch::zeros({2, 16}, torch::dtype(torch::kInt64));
  if (g_timing != nullptr) {
    C10_CUDA_CHECK(cudaDeviceSynchronize());
    C10_CUDA_CHECK(cudaMemcpy(out.data_ptr(), g_timing, 32 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  }
  if (enable) {
    if (g_timing == nullptr) C10_CUDA_CHECK(cudaMalloc(&g_timing, 32 * sizeof(unsigned long long)));
    C10_CUDA_CHECK(cudaMemset(g_timing, 0, 32 * sizeof(unsigned long long)));
  } else if (g_timing != nullptr) {
    C10_CUDA_CHECK(cudaFree(g_timing));
    g_timing = nullptr;
  }
  return out;
}

// Gradients of softmax(scale * Q K^T) V for [B, H, S, D] bf16 views (any strides the 4-D tensor map
// can describe, unit stride in D).  `out` and `lse` are what flash_attn_fwd returned.  The three
// gradients are token-major [B, S, H, D] buffers returned as [B, H, S, D] views.
std::vector<torch::Tensor> flash_attn_bwd(torch::Tensor dout, torch::Tensor q, torch::Tensor k, torch::Tensor v,
                                          torch::Tensor out, torch::Tensor lse, double scale, bool causal) {
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
  VRL_CHECK_OPERAND(dout, q);
  VRL_CHECK_OPERAND(k, q);
  VRL_CHECK_OPERAND(v, q);
  VRL_CHECK_OPERAND(out, q);
  VRL_CHECK_OPERAND(lse, q);
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
  TORCH_CHECK(!causal || sq <= skv, "flash_attn_bwd: causal attention needs Sq <= Skv");
  if (d == 64) attn_bwd::run<64>(dout, q, k, v, out, lse, delta, dq_tm, dk_tm, dv_tm, scale, causal, stream);
  else attn_bwd::run<128>(dout, q, k, v, out, lse, delta, dq_tm, dk_tm, dv_tm, scale, causal, stream);
  return grads;
}

}  // namespace vrl
