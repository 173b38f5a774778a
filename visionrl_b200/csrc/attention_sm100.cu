// Bidirectional flash attention forward for sm_100a: S = Q K^T and O += P V on tcgen05.mma with
// both accumulators in tensor memory, operands staged by TMA, online softmax in registers.
//
// One CTA owns 128 query rows of one (batch, head) and walks the keys in tiles of 128.
//   warp 0      TMA producer: Q once, then K and V tiles through two-stage rings
//   warp 1      MMA issuer and TMEM owner: S[j+1] = Q K[j+1]^T is issued before P[j] V[j], so the
//               tensor core works on the next score tile while the softmax warps handle this one
//   warps 2..9  softmax: two threads per query row, each owning 64 of the tile's 128 scores and
//               half of the output columns.  Scores are read from TMEM once, probabilities are
//               written as bf16 into a 128-byte-swizzled shared tile that is the A operand of P V;
//               the running output lives in registers and absorbs each P V partial product from
//               TMEM with the usual rescale.
// TMEM columns: S0, S1 (128 each), then O0, O1 (D each); one CTA per SM.  Every wait is bounded; on
// expiry the
// role records a status code, raises the CTA's abort flag and all roles fall through to the
// common exit where the TMEM is released.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cudaTypedefs.h>

#include <map>
#include <mutex>

#include "attn_host.cuh"
#include "common.cuh"
#include "ops.h"
#include "sm100_ptx.cuh"

namespace vrl {
namespace attn {

using namespace ptx;

constexpr int kTile = 128;                 // query rows per CTA and keys per step
constexpr int kThreads = 320;              // TMA warp, MMA warp, 8 softmax warps
constexpr uint32_t kBlockBytes = kTile * 128;   // one 64-column swizzle block of a 128-row tile
constexpr uint32_t kPBytes = 2 * kBlockBytes;

enum Status : int { kOk = 0, kTimeoutProducer = 11, kTimeoutMma = 12, kTimeoutSoftmax = 13,
                    kMisalignedSmem = 14 };

template <int D>
struct Cfg {
  static constexpr int kDBlocks = D / 64;
  static constexpr uint32_t kTileBytes = kDBlocks * kBlockBytes;      // Q, K or V tile
  static constexpr uint32_t kXchBytes = 12 * kTile * 4;               // max/tag [2][2][128], sum/tag [2][128]
  static constexpr uint32_t kSmemBytes = 5 * kTileBytes + kPBytes + kXchBytes + 256;
  static constexpr int kSBufs = 2;                                    // score buffers in TMEM
  static constexpr uint32_t kOCol = kSBufs * kTile;                   // first O column in TMEM
  static constexpr uint32_t kTmemCols = 512;                          // S0 S1 O0 O1 (power of two)
  static constexpr int kCtasPerSm = 1;
};

struct Params {
  __nv_bfloat16* out;     // token-major [B, Sq, H, D]
  float* lse;             // [B, H, Sq] natural-log sum of exponentials of the scaled scores
  int heads;
  int* status;
  int sq, skv;
  float scale_log2;       // softmax scale times log2(e)
  int causal;             // query row r attends keys 0 .. r + (skv - sq) (lazy-rescale kernel only)
  // Sequence-parallel output (sp_world > 1): this rank computed `heads` local heads over the FULL
  // sequence; query row r belongs to rank r / sp_sloc, whose [B, sp_sloc, sp_heads_total, D] buffer
  // (peer-mapped address out_peer[r / sp_sloc]) receives it at head offset sp_head0 — the
  // heads -> sequence exchange of Ulysses happens in the epilogue's stores.
  __nv_bfloat16* out_peer[16];
  int sp_world, sp_sloc, sp_heads_total, sp_head0;
};

// Address of the D output values of (batch bi, query row, local head hi).
template <int D>
__device__ __forceinline__ __nv_bfloat16* out_row(const Params& p, int bi, int row, int hi) {
  if (p.sp_world > 1) {
    const int owner = row / p.sp_sloc, local = row - owner * p.sp_sloc;
    return p.out_peer[owner] + (((int64_t)bi * p.sp_sloc + local) * p.sp_heads_total + p.sp_head0 + hi) * D;
  }
  return p.out + (((int64_t)bi * p.sq + row) * p.heads + hi) * D;
}

// Publish `mine` in slot `me` with tag `tag`, then read the partner's value once its slot carries the
// same tag.  Bounded: returns false when the partner does not show up.
__device__ __forceinline__ bool exchange(float* vals, int* tags, int me, int partner, float mine, int tag,
                                         float& theirs, volatile int* abort_flag) {
  volatile float* v = vals;
  volatile int* t = tags;
  v[me] = mine;
  __threadfence_block();
  t[me] = tag;
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (t[partner] == tag) {
      __threadfence_block();
      theirs = v[partner];
      return true;
    }
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}

template <int D>
__global__ void __launch_bounds__(kThreads, Cfg<D>::kCtasPerSm)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const Params p) {
  using C = Cfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {          // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(p.status, kMisalignedSmem);
    return;
  }
  uint8_t* sq = smem;
  uint8_t* sk = sq + C::kTileBytes;            // [2]
  uint8_t* sv = sk + 2 * C::kTileBytes;        // [2]
  uint8_t* sp = sv + 2 * C::kTileBytes;
  float* xmax = reinterpret_cast<float*>(sp + kPBytes);          // [2 parities][2 halves][128]
  int* xtag = reinterpret_cast<int*>(xmax + 4 * kTile);          // tile number + 1 of each xmax slot
  float* xsum = reinterpret_cast<float*>(xtag + 4 * kTile);      // [2 halves][128]
  int* xsum_tag = reinterpret_cast<int*>(xsum + 2 * kTile);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sp + kPBytes + C::kXchBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* k_empty = bars + 3;    // [2]
  uint64_t* v_full = bars + 5;     // [2]
  uint64_t* v_empty = bars + 7;    // [2] spare: the V stage is released through o_full
  uint64_t* s_full = bars + 9;     // [2]
  uint64_t* o_full = bars + 11;    // [2]
  uint64_t* p_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, q0 = blockIdx.x * kTile;
  const int bi = bh / p.heads, hi = bh % p.heads;
  const int n_tiles = (p.skv + kTile - 1) / kTile;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&o_full[s], 1);
    }
    mbar_init(p_full, 8);
    *abort_flag = 0;
    mbar_fence_init();
    fence_async_smem();
  }
  for (int i = threadIdx.x; i < 4 * kTile; i += kThreads) xtag[i] = 0;
  for (int i = threadIdx.x; i < 2 * kTile; i += kThreads) xsum_tag[i] = 0;
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ----------------------------------------------------------------------- TMA producer
    bool ok = true;
    mbar_expect_tx(q_full, C::kTileBytes);
#pragma unroll
    for (int c = 0; c < C::kDBlocks; ++c) tma_load_4d(sq + c * kBlockBytes, &map_q, q_full, c * 64, q0, hi, bi);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = ((j >> 1) & 1u) ^ 1u;
      if (!mbar_wait(&k_empty[s], ph, abort_flag)) { ok = false; break; }
      mbar_expect_tx(&k_full[s], C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
        tma_load_4d(sk + s * C::kTileBytes + c * kBlockBytes, &map_k, &k_full[s], c * 64, j * kTile, hi, bi);
      if (!mbar_wait(&o_full[s], ph, abort_flag)) { ok = false; break; }     // P V of step j-2 done
      mbar_expect_tx(&v_full[s], C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
        tma_load_4d(sv + s * C::kTileBytes + c * kBlockBytes, &map_v, &v_full[s], c * 64, j * kTile, hi, bi);
    }
    if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutProducer);
    if (*abort_flag) {
      // copies already issued write into this CTA's shared memory: give them time to land
      for (uint32_t spin = 0; spin < (1u << 20); ++spin)
        if (mbar_try(q_full, 0)) break;
      for (int s = 0; s < 2; ++s)
        for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
          if (mbar_try(&k_full[s], 0) || mbar_try(&k_full[s], 1)) break;
        }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_qk = make_idesc(kTile, kTile, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(kTile, D, 0, 1);
    // operand descriptors: constant high half, low half = base + (byte offset >> 4)
    constexpr uint32_t hi = desc_hi(1024);
    const uint32_t q_lo = desc_lo(smem_u32(sq), 16), k_lo = desc_lo(smem_u32(sk), 16);
    const uint32_t p_lo = desc_lo(smem_u32(sp), 16), v_lo = desc_lo(smem_u32(sv), kBlockBytes);
    bool ok = mbar_wait(q_full, 0, abort_flag);
    tmem_fence_after();
    auto issue_qk = [&](int j) -> bool {
      const int s = j & 1;
      const int sbuf = j % C::kSBufs;
      if (!mbar_wait(&k_full[s], (j >> 1) & 1u, abort_flag)) return false;
      tmem_fence_after();
      const uint32_t stage = (uint32_t)s * (C::kTileBytes >> 4);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_split(tmem_base + sbuf * kTile, q_lo + ((c * kBlockBytes + kk * 32) >> 4), hi,
                          k_lo + stage + ((c * kBlockBytes + kk * 32) >> 4), hi, idesc_qk, (c | kk) ? 1u : 0u);
      umma_commit(&k_empty[s]);
      umma_commit(&s_full[sbuf]);
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      // with two score buffers the next Q K^T runs while the softmax warps work on this tile;
      // with one it has to wait until they have consumed the scores (signalled with P)
      if (C::kSBufs == 2 && j + 1 < n_tiles && !issue_qk(j + 1)) { ok = false; break; }
      if (!mbar_wait(p_full, j & 1u, abort_flag)) { ok = false; break; }
      if (C::kSBufs == 1 && j + 1 < n_tiles && !issue_qk(j + 1)) { ok = false; break; }
      const int s = j & 1;
      if (!mbar_wait(&v_full[s], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      tmem_fence_after();
      const uint32_t vstage = (uint32_t)s * (C::kTileBytes >> 4);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16_split(tmem_base + C::kOCol + s * D, p_lo + (((kk >> 2) * kBlockBytes + (kk & 3) * 32) >> 4), hi,
                        v_lo + vstage + ((kk * 2048) >> 4), hi, idesc_pv, kk ? 1u : 0u);
      // one commit serves both readers of "P V of this step is done": the softmax warps (partial
      // output ready) and the producer (V stage free); a commit costs the issuing thread ~100 cycles
      umma_commit(&o_full[s]);
    }
    if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutMma);
  } else if (warp >= 2) {
    // --------------------------------------------------------------------------- softmax
    // Eight warps: warp w may read TMEM lanes 32 (w % 4) .. +31, so two warps share every block
    // of 32 query rows.  Partner threads split a row's 128 scores (and the D output columns) in
    // halves, exchange their half-row maxima through shared memory once per key tile, and keep
    // separate partial row sums that are combined at the very end.  Each thread reads its 64
    // scores from TMEM once (both 32-column loads in flight together).
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row_local = quarter * 32 + lane;
    const int row = q0 + row_local;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t p_row = smem_u32(sp) + half * kBlockBytes + row_local * 128;
    const int swz = row_local & 7;
    constexpr int DH = D / 2;                      // output columns owned by this thread
    float m = -INFINITY, l = 0.f;
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[sb], (j >> 1) & 1u, abort_flag));
      if (!ok) break;
      tmem_fence_after();
      const int valid = min(kTile, p.skv - j * kTile) - half * 64;     // valid columns of my half
      uint32_t r[64];
      tmem_ld32(lane_base + sb * kTile + half * 64, r);
      tmem_ld32(lane_base + sb * kTile + half * 64 + 32, r + 32);
      tmem_ld_wait();
      float mx = -INFINITY;
      if (valid >= 64) {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i < valid) mx = fmaxf(mx, __uint_as_float(r[i]));
      }
      // exchange with the partner thread of the other half (slots alternate with the tile parity;
      // a tagged slot is rewritten two tiles later, after the partner has published its next one)
      {
        float other;
        ok = __all_sync(0xffffffffu,
                        exchange(xmax, xtag, ((j & 1) * 2 + half) * kTile + row_local,
                                 ((j & 1) * 2 + (half ^ 1)) * kTile + row_local, mx, j + 1, other, abort_flag));
        if (!ok) break;
        mx = fmaxf(mx, other);
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float corr = exp2f(m - m_new);              // 0 on the first tile (m = -inf)
      // the previous P V must be done before its P operand is overwritten
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1u, abort_flag));
        if (!ok) break;
        tmem_fence_after();
      }
      float rowsum = 0.f;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        float pv[8];
        if (valid >= 64) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            pv[i] = exp2f(__uint_as_float(r[g * 8 + i]) * p.scale_log2 - m_new);
            rowsum += pv[i];
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float e = exp2f(__uint_as_float(r[g * 8 + i]) * p.scale_log2 - m_new);
            pv[i] = (g * 8 + i) < valid ? e : 0.f;
            rowsum += pv[i];
          }
        }
        const bf16x8 packed = pack8(pv);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                         p_row + (((uint32_t)g ^ (uint32_t)swz) << 4)),
                     "r"(packed.u.x), "r"(packed.u.y), "r"(packed.u.z), "r"(packed.u.w)
                     : "memory");
      }
      fence_async_smem();
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      // absorb my half of the previous partial product: o = (o + P[j-1] V[j-1]) * corr
      if (j > 0) {
        const uint32_t o_addr = lane_base + C::kOCol + ((j - 1) & 1) * D + half * DH;
        uint32_t q[DH];
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) tmem_ld32(o_addr + c * 32, q + c * 32);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < DH; ++i) o[i] = (o[i] + __uint_as_float(q[i])) * corr;
      }
      l = l * corr + rowsum;
      m = m_new;
    }
    if (ok) {
      const int last = n_tiles - 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[last & 1], (last >> 1) & 1u, abort_flag));
    }
    if (ok) {
      tmem_fence_after();
      const int last = n_tiles - 1;
      const uint32_t o_addr = lane_base + C::kOCol + (last & 1) * D + half * DH;
      // combine the partners' partial row sums (both are relative to the same running maximum)
      float other_l = 0.f;
      ok = __all_sync(0xffffffffu, exchange(xsum, xsum_tag, half * kTile + row_local,
                                            (half ^ 1) * kTile + row_local, l, 1, other_l, abort_flag));
      l += other_l;
      const float inv = 1.f / l;
      uint32_t q[DH];
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) tmem_ld32(o_addr + c * 32, q + c * 32);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < DH; ++i) o[i] = (o[i] + __uint_as_float(q[i])) * inv;
      if (ok && row < p.sq) {
        __nv_bfloat16* dst = out_row<D>(p, bi, row, hi) + half * DH;
#pragma unroll
        for (int g = 0; g < DH / 8; ++g) *reinterpret_cast<bf16x8*>(dst + g * 8) = pack8(&o[g * 8]);
        if (half == 0) p.lse[(int64_t)bh * p.sq + row] = (m + log2f(l)) * 0.6931471805599453f;
      }
    }
    if (!ok && lane == 0) {
      if (atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutSoftmax);
    }
  }

  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// Variant for head dimension 64: four softmax warps (one thread per query row, two TMEM passes over
// the scores), one score buffer, 256 TMEM columns and 115 KB of shared memory per CTA, so that TWO
// CTAs share an SM and overlap each other's softmax and MMA phases.  With d = 64 the softmax work
// per MMA flop doubles, and two independent CTAs hide it better than one wider CTA (0.43 ms
// against 0.52 ms on 16 x 24 x 1178 tokens); d = 128 is the other way round.
// ------------------------------------------------------------------------------------------
constexpr int kSmallThreads = 192;

template <int D>
struct SmallCfg {
  static constexpr int kDBlocks = D / 64;
  static constexpr uint32_t kTileBytes = kDBlocks * kBlockBytes;      // Q, K or V tile
  static constexpr uint32_t kSmemBytes = 5 * kTileBytes + kPBytes + 256;
  static constexpr int kSBufs = D == 64 ? 1 : 2;                      // score buffers in TMEM
  static constexpr uint32_t kOCol = kSBufs * kTile;                   // first O column in TMEM
  static constexpr uint32_t kTmemCols = kOCol + 2 * D;                // 256 or 512
  static constexpr int kCtasPerSm = D == 64 ? 2 : 1;
};

template <int D>
__global__ void __launch_bounds__(kSmallThreads, SmallCfg<D>::kCtasPerSm)
flash_fwd_small_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const Params p) {
  using C = SmallCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {          // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicExch(p.status, kMisalignedSmem);
    return;
  }
  uint8_t* sq = smem;
  uint8_t* sk = sq + C::kTileBytes;            // [2]
  uint8_t* sv = sk + 2 * C::kTileBytes;        // [2]
  uint8_t* sp = sv + 2 * C::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sp + kPBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* k_empty = bars + 3;    // [2]
  uint64_t* v_full = bars + 5;     // [2]
  uint64_t* v_empty = bars + 7;    // [2] spare: the V stage is released through o_full
  uint64_t* s_full = bars + 9;     // [2]
  uint64_t* o_full = bars + 11;    // [2]
  uint64_t* p_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, q0 = blockIdx.x * kTile;
  const int bi = bh / p.heads, hi = bh % p.heads;
  const int n_tiles = (p.skv + kTile - 1) / kTile;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&o_full[s], 1);
    }
    mbar_init(p_full, 4);
    *abort_flag = 0;
    mbar_fence_init();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ----------------------------------------------------------------------- TMA producer
    bool ok = true;
    mbar_expect_tx(q_full, C::kTileBytes);
#pragma unroll
    for (int c = 0; c < C::kDBlocks; ++c) tma_load_4d(sq + c * kBlockBytes, &map_q, q_full, c * 64, q0, hi, bi);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = ((j >> 1) & 1u) ^ 1u;
      if (!mbar_wait(&k_empty[s], ph, abort_flag)) { ok = false; break; }
      mbar_expect_tx(&k_full[s], C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
        tma_load_4d(sk + s * C::kTileBytes + c * kBlockBytes, &map_k, &k_full[s], c * 64, j * kTile, hi, bi);
      if (!mbar_wait(&o_full[s], ph, abort_flag)) { ok = false; break; }     // P V of step j-2 done
      mbar_expect_tx(&v_full[s], C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
        tma_load_4d(sv + s * C::kTileBytes + c * kBlockBytes, &map_v, &v_full[s], c * 64, j * kTile, hi, bi);
    }
    if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutProducer);
    if (*abort_flag) {
      // copies already issued write into this CTA's shared memory: give them time to land
      for (uint32_t spin = 0; spin < (1u << 20); ++spin)
        if (mbar_try(q_full, 0)) break;
      for (int s = 0; s < 2; ++s)
        for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
          if (mbar_try(&k_full[s], 0) || mbar_try(&k_full[s], 1)) break;
        }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_qk = make_idesc(kTile, kTile, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(kTile, D, 0, 1);
    // operand descriptors: constant high half, low half = base + (byte offset >> 4)
    constexpr uint32_t hi = desc_hi(1024);
    const uint32_t q_lo = desc_lo(smem_u32(sq), 16), k_lo = desc_lo(smem_u32(sk), 16);
    const uint32_t p_lo = desc_lo(smem_u32(sp), 16), v_lo = desc_lo(smem_u32(sv), kBlockBytes);
    bool ok = mbar_wait(q_full, 0, abort_flag);
    tmem_fence_after();
    auto issue_qk = [&](int j) -> bool {
      const int s = j & 1;
      const int sbuf = j % C::kSBufs;
      if (!mbar_wait(&k_full[s], (j >> 1) & 1u, abort_flag)) return false;
      tmem_fence_after();
      const uint32_t stage = (uint32_t)s * (C::kTileBytes >> 4);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_split(tmem_base + sbuf * kTile, q_lo + ((c * kBlockBytes + kk * 32) >> 4), hi,
                          k_lo + stage + ((c * kBlockBytes + kk * 32) >> 4), hi, idesc_qk, (c | kk) ? 1u : 0u);
      umma_commit(&k_empty[s]);
      umma_commit(&s_full[sbuf]);
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      // with two score buffers the next Q K^T runs while the softmax warps work on this tile;
      // with one it has to wait until they have consumed the scores (signalled with P)
      if (C::kSBufs == 2 && j + 1 < n_tiles && !issue_qk(j + 1)) { ok = false; break; }
      if (!mbar_wait(p_full, j & 1u, abort_flag)) { ok = false; break; }
      if (C::kSBufs == 1 && j + 1 < n_tiles && !issue_qk(j + 1)) { ok = false; break; }
      const int s = j & 1;
      if (!mbar_wait(&v_full[s], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      tmem_fence_after();
      const uint32_t vstage = (uint32_t)s * (C::kTileBytes >> 4);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16_split(tmem_base + C::kOCol + s * D, p_lo + (((kk >> 2) * kBlockBytes + (kk & 3) * 32) >> 4), hi,
                        v_lo + vstage + ((kk * 2048) >> 4), hi, idesc_pv, kk ? 1u : 0u);
      // one commit serves both readers of "P V of this step is done": the softmax warps (partial
      // output ready) and the producer (V stage free); a commit costs the issuing thread ~100 cycles
      umma_commit(&o_full[s]);
    }
    if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutMma);
  } else if (warp >= 2) {
    // --------------------------------------------------------------------------- softmax
    const int quarter = warp & 3;
    const int row_local = quarter * 32 + lane;
    const int row = q0 + row_local;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t p_row = smem_u32(sp) + row_local * 128;
    const int swz = row_local & 7;
    float m = -INFINITY, l = 0.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j % C::kSBufs;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[sb], (j / C::kSBufs) & 1u, abort_flag));
      if (!ok) break;
      tmem_fence_after();
      const int valid = min(kTile, p.skv - j * kTile);
      const uint32_t s_addr = lane_base + sb * kTile;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(s_addr + c * 32, r);
        tmem_ld_wait();
        if (valid == kTile) {                          // only the last key tile is ever partial
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < valid) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float corr = exp2f(m - m_new);              // 0 on the first tile (m = -inf)
      // the previous P V must be done before its P operand is overwritten
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1u, abort_flag));
        if (!ok) break;
        tmem_fence_after();
      }
      // pass 2: probabilities -> shared memory (bf16, swizzled K-major), row sum
      float rowsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(s_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float pv[8];
          if (valid == kTile) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              pv[i] = exp2f(__uint_as_float(r[g * 8 + i]) * p.scale_log2 - m_new);
              rowsum += pv[i];
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int col = c * 32 + g * 8 + i;
              const float e = exp2f(__uint_as_float(r[g * 8 + i]) * p.scale_log2 - m_new);
              pv[i] = col < valid ? e : 0.f;
              rowsum += pv[i];
            }
          }
          const bf16x8 packed = pack8(pv);
          const uint32_t chunk = (uint32_t)((c & 1) * 4 + g);
          const uint32_t addr = p_row + (c >> 1) * kBlockBytes + ((chunk ^ (uint32_t)swz) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed.u.x),
                       "r"(packed.u.y), "r"(packed.u.z), "r"(packed.u.w)
                       : "memory");
        }
      }
      fence_async_smem();
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      // absorb the previous partial product: o = (o + P[j-1] V[j-1]) * corr
      if (j > 0) {
        const uint32_t o_addr = lane_base + C::kOCol + ((j - 1) & 1) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(o_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(r[i])) * corr;
        }
      }
      l = l * corr + rowsum;
      m = m_new;
    }
    if (ok) {
      const int last = n_tiles - 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[last & 1], (last >> 1) & 1u, abort_flag));
    }
    if (ok) {
      tmem_fence_after();
      const int last = n_tiles - 1;
      const uint32_t o_addr = lane_base + C::kOCol + (last & 1) * D;
      const float inv = 1.f / l;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(o_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(r[i])) * inv;
      }
      if (row < p.sq) {
        __nv_bfloat16* dst = out_row<D>(p, bi, row, hi);
#pragma unroll
        for (int g = 0; g < D / 8; ++g) *reinterpret_cast<bf16x8*>(dst + g * 8) = pack8(&o[g * 8]);
        p.lse[(int64_t)bh * p.sq + row] = (m + log2f(l)) * 0.6931471805599453f;
      }
    } else if (lane == 0) {
      if (atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutSoftmax);
    }
  }

  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
// Lazy-rescale forward (the default for head dimension 64, and the causal path of both sizes).
//
// The softmax warps of the kernels above issue ~14 instructions per score; with the tensor pipe
// under 20 % busy and the issue slots 60 % busy, instruction count — not the MMA, not the exp
// unit — bounded them.  This variant removes the work that was not needed:
//   * the output accumulates in tensor memory across key tiles (the P V product adds into it);
//     it is rescaled only when a row's running maximum grows by more than 2^8, which after the
//     first tiles almost never happens, so the per-tile "read partial O, add, multiply" of the
//     register version is gone.  Probabilities are computed against the stale maximum (they stay
//     below 2^8, harmless in bf16 / fp32) and the final division by the row sum makes the result
//     exact in the usual sense;
//   * one thread owns one query row: no partner exchange, no shared-memory max hand-off;
//   * scale-and-subtract and the row sum use packed fp32x2 arithmetic, the row maximum three-input
//     max, so a score costs ~4 issued instructions (TMEM load, max, fma, ex2, add, cvt, store);
//   * `causal` skips the key tiles above the diagonal and masks inside the diagonal tile
//     (query row r attends keys 0 .. r + skv - sq).
// TMEM: S in columns [0, 128), O in [128, 128 + D); two CTAs per SM at D = 64.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %4};\n\t"
      "mov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr float kRescaleThreshold = 8.f;       // log2 units: rescale O when the maximum grows by > 2^8

template <int D>
struct LazyCfg {
  static constexpr int kDBlocks = D / 64;
  static constexpr uint32_t kTileBytes = kDBlocks * kBlockBytes;      // Q, K or V tile
  static constexpr uint32_t kSmemBytes = 5 * kTileBytes + kPBytes + 256;
  static constexpr uint32_t kOCol = kTile;                            // first O column in TMEM
  static constexpr uint32_t kTmemCols = 256;                          // S (128) + O (D <= 128)
  static constexpr int kCtasPerSm = D == 64 ? 2 : 1;
};

template <int D>
__global__ void __launch_bounds__(kSmallThreads, LazyCfg<D>::kCtasPerSm)
flash_fwd_lazy_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const Params p) {
  using C = LazyCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0) atomicExch(p.status, kMisalignedSmem);
    return;
  }
  uint8_t* sq = smem;
  uint8_t* sk = sq + C::kTileBytes;            // [2]
  uint8_t* sv = sk + 2 * C::kTileBytes;        // [2]
  uint8_t* sp = sv + 2 * C::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sp + kPBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* k_empty = bars + 3;    // [2]
  uint64_t* v_full = bars + 5;     // [2]
  uint64_t* s_full = bars + 7;
  uint64_t* o_full = bars + 8;     // [2] P V of step j done (also frees V stage j & 1 and the P tile)
  uint64_t* p_full = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, q0 = blockIdx.x * kTile;
  const int bi = bh / p.heads, hi = bh % p.heads;
  int n_tiles = (p.skv + kTile - 1) / kTile;
  const int causal_off = p.skv - p.sq;
  if (p.causal) {
    // last key any row of this tile may see: (q0 + 127, clipped to sq - 1) + causal_off
    const int last_key = min(q0 + kTile, p.sq) - 1 + causal_off;
    n_tiles = max(1, min(n_tiles, last_key / kTile + 1));
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&o_full[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    *abort_flag = 0;
    mbar_fence_init();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ----------------------------------------------------------------------- TMA producer
    bool ok = true;
    mbar_expect_tx(q_full, C::kTileBytes);
#pragma unroll
    for (int c = 0; c < C::kDBlocks; ++c) tma_load_4d(sq + c * kBlockBytes, &map_q, q_full, c * 64, q0, hi, bi);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = ((j >> 1) & 1u) ^ 1u;
      if (!mbar_wait(&k_empty[s], ph, abort_flag)) { ok = false; break; }
      mbar_expect_tx(&k_full[s], C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
        tma_load_4d(sk + s * C::kTileBytes + c * kBlockBytes, &map_k, &k_full[s], c * 64, j * kTile, hi, bi);
      if (!mbar_wait(&o_full[s], ph, abort_flag)) { ok = false; break; }     // P V of step j-2 done
      mbar_expect_tx(&v_full[s], C::kTileBytes);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
        tma_load_4d(sv + s * C::kTileBytes + c * kBlockBytes, &map_v, &v_full[s], c * 64, j * kTile, hi, bi);
    }
    if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutProducer);
    if (*abort_flag) {
      for (uint32_t spin = 0; spin < (1u << 20); ++spin)
        if (mbar_try(q_full, 0)) break;
      for (int s = 0; s < 2; ++s)
        for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
          if (mbar_try(&k_full[s], 0) || mbar_try(&k_full[s], 1)) break;
        }
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_qk = make_idesc(kTile, kTile, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(kTile, D, 0, 1);
    constexpr uint32_t hi = desc_hi(1024);
    const uint32_t q_lo = desc_lo(smem_u32(sq), 16), k_lo = desc_lo(smem_u32(sk), 16);
    const uint32_t p_lo = desc_lo(smem_u32(sp), 16), v_lo = desc_lo(smem_u32(sv), kBlockBytes);
    bool ok = mbar_wait(q_full, 0, abort_flag);
    tmem_fence_after();
    auto issue_qk = [&](int j) -> bool {
      const int s = j & 1;
      if (!mbar_wait(&k_full[s], (j >> 1) & 1u, abort_flag)) return false;
      tmem_fence_after();
      const uint32_t stage = (uint32_t)s * (C::kTileBytes >> 4);
#pragma unroll
      for (int c = 0; c < C::kDBlocks; ++c)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_split(tmem_base, q_lo + ((c * kBlockBytes + kk * 32) >> 4), hi,
                          k_lo + stage + ((c * kBlockBytes + kk * 32) >> 4), hi, idesc_qk, (c | kk) ? 1u : 0u);
      umma_commit(&k_empty[s]);
      umma_commit(s_full);
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      // P of tile j is in shared memory and the scores of tile j have been consumed
      if (!mbar_wait(p_full, j & 1u, abort_flag)) { ok = false; break; }
      if (j + 1 < n_tiles && !issue_qk(j + 1)) { ok = false; break; }
      const int s = j & 1;
      if (!mbar_wait(&v_full[s], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      tmem_fence_after();
      const uint32_t vstage = (uint32_t)s * (C::kTileBytes >> 4);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16_split(tmem_base + C::kOCol, p_lo + (((kk >> 2) * kBlockBytes + (kk & 3) * 32) >> 4), hi,
                        v_lo + vstage + ((kk * 2048) >> 4), hi, idesc_pv, (j | kk) ? 1u : 0u);
      umma_commit(&o_full[s]);
    }
    if (!ok && atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutMma);
  } else if (warp >= 2) {
    // --------------------------------------------------------------------------- softmax
    const int quarter = warp & 3;
    const int row_local = quarter * 32 + lane;
    const int row = q0 + row_local;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t p_row = smem_u32(sp) + row_local * 128;
    const uint32_t swz = (uint32_t)(row_local & 7);
    const float scale = p.scale_log2;
    float m = -INFINITY, l0 = 0.f, l1 = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, j & 1u, abort_flag));
      if (!ok) break;
      tmem_fence_after();
      uint32_t r[kTile];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(lane_base + c * 32, r + c * 32);
      tmem_ld_wait();
      // keys this row may see inside the tile
      int lim = min(kTile, p.skv - j * kTile);
      if (p.causal) lim = min(lim, row + causal_off - j * kTile + 1);
      if (lim < kTile) {
#pragma unroll
        for (int i = 0; i < kTile; ++i)
          if (i >= lim) r[i] = 0xff800000u;           // -inf: contributes exp2(-inf) = 0
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kTile; i += 8) {
        mx0 = max3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        mx1 = max3(mx1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
        mx2 = max3(mx2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
        mx3 = max3(mx3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
      }
      const float m_cand = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale;
      const bool grow = m_cand > m + kRescaleThreshold;        // always true on the first tile
      const bool any_grow = __any_sync(0xffffffffu, grow);
      // P V of the previous tile must be done before P is overwritten and before O is rescaled
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1u, abort_flag));
        if (!ok) break;
        tmem_fence_after();
      }
      if (any_grow) {
        const float m_new = grow ? m_cand : m;
        const float corr = j == 0 ? 0.f : ex2(m - m_new);     // 1 for rows whose maximum stayed
        if (j > 0) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t q[32];
            tmem_ld32(lane_base + C::kOCol + c * 32, q);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) q[i] = __float_as_uint(__uint_as_float(q[i]) * corr);
            tmem_st16(lane_base + C::kOCol + c * 32, q);
            tmem_st16(lane_base + C::kOCol + c * 32 + 16, q + 16);
          }
          tmem_st_wait();
        }
        l0 *= corr;
        l1 *= corr;
        m = m_new;
      }
      const float neg_m = -m;
#pragma unroll
      for (int g = 0; g < 16; ++g) {
        float pv[8];
#pragma unroll
        for (int i = 0; i < 8; i += 2)
          fma2(pv[i], pv[i + 1], __uint_as_float(r[g * 8 + i]), __uint_as_float(r[g * 8 + i + 1]), scale, neg_m);
#pragma unroll
        for (int i = 0; i < 8; ++i) pv[i] = ex2(pv[i]);
#pragma unroll
        for (int i = 0; i < 8; i += 2) add2(l0, l1, l0, l1, pv[i], pv[i + 1]);
        const bf16x8 packed = pack8(pv);
        const uint32_t c = (uint32_t)g >> 2;                    // which 32-column group
        const uint32_t chunk = (c & 1u) * 4u + ((uint32_t)g & 3u);
        const uint32_t addr = p_row + (c >> 1) * kBlockBytes + ((chunk ^ swz) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed.u.x),
                     "r"(packed.u.y), "r"(packed.u.z), "r"(packed.u.w)
                     : "memory");
      }
      fence_async_smem();
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) {
      const int last = n_tiles - 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&o_full[last & 1], (last >> 1) & 1u, abort_flag));
    }
    if (ok) {
      tmem_fence_after();
      const float l = l0 + l1;
      const float inv = 1.f / l;
      float o[D];
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t q[32];
        tmem_ld32(lane_base + C::kOCol + c * 32, q);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = __uint_as_float(q[i]) * inv;
      }
      if (row < p.sq) {
        __nv_bfloat16* dst = out_row<D>(p, bi, row, hi);
#pragma unroll
        for (int g = 0; g < D / 8; ++g) *reinterpret_cast<bf16x8*>(dst + g * 8) = pack8(&o[g * 8]);
        p.lse[(int64_t)bh * p.sq + row] = (m + log2f(l)) * 0.6931471805599453f;
      }
    } else if (lane == 0) {
      if (atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutSoftmax);
    }
  }

  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// --------------------------------------------------------------------------------- host side
int* status_word(int device) { return kernel_status_block(device) + kStatusAttention; }

static void launch_small(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p,
                         int q_tiles, int bh, cudaStream_t stream) {
  static const bool attr_set = [] {
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_small_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        SmallCfg<64>::kSmemBytes));
    return true;
  }();
  (void)attr_set;
  flash_fwd_small_kernel<64><<<dim3(q_tiles, bh), kSmallThreads, SmallCfg<64>::kSmemBytes, stream>>>(mq, mk, mv, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <int D>
static void launch_lazy(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p,
                        int q_tiles, int bh, cudaStream_t stream) {
  static const bool attr_set = [] {
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_lazy_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        LazyCfg<D>::kSmemBytes));
    return true;
  }();
  (void)attr_set;
  flash_fwd_lazy_kernel<D><<<dim3(q_tiles, bh), kSmallThreads, LazyCfg<D>::kSmemBytes, stream>>>(mq, mk, mv, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <int D>
static void launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p,
                   int q_tiles, int bh, cudaStream_t stream) {
  static const bool attr_set = [] {
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg<D>::kSmemBytes));
    return true;
  }();
  (void)attr_set;
  flash_fwd_kernel<D><<<dim3(q_tiles, bh), kThreads, Cfg<D>::kSmemBytes, stream>>>(mq, mk, mv, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace attn

// `causal`: query row r attends keys 0 .. r + (Skv - Sq) (needs Sq <= Skv).  `variant`: 0 picks the
// default kernel for the shape, 1 forces the register-accumulating kernels, 2 the lazy-rescale one.
static std::vector<torch::Tensor> flash_attn_fwd_impl(torch::Tensor q, torch::Tensor k, torch::Tensor v, double scale,
                                                      bool causal, int64_t variant, const torch::Tensor* out_peers,
                                                      int64_t sp_world, int64_t sp_rank, int64_t heads_total);

std::vector<torch::Tensor> flash_attn_fwd(torch::Tensor q, torch::Tensor k, torch::Tensor v, double scale,
                                          bool causal, int64_t variant) {
  return flash_attn_fwd_impl(q, k, v, scale, causal, variant, nullptr, 1, 0, 0);
}

// Sequence-parallel form: q, k, v hold this rank's `H / world` heads over the full sequence; the
// output rows are stored into the sequence owners' [B, S / world, heads_total, D] buffers
// (`out_peers`: CPU int64 table of their peer-mapped addresses).  Returns {lse}.
std::vector<torch::Tensor> flash_attn_fwd_peers(torch::Tensor q, torch::Tensor k, torch::Tensor v, double scale,
                                                torch::Tensor out_peers, int64_t world, int64_t rank,
                                                int64_t heads_total) {
  TORCH_CHECK(world >= 2 && world <= 16 && rank >= 0 && rank < world, "flash_attn_fwd_peers: 2..16 ranks");
  TORCH_CHECK(out_peers.device().is_cpu() && out_peers.scalar_type() == torch::kInt64 && out_peers.numel() >= world,
              "out_peers: CPU int64 tensor with one address per rank");
  TORCH_CHECK(q.dim() == 4 && q.size(2) % world == 0 && q.size(1) * world == heads_total,
              "flash_attn_fwd_peers: sequence must divide by the ranks and heads_total = local heads * world");
  auto outs = flash_attn_fwd_impl(q, k, v, scale, false, 0, &out_peers, world, rank, heads_total);
  return {outs[1]};
}

static std::vector<torch::Tensor> flash_attn_fwd_impl(torch::Tensor q, torch::Tensor k, torch::Tensor v, double scale,
                                                      bool causal, int64_t variant, const torch::Tensor* out_peers,
                                                      int64_t sp_world, int64_t sp_rank, int64_t heads_total) {
  using namespace attn;
  TORCH_CHECK(q.is_cuda() && q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "flash_attn_fwd: [B, H, S, D]");
  TORCH_CHECK(q.scalar_type() == torch::kBFloat16 && k.scalar_type() == torch::kBFloat16 &&
              v.scalar_type() == torch::kBFloat16);
  const int64_t b = q.size(0), h = q.size(1), sq = q.size(2), d = q.size(3), skv = k.size(2);
  TORCH_CHECK(d == 64 || d == 128, "flash_attn_fwd: head dimension 64 or 128");
  TORCH_CHECK(k.size(0) == b && k.size(1) == h && k.size(3) == d && v.sizes() == k.sizes());
  VRL_CHECK_OPERAND(k, q);
  VRL_CHECK_OPERAND(v, q);
  q = mappable(q);
  k = mappable(k);
  v = mappable(v);
  const c10::cuda::CUDAGuard guard(q.device());
  bind_context();
  // token-major output, returned as a [B, H, S, D] view: merging heads afterwards is free
  // (the sequence-parallel form writes into the peers' buffers instead and allocates nothing here)
  auto out_tm = out_peers != nullptr ? torch::empty({0, 0, h, d}, q.options())
                                     : torch::empty({b, sq, h, d}, q.options());
  auto out = out_tm.transpose(1, 2);
  auto lse = torch::empty({b, h, sq}, q.options().dtype(torch::kFloat32));
  if (b * h == 0 || sq == 0) return {out, lse};
  TORCH_CHECK(skv > 0, "flash_attn_fwd: empty key sequence");
  TORCH_CHECK(!causal || sq <= skv, "flash_attn_fwd: causal attention needs Sq <= Skv");
  TORCH_CHECK(variant >= 0 && variant <= 2 && !(causal && variant == 1),
              "flash_attn_fwd: variant 0 (default), 1 (register accumulation, no causal) or 2 (lazy rescale)");
  const CUtensorMap mq = make_map4(q, kTile);
  const CUtensorMap mk = make_map4(k, kTile);
  const CUtensorMap mv = make_map4(v, kTile);
  Params p{};
  p.out = reinterpret_cast<__nv_bfloat16*>(out_tm.data_ptr());
  p.heads = (int)h;
  p.lse = lse.data_ptr<float>();
  p.status = status_word(q.get_device());
  p.sq = (int)sq;
  p.skv = (int)skv;
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.causal = causal ? 1 : 0;
  if (out_peers != nullptr) {
    p.sp_world = (int)sp_world;
    p.sp_sloc = (int)(sq / sp_world);
    p.sp_heads_total = (int)heads_total;
    p.sp_head0 = (int)(sp_rank * h);
    for (int r = 0; r < sp_world; ++r) {
      const int64_t addr = out_peers->data_ptr<int64_t>()[r];
      TORCH_CHECK(addr != 0 && addr % 16 == 0, "flash_attn_fwd_peers: output addresses must be 16-byte aligned");
      p.out_peer[r] = reinterpret_cast<__nv_bfloat16*>(addr);
    }
  }
  const int q_tiles = (int)((sq + kTile - 1) / kTile);
  TORCH_CHECK(b * h <= 65535, "flash_attn_fwd: batch * heads exceeds the grid limit");
  auto stream = at::cuda::getCurrentCUDAStream();
  const bool lazy = variant == 2 || causal || (variant == 0 && d == 64);
  if (lazy && d == 64) launch_lazy<64>(mq, mk, mv, p, q_tiles, (int)(b * h), stream);
  else if (lazy) launch_lazy<128>(mq, mk, mv, p, q_tiles, (int)(b * h), stream);
  else if (d == 64) launch_small(mq, mk, mv, p, q_tiles, (int)(b * h), stream);
  else launch<128>(mq, mk, mv, p, q_tiles, (int)(b * h), stream);
  return {out, lse};
}

}  // namespace vrl
