// K1: persistent bf16 GEMM for sm_100a.  C[M,N] = epilogue(A · B^T) with fp32 accumulation.
//
//   * operands reach shared memory through TMA (cp.async.bulk.tensor, 128-byte swizzle,
//     no cluster multicast), four pipeline stages of a 128x64 A tile and a 256x64 B tile;
//   * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=256, K=16);
//     the accumulator lives in tensor memory, double-buffered (2 x 256 columns) so the
//     epilogue of tile i overlaps the main loop of tile i+1;
//   * four epilogue warps read the accumulator with tcgen05.ld (32 lanes x 32 columns),
//     apply bias / GELU-tanh / SiLU / adaLN gate-residual in registers and store bf16 or fp32;
//   * either operand may be "MN-major" (stored [K, M] resp. [K, N] with the non-contracted
//     dimension contiguous), which is what the backward GEMMs dX = dY·W and dW = dY^T·X need;
//   * every mbarrier wait is bounded: on expiry the kernel records where it gave up in a
//     status word, drains its own TMA copies (bounded as well), frees its tensor memory and
//     returns; the host raises after the launch completes.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..9 = epilogue.  Warp w may only touch TMEM lanes 32*(w%4) .. 32*(w%4)+31, so two
// warps share every lane quarter and split the 256 accumulator columns between them.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cudaTypedefs.h>
#include <torch/extension.h>

#include <cstdlib>
#include <string>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "ops.h"
#include "sm100_ptx.cuh"

namespace vrl {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kThreads = 320;      // TMA warp, MMA warp, 8 epilogue warps
constexpr uint32_t kABytes = BM * BK * 2;          // 16 KiB
constexpr uint32_t kBBytes = BN * BK * 2;          // 32 KiB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kTmemCols = 512;                // two 256-column fp32 accumulators
constexpr int kEpiWarps = 8;
constexpr uint32_t kStoreBytes = 32 * 128;         // one warp's 32-row x 64-column bf16 staging tile
constexpr uint32_t kStagingBytes = kEpiWarps * kStoreBytes;
constexpr uint32_t kSmemBytes =
    kStages * kStageBytes + kStagingBytes + 1024 /*align*/ + 256 /*barriers*/;

enum Status : int { kOk = 0, kTimeoutProducer = 1, kTimeoutMma = 2, kTimeoutEpilogue = 3 };

struct Params {
  void* c;
  const __nv_bfloat16* bias;       // [N] or null
  const __nv_bfloat16* gate;       // [M / rows_per_gate, N] or null
  const __nv_bfloat16* residual;   // [M, N] or null
  int* status;
  int m, n, k;
  int act;                         // 0 none, 1 gelu-tanh, 2 silu, 3 multiply by gelu'(residual)
  int dual;                        // also store the pre-activation (acc + bias) through map_c2
  int rows_per_gate;
  int64_t gate_ld;                 // elements between consecutive gate rows
  int a_mn, b_mn;
  int a_mn3, b_mn3;                // the MN-major operand's map is 3-D: one copy per stage instead of one per 64-wide chunk
  int out_fp32;
  // all-gather fused into the GEMM (B operand sharded by rows over `g_world` ranks)
  const __nv_bfloat16* g_peer[16]; // every rank's shard [g_rows, K] (peer-mapped pointers)
  __nv_bfloat16* g_full;           // local [N, K] buffer the shards are gathered into (= B operand)
  int* g_ready;                    // [g_world] arrival counters, zero before the launch
  int g_world, g_rank, g_rows;     // g_rows = N / g_world
  int g_first_tile;                // n-tile holding this rank's own rows: processed first
  int g_band;                      // m-tiles per band of the gathering variant's tile order
  // Grouped products (mixture of experts; 0 = off).  The rows of the activation are sorted by
  // expert and every expert's run is padded to a multiple of BM rows.
  //   1: C[r, :] = epilogue(A[r, :] B_e^T), e = grp_tile_expert[r / BM] (negative: unused tile).
  //      B holds all experts' matrices stacked along its outer dimension, grp_stride rows apart.
  //   2: C_e = A[rows of e]^T B[rows of e] for every expert e (weight gradients): the contraction
  //      runs over the expert's padded row range grp_offsets[e] .. grp_offsets[e + 1]; the tile
  //      index also enumerates the experts and C_e starts at row e * m of the output.
  int grp_mode;
  int grp_experts;
  int grp_stride;
  const int* grp_tile_expert;
  const int* grp_offsets;
  // log-sum-exp epilogues of the vocabulary head (0 = off).  1: nothing is stored but, per row and
  // 64-column chunk, the maximum and the exponential sum of (acc + bias) / T, plus the target's
  // value; 2: the stored bf16 value is g/T * (onehot(id) - exp((acc + bias) / T - lse)).
  int lse_mode;
  const int64_t* lse_ids;          // [M] target column (global index; lse_col0 is this product's first)
  int64_t lse_col0;
  float lse_inv_t;
  float* lse_part_max;             // [ceil(N / 64), M]
  float* lse_part_sum;             // [ceil(N / 64), M]
  float* lse_target;               // [M]
  const float* lse_lse;            // [M]  (mode 2)
  const float* lse_g;              // [M]  (mode 2)
};

constexpr int kGatherThreads = 128;
enum : int { kTimeoutGather = 4 };

// Tile index -> tile origin.  Plain GEMMs sweep n fastest.  The gathering variant works through
// bands of `g_band` m-tiles; inside a band it sweeps m fastest and starts at the n-tiles of the
// local shard, so the peers' rows are needed as late as the first band allows.  The band keeps the
// A rows that one pass over the n-tiles re-reads small enough to stay in L2: an m-fastest sweep
// over all of a large A would fetch it from DRAM once per n-tile.
template <bool kGather>
__device__ __forceinline__ void tile_origin(int tile, int m_tiles, int n_tiles, const Params& p, int& m0,
                                            int& n0) {
  if (kGather) {
    const int band_tiles = p.g_band * n_tiles;
    const int band = tile / band_tiles;
    const int mt0 = band * p.g_band;
    const int mb = min(p.g_band, m_tiles - mt0);
    const int t = tile - band * band_tiles;
    int nt = t / mb + p.g_first_tile;
    if (nt >= n_tiles) nt -= n_tiles;
    m0 = (mt0 + t % mb) * BM;
    n0 = nt * BN;
  } else {
    m0 = (tile / n_tiles) * BM;
    n0 = (tile % n_tiles) * BN;
  }
}

// Everything a role needs to know about one tile; the three roles derive it independently and
// must agree, so it is a pure function of the tile index and the launch parameters.
struct TileInfo {
  int m0, n0;        // tile origin in the (per-expert, for grouped mode 2) output
  int kb0, kbn;      // first k-block and number of k-blocks of the contraction
  int b_off;         // offset added to B's outer coordinate (expert's matrix)
  int c_row_off;     // offset added to the output row coordinate
  int bias_off;
  bool skip;
};

template <bool kGather>
__device__ __forceinline__ TileInfo tile_info(int tile, int m_tiles, int n_tiles, int k_blocks, const Params& p) {
  TileInfo t;
  t.kb0 = 0; t.kbn = k_blocks; t.b_off = 0; t.c_row_off = 0; t.bias_off = 0; t.skip = false;
  if (!kGather && p.grp_mode == 2) {
    const int per = m_tiles * n_tiles;
    const int e = tile / per, r = tile - e * per;
    t.m0 = (r / n_tiles) * BM;
    t.n0 = (r % n_tiles) * BN;
    const int lo = p.grp_offsets[e], hi = p.grp_offsets[e + 1];
    t.kb0 = lo / BK;
    t.kbn = (hi - lo) / BK;
    t.c_row_off = e * p.m;
    return t;
  }
  tile_origin<kGather>(tile, m_tiles, n_tiles, p, t.m0, t.n0);
  if (!kGather && p.grp_mode == 1) {
    const int e = p.grp_tile_expert[t.m0 / BM];
    if (e < 0) { t.skip = true; t.kbn = 0; return t; }
    t.b_off = e * p.grp_stride;
    t.bias_off = e * p.n;
  }
  return t;
}

using namespace ptx;

// ------------------------------------------------------------------------------------- kernel
template <bool kGather>
__global__ void __launch_bounds__(kGather ? kThreads + kGatherThreads : kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_r,
                 const __grid_constant__ CUtensorMap map_c2, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + kStages * kStageBytes;      // 1024-byte aligned (stage size is 48 KiB)
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kStagingBytes);
  uint64_t* full = bars;                       // [kStages]
  uint64_t* empty = bars + kStages;            // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;     // [2]
  uint64_t* acc_empty = bars + 2 * kStages + 2;  // [2]
  uint64_t* res_full = bars + 2 * kStages + 4;   // [kEpiWarps] residual tile landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4 + kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.m + BM - 1) / BM, n_tiles = (p.n + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles * (p.grp_mode == 2 ? p.grp_experts : 1);
  const int k_blocks = (p.k + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], kEpiWarps); }
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(&res_full[w], 1);
    *abort_flag = 0;
    mbar_fence_init();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tmem_fence_before();
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------------ TMA producer
    uint32_t it = 0;
    bool ok = true;
    uint32_t slabs_seen = 0;       // bit r: the rows of rank r are known to be in g_full
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const TileInfo ti = tile_info<kGather>(tile, m_tiles, n_tiles, k_blocks, p);
      if (ti.skip) continue;
      const int m0 = ti.m0, n0 = ti.n0;
      if (kGather) {
        // the B rows of this tile must have been copied by the gather warps of EVERY CTA
        const int lo = n0 / p.g_rows, hi = min(p.n - 1, n0 + BN - 1) / p.g_rows;
        for (int r = lo; r <= hi && ok; ++r) {
          if (slabs_seen & (1u << r)) continue;
          bool ready = false;
          for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.g_ready + r) : "memory");
            if (v >= (int)gridDim.x) { ready = true; break; }
            if ((spin & 1023u) == 1023u && *abort_flag) break;
          }
          if (!ready) { ok = false; break; }
          slabs_seen |= 1u << r;
          asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy writes -> TMA reads
        }
        if (!ok) break;
      }
      for (int kb = 0; kb < ti.kbn; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t parity = ((it / kStages) & 1u) ^ 1u;
        if (!mbar_wait(&empty[s], parity, abort_flag)) { ok = false; break; }
        uint8_t* sa = smem + s * kStageBytes;
        uint8_t* sb = sa + kABytes;
        mbar_expect_tx(&full[s], kStageBytes);
        const int k0 = (ti.kb0 + kb) * BK;
        if (!p.a_mn) {
          tma_load_2d(sa, &map_a, &full[s], k0, m0);
        } else if (p.a_mn3) {
          tma_load_3d(sa, &map_a, &full[s], 0, k0, m0 / 64);
        } else {
#pragma unroll
          for (int c = 0; c < BM / 64; ++c)
            tma_load_2d(sa + c * (BK * 128), &map_a, &full[s], m0 + c * 64, k0);
        }
        if (!p.b_mn) {
          tma_load_2d(sb, &map_b, &full[s], k0, n0 + ti.b_off);
        } else if (p.b_mn3) {
          tma_load_3d(sb, &map_b, &full[s], 0, k0 + ti.b_off, n0 / 64);
        } else {
          // grouped mode 1 with a row-major B: the expert's matrix starts b_off rows down the
          // contraction coordinate; mode 2 contracts over the rows themselves (b_off = 0)
#pragma unroll
          for (int c = 0; c < BN / 64; ++c)
            tma_load_2d(sb + c * (BK * 128), &map_b, &full[s], n0 + c * 64, k0 + ti.b_off);
        }
      }
    }
    if (!ok) {
      if (atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutProducer);
    }
    // copies still in flight target this CTA's shared memory: give them time to land
    if (*abort_flag) {
      const uint32_t issued = it;
      for (uint32_t j = issued > (uint32_t)kStages ? issued - kStages : 0; j < issued; ++j) {
        const int s = j % kStages;
        for (uint32_t spin = 0; spin < (1u << 20); ++spin)
          if (mbar_try(&full[s], (j / kStages) & 1u)) break;
      }
    }
  } else if (warp == 1 && lane == 0) {
    // -------------------------------------------------------------------- MMA issuer
    const uint32_t idesc = make_idesc(BM, BN, p.a_mn, p.b_mn);
    // Descriptor halves: the issuing thread is the scarcest resource of the CTA (a tcgen05.mma costs
    // it ~48 cycles, a commit ~100, a wait more), so per product only the low half changes, by one
    // add.  K-major operands advance 32 bytes per k-step, MN-major ones 16 rows of 128 bytes.
    const uint32_t a_lo0 = desc_lo(smem_u32(smem), p.a_mn ? BK * 128 : 16);
    const uint32_t b_lo0 = desc_lo(smem_u32(smem) + kABytes, p.b_mn ? BK * 128 : 16);
    const uint32_t a_step = p.a_mn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
    const uint32_t b_step = p.b_mn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
    uint32_t it = 0, tile_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const TileInfo ti = tile_info<kGather>(tile, m_tiles, n_tiles, k_blocks, p);
      if (ti.skip) continue;
      const uint32_t buf = tile_it & 1u;
      if (!mbar_wait(&acc_empty[buf], ((tile_it >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
      tmem_fence_after();
      const uint32_t tmem_c = tmem_base + buf * BN;
      for (int kb = 0; kb < ti.kbn; ++kb, ++it) {
        const int s = it % kStages;
        if (!mbar_wait(&full[s], (it / kStages) & 1u, abort_flag)) { ok = false; break; }
        tmem_fence_after();
        const uint32_t sa = a_lo0 + (uint32_t)s * (kStageBytes >> 4), sb = b_lo0 + (uint32_t)s * (kStageBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk)
          umma_bf16_split(tmem_c, sa + kk * a_step, desc_hi(1024), sb + kk * b_step, desc_hi(1024), idesc,
                          (kb | kk) ? 1u : 0u);
        umma_commit(&empty[s]);           // frees the stage once these MMAs have read it
      }
      if (ok) umma_commit(&acc_full[buf]);     // with no products issued it completes at once
      ++tile_it;
    }
    if (!ok) {
      if (atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutMma);
    }
  } else if (kGather && warp >= 2 + kEpiWarps) {
    // ------------------------------------------------------------------------ gather
    // The 128 extra threads of every CTA copy this CTA's share of each rank's shard into the
    // local full-weight buffer, own rows first, then peer (r + 1), (r + 2), ... over NVLink with
    // plain 16-byte loads.  After a shard's share is written the group publishes it with a
    // release (fence + atomic); a shard is complete when all gridDim.x CTAs have published.
    const int gt = threadIdx.x - (2 + kEpiWarps) * 32;
    const int64_t vec_per_shard = (int64_t)p.g_rows * p.k / 8;
    const int64_t v_lo = vec_per_shard * blockIdx.x / gridDim.x;
    const int64_t v_hi = vec_per_shard * (blockIdx.x + 1) / gridDim.x;
    for (int step = 0; step < p.g_world; ++step) {
      int r = p.g_rank + step;
      if (r >= p.g_world) r -= p.g_world;
      const uint4* src = reinterpret_cast<const uint4*>(p.g_peer[r]);
      uint4* dst = reinterpret_cast<uint4*>(p.g_full + (int64_t)r * p.g_rows * p.k);
      // four independent 16-byte loads in flight per thread: a peer load takes microseconds, so
      // bandwidth over NVLink needs many outstanding requests
      int64_t v = v_lo + gt;
      for (; v + 3 * kGatherThreads < v_hi; v += 4 * kGatherThreads) {
        const uint4 t0 = src[v], t1 = src[v + kGatherThreads], t2 = src[v + 2 * kGatherThreads],
                    t3 = src[v + 3 * kGatherThreads];
        dst[v] = t0;
        dst[v + kGatherThreads] = t1;
        dst[v + 2 * kGatherThreads] = t2;
        dst[v + 3 * kGatherThreads] = t3;
      }
      for (; v < v_hi; v += kGatherThreads) dst[v] = src[v];
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kGatherThreads) : "memory");
      if (gt == 0) {
        __threadfence();                            // cumulative release of the group's stores
        asm volatile("fence.proxy.async;" ::: "memory");
        atomicAdd(p.g_ready + r, 1);
      }
    }
  } else if (warp >= 2 && warp < 2 + kEpiWarps) {
    // ---------------------------------------------------------------------- epilogue
    // bf16 results leave through shared memory: each warp converts a 32-row x 64-column piece,
    // writes it 128-byte-swizzled into its own staging tile and lane 0 hands that tile to a TMA
    // store (full-line writes, rows and columns past the matrix edge clipped by the tensor map).
    // The residual operand arrives the same way (TMA load into the staging tile, combined in
    // place).  fp32 results are rare (final projections) and use plain 16-byte stores.
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
    const int ew = warp - 2;                      // epilogue warp index 0..7
    const int half = ew >> 2;                     // which 128 accumulator columns it handles
    uint8_t* stage = staging + ew * kStoreBytes;
    const uint32_t stage_row = smem_u32(stage) + lane * 128;
    const int swz = lane & 7;
    uint32_t tile_it = 0, res_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const TileInfo ti = tile_info<kGather>(tile, m_tiles, n_tiles, k_blocks, p);
      if (ti.skip) continue;
      const uint32_t buf = tile_it & 1u;
      const int m0 = ti.m0, n0 = ti.n0;
      const __nv_bfloat16* bias_t = p.bias ? p.bias + ti.bias_off : nullptr;
      if (!mbar_wait(&acc_full[buf], (tile_it >> 1) & 1u, abort_flag)) { ok = false; break; }
      tmem_fence_after();
      const int row0 = m0 + quarter * 32;
      const int row = row0 + lane;
      const bool row_ok = row < p.m;
      // grouped weight gradients: a 32-row piece past the expert's matrix would land in the next one
      const bool piece_ok = p.grp_mode != 2 || row0 < p.m;
      const int64_t gate_row = p.gate ? ((row_ok ? row : 0) / p.rows_per_gate) : 0;
#pragma unroll 1
      for (int cc = 0; cc < 2 && ok; ++cc) {
        const int colbase = n0 + half * 128 + cc * 64;
        if (colbase >= p.n) break;                // warp-uniform
        const uint32_t taddr =
            tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + half * 128 + cc * 64;
        if (!piece_ok) break;                     // warp-uniform
        uint32_t r[64];
        tmem_ld32(taddr, r);
        tmem_ld32(taddr + 32, r + 32);
        if (!p.out_fp32) {
          if (lane == 0) {
            tma_store_wait_read();                // the previous store has drained this tile
            if (p.residual) {
              mbar_expect_tx(&res_full[ew], kStoreBytes);
              tma_load_2d(stage, &map_r, &res_full[ew], colbase, row0);
            }
          }
          __syncwarp();
          if (p.residual) {
            if (!mbar_wait(&res_full[ew], res_it & 1u, abort_flag)) { ok = false; }
            ++res_it;
          }
        }
        tmem_ld_wait();
        if (!ok) break;
        if (ti.kbn == 0) {
          // an expert without rows: no product was issued, the accumulator columns hold old data
#pragma unroll
          for (int i = 0; i < 64; ++i) r[i] = 0u;
        }
        if (p.lse_mode == 1) {
          // one thread holds 64 consecutive logits of one row: fold them here, store 8 bytes
          const int t = row_ok ? (int)(p.lse_ids[row] - p.lse_col0 - colbase) : -1;
          float mx = -INFINITY;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int col = colbase + g * 8;
            float b[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) b[j] = 0.f;
            if (bias_t && col < p.n) unpack8(*reinterpret_cast<const bf16x8*>(bias_t + col), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float sv = (__uint_as_float(r[g * 8 + j]) + b[j]) * p.lse_inv_t;
              if (col >= p.n) sv = -INFINITY;
              r[g * 8 + j] = __float_as_uint(sv);
              mx = fmaxf(mx, sv);
            }
          }
          float sum = 0.f, tgt = 0.f;
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float sv = __uint_as_float(r[i]);
            sum += __expf(sv - mx);
            if (i == t) tgt = sv;
          }
          if (row_ok) {
            const int64_t slot = (int64_t)(colbase >> 6) * p.m + row;
            p.lse_part_max[slot] = mx;
            p.lse_part_sum[slot] = sum;
            if (t >= 0 && t < 64) p.lse_target[row] = tgt;
          }
          continue;
        }
        const float lse_r = (p.lse_mode == 2 && row_ok) ? p.lse_lse[row] : 0.f;
        const float lse_gs = (p.lse_mode == 2 && row_ok) ? p.lse_g[row] * p.lse_inv_t : 0.f;
        const int lse_id = (p.lse_mode == 2 && row_ok) ? (int)(p.lse_ids[row] - p.lse_col0) : -1;
        if (p.dual) {
          // first output: the pre-activation values, kept for the backward pass of the activation
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const int col = colbase + g * 8;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]);
            if (bias_t && col < p.n) {
              float b[8];
              unpack8(*reinterpret_cast<const bf16x8*>(bias_t + col), b);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] += b[j];
            }
            const bf16x8 o = pack8(v);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                             stage_row + ((uint32_t)(g ^ swz) << 4)),
                         "r"(o.u.x), "r"(o.u.y), "r"(o.u.z), "r"(o.u.w)
                         : "memory");
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(stage, &map_c2, colbase, row0 + ti.c_row_off);
            tma_store_wait_read();
          }
          __syncwarp();
        }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int col = colbase + g * 8;
          const bool col_ok = col < p.n;
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]);
          if (bias_t && col_ok) {
            float b[8];
            unpack8(*reinterpret_cast<const bf16x8*>(bias_t + col), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += b[j];
          }
          if (p.lse_mode == 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              v[j] = lse_gs * ((col + j == lse_id ? 1.f : 0.f) - __expf(v[j] * p.lse_inv_t - lse_r));
          }
          if (p.act == 1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
          } else if (p.act == 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = silu(v[j]);
          }
          const uint32_t saddr = stage_row + ((uint32_t)(g ^ swz) << 4);
          if (p.residual) {
            float rs[8];
            if (!p.out_fp32) {
              bf16x8 t;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(t.u.x), "=r"(t.u.y), "=r"(t.u.z), "=r"(t.u.w)
                           : "r"(saddr));
              unpack8(t, rs);
            } else if (row_ok && col_ok) {
              unpack8(*reinterpret_cast<const bf16x8*>(p.residual + (int64_t)row * p.n + col), rs);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) rs[j] = 0.f;
            }
            if (p.act == 3) {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] *= gelu_tanh_grad(rs[j]);
            } else if (p.gate) {
              float gt[8];
              if (col_ok) {
                unpack8(*reinterpret_cast<const bf16x8*>(p.gate + gate_row * p.gate_ld + col), gt);
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) gt[j] = 0.f;
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = rs[j] + gt[j] * v[j];
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] += rs[j];
            }
          }
          if (p.out_fp32) {
            if (row_ok && col_ok) {
              float* dst = reinterpret_cast<float*>(p.c) + (int64_t)row * p.n + col;
              *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
              *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
          } else {
            const bf16x8 o = pack8(v);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(o.u.x),
                         "r"(o.u.y), "r"(o.u.z), "r"(o.u.w)
                         : "memory");
          }
        }
        if (!p.out_fp32) {
          fence_async_smem();                     // generic-proxy writes -> visible to the TMA unit
          __syncwarp();
          if (lane == 0) tma_store_2d(stage, &map_c, colbase, row0 + ti.c_row_off);
        }
      }
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      ++tile_it;
    }
    if (lane == 0) tma_store_wait_all();          // staging must outlive the stores reading it
    if (!ok && lane == 0) {
      if (atomicCAS(const_cast<int*>(abort_flag), 0, 1) == 0) atomicExch(p.status, kTimeoutEpilogue);
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

static EncodeFn lookup_encode_fn() {
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult q;
  C10_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q));
  TORCH_CHECK(ptr != nullptr && q == cudaDriverEntryPointSuccess,
              "cuTensorMapEncodeTiled is not available from this driver");
  return reinterpret_cast<EncodeFn>(ptr);
}

static EncodeFn encode_fn() {
  static EncodeFn fn = lookup_encode_fn();     // thread-safe function-local static
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows of pitch `pitch_elems`.
static CUtensorMap make_map(const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_elems,
                            uint32_t box_inner, uint32_t box_outer) {
  CUtensorMap map;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem[2] = {1, 1};
  CUresult rc = encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(rc == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)rc,
              " (base must be 16-byte aligned, pitch a multiple of 16 bytes)");
  return map;
}

// 3-D map of an MN-major operand stored [rows = k, mn] with pitch `pitch_elems`: (64 mn, k, mn / 64).
// One box of (64, BK, chunks) lands in shared memory as `chunks` consecutive [BK x 128-byte] blocks,
// the layout the MN-major descriptors expect, with ONE copy instruction: the producer thread's
// issue slots are the scarce resource of the pipeline, and a copy per 64-wide chunk (up to six per
// stage) ate into the latency the four stages can hide.  The chunk dimension has a smaller stride
// than the row dimension; where the driver's encoder refuses that, the caller keeps the 2-D maps.
static bool make_map_mn3(CUtensorMap* map, const void* base, uint64_t mn, uint64_t k, uint64_t pitch_elems,
                         uint32_t chunks) {
  static int supported = -1;                     // -1 unknown, 0 refused once, 1 accepted
  if (supported == 0 || mn % 64 != 0) return false;
  cuuint64_t dims[3] = {64, k, mn / 64};
  cuuint64_t strides[2] = {pitch_elems * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)BK, chunks};
  cuuint32_t elem[3] = {1, 1, 1};
  const CUresult rc = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                                  box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (supported < 0) supported = rc == CUDA_SUCCESS ? 1 : 0;
  return rc == CUDA_SUCCESS;
}

static int* status_word(int device) { return kernel_status_block(device) + kStatusGemm; }

}  // namespace gemm

// VRL_GEMM_MN3D=0 keeps the one-copy-per-chunk form of MN-major operands (a comparison switch).
static bool gemm_mn3_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("VRL_GEMM_MN3D");
    return v == nullptr || std::string(v) != "0";
  }();
  return on;
}

// All-gather fused into the GEMM: the B operand [N, K] is sharded by rows over `world` ranks.
// `peer_ptrs` (CPU int64) holds every rank's shard address as mapped into this process, `ready`
// is an int32 [world] scratch; the gathered rows land in the tensor passed as `b`.
struct GatherSpec {
  torch::Tensor peer_ptrs, ready;
  int64_t rank, world;
};

// Log-sum-exp epilogues of the vocabulary head (Params::lse_mode).
struct LseSpec {
  int mode;                              // 1 = partial (max, sum, target) per 64-column chunk; 2 = softmax gradient
  torch::Tensor ids;                     // int64 [M]
  int64_t col0;                          // global index of this product's first column
  double inv_t;
  torch::Tensor part_max, part_sum, target;   // mode 1
  torch::Tensor lse, g;                        // mode 2
};

// Grouped products (Params::grp_mode).  Mode 1: `b` is the 2-D view of the experts' stacked matrices
// and `tile_expert` maps every BM-row tile of `a` to its expert (negative = unused).  Mode 2: `a` and
// `b` are both [rows, *] and `offsets` [experts + 1] gives every expert's padded row range.
struct GroupSpec {
  int mode;
  int64_t experts;
  torch::Tensor table;                   // tile_expert (mode 1) or offsets (mode 2), int32
};

static std::vector<torch::Tensor> gemm_impl(torch::Tensor a, torch::Tensor b,
                                            c10::optional<torch::Tensor> bias,
                                            c10::optional<torch::Tensor> gate,
                                            c10::optional<torch::Tensor> residual, int64_t act,
                                            int64_t rows_per_gate, bool a_mn_major, bool b_mn_major,
                                            bool out_fp32, bool dual,
                                            c10::optional<torch::Tensor> out_given = c10::nullopt,
                                            const struct GatherSpec* gather = nullptr,
                                            const struct LseSpec* lse = nullptr,
                                            const struct GroupSpec* grp = nullptr);

torch::Tensor gemm_bf16(torch::Tensor a, torch::Tensor b, c10::optional<torch::Tensor> bias,
                        c10::optional<torch::Tensor> gate, c10::optional<torch::Tensor> residual,
                        int64_t act, int64_t rows_per_gate, bool a_mn_major, bool b_mn_major,
                        bool out_fp32) {
  return gemm_impl(a, b, bias, gate, residual, act, rows_per_gate, a_mn_major, b_mn_major, out_fp32,
                   false)[0];
}

// acc += op(a) op(b)^T in place (weight-gradient accumulation straight into the flat gradient buffer:
// the existing values come in through the residual path and leave through the same tile's store).
void gemm_bf16_acc(torch::Tensor a, torch::Tensor b, torch::Tensor acc, bool a_mn_major, bool b_mn_major) {
  TORCH_CHECK(acc.is_cuda() && acc.dim() == 2 && acc.scalar_type() == torch::kBFloat16 && acc.is_contiguous() &&
              reinterpret_cast<uintptr_t>(acc.data_ptr()) % 16 == 0, "gemm_bf16_acc: contiguous aligned bf16 target");
  gemm_impl(a, b, c10::nullopt, c10::nullopt, acc, 0, 0, a_mn_major, b_mn_major, false, false, acc);
}

// (activation(a b^T + bias), a b^T + bias): the second tensor is what the activation's backward needs.
std::vector<torch::Tensor> gemm_bf16_dual(torch::Tensor a, torch::Tensor b,
                                          c10::optional<torch::Tensor> bias, int64_t act) {
  return gemm_impl(a, b, bias, c10::nullopt, c10::nullopt, act, 0, false, false, false, true);
}

static std::vector<torch::Tensor> gemm_impl(torch::Tensor a, torch::Tensor b,
                                            c10::optional<torch::Tensor> bias,
                                            c10::optional<torch::Tensor> gate,
                                            c10::optional<torch::Tensor> residual, int64_t act,
                                            int64_t rows_per_gate, bool a_mn_major, bool b_mn_major,
                                            bool out_fp32, bool dual,
                                            c10::optional<torch::Tensor> out_given,
                                            const GatherSpec* gather, const LseSpec* lse, const GroupSpec* grp) {
  using namespace gemm;
  TORCH_CHECK(grp == nullptr || (gather == nullptr && lse == nullptr && !out_fp32 && !gate.has_value() &&
                                 !out_given.has_value()),
              "gemm_bf16: grouped products take bias, activation, dual output and the gelu-gradient residual only");
  const bool lse_partial = lse != nullptr && lse->mode == 1;
  TORCH_CHECK(lse == nullptr || (!gate.has_value() && !residual.has_value() && !dual && act == 0 &&
                                 gather == nullptr && !out_given.has_value() && !out_fp32),
              "gemm_bf16: the log-sum-exp epilogues take bias only");
  TORCH_CHECK(act >= 0 && act <= 3, "gemm_bf16: unknown epilogue activation");
  TORCH_CHECK(act != 3 || (residual.has_value() && !gate.has_value() && !out_fp32),
              "gemm_bf16: the gelu-gradient epilogue needs the pre-activation as `residual`");
  TORCH_CHECK(!dual || (!residual.has_value() && !out_fp32), "gemm_bf16: dual output excludes residual/fp32");
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2);
  TORCH_CHECK(a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1, "gemm_bf16: innermost dimension must be contiguous");
  VRL_CHECK_OPERAND(b, a);
  VRL_CHECK_OPERAND(bias, a);
  VRL_CHECK_OPERAND(gate, a);
  VRL_CHECK_OPERAND(residual, a);
  VRL_CHECK_OPERAND(out_given, a);
  const c10::cuda::CUDAGuard guard(a.device());
  // The tensor-map encoder is a driver entry point.  A thread that has made no runtime call yet
  // (a fresh autograd worker) has no context bound, so bind the primary context once per thread.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    C10_CUDA_CHECK(cudaFree(nullptr));
    context_bound = true;
  }
  // logical sizes: A is [M, K] (or stored [K, M] when MN-major), B is [N, K] (or stored [K, N])
  const int64_t m = a_mn_major ? a.size(1) : a.size(0);
  const int64_t k = a_mn_major ? a.size(0) : a.size(1);
  int64_t n = b_mn_major ? b.size(1) : b.size(0);
  int64_t kb = b_mn_major ? b.size(0) : b.size(1);
  const int64_t experts = grp != nullptr ? grp->experts : 1;
  if (grp != nullptr && grp->mode == 1) {
    // b is the stack of the experts' matrices: [E * N, K] (K-major) or [E * K, N] (row-major)
    if (b_mn_major) { TORCH_CHECK(kb % experts == 0); kb /= experts; }
    else { TORCH_CHECK(n % experts == 0); n /= experts; }
  }
  TORCH_CHECK(k == kb, "gemm_bf16: contraction sizes differ: ", k, " vs ", kb);
  TORCH_CHECK(n % 8 == 0, "gemm_bf16: N must be a multiple of 8");
  TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "gemm_bf16: row pitch must be a multiple of 8");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 &&
              reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0, "gemm_bf16: 16-byte alignment");
  torch::Tensor out;
  if (out_given.has_value()) {
    out = *out_given;
    TORCH_CHECK(!out_fp32 && out.size(0) == m && out.size(1) == n, "gemm_bf16: output shape mismatch");
  } else if (lse_partial) {
    out = torch::empty({0}, a.options());      // this epilogue stores no product
  } else if (grp != nullptr && grp->mode == 2) {
    out = torch::empty({experts * m, n}, a.options());
  } else {
    out = torch::empty({m, n}, a.options().dtype(out_fp32 ? torch::kFloat32 : torch::kBFloat16));
  }
  torch::Tensor pre = dual ? torch::empty({m, n}, a.options()) : torch::Tensor();
  if (m == 0 || n == 0) return {out, pre};
  if (grp != nullptr && grp->mode == 2 && k == 0) { out.zero_(); return {out, pre}; }
  TORCH_CHECK(k > 0, "gemm_bf16: empty contraction");

  // grouped mode 1: B's outer extent covers every expert's matrix
  const int64_t b_outer = (grp != nullptr && grp->mode == 1) ? experts : 1;
  CUtensorMap map_a, map_b;
  const bool use_mn3 = gemm_mn3_enabled();
  const bool a_mn3 = a_mn_major && use_mn3 && make_map_mn3(&map_a, a.data_ptr(), m, k, a.stride(0), BM / 64);
  const bool b_mn3 = b_mn_major && use_mn3 && make_map_mn3(&map_b, b.data_ptr(), n, k * b_outer, b.stride(0), BN / 64);
  if (!a_mn3)
    map_a = a_mn_major ? make_map(a.data_ptr(), m, k, a.stride(0), 64, BK)
                       : make_map(a.data_ptr(), k, m, a.stride(0), BK, BM);
  if (!b_mn3)
    map_b = b_mn_major ? make_map(b.data_ptr(), n, k * b_outer, b.stride(0), 64, BK)
                       : make_map(b.data_ptr(), k, n * b_outer, b.stride(0), BK, BN);
  Params p{};
  p.a_mn3 = a_mn3 ? 1 : 0;
  p.b_mn3 = b_mn3 ? 1 : 0;
  p.c = out.data_ptr();
  torch::Tensor bias_c, gate_c, res_c;
  if (bias.has_value()) {
    bias_c = bias->to(torch::kBFloat16).contiguous();
    TORCH_CHECK(bias_c.numel() == n * ((grp != nullptr && grp->mode == 1) ? experts : 1));
    p.bias = reinterpret_cast<const __nv_bfloat16*>(bias_c.data_ptr());
  }
  if (gate.has_value()) {
    TORCH_CHECK(residual.has_value() && rows_per_gate > 0, "gate needs residual and rows_per_gate");
    gate_c = *gate;
    const bool strided_ok = gate_c.dim() == 2 && gate_c.scalar_type() == torch::kBFloat16 &&
                            gate_c.stride(1) == 1 && gate_c.stride(0) % 8 == 0 &&
                            reinterpret_cast<uintptr_t>(gate_c.data_ptr()) % 16 == 0;
    if (!strided_ok) gate_c = gate_c.to(torch::kBFloat16).contiguous().view({-1, n});
    TORCH_CHECK(gate_c.size(0) == m / rows_per_gate && gate_c.size(1) == n && m % rows_per_gate == 0,
                "gate must be [M / rows_per_gate, N]");
    p.gate = reinterpret_cast<const __nv_bfloat16*>(gate_c.data_ptr());
    p.gate_ld = gate_c.stride(0);
  }
  if (residual.has_value()) {
    res_c = residual->to(torch::kBFloat16).contiguous();
    TORCH_CHECK(res_c.numel() == m * n);
    if (reinterpret_cast<uintptr_t>(res_c.data_ptr()) % 16 != 0) {
      TORCH_CHECK(!out_given.has_value(), "gemm_bf16: in-place accumulation needs a 16-byte aligned target");
      res_c = res_c.clone();
    }
    p.residual = reinterpret_cast<const __nv_bfloat16*>(res_c.data_ptr());
  }
  p.status = status_word(a.get_device());
  p.m = (int)m; p.n = (int)n; p.k = (int)k;
  p.act = (int)act;
  p.rows_per_gate = (int)std::max<int64_t>(rows_per_gate, 1);
  p.a_mn = a_mn_major ? 1 : 0;
  p.b_mn = b_mn_major ? 1 : 0;
  p.out_fp32 = out_fp32 ? 1 : 0;
  p.dual = dual ? 1 : 0;
  if (grp != nullptr) {
    TORCH_CHECK(experts >= 1 && grp->table.is_contiguous(), "gemm_bf16: grouped table");
    p.grp_mode = grp->mode;
    p.grp_experts = (int)experts;
    if (grp->mode == 1) {
      TORCH_CHECK(!a_mn_major && m % BM == 0, "grouped product: rows padded to the tile height, K-major activations");
      VRL_CHECK_OPERAND(grp->table, a, torch::kInt32, m / BM);
      p.grp_tile_expert = grp->table.data_ptr<int>();
      p.grp_stride = (int)(b_mn_major ? k : n);
    } else {
      TORCH_CHECK(a_mn_major && b_mn_major && k % BM == 0 && m % 32 == 0 && !bias.has_value() &&
                  !residual.has_value() && !dual && act == 0,
                  "grouped weight gradient: row-major operands over padded rows, output rows a multiple of 32");
      VRL_CHECK_OPERAND(grp->table, a, torch::kInt32, experts + 1);
      p.grp_offsets = grp->table.data_ptr<int>();
    }
  }
  if (lse != nullptr) {
    const int64_t chunks = (n + 63) / 64;
    VRL_CHECK_OPERAND(lse->ids, a, torch::kInt64, m);
    p.lse_mode = lse->mode;
    p.lse_ids = lse->ids.data_ptr<int64_t>();
    p.lse_col0 = lse->col0;
    p.lse_inv_t = (float)lse->inv_t;
    if (lse_partial) {
      VRL_CHECK_OPERAND(lse->part_max, a, torch::kFloat32, chunks * m);
      VRL_CHECK_OPERAND(lse->part_sum, a, torch::kFloat32, chunks * m);
      VRL_CHECK_OPERAND(lse->target, a, torch::kFloat32, m);
      p.lse_part_max = lse->part_max.data_ptr<float>();
      p.lse_part_sum = lse->part_sum.data_ptr<float>();
      p.lse_target = lse->target.data_ptr<float>();
      p.out_fp32 = 1;                           // no staging tile, no TMA store
    } else {
      VRL_CHECK_OPERAND(lse->lse, a, torch::kFloat32, m);
      VRL_CHECK_OPERAND(lse->g, a, torch::kFloat32, m);
      p.lse_lse = lse->lse.data_ptr<float>();
      p.lse_g = lse->g.data_ptr<float>();
    }
  }

  static const bool attr_set = [] {
    C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        kSmemBytes));
    C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        kSmemBytes));
    return true;
  }();
  (void)attr_set;
  const int tiles = (int)(((m + BM - 1) / BM) * ((n + BN - 1) / BN) * ((grp != nullptr && grp->mode == 2) ? experts : 1));
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  // output / residual maps: 64-column x 32-row boxes matching one epilogue warp's staging tile
  const int64_t c_rows = (grp != nullptr && grp->mode == 2) ? experts * m : m;
  CUtensorMap map_c = (out_fp32 || lse_partial) ? map_a : make_map(out.data_ptr(), n, c_rows, n, 64, 32);
  CUtensorMap map_r = (p.residual && !out_fp32) ? make_map(p.residual, n, m, n, 64, 32) : map_c;
  CUtensorMap map_c2 = dual ? make_map(pre.data_ptr(), n, m, n, 64, 32) : map_c;
  auto stream = at::cuda::getCurrentCUDAStream();
  if (gather != nullptr) {
    const int64_t world = gather->world, rank = gather->rank;
    TORCH_CHECK(!a_mn_major && !b_mn_major && b.is_contiguous(),
                "gemm_allgather: K-major operands, contiguous gathered weight");
    TORCH_CHECK(world >= 1 && world <= 16 && rank >= 0 && rank < world && n % world == 0 && k % 8 == 0 &&
                ((n / world) * k) % 8 == 0, "gemm_allgather: rows must divide evenly into 16-byte aligned shards");
    TORCH_CHECK(gather->peer_ptrs.device().is_cpu() && gather->peer_ptrs.scalar_type() == torch::kInt64 &&
                gather->peer_ptrs.numel() == world, "peer_ptrs: CPU int64 tensor with one address per rank");
    VRL_CHECK_OPERAND(gather->ready, a, torch::kInt32);
    TORCH_CHECK(gather->ready.numel() >= world && gather->ready.is_contiguous());
    const int64_t* ptrs = gather->peer_ptrs.data_ptr<int64_t>();
    for (int r = 0; r < world; ++r) {
      TORCH_CHECK(ptrs[r] != 0 && ptrs[r] % 16 == 0, "gemm_allgather: shard addresses must be 16-byte aligned");
      p.g_peer[r] = reinterpret_cast<const __nv_bfloat16*>(ptrs[r]);
    }
    p.g_full = reinterpret_cast<__nv_bfloat16*>(b.data_ptr());
    p.g_ready = gather->ready.data_ptr<int>();
    p.g_world = (int)world; p.g_rank = (int)rank; p.g_rows = (int)(n / world);
    p.g_first_tile = (int)((rank * (n / world)) / BN);
    // a band's A rows (g_band * BM * K bf16) stay within a quarter of the L2
    const int64_t m_tiles_h = (m + BM - 1) / BM;
    const int64_t band = (32ll << 20) / ((int64_t)BM * k * 2);
    p.g_band = (int)std::max<int64_t>(1, std::min<int64_t>(m_tiles_h, band));
    C10_CUDA_CHECK(cudaMemsetAsync(p.g_ready, 0, sizeof(int) * world, stream));
    // One CTA per SM, all resident (the producers wait for every CTA's share of the gather), and
    // ALL of them even when the product has fewer tiles: the copy wants every SM's load slots.
    gemm_bf16_kernel<true><<<sms, kThreads + kGatherThreads, kSmemBytes, stream>>>(map_a, map_b, map_c, map_r,
                                                                                  map_c2, p);
  } else {
    const int grid = std::min(tiles, sms);
    gemm_bf16_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, map_c, map_r, map_c2, p);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {out, pre};
}

// op(a) op(b)^T written into a caller-provided bf16 [M, N] tensor (the weight-gradient staging
// buffers of sharded training are filled this way).
void gemm_bf16_out(torch::Tensor a, torch::Tensor b, torch::Tensor out, bool a_mn_major, bool b_mn_major) {
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.scalar_type() == torch::kBFloat16 && out.is_contiguous() &&
              reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0, "gemm_bf16_out: contiguous aligned bf16 target");
  gemm_impl(a, b, c10::nullopt, c10::nullopt, c10::nullopt, 0, 0, a_mn_major, b_mn_major, false, false, out);
}

// epilogue(x W^T + bias) where W [N, K] is sharded by rows over `world` ranks.  `peer_ptrs` holds the
// address of every rank's shard [N / world, K] as mapped into THIS process (own shard included),
// `full` is a local [N, K] buffer the kernel gathers the shards into while it computes (and that the
// caller may reuse afterwards, e.g. for dX = dY W), `ready` an int32 [world] scratch.  All ranks'
// shards must be final before the launch.  Returns {y} or, with `dual`, {act(y), y}.
std::vector<torch::Tensor> gemm_allgather(torch::Tensor x, torch::Tensor peer_ptrs, torch::Tensor full,
                                          torch::Tensor ready, c10::optional<torch::Tensor> bias, int64_t act,
                                          int64_t rank, int64_t world, c10::optional<torch::Tensor> gate,
                                          c10::optional<torch::Tensor> residual, int64_t rows_per_gate,
                                          bool dual) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.stride(1) == 1);
  TORCH_CHECK(full.is_cuda() && full.dim() == 2 && full.scalar_type() == torch::kBFloat16 && full.is_contiguous());
  TORCH_CHECK(act >= 0 && act <= 2, "gemm_allgather: activation none / gelu-tanh / silu");
  TORCH_CHECK(x.size(0) > 0, "gemm_allgather: empty activation (the gather would not run)");
  const GatherSpec spec{peer_ptrs, ready, rank, world};
  auto outs = gemm_impl(x, full, bias, gate, residual, act, rows_per_gate, false, false, false, dual,
                        c10::nullopt, &spec);
  if (!dual) outs.resize(1);
  return outs;
}

// ---------------------------------------------------------------------------- grouped products
// epilogue(a[r, :] W_e^T + bias_e) for rows sorted by expert, every expert's run padded to 128 rows.
// `w` is [E, N, K] (or, `w_row_major`, [E, K, N]: the input-gradient form), `tile_expert` int32
// [rows / 128].  Returns {y} or, with `dual`, {act(y), y}; `residual` with act 3 is the
// gelu-gradient epilogue.  No value is read on the host: the launch is the same for any routing.
std::vector<torch::Tensor> gemm_grouped(torch::Tensor a, torch::Tensor w, torch::Tensor tile_expert,
                                        c10::optional<torch::Tensor> bias, c10::optional<torch::Tensor> residual,
                                        int64_t act, bool w_row_major, bool dual) {
  TORCH_CHECK(a.is_cuda() && a.dim() == 2 && w.dim() == 3 && w.is_contiguous() && a.is_contiguous(),
              "gemm_grouped: a [rows, K] and w [E, N, K] contiguous");
  const int64_t experts = w.size(0);
  const GroupSpec spec{1, experts, tile_expert};
  auto outs = gemm_impl(a, w.view({experts * w.size(1), w.size(2)}), bias, c10::nullopt, residual, act, 0, false,
                        w_row_major, false, dual, c10::nullopt, nullptr, nullptr, &spec);
  if (!dual) outs.resize(1);
  return outs;
}

// dW_e = gy[rows of e]^T x[rows of e] for every expert: [E, N, K] from gy [rows, N], x [rows, K] and the
// experts' padded row offsets (int32 [E + 1], multiples of 128).  Rows of padding must be zero in `gy`.
torch::Tensor gemm_grouped_wgrad(torch::Tensor gy, torch::Tensor x, torch::Tensor offsets, int64_t experts) {
  TORCH_CHECK(gy.is_cuda() && gy.dim() == 2 && x.dim() == 2 && gy.size(0) == x.size(0) && gy.is_contiguous() &&
              x.is_contiguous(), "gemm_grouped_wgrad: gy [rows, N], x [rows, K] contiguous");
  const GroupSpec spec{2, experts, offsets};
  auto out = gemm_impl(gy, x, c10::nullopt, c10::nullopt, c10::nullopt, 0, 0, true, true, false, false, c10::nullopt,
                       nullptr, nullptr, &spec)[0];
  return out.view({experts, gy.size(1), x.size(1)});
}

// ------------------------------------------------------------- vocabulary head with log-sum-exp
namespace gemm {

// One thread per row: fold the per-chunk (max, sum) pairs into the row's log-sum-exp and finish
// the target's log-probability.
__global__ void lse_merge_kernel(const float* __restrict__ part_max, const float* __restrict__ part_sum,
                                 const float* __restrict__ target, int chunks, int m, float* __restrict__ logp,
                                 float* __restrict__ lse) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= m) return;
  float mx = -INFINITY;
  for (int c = 0; c < chunks; ++c) mx = fmaxf(mx, part_max[(int64_t)c * m + row]);
  float sum = 0.f;
  for (int c = 0; c < chunks; ++c)
    sum += part_sum[(int64_t)c * m + row] * __expf(part_max[(int64_t)c * m + row] - mx);
  const float l = mx + logf(sum);
  lse[row] = l;
  logp[row] = target[row] - l;
}

}  // namespace gemm

static void check_head_operands(const torch::Tensor& h, const torch::Tensor& w, const torch::Tensor& ids) {
  TORCH_CHECK(h.is_cuda() && h.dim() == 2 && h.scalar_type() == torch::kBFloat16 && h.is_contiguous(),
              "head log-probs: hidden must be a contiguous bf16 [rows, dim] CUDA tensor");
  TORCH_CHECK(w.dim() == 2 && w.scalar_type() == torch::kBFloat16 && w.is_contiguous() && w.size(1) == h.size(1),
              "head log-probs: weight must be contiguous bf16 [vocab, dim]");
  TORCH_CHECK(ids.dim() == 1 && ids.is_contiguous() && ids.size(0) == h.size(0), "head log-probs: ids must be [rows]");
}

// log_softmax((h W^T + bias) / T)[ids] and the row log-sum-exp, with the fold over the vocabulary
// done in the product's epilogue: what reaches memory per row is 8 bytes per 64 vocabulary
// columns instead of 256 bytes of fp32 logits.  Ids outside [0, vocab) are the caller's error.
std::vector<torch::Tensor> head_logprob_fwd(torch::Tensor h, torch::Tensor w, c10::optional<torch::Tensor> bias,
                                            torch::Tensor ids, double temperature) {
  check_head_operands(h, w, ids);
  TORCH_CHECK(temperature > 0, "head log-probs: temperature must be positive");
  const int64_t m = h.size(0), n = w.size(0), chunks = (n + 63) / 64;
  auto f32 = h.options().dtype(torch::kFloat32);
  torch::Tensor logp = torch::empty({m}, f32), lse = torch::empty({m}, f32);
  if (m == 0) return {logp, lse};
  LseSpec spec{1, ids, 0, 1.0 / temperature, torch::empty({chunks, m}, f32), torch::empty({chunks, m}, f32),
               torch::zeros({m}, f32), torch::Tensor(), torch::Tensor()};
  gemm_impl(h, w, bias, c10::nullopt, c10::nullopt, 0, 0, false, false, false, false, c10::nullopt, nullptr, &spec);
  const c10::cuda::CUDAGuard guard(h.device());
  gemm::lse_merge_kernel<<<(unsigned)((m + 127) / 128), 128, 0, at::cuda::getCurrentCUDAStream()>>>(
      spec.part_max.data_ptr<float>(), spec.part_sum.data_ptr<float>(), spec.target.data_ptr<float>(), (int)chunks,
      (int)m, logp.data_ptr<float>(), lse.data_ptr<float>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {logp, lse};
}

// d logits = g / T * (onehot(ids) - softmax) for the vocabulary slice [col0, col0 + w.size(0)), as bf16,
// produced in the epilogue of the recomputed product (no fp32 logits in memory).
torch::Tensor head_softmax_grad(torch::Tensor h, torch::Tensor w, c10::optional<torch::Tensor> bias,
                                torch::Tensor ids, torch::Tensor lse, torch::Tensor g, int64_t col0,
                                double temperature) {
  check_head_operands(h, w, ids);
  TORCH_CHECK(lse.is_contiguous() && g.is_contiguous(), "head_softmax_grad: contiguous lse and g");
  TORCH_CHECK(temperature > 0, "head_softmax_grad: temperature must be positive");
  LseSpec spec{2, ids, col0, 1.0 / temperature, torch::Tensor(), torch::Tensor(), torch::Tensor(), lse, g};
  return gemm_impl(h, w, bias, c10::nullopt, c10::nullopt, 0, 0, false, false, false, false, c10::nullopt, nullptr,
                   &spec)[0];
}

}  // namespace vrl
