// Normalisation kernels (K3/K4): adaLN-modulated LayerNorm, RMSNorm and the fused QKV
// post-processing (head split + per-head or full-width RMS norm of q/k + rotary embedding),
// forward and backward.  One thread block handles one token row (forward) or a short run of
// rows (backward, so per-column parameter gradients are accumulated in registers / shared
// memory before touching global atomics).  Statistics are fp32; data is bf16.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "ops.h"

namespace vrl {

constexpr int kNormThreads = 256;
constexpr int kMaxVec = 4;          // vectors of 8 per thread  => D <= 8192
constexpr int kBwdRows = 16;

using bf16 = __nv_bfloat16;

// A [B, D] bf16 operand whose rows may sit `stride(0)` apart (a column slice of a wider
// modulation tensor); copied only when it is not row-strided with 16-byte aligned rows.
static torch::Tensor strided_rows(torch::Tensor t, int64_t b, int64_t d) {
  TORCH_CHECK(t.dim() == 2 && t.size(0) == b && t.size(1) == d, "expected a [B, D] tensor");
  const bool ok = t.scalar_type() == torch::kBFloat16 && t.stride(1) == 1 && t.stride(0) % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0;
  return ok ? t : t.to(torch::kBFloat16).contiguous();
}


// ------------------------------------------------------------------ warp-per-row variants
// For D <= 2048 one warp owns a whole row: lane l holds vectors l, l+32, ... (512 contiguous
// bytes per warp-wide load), statistics are warp shuffles, and no block barrier is needed, so
// many rows are in flight per SM.  Rows stay packed (bf16) in registers between the passes.
constexpr int kRowWarps = 8;

template <int VPL>
__global__ void __launch_bounds__(kRowWarps * 32)
adaln_fwd_warp_kernel(const bf16* __restrict__ x, const bf16* __restrict__ shift,
                      const bf16* __restrict__ scale, bf16* __restrict__ y, float* __restrict__ mean_o,
                      float* __restrict__ rstd_o, int64_t rows, int rows_per_sample, int d, float eps,
                      int64_t shift_ld, int64_t scale_ld) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kRowWarps + warp;
  if (row >= rows) return;
  const int nvec = d / 8;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * d);
  bf16x8 raw[VPL];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int i = lane + k * 32;
    if (i < nvec) {
      raw[k] = xr[i];
      float f[8];
      unpack8(raw[k], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += f[j];
    }
  }
  const float mu = warp_sum(s) / (float)d;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    if (lane + k * 32 < nvec) {
      float f[8];
      unpack8(raw[k], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float c = f[j] - mu; q += c * c; }
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / (float)d + eps);
  if (lane == 0) { mean_o[row] = mu; rstd_o[row] = rstd; }
  const int sample = (int)(row / rows_per_sample);
  const bf16x8* sh = reinterpret_cast<const bf16x8*>(shift + (int64_t)sample * shift_ld);
  const bf16x8* sc = reinterpret_cast<const bf16x8*>(scale + (int64_t)sample * scale_ld);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * d);
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int i = lane + k * 32;
    if (i < nvec) {
      float f[8], a[8], b[8], o[8];
      unpack8(raw[k], f);
      unpack8(sh[i], a);
      unpack8(sc[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (f[j] - mu) * rstd * (1.f + b[j]) + a[j];
      yr[i] = pack8(o);
    }
  }
}

// Backward: a block of 8 warps covers `kAdaBlockRows` rows of ONE sample, 16 rows per warp.  Each
// lane keeps the per-column sums for d(shift) and d(scale) of its own columns in registers over
// those rows, adds them to a shared-memory copy once, and the block flushes that copy to global
// memory with one atomic per column.
constexpr int kAdaBlockRows = 128;

template <int VPL>
__global__ void __launch_bounds__(kRowWarps * 32)
adaln_bwd_warp_kernel(const bf16* __restrict__ gy, const bf16* __restrict__ x,
                      const bf16* __restrict__ scale, const float* __restrict__ mean,
                      const float* __restrict__ rstd, bf16* __restrict__ gx, float* __restrict__ gshift,
                      float* __restrict__ gscale, int rows_per_sample, int d, int64_t scale_ld) {
  extern __shared__ float col_acc[];         // [2][d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sample = blockIdx.y;
  const int nvec = d / 8;
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) col_acc[i] = 0.f;
  __syncthreads();
  const bf16x8* sc = reinterpret_cast<const bf16x8*>(scale + (int64_t)sample * scale_ld);
  float acc_sh[VPL][8], acc_sc[VPL][8];
#pragma unroll
  for (int k = 0; k < VPL; ++k)
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc_sh[k][j] = 0.f; acc_sc[k][j] = 0.f; }
  const int r_begin = blockIdx.x * kAdaBlockRows;
  for (int r = r_begin + warp; r < r_begin + kAdaBlockRows && r < rows_per_sample; r += kRowWarps) {
    const int64_t row = (int64_t)sample * rows_per_sample + r;
    const float mu = mean[row], rs = rstd[row];
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * d);
    const bf16x8* gr = reinterpret_cast<const bf16x8*>(gy + row * d);
    bf16x8 xraw[VPL], graw[VPL];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int i = lane + k * 32;
      if (i < nvec) {
        xraw[k] = xr[i];
        graw[k] = gr[i];
      }
    }
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int i = lane + k * 32;
      if (i < nvec) {
        float xv[8], gv[8], t[8];
        unpack8(xraw[k], xv);
        unpack8(graw[k], gv);
        unpack8(sc[i], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mu) * rs;
          const float gp = gv[j] * (1.f + t[j]);
          s1 += gp;
          s2 += gp * xh;
          acc_sh[k][j] += gv[j];
          acc_sc[k][j] += gv[j] * xh;
        }
      }
    }
    const float m1 = warp_sum(s1) / (float)d;
    const float m2 = warp_sum(s2) / (float)d;
    bf16x8* gxr = reinterpret_cast<bf16x8*>(gx + row * d);
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int i = lane + k * 32;
      if (i < nvec) {
        float xv[8], gv[8], t[8], o[8];
        unpack8(xraw[k], xv);
        unpack8(graw[k], gv);
        unpack8(sc[i], t);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mu) * rs;
          o[j] = rs * (gv[j] * (1.f + t[j]) - m1 - xh * m2);
        }
        gxr[i] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int i = lane + k * 32;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        atomicAdd(&col_acc[i * 8 + j], acc_sh[k][j]);
        atomicAdd(&col_acc[d + i * 8 + j], acc_sc[k][j]);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    atomicAdd(gshift + (int64_t)sample * d + i, col_acc[i]);
    atomicAdd(gscale + (int64_t)sample * d + i, col_acc[d + i]);
  }
}

template <int VPL>
__global__ void __launch_bounds__(kRowWarps * 32)
rmsnorm_fwd_warp_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                        float* __restrict__ rstd_o, int64_t rows, int d, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kRowWarps + warp;
  if (row >= rows) return;
  const int nvec = d / 8;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * d);
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8 raw[VPL];
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int i = lane + k * 32;
    if (i < nvec) {
      raw[k] = xr[i];
      float f[8];
      unpack8(raw[k], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) q += f[j] * f[j];
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / (float)d + eps);
  if (lane == 0) rstd_o[row] = rstd;
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * d);
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int i = lane + k * 32;
    if (i < nvec) {
      float f[8], ww[8], o[8];
      unpack8(raw[k], f);
      unpack8(wr[i], ww);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = f[j] * rstd * ww[j];
      yr[i] = pack8(o);
    }
  }
}

// Calls `fn.template operator()<VPL>()` with the smallest VPL in {2, 4, 6, 8} covering nvec / 32.
#define VRL_DISPATCH_VPL(nvec, ...)                     \
  do {                                                  \
    const int vpl_needed = ((nvec) + 31) / 32;          \
    if (vpl_needed <= 2) { constexpr int VPL = 2; __VA_ARGS__; }        \
    else if (vpl_needed <= 4) { constexpr int VPL = 4; __VA_ARGS__; }   \
    else if (vpl_needed <= 6) { constexpr int VPL = 6; __VA_ARGS__; }   \
    else { constexpr int VPL = 8; __VA_ARGS__; }                        \
  } while (0)

// ----------------------------------------------------------------- column-owner variants
// One thread owns ONE 8-column vector of the row (block = D / 8 threads rounded up to a warp) and
// walks over a run of rows, RB rows per pass: RB independent 16-byte loads per operand are in
// flight per thread, row statistics are block sums of RB values at a time (one barrier per RB rows),
// and a per-column gradient sum is 8 registers per thread instead of a whole row's worth per
// lane.  The register count stays low enough for several blocks per SM, which is what a
// bandwidth-bound pass needs.
constexpr int kColsRowsPerPass = 4;

__device__ __forceinline__ void red_add_v4(float* addr, const float* v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]),
               "f"(v[3])
               : "memory");
}

// Block-wide sums of NV values per thread, result in every thread.  `red` holds 32 * NV floats and
// must not be reused before the next barrier of the block (callers alternate two buffers).
template <int NV>
__device__ __forceinline__ void block_sum_vals(float (&v)[NV], float* red, int nwarps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int q = 0; q < NV; ++q) v[q] = warp_sum(v[q]);
  if (lane == 0) {
#pragma unroll
    for (int q = 0; q < NV; ++q) red[warp * NV + q] = v[q];
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < NV; ++q) {
    float t = 0.f;
    for (int w = 0; w < nwarps; ++w) t += red[w * NV + q];
    v[q] = t;
  }
}

// rows per block so that the grid has a few blocks per SM slot, in multiples of the pass size
static int cols_rows_per_block(int64_t total_rows, int rows_per_sample) {
  int64_t rpb = total_rows / (148 * 4);
  rpb = std::max<int64_t>(8, std::min<int64_t>(64, rpb));
  rpb = (rpb + kColsRowsPerPass - 1) / kColsRowsPerPass * kColsRowsPerPass;
  return (int)std::min<int64_t>(rpb, std::max(rows_per_sample, kColsRowsPerPass));
}

#define VRL_DISPATCH_COLS(threads, ...)                                  \
  do {                                                                   \
    if ((threads) <= 256) { constexpr int kMaxT = 256; __VA_ARGS__; }    \
    else if ((threads) <= 512) { constexpr int kMaxT = 512; __VA_ARGS__; } \
    else { constexpr int kMaxT = 1024; __VA_ARGS__; }                    \
  } while (0)

template <int kMaxT>
__global__ void __launch_bounds__(kMaxT)
adaln_fwd_cols_kernel(const bf16* __restrict__ x, const bf16* __restrict__ shift,
                      const bf16* __restrict__ scale, bf16* __restrict__ y, float* __restrict__ mean_o,
                      float* __restrict__ rstd_o, int rows_per_sample, int d, float eps, int64_t shift_ld,
                      int64_t scale_ld, int rows_per_block) {
  constexpr int RB = kColsRowsPerPass;
  __shared__ float red[2 * 32 * RB];
  const int i = threadIdx.x, nvec = d / 8, nwarps = blockDim.x >> 5;
  const bool act = i < nvec;
  const int sample = blockIdx.y;
  float sh[8], sc1[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { sh[j] = 0.f; sc1[j] = 1.f; }
  if (act) {
    float t[8];
    unpack8(reinterpret_cast<const bf16x8*>(shift + (int64_t)sample * shift_ld)[i], sh);
    unpack8(reinterpret_cast<const bf16x8*>(scale + (int64_t)sample * scale_ld)[i], t);
#pragma unroll
    for (int j = 0; j < 8; ++j) sc1[j] = 1.f + t[j];
  }
  const int r_begin = blockIdx.x * rows_per_block;
  const int r_end = min(r_begin + rows_per_block, rows_per_sample);
  for (int rb = r_begin; rb < r_end; rb += RB) {
    bf16x8 raw[RB];
#pragma unroll
    for (int q = 0; q < RB; ++q) {
      raw[q].u = make_uint4(0u, 0u, 0u, 0u);
      if (act && rb + q < r_end)
        raw[q] = reinterpret_cast<const bf16x8*>(x + ((int64_t)sample * rows_per_sample + rb + q) * d)[i];
    }
    float mu[RB], var[RB];
#pragma unroll
    for (int q = 0; q < RB; ++q) {
      float f[8];
      unpack8(raw[q], f);
      float t = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) t += f[j];
      mu[q] = t;
    }
    block_sum_vals<RB>(mu, red, nwarps);
#pragma unroll
    for (int q = 0; q < RB; ++q) {
      mu[q] /= (float)d;
      float f[8];
      unpack8(raw[q], f);
      float t = 0.f;
      if (act) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float c = f[j] - mu[q]; t += c * c; }
      }
      var[q] = t;
    }
    block_sum_vals<RB>(var, red + 32 * RB, nwarps);
#pragma unroll
    for (int q = 0; q < RB; ++q) {
      if (rb + q >= r_end) continue;
      const int64_t row = (int64_t)sample * rows_per_sample + rb + q;
      const float rstd = rsqrtf(var[q] / (float)d + eps);
      if (i == 0) { mean_o[row] = mu[q]; rstd_o[row] = rstd; }
      if (act) {
        float f[8], o[8];
        unpack8(raw[q], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (f[j] - mu[q]) * rstd * sc1[j] + sh[j];
        reinterpret_cast<bf16x8*>(y + row * d)[i] = pack8(o);
      }
    }
    __syncthreads();            // both halves of `red` are free again
  }
}

template <int kMaxT>
__global__ void __launch_bounds__(kMaxT)
adaln_bwd_cols_kernel(const bf16* __restrict__ gy, const bf16* __restrict__ x,
                      const bf16* __restrict__ scale, const float* __restrict__ mean,
                      const float* __restrict__ rstd, bf16* __restrict__ gx, float* __restrict__ gshift,
                      float* __restrict__ gscale, int rows_per_sample, int d, int64_t scale_ld,
                      int rows_per_block) {
  constexpr int RB = kColsRowsPerPass;
  __shared__ float red[2 * 32 * 2 * RB];
  const int i = threadIdx.x, nvec = d / 8, nwarps = blockDim.x >> 5;
  const bool act = i < nvec;
  const int sample = blockIdx.y;
  float one_plus[8], acc_sh[8], acc_sc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { one_plus[j] = 1.f; acc_sh[j] = 0.f; acc_sc[j] = 0.f; }
  if (act) {
    float t[8];
    unpack8(reinterpret_cast<const bf16x8*>(scale + (int64_t)sample * scale_ld)[i], t);
#pragma unroll
    for (int j = 0; j < 8; ++j) one_plus[j] = 1.f + t[j];
  }
  const int r_begin = blockIdx.x * rows_per_block;
  const int r_end = min(r_begin + rows_per_block, rows_per_sample);
  int parity = 0;
  for (int rb = r_begin; rb < r_end; rb += RB, parity ^= 1) {
    bf16x8 xr[RB], gr[RB];
    float mu[RB], rs[RB];
#pragma unroll
    for (int q = 0; q < RB; ++q) {
      const bool ok = rb + q < r_end;
      const int64_t row = (int64_t)sample * rows_per_sample + (ok ? rb + q : r_end - 1);
      mu[q] = mean[row];
      rs[q] = rstd[row];
      xr[q].u = make_uint4(0u, 0u, 0u, 0u);
      gr[q].u = make_uint4(0u, 0u, 0u, 0u);
      if (act && ok) {
        xr[q] = reinterpret_cast<const bf16x8*>(x + row * d)[i];
        gr[q] = reinterpret_cast<const bf16x8*>(gy + row * d)[i];
      }
    }
    float part[2 * RB];
#pragma unroll
    for (int q = 0; q < RB; ++q) {
      float xv[8], gv[8];
      unpack8(xr[q], xv);
      unpack8(gr[q], gv);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (xv[j] - mu[q]) * rs[q];
        const float gp = gv[j] * one_plus[j];
        s1 += gp;
        s2 += gp * xh;
        acc_sh[j] += gv[j];
        acc_sc[j] += gv[j] * xh;
      }
      part[2 * q] = s1;
      part[2 * q + 1] = s2;
    }
    block_sum_vals<2 * RB>(part, red + parity * 32 * 2 * RB, nwarps);
#pragma unroll
    for (int q = 0; q < RB; ++q) {
      if (!act || rb + q >= r_end) continue;
      const int64_t row = (int64_t)sample * rows_per_sample + rb + q;
      const float m1 = part[2 * q] / (float)d, m2 = part[2 * q + 1] / (float)d;
      float xv[8], gv[8], o[8];
      unpack8(xr[q], xv);
      unpack8(gr[q], gv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = (xv[j] - mu[q]) * rs[q];
        o[j] = rs[q] * (gv[j] * one_plus[j] - m1 - xh * m2);
      }
      reinterpret_cast<bf16x8*>(gx + row * d)[i] = pack8(o);
    }
  }
  if (act) {
    float* ds = gshift + (int64_t)sample * d + i * 8;
    float* dc = gscale + (int64_t)sample * d + i * 8;
    red_add_v4(ds, acc_sh);
    red_add_v4(ds + 4, acc_sh + 4);
    red_add_v4(dc, acc_sc);
    red_add_v4(dc + 4, acc_sc + 4);
  }
}

// d(out)/d(y) = g * gate and d(gate)[sample] = sum over the sample's rows of g * y, column owners.
template <int kMaxT>
__global__ void __launch_bounds__(kMaxT)
gate_residual_bwd_cols_kernel(const bf16* __restrict__ g, const bf16* __restrict__ y,
                              const bf16* __restrict__ gate, bf16* __restrict__ gy,
                              float* __restrict__ ggate, int rows_per_sample, int d, int64_t gate_ld,
                              int rows_per_block) {
  constexpr int RB = kColsRowsPerPass;
  const int i = threadIdx.x, nvec = d / 8;
  if (i >= nvec) return;                        // no barrier in this kernel
  const int sample = blockIdx.y;
  float gt[8], acc[8];
  unpack8(reinterpret_cast<const bf16x8*>(gate + (int64_t)sample * gate_ld)[i], gt);
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const int r_begin = blockIdx.x * rows_per_block;
  const int r_end = min(r_begin + rows_per_block, rows_per_sample);
  for (int rb = r_begin; rb < r_end; rb += RB) {
    bf16x8 graw[RB], yraw[RB];
#pragma unroll
    for (int q = 0; q < RB; ++q) {
      graw[q].u = make_uint4(0u, 0u, 0u, 0u);
      yraw[q].u = make_uint4(0u, 0u, 0u, 0u);
      if (rb + q < r_end) {
        const int64_t row = (int64_t)sample * rows_per_sample + rb + q;
        graw[q] = reinterpret_cast<const bf16x8*>(g + row * d)[i];
        yraw[q] = reinterpret_cast<const bf16x8*>(y + row * d)[i];
      }
    }
#pragma unroll
    for (int q = 0; q < RB; ++q) {
      if (rb + q >= r_end) continue;
      const int64_t row = (int64_t)sample * rows_per_sample + rb + q;
      float a[8], b[8], o[8];
      unpack8(graw[q], a);
      unpack8(yraw[q], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = a[j] * gt[j];
        acc[j] += a[j] * b[j];
      }
      reinterpret_cast<bf16x8*>(gy + row * d)[i] = pack8(o);
    }
  }
  float* dg = ggate + (int64_t)sample * d + i * 8;
  red_add_v4(dg, acc);
  red_add_v4(dg + 4, acc + 4);
}

// ------------------------------------------------------------------------------ adaLN forward
__global__ void __launch_bounds__(kNormThreads)
adaln_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ shift,
                 const bf16* __restrict__ scale, bf16* __restrict__ y, float* __restrict__ mean_o,
                 float* __restrict__ rstd_o, int rows_per_sample, int d, float eps,
                 int64_t shift_ld, int64_t scale_ld) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int sample = (int)(row / rows_per_sample);
  const int nvec = d / 8;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * d);
  float f[kMaxVec][8];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
    if (i < nvec) {
      unpack8(xr[i], f[k]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += f[k][j];
    }
  }
  const float mu = block_sum(s, red) / (float)d;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float c = f[k][j] - mu; q += c * c; }
    }
  }
  const float rstd = rsqrtf(block_sum(q, red) / (float)d + eps);
  if (threadIdx.x == 0) { mean_o[row] = mu; rstd_o[row] = rstd; }
  const bf16x8* sh = reinterpret_cast<const bf16x8*>(shift + (int64_t)sample * shift_ld);
  const bf16x8* sc = reinterpret_cast<const bf16x8*>(scale + (int64_t)sample * scale_ld);
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * d);
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
    if (i < nvec) {
      float a[8], b[8], o[8];
      unpack8(sh[i], a);
      unpack8(sc[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (f[k][j] - mu) * rstd * (1.f + b[j]) + a[j];
      yr[i] = pack8(o);
    }
  }
}

std::vector<torch::Tensor> adaln_fwd(torch::Tensor x, torch::Tensor shift, torch::Tensor scale,
                                     double eps) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.scalar_type() == torch::kBFloat16 && x.is_contiguous());
  VRL_CHECK_OPERAND(shift, x);
  VRL_CHECK_OPERAND(scale, x);
  const c10::cuda::CUDAGuard guard(x.device());
  const int b = (int)x.size(0), s = (int)x.size(1), d = (int)x.size(2);
  TORCH_CHECK(d % 8 == 0 && d <= 8 * kMaxVec * kNormThreads, "adaln: D must be a multiple of 8, <= 8192");
  shift = strided_rows(shift, b, d);
  scale = strided_rows(scale, b, d);
  auto y = torch::empty_like(x);
  auto mean = torch::empty({(int64_t)b * s}, x.options().dtype(torch::kFloat32));
  auto rstd = torch::empty_like(mean);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (b * s > 0 && b <= 65535) {
    const int threads = (d / 8 + 31) / 32 * 32;
    const int rpb = cols_rows_per_block((int64_t)b * s, s);
    dim3 grid((s + rpb - 1) / rpb, b);
    VRL_DISPATCH_COLS(threads, adaln_fwd_cols_kernel<kMaxT><<<grid, threads, 0, stream>>>(
        reinterpret_cast<const bf16*>(x.data_ptr()), reinterpret_cast<const bf16*>(shift.data_ptr()),
        reinterpret_cast<const bf16*>(scale.data_ptr()), reinterpret_cast<bf16*>(y.data_ptr()),
        mean.data_ptr<float>(), rstd.data_ptr<float>(), s, d, (float)eps, shift.stride(0), scale.stride(0),
        rpb));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {y, mean, rstd};
  }
  if (d <= 2048) {
    const int64_t rows = (int64_t)b * s;
    const unsigned blocks = (unsigned)((rows + kRowWarps - 1) / kRowWarps);
    VRL_DISPATCH_VPL(d / 8, adaln_fwd_warp_kernel<VPL><<<blocks, kRowWarps * 32, 0, stream>>>(
        reinterpret_cast<const bf16*>(x.data_ptr()), reinterpret_cast<const bf16*>(shift.data_ptr()),
        reinterpret_cast<const bf16*>(scale.data_ptr()), reinterpret_cast<bf16*>(y.data_ptr()),
        mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, s, d, (float)eps, shift.stride(0),
        scale.stride(0)));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {y, mean, rstd};
  }
  adaln_fwd_kernel<<<b * s, kNormThreads, 0, stream>>>(
      reinterpret_cast<const bf16*>(x.data_ptr()), reinterpret_cast<const bf16*>(shift.data_ptr()),
      reinterpret_cast<const bf16*>(scale.data_ptr()), reinterpret_cast<bf16*>(y.data_ptr()),
      mean.data_ptr<float>(), rstd.data_ptr<float>(), s, d, (float)eps, shift.stride(0),
      scale.stride(0));
  return {y, mean, rstd};
}

// ----------------------------------------------------------------------------- adaLN backward
__global__ void __launch_bounds__(kNormThreads)
adaln_bwd_kernel(const bf16* __restrict__ gy, const bf16* __restrict__ x,
                 const bf16* __restrict__ scale, const float* __restrict__ mean,
                 const float* __restrict__ rstd, bf16* __restrict__ gx, float* __restrict__ gshift,
                 float* __restrict__ gscale, int rows_per_sample, int d, int64_t scale_ld) {
  __shared__ float red[32];
  const int sample = blockIdx.y;
  const int nvec = d / 8;
  const int row0 = blockIdx.x * kBwdRows;
  const bf16x8* sc = reinterpret_cast<const bf16x8*>(scale + (int64_t)sample * scale_ld);
  float one_plus[kMaxVec][8], acc_sh[kMaxVec][8], acc_sc[kMaxVec][8];
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc_sh[k][j] = 0.f; acc_sc[k][j] = 0.f; one_plus[k][j] = 1.f; }
    if (i < nvec) {
      float t[8];
      unpack8(sc[i], t);
#pragma unroll
      for (int j = 0; j < 8; ++j) one_plus[k][j] = 1.f + t[j];
    }
  }
  for (int r = row0; r < row0 + kBwdRows && r < rows_per_sample; ++r) {
    const int64_t row = (int64_t)sample * rows_per_sample + r;
    const float mu = mean[row], rs = rstd[row];
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * d);
    const bf16x8* gr = reinterpret_cast<const bf16x8*>(gy + row * d);
    float xh[kMaxVec][8], gp[kMaxVec][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
      const int i = threadIdx.x + k * kNormThreads;
      if (i < nvec) {
        float xv[8], gv[8];
        unpack8(xr[i], xv);
        unpack8(gr[i], gv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[k][j] = (xv[j] - mu) * rs;
          gp[k][j] = gv[j] * one_plus[k][j];
          acc_sh[k][j] += gv[j];
          acc_sc[k][j] += gv[j] * xh[k][j];
          s1 += gp[k][j];
          s2 += gp[k][j] * xh[k][j];
        }
      }
    }
    const float m1 = block_sum(s1, red) / (float)d;
    const float m2 = block_sum(s2, red) / (float)d;
    bf16x8* gxr = reinterpret_cast<bf16x8*>(gx + row * d);
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
      const int i = threadIdx.x + k * kNormThreads;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (gp[k][j] - m1 - xh[k][j] * m2);
        gxr[i] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        atomicAdd(gshift + (int64_t)sample * d + i * 8 + j, acc_sh[k][j]);
        atomicAdd(gscale + (int64_t)sample * d + i * 8 + j, acc_sc[k][j]);
      }
    }
  }
}

std::vector<torch::Tensor> adaln_bwd(torch::Tensor gy, torch::Tensor x, torch::Tensor scale,
                                     torch::Tensor mean, torch::Tensor rstd) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.scalar_type() == torch::kBFloat16 && x.is_contiguous());
  VRL_CHECK_OPERAND(gy, x, c10::nullopt, x.numel());
  VRL_CHECK_OPERAND(scale, x);
  VRL_CHECK_OPERAND(mean, x, torch::kFloat32, x.size(0) * x.size(1));
  VRL_CHECK_OPERAND(rstd, x, torch::kFloat32, x.size(0) * x.size(1));
  TORCH_CHECK(mean.is_contiguous() && rstd.is_contiguous(), "adaln_bwd: row statistics must be contiguous");
  const c10::cuda::CUDAGuard guard(x.device());
  const int b = (int)x.size(0), s = (int)x.size(1), d = (int)x.size(2);
  gy = gy.to(torch::kBFloat16).contiguous();
  scale = strided_rows(scale, b, d);
  auto gx = torch::empty_like(x);
  auto gshift = torch::zeros({b, d}, x.options().dtype(torch::kFloat32));
  auto gscale = torch::zeros({b, d}, x.options().dtype(torch::kFloat32));
  if (b * s > 0 && b <= 65535) {
    const int threads = (d / 8 + 31) / 32 * 32;
    const int rpb = cols_rows_per_block((int64_t)b * s, s);
    dim3 grid((s + rpb - 1) / rpb, b);
    auto stream = at::cuda::getCurrentCUDAStream();
    VRL_DISPATCH_COLS(threads, adaln_bwd_cols_kernel<kMaxT><<<grid, threads, 0, stream>>>(
        reinterpret_cast<const bf16*>(gy.data_ptr()), reinterpret_cast<const bf16*>(x.data_ptr()),
        reinterpret_cast<const bf16*>(scale.data_ptr()), mean.data_ptr<float>(), rstd.data_ptr<float>(),
        reinterpret_cast<bf16*>(gx.data_ptr()), gshift.data_ptr<float>(), gscale.data_ptr<float>(), s, d,
        scale.stride(0), rpb));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {gx, gshift, gscale};
  }
  if (d <= 2048) {
    dim3 wgrid((s + kAdaBlockRows - 1) / kAdaBlockRows, b);
    auto stream = at::cuda::getCurrentCUDAStream();
    VRL_DISPATCH_VPL(d / 8, adaln_bwd_warp_kernel<VPL><<<wgrid, kRowWarps * 32, 2 * d * sizeof(float), stream>>>(
        reinterpret_cast<const bf16*>(gy.data_ptr()), reinterpret_cast<const bf16*>(x.data_ptr()),
        reinterpret_cast<const bf16*>(scale.data_ptr()), mean.data_ptr<float>(),
        rstd.data_ptr<float>(), reinterpret_cast<bf16*>(gx.data_ptr()), gshift.data_ptr<float>(),
        gscale.data_ptr<float>(), s, d, scale.stride(0)));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {gx, gshift, gscale};
  }
  dim3 grid((s + kBwdRows - 1) / kBwdRows, b);
  adaln_bwd_kernel<<<grid, kNormThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(gy.data_ptr()), reinterpret_cast<const bf16*>(x.data_ptr()),
      reinterpret_cast<const bf16*>(scale.data_ptr()), mean.data_ptr<float>(),
      rstd.data_ptr<float>(), reinterpret_cast<bf16*>(gx.data_ptr()), gshift.data_ptr<float>(),
      gscale.data_ptr<float>(), s, d, scale.stride(0));
  return {gx, gshift, gscale};
}

// ----------------------------------------------------------------------------------- RMSNorm
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                   float* __restrict__ rstd_o, int d, float eps) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int nvec = d / 8;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * d);
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  float f[kMaxVec][8];
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
    if (i < nvec) {
      unpack8(xr[i], f[k]);
#pragma unroll
      for (int j = 0; j < 8; ++j) q += f[k][j] * f[k][j];
    }
  }
  const float rstd = rsqrtf(block_sum(q, red) / (float)d + eps);
  if (threadIdx.x == 0) rstd_o[row] = rstd;
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + row * d);
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
    if (i < nvec) {
      float ww[8], o[8];
      unpack8(wr[i], ww);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = f[k][j] * rstd * ww[j];
      yr[i] = pack8(o);
    }
  }
}

std::vector<torch::Tensor> rmsnorm_fwd(torch::Tensor x, torch::Tensor w, double eps) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() >= 1);
  VRL_CHECK_OPERAND(w, x, c10::nullopt, x.size(-1));
  const c10::cuda::CUDAGuard guard(x.device());
  const int d = (int)x.size(-1);
  const int64_t rows = x.numel() / d;
  TORCH_CHECK(d % 8 == 0 && d <= 8 * kMaxVec * kNormThreads);
  w = w.to(torch::kBFloat16).contiguous();
  auto y = torch::empty_like(x);
  auto rstd = torch::empty({rows}, x.options().dtype(torch::kFloat32));
  if (d <= 2048) {
    auto stream = at::cuda::getCurrentCUDAStream();
    const unsigned blocks = (unsigned)((rows + kRowWarps - 1) / kRowWarps);
    VRL_DISPATCH_VPL(d / 8, rmsnorm_fwd_warp_kernel<VPL><<<blocks, kRowWarps * 32, 0, stream>>>(
        reinterpret_cast<const bf16*>(x.data_ptr()), reinterpret_cast<const bf16*>(w.data_ptr()),
        reinterpret_cast<bf16*>(y.data_ptr()), rstd.data_ptr<float>(), rows, d, (float)eps));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {y, rstd};
  }
  rmsnorm_fwd_kernel<<<(unsigned)rows, kNormThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(x.data_ptr()), reinterpret_cast<const bf16*>(w.data_ptr()),
      reinterpret_cast<bf16*>(y.data_ptr()), rstd.data_ptr<float>(), d, (float)eps);
  return {y, rstd};
}

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const bf16* __restrict__ gy, const bf16* __restrict__ x,
                   const bf16* __restrict__ w, const float* __restrict__ rstd,
                   bf16* __restrict__ gx, float* __restrict__ gw, int64_t rows, int d) {
  __shared__ float red[32];
  const int nvec = d / 8;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  float ww[kMaxVec][8], acc[kMaxVec][8];
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc[k][j] = 0.f; ww[k][j] = 0.f; }
    if (i < nvec) unpack8(wr[i], ww[k]);
  }
  const int64_t row0 = (int64_t)blockIdx.x * kBwdRows;
  for (int64_t row = row0; row < row0 + kBwdRows && row < rows; ++row) {
    const float rs = rstd[row];
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + row * d);
    const bf16x8* gr = reinterpret_cast<const bf16x8*>(gy + row * d);
    float xh[kMaxVec][8], gn[kMaxVec][8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
      const int i = threadIdx.x + k * kNormThreads;
      if (i < nvec) {
        float xv[8], gv[8];
        unpack8(xr[i], xv);
        unpack8(gr[i], gv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[k][j] = xv[j] * rs;
          gn[k][j] = gv[j] * ww[k][j];
          acc[k][j] += gv[j] * xh[k][j];
          s += gn[k][j] * xh[k][j];
        }
      }
    }
    const float m = block_sum(s, red) / (float)d;
    bf16x8* gxr = reinterpret_cast<bf16x8*>(gx + row * d);
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
      const int i = threadIdx.x + k * kNormThreads;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (gn[k][j] - xh[k][j] * m);
        gxr[i] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(gw + i * 8 + j, acc[k][j]);
    }
  }
}

std::vector<torch::Tensor> rmsnorm_bwd(torch::Tensor gy, torch::Tensor x, torch::Tensor w,
                                       torch::Tensor rstd) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() >= 1);
  VRL_CHECK_OPERAND(gy, x, c10::nullopt, x.numel());
  VRL_CHECK_OPERAND(w, x, c10::nullopt, x.size(-1));
  VRL_CHECK_OPERAND(rstd, x, torch::kFloat32, x.numel() / x.size(-1));
  TORCH_CHECK(rstd.is_contiguous(), "rmsnorm_bwd: rstd must be contiguous");
  const c10::cuda::CUDAGuard guard(x.device());
  const int d = (int)x.size(-1);
  const int64_t rows = x.numel() / d;
  gy = gy.to(torch::kBFloat16).contiguous();
  w = w.to(torch::kBFloat16).contiguous();
  auto gx = torch::empty_like(x);
  auto gw = torch::zeros({d}, x.options().dtype(torch::kFloat32));
  rmsnorm_bwd_kernel<<<(unsigned)((rows + kBwdRows - 1) / kBwdRows), kNormThreads, 0,
                       at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(gy.data_ptr()), reinterpret_cast<const bf16*>(x.data_ptr()),
      reinterpret_cast<const bf16*>(w.data_ptr()), rstd.data_ptr<float>(),
      reinterpret_cast<bf16*>(gx.data_ptr()), gw.data_ptr<float>(), rows, d);
  return {gx, gw};
}

// ------------------------------------------------------------------ gated residual (adaLN-Zero)
// out = residual + gate[sample] * y, and its backward: gy = g * gate, d(gate)[sample] = sum_s g * y
// (d(residual) is g itself).  One warp per row; the per-sample column sums of the backward are
// collected in shared memory per block and flushed once with global atomics.
__global__ void __launch_bounds__(kRowWarps * 32)
gate_residual_fwd_kernel(const bf16* __restrict__ y, const bf16* __restrict__ gate,
                         const bf16* __restrict__ residual, bf16* __restrict__ out, int64_t rows,
                         int rows_per_sample, int d, int64_t gate_ld) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kRowWarps + warp;
  if (row >= rows) return;
  const int nvec = d / 8;
  const bf16x8* yr = reinterpret_cast<const bf16x8*>(y + row * d);
  const bf16x8* rr = reinterpret_cast<const bf16x8*>(residual + row * d);
  const bf16x8* gr = reinterpret_cast<const bf16x8*>(gate + (row / rows_per_sample) * gate_ld);
  bf16x8* orow = reinterpret_cast<bf16x8*>(out + row * d);
  for (int i = lane; i < nvec; i += 32) {
    float a[8], b[8], c[8], o[8];
    unpack8(yr[i], a);
    unpack8(gr[i], b);
    unpack8(rr[i], c);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = c[j] + b[j] * a[j];
    orow[i] = pack8(o);
  }
}

constexpr int kGateBlockRows = 128;

template <int VPL>
__global__ void __launch_bounds__(kRowWarps * 32)
gate_residual_bwd_kernel(const bf16* __restrict__ g, const bf16* __restrict__ y,
                         const bf16* __restrict__ gate, bf16* __restrict__ gy,
                         float* __restrict__ ggate, int rows_per_sample, int d, int64_t gate_ld) {
  extern __shared__ float col_acc[];         // [d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sample = blockIdx.y;
  const int nvec = d / 8;
  for (int i = threadIdx.x; i < d; i += blockDim.x) col_acc[i] = 0.f;
  __syncthreads();
  const bf16x8* gt = reinterpret_cast<const bf16x8*>(gate + (int64_t)sample * gate_ld);
  float acc[VPL][8], gtv[VPL][8];
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int i = lane + k * 32;
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc[k][j] = 0.f; gtv[k][j] = 0.f; }
    if (i < nvec) unpack8(gt[i], gtv[k]);
  }
  const int r_begin = blockIdx.x * kGateBlockRows;
  for (int r = r_begin + warp; r < r_begin + kGateBlockRows && r < rows_per_sample; r += kRowWarps) {
    const int64_t row = (int64_t)sample * rows_per_sample + r;
    const bf16x8* gr = reinterpret_cast<const bf16x8*>(g + row * d);
    const bf16x8* yr = reinterpret_cast<const bf16x8*>(y + row * d);
    bf16x8* orow = reinterpret_cast<bf16x8*>(gy + row * d);
    bf16x8 graw[VPL], yraw[VPL];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int i = lane + k * 32;
      if (i < nvec) { graw[k] = gr[i]; yraw[k] = yr[i]; }
    }
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int i = lane + k * 32;
      if (i < nvec) {
        float a[8], b[8], o[8];
        unpack8(graw[k], a);
        unpack8(yraw[k], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = a[j] * gtv[k][j];
          acc[k][j] += a[j] * b[j];
        }
        orow[i] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < VPL; ++k) {
    const int i = lane + k * 32;
    if (i < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(&col_acc[i * 8 + j], acc[k][j]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < d; i += blockDim.x) atomicAdd(ggate + (int64_t)sample * d + i, col_acc[i]);
}

torch::Tensor gate_residual_fwd(torch::Tensor y, torch::Tensor gate, torch::Tensor residual) {
  TORCH_CHECK(y.is_cuda() && y.dim() == 3 && y.scalar_type() == torch::kBFloat16 && y.is_contiguous());
  TORCH_CHECK(residual.scalar_type() == torch::kBFloat16 && residual.is_contiguous() &&
              residual.sizes() == y.sizes());
  VRL_CHECK_OPERAND(gate, y);
  VRL_CHECK_OPERAND(residual, y);
  const c10::cuda::CUDAGuard guard(y.device());
  const int b = (int)y.size(0), s = (int)y.size(1), d = (int)y.size(2);
  TORCH_CHECK(d % 8 == 0);
  gate = strided_rows(gate, b, d);
  auto out = torch::empty_like(y);
  const int64_t rows = (int64_t)b * s;
  if (rows == 0) return out;
  gate_residual_fwd_kernel<<<(unsigned)((rows + kRowWarps - 1) / kRowWarps), kRowWarps * 32, 0,
                             at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(y.data_ptr()), reinterpret_cast<const bf16*>(gate.data_ptr()),
      reinterpret_cast<const bf16*>(residual.data_ptr()), reinterpret_cast<bf16*>(out.data_ptr()), rows, s,
      d, gate.stride(0));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

std::vector<torch::Tensor> gate_residual_bwd(torch::Tensor g, torch::Tensor y, torch::Tensor gate) {
  TORCH_CHECK(y.is_cuda() && y.dim() == 3 && y.scalar_type() == torch::kBFloat16 && y.is_contiguous());
  VRL_CHECK_OPERAND(g, y);
  VRL_CHECK_OPERAND(gate, y);
  const c10::cuda::CUDAGuard guard(y.device());
  const int b = (int)y.size(0), s = (int)y.size(1), d = (int)y.size(2);
  g = g.to(torch::kBFloat16).contiguous();
  TORCH_CHECK(g.sizes() == y.sizes() && d % 8 == 0 && d <= 8192, "gate_residual_bwd: D <= 8192");
  gate = strided_rows(gate, b, d);
  auto gy = torch::empty_like(y);
  auto ggate = torch::zeros({b, d}, y.options().dtype(torch::kFloat32));
  if (b * s == 0) return {gy, ggate};
  if (b <= 65535) {
    const int threads = (d / 8 + 31) / 32 * 32;
    const int rpb = cols_rows_per_block((int64_t)b * s, s);
    dim3 cgrid((s + rpb - 1) / rpb, b);
    VRL_DISPATCH_COLS(threads, gate_residual_bwd_cols_kernel<kMaxT><<<cgrid, threads, 0,
                                                                   at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const bf16*>(g.data_ptr()), reinterpret_cast<const bf16*>(y.data_ptr()),
        reinterpret_cast<const bf16*>(gate.data_ptr()), reinterpret_cast<bf16*>(gy.data_ptr()),
        ggate.data_ptr<float>(), s, d, gate.stride(0), rpb));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {gy, ggate};
  }
  TORCH_CHECK(d <= 2048, "gate_residual_bwd: D <= 2048 for more than 65535 samples");
  dim3 grid((s + kGateBlockRows - 1) / kGateBlockRows, b);
  auto stream = at::cuda::getCurrentCUDAStream();
  VRL_DISPATCH_VPL(d / 8, gate_residual_bwd_kernel<VPL><<<grid, kRowWarps * 32, d * sizeof(float), stream>>>(
      reinterpret_cast<const bf16*>(g.data_ptr()), reinterpret_cast<const bf16*>(y.data_ptr()),
      reinterpret_cast<const bf16*>(gate.data_ptr()), reinterpret_cast<bf16*>(gy.data_ptr()),
      ggate.data_ptr<float>(), s, d, gate.stride(0)));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {gy, ggate};
}

// ------------------------------------------------------------------------- QKV post-processing
// qkv[b, s, which, h, :] -> out_which[b, seq_offset + s, h, :] of a token-major [B, S_total, H, Dh]
// buffer (callers view it as [B, H, S_total, Dh] through strides; two streams of a joint-attention
// block write into one buffer at different offsets, so no concatenation copy is needed).  Norm modes: 0 none, 1 per head (weights of
// Dh elements), 2 full width (weights of H*Dh elements).  rstd layout: [b, s, 2, H] (mode 1)
// or [b, s, 2] (mode 2).  Rotary tables are [S, Dh/2]; pairs are (2i, 2i+1).
constexpr int kQkvTokensPerPass = 4;

__device__ __forceinline__ float group_sum(float v, int lanes) {
  for (int o = lanes >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Destinations of the sequence-parallel form: head group g = h / (heads / world) of every token goes
// to rank g's [B, seq_total, heads / world, Dh] buffer (peer-mapped addresses), at this rank's
// sequence offset.  world <= 1 means "local destinations" and the table is not read.
struct QkvPeers {
  bf16* q[16];
  bf16* k[16];
  bf16* v[16];
  int world;
};

// tokens per block so that the three grids together give every SM a few blocks
static int qkv_tokens_per_block(int64_t tokens) {
  int64_t tpb = tokens * 3 / (148 * 6);
  tpb = std::max<int64_t>(kQkvTokensPerPass, std::min<int64_t>(32, tpb));
  return (int)((tpb + kQkvTokensPerPass - 1) / kQkvTokensPerPass * kQkvTokensPerPass);
}

// Column owners: blockIdx.y picks q, k or v; thread i owns vector i of that part's H * Dh / 8 (head
// i / (Dh / 8)) and walks over a run of tokens, four per pass, so four independent 16-byte loads are
// in flight per thread.  The per-head statistics are sums over the Dh / 8 neighbouring lanes; the
// full-width ones are block sums of four values at a time.
template <int kMaxT>
__global__ void __launch_bounds__(kMaxT)
qkv_prepare_fwd_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ qw,
                       const bf16* __restrict__ kw, const float* __restrict__ cosT,
                       const float* __restrict__ sinT, bf16* __restrict__ q, bf16* __restrict__ k,
                       bf16* __restrict__ v, float* __restrict__ rstd_o, int64_t tokens, int seq, int heads,
                       int dh, int mode, float eps, int seq_total, int seq_offset, int tokens_per_block,
                       const QkvPeers peers) {
  constexpr int TB = kQkvTokensPerPass;
  __shared__ float red[2 * 32 * TB];
  const int i = threadIdx.x, nwarps = blockDim.x >> 5;
  const int which = blockIdx.y;
  const int dmodel = heads * dh;
  const int vec_per_head = dh / 8, vec_per_which = dmodel / 8;
  const bool act = i < vec_per_which;
  const int h = i / vec_per_head, j8 = i - h * vec_per_head;
  const bool normed = which < 2 && mode != 0;
  float ww[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) ww[j] = 1.f;
  if (act && normed)
    unpack8(*reinterpret_cast<const bf16x8*>((which == 0 ? qw : kw) + (mode == 1 ? j8 * 8 : i * 8)), ww);
  bf16* dst_local = which == 0 ? q : (which == 1 ? k : v);
  const int hp = peers.world > 1 ? heads / peers.world : heads;
  const int pg = h / hp, hl = h - pg * hp;
  bf16* dst_peer = nullptr;
  if (peers.world > 1 && act) dst_peer = which == 0 ? peers.q[pg] : (which == 1 ? peers.k[pg] : peers.v[pg]);
  const int64_t tok_begin = (int64_t)blockIdx.x * tokens_per_block;
  const int64_t tok_end = min(tok_begin + (int64_t)tokens_per_block, tokens);
  int parity = 0;
  for (int64_t tb = tok_begin; tb < tok_end; tb += TB) {
    bf16x8 raw[TB];
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      raw[t].u = make_uint4(0u, 0u, 0u, 0u);
      if (act && tb + t < tok_end)
        raw[t] = *reinterpret_cast<const bf16x8*>(qkv + ((tb + t) * 3 + which) * dmodel + i * 8);
    }
    float ssq[TB];
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      float f[8];
      unpack8(raw[t], f);
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) a += f[j] * f[j];
      ssq[t] = a;
    }
    if (normed) {                                   // uniform over the block
      if (mode == 1) {
#pragma unroll
        for (int t = 0; t < TB; ++t) ssq[t] = group_sum(ssq[t], vec_per_head);
      } else {
        block_sum_vals<TB>(ssq, red + parity * 32 * TB, nwarps);
        parity ^= 1;
      }
    }
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      const int64_t tok = tb + t;
      if (!act || tok >= tok_end) continue;
      // 32-bit index arithmetic: a 64-bit division per token and thread costs more than the token's math
      int b = (int)((unsigned)tb / (unsigned)seq), sidx = (int)tb - b * seq + t;
      while (sidx >= seq) { sidx -= seq; ++b; }
      float o[8];
      unpack8(raw[t], o);
      if (normed) {
        const float rs = rsqrtf(ssq[t] / (float)(mode == 1 ? dh : dmodel) + eps);
        if (mode == 1) {
          if (j8 == 0) rstd_o[(tok * 2 + which) * heads + h] = rs;
        } else if (i == 0) {
          rstd_o[tok * 2 + which] = rs;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = o[j] * rs * ww[j];
      }
      if (which < 2 && cosT != nullptr) {
        const float4 c = *reinterpret_cast<const float4*>(cosT + (int64_t)sidx * (dh / 2) + j8 * 4);
        const float4 sn = *reinterpret_cast<const float4*>(sinT + (int64_t)sidx * (dh / 2) + j8 * 4);
        const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float x0 = o[2 * p], x1 = o[2 * p + 1];
          o[2 * p] = x0 * cc[p] - x1 * sv[p];
          o[2 * p + 1] = x0 * sv[p] + x1 * cc[p];
        }
      }
      const int64_t drow = (int64_t)b * seq_total + seq_offset + sidx;
      if (peers.world > 1) {
        // the head <-> sequence exchange of sequence parallelism happens in this store: the head's
        // owner receives the token at this rank's place in the full sequence, over NVLink
        *reinterpret_cast<bf16x8*>(dst_peer + (drow * hp + hl) * dh + j8 * 8) = pack8(o);
      } else {
        // token-major destination [B, seq_total, H, Dh]: one token's heads are contiguous
        *reinterpret_cast<bf16x8*>(dst_local + (drow * heads + h) * dh + j8 * 8) = pack8(o);
      }
    }
  }
}

// shared launch of the forward kernel (local or peer destinations)
static void launch_qkv_fwd(const torch::Tensor& qkv, const bf16* qw, const bf16* kw, const float* cosT,
                           const float* sinT, bf16* q, bf16* k, bf16* v, float* rstd, int b, int s, int heads,
                           int dh, int mode, float eps, int seq_total, int seq_offset, const QkvPeers& peers) {
  const int64_t tokens = (int64_t)b * s;
  if (tokens == 0) return;
  TORCH_CHECK(tokens < (1ll << 31), "qkv_prepare: token count must fit 31 bits");
  const int threads = (heads * dh / 8 + 31) / 32 * 32;
  const int tpb = qkv_tokens_per_block(tokens);
  dim3 grid((unsigned)((tokens + tpb - 1) / tpb), 3);
  auto stream = at::cuda::getCurrentCUDAStream();
  VRL_DISPATCH_COLS(threads, qkv_prepare_fwd_kernel<kMaxT><<<grid, threads, 0, stream>>>(
      reinterpret_cast<const bf16*>(qkv.data_ptr()), qw, kw, cosT, sinT, q, k, v, rstd, tokens, s, heads, dh,
      mode, eps, seq_total, seq_offset, tpb, peers));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// head dims whose Dh / 8 lanes form a power-of-two group inside a warp, widths of at most 1024 owners
static void check_qkv_geometry(int dmodel, int dh) {
  const int vph = dh / 8;
  TORCH_CHECK(dh % 8 == 0 && vph >= 1 && vph <= 32 && (vph & (vph - 1)) == 0, "unsupported head dim");
  TORCH_CHECK(dmodel / 8 <= 1024, "model width too large for qkv_prepare");
}

std::vector<torch::Tensor> qkv_prepare_fwd(torch::Tensor qkv, c10::optional<torch::Tensor> qw,
                                           c10::optional<torch::Tensor> kw,
                                           c10::optional<torch::Tensor> cos,
                                           c10::optional<torch::Tensor> sin, int64_t heads,
                                           double eps, c10::optional<torch::Tensor> dst_q,
                                           c10::optional<torch::Tensor> dst_k,
                                           c10::optional<torch::Tensor> dst_v, int64_t seq_offset) {
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 3 && qkv.scalar_type() == torch::kBFloat16 &&
              qkv.is_contiguous());
  TORCH_CHECK(qw.has_value() == kw.has_value() && cos.has_value() == sin.has_value() &&
              dst_q.has_value() == dst_k.has_value() && dst_q.has_value() == dst_v.has_value(),
              "qkv_prepare: q/k norm weights, cos/sin tables and destinations come in complete sets");
  VRL_CHECK_OPERAND(qw, qkv);
  VRL_CHECK_OPERAND(kw, qkv);
  VRL_CHECK_OPERAND(cos, qkv);
  VRL_CHECK_OPERAND(sin, qkv);
  VRL_CHECK_OPERAND(dst_q, qkv);
  VRL_CHECK_OPERAND(dst_k, qkv);
  VRL_CHECK_OPERAND(dst_v, qkv);
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int b = (int)qkv.size(0), s = (int)qkv.size(1);
  const int dmodel = (int)(qkv.size(2) / 3), dh = dmodel / (int)heads;
  check_qkv_geometry(dmodel, dh);
  int mode = 0;
  torch::Tensor qwc, kwc;
  if (qw.has_value()) {
    qwc = qw->to(torch::kBFloat16).contiguous();
    kwc = kw->to(torch::kBFloat16).contiguous();
    mode = (qwc.numel() == dh && heads > 1) || (heads == 1) ? 1 : 2;
    TORCH_CHECK(qwc.numel() == (mode == 1 ? dh : dmodel));
  }
  torch::Tensor cosc, sinc;
  if (cos.has_value()) {
    cosc = cos->to(torch::kFloat32).contiguous();
    sinc = sin->to(torch::kFloat32).contiguous();
    TORCH_CHECK(cosc.size(0) == s && cosc.size(1) == dh / 2);
  }
  auto opt = qkv.options();
  torch::Tensor q, k, v;
  int64_t seq_total = s;
  if (dst_q.has_value()) {
    q = *dst_q; k = *dst_k; v = *dst_v;
    for (const auto& t : {q, k, v})
      TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 4 && t.is_contiguous() &&
                  t.size(0) == b && t.size(2) == heads && t.size(3) == dh,
                  "qkv_prepare: destinations must be contiguous [B, S_total, H, Dh]");
    seq_total = q.size(1);
    TORCH_CHECK(k.size(1) == seq_total && v.size(1) == seq_total && seq_offset >= 0 &&
                seq_offset + s <= seq_total, "qkv_prepare: sequence window out of range");
  } else {
    TORCH_CHECK(seq_offset == 0);
    q = torch::empty({b, s, (int64_t)heads, dh}, opt);
    k = torch::empty_like(q);
    v = torch::empty_like(q);
  }
  auto rstd = torch::empty({(int64_t)b * s * 2 * (mode == 1 ? heads : 1)},
                           opt.dtype(torch::kFloat32));
  launch_qkv_fwd(qkv, mode ? reinterpret_cast<const bf16*>(qwc.data_ptr()) : nullptr,
                 mode ? reinterpret_cast<const bf16*>(kwc.data_ptr()) : nullptr,
                 cos.has_value() ? cosc.data_ptr<float>() : nullptr,
                 cos.has_value() ? sinc.data_ptr<float>() : nullptr, reinterpret_cast<bf16*>(q.data_ptr()),
                 reinterpret_cast<bf16*>(k.data_ptr()), reinterpret_cast<bf16*>(v.data_ptr()),
                 rstd.data_ptr<float>(), b, s, (int)heads, dh, mode, (float)eps, (int)seq_total,
                 (int)seq_offset, QkvPeers{});
  return {q, k, v, rstd};
}

// Sequence-parallel form: q / k / v of this rank's tokens are stored straight into the head owners'
// [B, seq_total, heads / world, Dh] buffers.  `peers_*` are CPU int64 tables of the peer-mapped base
// addresses of those buffers (one per rank).  Returns the norm statistics the backward pass needs.
torch::Tensor qkv_prepare_fwd_peers(torch::Tensor qkv, c10::optional<torch::Tensor> qw,
                                    c10::optional<torch::Tensor> kw, c10::optional<torch::Tensor> cos,
                                    c10::optional<torch::Tensor> sin, int64_t heads, double eps,
                                    torch::Tensor peers_q, torch::Tensor peers_k, torch::Tensor peers_v,
                                    int64_t world, int64_t seq_total, int64_t seq_offset) {
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 3 && qkv.scalar_type() == torch::kBFloat16 && qkv.is_contiguous());
  TORCH_CHECK(qw.has_value() == kw.has_value() && cos.has_value() == sin.has_value());
  VRL_CHECK_OPERAND(qw, qkv);
  VRL_CHECK_OPERAND(kw, qkv);
  VRL_CHECK_OPERAND(cos, qkv);
  VRL_CHECK_OPERAND(sin, qkv);
  TORCH_CHECK(world >= 2 && world <= 16 && heads % world == 0, "qkv_prepare_fwd_peers: heads must divide by 2..16 ranks");
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int b = (int)qkv.size(0), s = (int)qkv.size(1);
  const int dmodel = (int)(qkv.size(2) / 3), dh = dmodel / (int)heads;
  check_qkv_geometry(dmodel, dh);
  TORCH_CHECK(seq_offset >= 0 && seq_offset + s <= seq_total, "qkv_prepare_fwd_peers: sequence window out of range");
  int mode = 0;
  torch::Tensor qwc, kwc;
  if (qw.has_value()) {
    qwc = qw->to(torch::kBFloat16).contiguous();
    kwc = kw->to(torch::kBFloat16).contiguous();
    mode = (qwc.numel() == dh && heads > 1) || (heads == 1) ? 1 : 2;
    TORCH_CHECK(qwc.numel() == (mode == 1 ? dh : dmodel));
  }
  torch::Tensor cosc, sinc;
  if (cos.has_value()) {
    cosc = cos->to(torch::kFloat32).contiguous();
    sinc = sin->to(torch::kFloat32).contiguous();
    TORCH_CHECK(cosc.size(0) == s && cosc.size(1) == dh / 2);
  }
  QkvPeers peers{};
  peers.world = (int)world;
  const torch::Tensor* tables[3] = {&peers_q, &peers_k, &peers_v};
  bf16** slots[3] = {peers.q, peers.k, peers.v};
  for (int t = 0; t < 3; ++t) {
    TORCH_CHECK(tables[t]->device().is_cpu() && tables[t]->scalar_type() == torch::kInt64 &&
                tables[t]->numel() >= world, "peer tables: CPU int64 tensors with one address per rank");
    for (int r = 0; r < world; ++r) {
      const int64_t addr = tables[t]->data_ptr<int64_t>()[r];
      TORCH_CHECK(addr != 0 && addr % 16 == 0, "peer destinations must be 16-byte aligned");
      slots[t][r] = reinterpret_cast<bf16*>(addr);
    }
  }
  auto rstd = torch::empty({(int64_t)b * s * 2 * (mode == 1 ? heads : 1)}, qkv.options().dtype(torch::kFloat32));
  launch_qkv_fwd(qkv, mode ? reinterpret_cast<const bf16*>(qwc.data_ptr()) : nullptr,
                 mode ? reinterpret_cast<const bf16*>(kwc.data_ptr()) : nullptr,
                 cos.has_value() ? cosc.data_ptr<float>() : nullptr,
                 cos.has_value() ? sinc.data_ptr<float>() : nullptr, nullptr, nullptr, nullptr,
                 rstd.data_ptr<float>(), b, s, (int)heads, dh, mode, (float)eps, (int)seq_total,
                 (int)seq_offset, peers);
  return rstd;
}

// Backward of the above, the same column-owner layout: thread i owns vector i of q, k or v
// (blockIdx.y) over a run of tokens, four per pass.  The weight gradient of the norm is eight
// registers per thread, combined over the heads in shared memory (per-head weights) or sent
// straight to memory (full-width weights) once per block.
template <int kMaxT>
__global__ void __launch_bounds__(kMaxT)
qkv_prepare_bwd_kernel(const bf16* __restrict__ gq, const bf16* __restrict__ gk,
                       const bf16* __restrict__ gv, const bf16* __restrict__ qkv,
                       const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                       const float* __restrict__ cosT, const float* __restrict__ sinT,
                       const float* __restrict__ rstd, bf16* __restrict__ gqkv,
                       float* __restrict__ gqw, float* __restrict__ gkw, int64_t tokens, int seq,
                       int heads, int dh, int mode, int seq_offset, int tokens_per_block, int64_t gq_sb,
                       int64_t gq_sh, int64_t gq_ss, int64_t gk_sb, int64_t gk_sh, int64_t gk_ss,
                       int64_t gv_sb, int64_t gv_sh, int64_t gv_ss) {
  constexpr int TB = kQkvTokensPerPass;
  __shared__ float red[2 * 32 * TB];
  __shared__ float wacc[256];                  // per-head weights: Dh <= 256 column sums over the heads
  const int i = threadIdx.x, nwarps = blockDim.x >> 5;
  const int which = blockIdx.y;
  const int dmodel = heads * dh;
  const int vec_per_head = dh / 8, vec_per_which = dmodel / 8;
  const bool act = i < vec_per_which;
  const int h = i / vec_per_head, j8 = i - h * vec_per_head;
  const bool normed = which < 2 && mode != 0;
  const bf16* gsrc = which == 0 ? gq : (which == 1 ? gk : gv);
  const int64_t sb = which == 0 ? gq_sb : (which == 1 ? gk_sb : gv_sb);
  const int64_t sh = which == 0 ? gq_sh : (which == 1 ? gk_sh : gv_sh);
  const int64_t ss = which == 0 ? gq_ss : (which == 1 ? gk_ss : gv_ss);
  float ww[8], wg[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { ww[j] = 1.f; wg[j] = 0.f; }
  if (act && normed)
    unpack8(*reinterpret_cast<const bf16x8*>((which == 0 ? qw : kw) + (mode == 1 ? j8 * 8 : i * 8)), ww);
  if (normed && mode == 1) {
    for (int t = i; t < dh; t += blockDim.x) wacc[t] = 0.f;
    __syncthreads();
  }
  const int64_t tok_begin = (int64_t)blockIdx.x * tokens_per_block;
  const int64_t tok_end = min(tok_begin + (int64_t)tokens_per_block, tokens);
  int parity = 0;
  for (int64_t tb = tok_begin; tb < tok_end; tb += TB) {
    bf16x8 graw[TB], xraw[TB];
    float rs[TB];
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      const int64_t tok = tb + t;
      graw[t].u = make_uint4(0u, 0u, 0u, 0u);
      xraw[t].u = make_uint4(0u, 0u, 0u, 0u);
      rs[t] = 0.f;
      if (act && tok < tok_end) {
        int b = (int)((unsigned)tb / (unsigned)seq), sidx = (int)tb - b * seq + t;     // 32-bit on purpose
        while (sidx >= seq) { sidx -= seq; ++b; }
        graw[t] = *reinterpret_cast<const bf16x8*>(gsrc + b * sb + h * sh + (int64_t)(seq_offset + sidx) * ss + j8 * 8);
        if (normed) {
          xraw[t] = *reinterpret_cast<const bf16x8*>(qkv + (tok * 3 + which) * dmodel + i * 8);
          rs[t] = mode == 1 ? rstd[(tok * 2 + which) * heads + h] : rstd[tok * 2 + which];
        }
      }
    }
    float g[TB][8], dot[TB];
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      unpack8(graw[t], g[t]);
      dot[t] = 0.f;
      const int64_t tok = tb + t;
      if (which < 2 && cosT != nullptr && act && tok < tok_end) {     // transpose of the rotation
        const int sidx = (int)((unsigned)tok % (unsigned)seq);
        const float4 c = *reinterpret_cast<const float4*>(cosT + (int64_t)sidx * (dh / 2) + j8 * 4);
        const float4 sn = *reinterpret_cast<const float4*>(sinT + (int64_t)sidx * (dh / 2) + j8 * 4);
        const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float g0 = g[t][2 * p], g1 = g[t][2 * p + 1];
          g[t][2 * p] = g0 * cc[p] + g1 * sv[p];
          g[t][2 * p + 1] = -g0 * sv[p] + g1 * cc[p];
        }
      }
      if (normed) {
        float xv[8];
        unpack8(xraw[t], xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = xv[j] * rs[t];
          dot[t] += g[t][j] * ww[j] * xh;
          wg[j] += g[t][j] * xh;
        }
      }
    }
    if (normed) {                                   // uniform over the block
      if (mode == 1) {
#pragma unroll
        for (int t = 0; t < TB; ++t) dot[t] = group_sum(dot[t], vec_per_head) / (float)dh;
      } else {
        block_sum_vals<TB>(dot, red + parity * 32 * TB, nwarps);
        parity ^= 1;
#pragma unroll
        for (int t = 0; t < TB; ++t) dot[t] /= (float)dmodel;
      }
    }
#pragma unroll
    for (int t = 0; t < TB; ++t) {
      const int64_t tok = tb + t;
      if (!act || tok >= tok_end) continue;
      float o[8];
      if (normed) {
        float xv[8];
        unpack8(xraw[t], xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs[t] * (g[t][j] * ww[j] - xv[j] * rs[t] * dot[t]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = g[t][j];
      }
      *reinterpret_cast<bf16x8*>(gqkv + (tok * 3 + which) * dmodel + i * 8) = pack8(o);
    }
  }
  if (!normed) return;
  float* gw = which == 0 ? gqw : gkw;
  if (mode == 1) {
    if (act) {
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(&wacc[j8 * 8 + j], wg[j]);
    }
    __syncthreads();
    for (int t = i; t < dh; t += blockDim.x) atomicAdd(gw + t, wacc[t]);
  } else if (act) {
    red_add_v4(gw + i * 8, wg);
    red_add_v4(gw + i * 8 + 4, wg + 4);
  }
}

std::vector<torch::Tensor> qkv_prepare_bwd(torch::Tensor gq, torch::Tensor gk, torch::Tensor gv,
                                           torch::Tensor qkv, c10::optional<torch::Tensor> qw,
                                           c10::optional<torch::Tensor> kw,
                                           c10::optional<torch::Tensor> cos,
                                           c10::optional<torch::Tensor> sin, torch::Tensor rstd,
                                           int64_t heads, int64_t seq_offset) {
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 3 && qkv.scalar_type() == torch::kBFloat16 &&
              qkv.is_contiguous());
  TORCH_CHECK(qw.has_value() == kw.has_value() && cos.has_value() == sin.has_value(),
              "qkv_prepare_bwd: q/k norm weights and cos/sin tables come in pairs");
  VRL_CHECK_OPERAND(gq, qkv);
  VRL_CHECK_OPERAND(gk, qkv);
  VRL_CHECK_OPERAND(gv, qkv);
  VRL_CHECK_OPERAND(qw, qkv);
  VRL_CHECK_OPERAND(kw, qkv);
  VRL_CHECK_OPERAND(cos, qkv);
  VRL_CHECK_OPERAND(sin, qkv);
  VRL_CHECK_OPERAND(rstd, qkv, torch::kFloat32);
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int b = (int)qkv.size(0), s = (int)qkv.size(1);
  const int dmodel = (int)(qkv.size(2) / 3), dh = dmodel / (int)heads;
  // gradients arrive as [B, H, S_total, Dh] views with arbitrary (16-byte aligned) strides
  auto usable = [&](torch::Tensor& g) {
    TORCH_CHECK(g.dim() == 4 && g.size(0) == b && g.size(1) == heads && g.size(3) == dh &&
                seq_offset + s <= g.size(2), "qkv_prepare_bwd: gradient shape");
    const bool ok = g.scalar_type() == torch::kBFloat16 && g.stride(3) == 1 && g.stride(0) % 8 == 0 &&
                    g.stride(1) % 8 == 0 && g.stride(2) % 8 == 0 &&
                    reinterpret_cast<uintptr_t>(g.data_ptr()) % 16 == 0;
    if (!ok) g = g.to(torch::kBFloat16).contiguous();
  };
  usable(gq);
  usable(gk);
  usable(gv);
  int mode = 0;
  torch::Tensor qwc, kwc;
  if (qw.has_value()) {
    qwc = qw->to(torch::kBFloat16).contiguous();
    kwc = kw->to(torch::kBFloat16).contiguous();
    mode = (qwc.numel() == dh && heads > 1) || (heads == 1) ? 1 : 2;
  }
  torch::Tensor cosc, sinc;
  if (cos.has_value()) {
    cosc = cos->to(torch::kFloat32).contiguous();
    sinc = sin->to(torch::kFloat32).contiguous();
  }
  const int wlen = mode == 1 ? dh : dmodel;
  auto gqkv = torch::empty_like(qkv);
  auto gqw = torch::zeros({mode ? wlen : 1}, qkv.options().dtype(torch::kFloat32));
  auto gkw = torch::zeros_like(gqw);
  const int64_t tokens = (int64_t)b * s;
  check_qkv_geometry(dmodel, dh);
  TORCH_CHECK(tokens < (1ll << 31), "qkv_prepare_bwd: token count must fit 31 bits");
  if (tokens == 0) return {gqkv, gqw, gkw};
  auto stream = at::cuda::getCurrentCUDAStream();
  const int threads = (dmodel / 8 + 31) / 32 * 32;
  const int tpb = qkv_tokens_per_block(tokens);
  dim3 grid((unsigned)((tokens + tpb - 1) / tpb), 3);
  VRL_DISPATCH_COLS(threads, qkv_prepare_bwd_kernel<kMaxT><<<grid, threads, 0, stream>>>(
      reinterpret_cast<const bf16*>(gq.data_ptr()), reinterpret_cast<const bf16*>(gk.data_ptr()),
      reinterpret_cast<const bf16*>(gv.data_ptr()), reinterpret_cast<const bf16*>(qkv.data_ptr()),
      mode ? reinterpret_cast<const bf16*>(qwc.data_ptr()) : nullptr,
      mode ? reinterpret_cast<const bf16*>(kwc.data_ptr()) : nullptr,
      cos.has_value() ? cosc.data_ptr<float>() : nullptr,
      cos.has_value() ? sinc.data_ptr<float>() : nullptr, rstd.data_ptr<float>(),
      reinterpret_cast<bf16*>(gqkv.data_ptr()), gqw.data_ptr<float>(), gkw.data_ptr<float>(),
      tokens, s, (int)heads, dh, mode, (int)seq_offset, tpb, gq.stride(0), gq.stride(1), gq.stride(2),
      gk.stride(0), gk.stride(1), gk.stride(2), gv.stride(0), gv.stride(1), gv.stride(2)));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {gqkv, gqw, gkw};
}

}  // namespace vrl
