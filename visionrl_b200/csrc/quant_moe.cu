// Weight-only int4 skinny GEMM for decode (M <= 32 rows) and the mixture-of-experts routing
// kernels (gate softmax + top-k, stable expert-major permutation, row gather, weighted combine).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "ops.h"

namespace vrl {

namespace {

// ------------------------------------------------------------------------------------------
// y[M, N] = x[M, K] . dequant(W)[N, K]^T.  W is stored as int32 words of eight 4-bit codes
// (code c -> (c - 8) * scale, low nibble = lowest k), scales bf16 per (row, group of `group` k).
// Decode is bound by the weight bytes, so every weight word is read once per 16 activation rows
// and the activations are staged in shared memory in 256-wide K chunks.
// Block = 8 warps, each warp owns 4 output columns; lane owns 8 consecutive k of the chunk.
// ------------------------------------------------------------------------------------------
constexpr int kGemvWarps = 8, kGemvCols = 4, kGemvChunk = 256, kGemvRows = 16;

__global__ void __launch_bounds__(kGemvWarps * 32)
int4_gemv_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ qw,
                 const __nv_bfloat16* __restrict__ scales, const __nv_bfloat16* __restrict__ bias,
                 __nv_bfloat16* __restrict__ y, int m, int n, int k, int group) {
  __shared__ __align__(16) __nv_bfloat16 xs[kGemvRows][kGemvChunk];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col0 = (blockIdx.x * kGemvWarps + warp) * kGemvCols;
  const int words_per_row = k / 8, groups_per_row = k / group;
  for (int r0 = 0; r0 < m; r0 += kGemvRows) {
    float acc[kGemvRows][kGemvCols];
#pragma unroll
    for (int i = 0; i < kGemvRows; ++i)
#pragma unroll
      for (int c = 0; c < kGemvCols; ++c) acc[i][c] = 0.f;
    for (int k0 = 0; k0 < k; k0 += kGemvChunk) {
      __syncthreads();
      // stage activations: 16 rows x 256 k = 512 vectors of 8
      for (int v = threadIdx.x; v < kGemvRows * (kGemvChunk / 8); v += kGemvWarps * 32) {
        const int rr = v / (kGemvChunk / 8), kk = (v % (kGemvChunk / 8)) * 8;
        bf16x8 val;
        val.u = make_uint4(0u, 0u, 0u, 0u);
        if (r0 + rr < m) val = *reinterpret_cast<const bf16x8*>(x + (int64_t)(r0 + rr) * k + k0 + kk);
        *reinterpret_cast<bf16x8*>(&xs[rr][kk]) = val;
      }
      __syncthreads();
      float wv[kGemvCols][8];
#pragma unroll
      for (int c = 0; c < kGemvCols; ++c) {
        const int col = col0 + c;
        if (col < n) {
          const int kidx = k0 + lane * 8;
          const uint32_t word = (uint32_t)qw[(int64_t)col * words_per_row + kidx / 8];
          const float sc = __bfloat162float(scales[(int64_t)col * groups_per_row + kidx / group]);
#pragma unroll
          for (int j = 0; j < 8; ++j) wv[c][j] = (float)((int)((word >> (4 * j)) & 15u) - 8) * sc;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) wv[c][j] = 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < kGemvRows; ++i) {
        float xv[8];
        unpack8(*reinterpret_cast<const bf16x8*>(&xs[i][lane * 8]), xv);
#pragma unroll
        for (int c = 0; c < kGemvCols; ++c)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][c] = fmaf(xv[j], wv[c][j], acc[i][c]);
      }
    }
#pragma unroll
    for (int i = 0; i < kGemvRows; ++i)
#pragma unroll
      for (int c = 0; c < kGemvCols; ++c) {
        const float v = warp_sum(acc[i][c]);
        const int col = col0 + c;
        if (lane == 0 && r0 + i < m && col < n) {
          const float b = bias ? __bfloat162float(bias[col]) : 0.f;
          y[(int64_t)(r0 + i) * n + col] = __float2bfloat16_rn(v + b);
        }
      }
  }
}

// ------------------------------------------------------------------------------------------
// Gate: softmax over experts, top-k by probability (ties -> lower index), weights renormalised
// to sum 1.  One thread per token; E <= 64.
// ------------------------------------------------------------------------------------------
constexpr int kMaxExperts = 64, kMaxTopK = 8;

template <typename T>
__global__ void moe_gate_topk_kernel(const T* __restrict__ logits, float* __restrict__ weights,
                                     int32_t* __restrict__ experts, int tokens, int e, int topk) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  float p[kMaxExperts];
  float mx = -INFINITY;
  for (int i = 0; i < e; ++i) { p[i] = to_f<T>(logits[(int64_t)t * e + i]); mx = fmaxf(mx, p[i]); }
  float sum = 0.f;
  for (int i = 0; i < e; ++i) { p[i] = __expf(p[i] - mx); sum += p[i]; }
  float chosen_w[kMaxTopK];
  int chosen_i[kMaxTopK];
  float tot = 0.f;
  for (int s = 0; s < topk; ++s) {
    int best = 0;
    float bv = -1.f;
    for (int i = 0; i < e; ++i)
      if (p[i] > bv) { bv = p[i]; best = i; }
    chosen_w[s] = bv / sum;
    chosen_i[s] = best;
    tot += chosen_w[s];
    p[best] = -2.f;
  }
  for (int s = 0; s < topk; ++s) {
    weights[(int64_t)t * topk + s] = chosen_w[s] / tot;
    experts[(int64_t)t * topk + s] = chosen_i[s];
  }
}

// ------------------------------------------------------------------------------------------
// Stable expert-major permutation of the flat (token, slot) list.  One block of 1024 threads;
// thread t owns a contiguous run of entries, experts are placed one after another with a block
// exclusive scan of the per-thread counts.
//   perm[pos]  = flat index of the entry placed at sorted position pos
//   inv[flat]  = sorted position of the flat entry
//   offsets[e] = first sorted position of expert e, offsets[E] = total
// With pad > 1 every expert's run starts on a multiple of `pad` (the tile height of the grouped
// product): the sorted positions then live in a padded row space whose unused slots keep the
// perm value they were initialised with (-1), and tile_expert[t] names the expert of padded tile t.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_permute_kernel(const int32_t* __restrict__ experts, int32_t* __restrict__ perm,
                   int32_t* __restrict__ inv, int32_t* __restrict__ offsets,
                   int32_t* __restrict__ tile_expert, int n, int e, int pad) {
  __shared__ int warp_tot[32];
  __shared__ int base_s;
  const int per = (n + 1023) / 1024;
  const int lo = min(n, (int)threadIdx.x * per), hi = min(n, lo + per);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) { base_s = 0; offsets[0] = 0; }
  __syncthreads();
  for (int ex = 0; ex < e; ++ex) {
    int c = 0;
    for (int i = lo; i < hi; ++i) c += (experts[i] == ex);
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = warp_tot[lane], wi = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += v;
      }
      warp_tot[lane] = wi - w;            // exclusive prefix of the warp totals
      if (lane == 31) offsets[ex + 1] = (base_s + wi + pad - 1) / pad * pad;
    }
    __syncthreads();
    if (tile_expert != nullptr) {
      for (int t = base_s / pad + threadIdx.x; t < offsets[ex + 1] / pad; t += blockDim.x) tile_expert[t] = ex;
    }
    int pos = base_s + warp_tot[warp] + incl - c;
    for (int i = lo; i < hi; ++i)
      if (experts[i] == ex) { perm[pos] = i; inv[i] = pos; ++pos; }
    __syncthreads();
    if (threadIdx.x == 0) base_s = offsets[ex + 1];
    __syncthreads();
  }
}

// xp[pos, :] = x[perm[pos] / topk, :]
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                       const int32_t* __restrict__ perm,
                                       __nv_bfloat16* __restrict__ xp, int dim, int topk) {
  const int64_t pos = blockIdx.x;
  const int flat = perm[pos];
  bf16x8* dst = reinterpret_cast<bf16x8*>(xp + pos * dim);
  if (flat < 0) {                      // a padding row of the padded layout
    bf16x8 z;
    z.u = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = z;
    return;
  }
  const int64_t tok = flat / topk;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(x + tok * dim);
  for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = src[i];
}

// Backward of the combine with respect to the permuted rows: every row has exactly one consumer,
// g_yp[pos, :] = w[perm[pos]] * gy[perm[pos] / topk, :] (zero for padding rows).
__global__ void moe_combine_bwd_rows_kernel(const __nv_bfloat16* __restrict__ gy,
                                            const int32_t* __restrict__ perm, const float* __restrict__ w,
                                            __nv_bfloat16* __restrict__ g_yp, int dim, int topk) {
  const int64_t pos = blockIdx.x;
  const int flat = perm[pos];
  bf16x8* dst = reinterpret_cast<bf16x8*>(g_yp + pos * dim);
  if (flat < 0) {
    bf16x8 z;
    z.u = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = z;
    return;
  }
  const float ws = w[flat];
  const bf16x8* src = reinterpret_cast<const bf16x8*>(gy + (int64_t)(flat / topk) * dim);
  for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) {
    float f[8];
    unpack8(src[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= ws;
    dst[i] = pack8(f);
  }
}

// Backward of the combine with respect to the gate weights: g_w[t, s] = <yp[inv[t, s], :], gy[t, :]>.
__global__ void __launch_bounds__(128)
moe_combine_bwd_weights_kernel(const __nv_bfloat16* __restrict__ yp, const __nv_bfloat16* __restrict__ gy,
                               const int32_t* __restrict__ inv, float* __restrict__ g_w, int dim, int topk) {
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  for (int sl = 0; sl < topk; ++sl) {
    const int64_t pos = inv[t * topk + sl];
    float acc = 0.f;
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) {
      float a[8], b[8];
      unpack8(reinterpret_cast<const bf16x8*>(yp + pos * dim)[i], a);
      unpack8(reinterpret_cast<const bf16x8*>(gy + t * dim)[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(a[j], b[j], acc);
    }
    const float total = block_sum(acc, red);
    if (threadIdx.x == 0) g_w[t * topk + sl] = total;
  }
}

// Per-expert column sums of a padded, expert-sorted matrix (bias gradients): out[e, c] += sum of
// g[r, c] over a chunk of the expert's rows; one thread per column, chunks of rows in blockIdx.z.
constexpr int kSegRows = 256;
__global__ void moe_segment_colsum_kernel(const __nv_bfloat16* __restrict__ g, const int32_t* __restrict__ offsets,
                                          float* __restrict__ out, int n) {
  const int e = blockIdx.y;
  const int lo = offsets[e] + blockIdx.z * kSegRows, hi = min(offsets[e + 1], lo + kSegRows);
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n || lo >= hi) return;
  float acc = 0.f;
  for (int r = lo; r < hi; ++r) acc += __bfloat162float(g[(int64_t)r * n + c]);
  atomicAdd(out + (int64_t)e * n + c, acc);
}

// y[t, :] = sum_s w[t, s] * yp[inv[t * topk + s], :]
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ yp,
                                   const int32_t* __restrict__ inv, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, int dim, int topk) {
  const int64_t t = blockIdx.x;
  for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < topk; ++s) {
      const int64_t pos = inv[t * topk + s];
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(yp + pos * dim)[i], f);
      const float ws = w[t * topk + s];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(ws, f[j], acc[j]);
    }
    reinterpret_cast<bf16x8*>(y + t * dim)[i] = pack8(acc);
  }
}

}  // namespace

// ============================================================================== host wrappers
torch::Tensor int4_gemv(torch::Tensor x, torch::Tensor qweight, torch::Tensor scales,
                        c10::optional<torch::Tensor> bias, int64_t group) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.is_contiguous());
  TORCH_CHECK(qweight.scalar_type() == torch::kInt32 && qweight.dim() == 2 && qweight.is_contiguous());
  TORCH_CHECK(scales.scalar_type() == torch::kBFloat16 && scales.is_contiguous());
  const int64_t m = x.size(0), k = x.size(1), n = qweight.size(0);
  TORCH_CHECK(m <= 32, "int4_gemv: at most 32 activation rows (decode batches)");
  TORCH_CHECK(k % kGemvChunk == 0 && qweight.size(1) * 8 == k, "int4_gemv: K must be a multiple of 256");
  TORCH_CHECK(group > 0 && group % 8 == 0 && k % group == 0 && scales.numel() == n * (k / group),
              "int4_gemv: scales must be [N, K / group]");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0);
  VRL_CHECK_OPERAND(qweight, x);
  VRL_CHECK_OPERAND(scales, x);
  VRL_CHECK_OPERAND(bias, x);
  const c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty({m, n}, x.options());
  if (m == 0 || n == 0) return y;
  const __nv_bfloat16* bias_p = nullptr;
  torch::Tensor bias_c;
  if (bias.has_value()) {
    bias_c = bias->to(torch::kBFloat16).contiguous();
    TORCH_CHECK(bias_c.numel() == n);
    bias_p = reinterpret_cast<const __nv_bfloat16*>(bias_c.data_ptr());
  }
  const int cols_per_block = kGemvWarps * kGemvCols;
  int4_gemv_kernel<<<(int)((n + cols_per_block - 1) / cols_per_block), kGemvWarps * 32, 0,
                     at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), qweight.data_ptr<int32_t>(),
      reinterpret_cast<const __nv_bfloat16*>(scales.data_ptr()), bias_p,
      reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), (int)m, (int)n, (int)k, (int)group);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

std::vector<torch::Tensor> moe_gate_topk(torch::Tensor logits, int64_t topk) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  const int64_t tokens = logits.size(0), e = logits.size(1);
  TORCH_CHECK(e <= kMaxExperts && topk >= 1 && topk <= kMaxTopK && topk <= e,
              "moe_gate_topk: at most 64 experts and top-8");
  const c10::cuda::CUDAGuard guard(logits.device());
  auto w = torch::empty({tokens, topk}, logits.options().dtype(torch::kFloat32));
  auto idx = torch::empty({tokens, topk}, logits.options().dtype(torch::kInt32));
  if (tokens == 0) return {w, idx};
  auto stream = at::cuda::getCurrentCUDAStream();
  const int threads = 128, blocks = (int)((tokens + threads - 1) / threads);
  if (logits.scalar_type() == torch::kBFloat16) {
    moe_gate_topk_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits.data_ptr()), w.data_ptr<float>(),
        idx.data_ptr<int32_t>(), (int)tokens, (int)e, (int)topk);
  } else {
    TORCH_CHECK(logits.scalar_type() == torch::kFloat32);
    moe_gate_topk_kernel<float><<<blocks, threads, 0, stream>>>(
        logits.data_ptr<float>(), w.data_ptr<float>(), idx.data_ptr<int32_t>(), (int)tokens, (int)e,
        (int)topk);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {w, idx};
}

// {perm, inv, offsets, tile_expert}.  pad <= 1: dense layout (perm has one entry per (token, slot),
// tile_expert is empty).  pad > 1: every expert's run is padded to a multiple of `pad` rows; perm
// then has (ceil(n / pad) + E) * pad entries, -1 in the padding, and tile_expert has one entry per
// `pad` rows (-1 past the last expert).  The sizes depend on n and E only, never on the routing.
std::vector<torch::Tensor> moe_permute(torch::Tensor experts, int64_t num_experts, int64_t pad) {
  TORCH_CHECK(experts.is_cuda() && experts.scalar_type() == torch::kInt32 && experts.is_contiguous());
  const c10::cuda::CUDAGuard guard(experts.device());
  const int64_t n = experts.numel();
  TORCH_CHECK(n < (1 << 30) && num_experts >= 1);
  if (pad < 1) pad = 1;
  const int64_t slots = pad > 1 ? ((n + pad - 1) / pad + num_experts) * pad : n;
  auto perm = pad > 1 ? torch::full({slots}, -1, experts.options()) : torch::empty({n}, experts.options());
  auto inv = torch::empty({n}, experts.options());
  auto offsets = torch::zeros({num_experts + 1}, experts.options());
  auto tile_expert = pad > 1 ? torch::full({slots / pad}, -1, experts.options()) : torch::empty({0}, experts.options());
  if (n == 0) return {perm, inv, offsets, tile_expert};
  moe_permute_kernel<<<1, 1024, 0, at::cuda::getCurrentCUDAStream()>>>(
      experts.data_ptr<int32_t>(), perm.data_ptr<int32_t>(), inv.data_ptr<int32_t>(),
      offsets.data_ptr<int32_t>(), pad > 1 ? tile_expert.data_ptr<int32_t>() : nullptr, (int)n,
      (int)num_experts, (int)pad);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {perm, inv, offsets, tile_expert};
}

// {d(yp) [rows, D] bf16, d(weights) [T, k] fp32} of y[t] = sum_s w[t, s] yp[inv[t, s]]
std::vector<torch::Tensor> moe_combine_bwd(torch::Tensor gy, torch::Tensor yp, torch::Tensor perm,
                                           torch::Tensor inv, torch::Tensor weights) {
  TORCH_CHECK(yp.is_cuda() && yp.dim() == 2 && yp.scalar_type() == torch::kBFloat16 && yp.is_contiguous());
  TORCH_CHECK(gy.dim() == 2 && gy.scalar_type() == torch::kBFloat16 && gy.is_contiguous() && gy.size(1) == yp.size(1));
  TORCH_CHECK(weights.dim() == 2 && weights.scalar_type() == torch::kFloat32 && weights.is_contiguous() &&
              weights.size(0) == gy.size(0));
  TORCH_CHECK(perm.scalar_type() == torch::kInt32 && perm.is_contiguous() && perm.numel() == yp.size(0) &&
              inv.scalar_type() == torch::kInt32 && inv.is_contiguous() && inv.numel() == weights.numel() &&
              yp.size(1) % 8 == 0, "moe_combine_bwd: permutation tables");
  VRL_CHECK_OPERAND(gy, yp);
  VRL_CHECK_OPERAND(perm, yp);
  VRL_CHECK_OPERAND(inv, yp);
  VRL_CHECK_OPERAND(weights, yp);
  const c10::cuda::CUDAGuard guard(yp.device());
  auto g_yp = torch::empty_like(yp);
  auto g_w = torch::empty_like(weights);
  auto stream = at::cuda::getCurrentCUDAStream();
  const int dim = (int)yp.size(1), topk = (int)weights.size(1);
  if (yp.size(0) > 0)
    moe_combine_bwd_rows_kernel<<<(int)yp.size(0), 128, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(gy.data_ptr()), perm.data_ptr<int32_t>(), weights.data_ptr<float>(),
        reinterpret_cast<__nv_bfloat16*>(g_yp.data_ptr()), dim, topk);
  if (gy.size(0) > 0)
    moe_combine_bwd_weights_kernel<<<(int)gy.size(0), 128, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(yp.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(gy.data_ptr()),
        inv.data_ptr<int32_t>(), g_w.data_ptr<float>(), dim, topk);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {g_yp, g_w};
}

// fp32 [E, N]: column sums of g [rows, N] over every expert's row range offsets[e] .. offsets[e + 1]
torch::Tensor moe_segment_colsum(torch::Tensor g, torch::Tensor offsets, int64_t num_experts) {
  TORCH_CHECK(g.is_cuda() && g.dim() == 2 && g.scalar_type() == torch::kBFloat16 && g.is_contiguous());
  VRL_CHECK_OPERAND(offsets, g, torch::kInt32, num_experts + 1);
  TORCH_CHECK(offsets.is_contiguous());
  const c10::cuda::CUDAGuard guard(g.device());
  auto out = torch::zeros({num_experts, g.size(1)}, g.options().dtype(torch::kFloat32));
  if (g.numel() == 0) return out;
  const int n = (int)g.size(1);
  dim3 grid((n + 255) / 256, (unsigned)num_experts, (unsigned)((g.size(0) + kSegRows - 1) / kSegRows));
  TORCH_CHECK(grid.z <= 65535, "moe_segment_colsum: too many rows");
  moe_segment_colsum_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(g.data_ptr()), offsets.data_ptr<int32_t>(), out.data_ptr<float>(), n);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

torch::Tensor moe_gather_rows(torch::Tensor x, torch::Tensor perm, int64_t topk) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.is_contiguous());
  TORCH_CHECK(x.size(1) % 8 == 0 && perm.scalar_type() == torch::kInt32 && perm.is_contiguous());
  VRL_CHECK_OPERAND(perm, x);
  const c10::cuda::CUDAGuard guard(x.device());
  auto xp = torch::empty({perm.numel(), x.size(1)}, x.options());
  if (perm.numel() == 0) return xp;
  moe_gather_rows_kernel<<<(int)perm.numel(), 128, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), perm.data_ptr<int32_t>(),
      reinterpret_cast<__nv_bfloat16*>(xp.data_ptr()), (int)x.size(1), (int)topk);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return xp;
}

torch::Tensor moe_combine(torch::Tensor yp, torch::Tensor inv, torch::Tensor weights) {
  TORCH_CHECK(yp.is_cuda() && yp.dim() == 2 && yp.scalar_type() == torch::kBFloat16 && yp.is_contiguous());
  TORCH_CHECK(weights.dim() == 2 && weights.scalar_type() == torch::kFloat32 && weights.is_contiguous());
  TORCH_CHECK(inv.scalar_type() == torch::kInt32 && inv.numel() == weights.numel() && yp.size(1) % 8 == 0);
  VRL_CHECK_OPERAND(inv, yp);
  VRL_CHECK_OPERAND(weights, yp);
  TORCH_CHECK(inv.is_contiguous(), "moe_combine: inverse permutation must be contiguous");
  const c10::cuda::CUDAGuard guard(yp.device());
  const int64_t tokens = weights.size(0), topk = weights.size(1);
  auto y = torch::empty({tokens, yp.size(1)}, yp.options());
  if (tokens == 0) return y;
  moe_combine_kernel<<<(int)tokens, 128, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(yp.data_ptr()), inv.data_ptr<int32_t>(),
      weights.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), (int)yp.size(1),
      (int)topk);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

}  // namespace vrl
