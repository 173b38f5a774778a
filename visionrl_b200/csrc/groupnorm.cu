// GroupNorm (+ optional SiLU) for channels-last bf16 activations, forward only: the convolutional
// decoders that turn latents into reward-model inputs run without gradients, and their group
// norms over [N, H, W, C] tensors of half a gigabyte each are pure bandwidth.
// Two passes: per-(sample, group) sums with fp32 atomics, then one streaming normalise pass.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"
#include "ops.h"

namespace vrl {

namespace {

constexpr int kGnThreads = 256;
constexpr int kGnPixelsPerBlock = 1024;

// x viewed as [N, HW, C]; thread t owns channel vector (t % V) of pixels t / V, t / V + 256 / V, ...
__global__ void __launch_bounds__(kGnThreads)
groupnorm_stats_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ stats, int64_t hw,
                       int c, int groups) {
  extern __shared__ float ch_acc[];          // [2][c]
  const int n = blockIdx.y;
  const int vecs = c / 8;
  const int v = threadIdx.x % vecs, p0 = threadIdx.x / vecs, pstride = kGnThreads / vecs;
  for (int i = threadIdx.x; i < 2 * c; i += kGnThreads) ch_acc[i] = 0.f;
  __syncthreads();
  const int64_t begin = (int64_t)blockIdx.x * kGnPixelsPerBlock;
  const int64_t end = min(hw, begin + kGnPixelsPerBlock);
  const __nv_bfloat16* base = x + (int64_t)n * hw * c;
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, q[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int64_t p = begin + p0; p < end; p += pstride) {
    float f[8];
    unpack8(*reinterpret_cast<const bf16x8*>(base + p * c + v * 8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) { s[j] += f[j]; q[j] += f[j] * f[j]; }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    atomicAdd(&ch_acc[v * 8 + j], s[j]);
    atomicAdd(&ch_acc[c + v * 8 + j], q[j]);
  }
  __syncthreads();
  const int cpg = c / groups;
  for (int g = threadIdx.x; g < groups; g += kGnThreads) {
    float gs = 0.f, gq = 0.f;
    for (int k = 0; k < cpg; ++k) { gs += ch_acc[g * cpg + k]; gq += ch_acc[c + g * cpg + k]; }
    atomicAdd(&stats[((int64_t)n * groups + g) * 2], gs);
    atomicAdd(&stats[((int64_t)n * groups + g) * 2 + 1], gq);
  }
}

__global__ void __launch_bounds__(kGnThreads)
groupnorm_apply_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ stats,
                       const __nv_bfloat16* __restrict__ weight, const __nv_bfloat16* __restrict__ bias,
                       __nv_bfloat16* __restrict__ y, int64_t hw, int c, int groups, float eps,
                       int apply_silu) {
  const int n = blockIdx.y;
  const int vecs = c / 8;
  const int v = threadIdx.x % vecs, p0 = threadIdx.x / vecs, pstride = kGnThreads / vecs;
  const int cpg = c / groups;
  const float inv_count = 1.f / ((float)hw * (float)cpg);
  float scale[8], shift[8], w[8], b[8];
  unpack8(*reinterpret_cast<const bf16x8*>(weight + v * 8), w);
  unpack8(*reinterpret_cast<const bf16x8*>(bias + v * 8), b);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int g = (v * 8 + j) / cpg;
    const float mean = stats[((int64_t)n * groups + g) * 2] * inv_count;
    const float var = fmaxf(stats[((int64_t)n * groups + g) * 2 + 1] * inv_count - mean * mean, 0.f);
    const float rstd = rsqrtf(var + eps);
    scale[j] = rstd * w[j];
    shift[j] = b[j] - mean * scale[j];
  }
  const int64_t begin = (int64_t)blockIdx.x * kGnPixelsPerBlock;
  const int64_t end = min(hw, begin + kGnPixelsPerBlock);
  const __nv_bfloat16* base = x + (int64_t)n * hw * c;
  __nv_bfloat16* out = y + (int64_t)n * hw * c;
  for (int64_t p = begin + p0; p < end; p += pstride) {
    float f[8], o[8];
    unpack8(*reinterpret_cast<const bf16x8*>(base + p * c + v * 8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float t = f[j] * scale[j] + shift[j];
      o[j] = apply_silu ? silu(t) : t;
    }
    *reinterpret_cast<bf16x8*>(out + p * c + v * 8) = pack8(o);
  }
}

}  // namespace

// x: [N, C, H, W] bf16 in channels-last memory format.  Returns a tensor of the same format.
torch::Tensor groupnorm_nhwc(torch::Tensor x, torch::Tensor weight, torch::Tensor bias, int64_t groups,
                             double eps, bool apply_silu) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(x.is_contiguous(at::MemoryFormat::ChannelsLast), "groupnorm_nhwc: channels-last input");
  const int64_t n = x.size(0), c = x.size(1), hw = x.size(2) * x.size(3);
  TORCH_CHECK(c % 8 == 0 && c % groups == 0 && kGnThreads % (c / 8) == 0 && c / 8 <= kGnThreads,
              "groupnorm_nhwc: unsupported channel count ", c);
  TORCH_CHECK(n <= 65535 && weight.numel() == c && bias.numel() == c);
  VRL_CHECK_OPERAND(weight, x);
  VRL_CHECK_OPERAND(bias, x);
  const c10::cuda::CUDAGuard guard(x.device());
  auto w = weight.to(torch::kBFloat16).contiguous();
  auto b = bias.to(torch::kBFloat16).contiguous();
  auto y = torch::empty_like(x);          // preserves the channels-last strides
  if (n == 0 || hw == 0) return y;
  auto stats = torch::zeros({n, groups, 2}, x.options().dtype(torch::kFloat32));
  auto stream = at::cuda::getCurrentCUDAStream();
  dim3 grid((unsigned)((hw + kGnPixelsPerBlock - 1) / kGnPixelsPerBlock), (unsigned)n);
  groupnorm_stats_kernel<<<grid, kGnThreads, 2 * c * sizeof(float), stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), stats.data_ptr<float>(), hw, (int)c, (int)groups);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  groupnorm_apply_kernel<<<grid, kGnThreads, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), stats.data_ptr<float>(),
      reinterpret_cast<const __nv_bfloat16*>(w.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(b.data_ptr()),
      reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), hw, (int)c, (int)groups, (float)eps, apply_silu ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

}  // namespace vrl
