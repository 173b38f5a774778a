// Fused element-wise / reduction kernels: SDE step + Gaussian log-prob (K5), GRPO and
// TokenGRPO losses (K6), per-sample MSE (K14), flat AdamW and gradient norm (K11).
// All reductions are two-stage with a fixed summation order, so results are bitwise
// reproducible between the rollout and the training replay of the same step.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <curand_kernel.h>

#include "common.cuh"
#include "ops.h"

namespace vrl {

// ------------------------------------------------------------------------------------------
// K5: mu = a x + b v ; x' = mu + scale * eps (or given, or x + dt v) ; sum (x' - mu)^2
// ------------------------------------------------------------------------------------------
constexpr int kSdeThreads = 256;
constexpr int kSdeElemsPerBlock = kSdeThreads * 4 * 4;   // 4 float4 per thread

// The step's arithmetic, spelled with explicitly rounded operations: the rollout kernel and the
// replay kernel must produce the same bits for the same inputs, which an expression left to the
// compiler's choice of multiply-add contraction does not guarantee across two kernels.
__device__ __forceinline__ float sde_mean(float ca, float x, float cb, float v) {
  return __fmaf_rn(ca, x, __fmul_rn(cb, v));
}
__device__ __forceinline__ float sde_sample(float mu, float cs, float e) { return __fmaf_rn(cs, e, mu); }
__device__ __forceinline__ float sde_ode(float x, float cdt, float v) { return __fmaf_rn(cdt, v, x); }
__device__ __forceinline__ float sde_sq4(float acc, const float4& pr, const float4& mu) {
  const float d0 = __fsub_rn(pr.x, mu.x), d1 = __fsub_rn(pr.y, mu.y), d2 = __fsub_rn(pr.z, mu.z),
              d3 = __fsub_rn(pr.w, mu.w);
  return __fmaf_rn(d3, d3, __fmaf_rn(d2, d2, __fmaf_rn(d1, d1, __fmaf_rn(d0, d0, acc))));
}

__global__ void __launch_bounds__(kSdeThreads)
sde_step_fwd_kernel(const float* __restrict__ v, const float* __restrict__ x,
                    const float* __restrict__ a, const float* __restrict__ b,
                    const float* __restrict__ scale, const float* __restrict__ dt,
                    const float* __restrict__ prev_in, const float* __restrict__ noise,
                    float* __restrict__ prev_out, float* __restrict__ mean_out,
                    float* __restrict__ partial, int64_t n, int blocks_per_sample,
                    int deterministic, int vec_ok) {
  __shared__ float red[32];
  const int sample = blockIdx.y;
  const float ca = a[sample], cb = b[sample], cs = scale[sample], cdt = dt[sample];
  const int64_t base = (int64_t)sample * n;
  const int64_t start = (int64_t)blockIdx.x * kSdeElemsPerBlock;
  float acc = 0.f;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int64_t i = start + ((int64_t)it * kSdeThreads + threadIdx.x) * 4;
    if (vec_ok && i + 3 < n) {
      const float4 vv = *reinterpret_cast<const float4*>(v + base + i);
      const float4 xx = *reinterpret_cast<const float4*>(x + base + i);
      float4 mu, pr;
      mu.x = sde_mean(ca, xx.x, cb, vv.x); mu.y = sde_mean(ca, xx.y, cb, vv.y);
      mu.z = sde_mean(ca, xx.z, cb, vv.z); mu.w = sde_mean(ca, xx.w, cb, vv.w);
      if (prev_in != nullptr) {
        pr = *reinterpret_cast<const float4*>(prev_in + base + i);
      } else {
        const float4 e = *reinterpret_cast<const float4*>(noise + base + i);
        pr.x = sde_sample(mu.x, cs, e.x); pr.y = sde_sample(mu.y, cs, e.y);
        pr.z = sde_sample(mu.z, cs, e.z); pr.w = sde_sample(mu.w, cs, e.w);
      }
      if (deterministic) {
        pr.x = sde_ode(xx.x, cdt, vv.x); pr.y = sde_ode(xx.y, cdt, vv.y);
        pr.z = sde_ode(xx.z, cdt, vv.z); pr.w = sde_ode(xx.w, cdt, vv.w);
      }
      *reinterpret_cast<float4*>(mean_out + base + i) = mu;
      *reinterpret_cast<float4*>(prev_out + base + i) = pr;
      acc = sde_sq4(acc, pr, mu);
    } else {
      // ragged end (or unaligned operands): the same operations in the same order, element by element
      float4 mu = make_float4(0.f, 0.f, 0.f, 0.f), pr = mu;
      float* mu_e = &mu.x;
      float* pr_e = &pr.x;
      for (int64_t j = i; j < n && j < i + 4; ++j) {
        const float vv = v[base + j], xx = x[base + j];
        const float m = sde_mean(ca, xx, cb, vv);
        float q = (prev_in != nullptr) ? prev_in[base + j] : sde_sample(m, cs, noise[base + j]);
        if (deterministic) q = sde_ode(xx, cdt, vv);
        mean_out[base + j] = m;
        prev_out[base + j] = q;
        mu_e[j - i] = m;
        pr_e[j - i] = q;
      }
      acc = sde_sq4(acc, pr, mu);
    }
  }
  const float total = block_sum(acc, red);
  if (threadIdx.x == 0) partial[(int64_t)sample * blocks_per_sample + blockIdx.x] = total;
}

__global__ void sde_logprob_finalize_kernel(const float* __restrict__ partial,
                                            const float* __restrict__ scale,
                                            float* __restrict__ logp, int blocks_per_sample,
                                            int64_t n, int gaussian, int batch) {
  const int sample = blockIdx.x * blockDim.x + threadIdx.x;
  if (sample >= batch) return;
  float s = 0.f;
  for (int i = 0; i < blocks_per_sample; ++i) s += partial[(int64_t)sample * blocks_per_sample + i];
  const float mean_sq = s / (float)n;
  if (gaussian) {
    const float nu = scale[sample];
    logp[sample] = -mean_sq / (2.f * nu * nu) - logf(nu) - 0.9189385332046727f;
  } else {
    logp[sample] = -mean_sq;
  }
}

// ------------------------------------------------------------------------------------------
// K5, rollout form: classifier-free-guidance combine + SDE / CPS step + Gaussian log-density + the
// write into the trajectory buffer, in ONE pass over the model output.
//   v   = cond                                   (no guidance)
//       = uncond + g (cond - uncond)             (cfg_form 0)   or   cond + g (cond - uncond)  (cfg_form 1)
//   mu  = a x + b v ;  x' = mu + scale * eps  (or x + dt v when deterministic)
// `pred` is the transformer output in its own dtype, [uncond ; cond] stacked along the batch when
// guidance is on.  x is row i of the trajectory buffer, x' goes to row i + 1 (both addressed with the
// buffer's batch stride), the per-sample log-density goes to column i of the [B, T] log-prob table.
// eps comes from `noise` when given, otherwise from Philox-4x32-10 keyed by (seed, element, step),
// so a rollout is a pure function of its seed and no noise tensor is materialised.
// ------------------------------------------------------------------------------------------
template <typename TV>
__device__ __forceinline__ float4 load4(const TV* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 lo = bf16pair_to_float2(u.x), hi = bf16pair_to_float2(u.y);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

template <typename TV>
__global__ void __launch_bounds__(kSdeThreads)
sde_rollout_step_kernel(const TV* __restrict__ pred, int has_cfg, float guidance, int cfg_form,
                        const float* __restrict__ x, float* __restrict__ next, int64_t path_bstride,
                        const float* __restrict__ a, const float* __restrict__ b,
                        const float* __restrict__ scale, const float* __restrict__ dt,
                        const float* __restrict__ noise, unsigned long long seed,
                        unsigned long long offset, float* __restrict__ partial, int64_t n,
                        int blocks_per_sample, int batch, int deterministic) {
  __shared__ float red[32];
  const int sample = blockIdx.y;
  const float ca = a[sample], cb = b[sample], cs = scale[sample], cdt = dt[sample];
  const TV* cond = pred + ((int64_t)(has_cfg ? batch : 0) + sample) * n;
  const TV* uncond = pred + (int64_t)sample * n;
  const float* xs = x + (int64_t)sample * path_bstride;
  float* out = next + (int64_t)sample * path_bstride;
  const int64_t start = (int64_t)blockIdx.x * kSdeElemsPerBlock;
  curandStatePhilox4_32_10_t rng;
  if (noise == nullptr && !deterministic)
    curand_init(seed, ((unsigned long long)sample * blocks_per_sample + blockIdx.x) * kSdeThreads + threadIdx.x,
                offset, &rng);
  float acc = 0.f;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int64_t i = start + ((int64_t)it * kSdeThreads + threadIdx.x) * 4;
    float4 e = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!deterministic) {
      // every thread draws in every iteration so the Philox counters do not depend on n
      if (noise == nullptr) e = curand_normal4(&rng);
      else if (i + 3 < n) e = *reinterpret_cast<const float4*>(noise + (int64_t)sample * n + i);
    }
    if (i + 3 < n) {
      float4 vv = load4<TV>(cond + i);
      if (has_cfg) {
        const float4 uu = load4<TV>(uncond + i);
        const float4 base = cfg_form == 0 ? uu : vv;
        // three separately rounded operations, exactly what the training replay's tensor expression
        // `base + g * (cond - uncond)` does: rollout and replay must see the same v bit for bit
        vv = make_float4(__fadd_rn(base.x, __fmul_rn(guidance, __fsub_rn(vv.x, uu.x))),
                         __fadd_rn(base.y, __fmul_rn(guidance, __fsub_rn(vv.y, uu.y))),
                         __fadd_rn(base.z, __fmul_rn(guidance, __fsub_rn(vv.z, uu.z))),
                         __fadd_rn(base.w, __fmul_rn(guidance, __fsub_rn(vv.w, uu.w))));
      }
      const float4 xx = *reinterpret_cast<const float4*>(xs + i);
      float4 mu, pr;
      mu.x = sde_mean(ca, xx.x, cb, vv.x); mu.y = sde_mean(ca, xx.y, cb, vv.y);
      mu.z = sde_mean(ca, xx.z, cb, vv.z); mu.w = sde_mean(ca, xx.w, cb, vv.w);
      if (deterministic) {
        pr.x = sde_ode(xx.x, cdt, vv.x); pr.y = sde_ode(xx.y, cdt, vv.y);
        pr.z = sde_ode(xx.z, cdt, vv.z); pr.w = sde_ode(xx.w, cdt, vv.w);
      } else {
        pr.x = sde_sample(mu.x, cs, e.x); pr.y = sde_sample(mu.y, cs, e.y);
        pr.z = sde_sample(mu.z, cs, e.z); pr.w = sde_sample(mu.w, cs, e.w);
      }
      *reinterpret_cast<float4*>(out + i) = pr;
      acc = sde_sq4(acc, pr, mu);
    }
  }
  const float total = block_sum(acc, red);
  if (threadIdx.x == 0) partial[(int64_t)sample * blocks_per_sample + blockIdx.x] = total;
}

__global__ void sde_logprob_finalize_strided_kernel(const float* __restrict__ partial,
                                                    const float* __restrict__ scale,
                                                    float* __restrict__ logp, int64_t logp_stride,
                                                    int blocks_per_sample, int64_t n, int gaussian,
                                                    int batch) {
  const int sample = blockIdx.x * blockDim.x + threadIdx.x;
  if (sample >= batch) return;
  float s = 0.f;
  for (int i = 0; i < blocks_per_sample; ++i) s += partial[(int64_t)sample * blocks_per_sample + i];
  const float mean_sq = s / (float)n;
  float value = -mean_sq;
  if (gaussian) {
    const float nu = scale[sample];
    value = -mean_sq / (2.f * nu * nu) - logf(nu) - 0.9189385332046727f;
  }
  logp[(int64_t)sample * logp_stride] = value;
}

void sde_rollout_step(torch::Tensor pred, bool has_cfg, double guidance, int64_t cfg_form,
                      torch::Tensor path, int64_t step, torch::Tensor a, torch::Tensor b,
                      torch::Tensor scale, torch::Tensor dt, c10::optional<torch::Tensor> noise,
                      int64_t seed, int64_t offset, torch::Tensor log_probs, bool deterministic,
                      bool gaussian) {
  TORCH_CHECK(path.is_cuda() && path.scalar_type() == torch::kFloat32 && path.is_contiguous() &&
              path.dim() >= 3, "sde_rollout_step: path must be a contiguous fp32 [B, T + 1, ...] buffer");
  const int64_t batch = path.size(0), rows = path.size(1);
  TORCH_CHECK(batch >= 1 && batch <= 65535 && step >= 0 && step + 1 < rows, "sde_rollout_step: step out of range");
  const int64_t n = path.numel() / (batch * rows);
  TORCH_CHECK(n % 4 == 0 && reinterpret_cast<uintptr_t>(path.data_ptr()) % 16 == 0,
              "sde_rollout_step: the per-sample latent size must be a multiple of 4 floats");
  VRL_CHECK_OPERAND(pred, path);
  TORCH_CHECK(pred.is_contiguous() && pred.numel() == (has_cfg ? 2 : 1) * batch * n &&
              reinterpret_cast<uintptr_t>(pred.data_ptr()) % 16 == 0 &&
              (pred.scalar_type() == torch::kFloat32 || pred.scalar_type() == torch::kBFloat16),
              "sde_rollout_step: pred must be contiguous fp32 / bf16 [(2) B, ...] matching the latents");
  VRL_CHECK_OPERAND(a, path, torch::kFloat32, batch);
  VRL_CHECK_OPERAND(b, path, torch::kFloat32, batch);
  VRL_CHECK_OPERAND(scale, path, torch::kFloat32, batch);
  VRL_CHECK_OPERAND(dt, path, torch::kFloat32, batch);
  VRL_CHECK_OPERAND(noise, path, torch::kFloat32, batch * n);
  VRL_CHECK_OPERAND(log_probs, path, torch::kFloat32);
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && scale.is_contiguous() && dt.is_contiguous() &&
              (!noise.has_value() || noise->is_contiguous()), "sde_rollout_step: contiguous per-sample operands");
  TORCH_CHECK(log_probs.dim() == 2 && log_probs.size(0) == batch && step < log_probs.size(1),
              "sde_rollout_step: log_probs must be [B, T]");
  TORCH_CHECK(cfg_form == 0 || cfg_form == 1, "sde_rollout_step: cfg_form 0 (uncond + g d) or 1 (cond + g d)");
  const c10::cuda::CUDAGuard guard(path.device());
  const int bps = sde_blocks_per_sample(n);
  auto partial = torch::empty({batch, bps}, path.options());
  auto stream = at::cuda::getCurrentCUDAStream();
  const float* x = path.data_ptr<float>() + step * n;
  float* next = path.data_ptr<float>() + (step + 1) * n;
  const float* noise_ptr = noise.has_value() ? noise->data_ptr<float>() : nullptr;
  dim3 grid(bps, (unsigned)batch);
#define VRL_LAUNCH_ROLLOUT(TV)                                                                        \
  sde_rollout_step_kernel<TV><<<grid, kSdeThreads, 0, stream>>>(                                      \
      reinterpret_cast<const TV*>(pred.data_ptr()), has_cfg ? 1 : 0, (float)guidance, (int)cfg_form, x,  \
      next, rows * n, a.data_ptr<float>(), b.data_ptr<float>(), scale.data_ptr<float>(),              \
      dt.data_ptr<float>(), noise_ptr, (unsigned long long)seed, (unsigned long long)offset,          \
      partial.data_ptr<float>(), n, bps, (int)batch, deterministic ? 1 : 0)
  if (pred.scalar_type() == torch::kBFloat16) VRL_LAUNCH_ROLLOUT(__nv_bfloat16);
  else VRL_LAUNCH_ROLLOUT(float);
#undef VRL_LAUNCH_ROLLOUT
  sde_logprob_finalize_strided_kernel<<<(unsigned)((batch + 127) / 128), 128, 0, stream>>>(
      partial.data_ptr<float>(), scale.data_ptr<float>(), log_probs.data_ptr<float>() + step,
      log_probs.stride(0), bps, n, gaussian ? 1 : 0, (int)batch);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// float4 accesses need every sample's base (sample * n floats) on a 16-byte boundary
static int sde_vector_ok(const float* v, const float* x, const float* prev_in, const float* noise,
                         const float* prev_out, const float* mean_out, int64_t n) {
  auto aligned = [](const void* p) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  return (n % 4 == 0 && aligned(v) && aligned(x) && aligned(prev_in) && aligned(noise) &&
          aligned(prev_out) && aligned(mean_out)) ? 1 : 0;
}

void sde_step_launch(const float* v, const float* x, const float* a, const float* b,
                     const float* scale, const float* dt, const float* prev_in,
                     const float* noise, float* prev_out, float* mean_out, float* logp,
                     float* partial, int batch, int64_t n, bool deterministic, bool gaussian,
                     cudaStream_t stream) {
  const int bps = sde_blocks_per_sample(n);
  dim3 grid(bps, batch);
  sde_step_fwd_kernel<<<grid, kSdeThreads, 0, stream>>>(v, x, a, b, scale, dt, prev_in, noise,
                                                        prev_out, mean_out, partial, n, bps,
                                                        deterministic ? 1 : 0,
                                                        sde_vector_ok(v, x, prev_in, noise, prev_out,
                                                                      mean_out, n));
  sde_logprob_finalize_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(partial, scale, logp, bps,
                                                                       n, gaussian ? 1 : 0, batch);
}

int sde_blocks_per_sample(int64_t n) {
  return (int)((n + kSdeElemsPerBlock - 1) / kSdeElemsPerBlock);
}

std::vector<torch::Tensor> sde_step_fwd(torch::Tensor v, torch::Tensor x, torch::Tensor a,
                                        torch::Tensor b, torch::Tensor scale, torch::Tensor dt,
                                        c10::optional<torch::Tensor> prev_sample,
                                        c10::optional<torch::Tensor> noise, bool deterministic,
                                        bool gaussian) {
  TORCH_CHECK(v.is_cuda() && v.scalar_type() == torch::kFloat32 && v.is_contiguous());
  TORCH_CHECK(x.scalar_type() == torch::kFloat32 && x.is_contiguous() && x.sizes() == v.sizes());
  TORCH_CHECK(prev_sample.has_value() || noise.has_value(), "need prev_sample or noise");
  TORCH_CHECK(v.dim() >= 1 && v.size(0) > 0, "sde_step_fwd: empty batch");
  VRL_CHECK_OPERAND(x, v);
  VRL_CHECK_OPERAND(a, v, c10::nullopt, v.size(0));
  VRL_CHECK_OPERAND(b, v, c10::nullopt, v.size(0));
  VRL_CHECK_OPERAND(scale, v, c10::nullopt, v.size(0));
  VRL_CHECK_OPERAND(dt, v, c10::nullopt, v.size(0));
  VRL_CHECK_OPERAND(prev_sample, v);
  VRL_CHECK_OPERAND(noise, v);
  const c10::cuda::CUDAGuard guard(v.device());
  const int batch = (int)v.size(0);
  const int64_t n = v.numel() / batch;
  auto prev_out = torch::empty_like(v);
  auto mean_out = torch::empty_like(v);
  auto logp = torch::empty({batch}, v.options());
  auto partial = torch::empty({batch, sde_blocks_per_sample(n)}, v.options());
  const float* prev_ptr = nullptr;
  const float* noise_ptr = nullptr;
  torch::Tensor prev_c, noise_c;
  if (prev_sample.has_value()) {
    prev_c = prev_sample->contiguous();
    TORCH_CHECK(prev_c.scalar_type() == torch::kFloat32 && prev_c.numel() == v.numel());
    prev_ptr = prev_c.data_ptr<float>();
  } else {
    noise_c = noise->contiguous();
    TORCH_CHECK(noise_c.scalar_type() == torch::kFloat32 && noise_c.numel() == v.numel());
    noise_ptr = noise_c.data_ptr<float>();
  }
  auto f = [](torch::Tensor& t) { t = t.to(torch::kFloat32).contiguous(); return t.data_ptr<float>(); };
  sde_step_launch(v.data_ptr<float>(), x.data_ptr<float>(), f(a), f(b), f(scale), f(dt), prev_ptr,
                  noise_ptr, prev_out.data_ptr<float>(), mean_out.data_ptr<float>(),
                  logp.data_ptr<float>(), partial.data_ptr<float>(), batch, n, deterministic,
                  gaussian, at::cuda::getCurrentCUDAStream());
  return {prev_out, logp, mean_out};
}

__global__ void sde_step_bwd_kernel(const float* __restrict__ prev, const float* __restrict__ mean,
                                    const float* __restrict__ a, const float* __restrict__ b,
                                    const float* __restrict__ scale,
                                    const float* __restrict__ g_logp,
                                    const float* __restrict__ g_mean, float* __restrict__ g_v,
                                    float* __restrict__ g_x, int64_t n, int gaussian) {
  const int sample = blockIdx.y;
  const float ca = a[sample], cb = b[sample], nu = scale[sample];
  // d logp / d mu_i = (x'_i - mu_i) * k
  const float k = g_logp[sample] * (gaussian ? 1.f / (nu * nu * (float)n) : 2.f / (float)n);
  const int64_t base = (int64_t)sample * n;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (int64_t)gridDim.x * blockDim.x * 4) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (i + j < n) {
        float gm = (prev[base + i + j] - mean[base + i + j]) * k;
        if (g_mean != nullptr) gm += g_mean[base + i + j];
        g_v[base + i + j] = gm * cb;
        g_x[base + i + j] = gm * ca;
      }
    }
  }
}

std::vector<torch::Tensor> sde_step_bwd(torch::Tensor prev, torch::Tensor mean, torch::Tensor a,
                                        torch::Tensor b, torch::Tensor scale, torch::Tensor g_logp,
                                        c10::optional<torch::Tensor> g_mean, bool gaussian) {
  TORCH_CHECK(prev.is_cuda() && prev.scalar_type() == torch::kFloat32 && prev.is_contiguous() &&
              prev.dim() >= 1 && prev.size(0) > 0, "sde_step_bwd: prev must be contiguous fp32 CUDA");
  VRL_CHECK_OPERAND(mean, prev, torch::kFloat32, prev.numel());
  TORCH_CHECK(mean.is_contiguous(), "sde_step_bwd: mean must be contiguous");
  VRL_CHECK_OPERAND(a, prev, c10::nullopt, prev.size(0));
  VRL_CHECK_OPERAND(b, prev, c10::nullopt, prev.size(0));
  VRL_CHECK_OPERAND(scale, prev, c10::nullopt, prev.size(0));
  VRL_CHECK_OPERAND(g_logp, prev, c10::nullopt, prev.size(0));
  VRL_CHECK_OPERAND(g_mean, prev, c10::nullopt, prev.numel());
  const c10::cuda::CUDAGuard guard(prev.device());
  const int batch = (int)prev.size(0);
  const int64_t n = prev.numel() / batch;
  auto g_v = torch::empty_like(prev);
  auto g_x = torch::empty_like(prev);
  torch::Tensor gm;
  const float* gm_ptr = nullptr;
  if (g_mean.has_value()) {
    gm = g_mean->to(torch::kFloat32).contiguous();
    gm_ptr = gm.data_ptr<float>();
  }
  a = a.to(torch::kFloat32).contiguous();
  b = b.to(torch::kFloat32).contiguous();
  scale = scale.to(torch::kFloat32).contiguous();
  g_logp = g_logp.to(torch::kFloat32).contiguous();
  const int bx = (int)std::min<int64_t>((n / 4 + 255) / 256, 64);
  sde_step_bwd_kernel<<<dim3(std::max(bx, 1), batch), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      prev.data_ptr<float>(), mean.data_ptr<float>(), a.data_ptr<float>(), b.data_ptr<float>(),
      scale.data_ptr<float>(), g_logp.data_ptr<float>(), gm_ptr, g_v.data_ptr<float>(),
      g_x.data_ptr<float>(), n, gaussian ? 1 : 0);
  return {g_v, g_x};
}

// ------------------------------------------------------------------------------------------
// K6: clipped surrogate over [B, L] tokens (L = 1 gives the per-sample GRPO loss)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
token_loss_kernel(const float* __restrict__ lp, const float* __restrict__ old,
                  const float* __restrict__ adv, const float* __restrict__ mask,
                  const float* __restrict__ ref, float* __restrict__ out,
                  float* __restrict__ g_pol, float* __restrict__ g_kl, int batch, int len,
                  float eps_clip, int k3) {
  __shared__ float red[32];
  const int total = batch * len;
  float s_loss = 0.f, s_kl = 0.f, s_clip = 0.f, s_akl = 0.f, s_mask = 0.f, s_valid = 0.f;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const float m = mask ? mask[i] : 1.f;
    const float a = adv[i / len];
    const float d = lp[i] - old[i];
    const float r = __expf(d);
    const float rc = fminf(fmaxf(r, 1.f - eps_clip), 1.f + eps_clip);
    const float un = -a * r, cl = -a * rc;
    s_loss += fmaxf(un, cl) * m;
    if (ref) {
      const float dr = lp[i] - ref[i];
      s_kl += (k3 ? (__expf(dr) * (dr - 1.f) + 1.f) : dr) * m;
    }
    const float valid = m > 0.f ? 1.f : 0.f;
    s_clip += (fabsf(r - 1.f) > eps_clip ? 1.f : 0.f) * valid;
    s_akl += 0.5f * d * d * valid;
    s_mask += m;
    s_valid += valid;
  }
  s_loss = block_sum(s_loss, red);
  s_kl = block_sum(s_kl, red);
  s_clip = block_sum(s_clip, red);
  s_akl = block_sum(s_akl, red);
  s_mask = block_sum(s_mask, red);
  s_valid = block_sum(s_valid, red);
  const float denom = fmaxf(s_mask, 1.f), nvalid = fmaxf(s_valid, 1.f);
  if (threadIdx.x == 0) {
    out[0] = s_loss / denom;
    out[1] = s_kl / denom;
    out[2] = s_clip / nvalid;
    out[3] = s_akl / nvalid;
  }
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const float m = mask ? mask[i] : 1.f;
    const float a = adv[i / len];
    const float r = __expf(lp[i] - old[i]);
    const bool inside = (r >= 1.f - eps_clip) && (r <= 1.f + eps_clip);
    const float rc = fminf(fmaxf(r, 1.f - eps_clip), 1.f + eps_clip);
    const bool unclipped_active = inside || (-a * r > -a * rc);
    g_pol[i] = unclipped_active ? (-a * r) * m / denom : 0.f;
    if (ref) {
      const float dr = lp[i] - ref[i];
      g_kl[i] = (k3 ? __expf(dr) * dr : 1.f) * m / denom;
    } else {
      g_kl[i] = 0.f;
    }
  }
}

std::vector<torch::Tensor> token_loss_fwd(torch::Tensor lp, torch::Tensor old, torch::Tensor adv,
                                          c10::optional<torch::Tensor> mask,
                                          c10::optional<torch::Tensor> ref, double eps_clip,
                                          bool k3) {
  TORCH_CHECK(lp.is_cuda() && lp.dim() == 2 && lp.scalar_type() == torch::kFloat32 && lp.is_contiguous());
  VRL_CHECK_OPERAND(old, lp, c10::nullopt, lp.numel());
  VRL_CHECK_OPERAND(adv, lp, c10::nullopt, lp.size(0));
  VRL_CHECK_OPERAND(mask, lp, c10::nullopt, lp.numel());
  VRL_CHECK_OPERAND(ref, lp, c10::nullopt, lp.numel());
  const c10::cuda::CUDAGuard guard(lp.device());
  const int batch = (int)lp.size(0), len = (int)lp.size(1);
  old = old.to(torch::kFloat32).contiguous();
  adv = adv.to(torch::kFloat32).contiguous();
  TORCH_CHECK(old.numel() == lp.numel() && adv.numel() == batch);
  torch::Tensor m, r;
  const float* mp = nullptr;
  const float* rp = nullptr;
  if (mask.has_value()) { m = mask->to(torch::kFloat32).contiguous(); mp = m.data_ptr<float>(); }
  if (ref.has_value()) { r = ref->to(torch::kFloat32).contiguous(); rp = r.data_ptr<float>(); }
  auto out = torch::empty({4}, lp.options());
  auto g_pol = torch::empty_like(lp);
  auto g_kl = torch::empty_like(lp);
  token_loss_kernel<<<1, 1024, 0, at::cuda::getCurrentCUDAStream()>>>(
      lp.data_ptr<float>(), old.data_ptr<float>(), adv.data_ptr<float>(), mp, rp,
      out.data_ptr<float>(), g_pol.data_ptr<float>(), g_kl.data_ptr<float>(), batch, len,
      (float)eps_clip, k3 ? 1 : 0);
  return {out, g_pol, g_kl};
}

// ------------------------------------------------------------------------------------------
// K14 helper: per-sample mean squared error, any of fp32 / bf16 inputs
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void mse_partial_kernel(const T* __restrict__ p, const T* __restrict__ t,
                                   float* __restrict__ partial, int64_t n, int bps) {
  __shared__ float red[32];
  const int sample = blockIdx.y;
  const int64_t base = (int64_t)sample * n;
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float d = to_f<T>(p[base + i]) - to_f<T>(t[base + i]);
    acc += d * d;
  }
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) partial[(int64_t)sample * bps + blockIdx.x] = s;
}

__global__ void mean_finalize_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                     int bps, float inv_n, int batch) {
  const int sample = blockIdx.x * blockDim.x + threadIdx.x;
  if (sample >= batch) return;
  float s = 0.f;
  for (int i = 0; i < bps; ++i) s += partial[(int64_t)sample * bps + i];
  out[sample] = s * inv_n;
}

torch::Tensor per_sample_mse(torch::Tensor pred, torch::Tensor target) {
  TORCH_CHECK(pred.is_cuda() && pred.sizes() == target.sizes() && pred.dtype() == target.dtype());
  VRL_CHECK_OPERAND(target, pred);
  const c10::cuda::CUDAGuard guard(pred.device());
  pred = pred.contiguous();
  target = target.contiguous();
  const int batch = (int)pred.size(0);
  const int64_t n = pred.numel() / batch;
  const int bps = (int)std::min<int64_t>((n + 4095) / 4096, 128);
  auto partial = torch::empty({batch, bps}, pred.options().dtype(torch::kFloat32));
  auto out = torch::empty({batch}, pred.options().dtype(torch::kFloat32));
  auto stream = at::cuda::getCurrentCUDAStream();
  if (pred.scalar_type() == torch::kFloat32) {
    mse_partial_kernel<float><<<dim3(bps, batch), 256, 0, stream>>>(
        pred.data_ptr<float>(), target.data_ptr<float>(), partial.data_ptr<float>(), n, bps);
  } else {
    TORCH_CHECK(pred.scalar_type() == torch::kBFloat16, "per_sample_mse: fp32 or bf16");
    mse_partial_kernel<__nv_bfloat16><<<dim3(bps, batch), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(pred.data_ptr()),
        reinterpret_cast<const __nv_bfloat16*>(target.data_ptr()), partial.data_ptr<float>(), n, bps);
  }
  mean_finalize_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(
      partial.data_ptr<float>(), out.data_ptr<float>(), bps, 1.f / (float)n, batch);
  return out;
}

// ------------------------------------------------------------------------------------------
// K11: sum of squares of a flat gradient buffer and the flat AdamW update
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ g, float* __restrict__ partial,
                                     int64_t n) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float x = to_f<T>(g[i]);
    acc += x * x;
  }
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void sumsq_partial_bf16x8_kernel(const bf16x8* __restrict__ g,
                                            float* __restrict__ partial, int64_t nvec) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(g[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += f[j] * f[j];
  }
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void sum_finalize_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                    int count) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < count; i += blockDim.x) acc += partial[i];
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = s;
}

torch::Tensor sum_squares(torch::Tensor g) {
  TORCH_CHECK(g.is_cuda() && g.is_contiguous());
  const c10::cuda::CUDAGuard guard(g.device());
  const int64_t n = g.numel();
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((n + 8191) / 8192, 148 * 8));
  auto partial = torch::empty({blocks}, g.options().dtype(torch::kFloat32));
  auto out = torch::empty({}, g.options().dtype(torch::kFloat32));
  auto stream = at::cuda::getCurrentCUDAStream();
  if (g.scalar_type() == torch::kBFloat16 && n % 8 == 0 &&
      reinterpret_cast<uintptr_t>(g.data_ptr()) % 16 == 0) {
    sumsq_partial_bf16x8_kernel<<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const bf16x8*>(g.data_ptr()), partial.data_ptr<float>(), n / 8);
  } else if (g.scalar_type() == torch::kBFloat16) {
    sumsq_partial_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(g.data_ptr()), partial.data_ptr<float>(), n);
  } else {
    TORCH_CHECK(g.scalar_type() == torch::kFloat32, "sum_squares: fp32 or bf16");
    sumsq_partial_kernel<float><<<blocks, 256, 0, stream>>>(g.data_ptr<float>(),
                                                           partial.data_ptr<float>(), n);
  }
  sum_finalize_kernel<<<1, 256, 0, stream>>>(partial.data_ptr<float>(), out.data_ptr<float>(), blocks);
  return out;
}

template <typename TP, typename TG>
__global__ void adamw_flat_kernel(TP* __restrict__ p, const TG* __restrict__ g,
                                  float* __restrict__ master, float* __restrict__ m,
                                  float* __restrict__ v, int64_t n, float lr, float b1, float b2,
                                  float eps, float wd, float bc1, float bc2,
                                  const float* __restrict__ clip, int master_is_param) {
  const float coef = clip ? clip[0] : 1.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float grad = to_f<TG>(g[i]) * coef;
    const float mi = b1 * m[i] + (1.f - b1) * grad;
    const float vi = b2 * v[i] + (1.f - b2) * grad * grad;
    m[i] = mi;
    v[i] = vi;
    float w = master[i];
    w = w * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    master[i] = w;
    if (!master_is_param) p[i] = from_f<TP>(w);
  }
}

void adamw_flat(torch::Tensor p, torch::Tensor g, torch::Tensor master, torch::Tensor m,
                torch::Tensor v, double lr, double b1, double b2, double eps, double wd,
                int64_t step, c10::optional<torch::Tensor> clip) {
  TORCH_CHECK(p.is_cuda() && p.is_contiguous() && g.is_contiguous());
  VRL_CHECK_OPERAND(g, p, c10::nullopt, p.numel());
  VRL_CHECK_OPERAND(master, p, torch::kFloat32, p.numel());
  VRL_CHECK_OPERAND(m, p, torch::kFloat32, p.numel());
  VRL_CHECK_OPERAND(v, p, torch::kFloat32, p.numel());
  VRL_CHECK_OPERAND(clip, p);
  TORCH_CHECK(master.is_contiguous() && m.is_contiguous() && v.is_contiguous(),
              "adamw_flat: optimizer state must be contiguous");
  const c10::cuda::CUDAGuard guard(p.device());
  const int64_t n = p.numel();
  TORCH_CHECK(g.numel() == n && master.numel() == n && m.numel() == n && v.numel() == n);
  const float bc1 = 1.f - (float)std::pow(b1, (double)step);
  const float bc2 = 1.f - (float)std::pow(b2, (double)step);
  torch::Tensor c;
  const float* cp = nullptr;
  if (clip.has_value()) { c = clip->to(torch::kFloat32).contiguous(); cp = c.data_ptr<float>(); }
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((n + 1023) / 1024, 148 * 16));
  auto stream = at::cuda::getCurrentCUDAStream();
  const int same = master.data_ptr() == p.data_ptr() ? 1 : 0;
#define LAUNCH(TP, TG)                                                                         \
  adamw_flat_kernel<TP, TG><<<blocks, 256, 0, stream>>>(                                       \
      reinterpret_cast<TP*>(p.data_ptr()), reinterpret_cast<const TG*>(g.data_ptr()),          \
      master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), n, (float)lr,        \
      (float)b1, (float)b2, (float)eps, (float)wd, bc1, bc2, cp, same)
  const bool pb = p.scalar_type() == torch::kBFloat16, gb = g.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(pb || p.scalar_type() == torch::kFloat32);
  TORCH_CHECK(gb || g.scalar_type() == torch::kFloat32);
  if (pb && gb) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (pb && !gb) LAUNCH(__nv_bfloat16, float);
  else if (!pb && gb) LAUNCH(float, __nv_bfloat16);
  else LAUNCH(float, float);
#undef LAUNCH
}

// ------------------------------------------------------------------------------------------
// Column sums of a [rows, cols] bf16 matrix (bias gradients): fp32 accumulation, bf16 result.
// Each block owns 64 columns x a slab of rows; slabs are combined with fp32 atomics.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, int64_t rows, int cols,
              int rows_per_block) {
  __shared__ float tile[32][8 * 8 + 1];
  const int cvec = threadIdx.x & 7;               // 8 vectors of 8 columns = 64 columns
  const int rlane = threadIdx.x >> 3;             // 32 row lanes
  const int col = blockIdx.x * 64 + cvec * 8;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_block;
  const int64_t r1 = min(rows, r0 + rows_per_block);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < cols) {
    for (int64_t r = r0 + rlane; r < r1; r += 32) {
      float f[8];
      unpack8(*reinterpret_cast<const bf16x8*>(x + r * cols + col), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) tile[rlane][cvec * 8 + j] = acc[j];
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) s += tile[r][threadIdx.x];
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < cols) atomicAdd(out + c, s);
  }
}

torch::Tensor colsum(torch::Tensor x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.is_contiguous());
  TORCH_CHECK(x.size(1) % 8 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0);
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0);
  const int cols = (int)x.size(1);
  auto out = torch::zeros({cols}, x.options().dtype(torch::kFloat32));
  const int col_blocks = (cols + 63) / 64;
  const int row_blocks = (int)std::max<int64_t>(1, std::min<int64_t>((rows + 511) / 512, 1184 / col_blocks + 1));
  const int rows_per_block = (int)((rows + row_blocks - 1) / row_blocks);
  colsum_kernel<<<dim3(col_blocks, row_blocks), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), out.data_ptr<float>(), rows, cols,
      rows_per_block);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

}  // namespace vrl
