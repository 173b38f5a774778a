// Autoregressive-path kernels: token log-probabilities over a large vocabulary (whole-row and
// vocabulary-chunked online forms), guided categorical sampling, single-position attention
// against a static KV cache, and group-normalised advantages.
//
// Reduction orders are fixed by the launch shape (no atomics on results), so two calls with the
// same inputs return bit-identical values: the rollout's recorded log-probability and the
// trainer's replayed one must agree exactly for the first policy-ratio to be 1.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cstdlib>
#include <string>

#include "common.cuh"
#include "ops.h"
#include "sm100_ptx.cuh"

namespace vrl {

namespace {

constexpr int kRowThreads = 256;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* f);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  unpack8(*reinterpret_cast<const bf16x8*>(p), f);
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// (max, sum of exp(x - max)) pairs combine associatively.
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  const float mn = fmaxf(m, m2);
  const float a = (m == -INFINITY) ? 0.f : s * __expf(m - mn);
  const float b = (m2 == -INFINITY) ? 0.f : s2 * __expf(m2 - mn);
  m = mn;
  s = a + b;
}

__device__ __forceinline__ void block_lse(float& m, float& s, float* sm, float* ss) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    lse_merge(m, s, m2, s2);
  }
  __syncthreads();
  if (lane == 0) { sm[warp] = m; ss[warp] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mm = sm[0], sv = ss[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) lse_merge(mm, sv, sm[w], ss[w]);
    sm[0] = mm; ss[0] = sv;
  }
  __syncthreads();
  m = sm[0]; s = ss[0];
  __syncthreads();
}

// ------------------------------------------------------------------------------------------
// log_softmax(logits / T)[id] for every row.  One block per row, one pass over the row.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
token_logprob_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ ids,
                         float* __restrict__ lp, float* __restrict__ lse, int vocab, float inv_t) {
  __shared__ float sm[32], ss[32];
  const int64_t row = blockIdx.x;
  const T* x = logits + row * vocab;
  float m = -INFINITY, s = 0.f;
  const int vec_end = (vocab / 8) * 8;
  for (int i = threadIdx.x * 8; i < vec_end; i += kRowThreads * 8) {
    float f[8];
    load8<T>(x + i, f);
    float cm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
    cm *= inv_t;
    float cs = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) cs += __expf(f[j] * inv_t - cm);
    lse_merge(m, s, cm, cs);
  }
  for (int i = vec_end + threadIdx.x; i < vocab; i += kRowThreads) lse_merge(m, s, to_f<T>(x[i]) * inv_t, 1.f);
  block_lse(m, s, sm, ss);
  if (threadIdx.x == 0) {
    const float l = m + __logf(s);
    lse[row] = l;
    int64_t id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    lp[row] = to_f<T>(x[id]) * inv_t - l;
  }
}

// grad_logits = g / T * (onehot(id) - softmax(logits / T))
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
token_logprob_bwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ ids,
                         const float* __restrict__ lse, const float* __restrict__ g,
                         T* __restrict__ grad, int vocab, float inv_t) {
  const int64_t row = blockIdx.x;
  const T* x = logits + row * vocab;
  T* o = grad + row * vocab;
  const float l = lse[row], gs = g[row] * inv_t;
  const int id = (int)ids[row];
  for (int i = threadIdx.x; i < vocab; i += kRowThreads) {
    const float p = __expf(to_f<T>(x[i]) * inv_t - l);
    o[i] = from_f<T>(gs * ((i == id ? 1.f : 0.f) - p));
  }
}

// ------------------------------------------------------------------------------------------
// Vocabulary-chunked form.  `chunk` is the fp32 head output for columns [col0, col0 + width);
// the running (max, sum) and the target logit are updated in place, so the full [rows, vocab]
// logits never exist at once.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kRowThreads)
lse_chunk_update_kernel(const float* __restrict__ chunk, const int64_t* __restrict__ ids,
                        float* __restrict__ run_max, float* __restrict__ run_sum,
                        float* __restrict__ target, int width, int col0, float inv_t) {
  __shared__ float sm[32], ss[32];
  const int64_t row = blockIdx.x;
  const float* x = chunk + row * width;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < width; i += kRowThreads) lse_merge(m, s, x[i] * inv_t, 1.f);
  block_lse(m, s, sm, ss);
  if (threadIdx.x == 0) {
    float rm = run_max[row], rs = run_sum[row];
    lse_merge(rm, rs, m, s);
    run_max[row] = rm;
    run_sum[row] = rs;
    const int64_t id = ids[row] - col0;
    if (id >= 0 && id < width) target[row] = x[id] * inv_t;
  }
}

// dlogits chunk (bf16) = g / T * (onehot - softmax) for columns [col0, col0 + width)
__global__ void __launch_bounds__(kRowThreads)
softmax_grad_chunk_kernel(const float* __restrict__ chunk, const int64_t* __restrict__ ids,
                          const float* __restrict__ lse, const float* __restrict__ g,
                          __nv_bfloat16* __restrict__ out, int width, int col0, float inv_t) {
  const int64_t row = blockIdx.x;
  const float* x = chunk + row * width;
  __nv_bfloat16* o = out + row * width;
  const float l = lse[row], gs = g[row] * inv_t;
  const int id = (int)(ids[row] - col0);
  for (int i = threadIdx.x; i < width; i += kRowThreads) {
    const float p = __expf(x[i] * inv_t - l);
    o[i] = __float2bfloat16_rn(gs * ((i == id ? 1.f : 0.f) - p));
  }
}

// ------------------------------------------------------------------------------------------
// Guided sampling.  One block per row.  The token is the first index whose inclusive cumulative
// probability under softmax((u + w (c - u)) / T) exceeds `uniform * total`; the recorded
// log-probability is log_softmax(c / T)[token].  Threads own contiguous index ranges so the
// cumulative sum is taken in index order.
// ------------------------------------------------------------------------------------------
constexpr int kSampleThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_tokens_kernel(const T* __restrict__ cond, const T* __restrict__ uncond,
                     const float* __restrict__ uniform, int64_t* __restrict__ tokens,
                     float* __restrict__ logp, int vocab, float w, float inv_t) {
  __shared__ float sm[32], ss[32];
  __shared__ float part[kSampleThreads];
  const int64_t row = blockIdx.x;
  const T* c = cond + row * vocab;
  const T* u = uncond + row * vocab;
  const int per = (vocab + kSampleThreads - 1) / kSampleThreads;
  const int lo = min(vocab, (int)threadIdx.x * per), hi = min(vocab, lo + per);

  // pass 1: maxima and sums of both distributions
  float gm = -INFINITY, gsum = 0.f, cm = -INFINITY, csum = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float cv = to_f<T>(c[i]), uv = to_f<T>(u[i]);
    lse_merge(gm, gsum, (uv + w * (cv - uv)) * inv_t, 1.f);
    lse_merge(cm, csum, cv * inv_t, 1.f);
  }
  float gmax = gm, gtot = gsum;
  block_lse(gmax, gtot, sm, ss);
  float cmax = cm, ctot = csum;
  block_lse(cmax, ctot, sm, ss);

  // pass 2: per-thread mass relative to the row maximum, then the owning thread scans its range
  float mass = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float cv = to_f<T>(c[i]), uv = to_f<T>(u[i]);
    mass += __expf((uv + w * (cv - uv)) * inv_t - gmax);
  }
  part[threadIdx.x] = mass;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int t = 0; t < kSampleThreads; ++t) total += part[t];
    const float uu = fminf(fmaxf(uniform[row], 0.f), 1.f - 1e-7f);
    const float tgt = uu * total;
    float acc = 0.f;
    int owner = kSampleThreads - 1;
    for (int t = 0; t < kSampleThreads; ++t) {
      if (acc + part[t] > tgt) { owner = t; break; }
      acc += part[t];
    }
    // sequential scan inside the owner's range
    const int olo = min(vocab, owner * per), ohi = min(vocab, olo + per);
    int tok = max(0, min(vocab, ohi) - 1);      // rounding may leave the target just out of reach
    for (int i = olo; i < ohi; ++i) {
      const float cv = to_f<T>(c[i]), uv = to_f<T>(u[i]);
      acc += __expf((uv + w * (cv - uv)) * inv_t - gmax);
      if (acc > tgt) { tok = i; break; }
    }
    tokens[row] = tok;
    logp[row] = to_f<T>(c[tok]) * inv_t - (cmax + __logf(ctot));
  }
}

// ------------------------------------------------------------------------------------------
// Decode attention: one query position per (row, head) against a static cache.
// q [R, H, D], caches [R, H, L, D] (strided), valid [R, L]; D = 128.  One block of 4 warps per
// (row, head); every warp walks runs of 16 keys with an online softmax, lanes own 4 dims.
// ------------------------------------------------------------------------------------------
constexpr int kDecodeWarps = 4;
constexpr int kDecodeKeys = 16;

__global__ void __launch_bounds__(kDecodeWarps * 32)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                        const __nv_bfloat16* __restrict__ vc, const bool* __restrict__ valid,
                        __nv_bfloat16* __restrict__ out, int heads, int length, int64_t k_sr,
                        int64_t k_sh, int64_t k_sl, int64_t v_sr, int64_t v_sh, int64_t v_sl,
                        int64_t valid_sr, float scale) {
  __shared__ float sm_m[kDecodeWarps], sm_s[kDecodeWarps];
  __shared__ float sm_o[kDecodeWarps][128];
  const int r = blockIdx.x / heads, h = blockIdx.x % heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* qp = q + ((int64_t)r * heads + h) * 128 + lane * 4;
  const uint2 qraw = *reinterpret_cast<const uint2*>(qp);
  const float2 q01 = bf16pair_to_float2(qraw.x), q23 = bf16pair_to_float2(qraw.y);
  const __nv_bfloat16* kbase = kc + r * k_sr + h * k_sh + lane * 4;
  const __nv_bfloat16* vbase = vc + r * v_sr + h * v_sh + lane * 4;
  const bool* vrow = valid + r * valid_sr;
  float m = -INFINITY, s = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
  // kDecodeKeys keys per pass: their loads, dot products and reductions are independent of one
  // another, so one pass costs about one memory round trip instead of kDecodeKeys of them; the
  // running maximum is raised once per pass.
  for (int j0 = warp * kDecodeKeys; j0 < length; j0 += kDecodeWarps * kDecodeKeys) {
    bool ok[kDecodeKeys];
    bool any = false;
#pragma unroll
    for (int i = 0; i < kDecodeKeys; ++i) {
      ok[i] = (j0 + i < length) && vrow[j0 + i];
      any = any || ok[i];
    }
    if (!any) continue;                                       // warp-uniform
    uint2 kraw[kDecodeKeys], vraw[kDecodeKeys];
#pragma unroll
    for (int i = 0; i < kDecodeKeys; ++i) {
      kraw[i] = make_uint2(0u, 0u);
      vraw[i] = make_uint2(0u, 0u);
      if (ok[i]) {                                            // never touch a slot that was not written
        kraw[i] = *reinterpret_cast<const uint2*>(kbase + (int64_t)(j0 + i) * k_sl);
        vraw[i] = *reinterpret_cast<const uint2*>(vbase + (int64_t)(j0 + i) * v_sl);
      }
    }
    float dot[kDecodeKeys];
#pragma unroll
    for (int i = 0; i < kDecodeKeys; ++i) {
      const float2 k01 = bf16pair_to_float2(kraw[i].x), k23 = bf16pair_to_float2(kraw[i].y);
      dot[i] = q01.x * k01.x + q01.y * k01.y + q23.x * k23.x + q23.y * k23.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int i = 0; i < kDecodeKeys; ++i) dot[i] += __shfl_xor_sync(0xffffffffu, dot[i], o);
    }
    float mn = m;
#pragma unroll
    for (int i = 0; i < kDecodeKeys; ++i) {
      dot[i] = ok[i] ? dot[i] * scale : -INFINITY;
      mn = fmaxf(mn, dot[i]);
    }
    const float corr = (m == -INFINITY) ? 0.f : __expf(m - mn);
    o0 *= corr; o1 *= corr; o2 *= corr; o3 *= corr;
    s *= corr;
#pragma unroll
    for (int i = 0; i < kDecodeKeys; ++i) {
      const float p = ok[i] ? __expf(dot[i] - mn) : 0.f;
      const float2 v01 = bf16pair_to_float2(vraw[i].x), v23 = bf16pair_to_float2(vraw[i].y);
      o0 = fmaf(p, v01.x, o0); o1 = fmaf(p, v01.y, o1);
      o2 = fmaf(p, v23.x, o2); o3 = fmaf(p, v23.y, o3);
      s += p;
    }
    m = mn;
  }
  if (lane == 0) { sm_m[warp] = m; sm_s[warp] = s; }
  __syncthreads();
  float gm = -INFINITY;
#pragma unroll
  for (int w2 = 0; w2 < kDecodeWarps; ++w2) gm = fmaxf(gm, sm_m[w2]);
  const float mine = (m == -INFINITY) ? 0.f : __expf(m - gm);
  sm_o[warp][lane * 4 + 0] = o0 * mine; sm_o[warp][lane * 4 + 1] = o1 * mine;
  sm_o[warp][lane * 4 + 2] = o2 * mine; sm_o[warp][lane * 4 + 3] = o3 * mine;
  __syncthreads();
  if (threadIdx.x < 128) {
    float tot = 0.f, acc = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < kDecodeWarps; ++w2) {
      tot += (sm_m[w2] == -INFINITY) ? 0.f : sm_s[w2] * __expf(sm_m[w2] - gm);
      acc += sm_o[w2][threadIdx.x];
    }
    out[((int64_t)r * heads + h) * 128 + threadIdx.x] = __float2bfloat16_rn(tot > 0.f ? acc / tot : 0.f);
  }
}

// ------------------------------------------------------------------------------------------
// Decode attention, streaming form (caches with contiguous keys: stride(2) == 128).  The keys and
// values of a (row, head) are one contiguous run each, so they are brought into shared memory by
// bulk asynchronous copies, 32 keys (8 KB + 8 KB) per stage through a three-stage ring: two stages
// per block are always in flight without costing a register, four blocks fit on an SM, and the
// arithmetic reads shared memory.  (The register form above keeps too little in flight: it reached
// 1.3 TB/s of cache traffic with every warp stalled on its loads.)  Chunks without a valid key are
// never copied; keys that are masked out are copied with their chunk but never read into the sums.
// A wait that runs out sets the attention status word and the block writes zeros.
// ------------------------------------------------------------------------------------------
constexpr int kDaChunk = 32;
constexpr int kDaStages = 3;
constexpr int kDaThreads = 128;
constexpr uint32_t kDaStageBytes = 2 * kDaChunk * 256;          // K then V
enum : int { kDecodeAttnTimeout = 31 };

__global__ void __launch_bounds__(kDaThreads)
decode_attention_bulk_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                             const __nv_bfloat16* __restrict__ vc, const bool* __restrict__ valid,
                             __nv_bfloat16* __restrict__ out, int heads, int length, int64_t k_sr, int64_t k_sh,
                             int64_t v_sr, int64_t v_sh, int64_t valid_sr, float scale, int* status) {
  using namespace ptx;
  extern __shared__ uint8_t da_raw[];
  uint8_t* stages = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(da_raw) + 127) & ~static_cast<uintptr_t>(127));
  __shared__ uint64_t full[kDaStages];
  __shared__ unsigned chunk_mask;
  __shared__ int abort_flag;
  __shared__ float sm_m[4], sm_s[4];
  __shared__ float sm_o[4][128];
  const int r = blockIdx.x / heads, h = blockIdx.x % heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool* vrow = valid + r * valid_sr;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kDaStages; ++s) mbar_init(&full[s], 1);
    chunk_mask = 0u;
    abort_flag = 0;
    mbar_fence_init();
    fence_async_smem();
  }
  __syncthreads();
  // which 32-key chunks hold at least one valid key (length <= 1024: thread t looks at 8 positions)
  {
    bool any = false;
    const int p0 = threadIdx.x * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) any = any || (p0 + i < length && vrow[p0 + i]);
    if (any) atomicOr(&chunk_mask, 1u << (p0 / kDaChunk));
  }
  __syncthreads();
  const unsigned mask = chunk_mask;
  const int count = __popc(mask);
  const __nv_bfloat16* kbase = kc + r * k_sr + h * k_sh;
  const __nv_bfloat16* vbase = vc + r * v_sr + h * v_sh;
  auto issue = [&](int chunk, int s) {
    const int nkeys = min(kDaChunk, length - chunk * kDaChunk);
    uint8_t* dst = stages + s * kDaStageBytes;
    mbar_expect_tx(&full[s], 2u * (uint32_t)nkeys * 256u);
    bulk_load(dst, kbase + (int64_t)chunk * kDaChunk * 128, (uint32_t)nkeys * 256u, &full[s]);
    bulk_load(dst + kDaChunk * 256, vbase + (int64_t)chunk * kDaChunk * 128, (uint32_t)nkeys * 256u, &full[s]);
  };
  unsigned prod_rem = mask;                    // thread 0: chunks not yet requested
  if (threadIdx.x == 0) {
    for (int s = 0; s < kDaStages && prod_rem; ++s) {
      issue(__ffs(prod_rem) - 1, s);
      prod_rem &= prod_rem - 1;
    }
  }
  const uint2 qraw = *reinterpret_cast<const uint2*>(q + ((int64_t)r * heads + h) * 128 + lane * 4);
  const float2 q01 = bf16pair_to_float2(qraw.x), q23 = bf16pair_to_float2(qraw.y);
  float m = -INFINITY, sum = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
  unsigned cons_rem = mask;
  bool ok_all = true;
  for (int it = 0; it < count; ++it) {
    const int s = it % kDaStages;
    const int chunk = __ffs(cons_rem) - 1;
    cons_rem &= cons_rem - 1;
    // this warp's eight keys of the chunk: their mask bytes are requested before the wait
    const int j0 = chunk * kDaChunk + warp * 8;
    bool ok[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) ok[i] = (j0 + i < length) && vrow[j0 + i];
    if (!mbar_wait(&full[s], (it / kDaStages) & 1u, &abort_flag)) { ok_all = false; }
    ok_all = __syncthreads_and(ok_all ? 1 : 0) != 0;
    if (!ok_all) break;
    const uint8_t* ks = stages + s * kDaStageBytes + warp * 8 * 256 + lane * 8;
    const uint8_t* vs = ks + kDaChunk * 256;
    float dot[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint2 kraw = *reinterpret_cast<const uint2*>(ks + i * 256);
      const float2 k01 = bf16pair_to_float2(kraw.x), k23 = bf16pair_to_float2(kraw.y);
      dot[i] = q01.x * k01.x + q01.y * k01.y + q23.x * k23.x + q23.y * k23.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i) dot[i] += __shfl_xor_sync(0xffffffffu, dot[i], o);
    }
    float mn = m;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      dot[i] = ok[i] ? dot[i] * scale : -INFINITY;
      mn = fmaxf(mn, dot[i]);
    }
    if (mn != -INFINITY) {                                      // warp-uniform
      const float corr = (m == -INFINITY) ? 0.f : __expf(m - mn);
      o0 *= corr; o1 *= corr; o2 *= corr; o3 *= corr;
      sum *= corr;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (!ok[i]) continue;                                   // a masked slot may hold anything
        const float p = __expf(dot[i] - mn);
        const uint2 vraw = *reinterpret_cast<const uint2*>(vs + i * 256);
        const float2 v01 = bf16pair_to_float2(vraw.x), v23 = bf16pair_to_float2(vraw.y);
        o0 = fmaf(p, v01.x, o0); o1 = fmaf(p, v01.y, o1);
        o2 = fmaf(p, v23.x, o2); o3 = fmaf(p, v23.y, o3);
        sum += p;
      }
      m = mn;
    }
    __syncthreads();                                            // every warp is done with stage s
    if (threadIdx.x == 0 && prod_rem) {
      issue(__ffs(prod_rem) - 1, s);
      prod_rem &= prod_rem - 1;
    }
  }
  if (!ok_all) {
    // copies already requested still target this block's shared memory: wait (bounded) for them
    if (threadIdx.x == 0) {
      atomicExch(status, kDecodeAttnTimeout);
      for (int spin = 0; spin < 2000; ++spin) __nanosleep(1000);       // ~2 ms, far longer than any copy
    }
    __syncthreads();
    if (threadIdx.x < 128) out[((int64_t)r * heads + h) * 128 + threadIdx.x] = __float2bfloat16_rn(0.f);
    return;
  }
  if (lane == 0) { sm_m[warp] = m; sm_s[warp] = sum; }
  __syncthreads();
  float gm = -INFINITY;
#pragma unroll
  for (int w2 = 0; w2 < 4; ++w2) gm = fmaxf(gm, sm_m[w2]);
  const float mine = (m == -INFINITY) ? 0.f : __expf(m - gm);
  sm_o[warp][lane * 4 + 0] = o0 * mine; sm_o[warp][lane * 4 + 1] = o1 * mine;
  sm_o[warp][lane * 4 + 2] = o2 * mine; sm_o[warp][lane * 4 + 3] = o3 * mine;
  __syncthreads();
  {
    float tot = 0.f, acc = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < 4; ++w2) {
      tot += (sm_m[w2] == -INFINITY) ? 0.f : sm_s[w2] * __expf(sm_m[w2] - gm);
      acc += sm_o[w2][threadIdx.x];
    }
    out[((int64_t)r * heads + h) * 128 + threadIdx.x] = __float2bfloat16_rn(tot > 0.f ? acc / tot : 0.f);
  }
}

// ------------------------------------------------------------------------------------------
// Group-normalised advantages: a = clamp((r - mean_g) / max(std_g, eps), +-clip), unbiased std,
// singleton groups -> 0.  One block; every thread owns samples i, i + blockDim, ...
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
group_advantages_kernel(const float* __restrict__ rewards, const int64_t* __restrict__ gids,
                        float* __restrict__ adv, int n, float eps, float clip, int global_std) {
  __shared__ float scratch[32];
  float gstd = 0.f;
  if (global_std) {
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += rewards[i];
    const float mean = block_sum(s, scratch) / (float)max(n, 1);
    float q = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float d = rewards[i] - mean; q += d * d; }
    gstd = n > 1 ? sqrtf(block_sum(q, scratch) / (float)(n - 1)) : 0.f;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int64_t g = gids[i];
    float sum = 0.f;
    int cnt = 0;
    for (int j = 0; j < n; ++j)
      if (gids[j] == g) { sum += rewards[j]; ++cnt; }
    const float mean = sum / (float)cnt;
    float sq = 0.f;
    for (int j = 0; j < n; ++j)
      if (gids[j] == g) { const float d = rewards[j] - mean; sq += d * d; }
    const float std = global_std ? gstd : sqrtf(sq / (float)max(cnt - 1, 1));
    float a = (rewards[i] - mean) / fmaxf(std, eps);
    a = fminf(fmaxf(a, -clip), clip);
    adv[i] = cnt > 1 ? a : 0.f;
  }
}

}  // namespace

// ============================================================================== host wrappers
std::vector<torch::Tensor> token_logprob_fwd(torch::Tensor logits, torch::Tensor ids, double temperature) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == torch::kInt64 && ids.numel() == logits.size(0));
  VRL_CHECK_OPERAND(ids, logits);
  const c10::cuda::CUDAGuard guard(logits.device());
  const int64_t rows = logits.size(0);
  const int vocab = (int)logits.size(1);
  auto opts = logits.options().dtype(torch::kFloat32);
  auto lp = torch::empty({rows}, opts), lse = torch::empty({rows}, opts);
  if (rows == 0) return {lp, lse};
  auto stream = at::cuda::getCurrentCUDAStream();
  const float inv_t = (float)(1.0 / temperature);
  ids = ids.contiguous();
  if (logits.scalar_type() == torch::kBFloat16) {
    TORCH_CHECK(vocab % 8 == 0, "token_logprob_fwd: bf16 vocabulary must be a multiple of 8");
    token_logprob_fwd_kernel<__nv_bfloat16><<<rows, kRowThreads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits.data_ptr()), ids.data_ptr<int64_t>(),
        lp.data_ptr<float>(), lse.data_ptr<float>(), vocab, inv_t);
  } else {
    TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && vocab % 4 == 0);
    token_logprob_fwd_kernel<float><<<rows, kRowThreads, 0, stream>>>(
        logits.data_ptr<float>(), ids.data_ptr<int64_t>(), lp.data_ptr<float>(),
        lse.data_ptr<float>(), vocab, inv_t);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {lp, lse};
}

torch::Tensor token_logprob_bwd(torch::Tensor logits, torch::Tensor ids, torch::Tensor lse,
                                torch::Tensor g, double temperature) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  VRL_CHECK_OPERAND(ids, logits, torch::kInt64, logits.size(0));
  VRL_CHECK_OPERAND(lse, logits, torch::kFloat32, logits.size(0));
  VRL_CHECK_OPERAND(g, logits, c10::nullopt, logits.size(0));
  const c10::cuda::CUDAGuard guard(logits.device());
  const int64_t rows = logits.size(0);
  const int vocab = (int)logits.size(1);
  auto grad = torch::empty_like(logits);
  if (rows == 0) return grad;
  auto stream = at::cuda::getCurrentCUDAStream();
  const float inv_t = (float)(1.0 / temperature);
  ids = ids.contiguous();
  lse = lse.contiguous();
  g = g.to(torch::kFloat32).contiguous();
  if (logits.scalar_type() == torch::kBFloat16) {
    token_logprob_bwd_kernel<__nv_bfloat16><<<rows, kRowThreads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(logits.data_ptr()), ids.data_ptr<int64_t>(),
        lse.data_ptr<float>(), g.data_ptr<float>(),
        reinterpret_cast<__nv_bfloat16*>(grad.data_ptr()), vocab, inv_t);
  } else {
    TORCH_CHECK(logits.scalar_type() == torch::kFloat32);
    token_logprob_bwd_kernel<float><<<rows, kRowThreads, 0, stream>>>(
        logits.data_ptr<float>(), ids.data_ptr<int64_t>(), lse.data_ptr<float>(),
        g.data_ptr<float>(), grad.data_ptr<float>(), vocab, inv_t);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return grad;
}

void lse_chunk_update(torch::Tensor chunk, torch::Tensor ids, torch::Tensor run_max,
                      torch::Tensor run_sum, torch::Tensor target, int64_t col0, double temperature) {
  TORCH_CHECK(chunk.is_cuda() && chunk.dim() == 2 && chunk.is_contiguous() &&
              chunk.scalar_type() == torch::kFloat32);
  TORCH_CHECK(run_max.scalar_type() == torch::kFloat32 && run_sum.scalar_type() == torch::kFloat32 &&
              target.scalar_type() == torch::kFloat32 && ids.scalar_type() == torch::kInt64);
  VRL_CHECK_OPERAND(ids, chunk, torch::kInt64, chunk.size(0));
  VRL_CHECK_OPERAND(run_max, chunk, torch::kFloat32, chunk.size(0));
  VRL_CHECK_OPERAND(run_sum, chunk, torch::kFloat32, chunk.size(0));
  VRL_CHECK_OPERAND(target, chunk, torch::kFloat32, chunk.size(0));
  TORCH_CHECK(ids.is_contiguous() && run_max.is_contiguous() && run_sum.is_contiguous() && target.is_contiguous(),
              "lse_chunk_update: per-row operands must be contiguous");
  const c10::cuda::CUDAGuard guard(chunk.device());
  const int64_t rows = chunk.size(0);
  if (rows == 0) return;
  lse_chunk_update_kernel<<<rows, kRowThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
      chunk.data_ptr<float>(), ids.data_ptr<int64_t>(), run_max.data_ptr<float>(),
      run_sum.data_ptr<float>(), target.data_ptr<float>(), (int)chunk.size(1), (int)col0,
      (float)(1.0 / temperature));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

torch::Tensor softmax_grad_chunk(torch::Tensor chunk, torch::Tensor ids, torch::Tensor lse,
                                 torch::Tensor g, int64_t col0, double temperature) {
  TORCH_CHECK(chunk.is_cuda() && chunk.dim() == 2 && chunk.is_contiguous() &&
              chunk.scalar_type() == torch::kFloat32);
  VRL_CHECK_OPERAND(ids, chunk, torch::kInt64, chunk.size(0));
  VRL_CHECK_OPERAND(lse, chunk, torch::kFloat32, chunk.size(0));
  VRL_CHECK_OPERAND(g, chunk, torch::kFloat32, chunk.size(0));
  TORCH_CHECK(ids.is_contiguous() && lse.is_contiguous() && g.is_contiguous(),
              "softmax_grad_chunk: per-row operands must be contiguous");
  const c10::cuda::CUDAGuard guard(chunk.device());
  auto out = torch::empty(chunk.sizes(), chunk.options().dtype(torch::kBFloat16));
  const int64_t rows = chunk.size(0);
  if (rows == 0) return out;
  softmax_grad_chunk_kernel<<<rows, kRowThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
      chunk.data_ptr<float>(), ids.data_ptr<int64_t>(), lse.data_ptr<float>(), g.data_ptr<float>(),
      reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), (int)chunk.size(1), (int)col0,
      (float)(1.0 / temperature));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

std::vector<torch::Tensor> sample_tokens(torch::Tensor cond, torch::Tensor uncond, torch::Tensor u,
                                         double cfg_weight, double temperature) {
  TORCH_CHECK(cond.is_cuda() && cond.dim() == 2 && cond.is_contiguous() && uncond.is_contiguous());
  TORCH_CHECK(cond.sizes() == uncond.sizes() && cond.scalar_type() == uncond.scalar_type());
  TORCH_CHECK(u.scalar_type() == torch::kFloat32 && u.numel() == cond.size(0) && u.is_contiguous());
  VRL_CHECK_OPERAND(uncond, cond);
  VRL_CHECK_OPERAND(u, cond);
  const c10::cuda::CUDAGuard guard(cond.device());
  const int64_t rows = cond.size(0);
  auto tokens = torch::empty({rows}, cond.options().dtype(torch::kInt64));
  auto logp = torch::empty({rows}, cond.options().dtype(torch::kFloat32));
  if (rows == 0) return {tokens, logp};
  auto stream = at::cuda::getCurrentCUDAStream();
  const float inv_t = (float)(1.0 / temperature);
  if (cond.scalar_type() == torch::kBFloat16) {
    sample_tokens_kernel<__nv_bfloat16><<<rows, kSampleThreads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(cond.data_ptr()),
        reinterpret_cast<const __nv_bfloat16*>(uncond.data_ptr()), u.data_ptr<float>(),
        tokens.data_ptr<int64_t>(), logp.data_ptr<float>(), (int)cond.size(1), (float)cfg_weight, inv_t);
  } else {
    TORCH_CHECK(cond.scalar_type() == torch::kFloat32);
    sample_tokens_kernel<float><<<rows, kSampleThreads, 0, stream>>>(
        cond.data_ptr<float>(), uncond.data_ptr<float>(), u.data_ptr<float>(),
        tokens.data_ptr<int64_t>(), logp.data_ptr<float>(), (int)cond.size(1), (float)cfg_weight, inv_t);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {tokens, logp};
}

// VRL_DECODE_ATTENTION=registers keeps the register form for caches the streaming form could serve
static bool decode_attention_bulk_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("VRL_DECODE_ATTENTION");
    return v == nullptr || std::string(v) != "registers";
  }();
  return on;
}

torch::Tensor decode_attention(torch::Tensor q, torch::Tensor k_cache, torch::Tensor v_cache,
                               torch::Tensor valid, int64_t length, double scale) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == torch::kBFloat16 && q.dim() == 4 && q.size(2) == 1 &&
              q.size(3) == 128 && q.is_contiguous(), "decode_attention: q must be [R, H, 1, 128] bf16");
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.dim() == 4 && k_cache.stride(3) == 1 && v_cache.stride(3) == 1 &&
              k_cache.scalar_type() == torch::kBFloat16 && v_cache.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(valid.scalar_type() == torch::kBool && valid.dim() == 2 && valid.stride(1) == 1);
  TORCH_CHECK(length <= k_cache.size(2) && length <= valid.size(1));
  TORCH_CHECK(k_cache.stride(0) % 4 == 0 && k_cache.stride(1) % 4 == 0 && k_cache.stride(2) % 4 == 0 &&
              v_cache.stride(0) % 4 == 0 && v_cache.stride(1) % 4 == 0 && v_cache.stride(2) % 4 == 0 &&
              reinterpret_cast<uintptr_t>(k_cache.data_ptr()) % 8 == 0 &&
              reinterpret_cast<uintptr_t>(v_cache.data_ptr()) % 8 == 0, "decode_attention: cache alignment");
  VRL_CHECK_OPERAND(k_cache, q);
  VRL_CHECK_OPERAND(v_cache, q);
  VRL_CHECK_OPERAND(valid, q);
  TORCH_CHECK(k_cache.size(0) >= q.size(0) && v_cache.size(0) >= q.size(0) && valid.size(0) >= q.size(0) &&
              k_cache.size(1) == q.size(1) && v_cache.size(1) == q.size(1) && length <= v_cache.size(2),
              "decode_attention: cache / mask shapes do not cover the query rows");
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t rows = q.size(0), heads = q.size(1);
  auto out = torch::empty_like(q);
  if (rows == 0) return out;
  // contiguous keys, 16-byte aligned runs, at most 1024 positions: the streaming form
  const bool bulk = k_cache.stride(2) == 128 && v_cache.stride(2) == 128 && length <= 1024 &&
                    k_cache.stride(0) % 8 == 0 && k_cache.stride(1) % 8 == 0 && v_cache.stride(0) % 8 == 0 &&
                    v_cache.stride(1) % 8 == 0 && reinterpret_cast<uintptr_t>(k_cache.data_ptr()) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(v_cache.data_ptr()) % 16 == 0 && decode_attention_bulk_enabled();
  if (bulk) {
    constexpr size_t smem = kDaStages * kDaStageBytes + 128;
    static const bool attr_set = [] {
      C10_CUDA_CHECK(cudaFuncSetAttribute(decode_attention_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
      return true;
    }();
    (void)attr_set;
    decode_attention_bulk_kernel<<<rows * heads, kDaThreads, smem, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(q.data_ptr()),
        reinterpret_cast<const __nv_bfloat16*>(k_cache.data_ptr()),
        reinterpret_cast<const __nv_bfloat16*>(v_cache.data_ptr()), valid.data_ptr<bool>(),
        reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), (int)heads, (int)length, k_cache.stride(0),
        k_cache.stride(1), v_cache.stride(0), v_cache.stride(1), valid.stride(0), (float)scale,
        kernel_status_block(q.get_device()) + kStatusAttention);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return out;
  }
  decode_attention_kernel<<<rows * heads, kDecodeWarps * 32, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(q.data_ptr()),
      reinterpret_cast<const __nv_bfloat16*>(k_cache.data_ptr()),
      reinterpret_cast<const __nv_bfloat16*>(v_cache.data_ptr()), valid.data_ptr<bool>(),
      reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), (int)heads, (int)length, k_cache.stride(0),
      k_cache.stride(1), k_cache.stride(2), v_cache.stride(0), v_cache.stride(1), v_cache.stride(2),
      valid.stride(0), (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// ------------------------------------------------------------------------------------------
// Decode-step glue of the LLaMA trunk (one query position per row, launch-latency bound): each of
// the three kernels below replaces a chain of tiny tensor ops that would otherwise cost a launch
// apiece inside the replayed CUDA graph.
//   decode_qkv_rope_append   fused QKV output [R, 3 H Dh] -> rotated q [R, H, 1, Dh]; rotated k and
//                            v are written straight into the caches at the position held in `pos`
//   swiglu_rows              [R, 2 F] (gate | up) -> silu(gate) * up  [R, F]
//   add_rmsnorm_rows         x += delta ; y = rmsnorm(x) * w   (residual add fused with the next norm)
// ------------------------------------------------------------------------------------------
namespace {

__global__ void __launch_bounds__(128)
decode_qkv_rope_append_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosT,
                              const float* __restrict__ sinT, const int64_t* __restrict__ pos,
                              __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ kc,
                              __nv_bfloat16* __restrict__ vc, int heads, int dh, int max_len,
                              int64_t c_sr, int64_t c_sh, int64_t c_sl) {
  // one block per (row, head); thread t owns the element pair (2t, 2t + 1) of q, k and v
  const int r = blockIdx.x / heads, h = blockIdx.x % heads;
  const int t = threadIdx.x;
  if (2 * t >= dh) return;
  const int64_t p = pos[0];
  if (p < 0 || p >= max_len) return;                       // a bad position must not write anywhere
  const int dmodel = heads * dh;
  const __nv_bfloat16* row = qkv + (int64_t)r * 3 * dmodel + h * dh + 2 * t;
  const float2 q2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row));
  const float2 k2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + dmodel));
  const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(row + 2 * dmodel);
  const float c = cosT[t], s = sinT[t];
  // bf16 rounding of the rotated values happens once, as in the tensor formulation
  const __nv_bfloat162 qr = __floats2bfloat162_rn(q2.x * c - q2.y * s, q2.x * s + q2.y * c);
  const __nv_bfloat162 kr = __floats2bfloat162_rn(k2.x * c - k2.y * s, k2.x * s + k2.y * c);
  *reinterpret_cast<__nv_bfloat162*>(q_out + ((int64_t)r * heads + h) * dh + 2 * t) = qr;
  const int64_t off = r * c_sr + h * c_sh + p * c_sl + 2 * t;
  *reinterpret_cast<__nv_bfloat162*>(kc + off) = kr;
  *reinterpret_cast<__nv_bfloat162*>(vc + off) = v2;
}

__global__ void __launch_bounds__(256)
swiglu_rows_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int64_t rows, int f) {
  const int64_t vec_per_row = f / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * vec_per_row;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row, v = i - r * vec_per_row;
    float g[8], u[8];
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * f + v * 8), g);
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * f + f + v * 8), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // silu in fp32, rounded to bf16 before the product, like F.silu(g) * u on bf16 tensors
      const float sg = __bfloat162float(__float2bfloat16_rn(g[j] / (1.f + __expf(-g[j]))));
      g[j] = sg * u[j];
    }
    *reinterpret_cast<bf16x8*>(out + r * f + v * 8) = pack8(g);
  }
}

__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                        const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int d, float eps) {
  __shared__ float red[32];
  const int64_t r = blockIdx.x;
  float acc = 0.f;
  for (int v = threadIdx.x; v < d / 8; v += blockDim.x) {
    float a[8], b[8];
    unpack8(*reinterpret_cast<const bf16x8*>(x + r * d + v * 8), a);
    if (delta != nullptr) {
      unpack8(*reinterpret_cast<const bf16x8*>(delta + r * d + v * 8), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = __bfloat162float(__float2bfloat16_rn(a[j] + b[j]));
      *reinterpret_cast<bf16x8*>(x + r * d + v * 8) = pack8(a);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += a[j] * a[j];
  }
  const float rs = rsqrtf(block_sum(acc, red) / (float)d + eps);
  for (int v = threadIdx.x; v < d / 8; v += blockDim.x) {
    float a[8], ww[8];
    unpack8(*reinterpret_cast<const bf16x8*>(x + r * d + v * 8), a);
    unpack8(*reinterpret_cast<const bf16x8*>(w + v * 8), ww);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = a[j] * rs * ww[j];
    *reinterpret_cast<bf16x8*>(y + r * d + v * 8) = pack8(a);
  }
}

}  // namespace

torch::Tensor decode_qkv_rope_append(torch::Tensor qkv, torch::Tensor cos, torch::Tensor sin, torch::Tensor pos,
                                     torch::Tensor k_cache, torch::Tensor v_cache, int64_t heads) {
  TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 2 && qkv.scalar_type() == torch::kBFloat16 && qkv.is_contiguous(),
              "decode_qkv_rope_append: qkv must be contiguous bf16 [R, 3 * H * Dh]");
  const int64_t rows = qkv.size(0), dmodel = qkv.size(1) / 3, dh = dmodel / heads;
  TORCH_CHECK(qkv.size(1) == 3 * heads * dh && dh % 2 == 0 && dh <= 256, "decode_qkv_rope_append: head size");
  VRL_CHECK_OPERAND(cos, qkv, torch::kFloat32, dh / 2);
  VRL_CHECK_OPERAND(sin, qkv, torch::kFloat32, dh / 2);
  VRL_CHECK_OPERAND(pos, qkv, torch::kInt64, 1);
  VRL_CHECK_OPERAND(k_cache, qkv, torch::kBFloat16);
  VRL_CHECK_OPERAND(v_cache, qkv, torch::kBFloat16);
  TORCH_CHECK(cos.is_contiguous() && sin.is_contiguous());
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.sizes() == v_cache.sizes() && k_cache.strides() == v_cache.strides() &&
              k_cache.size(0) >= rows && k_cache.size(1) == heads && k_cache.size(3) == dh &&
              k_cache.stride(3) == 1 && k_cache.stride(0) % 2 == 0 && k_cache.stride(1) % 2 == 0 &&
              k_cache.stride(2) % 2 == 0, "decode_qkv_rope_append: caches must be [R, H, L, Dh] with unit inner stride");
  const c10::cuda::CUDAGuard guard(qkv.device());
  auto q = torch::empty({rows, heads, 1, dh}, qkv.options());
  if (rows == 0) return q;
  decode_qkv_rope_append_kernel<<<(unsigned)(rows * heads), 128, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(qkv.data_ptr()), cos.data_ptr<float>(), sin.data_ptr<float>(),
      pos.data_ptr<int64_t>(), reinterpret_cast<__nv_bfloat16*>(q.data_ptr()),
      reinterpret_cast<__nv_bfloat16*>(k_cache.data_ptr()), reinterpret_cast<__nv_bfloat16*>(v_cache.data_ptr()),
      (int)heads, (int)dh, (int)k_cache.size(2), k_cache.stride(0), k_cache.stride(1), k_cache.stride(2));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return q;
}

torch::Tensor swiglu_rows(torch::Tensor gate_up) {
  TORCH_CHECK(gate_up.is_cuda() && gate_up.dim() == 2 && gate_up.scalar_type() == torch::kBFloat16 &&
              gate_up.is_contiguous() && gate_up.size(1) % 16 == 0, "swiglu_rows: contiguous bf16 [R, 2 F], F % 8 == 0");
  const c10::cuda::CUDAGuard guard(gate_up.device());
  const int64_t rows = gate_up.size(0), f = gate_up.size(1) / 2;
  auto out = torch::empty({rows, f}, gate_up.options());
  if (rows == 0) return out;
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((rows * f / 8 + 255) / 256, 148 * 4));
  swiglu_rows_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(gate_up.data_ptr()), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()),
      rows, (int)f);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// x (updated in place when `delta` is given) and the normalised rows.
torch::Tensor add_rmsnorm_rows(torch::Tensor x, c10::optional<torch::Tensor> delta, torch::Tensor w, double eps) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() &&
              x.size(1) % 8 == 0, "add_rmsnorm_rows: contiguous bf16 [R, D], D % 8 == 0");
  VRL_CHECK_OPERAND(delta, x, torch::kBFloat16, x.numel());
  VRL_CHECK_OPERAND(w, x, torch::kBFloat16, x.size(1));
  TORCH_CHECK(w.is_contiguous() && (!delta.has_value() || delta->is_contiguous()));
  const c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty_like(x);
  if (x.size(0) == 0) return y;
  add_rmsnorm_rows_kernel<<<(unsigned)x.size(0), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<__nv_bfloat16*>(x.data_ptr()),
      delta.has_value() ? reinterpret_cast<const __nv_bfloat16*>(delta->data_ptr()) : nullptr,
      reinterpret_cast<const __nv_bfloat16*>(w.data_ptr()), reinterpret_cast<__nv_bfloat16*>(y.data_ptr()),
      (int)x.size(1), (float)eps);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

// ------------------------------------------------------------------------------------------
// Low-rank adapter for decode-sized inputs: y += scale * (x A^T) B^T with R <= 64 rows.  Two tiny
// CUDA-core kernels (the contraction over K is split over blocks; the rank-r update is a few
// multiply-adds per output) instead of two tensor-core launches whose single tile would stream
// K serially, plus the scaling and the add.
//   lora_down_rows   low[R, r] (fp32) = x[R, K] A[r, K]^T        one warp per (row, adapter row)
//   lora_up_add_rows y[R, N] += scale * low[R, r] B[N, r]^T      one thread per (8 rows, column)
// ------------------------------------------------------------------------------------------
namespace {

constexpr int kLoraRowsPerBlock = 8;

__global__ void __launch_bounds__(kLoraRowsPerBlock * 32)
lora_down_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ a,
                      float* __restrict__ low, int rows, int k, int rank) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y * kLoraRowsPerBlock + warp, j = blockIdx.x;
  if (row >= rows) return;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (int64_t)row * k);
  const bf16x8* ar = reinterpret_cast<const bf16x8*>(a + (int64_t)j * k);
  float acc = 0.f;
  for (int i = lane; i < k / 8; i += 32) {
    float xv[8], av[8];
    unpack8(xr[i], xv);
    unpack8(ar[i], av);
#pragma unroll
    for (int t = 0; t < 8; ++t) acc = fmaf(xv[t], av[t], acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) low[(int64_t)row * rank + j] = acc;
}

constexpr int kLoraRankChunk = 32;

__global__ void __launch_bounds__(256)
lora_up_add_rows_kernel(__nv_bfloat16* __restrict__ y, const float* __restrict__ low,
                        const __nv_bfloat16* __restrict__ b, int rows, int n, int rank, float scale) {
  extern __shared__ __align__(16) float low_s[];                 // [kLoraRowsPerBlock][rank]
  const int row0 = blockIdx.y * kLoraRowsPerBlock;
  const int nrows = min(kLoraRowsPerBlock, rows - row0);
  for (int i = threadIdx.x; i < kLoraRowsPerBlock * rank; i += blockDim.x)
    low_s[i] = i < nrows * rank ? low[(int64_t)row0 * rank + i] * scale : 0.f;
  __syncthreads();
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= n) return;
  float acc[kLoraRowsPerBlock];
#pragma unroll
  for (int r = 0; r < kLoraRowsPerBlock; ++r) acc[r] = 0.f;
  const bf16x8* br = reinterpret_cast<const bf16x8*>(b + (int64_t)col * rank);
  // the adapter row goes through registers 32 values at a time; the rows' low-rank activations are
  // broadcast reads of shared memory, four values per load
  for (int c0 = 0; c0 < rank; c0 += kLoraRankChunk) {
    const int width = min(kLoraRankChunk, rank - c0);            // a multiple of 8
    float bv[kLoraRankChunk];
#pragma unroll
    for (int i = 0; i < kLoraRankChunk / 8; ++i) {
      if (i * 8 < width) {
        unpack8(br[c0 / 8 + i], bv + i * 8);
      } else {
#pragma unroll
        for (int t = 0; t < 8; ++t) bv[i * 8 + t] = 0.f;
      }
    }
#pragma unroll
    for (int r = 0; r < kLoraRowsPerBlock; ++r) {
      const float4* lr = reinterpret_cast<const float4*>(low_s + r * rank + c0);
      float a = acc[r];
#pragma unroll
      for (int i = 0; i < kLoraRankChunk / 4; ++i) {
        if (i * 4 < width) {
          const float4 l4 = lr[i];
          a = fmaf(l4.x, bv[4 * i], a);
          a = fmaf(l4.y, bv[4 * i + 1], a);
          a = fmaf(l4.z, bv[4 * i + 2], a);
          a = fmaf(l4.w, bv[4 * i + 3], a);
        }
      }
      acc[r] = a;
    }
  }
  for (int r = 0; r < nrows; ++r) {
    __nv_bfloat16* dst = y + (int64_t)(row0 + r) * n + col;
    *dst = __float2bfloat16_rn(__bfloat162float(*dst) + acc[r]);
  }
}

}  // namespace

// y (bf16 [R, N], updated in place) += scale * (x A^T) B^T for R <= 64 rows.
void lora_apply_rows(torch::Tensor y, torch::Tensor x, torch::Tensor a, torch::Tensor b, double scale) {
  TORCH_CHECK(y.is_cuda() && y.dim() == 2 && y.scalar_type() == torch::kBFloat16 && y.is_contiguous(),
              "lora_apply_rows: y must be a contiguous bf16 [R, N] CUDA tensor");
  VRL_CHECK_OPERAND(x, y, torch::kBFloat16);
  VRL_CHECK_OPERAND(a, y, torch::kBFloat16);
  VRL_CHECK_OPERAND(b, y, torch::kBFloat16);
  const int64_t rows = y.size(0), n = y.size(1);
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.size(0) == rows && a.dim() == 2 && a.is_contiguous() &&
              b.dim() == 2 && b.is_contiguous() && a.size(1) == x.size(1) && b.size(0) == n && b.size(1) == a.size(0),
              "lora_apply_rows: x [R, K], A [r, K], B [N, r]");
  const int64_t k = x.size(1), rank = a.size(0);
  TORCH_CHECK(rows <= 64 && k % 8 == 0 && rank % 8 == 0 && rank >= 8 && rank <= 256,
              "lora_apply_rows: R <= 64, K % 8 == 0, adapter rank a multiple of 8 up to 256");
  if (rows == 0 || n == 0) return;
  const c10::cuda::CUDAGuard guard(y.device());
  auto low = torch::empty({rows, rank}, y.options().dtype(torch::kFloat32));
  auto stream = at::cuda::getCurrentCUDAStream();
  const unsigned row_blocks = (unsigned)((rows + kLoraRowsPerBlock - 1) / kLoraRowsPerBlock);
  lora_down_rows_kernel<<<dim3((unsigned)rank, row_blocks), kLoraRowsPerBlock * 32, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(a.data_ptr()),
      low.data_ptr<float>(), (int)rows, (int)k, (int)rank);
  lora_up_add_rows_kernel<<<dim3((unsigned)((n + 255) / 256), row_blocks), 256,
                            kLoraRowsPerBlock * rank * sizeof(float), stream>>>(
      reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), low.data_ptr<float>(),
      reinterpret_cast<const __nv_bfloat16*>(b.data_ptr()), (int)rows, (int)n, (int)rank, (float)scale);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

torch::Tensor group_advantages(torch::Tensor rewards, torch::Tensor group_ids, double eps, double clip,
                               bool global_std) {
  TORCH_CHECK(rewards.is_cuda() && rewards.dim() == 1 && group_ids.numel() == rewards.numel());
  VRL_CHECK_OPERAND(group_ids, rewards);
  const c10::cuda::CUDAGuard guard(rewards.device());
  auto r = rewards.to(torch::kFloat32).contiguous();
  auto g = group_ids.to(torch::kInt64).contiguous();
  auto adv = torch::empty_like(r);
  const int n = (int)r.numel();
  if (n == 0) return adv;
  TORCH_CHECK(n <= 16384, "group_advantages: batch larger than the single-block kernel supports");
  group_advantages_kernel<<<1, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      r.data_ptr<float>(), g.data_ptr<int64_t>(), adv.data_ptr<float>(), n, (float)eps, (float)clip,
      global_std ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return adv;
}

}  // namespace vrl
