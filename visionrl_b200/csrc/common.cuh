// Shared device helpers for the sm_100a kernels of visionrl_b200.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vrl {

constexpr int kWarp = 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread receives the result.  `scratch` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nwarps) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) {
    r = warp_sum(r);
    if (lane == 0) scratch[0] = r;
  }
  __syncthreads();
  return scratch[0];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nwarps) ? scratch[threadIdx.x] : -INFINITY;
  if (warp == 0) {
    r = warp_max(r);
    if (lane == 0) scratch[0] = r;
  }
  __syncthreads();
  return scratch[0];
}

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 16-byte vector of 8 bf16 values.
// Eight bf16 values moved as ONE 128-bit access.  The payload is a single uint4 member so that
// copying the struct through a pointer compiles to one LDG.128 / STG.128 (a struct of four
// 32-bit members is copied member by member, i.e. four 4-byte accesses per thread).
struct alignas(16) bf16x8 {
  uint4 u;
};

__device__ __forceinline__ float2 bf16pair_to_float2(uint32_t w) {
  __nv_bfloat162 h;
  memcpy(&h, &w, sizeof(w));
  return __bfloat1622float2(h);
}

__device__ __forceinline__ uint32_t float2_to_bf16pair(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  uint32_t w;
  memcpy(&w, &h, sizeof(w));
  return w;
}

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
  const uint4 u = p.u;
  float2 t;
  t = bf16pair_to_float2(u.x); f[0] = t.x; f[1] = t.y;
  t = bf16pair_to_float2(u.y); f[2] = t.x; f[3] = t.y;
  t = bf16pair_to_float2(u.z); f[4] = t.x; f[5] = t.y;
  t = bf16pair_to_float2(u.w); f[6] = t.x; f[7] = t.y;
}

__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
  p.u = make_uint4(float2_to_bf16pair(f[0], f[1]), float2_to_bf16pair(f[2], f[3]),
                   float2_to_bf16pair(f[4], f[5]), float2_to_bf16pair(f[6], f[7]));
  return p;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}

// d/dx of gelu_tanh
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (x + k1 * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

}  // namespace vrl
