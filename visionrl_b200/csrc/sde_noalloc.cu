// Allocation-free C entry point of the SDE step (declaration and contract: sde_noalloc.h).
#include "sde_noalloc.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>

namespace vrl {
// raw-pointer launcher and grid sizing of the step kernels (elementwise.cu)
int sde_blocks_per_sample(int64_t n);
void sde_step_launch(const float* v, const float* x, const float* a, const float* b,
                     const float* scale, const float* dt, const float* prev_in,
                     const float* noise, float* prev_out, float* mean_out, float* logp,
                     float* partial, int batch, int64_t n, bool deterministic, bool gaussian,
                     cudaStream_t stream);
}  // namespace vrl

namespace {

// Per-block partial sums of the log-density reduction live here instead of in a per-call
// allocation.  The array belongs to the module image on every device that loads it.
static __device__ __align__(256) float g_sde_scratch[VRL_SDE_NOALLOC_MAX_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
// address of g_sde_scratch on each device, resolved on the first call with that device current
std::atomic<float*> g_scratch_addr[kMaxDevices];

int fail(int code, char* err, size_t err_len, const char* what, const char* detail) {
  if (err != nullptr && err_len > 0) snprintf(err, err_len, "vrl_sde_step_noalloc: %s%s%s", what,
                                             detail ? ": " : "", detail ? detail : "");
  return code;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int vrl_sde_step_noalloc(
    const float* v, const float* x, const float* a, const float* b, const float* scale,
    const float* dt, const float* prev_in, const float* noise, float* next_out, float* mean_out,
    float* logp, int batch, int64_t n, int deterministic, int gaussian, void* stream, char* err,
    size_t err_len) {
  if (v == nullptr || x == nullptr || a == nullptr || b == nullptr || scale == nullptr ||
      dt == nullptr || next_out == nullptr || mean_out == nullptr || logp == nullptr)
    return fail(1, err, err_len, "null pointer argument", nullptr);
  if (prev_in == nullptr && noise == nullptr)
    return fail(1, err, err_len, "one of prev_in and noise is required", nullptr);
  if (batch <= 0 || n <= 0) return fail(1, err, err_len, "batch and n must be positive", nullptr);
  if (batch > 65535) return fail(1, err, err_len, "batch exceeds the grid limit of 65535", nullptr);

  // blocks per sample in 64-bit arithmetic BEFORE any narrowing: an absurd n must be rejected
  // here (rc 2) instead of wrapping through `int` and reaching the launch
  constexpr int64_t kElemsPerBlock = 4096;
  const int64_t blocks_per_sample = n / kElemsPerBlock + (n % kElemsPerBlock != 0 ? 1 : 0);
  const int64_t need = blocks_per_sample <= VRL_SDE_NOALLOC_MAX_SCRATCH_FLOATS
                           ? (int64_t)batch * blocks_per_sample
                           : (int64_t)VRL_SDE_NOALLOC_MAX_SCRATCH_FLOATS + 1;
  if (need > VRL_SDE_NOALLOC_MAX_SCRATCH_FLOATS ||
      blocks_per_sample != (int64_t)vrl::sde_blocks_per_sample(n)) {
    char detail[160];
    snprintf(detail, sizeof(detail), "batch * ceil(n / 4096) = %lld floats of scratch needed, %d available",
             (long long)need, VRL_SDE_NOALLOC_MAX_SCRATCH_FLOATS);
    return fail(2, err, err_len, "problem too large for the fixed scratch array", detail);
  }

  int device = -1;
  cudaError_t rc = cudaGetDevice(&device);
  if (rc != cudaSuccess) return fail(3, err, err_len, "cudaGetDevice failed", cudaGetErrorString(rc));
  if (device < 0 || device >= kMaxDevices) return fail(3, err, err_len, "device index out of range", nullptr);
  float* scratch = g_scratch_addr[device].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // one-time set-up for this device (not capturable: keep the first call out of stream capture)
    rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_sde_scratch);
    if (rc != cudaSuccess || scratch == nullptr)
      return fail(3, err, err_len, "cudaGetSymbolAddress failed", cudaGetErrorString(rc));
    g_scratch_addr[device].store(scratch, std::memory_order_release);
  }

  // An error left behind by unrelated earlier work would otherwise be reported (and cleared) as
  // this call's launch failure: look without clearing, and name it for what it is.
  rc = cudaPeekAtLastError();
  if (rc != cudaSuccess)
    return fail(5, err, err_len, "a CUDA error from earlier work is pending; nothing was launched",
                cudaGetErrorString(rc));
  vrl::sde_step_launch(v, x, a, b, scale, dt, prev_in, noise, next_out, mean_out, logp, scratch, batch,
                       n, deterministic != 0, gaussian != 0, static_cast<cudaStream_t>(stream));
  rc = cudaGetLastError();
  if (rc != cudaSuccess) return fail(4, err, err_len, "kernel launch failed", cudaGetErrorString(rc));
  if (err != nullptr && err_len > 0) err[0] = '\0';
  return 0;
}
