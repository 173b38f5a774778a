// Collectives fused into compute over NVLink peer memory (F2, F3, F4).
//
// Every kernel receives a device array of peer base pointers into one symmetric allocation
// (the same offset means the same logical element on every rank) and moves data with plain
// peer loads / stores issued from inside the kernel — no library collective is called.
//
//   rs_sum_slice            gradient reduce-scatter fused with the bf16->fp32 cast, the 1/world
//                           scale and the sum of squares of the reduced slice (for clipping)
//   adamw_slice_broadcast   sharded AdamW on the owned slice fused with the all-gather: the new
//                           bf16 parameters are stored straight into every rank's buffer
//   p2p_broadcast_versioned trainer -> rollout weight broadcast with a release-ordered version
//   wait_flag               bounded wait on a flag word; reports instead of hanging
//   ulysses_scatter         head<->sequence exchange of sequence parallelism as peer stores
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "ops.h"

namespace vrl {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
  void* p[kMaxPeers];
};

static PeerPtrs load_peers(const torch::Tensor& peers, int world) {
  TORCH_CHECK(world >= 1 && world <= kMaxPeers, "world size must be in [1, 16]");
  TORCH_CHECK(peers.device().is_cpu() && peers.scalar_type() == torch::kInt64 &&
              peers.numel() >= world, "peer pointer table must be a CPU int64 tensor");
  PeerPtrs out{};
  const int64_t* src = peers.data_ptr<int64_t>();
  for (int i = 0; i < world; ++i) out.p[i] = reinterpret_cast<void*>(src[i]);
  return out;
}

// ------------------------------------------------------------------------------------------
// F2 part 1: out[i] = scale * sum_r peer_r[lo + i]; partial[block] = sum out[i]^2
// ------------------------------------------------------------------------------------------
template <bool kBf16>
__global__ void __launch_bounds__(256)
rs_sum_slice_kernel(PeerPtrs peers, float* __restrict__ out, float* __restrict__ partial,
                    int64_t lo, int64_t n, int world, int rank, float inv) {
  __shared__ float red[32];
  float acc = 0.f;
  if (kBf16) {
    const int64_t nvec = n / 8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (int64_t)gridDim.x * blockDim.x) {
      float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < world; ++r) {
        // start with this rank's own copy, then walk the ring so peers are read evenly
        const int src = (rank + r) % world;
        const bf16x8 v = *(reinterpret_cast<const bf16x8*>(
                               reinterpret_cast<const __nv_bfloat16*>(peers.p[src]) + lo) + i);
        float f[8];
        unpack8(v, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j] += f[j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s[j] *= inv; acc += s[j] * s[j]; }
      *reinterpret_cast<float4*>(out + i * 8) = make_float4(s[0], s[1], s[2], s[3]);
      *reinterpret_cast<float4*>(out + i * 8 + 4) = make_float4(s[4], s[5], s[6], s[7]);
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
      float s = 0.f;
      for (int r = 0; r < world; ++r) {
        const int src = (rank + r) % world;
        s += reinterpret_cast<const float*>(peers.p[src])[lo + i];
      }
      s *= inv;
      out[i] = s;
      acc += s * s;
    }
  }
  const float total = block_sum(acc, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = total;
}

__global__ void collective_sum_finalize(const float* __restrict__ partial, float* __restrict__ out,
                                        int count) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < count; i += blockDim.x) acc += partial[i];
  const float s = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = s;
}

torch::Tensor rs_sum_slice(torch::Tensor peers, torch::Tensor out, int64_t lo, int64_t n,
                           int64_t world, int64_t rank, bool is_bf16, double scale) {
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kFloat32 && out.numel() >= n);
  TORCH_CHECK(lo % 8 == 0 && n % 8 == 0, "slice bounds must be multiples of 8 elements");
  const c10::cuda::CUDAGuard guard(out.device());
  const PeerPtrs pp = load_peers(peers, (int)world);
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((n / 8 + 255) / 256, 148 * 8));
  auto partial = torch::empty({blocks}, out.options());
  auto sumsq = torch::empty({}, out.options());
  auto stream = at::cuda::getCurrentCUDAStream();
  if (is_bf16) {
    rs_sum_slice_kernel<true><<<blocks, 256, 0, stream>>>(pp, out.data_ptr<float>(),
                                                          partial.data_ptr<float>(), lo, n,
                                                          (int)world, (int)rank, (float)scale);
  } else {
    rs_sum_slice_kernel<false><<<blocks, 256, 0, stream>>>(pp, out.data_ptr<float>(),
                                                           partial.data_ptr<float>(), lo, n,
                                                           (int)world, (int)rank, (float)scale);
  }
  collective_sum_finalize<<<1, 256, 0, stream>>>(partial.data_ptr<float>(), sumsq.data_ptr<float>(),
                                                 blocks);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return sumsq;
}

// ------------------------------------------------------------------------------------------
// F2 part 2 + all-gather: AdamW on the owned slice, result stored into every rank's buffer
// ------------------------------------------------------------------------------------------
template <bool kBf16>
__global__ void __launch_bounds__(256)
adamw_slice_broadcast_kernel(PeerPtrs peers, const float* __restrict__ g,
                             float* __restrict__ master, float* __restrict__ m,
                             float* __restrict__ v, int64_t lo, int64_t n, int world, int rank,
                             float lr, float b1, float b2, float eps, float wd, float bc1,
                             float bc2, const float* __restrict__ clip) {
  const float coef = clip ? clip[0] : 1.f;
  const int64_t nvec = n / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t e = i * 8 + j;
      const float grad = g[e] * coef;
      const float mi = b1 * m[e] + (1.f - b1) * grad;
      const float vi = b2 * v[e] + (1.f - b2) * grad * grad;
      m[e] = mi;
      v[e] = vi;
      float x = master[e];
      x = x * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
      master[e] = x;
      w[j] = x;
    }
    if (kBf16) {
      const bf16x8 packed = pack8(w);
      for (int r = 0; r < world; ++r) {
        const int dst = (rank + r) % world;
        *(reinterpret_cast<bf16x8*>(reinterpret_cast<__nv_bfloat16*>(peers.p[dst]) + lo) + i) = packed;
      }
    } else {
      for (int r = 0; r < world; ++r) {
        const int dst = (rank + r) % world;
        float* base = reinterpret_cast<float*>(peers.p[dst]) + lo + i * 8;
        // when the parameters are fp32 the local copy *is* the master buffer
        if (base == master + i * 8) continue;
        *reinterpret_cast<float4*>(base) = make_float4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<float4*>(base + 4) = make_float4(w[4], w[5], w[6], w[7]);
      }
    }
  }
}

void adamw_slice_broadcast(torch::Tensor peers, torch::Tensor g, torch::Tensor master,
                           torch::Tensor m, torch::Tensor v, int64_t lo, int64_t n, int64_t world,
                           int64_t rank, double lr, double b1, double b2, double eps, double wd,
                           int64_t step, c10::optional<torch::Tensor> clip, bool is_bf16) {
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == torch::kFloat32 && g.numel() >= n && g.is_contiguous());
  VRL_CHECK_OPERAND(master, g, torch::kFloat32);
  VRL_CHECK_OPERAND(m, g, torch::kFloat32);
  VRL_CHECK_OPERAND(v, g, torch::kFloat32);
  VRL_CHECK_OPERAND(clip, g);
  TORCH_CHECK(master.numel() >= n && m.numel() >= n && v.numel() >= n && master.is_contiguous() &&
              m.is_contiguous() && v.is_contiguous(),
              "adamw_slice_broadcast: master / moments must be contiguous and cover the slice");
  TORCH_CHECK(lo % 8 == 0 && n % 8 == 0, "slice bounds must be multiples of 8 elements");
  const c10::cuda::CUDAGuard guard(g.device());
  const PeerPtrs pp = load_peers(peers, (int)world);
  const float bc1 = 1.f - (float)std::pow(b1, (double)step);
  const float bc2 = 1.f - (float)std::pow(b2, (double)step);
  torch::Tensor c;
  const float* cp = nullptr;
  if (clip.has_value()) { c = clip->to(torch::kFloat32).contiguous(); cp = c.data_ptr<float>(); }
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((n / 8 + 255) / 256, 148 * 8));
  auto stream = at::cuda::getCurrentCUDAStream();
  if (is_bf16) {
    adamw_slice_broadcast_kernel<true><<<blocks, 256, 0, stream>>>(
        pp, g.data_ptr<float>(), master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
        lo, n, (int)world, (int)rank, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, bc1,
        bc2, cp);
  } else {
    adamw_slice_broadcast_kernel<false><<<blocks, 256, 0, stream>>>(
        pp, g.data_ptr<float>(), master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
        lo, n, (int)world, (int)rank, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, bc1,
        bc2, cp);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// F4: broadcast of a local buffer into every peer's buffer, then a release-ordered version
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
p2p_broadcast_kernel(const uint4* __restrict__ src, PeerPtrs dst, int64_t dst_off_vec,
                     int64_t nvec, int world, int rank, int include_self) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 val = src[i];
    for (int r = include_self ? 0 : 1; r < world; ++r) {
      const int d = (rank + r) % world;
      reinterpret_cast<uint4*>(dst.p[d])[dst_off_vec + i] = val;
    }
  }
}

__global__ void publish_version_kernel(PeerPtrs flags, int64_t slot, int world, int version) {
  // the broadcast kernel ran before this one on the same stream; make its peer stores visible
  // system-wide before any peer can observe the new version
  __threadfence_system();
  if (threadIdx.x < world) {
    int* f = reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f), "r"(version) : "memory");
  }
}

void p2p_broadcast_versioned(torch::Tensor src, torch::Tensor dst_peers, int64_t dst_offset_bytes,
                             torch::Tensor flag_peers, int64_t flag_slot, int64_t world,
                             int64_t rank, int64_t version, bool include_self) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous());
  const int64_t bytes = src.numel() * src.element_size();
  TORCH_CHECK(bytes % 16 == 0 && dst_offset_bytes % 16 == 0 &&
              reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0,
              "p2p_broadcast: sizes, offsets and the source must be 16-byte aligned");
  const c10::cuda::CUDAGuard guard(src.device());
  const PeerPtrs dp = load_peers(dst_peers, (int)world);
  const PeerPtrs fp = load_peers(flag_peers, (int)world);
  const int64_t nvec = bytes / 16;
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((nvec + 255) / 256, 148 * 8));
  auto stream = at::cuda::getCurrentCUDAStream();
  p2p_broadcast_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(src.data_ptr()), dp,
                                                   dst_offset_bytes / 16, nvec, (int)world,
                                                   (int)rank, include_self ? 1 : 0);
  publish_version_kernel<<<1, 32, 0, stream>>>(fp, flag_slot, (int)world, (int)version);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Table-driven form of the broadcast: segment j copies `count` 16-bit elements from
// src_flat + src_off to offset dst_off of EVERY rank's destination buffer.  One launch publishes
// all of a rank's parameter shards into the rollout replicas of the whole group.
// Blocks per segment of the table-driven kernels: enough blocks in total to give every SM several
// (a peer access takes microseconds, so bandwidth over NVLink needs many requests in flight),
// however few segments the table has, and never more than the longest segment can feed.
static int table_grid_x(int64_t segments, int64_t max_segment) {
  const int64_t wanted = (148 * 8 + segments - 1) / segments;
  const int64_t useful = (max_segment / 8 + 255) / 256;
  return (int)std::max<int64_t>(1, std::min<int64_t>(std::min(wanted, useful), 65535));
}

__global__ void __launch_bounds__(256)
p2p_broadcast_table_kernel(const uint4* __restrict__ src, PeerPtrs dst, const int64_t* __restrict__ table,
                           int world, int rank) {
  const int64_t src_vec = table[blockIdx.y * 3 + 0] / 8, dst_vec = table[blockIdx.y * 3 + 1] / 8;
  const int64_t nvec = table[blockIdx.y * 3 + 2] / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 val = src[src_vec + i];
    for (int r = 0; r < world; ++r) {
      const int d = (rank + r) % world;          // own copy first, then round the ring
      reinterpret_cast<uint4*>(dst.p[d])[dst_vec + i] = val;
    }
  }
}

void p2p_broadcast_table(torch::Tensor src_flat, torch::Tensor dst_peers, torch::Tensor table,
                         int64_t world, int64_t rank, int64_t max_segment) {
  TORCH_CHECK(src_flat.is_cuda() && src_flat.is_contiguous() && src_flat.element_size() == 2 &&
              reinterpret_cast<uintptr_t>(src_flat.data_ptr()) % 16 == 0,
              "p2p_broadcast_table: contiguous 16-bit source, 16-byte aligned");
  VRL_CHECK_OPERAND(table, src_flat, torch::kInt64);
  TORCH_CHECK(table.dim() == 2 && table.size(1) == 3 && table.is_contiguous() && table.size(0) >= 1 &&
              table.size(0) <= 65535, "p2p_broadcast_table: segment table [segments, 3] (src, dst, count), "
              "all multiples of 8 elements");
  TORCH_CHECK(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world && max_segment > 0);
  const c10::cuda::CUDAGuard guard(src_flat.device());
  const PeerPtrs dp = load_peers(dst_peers, (int)world);
  const int bx = table_grid_x(table.size(0), max_segment);
  p2p_broadcast_table_kernel<<<dim3(bx, (unsigned)table.size(0)), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const uint4*>(src_flat.data_ptr()), dp, table.data_ptr<int64_t>(), (int)world, (int)rank);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Bounded wait: status[0] = 0 when flag >= expected was observed, 1 when the limit ran out.
__global__ void wait_flag_kernel(const int* __restrict__ flag, int expected, int* __restrict__ status,
                                 long long max_spins) {
  if (threadIdx.x != 0) return;
  int seen = 0;
  for (long long spin = 0; spin < max_spins; ++spin) {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (seen >= expected) { status[0] = 0; status[1] = seen; return; }
    __nanosleep(200);
  }
  status[0] = 1;
  status[1] = seen;
}

torch::Tensor wait_flag(torch::Tensor flags, int64_t slot, int64_t expected, double timeout_s) {
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == torch::kInt32);
  const c10::cuda::CUDAGuard guard(flags.device());
  auto status = torch::zeros({2}, flags.options());
  const long long spins = (long long)std::max(1.0, timeout_s * 2.0e6);   // ~0.5 us per poll
  wait_flag_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(
      flags.data_ptr<int>() + slot, (int)expected, status.data_ptr<int>(), spins);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return status;
}

// ------------------------------------------------------------------------------------------
// Flag signalling between ranks.  A flag array is a small symmetric int32 allocation; slot
// (base + r) of every rank's array is written only by rank r, so no slot has two writers.
// Every wait is bounded by wall-clock time (%globaltimer): on expiry the kernel records
// {1, peer slot, last value seen, value expected} in `status` (first failure wins) and RETURNS,
// so a departed peer costs the others a timeout and a Python exception, never a hung GPU.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// true when `flag` reached `expected` (wrap-safe signed distance) before the deadline
__device__ __forceinline__ bool bounded_flag_wait(const int* flag, int expected, unsigned long long timeout_ns,
                                                  int* seen_out) {
  const unsigned long long t0 = global_ns();
  int seen = 0;
  for (;;) {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (seen - expected >= 0) { *seen_out = seen; return true; }
    if (global_ns() - t0 > timeout_ns) { *seen_out = seen; return false; }
    __nanosleep(100);
  }
}

__device__ __forceinline__ void report_timeout(int* status, int slot, int seen, int expected) {
  if (atomicCAS(status, 0, 1) == 0) {
    status[1] = slot;
    status[2] = seen;
    status[3] = expected;
  }
}

// Lane r stores `value` into slot `slot` of rank r's flag array.  Everything this rank wrote
// before (earlier kernels of the stream included) is visible to a peer that acquires the flag.
__global__ void flag_signal_kernel(PeerPtrs flags, int slot, int world, int value) {
  __threadfence_system();
  if (threadIdx.x < world) {
    int* f = reinterpret_cast<int*>(flags.p[threadIdx.x]) + slot;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f), "r"(value) : "memory");
  }
}

// Lane i waits until local slot (slot0 + i) has reached `expected`.
__global__ void flag_wait_kernel(const int* __restrict__ flags, int slot0, int count, int expected,
                                 unsigned long long timeout_ns, int* __restrict__ status) {
  if (threadIdx.x < count) {
    int seen = 0;
    if (!bounded_flag_wait(flags + slot0 + threadIdx.x, expected, timeout_ns, &seen))
      report_timeout(status, slot0 + threadIdx.x, seen, expected);
  }
  __threadfence_system();
}

// Barrier = signal every peer, then wait for every peer, in one launch.
__global__ void flag_barrier_kernel(PeerPtrs flags, const int* __restrict__ local, int base, int world,
                                    int rank, int epoch, unsigned long long timeout_ns,
                                    int* __restrict__ status) {
  __threadfence_system();
  if (threadIdx.x < world) {
    int* f = reinterpret_cast<int*>(flags.p[threadIdx.x]) + base + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    int seen = 0;
    if (!bounded_flag_wait(local + base + threadIdx.x, epoch, timeout_ns, &seen))
      report_timeout(status, base + threadIdx.x, seen, epoch);
  }
  __threadfence_system();
}

static unsigned long long to_ns(double timeout_s) {
  return (unsigned long long)(std::max(1e-4, std::min(timeout_s, 600.0)) * 1e9);
}

static void check_flags(const torch::Tensor& flags, const torch::Tensor& status, int64_t last_slot) {
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == torch::kInt32 && flags.is_contiguous() &&
              last_slot < flags.numel(), "flag array: contiguous int32 CUDA tensor covering the slots");
  VRL_CHECK_OPERAND(status, flags, torch::kInt32);
  TORCH_CHECK(status.numel() >= 4 && status.is_contiguous(), "status: int32[>=4]");
}

void flag_signal(torch::Tensor flag_peers, torch::Tensor flags, int64_t slot, int64_t world, int64_t value) {
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == torch::kInt32 && slot >= 0 && slot < flags.numel());
  const c10::cuda::CUDAGuard guard(flags.device());
  const PeerPtrs fp = load_peers(flag_peers, (int)world);
  flag_signal_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(fp, (int)slot, (int)world, (int)value);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void flag_wait(torch::Tensor flags, int64_t slot0, int64_t count, int64_t expected, double timeout_s,
               torch::Tensor status) {
  TORCH_CHECK(count >= 1 && count <= 32 && slot0 >= 0, "flag_wait: 1..32 consecutive slots");
  check_flags(flags, status, slot0 + count - 1);
  const c10::cuda::CUDAGuard guard(flags.device());
  flag_wait_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(
      flags.data_ptr<int>(), (int)slot0, (int)count, (int)expected, to_ns(timeout_s), status.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void flag_barrier(torch::Tensor flag_peers, torch::Tensor flags, int64_t base, int64_t world, int64_t rank,
                  int64_t epoch, double timeout_s, torch::Tensor status) {
  TORCH_CHECK(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world && base >= 0);
  check_flags(flags, status, base + world - 1);
  const c10::cuda::CUDAGuard guard(flags.device());
  const PeerPtrs fp = load_peers(flag_peers, (int)world);
  flag_barrier_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(
      fp, flags.data_ptr<int>(), (int)base, (int)world, (int)rank, (int)epoch, to_ns(timeout_s),
      status.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// Sharded-parameter training (F1 / F2 support kernels).
//
//   bucket_reduce_acc   gradient reduce-scatter of one bucket fused with the bf16 -> fp32 cast,
//                       the scale and the accumulation into this rank's persistent fp32 gradient
//                       shard: for every segment (one per weight of the bucket)
//                           gshard[dst + i] += scale * sum_r stage_r[src + i]
//                       where stage_r is rank r's staging buffer read over NVLink.
//   p2p_gather_rows     stand-alone all-gather of a row-sharded weight into a local full buffer
//                       (the fused form lives in the GEMM; this one serves checkpoints and the
//                       rare backward that finds its gathered copy evicted).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
bucket_reduce_acc_kernel(PeerPtrs stage, const int64_t* __restrict__ table, float* __restrict__ gshard,
                         float scale, int world, int rank) {
  const int64_t src = table[blockIdx.y * 3 + 0], dst = table[blockIdx.y * 3 + 1];
  const int64_t nvec = table[blockIdx.y * 3 + 2] / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (int64_t)gridDim.x * blockDim.x) {
    bf16x8 part[kMaxPeers];
    // issue every peer's load before the first use: NVLink latency overlaps across peers
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r < world) {
        const int from = (rank + r) % world;
        part[r] = *(reinterpret_cast<const bf16x8*>(reinterpret_cast<const __nv_bfloat16*>(stage.p[from]) + src) + i);
      }
    }
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r < world) {
        float f[8];
        unpack8(part[r], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j] += f[j];
      }
    }
    float4* out = reinterpret_cast<float4*>(gshard + dst + i * 8);
    float4 lo = out[0], hi = out[1];
    lo.x += scale * s[0]; lo.y += scale * s[1]; lo.z += scale * s[2]; lo.w += scale * s[3];
    hi.x += scale * s[4]; hi.y += scale * s[5]; hi.z += scale * s[6]; hi.w += scale * s[7];
    out[0] = lo;
    out[1] = hi;
  }
}

void bucket_reduce_acc(torch::Tensor stage_peers, torch::Tensor table, torch::Tensor gshard, double scale,
                       int64_t world, int64_t rank, int64_t max_segment) {
  TORCH_CHECK(gshard.is_cuda() && gshard.scalar_type() == torch::kFloat32 && gshard.is_contiguous() &&
              reinterpret_cast<uintptr_t>(gshard.data_ptr()) % 16 == 0, "bucket_reduce_acc: fp32 gradient shard");
  VRL_CHECK_OPERAND(table, gshard, torch::kInt64);
  TORCH_CHECK(table.dim() == 2 && table.size(1) == 3 && table.is_contiguous() && table.size(0) >= 1 &&
              table.size(0) <= 65535, "bucket_reduce_acc: segment table [segments, 3] (src, dst, count)");
  TORCH_CHECK(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world && max_segment > 0);
  const c10::cuda::CUDAGuard guard(gshard.device());
  const PeerPtrs sp = load_peers(stage_peers, (int)world);
  const int bx = table_grid_x(table.size(0), max_segment);
  bucket_reduce_acc_kernel<<<dim3(bx, (unsigned)table.size(0)), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      sp, table.data_ptr<int64_t>(), gshard.data_ptr<float>(), (float)scale, (int)world, (int)rank);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

__global__ void __launch_bounds__(256)
p2p_gather_rows_kernel(PeerPtrs shards, uint4* __restrict__ full, int64_t vec_per_shard, int world, int rank) {
  for (int step = 0; step < world; ++step) {
    const int r = (rank + step) % world;
    const uint4* src = reinterpret_cast<const uint4*>(shards.p[r]);
    uint4* dst = full + (int64_t)r * vec_per_shard;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i + 3 * stride < vec_per_shard; i += 4 * stride) {
      const uint4 v0 = src[i], v1 = src[i + stride], v2 = src[i + 2 * stride], v3 = src[i + 3 * stride];
      dst[i] = v0; dst[i + stride] = v1; dst[i + 2 * stride] = v2; dst[i + 3 * stride] = v3;
    }
    for (; i < vec_per_shard; i += stride) dst[i] = src[i];
  }
}

// Table-driven all-gather of many row-sharded weights in one launch: segment j pulls `count`
// elements from offset src_off of EVERY rank's shard buffer into dst + dst_off + peer * count, so
// the destination holds the full [world * count] weight.  Used to fetch a whole block's weights
// ahead of the block's backward pass, on a side stream.
__global__ void __launch_bounds__(256)
p2p_gather_table_kernel(PeerPtrs shards, uint4* __restrict__ dst, const int64_t* __restrict__ table, int world,
                        int rank) {
  const int64_t src_vec = table[blockIdx.y * 3 + 0] / 8, dst_vec = table[blockIdx.y * 3 + 1] / 8;
  const int64_t nvec = table[blockIdx.y * 3 + 2] / 8;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int step = 0; step < world; ++step) {
    const int r = (rank + step) % world;
    const uint4* src = reinterpret_cast<const uint4*>(shards.p[r]) + src_vec;
    uint4* out = dst + dst_vec + (int64_t)r * nvec;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      const uint4 v0 = src[i], v1 = src[i + stride], v2 = src[i + 2 * stride], v3 = src[i + 3 * stride];
      out[i] = v0; out[i + stride] = v1; out[i + 2 * stride] = v2; out[i + 3 * stride] = v3;
    }
    for (; i < nvec; i += stride) out[i] = src[i];
  }
}

void p2p_gather_table(torch::Tensor shard_peers, torch::Tensor dst, torch::Tensor table, int64_t world,
                      int64_t rank, int64_t max_segment) {
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && dst.element_size() == 2 &&
              reinterpret_cast<uintptr_t>(dst.data_ptr()) % 16 == 0,
              "p2p_gather_table: contiguous 16-bit destination, 16-byte aligned");
  VRL_CHECK_OPERAND(table, dst, torch::kInt64);
  TORCH_CHECK(table.dim() == 2 && table.size(1) == 3 && table.is_contiguous() && table.size(0) >= 1 &&
              table.size(0) <= 65535, "p2p_gather_table: segment table [segments, 3] (src, dst, count), "
              "all multiples of 8 elements");
  TORCH_CHECK(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world && max_segment > 0);
  const c10::cuda::CUDAGuard guard(dst.device());
  const PeerPtrs sp = load_peers(shard_peers, (int)world);
  const int bx = table_grid_x(table.size(0), max_segment);
  p2p_gather_table_kernel<<<dim3(bx, (unsigned)table.size(0)), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      sp, reinterpret_cast<uint4*>(dst.data_ptr()), table.data_ptr<int64_t>(), (int)world, (int)rank);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void p2p_gather_rows(torch::Tensor shard_peers, torch::Tensor full, int64_t shard_elems, int64_t world,
                     int64_t rank) {
  TORCH_CHECK(full.is_cuda() && full.is_contiguous() && full.element_size() == 2 &&
              full.numel() == shard_elems * world && shard_elems % 8 == 0 &&
              reinterpret_cast<uintptr_t>(full.data_ptr()) % 16 == 0,
              "p2p_gather_rows: `full` must hold world * shard_elems 16-bit elements, 16-byte aligned");
  TORCH_CHECK(world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world);
  const c10::cuda::CUDAGuard guard(full.device());
  const PeerPtrs sp = load_peers(shard_peers, (int)world);
  for (int r = 0; r < world; ++r)
    TORCH_CHECK(reinterpret_cast<uintptr_t>(sp.p[r]) % 16 == 0, "p2p_gather_rows: shard addresses must be 16-byte aligned");
  const int64_t vec = shard_elems / 8;
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((vec + 1023) / 1024, 148 * 4));
  p2p_gather_rows_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      sp, reinterpret_cast<uint4*>(full.data_ptr()), vec, (int)world, (int)rank);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------------
// F3: Ulysses exchange as peer stores.
//   to_heads  : src [B, H, S_loc, D] (all heads, local sequence slice)
//               -> peer g's dst [B, H/P, S, D] at sequence offset rank * S_loc, for head group g
//   to_seq    : src [B, H/P, S, D] (local heads, full sequence)
//               -> peer r's dst [B, S_loc, H, D] (merged-head layout) at head offset rank * H/P
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
ulysses_to_heads_kernel(const uint4* __restrict__ src, PeerPtrs dst, int batch, int heads,
                        int s_loc, int vec_per_row, int world, int rank) {
  const int hp = heads / world;
  const int64_t total = (int64_t)batch * heads * s_loc * vec_per_row;
  const int64_t s_full = (int64_t)s_loc * world;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_row);
    int64_t t = i / vec_per_row;
    const int s = (int)(t % s_loc); t /= s_loc;
    const int h = (int)(t % heads);
    const int b = (int)(t / heads);
    const int peer = h / hp, hl = h % hp;
    const int64_t o = ((((int64_t)b * hp + hl) * s_full) + (int64_t)rank * s_loc + s) * vec_per_row + v;
    reinterpret_cast<uint4*>(dst.p[peer])[o] = src[i];
  }
}

__global__ void __launch_bounds__(256)
ulysses_to_seq_kernel(const uint4* __restrict__ src, PeerPtrs dst, int batch, int heads, int s_loc,
                      int vec_per_row, int world, int rank) {
  const int hp = heads / world;
  const int64_t s_full = (int64_t)s_loc * world;
  const int64_t total = (int64_t)batch * hp * s_full * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_row);
    int64_t t = i / vec_per_row;
    const int64_t s = t % s_full; t /= s_full;
    const int hl = (int)(t % hp);
    const int b = (int)(t / hp);
    const int peer = (int)(s / s_loc);
    const int sl = (int)(s % s_loc);
    const int64_t o = ((((int64_t)b * s_loc + sl) * heads) + (int64_t)rank * hp + hl) * vec_per_row + v;
    reinterpret_cast<uint4*>(dst.p[peer])[o] = src[i];
  }
}

// Token-major forms of the same exchange (what the backward pass of fused sequence-parallel attention
// needs: gradients arrive and leave token-major).  A "chunk" is one rank's heads of one token,
// C = (H / P) * D contiguous elements.
//   to_heads : src [B, S_loc, P, C]  -> peer g's dst [B, S, C]          at row rank * S_loc + s
//   to_seq   : src [B, S, C]         -> peer (s / S_loc)'s dst [B, S_loc, P, C] at chunk `rank`
__global__ void __launch_bounds__(256)
ulysses_tm_kernel(const uint4* __restrict__ src, PeerPtrs dst, int batch, int s_loc, int world, int rank,
                  int cvec, int to_heads) {
  const int64_t s_full = (int64_t)s_loc * world;
  const int64_t total = (int64_t)batch * s_full * cvec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % cvec);
    int64_t t = i / cvec;
    if (to_heads) {
      const int g = (int)(t % world); t /= world;
      const int s = (int)(t % s_loc);
      const int64_t b = t / s_loc;
      const int64_t o = ((b * s_full + (int64_t)rank * s_loc + s) * cvec) + v;
      reinterpret_cast<uint4*>(dst.p[g])[o] = src[i];
    } else {
      const int64_t s = t % s_full;
      const int64_t b = t / s_full;
      const int peer = (int)(s / s_loc);
      const int64_t sl = s - (int64_t)peer * s_loc;
      const int64_t o = (((b * s_loc + sl) * world + rank) * cvec) + v;
      reinterpret_cast<uint4*>(dst.p[peer])[o] = src[i];
    }
  }
}

void ulysses_exchange_tm(torch::Tensor src, torch::Tensor dst_peers, int64_t batch, int64_t s_loc,
                         int64_t chunk_elems, int64_t world, int64_t rank, bool to_heads) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && src.element_size() == 2 &&
              reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0, "ulysses_exchange_tm: contiguous 16-bit source");
  TORCH_CHECK(chunk_elems % 8 == 0 && world >= 1 && world <= kMaxPeers && rank >= 0 && rank < world);
  TORCH_CHECK(src.numel() == batch * s_loc * world * chunk_elems, "ulysses_exchange_tm: source size mismatch");
  const c10::cuda::CUDAGuard guard(src.device());
  const PeerPtrs dp = load_peers(dst_peers, (int)world);
  const int64_t total = src.numel() / 8;
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((total + 255) / 256, 148 * 8));
  ulysses_tm_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const uint4*>(src.data_ptr()), dp, (int)batch, (int)s_loc, (int)world, (int)rank,
      (int)(chunk_elems / 8), to_heads ? 1 : 0);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void ulysses_scatter(torch::Tensor src, torch::Tensor dst_peers, int64_t batch, int64_t heads,
                     int64_t s_loc, int64_t head_dim, int64_t world, int64_t rank, bool to_heads) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && src.element_size() == 2);
  TORCH_CHECK(head_dim % 8 == 0 && heads % world == 0);
  TORCH_CHECK(reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0);
  const c10::cuda::CUDAGuard guard(src.device());
  const PeerPtrs dp = load_peers(dst_peers, (int)world);
  const int vec = (int)(head_dim / 8);
  const int64_t total = src.numel() / 8;
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((total + 255) / 256, 148 * 8));
  auto stream = at::cuda::getCurrentCUDAStream();
  if (to_heads) {
    TORCH_CHECK(src.numel() == batch * heads * s_loc * head_dim);
    ulysses_to_heads_kernel<<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(src.data_ptr()), dp, (int)batch, (int)heads, (int)s_loc, vec,
        (int)world, (int)rank);
  } else {
    TORCH_CHECK(src.numel() == batch * (heads / world) * s_loc * world * head_dim);
    ulysses_to_seq_kernel<<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const uint4*>(src.data_ptr()), dp, (int)batch, (int)heads, (int)s_loc, vec,
        (int)world, (int)rank);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace vrl
