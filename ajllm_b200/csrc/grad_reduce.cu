// Reduce-scatter of a unit's fp32 gradients over NVLink peer memory, fused with the accumulation into
// this rank's gradient shard and with the partial sums of squares that the global-norm clip needs.
//
// Every rank holds the unit's full gradient (written by the weight-gradient GEMM epilogues) in a
// symmetric buffer. One kernel per rank: announce "my buffer is complete" to the peers, wait for their
// announcements, then pull slice `rank` of every peer's buffer with 16-byte loads, add the slices in
// rank order (the same order on every rank, so the result does not depend on timing), add the sum to
// the shard (`dst += ...` over micro-batches) and leave one partial sum of squares per CTA of the
// updated shard. A closing handshake keeps every rank inside the kernel until all peers have finished
// reading its buffer, so whatever follows on the stream may overwrite it.
//
// Every wait on another GPU is bounded; on expiry the kernel records a status word and returns.
#include <string.h>

#include "common.cuh"

namespace ajb {
namespace gradrs {

constexpr int kThreads = 256;
constexpr int kMaxRanks = 8;
constexpr int kKernelId = 9;

struct Params {
  int world, rank;
  long long shard_vec4;                 // float4 elements per shard
  const float4* full_ptrs[kMaxRanks];   // each rank's symmetric full-gradient buffer (peer addresses)
  float4* dst;                          // this rank's shard accumulator
  int accumulate;                       // 1: dst += sum, 0: dst = sum
  float scale;
  float* sumsq_partials;                // gridDim.x floats or nullptr
  unsigned int* ready_ptrs[kMaxRanks];  // ready_ptrs[p][r]: rank r's buffer holds the gradients of this call
  unsigned int* done_ptrs[kMaxRanks];   // done_ptrs[p][r]: rank r has finished reading rank p's buffer
  unsigned int epoch;
  unsigned int* local_counter;          // zeroed by the host before the launch
  DeviceStatus* status;
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer(const float4* p) {
  float4 v;
  asm volatile("ld.global.relaxed.sys.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool wait_epoch(const unsigned int* p, unsigned int want, DeviceStatus* status, int stage) {
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    const unsigned int v = ld_acquire_sys(p);
    if ((int)(v - want) >= 0) return true;
    if ((++spins & 0xff) == 0 && global_timer_ns() - t0 > kWaitBudgetNs) {
      if (status != nullptr && atomicCAS(&status[kKernelId].code, 0u, (unsigned)((stage << 8) | (kKernelId + 1))) == 0u) {
        status[kKernelId].block = blockIdx.x;
        status[kKernelId].detail0 = want;
        status[kKernelId].detail1 = v;
      }
      return false;
    }
    __nanosleep(64);
  }
}

// U vectors per thread and trip (WMAX bounds the rank count): with `world` peers that is world * U independent 16-byte loads in flight per
// thread before the first add, which is what hides the NVLink round trip with only a few dozen CTAs.
template <int WMAX, int U>
__device__ __forceinline__ float reduce_slices(const Params& p) {
  float ss = 0.0f;
  const long long stride = (long long)gridDim.x * kThreads;
  for (long long i0 = (long long)blockIdx.x * kThreads + threadIdx.x; i0 < p.shard_vec4; i0 += stride * U) {
    float4 part[WMAX][U];
#pragma unroll
    for (int r = 0; r < WMAX; ++r)
      if (r < p.world) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          part[r][u] = i < p.shard_vec4 ? ld_peer(p.full_ptrs[r] + (long long)p.rank * p.shard_vec4 + i)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= p.shard_vec4) break;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < WMAX; ++r)
        if (r < p.world) { acc.x += part[r][u].x; acc.y += part[r][u].y; acc.z += part[r][u].z; acc.w += part[r][u].w; }
      float4 out = make_float4(acc.x * p.scale, acc.y * p.scale, acc.z * p.scale, acc.w * p.scale);
      if (p.accumulate) {
        const float4 old = p.dst[i];
        out.x += old.x; out.y += old.y; out.z += old.z; out.w += old.w;
      }
      p.dst[i] = out;
      ss += out.x * out.x + out.y * out.y + out.z * out.z + out.w * out.w;
    }
  }
  return ss;
}

__global__ void __launch_bounds__(kThreads) grad_reduce_scatter_kernel(const Params p) {
  __shared__ int s_ok;
  __shared__ float s_red[kThreads / 32];
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();     // the GEMM epilogues of earlier kernels on this stream wrote the buffer
      for (int r = 0; r < p.world; ++r) st_release_sys(p.ready_ptrs[r] + p.rank, p.epoch);
    }
    bool ok = true;
    for (int r = 0; r < p.world && ok; ++r) ok = wait_epoch(p.ready_ptrs[p.rank] + r, p.epoch, p.status, 1);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  float ss = 0.0f;
  if (s_ok) {
    if (p.world <= 2) ss = reduce_slices<2, 8>(p);
    else if (p.world <= 4) ss = reduce_slices<4, 4>(p);
    else ss = reduce_slices<kMaxRanks, 2>(p);
  }
  if (p.sumsq_partials != nullptr) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.0f;
      for (int w = 0; w < kThreads / 32; ++w) total += s_red[w];
      p.sumsq_partials[blockIdx.x] = total;
    }
  }
  __syncthreads();
  // closing handshake: the last CTA of this rank tells every peer that this rank no longer reads their
  // buffers, then waits for the same message from everyone
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.local_counter, 1u) == gridDim.x - 1) {
      for (int r = 0; r < p.world; ++r) st_release_sys(p.done_ptrs[r] + p.rank, p.epoch);
      for (int r = 0; r < p.world; ++r)
        if (!wait_epoch(p.done_ptrs[p.rank] + r, p.epoch, p.status, 2)) break;
    }
  }
}

}  // namespace gradrs
}  // namespace ajb

struct AjbGradReduceArgs {
  int world, rank;
  long long shard_elems;            // multiple of 4
  const void* full_ptrs[8];         // symmetric full-gradient buffers, world * shard_elems floats each
  void* dst;                        // [shard_elems] fp32
  int accumulate;
  float scale;
  void* sumsq_partials;             // [ctas] fp32 or nullptr
  int ctas;                         // grid size (<= SM count); also the length of sumsq_partials
  unsigned int* ready_ptrs[8];
  unsigned int* done_ptrs[8];
  unsigned int epoch;
  unsigned int* local_counter;      // one word of local scratch
};

extern "C" int ajb_grad_reduce_scatter(const AjbGradReduceArgs* args, void* stream) {
  using namespace ajb;
  using namespace ajb::gradrs;
  const AjbGradReduceArgs& a = *args;
  AJB_REQUIRE(a.world >= 1 && a.world <= kMaxRanks, "grad_reduce_scatter: world must be in [1, %d]", kMaxRanks);
  AJB_REQUIRE(a.shard_elems > 0 && a.shard_elems % 4 == 0, "grad_reduce_scatter: shard length must be a positive multiple of 4");
  AJB_REQUIRE(a.ctas >= 1 && a.ctas <= sm_count(), "grad_reduce_scatter: grid of %d CTAs does not fit the device at once", a.ctas);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  Params p;
  memset(&p, 0, sizeof(p));
  p.world = a.world; p.rank = a.rank; p.shard_vec4 = a.shard_elems / 4;
  for (int r = 0; r < a.world; ++r) {
    p.full_ptrs[r] = reinterpret_cast<const float4*>(a.full_ptrs[r]);
    p.ready_ptrs[r] = a.ready_ptrs[r];
    p.done_ptrs[r] = a.done_ptrs[r];
  }
  p.dst = reinterpret_cast<float4*>(a.dst);
  p.accumulate = a.accumulate; p.scale = a.scale;
  p.sumsq_partials = reinterpret_cast<float*>(a.sumsq_partials);
  p.epoch = a.epoch; p.local_counter = a.local_counter;
  p.status = device_status_buffer();
  AJB_CUDA_OK(cudaMemsetAsync(a.local_counter, 0, sizeof(unsigned int), s));
  // every CTA waits for the peers before it starts, and the last one waits again at the end: all CTAs of
  // the grid must be resident together, hence the bound by the SM count above
  grad_reduce_scatter_kernel<<<a.ctas, kThreads, 0, s>>>(p);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}
