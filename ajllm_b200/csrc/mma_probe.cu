// Tensor-pipe probe: how many cycles one tcgen05.mma (M = 128, K = 16, bf16) costs as a function of N, of
// where the A operand comes from (shared memory K-major / MN-major, tensor memory) and of the B layout,
// measured with a lean issue loop (descriptor low words precomputed, one add per operand per product).
// One CTA per SM, one issuing thread, operands zero-filled in shared memory; cycles are SM clocks
// (clock64) from the first issue to the completion of a final tcgen05.commit.
//
// The kernels of this library are sized with these numbers: an SS product with N = 128 keeps the pipe
// busy (64 cycles), N = 64 does not (about 51 cycles instead of 32: the operand fetch from shared memory
// is the limit), N = 256 and products with A in tensor memory leave shared-memory bandwidth to spare.
#include "common.cuh"

namespace ajb {
namespace probe {

// A_SRC: 0 shared K-major, 1 shared MN-major, 2 tensor memory. COMMIT_EVERY: a tcgen05.commit after every so many
// products (0: none). Everything that varies is a template parameter: a run-time test between two products
// already doubles the measured cost.
template <int N, int A_SRC, int B_MN, int COMMIT_EVERY>
__global__ void __launch_bounds__(192, 1) mma_probe_kernel(long long* out, int iters) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar, scratch_bar;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 192 * 1024 / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init(&scratch_bar, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 1 && lane == 0) {
    constexpr uint32_t idesc = make_idesc(128, N, 1, A_SRC == 1, B_MN != 0);
    const uint32_t a_lo0 = A_SRC == 1 ? desc_lo_mn_major(smem_u32(smem), 128 * 128) : desc_lo_k_major(smem_u32(smem));
    const uint32_t b_lo0 = B_MN ? desc_lo_mn_major(smem_u32(smem + 64 * 1024), 128 * 128) : desc_lo_k_major(smem_u32(smem + 64 * 1024));
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      const uint32_t a_lo = a_lo0 + (uint32_t)(it & 1) * (32768 >> 4);
      const uint32_t b_lo = b_lo0 + (uint32_t)(it & 1) * (49152 >> 4);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t a_off = A_SRC == 1 ? mn_major_step(k) : k_major_step(k, 128 * 128);
        const uint32_t b_off = B_MN ? mn_major_step(k) : k_major_step(k, N * 128);
        const uint32_t d = tmem_base + 256;
        if (A_SRC == 2) {
          if (k) umma_f16_ts_c<true>(d, tmem_base + (uint32_t)(k * 8), desc_at(b_lo, b_off), idesc);
          else umma_f16_ts_c<false>(d, tmem_base, desc_at(b_lo, b_off), idesc);
        } else {
          if (k) umma_f16_c<true>(d, desc_at(a_lo, a_off), desc_at(b_lo, b_off), idesc);
          else umma_f16_c<false>(d, desc_at(a_lo, a_off), desc_at(b_lo, b_off), idesc);
        }
        if (COMMIT_EVERY > 0 && (k + 1) % COMMIT_EVERY == 0) tc_commit(&scratch_bar);
      }
    }
    tc_commit(&bar);
    for (int spin = 0; spin < 20000000 && !mbar_try_wait(&bar, 0); ++spin) {}
    const long long t1 = clock64();
    if (blockIdx.x == 0) out[0] = t1 - t0;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int N, int A_SRC, int B_MN, int COMMIT_EVERY>
static int run(long long* out, int iters, cudaStream_t s) {
  constexpr int kSmem = 200 * 1024;
  AJB_CUDA_OK(cudaFuncSetAttribute(mma_probe_kernel<N, A_SRC, B_MN, COMMIT_EVERY>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  mma_probe_kernel<N, A_SRC, B_MN, COMMIT_EVERY><<<sm_count(), 192, kSmem, s>>>(out, iters);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int N>
static int run_n(int a_src, int b_mn, int commit_every, long long* out, int iters, cudaStream_t s) {
  if (commit_every == 4 && a_src == 0 && !b_mn) return run<N, 0, 0, 4>(out, iters, s);
  if (commit_every == 1 && a_src == 0 && !b_mn) return run<N, 0, 0, 1>(out, iters, s);
  if (commit_every != 0) {
    set_error("mma_probe: commits are measured with both operands K-major in shared memory, every 1 or 4 products");
    return 2;
  }
  if (a_src == 0) return b_mn ? run<N, 0, 1, 0>(out, iters, s) : run<N, 0, 0, 0>(out, iters, s);
  if (a_src == 1) return b_mn ? run<N, 1, 1, 0>(out, iters, s) : run<N, 1, 0, 0>(out, iters, s);
  return b_mn ? run<N, 2, 1, 0>(out, iters, s) : run<N, 2, 0, 0>(out, iters, s);
}

}  // namespace probe
}  // namespace ajb

// cycles_out: one int64 on the device, receives the SM cycles of `iters` * 8 products on CTA 0.
extern "C" int ajb_mma_probe(int n, int a_source, int b_mn_major, int commit_every, int iters, void* cycles_out, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(n == 64 || n == 128 || n == 256, "mma_probe: n must be 64, 128 or 256");
  AJB_REQUIRE(a_source >= 0 && a_source <= 2 && iters > 0 && iters <= 4096, "mma_probe: bad arguments");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  long long* out = reinterpret_cast<long long*>(cycles_out);
  if (n == 64) return probe::run_n<64>(a_source, b_mn_major, commit_every, out, iters, s);
  if (n == 128) return probe::run_n<128>(a_source, b_mn_major, commit_every, out, iters, s);
  return probe::run_n<256>(a_source, b_mn_major, commit_every, out, iters, s);
}
