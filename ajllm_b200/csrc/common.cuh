// Shared sm_100a primitives: error reporting, bounded mbarrier waits, TMA loads, tcgen05 MMA /
// TMEM management, shared-memory matrix descriptors.
//
// Every device-side wait in this library is bounded: a wait that exceeds its time budget records a
// status word in global memory, raises a CTA-wide abort flag and returns false, and the kernel then
// leaves through its normal teardown path (TMEM is released, nothing traps).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ajb {

// ---------------------------------------------------------------------------------------------
// Host-side error plumbing
// ---------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
const char* last_error();

#define AJB_CUDA_OK(expr)                                                                   \
  do {                                                                                      \
    cudaError_t err__ = (expr);                                                             \
    if (err__ != cudaSuccess) {                                                             \
      ajb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__), __FILE__,   \
                     __LINE__);                                                             \
      return 1;                                                                             \
    }                                                                                       \
  } while (0)

#define AJB_REQUIRE(cond, ...)              \
  do {                                      \
    if (!(cond)) {                          \
      ajb::set_error(__VA_ARGS__);          \
      return 2;                             \
    }                                       \
  } while (0)

// Device status words written by kernels whose bounded waits expired. Index = kernel id.
enum KernelId : int { kGemm = 0, kFlashFwd = 1, kFlashBwdKV = 2, kFlashBwdQ = 3, kCommGemm = 4, kFlashBwdFused = 8, kNumKernelIds = 16 };
struct DeviceStatus {
  unsigned int code;    // 0 = ok, otherwise (stage << 8) | kernel id + 1
  unsigned int block;
  unsigned int detail0;
  unsigned int detail1;
};
DeviceStatus* device_status_buffer();   // kNumKernelIds entries, zero-initialised, per device
int check_device_status_all();          // host: first non-zero status word of the current device (0 = none), cleared once read

// Encodes a 2-D bf16/fp8/fp32 row-major tensor [rows, cols] (row pitch in bytes) for TMA with a
// 128-byte swizzle. box_cols * elem_bytes must be <= 128.
int make_tensor_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                       uint64_t rows, uint64_t cols, uint64_t row_pitch_bytes, uint32_t box_rows,
                       uint32_t box_cols);
int make_tensor_map_3d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                       uint64_t d2, uint64_t rows, uint64_t cols, uint64_t d2_pitch_bytes,
                       uint64_t row_pitch_bytes, uint32_t box_rows, uint32_t box_cols);

int sm_count();            // SMs a kernel launched by this host thread may fill (the thread's budget, else all)
int sm_count_physical();   // SMs of the current device

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------------
// Device primitives
// ---------------------------------------------------------------------------------------------
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;  // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. `abort_flag` is a CTA-shared word; once any role sets it, every wait returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          DeviceStatus* status, int kernel_id, int stage) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((++spins & 0x3ff) == 0 && global_timer_ns() - t0 > kWaitBudgetNs) {
      *abort_flag = 1;
      if (status != nullptr && atomicCAS(&status[kernel_id].code, 0u, (unsigned)((stage << 8) | (kernel_id + 1))) == 0u) {
        status[kernel_id].block = blockIdx.x;
        status[kernel_id].detail0 = parity;
        status[kernel_id].detail1 = threadIdx.x;
      }
      return false;
    }
  }
}

// Swizzled operand tiles need a 1024-byte aligned base. The dynamic shared array is declared with that
// alignment; should the runtime ever place it elsewhere, the CTA reports it and leaves before touching
// any barrier or tensor memory. A CTA also leaves at once when an earlier CTA of the same kernel has
// already recorded an expired wait, so a protocol bug costs one time budget, not one per wave.
// `skip_word` is a word of the CTA's dynamic shared memory that nothing else uses.
__device__ __forceinline__ bool smem_misaligned(const void* base, DeviceStatus* status, int kernel_id,
                                                volatile uint32_t* skip_word) {
  if (threadIdx.x == 0) {
    const bool bad = (smem_u32(base) & 1023u) != 0;
    if (bad && status != nullptr &&
        atomicCAS(&status[kernel_id].code, 0u, (unsigned)((0xff << 8) | (kernel_id + 1))) == 0u) {
      status[kernel_id].block = blockIdx.x;
      status[kernel_id].detail0 = smem_u32(base);
    }
    const bool failed_before = status != nullptr && *reinterpret_cast<volatile unsigned int*>(&status[kernel_id].code) != 0u;
    *skip_word = (bad || failed_before) ? 1u : 0u;
  }
  __syncthreads();
  return *skip_word != 0u;
}

// TMA tile loads (no multicast anywhere in this library).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensor_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], bf16/fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand read from tensor memory (lane = row of A; 16-bit elements packed two per 32-bit column along K,
// even k in the low half), B from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same for e4m3/e5m2 inputs.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane (base lane + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// Vector reduction into global memory: four consecutive fp32 values (16-byte aligned address).
__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// ---- descriptors (128-byte swizzle everywhere)
// Instruction descriptor for kind::f16 / kind::f8f6f4 with fp32 accumulation.
//   ab_format: f16 kinds 0 = fp16, 1 = bf16; f8 kinds 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int ab_format, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (uint32_t(ab_format) << 7) | (uint32_t(ab_format) << 10) | (uint32_t(a_mn_major) << 15) |
         (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Shared-memory matrix descriptor. Byte offsets are encoded in 16-byte units.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3ffff) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= uint64_t(1) << 46;  // descriptor version for sm_100
  d |= uint64_t(2) << 61;  // SWIZZLE_128B
  return d;
}
// K-major operand tile: rows of 128 bytes (64 bf16 along K), 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t tile_addr, uint32_t k_byte_offset) {
  return make_smem_desc(tile_addr + k_byte_offset, 16, 1024);
}
// MN-major operand tile made of [k rows][64 elements along MN] boxes of `box_bytes` each
// (box_bytes = k rows * 128). `k_index` is the first k row of this MMA (multiple of 8).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t tile_addr, uint32_t box_bytes, uint32_t k_index) {
  return make_smem_desc(tile_addr + k_index * 128, box_bytes, 1024);
}

// ---- lean descriptor arithmetic for MMA issue loops
// One thread issues every tcgen05.mma of a CTA, and a 128 x 128 x 16 product takes only 64 cycles, so the
// issue loop has a budget of a handful of instructions per product. All tiles here share the upper
// descriptor word (1024-byte row groups, version 1, 128-byte swizzle); the lower word is the start
// address in 16-byte units plus the leading-dimension offset, so stepping through a tile is one add.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo_k_major(uint32_t tile_addr) {
  return ((tile_addr & 0x3ffff) >> 4) | (1u << 16);
}
__device__ __forceinline__ uint32_t desc_lo_mn_major(uint32_t tile_addr, uint32_t box_bytes) {
  return ((tile_addr & 0x3ffff) >> 4) | ((box_bytes >> 4) << 16);
}
__device__ __forceinline__ uint64_t desc_at(uint32_t lo, uint32_t byte_offset) {
  return (uint64_t(kDescHi) << 32) | (lo + (byte_offset >> 4));
}
// Byte offset of k-step `k` (16 elements) inside a K-major tile whose 64-element boxes are `box_bytes` apart.
__host__ __device__ constexpr uint32_t k_major_step(int k, uint32_t box_bytes) {
  return uint32_t(k / 4) * box_bytes + uint32_t(k % 4) * 32u;
}
// Byte offset of k-step `k` inside an MN-major tile (16 rows of 128 bytes per step).
__host__ __device__ constexpr uint32_t mn_major_step(int k) { return uint32_t(k) * 2048u; }

// Products with the accumulate flag fixed at compile time (no predicate set-up from a register).
template <bool kAccumulate>
__device__ __forceinline__ void umma_f16_c(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  if (kAccumulate)
    asm volatile("{\n.reg .pred p;\nsetp.eq.u32 p, 1, 1;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc) : "memory");
  else
    asm volatile("{\n.reg .pred p;\nsetp.eq.u32 p, 1, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc) : "memory");
}
template <bool kAccumulate>
__device__ __forceinline__ void umma_f16_ts_c(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc) {
  if (kAccumulate)
    asm volatile("{\n.reg .pred p;\nsetp.eq.u32 p, 1, 1;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
                 "r"(tmem_a), "l"(desc_b), "r"(idesc) : "memory");
  else
    asm volatile("{\n.reg .pred p;\nsetp.eq.u32 p, 1, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
                 "r"(tmem_a), "l"(desc_b), "r"(idesc) : "memory");
}

// ---- CTA pairs (clusters of two CTAs, tcgen05 cta_group::2): one thread of the even CTA issues products that read
// A and B from both CTAs' shared memory and accumulate 128 rows in each CTA's tensor memory.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t value) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(value) : "memory");
}
// Wait on a barrier of this CTA whose arrivals (and the data they publish) come from the other CTA of the cluster.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                  DeviceStatus* status, int kernel_id, int stage) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*abort_flag) return false;
    if ((++spins & 0x3ff) == 0 && global_timer_ns() - t0 > kWaitBudgetNs) {
      *abort_flag = 1;
      if (status != nullptr && atomicCAS(&status[kernel_id].code, 0u, (unsigned)((stage << 8) | (kernel_id + 1))) == 0u) {
        status[kernel_id].block = blockIdx.x;
        status[kernel_id].detail0 = parity;
        status[kernel_id].detail1 = threadIdx.x;
      }
      return false;
    }
  }
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load into this CTA's shared memory whose completion is reported to a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
// arrive on one barrier (shared::cluster address, either CTA) when the pair's earlier products are complete
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
template <bool kAccumulate>
__device__ __forceinline__ void umma_pair_f16_c(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  if (kAccumulate)
    asm volatile("{\n.reg .pred p;\nsetp.eq.u32 p, 1, 1;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc) : "memory");
  else
    asm volatile("{\n.reg .pred p;\nsetp.eq.u32 p, 1, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc) : "memory");
}
__device__ __forceinline__ void umma_pair_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}


__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 16 bytes of read-only global memory (written by an earlier launch) through the non-coherent path.
__device__ __forceinline__ uint4 ld_nc_v4(const uint4* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}

// ---- bulk copies (async proxy, no multicast)
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all_but_two() { asm volatile("cp.async.bulk.wait_group 2;" ::: "memory"); }
// SwiGLU in a GEMM epilogue. A thread holds 32 consecutive accumulator columns of one row.
// Forward: the columns are 16 (gate, up) pairs, already packed to bf16 in w[16]; 16 activations silu(gate) * up leave
// as two 16-byte stores to act (32-byte aligned row position).
__device__ __forceinline__ void swiglu_store_activation(const uint32_t (&w)[16], uint4* act) {
  float a[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float2 pair = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
    a[j] = pair.x / (1.0f + __expf(-pair.x)) * pair.y;
  }
  act[0] = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
  act[1] = make_uint4(pack_bf16x2(a[8], a[9]), pack_bf16x2(a[10], a[11]), pack_bf16x2(a[12], a[13]), pack_bf16x2(a[14], a[15]));
}
// Backward: the columns are 32 values of d_act (fp32 bits in v); g holds the 32 saved (gate, up) words of the same
// positions; 32 (d_gate, d_up) words leave as eight 16-byte stores.
__device__ __forceinline__ void swiglu_store_gradient(const uint32_t (&v)[32], const uint4 (&g)[8], uint4* out) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t w[4] = {g[j].x, g[j].y, g[j].z, g[j].w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 pair = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      const float d = __uint_as_float(v[4 * j + i]);
      const float sig = 1.0f / (1.0f + __expf(-pair.x));
      o[i] = pack_bf16x2(d * pair.y * sig * (1.0f + pair.x * (1.0f - sig)), d * pair.x * sig);
    }
    out[j] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// SwiGLU backward for one warp of an epilogue: 32 rows x `cols` columns of d_act in tensor memory (lane l owns row l)
// meet the saved (gate, up) words of the same positions, 32 columns = 128 bytes per row at a time. Global memory is
// read and written with whole 128-byte row segments (8 lanes per row, 4 rows per instruction); a padded block of
// shared memory turns them into the row-per-lane layout of the accumulators and back. `in` / `out` point at the
// first of the warp's rows, at the tile's first pair; rows at or past `rows_valid` are neither read nor written.
constexpr int kSwigluRowPitch = 144;                         // 128 bytes + 16: 16-byte accesses of 8 lanes cover all banks
constexpr int kSwigluWarpBytes = 32 * kSwigluRowPitch;
__device__ __forceinline__ void swiglu_backward_rows(uint32_t taddr, const __nv_bfloat16* in, long long ld_in,
                                                     __nv_bfloat16* out, long long ld_out, int rows_valid, int cols,
                                                     uint8_t* stage, int lane) {
  const int chunks = cols >> 5;
  const int sub = lane >> 3, piece = lane & 7;
  uint4 g[8];
  auto fetch = [&](int c) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = 4 * i + sub;
      if (r < rows_valid) g[i] = ld_nc_v4(reinterpret_cast<const uint4*>(in + (long long)r * ld_in + c * 64) + piece);
    }
  };
  if (chunks > 0) fetch(0);
  uint4* mine = reinterpret_cast<uint4*>(stage + lane * kSwigluRowPitch);
#pragma unroll 1
  for (int c = 0; c < chunks; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(taddr + (uint32_t)(c * 32), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4*>(stage + (4 * i + sub) * kSwigluRowPitch + piece * 16) = g[i];
    __syncwarp();
    if (c + 1 < chunks) fetch(c + 1);
    uint4 row[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) row[j] = mine[j];
    tc_wait_ld();
    swiglu_store_gradient(v, row, mine);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = 4 * i + sub;
      const uint4 q = *reinterpret_cast<const uint4*>(stage + r * kSwigluRowPitch + piece * 16);
      if (r < rows_valid) reinterpret_cast<uint4*>(out + (long long)r * ld_out + c * 64)[piece] = q;
    }
    __syncwarp();
  }
}

// Row-per-lane registers to whole row segments in memory, for one warp of an epilogue (same padded block of shared
// memory as above). w: 64 bf16 columns of lane l's row; they leave as 128 contiguous bytes per row, 8 lanes per row.
__device__ __forceinline__ void store_rows_128(const uint32_t (&w)[32], __nv_bfloat16* out, long long ld, int rows_valid,
                                               uint8_t* stage, int lane) {
  uint4* mine = reinterpret_cast<uint4*>(stage + lane * kSwigluRowPitch);
#pragma unroll
  for (int j = 0; j < 8; ++j) mine[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
  __syncwarp();
  const int sub = lane >> 3, piece = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = 4 * i + sub;
    const uint4 q = *reinterpret_cast<const uint4*>(stage + r * kSwigluRowPitch + piece * 16);
    if (r < rows_valid) reinterpret_cast<uint4*>(out + (long long)r * ld)[piece] = q;
  }
  __syncwarp();
}
// The same for 32 bf16 columns (64 bytes per row, 4 lanes per row).
__device__ __forceinline__ void store_rows_64(const uint32_t (&w)[16], __nv_bfloat16* out, long long ld, int rows_valid,
                                              uint8_t* stage, int lane) {
  uint4* mine = reinterpret_cast<uint4*>(stage + lane * kSwigluRowPitch);
#pragma unroll
  for (int j = 0; j < 4; ++j) mine[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
  __syncwarp();
  const int sub = lane >> 2, piece = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 8 * i + sub;
    const uint4 q = *reinterpret_cast<const uint4*>(stage + r * kSwigluRowPitch + piece * 16);
    if (r < rows_valid) reinterpret_cast<uint4*>(out + (long long)r * ld)[piece] = q;
  }
  __syncwarp();
}
#endif  // __CUDACC__

}  // namespace ajb
