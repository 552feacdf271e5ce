// Block-scaled fp8 (e4m3) serving GEMM for sm_100a and the activation quantiser that feeds it.
//
//   C[M, N] (bf16) = sum over 128-wide K blocks kb of
//        ( Aq[M, kb] . Bq[N, kb]^T )  *  sa[M, kb]  *  sb[N / 128, kb]
//
// Aq: per-token activations, one fp32 scale per 1 x 128 slice. Bq: weights, one fp32 scale per
// 128 x 128 block. The scales are arbitrary fp32 values, so they cannot ride on the tensor core's own
// block scaling (which wants power-of-two scales per 32 elements); instead every K block is multiplied
// exactly in fp8 -> fp32 by tcgen05.mma kind::f8f6f4 into a fresh tensor-memory accumulator, and the
// epilogue warps fold it into per-thread fp32 running sums with the product of the two scales while the
// tensor core already works on the next K block (two partial accumulators in tensor memory).
// One CTA computes a 128 x 128 tile: one weight scale per K block, one activation scale per row.
//
// Decoding has few rows and therefore few tiles; a tile that walks the whole K on its own is a long serial chain
// on a mostly idle device. With `splits` > 1 the K blocks of a tile are divided over that many CTAs (grid z), each
// writes its fp32 partial tile to a workspace, and a second small kernel sums the parts in a fixed order and rounds
// to bf16.
#include <cuda_fp8.h>

#include "common.cuh"

namespace ajb {
namespace fp8 {

constexpr int BM = 128, BN = 128, BK = 128;   // BK fp8 elements = 128 bytes = one swizzle row
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kABytes = BM * BK, kBBytes = BN * BK, kStageBytes = kABytes + kBBytes;
constexpr int kSmem = kStages * kStageBytes + 256;
constexpr int kFp8KernelId = 6;

struct Params {
  __nv_bfloat16* c;
  const float* a_scale;   // [M, kblocks]
  const float* b_scale;   // [ceil(N / 128), kblocks]
  int m, n, k;
  long long ldc;
  int splits;        // CTAs per tile along K
  float* partial;    // splits > 1: [splits, m, n] fp32
  DeviceStatus* status;
};

__global__ void __launch_bounds__(kThreads, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  if (smem_misaligned(smem, p.status, kFp8KernelId, reinterpret_cast<uint32_t*>(bars) + 60)) return;
  uint64_t* full = bars;                  // kStages
  uint64_t* empty = bars + kStages;       // kStages
  uint64_t* part_full = empty + kStages;  // 2
  uint64_t* part_empty = part_full + 2;   // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tn = blockIdx.x, tm = blockIdx.y;
  const int num_kb = (p.k + BK - 1) / BK;          // K blocks of the whole problem (scale tables are indexed by these)
  const int per_split = (num_kb + p.splits - 1) / p.splits;
  const int kb_begin = min(num_kb, (int)blockIdx.z * per_split);
  const int kb_count = min(num_kb - kb_begin, per_split);      // this CTA's blocks: [kb_begin, kb_begin + kb_count)

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&part_full[b], 1);
      mbar_init(&part_empty[b], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_a);
    prefetch_tensor_map(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < kb_count; ++i) {
        const int s = i % kStages, kb = kb_begin + i;
        if (!mbar_wait(&empty[s], ((i / kStages) & 1) ^ 1, abort_flag, p.status, kFp8KernelId, 1)) break;
        uint8_t* sa = smem + s * kStageBytes;
        mbar_arrive_expect_tx(&full[s], kStageBytes);
        tma_load_2d(sa, &map_a, &full[s], kb * BK, tm * BM);
        tma_load_2d(sa + kABytes, &map_b, &full[s], kb * BK, tn * BN);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc(BM, BN, /*e4m3*/ 0, false, false);
    for (int kb = 0; kb < kb_count; ++kb) {          // local block index
      const int s = kb % kStages, buf = kb & 1;
      if (!mbar_wait(&part_empty[buf], (((uint32_t)kb >> 1) & 1) ^ 1, abort_flag, p.status, kFp8KernelId, 2)) break;
      if (!mbar_wait(&full[s], (kb / kStages) & 1, abort_flag, p.status, kFp8KernelId, 3)) break;
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t sa = smem_u32(smem + s * kStageBytes), sb = sa + kABytes;
#pragma unroll
        for (int k = 0; k < BK / 32; ++k)
          umma_f8(tmem_base + (uint32_t)(buf * BN), desc_k_major(sa, k * 32), desc_k_major(sb, k * 32), idesc, k != 0);
        tc_commit(&empty[s]);
        tc_commit(&part_full[buf]);
      }
      __syncwarp();
    }
  } else {
    const int quarter = warp & 3;
    const int row = tm * BM + quarter * 32 + lane;
    const bool row_ok = row < p.m;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float acc[BN];
#pragma unroll
    for (int i = 0; i < BN; ++i) acc[i] = 0.0f;
    bool ok = true;
    for (int i = 0; i < kb_count && ok; ++i) {
      const int buf = i & 1, kb = kb_begin + i;
      const float scale = (row_ok ? p.a_scale[(size_t)row * num_kb + kb] : 0.0f) * p.b_scale[(size_t)tn * num_kb + kb];
      if (!mbar_wait(&part_full[buf], ((uint32_t)i >> 1) & 1, abort_flag, p.status, kFp8KernelId, 4)) { ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(buf * BN + c * 32), v);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(v[i]), scale, acc[c * 32 + i]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&part_empty[buf]);
    }
    if (ok && row_ok && p.splits > 1) {
      // this part's fp32 sums (zeros when it had no K block); n is a multiple of 4 on this path
      const int col0 = tn * BN;
      float* dst = p.partial + ((size_t)blockIdx.z * p.m + row) * p.n + col0;
      const int valid = min(BN, p.n - col0);
#pragma unroll
      for (int j = 0; j < BN / 4; ++j)
        if (4 * j < valid) reinterpret_cast<float4*>(dst)[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
    } else if (ok && row_ok) {
      const int col0 = tn * BN;
      __nv_bfloat16* dst = p.c + (long long)row * p.ldc + col0;
      const int valid = min(BN, p.n - col0);
      if (valid == BN && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
          uint4 q;
          q.x = pack_bf16x2(acc[8 * j + 0], acc[8 * j + 1]);
          q.y = pack_bf16x2(acc[8 * j + 2], acc[8 * j + 3]);
          q.z = pack_bf16x2(acc[8 * j + 4], acc[8 * j + 5]);
          q.w = pack_bf16x2(acc[8 * j + 6], acc[8 * j + 7]);
          reinterpret_cast<uint4*>(dst)[j] = q;
        }
      } else {
#pragma unroll
        for (int j = 0; j < BN; ++j)
          if (j < valid) dst[j] = __float2bfloat16(acc[j]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// c[r, :] = bf16(sum over the parts of partial[part, r, :]), four columns per thread, parts in index order.
__global__ void sum_parts_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ c, int m, int n, long long ldc,
                                 int splits) {
  const long long vecs = (long long)m * (n >> 2);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < vecs; idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / (n >> 2);
    const int col = (int)(idx - row * (n >> 2)) * 4;
    float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int z = 0; z < splits; ++z) {
      const float4 v = *reinterpret_cast<const float4*>(partial + ((size_t)z * m + row) * n + col);
      total.x += v.x; total.y += v.y; total.z += v.z; total.w += v.w;
    }
    uint2 packed;
    packed.x = pack_bf16x2(total.x, total.y);
    packed.y = pack_bf16x2(total.z, total.w);
    *reinterpret_cast<uint2*>(c + row * ldc + col) = packed;
  }
}

// One warp per (row, 128-wide group): scale = amax / 448, q = x / scale.
__global__ void quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_storage_t* __restrict__ q,
                                     float* __restrict__ scales, int rows, int cols, int groups) {
  const long long warp_id = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_id >= (long long)rows * groups) return;
  const int row = (int)(warp_id / groups), g = (int)(warp_id % groups);
  const int col = g * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (col + 3 < cols) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)row * cols + col);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    for (int i = 0; i < 4; ++i)
      if (col + i < cols) v[i] = __bfloat162float(x[(size_t)row * cols + col + i]);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / 448.0f;
  const float inv = 1.0f / scale;
  if (lane == 0) scales[(size_t)row * groups + g] = scale;
  for (int i = 0; i < 4; ++i)
    if (col + i < cols)
      q[(size_t)row * cols + col + i] = __nv_cvt_float_to_fp8(v[i] * inv, __NV_SATFINITE, __NV_E4M3);
}

}  // namespace fp8
}  // namespace ajb

// x [rows, cols] bf16 -> q [rows, cols] e4m3, scales [rows, ceil(cols / 128)] fp32.
extern "C" int ajb_fp8_quantize_rows(const void* x, void* q, void* scales, int rows, int cols, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(cols % 4 == 0, "fp8 quantize: the feature dimension must be a multiple of 4");
  if (rows <= 0) return 0;
  const int groups = (cols + 127) / 128;
  const long long threads = (long long)rows * groups * 32;
  fp8::quantize_rows_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)x, (__nv_fp8_storage_t*)q, (float*)scales, rows, cols, groups);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

// How many K parts ajb_fp8_block_gemm would like for this problem (1 = none): enough CTAs to cover the device when
// the tiles alone do not, each part at least four K blocks long.
extern "C" int ajb_fp8_block_gemm_splits(int m, int n, int k) {
  using namespace ajb;
  const int tiles = ((n + fp8::BN - 1) / fp8::BN) * ((m + fp8::BM - 1) / fp8::BM);
  const int num_kb = (k + fp8::BK - 1) / fp8::BK;
  if (n % 4 != 0 || tiles >= sm_count()) return 1;
  int want = (sm_count() + tiles - 1) / tiles;
  if (want > num_kb / 4) want = num_kb / 4;
  return want < 1 ? 1 : want;
}

// a [m, k] e4m3 (row pitch lda bytes), b [n, k] e4m3 (row pitch ldb bytes), scales as described above.
// splits > 1 (see ajb_fp8_block_gemm_splits) needs `workspace` of splits * m * n floats.
extern "C" int ajb_fp8_block_gemm(const void* a, const void* b, const void* a_scale, const void* b_scale, void* c, int m,
                                  int n, int k, long long lda, long long ldb, long long ldc, int splits, void* workspace,
                                  void* stream) {
  using namespace ajb;
  AJB_REQUIRE(m > 0 && n > 0 && k > 0, "fp8 gemm: empty problem");
  AJB_REQUIRE(k % 16 == 0, "fp8 gemm: k must be a multiple of 16");
  AJB_REQUIRE(splits >= 1 && (splits == 1 || (workspace != nullptr && n % 4 == 0 && ldc % 4 == 0)),
              "fp8 gemm: K parts need a workspace and n, ldc multiples of 4");
  CUtensorMap map_a, map_b;
  int rc = make_tensor_map_2d(&map_a, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, m, k, lda, fp8::BM, fp8::BK);
  if (rc) return rc;
  rc = make_tensor_map_2d(&map_b, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, n, k, ldb, fp8::BN, fp8::BK);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    AJB_CUDA_OK(cudaFuncSetAttribute(fp8::fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fp8::kSmem));
    configured = true;
  }
  fp8::Params p;
  p.c = (__nv_bfloat16*)c; p.a_scale = (const float*)a_scale; p.b_scale = (const float*)b_scale;
  p.m = m; p.n = n; p.k = k; p.ldc = ldc; p.status = device_status_buffer();
  p.splits = splits; p.partial = (float*)workspace;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((n + fp8::BN - 1) / fp8::BN, (m + fp8::BM - 1) / fp8::BM, splits);
  fp8::fp8_gemm_kernel<<<grid, fp8::kThreads, fp8::kSmem, s>>>(map_a, map_b, p);
  AJB_CUDA_OK(cudaGetLastError());
  if (splits > 1) {
    const long long vecs = (long long)m * (n / 4);
    const long long blocks = (vecs + 255) / 256;
    fp8::sum_parts_kernel<<<(unsigned)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8), 256, 0, s>>>(
        (const float*)workspace, (__nv_bfloat16*)c, m, n, ldc, splits);
    AJB_CUDA_OK(cudaGetLastError());
  }
  return 0;
}
