// Decoding GEMM whose K slices are summed inside a thread-block cluster (sm_100a).
//
//   out[rows, n] (bf16) = x[rows, k] * w[n, k]^T        rows <= 128
//
// computed as (w x^T)^T so that the weight rows fill the 128-row side of the tensor-core tile. A cluster of S CTAs
// (S = 2..8) owns one 128-row strip of w: CTA r streams k-blocks [r * per, (r + 1) * per) of the strip through a TMA
// ring into tcgen05.mma, leaves its fp32 partial tile [rows, 128] in its own shared memory, and after a cluster
// barrier every CTA sums 1/S of the output columns over all S partial tiles through distributed shared memory and
// stores them as bf16. No workspace, no second kernel: the form used when n / 128 strips times S CTAs fit on the
// device at once; wider weights keep the persistent split-K kernel of gemm_bf16.cu.
//
// Every mbarrier wait is bounded (common.cuh); the two cluster barriers are reached by every thread of every CTA
// whatever happened before them.
#include "common.cuh"

namespace ajb {
namespace gemm_decode {

constexpr int BM = 128;          // weight rows per strip (TMEM lanes)
constexpr int BN = 128;          // activation rows per tile (TMEM columns); rows beyond `rows` read zeros
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kStages = 5;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kPartialBytes = BN * BM * 4;                 // [column][row] fp32, overlays the ring after the main loop
constexpr int kSmemBytes = kStages * kStageBytes + 256;
constexpr int kKernelId = 11;
static_assert(kPartialBytes <= kStages * kStageBytes, "partial tile must fit into the ring");

struct Params {
  __nv_bfloat16* out;
  int rows, n, k;
  long long ldo;
  int kb_per_cta;            // k-blocks per CTA of a cluster
  DeviceStatus* status;
};

__device__ __forceinline__ float ld_shared_cluster_f32(uint32_t cluster_addr) {
  float v;
  // volatile keeps it behind the cluster barrier; no memory clobber, so the stores of a trip do not serialise the loads
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr));
  return v;
}
__device__ __forceinline__ uint32_t cluster_size_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(r));
  return r;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_decode_cluster_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* ring = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + kStages * kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t slices = cluster_size_x();
  const int strip = blockIdx.x / (int)slices;
  const int total_kb = (p.k + BK - 1) / BK;
  const int kb_begin = (int)rank * p.kb_per_cta;
  const int kb_end = min(total_kb, kb_begin + p.kb_per_cta);
  const int num_kb = max(0, kb_end - kb_begin);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_w);
    prefetch_tensor_map(&map_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, kKernelId, 1)) break;
        uint8_t* sa = ring + stage * kStageBytes;
        mbar_arrive_expect_tx(&full[stage], kStageBytes);
        tma_load_2d(sa, &map_w, &full[stage], kb * BK, strip * BM);
        tma_load_2d(sa + kABytes, &map_x, &full[stage], kb * BK, 0);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc(BM, BN, /*bf16*/ 1, false, false);
    const uint32_t a_lo0 = desc_lo_k_major(smem_u32(ring));
    const uint32_t b_lo0 = desc_lo_k_major(smem_u32(ring) + kABytes);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int kb = 0; kb < num_kb; ++kb) {
      if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kKernelId, 3)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t a_lo = a_lo0 + (uint32_t)stage * (uint32_t)(kStageBytes >> 4);
        const uint32_t b_lo = b_lo0 + (uint32_t)stage * (uint32_t)(kStageBytes >> 4);
        umma_f16(tmem_base, desc_at(a_lo, 0), desc_at(b_lo, 0), idesc, kb != 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 1; ks < BK / UMMA_K; ++ks)
          umma_f16_c<true>(tmem_base, desc_at(a_lo, (uint32_t)ks * UMMA_K * 2), desc_at(b_lo, (uint32_t)ks * UMMA_K * 2), idesc);
        tc_commit(&empty[stage]);
      }
      __syncwarp();
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }
    if (ok && lane == 0) tc_commit(acc_full);      // with no k-blocks this completes at once
    __syncwarp();
  } else {
    // ---- accumulator -> fp32 partial tile in shared memory, [column][row]: a warp's 32 rows are 128 contiguous bytes
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    float* partial = reinterpret_cast<float*>(ring);
    const bool have = num_kb > 0 && mbar_wait(acc_full, 0, abort_flag, p.status, kKernelId, 4);
    tc_fence_after_sync();
    // all products have completed, so every stage of the ring has been read and may be overwritten
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      if (c >= p.rows) break;
      uint32_t v[32];
      if (have) {
        tmem_ld_32x32(taddr + (uint32_t)c, v);
        tc_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) partial[(c + j) * BM + row] = __uint_as_float(v[j]);
    }
  }

  // ---- every CTA's partial tile is complete: sum 1/S of the columns over the cluster and store them
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp >= 2 && *abort_flag == 0) {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int out_col = strip * BM + row;                  // column of `out` = row of w
    const uint32_t mine = smem_u32(ring) + (uint32_t)row * 4u;
    uint32_t base[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) base[q] = q < (int)slices ? map_to_cta(mine, (uint32_t)q) : 0u;
    // eight columns per trip: up to 64 independent loads in flight per thread hide the shared-memory round trip
    for (int c0 = (int)rank; c0 < p.rows; c0 += 8 * (int)slices) {
      float part[8][8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int c = c0 + u * (int)slices;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          part[u][q] = (q < (int)slices && c < p.rows) ? ld_shared_cluster_f32(base[q] + (uint32_t)c * (uint32_t)(BM * 4)) : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int c = c0 + u * (int)slices;
        float acc = 0.0f;
#pragma unroll
        for (int q = 0; q < 8; ++q) acc += part[u][q];
        if (c < p.rows && out_col < p.n) p.out[(long long)c * p.ldo + out_col] = __float2bfloat16(acc);
      }
    }
  }
  // nobody leaves while a peer may still read its shared memory
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, BN);
  }
}

}  // namespace gemm_decode
}  // namespace ajb

namespace ajb {
namespace gemm_decode {

static void fill_config(cudaLaunchConfig_t& config, cudaLaunchAttribute* attr, int ctas, int slices, cudaStream_t stream) {
  config = cudaLaunchConfig_t{};
  config.gridDim = dim3((unsigned)ctas, 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)slices;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = 1;
}

static bool configure() {
  static int state = 0;     // 0: not tried, 1: ok, -1: failed
  if (state == 0) {
    state = cudaFuncSetAttribute(gemm_decode_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) == cudaSuccess ? 1 : -1;
    if (state < 0) cudaGetLastError();
  }
  return state > 0;
}

// Clusters of `slices` CTAs that the device holds at once (0 when the query fails).
static int resident_clusters(int slices) {
  static int cached[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (cached[slices] == 0) {
    cudaLaunchConfig_t config;
    cudaLaunchAttribute attr[1];
    fill_config(config, attr, slices * (sm_count() / slices), slices, nullptr);
    int clusters = 0;
    if (!configure() || cudaOccupancyMaxActiveClusters(&clusters, gemm_decode_cluster_kernel, &config) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = -1;
    }
    cached[slices] = clusters;
  }
  return cached[slices] > 0 ? cached[slices] : 0;
}

}  // namespace gemm_decode
}  // namespace ajb

// How many CTAs per 128-row strip of w[n, k] the cluster kernel should use: the largest count (8..2) for which all
// ceil(n / 128) clusters are resident at once and every CTA gets at least four 64-wide k-blocks; 0 = use the
// persistent split-K kernel instead.
extern "C" int ajb_gemm_decode_cluster_slices(int n, int k) {
  using namespace ajb::gemm_decode;
  const int strips = (n + BM - 1) / BM;
  const int k_blocks = (k + BK - 1) / BK;
  for (int slices = 8; slices >= 2; --slices)
    if (k_blocks / slices >= 4 && resident_clusters(slices) >= strips) return slices;
  return 0;
}

// out[rows, n] = x[rows, k] w[n, k]^T with `slices` (2..8) CTAs per 128-row strip of w; ceil(n / 128) * slices CTAs
// should fit on the device at once (the caller checks). Returns non-zero on a bad argument or a failed launch.
extern "C" int ajb_gemm_bf16_decode_cluster(const void* x, const void* w, void* out, int rows, int n, int k, long long ldx,
                                            long long ldw, long long ldo, int slices, void* stream) {
  using namespace ajb;
  using namespace ajb::gemm_decode;
  AJB_REQUIRE(rows > 0 && rows <= BN && n > 0 && k > 0, "decode gemm (cluster): bad problem %d x %d x %d", rows, n, k);
  AJB_REQUIRE(slices >= 2 && slices <= 8, "decode gemm (cluster): %d slices", slices);
  CUtensorMap map_w, map_x;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int rc = make_tensor_map_2d(&map_w, w, bf, 2, n, k, ldw * 2, BM, 64);
  if (rc) return rc;
  rc = make_tensor_map_2d(&map_x, x, bf, 2, rows, k, ldx * 2, BN, 64);
  if (rc) return rc;
  AJB_REQUIRE(configure(), "decode gemm (cluster): %d bytes of shared memory are not available", kSmemBytes);
  Params p;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.rows = rows; p.n = n; p.k = k; p.ldo = ldo;
  const int total_kb = (k + BK - 1) / BK;
  p.kb_per_cta = (total_kb + slices - 1) / slices;
  p.status = device_status_buffer();
  const int strips = (n + BM - 1) / BM;
  cudaLaunchConfig_t config;
  cudaLaunchAttribute attr[1];
  fill_config(config, attr, strips * slices, slices, reinterpret_cast<cudaStream_t>(stream));
  AJB_CUDA_OK(cudaLaunchKernelEx(&config, gemm_decode_cluster_kernel, map_w, map_x, p));
  return 0;
}
