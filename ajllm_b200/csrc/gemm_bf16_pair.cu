// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): two CTAs of a cluster, on neighbouring SMs, work on one
// 256 x 256 output tile.
//
//   C[M,N] (+)= op(A)[M,K] * op(B)[K,N]        (same operand layouts as gemm_bf16.cu)
//
// Each CTA of a pair loads 128 rows of A and HALF of the B tile (128 of its 256 columns) per k-block; one
// thread of the even CTA (the leader) issues tcgen05.mma.cta_group::2 with M = 256, N = 256, which reads A and
// B from both CTAs' shared memory and accumulates 128 rows x 256 columns in each CTA's tensor memory. Against
// the single-CTA kernel every CTA fetches one third fewer operand bytes from L2 and the tensor pipe reads one
// third fewer bytes from shared memory per product (32 KB instead of 48 KB per k-block and CTA), which is what
// counts on a part that runs dense GEMMs against its power limit; the smaller stages also make the ring six
// deep.
//
// Synchronisation (all waits bounded, see common.cuh):
//   full[s]      leader only. Armed by the leader's producer with the bytes of BOTH CTAs; both producers'
//                TMA loads complete on it (the peer's through the cta_group::2 form of the load).
//   empty[s]     one per CTA, signalled by tcgen05.commit from the leader's issuing thread (one commit per CTA).
//   acc_full[b]  one per CTA, same mechanism.
//   acc_empty[b] leader only, 8 arrivals: the four epilogue warps of each CTA (the peer's arrive remotely).
// Every CTA fetches its own bytes with its own TMA loads.
#include <cstdlib>

#include "common.cuh"
#include "gemm_pair.h"

namespace ajb {
namespace gemm_pair {

constexpr int BM = 128;          // rows per CTA; the pair covers 256
constexpr int BN = 256;          // columns of the pair's tile; each CTA stages 128 of them
constexpr int BNH = BN / 2;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kGroupM = 8;       // pair-tiles per column sweep (8 x 256 rows share their B panel through L2)
constexpr int kStages = 6;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BNH * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 2 * BN;
constexpr int kSmemBytes = kStages * kStageBytes + 256 + 4 * kSwigluWarpBytes;   // ring, barriers, a row block per epilogue warp
constexpr int kKernelId = 10;

// kStoreBf16Swiglu: C holds (gate, up) pairs in neighbouring columns; besides C (skipped when c is null) the epilogue
//   writes act[m, n / 2] = silu(gate) * up to c2, computed from the bf16-rounded pair.
// kSwigluBackward: the accumulators are d_act[m, n]; c2 is the saved gate_up[m, 2 n] and the epilogue writes
//   d_gate_up[m, 2 n] to c. d_act itself never reaches memory.
enum Epilogue : int { kStoreBf16 = 0, kAccumF32 = 1, kStoreF32 = 2, kAtomicAddF32 = 3, kStoreBf16Swiglu = 4,
                      kSwigluBackward = 5 };

struct Params {
  void* c;
  void* c2;
  long long ldc2;
  int row_stores;           // bf16 outputs leave as whole row segments through shared memory (AJB_GEMM_ROW_STORES=0: 16-byte pieces)
  int m, n, k;
  long long ldc;
  int epilogue;
  int tiles_m, tiles_n;     // in pair tiles (256 x 256)
  int split_k;              // K slices; slice s of a tile is work item s * tiles_m * tiles_n + tile (add epilogue only)
  DeviceStatus* status;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int group_span = kGroupM * tiles_n;
  const int group = tile / group_span;
  const int first_m = group * kGroupM;
  const int rows = min(kGroupM, tiles_m - first_m);
  const int within = tile - group * group_span;
  tm = first_m + within % rows;
  tn = within / rows;
}

// SWIGLU_BWD: the kernel of the kSwigluBackward epilogue (a row block per epilogue warp behind the barriers).
template <bool A_MN, bool B_MN, bool SWIGLU_BWD = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* stage_base = smem_raw;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + kStages * kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* acc_full = bars + 2 * kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint8_t* row_stage = smem_raw + kStages * kStageBytes + 256;          // 4 epilogue warps x kSwigluWarpBytes
  // both CTAs of a pair take the same branch here (same dynamic shared memory offset in both)
  const bool misaligned = smem_misaligned(smem_raw, p.status, kKernelId, reinterpret_cast<uint32_t*>(bars) + 60);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int per_slice = p.tiles_m * p.tiles_n;
  const int num_tiles = per_slice * p.split_k;
  const int total_kb = (p.k + BK - 1) / BK;
  const int kb_per_split = (total_kb + p.split_k - 1) / p.split_k;

  if (misaligned) return;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_a);
    prefetch_tensor_map(&map_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();            // the peer's barriers exist before anything is signalled across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      const uint32_t full_leader = map_to_cta(smem_u32(&full[0]), 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        const int slice = tile / per_slice;
        tile_coords(tile - slice * per_slice, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * (2 * BM) + (int)rank * BM;
        const int n0 = tn * BN + (int)rank * BNH;
        const int kb_begin = slice * kb_per_split;
        const int kb_end = min(total_kb, kb_begin + kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, kKernelId, 1)) { ok = false; break; }
          uint8_t* sa = stage_base + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          if (leader) mbar_arrive_expect_tx(&full[stage], 2 * kStageBytes);
          const uint32_t bar = full_leader + (uint32_t)stage * 8u;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * (BK * 128), &map_a, bar, m0 + 64 * j, k0);
          } else {
            tma_load_2d_pair(sa, &map_a, bar, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * (BK * 128), &map_b, bar, n0 + 64 * j, k0);
          } else {
            tma_load_2d_pair(sb, &map_b, bar, k0, n0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader) {
      constexpr uint32_t idesc = make_idesc(2 * BM, BN, /*bf16*/ 1, A_MN, B_MN);
      const uint32_t a_lo0 = A_MN ? desc_lo_mn_major(smem_u32(stage_base), BK * 128) : desc_lo_k_major(smem_u32(stage_base));
      const uint32_t b_lo0 = B_MN ? desc_lo_mn_major(smem_u32(stage_base) + kABytes, BK * 128)
                                  : desc_lo_k_major(smem_u32(stage_base) + kABytes);
      const uint32_t empty_mine = smem_u32(&empty[0]);
      const uint32_t empty_peer = map_to_cta(empty_mine, 1);
      const uint32_t acc_full_mine = smem_u32(&acc_full[0]);
      const uint32_t acc_full_peer = map_to_cta(acc_full_mine, 1);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int buf = iter & 1;
        const uint32_t use = (uint32_t)(iter >> 1);
        ++iter;
        if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, abort_flag, p.status, kKernelId, 2)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        const int slice = tile / per_slice;
        const int num_kb = min(total_kb, (slice + 1) * kb_per_split) - slice * kb_per_split;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kKernelId, 3)) { ok = false; break; }
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t a_lo = a_lo0 + (uint32_t)stage * (uint32_t)(kStageBytes >> 4);
            const uint32_t b_lo = b_lo0 + (uint32_t)stage * (uint32_t)(kStageBytes >> 4);
            umma_pair_f16(tmem_d, desc_at(a_lo, 0), desc_at(b_lo, 0), idesc, kb != 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < BK / UMMA_K; ++k)
              umma_pair_f16_c<true>(tmem_d, desc_at(a_lo, A_MN ? mn_major_step(k) : (uint32_t)k * UMMA_K * 2),
                                    desc_at(b_lo, B_MN ? mn_major_step(k) : (uint32_t)k * UMMA_K * 2), idesc);
            // the slot is free in both CTAs once these products have read it
            tc_commit_pair(empty_mine + (uint32_t)stage * 8u);
            tc_commit_pair(empty_peer + (uint32_t)stage * 8u);
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok && lane == 0) {
          tc_commit_pair(acc_full_mine + (uint32_t)buf * 8u);
          tc_commit_pair(acc_full_peer + (uint32_t)buf * 8u);
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    const uint32_t acc_empty_leader = map_to_cta(smem_u32(&acc_empty[0]), 0);
    int iter = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int tm, tn;
      tile_coords(tile % per_slice, p.tiles_m, p.tiles_n, tm, tn);
      const int buf = iter & 1;
      const uint32_t use = (uint32_t)(iter >> 1);
      ++iter;
      if (!mbar_wait(&acc_full[buf], use & 1, abort_flag, p.status, kKernelId, 4)) break;
      tc_fence_after_sync();
      const int row = tm * (2 * BM) + (int)rank * BM + quarter * 32 + lane;
      const int col0 = tn * BN;
      const uint32_t taddr = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(quarter * 32) << 16);
      const bool row_ok = row < p.m;
      // bf16 outputs whose rows start on 16-byte boundaries go out as whole row segments
      const bool bf16_rows = p.row_stores && (p.epilogue == kStoreBf16 || p.epilogue == kStoreBf16Swiglu) && (p.ldc & 7) == 0 &&
                             (reinterpret_cast<uintptr_t>(p.c) & 15) == 0;
      if (SWIGLU_BWD) {
        // the accumulators are d_act: turned into the gradient of the saved (gate, up) pairs, 32 columns at a time
        // (n is a multiple of 32: a chunk is whole or absent)
        const int row0 = row - lane;
        const long long at = 2 * col0;
        swiglu_backward_rows(taddr, reinterpret_cast<const __nv_bfloat16*>(p.c2) + (long long)row0 * p.ldc2 + at, p.ldc2,
                             reinterpret_cast<__nv_bfloat16*>(p.c) + (long long)row0 * p.ldc + at, p.ldc,
                             min(32, p.m - row0), min(BN, p.n - col0), row_stage + quarter * kSwigluWarpBytes, lane);
      } else
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        const int col = col0 + c;
        if (bf16_rows && (c & 63) == 0 && col + 64 <= p.n) {
          // 64 whole columns: bf16 rows leave as 128-byte segments through the warp's row block
          const int row0 = row - lane;
          uint32_t w[32];
          {
            uint32_t v[32];
            tmem_ld_32x32(taddr + (uint32_t)c, v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
            tmem_ld_32x32(taddr + (uint32_t)(c + 32), v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) w[16 + j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          }
          uint8_t* stage = row_stage + quarter * kSwigluWarpBytes;
          if (p.c != nullptr)
            store_rows_128(w, reinterpret_cast<__nv_bfloat16*>(p.c) + (long long)row0 * p.ldc + col, p.ldc, p.m - row0, stage, lane);
          if (p.epilogue == kStoreBf16Swiglu) {
            uint32_t a[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float2 p0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[2 * j]));
              const float2 p1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[2 * j + 1]));
              a[j] = pack_bf16x2(p0.x / (1.0f + __expf(-p0.x)) * p0.y, p1.x / (1.0f + __expf(-p1.x)) * p1.y);
            }
            store_rows_64(a, reinterpret_cast<__nv_bfloat16*>(p.c2) + (long long)row0 * p.ldc2 + (col >> 1), p.ldc2,
                          p.m - row0, stage, lane);
          }
          c += 32;
          continue;
        }
        uint32_t v[32];
        tmem_ld_32x32(taddr + (uint32_t)c, v);
        tc_wait_ld();
        if (!row_ok || col >= p.n) continue;
        const int valid = min(32, p.n - col);
        if (p.epilogue == kStoreBf16Swiglu) {
          // n is a multiple of 32 here
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) w[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          if (p.c != nullptr) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.c) + (long long)row * p.ldc + col);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          }
          swiglu_store_activation(w, reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.c2) +
                                                             (long long)row * p.ldc2 + (col >> 1)));
        } else if (p.epilogue == kStoreBf16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + (long long)row * p.ldc + col;
          if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 q;
              q.x = pack_bf16x2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
              q.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
              q.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
              q.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
              reinterpret_cast<uint4*>(dst)[j] = q;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) dst[j] = __float2bfloat16(__uint_as_float(v[j]));
          }
        } else {
          float* dst = reinterpret_cast<float*>(p.c) + (long long)row * p.ldc + col;
          const bool accumulate = p.epilogue == kAccumF32;
          if (p.epilogue == kAtomicAddF32) {
            // several K slices add into the same tile: 16-byte reductions, order not fixed
            if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                red_add_f32x4(dst + 4 * j, __uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                              __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < valid) atomicAdd(dst + j, __uint_as_float(v[j]));
            }
          } else if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 q = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                     __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
              if (accumulate) {
                const float4 old = reinterpret_cast<float4*>(dst)[j];
                q.x += old.x; q.y += old.y; q.z += old.z; q.w += old.w;
              }
              reinterpret_cast<float4*>(dst)[j] = q;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) dst[j] = (accumulate ? dst[j] : 0.0f) + __uint_as_float(v[j]);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_leader + (uint32_t)buf * 8u);
    }
  }

  // neither CTA may leave (or free tensor memory) while the other still reads its shared memory or writes its
  // accumulators: every role of both CTAs has finished, or given up after its bounded wait, before this point
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// How many pairs can be resident at once (a pair needs two free SMs of one cluster-capable group).
template <typename Kernel>
static int resident_pairs(Kernel kernel) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)sm_count_physical() / 2 * 2, 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters <= 0) {
    cudaGetLastError();
    clusters = sm_count_physical() / 2;
  }
  return clusters < sm_count_physical() / 2 ? clusters : sm_count_physical() / 2;
}

template <bool A_MN, bool B_MN, bool SWIGLU_BWD = false>
static int launch(const void* a, const void* b, void* c, int m, int n, int k, long long lda, long long ldb, long long ldc,
                  int epilogue, int split_k, cudaStream_t stream, void* c2 = nullptr, long long ldc2 = 0) {
  CUtensorMap map_a, map_b;
  int rc;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (A_MN) rc = make_tensor_map_2d(&map_a, a, bf, 2, k, m, lda * 2, BK, 64);
  else      rc = make_tensor_map_2d(&map_a, a, bf, 2, m, k, lda * 2, BM, 64);
  if (rc) return rc;
  if (B_MN) rc = make_tensor_map_2d(&map_b, b, bf, 2, k, n, ldb * 2, BK, 64);
  else      rc = make_tensor_map_2d(&map_b, b, bf, 2, n, k, ldb * 2, BNH, 64);
  if (rc) return rc;

  static bool configured = false;
  auto kernel = gemm_pair_kernel<A_MN, B_MN, SWIGLU_BWD>;
  if (!configured) {
    AJB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured = true;
  }
  const int pairs = capacity();
  Params p;
  static const bool row_stores = [] {
    const char* v = std::getenv("AJB_GEMM_ROW_STORES");
    return v == nullptr || v[0] != '0';
  }();
  p.row_stores = row_stores ? 1 : 0;
  p.c = c; p.c2 = c2; p.ldc2 = ldc2; p.m = m; p.n = n; p.k = k; p.ldc = ldc; p.epilogue = epilogue;
  p.tiles_m = (m + 2 * BM - 1) / (2 * BM);
  p.tiles_n = (n + BN - 1) / BN;
  p.split_k = split_k;
  p.status = device_status_buffer();
  const long long tiles = (long long)p.tiles_m * p.tiles_n * split_k;
  const int grid = 2 * (int)(tiles < pairs ? tiles : pairs);
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

int capacity() {
  static int pairs = 0;
  if (pairs == 0) {
    auto kernel = gemm_pair_kernel<false, false>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
      cudaGetLastError();
      return sm_count() / 2;
    }
    pairs = resident_pairs(kernel);
  }
  // under an SM budget (see sm_count) only that many SMs' worth of pairs are launched
  return pairs < sm_count() / 2 ? pairs : sm_count() / 2;
}

int run(const void* a, const void* b, void* c, int m, int n, int k, long long lda, long long ldb, long long ldc,
        int a_mn_major, int b_mn_major, int epilogue, int split_k, cudaStream_t s) {
  const int sel = (a_mn_major ? 2 : 0) | (b_mn_major ? 1 : 0);
  switch (sel) {
    case 0: return launch<false, false>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, split_k, s);
    case 1: return launch<false, true>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, split_k, s);
    case 2: return launch<true, false>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, split_k, s);
    default: return launch<true, true>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, split_k, s);
  }
}

int run_swiglu(const void* a, const void* b, void* c, void* c2, int m, int n, int k, long long lda, long long ldb,
               long long ldc, long long ldc2, int backward, cudaStream_t s) {
  if (backward) return launch<false, true, true>(a, b, c, m, n, k, lda, ldb, ldc, kSwigluBackward, 1, s, c2, ldc2);
  return launch<false, false>(a, b, c, m, n, k, lda, ldb, ldc, kStoreBf16Swiglu, 1, s, c2, ldc2);
}

}  // namespace gemm_pair
}  // namespace ajb

// SwiGLU inside the projections around it, on CTA pairs (the reference applies it as three eager ops between the
// matmuls, ajllm/modeling/activations.py:25).
//   forward  (backward = 0): gate_up[m, n] = x[m, k] w13[n, k]^T with (gate, up) pairs in neighbouring columns, and
//            act[m, n / 2] = silu(gate) * up from the same accumulators. gate_up may be null (inference): only act is
//            written.
//   backward (backward = 1): d_act[m, n] = d_out[m, k] w2[k, n] stays in tensor memory; the epilogue reads the saved
//            gate_up[m, 2 n] and writes d_gate_up[m, 2 n].
// n must be a multiple of 32, all row strides multiples of 8 elements, all bases 16-byte aligned.
extern "C" int ajb_gemm_bf16_swiglu(const void* a, const void* b, void* gate_up, void* other, int m, int n, int k,
                                    long long lda, long long ldb, long long ld_gate_up, long long ld_other, int backward,
                                    void* stream) {
  using namespace ajb;
  AJB_REQUIRE(m > 0 && n > 0 && k > 0, "gemm_swiglu: empty problem %dx%dx%d", m, n, k);
  AJB_REQUIRE(n % 32 == 0, "gemm_swiglu: n = %d must be a multiple of 32", n);
  AJB_REQUIRE(ld_gate_up % 8 == 0 && ld_other % 8 == 0, "gemm_swiglu: row strides must be multiples of 8 elements");
  AJB_REQUIRE(other != nullptr && (backward == 0 || gate_up != nullptr), "gemm_swiglu: missing operand");
  AJB_REQUIRE(((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(other)) & 15) == 0,
              "gemm_swiglu: outputs must be 16-byte aligned");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // forward: C = gate_up, c2 = act; backward: C = d_gate_up (`other`), c2 = the saved gate_up
  if (backward) return gemm_pair::run_swiglu(a, b, other, gate_up, m, n, k, lda, ldb, ld_other, ld_gate_up, 1, s);
  return gemm_pair::run_swiglu(a, b, gate_up, other, m, n, k, lda, ldb, ld_gate_up, ld_other, 0, s);
}

// The pair kernel on its own (tests and benchmarks; ajb_gemm_bf16 chooses between the two kernels itself).
// Epilogues 0 (bf16 store), 1 (fp32 accumulate), 2 (fp32 store); 3 (fp32 add with reductions) takes `split_k` K slices.
extern "C" int ajb_gemm_bf16_pair(const void* a, const void* b, void* c, int m, int n, int k, long long lda, long long ldb,
                                  long long ldc, int a_mn_major, int b_mn_major, int epilogue, int split_k, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(m > 0 && n > 0 && k > 0, "gemm_pair: empty problem %dx%dx%d", m, n, k);
  AJB_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm_pair: unknown epilogue %d", epilogue);
  AJB_REQUIRE(split_k >= 1 && (split_k == 1 || epilogue == 3), "gemm_pair: K slices need the add epilogue");
  AJB_REQUIRE((k + gemm_pair::BK - 1) / gemm_pair::BK >= split_k, "gemm_pair: more K slices than k-blocks");
  return gemm_pair::run(a, b, c, m, n, k, lda, ldb, ldc, a_mn_major, b_mn_major, epilogue, split_k,
                        reinterpret_cast<cudaStream_t>(stream));
}

// Resident CTA pairs on the current device (what the dispatcher plans its rounds with).
extern "C" int ajb_gemm_pair_capacity() { return ajb::gemm_pair::capacity(); }
