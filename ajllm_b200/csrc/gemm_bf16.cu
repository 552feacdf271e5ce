// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory ring -> tcgen05.mma with
// fp32 accumulators in tensor memory -> tcgen05.ld epilogue.
//
//   C[M,N] (+)= op(A)[M,K] * op(B)[K,N]
//
// A is stored [M,K] (K contiguous) or, MN-major, [K,M] (M contiguous); B is stored [N,K] (K contiguous)
// or, MN-major, [K,N] (N contiguous). The three combinations used by a linear layer are
//   forward  y  = x W^T      : A K-major,  B K-major
//   dgrad    dx = dy W       : A K-major,  B MN-major
//   wgrad    dW = dy^T x     : A MN-major, B MN-major
// so no operand is ever transposed in memory.
//
// CTA = 6 warps: warp 0 issues TMA loads, warp 1 owns TMEM and issues the MMAs (one elected lane),
// warps 2..5 drain accumulators. Two 128x256 fp32 accumulators live in TMEM (512 columns) so the
// epilogue of tile i overlaps the main loop of tile i+1. Tiles are visited in groups of 16 row-blocks
// so that a wave of CTAs shares its A and B panels through L2.
#include "common.cuh"
#include "gemm_pair.h"

#include <cstdlib>

namespace ajb {

namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kGroupM = 16;

// kStoreBf16Swiglu / kSwigluBackward: as in gemm_bf16_pair.cu (activation from the (gate, up) product's epilogue; gradient
// of the pairs from the epilogue of d_out W2), here for the batched per-expert form as well.
enum Epilogue : int { kStoreBf16 = 0, kAccumF32 = 1, kStoreF32 = 2, kAtomicAddF32 = 3, kStoreBf16Swiglu = 4,
                      kSwigluBackward = 5 };

template <int BN>
struct Config {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;  // two accumulators
  static constexpr int kSmemBytes = kStages * kStageBytes + 256 /*barriers*/ + 4 * kSwigluWarpBytes /*a row block per epilogue warp*/;
};

struct Params {
  void* c;
  void* c2;                 // SwiGLU epilogues: the activation (written) or the saved (gate, up) pairs (read)
  long long ldc2, c2_batch_stride;
  int m, n, k;
  long long ldc;
  int epilogue;
  int tiles_m, tiles_n;
  // batched problems (one GEMM per expert): `batch` equal-shaped problems, outputs `c_batch_stride` elements apart.
  // Rows of a problem may be cut into segments of `segment_rows`; valid_rows[b * segments + s] says how many
  // leading rows of segment s hold data, and row blocks wholly past that count are skipped.
  int batch;
  long long c_batch_stride;
  const int* valid_rows;
  int segment_rows;
  // split-K (skinny problems): the K range is cut into `split_k` slices, slice s writes its partial product to
  // c + s * split_stride (fp32 store epilogue) and a small kernel sums the slices afterwards.
  int split_k;
  long long split_stride;
  // transposed store: element (row, col) of the product goes to c[col * ldc + row]. Decoding computes
  // (W x^T)^T this way: the weight rows fill the 128-row side of the tile whatever the batch size, and
  // the few activation rows are the narrow side.
  int transpose_c;
  DeviceStatus* status;
};

// Tile number -> (problem, row block, column block); returns false for a row block that holds no data.
__device__ __forceinline__ bool decode_tile(const Params& p, int tile, int& b, int& tm, int& tn);

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int group_span = kGroupM * tiles_n;
  const int group = tile / group_span;
  const int first_m = group * kGroupM;
  const int rows = min(kGroupM, tiles_m - first_m);
  const int within = tile - group * group_span;
  tm = first_m + within % rows;
  tn = within / rows;
}

template <bool BATCHED>
__device__ __forceinline__ void load_box(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int b) {
  if (BATCHED) tma_load_3d(dst, map, bar, c0, c1, b);
  else tma_load_2d(dst, map, bar, c0, c1);
}

__device__ __forceinline__ bool decode_tile(const Params& p, int tile, int& b, int& tm, int& tn) {
  const int per_problem = p.tiles_m * p.tiles_n;
  if (p.split_k > 1) {          // b carries the K slice
    b = tile / per_problem;
    tile_coords(tile - b * per_problem, p.tiles_m, p.tiles_n, tm, tn);
    return true;
  }
  b = tile / per_problem;
  tile_coords(tile - b * per_problem, p.tiles_m, p.tiles_n, tm, tn);
  if (p.valid_rows == nullptr) return true;
  const int m0 = tm * BM;
  const int seg = m0 / p.segment_rows;
  const int segments = (p.m + p.segment_rows - 1) / p.segment_rows;
  return m0 - seg * p.segment_rows < p.valid_rows[b * segments + seg];
}

template <int BN, bool A_MN, bool B_MN, bool BATCHED>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  using Cfg = Config<BN>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  if (smem_misaligned(smem, p.status, kGemm, reinterpret_cast<uint32_t*>(bars) + 60)) return;
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::kStages;
  uint64_t* acc_full = bars + 2 * Cfg::kStages;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n * p.batch * p.split_k;
  const int total_kb = (p.k + BK - 1) / BK;
  const int kb_per_split = (total_kb + p.split_k - 1) / p.split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_a);
    prefetch_tensor_map(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int b, tm, tn;
        if (!decode_tile(p, tile, b, tm, tn)) continue;
        const int m0 = tm * BM, n0 = tn * BN;
        const int kb_begin = p.split_k > 1 ? b * kb_per_split : 0;
        const int kb_end = p.split_k > 1 ? min(total_kb, kb_begin + kb_per_split) : total_kb;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, kGemm, 1)) { ok = false; break; }
          uint8_t* sa = stage_base + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_arrive_expect_tx(&full[stage], Cfg::kStageBytes);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) load_box<BATCHED>(sa + j * (BK * 128), &map_a, &full[stage], m0 + 64 * j, k0, p.split_k > 1 ? 0 : b);
          } else {
            load_box<BATCHED>(sa, &map_a, &full[stage], k0, m0, p.split_k > 1 ? 0 : b);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) load_box<BATCHED>(sb + j * (BK * 128), &map_b, &full[stage], n0 + 64 * j, k0, p.split_k > 1 ? 0 : b);
          } else {
            load_box<BATCHED>(sb, &map_b, &full[stage], k0, n0, p.split_k > 1 ? 0 : b);
          }
          ++issued;
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // drain: wait (bounded) for the copies this thread still has in flight before leaving
        const int pending = min(issued, Cfg::kStages);
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) { s = Cfg::kStages - 1; ph ^= 1; }
          const unsigned long long t0 = global_timer_ns();
          while (!mbar_try_wait(&full[s], ph) && global_timer_ns() - t0 < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc(BM, BN, /*bf16*/ 1, A_MN, B_MN);
    // The issuing thread has 128 cycles per product (N = 256): descriptor low words are formed once, a
    // stage is one multiply-add away and a k-step a compile-time offset (see common.cuh).
    const uint32_t a_lo0 = A_MN ? desc_lo_mn_major(smem_u32(stage_base), BK * 128) : desc_lo_k_major(smem_u32(stage_base));
    const uint32_t b_lo0 = B_MN ? desc_lo_mn_major(smem_u32(stage_base) + Cfg::kABytes, BK * 128)
                                : desc_lo_k_major(smem_u32(stage_base) + Cfg::kABytes);
    int stage = 0;
    uint32_t phase = 0;
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int num_kb = total_kb;
      {
        int b, tm, tn;
        if (!decode_tile(p, tile, b, tm, tn)) continue;
        if (p.split_k > 1) num_kb = min(total_kb, (b + 1) * kb_per_split) - b * kb_per_split;
      }
      const int buf = iter & 1;
      const uint32_t use = (uint32_t)(iter >> 1);
      ++iter;
      if (!mbar_wait(&acc_empty[buf], (use & 1) ^ 1, abort_flag, p.status, kGemm, 2)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kGemm, 3)) { ok = false; break; }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_lo = a_lo0 + (uint32_t)stage * (uint32_t)(Cfg::kStageBytes >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)stage * (uint32_t)(Cfg::kStageBytes >> 4);
          umma_f16(tmem_d, desc_at(a_lo, 0), desc_at(b_lo, 0), idesc, kb != 0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < BK / UMMA_K; ++k)
            umma_f16_c<true>(tmem_d, desc_at(a_lo, A_MN ? mn_major_step(k) : (uint32_t)k * UMMA_K * 2),
                             desc_at(b_lo, B_MN ? mn_major_step(k) : (uint32_t)k * UMMA_K * 2), idesc);
          tc_commit(&empty[stage]);  // frees the smem slot once these MMAs have read it
        }
        __syncwarp();
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
      if (ok && lane == 0) tc_commit(&acc_full[buf]);
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int b, tm, tn;
      if (!decode_tile(p, tile, b, tm, tn)) continue;
      const int buf = iter & 1;
      const uint32_t use = (uint32_t)(iter >> 1);
      ++iter;
      if (!mbar_wait(&acc_full[buf], use & 1, abort_flag, p.status, kGemm, 4)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = tm * BM + quarter * 32 + lane;
      const int col0 = tn * BN;
      const uint32_t taddr = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(quarter * 32) << 16);
      const bool row_ok = row < p.m;
      if (p.epilogue == kSwigluBackward) {
        // the accumulators are d_act; c2 holds the saved (gate, up) pairs, c receives their gradient (n % 32 == 0)
        const int row0 = row - lane;
        const long long at = 2 * col0;
        swiglu_backward_rows(taddr, reinterpret_cast<const __nv_bfloat16*>(p.c2) + b * p.c2_batch_stride + (long long)row0 * p.ldc2 + at,
                             p.ldc2, reinterpret_cast<__nv_bfloat16*>(p.c) + b * p.c_batch_stride + (long long)row0 * p.ldc + at, p.ldc,
                             min(32, p.m - row0), min(BN, p.n - col0),
                             smem + Cfg::kStages * Cfg::kStageBytes + 256 + quarter * kSwigluWarpBytes, lane);
      } else
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + (uint32_t)c, v);
        tc_wait_ld();
        const int col = col0 + c;
        if (!row_ok || col >= p.n) continue;
        const int valid = min(32, p.n - col);
        if (p.epilogue == kStoreBf16Swiglu) {
          // (gate, up) pairs in neighbouring columns (n % 32 == 0): the pairs go to c (when given), silu(gate) * up to c2
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) w[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
          if (p.c != nullptr) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.c) + b * p.c_batch_stride + (long long)row * p.ldc + col);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          }
          swiglu_store_activation(w, reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.c2) + b * p.c2_batch_stride +
                                                             (long long)row * p.ldc2 + (col >> 1)));
          continue;
        }
        if (p.transpose_c) {
          // consecutive lanes hold consecutive rows: each store instruction writes 32 neighbours of one output row
          const long long base = b * (p.split_k > 1 ? p.split_stride : p.c_batch_stride) + (long long)col * p.ldc + row;
          if (p.epilogue == kStoreBf16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + base;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) dst[(long long)j * p.ldc] = __float2bfloat16(__uint_as_float(v[j]));
          } else {
            float* dst = reinterpret_cast<float*>(p.c) + base;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) dst[(long long)j * p.ldc] = __uint_as_float(v[j]);
          }
          continue;
        }
        if (p.epilogue == kStoreBf16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + b * (p.split_k > 1 ? p.split_stride : p.c_batch_stride) + (long long)row * p.ldc + col;
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
          float* dst = reinterpret_cast<float*>(p.c) + b * (p.split_k > 1 ? p.split_stride : p.c_batch_stride) + (long long)row * p.ldc + col;
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
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

struct BatchSpec {
  int batch = 1;
  long long a_stride = 0, b_stride = 0, c_stride = 0;   // elements between consecutive problems
  void* c2 = nullptr;                                    // SwiGLU epilogues: second array, its row and problem strides
  long long ldc2 = 0, c2_stride = 0;
  const int* valid_rows = nullptr;
  int segment_rows = 0;
  int split_k = 1;
  long long split_stride = 0;
  int transpose_c = 0;
};

template <int BN, bool A_MN, bool B_MN, bool BATCHED>
static int launch(const void* a, const void* b, void* c, int m, int n, int k, long long lda, long long ldb,
                  long long ldc, int epilogue, const BatchSpec& spec, cudaStream_t stream) {
  using Cfg = Config<BN>;
  CUtensorMap map_a, map_b;
  int rc;
  const CUtensorMapDataType bf = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (BATCHED) {
    if (A_MN) rc = make_tensor_map_3d(&map_a, a, bf, 2, spec.batch, k, m, spec.a_stride * 2, lda * 2, BK, 64);
    else      rc = make_tensor_map_3d(&map_a, a, bf, 2, spec.batch, m, k, spec.a_stride * 2, lda * 2, BM, 64);
    if (rc) return rc;
    if (B_MN) rc = make_tensor_map_3d(&map_b, b, bf, 2, spec.batch, k, n, spec.b_stride * 2, ldb * 2, BK, 64);
    else      rc = make_tensor_map_3d(&map_b, b, bf, 2, spec.batch, n, k, spec.b_stride * 2, ldb * 2, BN, 64);
  } else {
    if (A_MN) rc = make_tensor_map_2d(&map_a, a, bf, 2, k, m, lda * 2, BK, 64);
    else      rc = make_tensor_map_2d(&map_a, a, bf, 2, m, k, lda * 2, BM, 64);
    if (rc) return rc;
    if (B_MN) rc = make_tensor_map_2d(&map_b, b, bf, 2, k, n, ldb * 2, BK, 64);
    else      rc = make_tensor_map_2d(&map_b, b, bf, 2, n, k, ldb * 2, BN, 64);
  }
  if (rc) return rc;

  static bool configured = false;
  auto kernel = gemm_kernel<BN, A_MN, B_MN, BATCHED>;
  if (!configured) {
    AJB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  Params p;
  p.c = c; p.m = m; p.n = n; p.k = k; p.ldc = ldc; p.epilogue = epilogue;
  p.c2 = spec.c2; p.ldc2 = spec.ldc2; p.c2_batch_stride = spec.c2_stride;
  p.tiles_m = (m + BM - 1) / BM;
  p.tiles_n = (n + BN - 1) / BN;
  p.batch = spec.batch;
  p.c_batch_stride = spec.c_stride;
  p.valid_rows = spec.valid_rows;
  p.segment_rows = spec.segment_rows > 0 ? spec.segment_rows : m;
  p.split_k = spec.split_k;
  p.split_stride = spec.split_stride;
  p.transpose_c = spec.transpose_c;
  p.status = device_status_buffer();
  const long long tiles = (long long)p.tiles_m * p.tiles_n * spec.batch * spec.split_k;
  const int grid = tiles < sm_count() ? (int)tiles : sm_count();
  kernel<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(map_a, map_b, p);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

template <bool BATCHED>
static int dispatch(const void* a, const void* b, void* c, int m, int n, int k, long long lda, long long ldb,
                    long long ldc, int a_mn_major, int b_mn_major, int epilogue, const BatchSpec& spec, cudaStream_t s) {
  // narrow outputs waste less of a 128-wide tile than of a 256-wide one
  const bool narrow = (n % 256 != 0) && ((n + 127) / 128 * 128 < (n + 255) / 256 * 256);
  const int sel = (a_mn_major ? 2 : 0) | (b_mn_major ? 1 : 0);
  if (narrow) {
    switch (sel) {
      case 0: return launch<128, false, false, BATCHED>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, spec, s);
      case 1: return launch<128, false, true, BATCHED>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, spec, s);
      case 2: return launch<128, true, false, BATCHED>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, spec, s);
      default: return launch<128, true, true, BATCHED>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, spec, s);
    }
  }
  switch (sel) {
    case 0: return launch<256, false, false, BATCHED>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, spec, s);
    case 1: return launch<256, false, true, BATCHED>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, spec, s);
    case 2: return launch<256, true, false, BATCHED>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, spec, s);
    default: return launch<256, true, true, BATCHED>(a, b, c, m, n, k, lda, ldb, ldc, epilogue, spec, s);
  }
}

// out[i] = sum_s partial[s * stride + i], fp32 -> bf16 (8 elements per thread)
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, long long vecs,
                                     long long stride, int splits) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < splits; ++s) {
      const float4 a = reinterpret_cast<const float4*>(partial + s * stride)[2 * i];
      const float4 b = reinterpret_cast<const float4*>(partial + s * stride)[2 * i + 1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint4 q;
    q.x = pack_bf16x2(acc[0], acc[1]);
    q.y = pack_bf16x2(acc[2], acc[3]);
    q.z = pack_bf16x2(acc[4], acc[5]);
    q.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = q;
  }
}

}  // namespace gemm
}  // namespace ajb

// C[m,n] (+)= op(A) op(B). lda/ldb/ldc are in elements. epilogue: 0 = bf16 store, 1 = fp32 accumulate,
// 2 = fp32 store.
extern "C" int ajb_gemm_bf16(const void* a, const void* b, void* c, int m, int n, int k, long long lda, long long ldb,
                             long long ldc, int a_mn_major, int b_mn_major, int epilogue, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(m > 0 && n > 0 && k > 0, "gemm: empty problem %dx%dx%d", m, n, k);
  AJB_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm: unknown epilogue %d", epilogue);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int sms = sm_count();
  const int k_blocks = (k + gemm::BK - 1) / gemm::BK;
  // Accumulating products with a long K (weight gradients: K = tokens) often have a tile count that fills the
  // SMs badly, e.g. 352 tiles on 148 SMs run as three rounds, the last one 40 % full. Cutting K into slices that
  // add into the same tile with reductions evens that out; with one slice this is the plain accumulate epilogue.
  auto pick_split = [&](int tiles, int units_per_round) {
    int best = 1;
    double best_eff = (double)tiles / (((tiles + units_per_round - 1) / units_per_round) * (double)units_per_round);
    if (epilogue != gemm::kAtomicAddF32) return best;
    for (int split = 2; split <= 4 && k_blocks / split >= 32; ++split) {
      const int units = tiles * split;
      const double eff = (double)units / (((units + units_per_round - 1) / units_per_round) * (double)units_per_round);
      if (eff > best_eff + 0.04) { best = split; best_eff = eff; }
    }
    return best;
  };
  const int tiles_single = ((m + gemm::BM - 1) / gemm::BM) * ((n + 255) / 256);
  const int split_single = pick_split(tiles_single, sms);

  // Two kernels: CTA pairs on 256 x 256 tiles (a third fewer operand bytes per CTA, about 1.1 x faster per tile)
  // and single CTAs on 128 x 256 or 128 x 128 tiles. Time is rounds x k-blocks per round; the pair kernel gets
  // the problem unless its coarser tiles cost more rounds than its per-tile advantage buys back.
  static const bool pairs_enabled = [] {
    const char* v = std::getenv("AJB_GEMM_PAIR");
    return v == nullptr || v[0] != '0';
  }();
  const bool narrow = (n % 256 != 0) && ((n + 127) / 128 * 128 < (n + 255) / 256 * 256);
  if (pairs_enabled && !narrow && m > gemm::BM) {
    const int pairs = gemm_pair::capacity();
    const int tiles_pair = ((m + 2 * gemm::BM - 1) / (2 * gemm::BM)) * ((n + 255) / 256);
    const int split_pair = pick_split(tiles_pair, pairs);
    const double rounds_single = (double)((tiles_single * split_single + sms - 1) / sms) / split_single;
    const double rounds_pair = (double)((tiles_pair * split_pair + pairs - 1) / pairs) / split_pair;
    if (rounds_pair * 0.93 <= rounds_single) {
      const int epi = (epilogue == gemm::kAtomicAddF32 && split_pair == 1) ? (int)gemm::kAccumF32 : epilogue;
      return gemm_pair::run(a, b, c, m, n, k, lda, ldb, ldc, a_mn_major, b_mn_major, epi, split_pair, s);
    }
  }
  gemm::BatchSpec spec;
  if (epilogue == gemm::kAtomicAddF32) {
    if (split_single == 1) epilogue = gemm::kAccumF32;
    else { spec.split_k = split_single; spec.split_stride = 0; }
  }
  return gemm::dispatch<false>(a, b, c, m, n, k, lda, ldb, ldc, a_mn_major, b_mn_major, epilogue, spec, s);
}

// `batch` equal-shaped problems (one per expert), operands / outputs `*_stride` elements apart. When valid_rows is
// given, the rows of each problem are cut into segments of `segment_rows` rows and valid_rows[problem * segments +
// segment] (device memory) tells how many leading rows of that segment hold data: row blocks past it are skipped,
// their outputs are left untouched.
extern "C" int ajb_gemm_bf16_batched(const void* a, const void* b, void* c, int batch, int m, int n, int k, long long lda,
                                     long long ldb, long long ldc, long long a_stride, long long b_stride,
                                     long long c_stride, int a_mn_major, int b_mn_major, int epilogue,
                                     const void* valid_rows, int segment_rows, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(batch > 0 && m > 0 && n > 0 && k > 0, "batched gemm: empty problem");
  AJB_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm: unknown epilogue %d", epilogue);
  AJB_REQUIRE(valid_rows == nullptr || (segment_rows > 0 && segment_rows % gemm::BM == 0),
              "batched gemm: segment_rows must be a positive multiple of %d", gemm::BM);
  gemm::BatchSpec spec;
  spec.batch = batch; spec.a_stride = a_stride; spec.b_stride = b_stride; spec.c_stride = c_stride;
  spec.valid_rows = (const int*)valid_rows; spec.segment_rows = segment_rows;
  return gemm::dispatch<true>(a, b, c, m, n, k, lda, ldb, ldc, a_mn_major, b_mn_major, epilogue, spec,
                              reinterpret_cast<cudaStream_t>(stream));
}

// Per-expert SwiGLU projections (`batch` problems, operands and outputs `*_stride` elements apart, valid_rows as in
// ajb_gemm_bf16_batched).
//   backward = 0: gate_up[b][m, n] = x[b][m, k] w13[b][n, k]^T with (gate, up) pairs in neighbouring columns (gate_up may be
//                 null) and other[b][m, n / 2] = silu(gate) * up from the same accumulators.
//   backward = 1: d_act[b][m, n] = d_out[b][m, k] w2[b][k, n] stays in tensor memory; the epilogue reads the saved
//                 gate_up[b][m, 2 n] and writes other[b][m, 2 n], the gradient of the pairs.
// n % 32 == 0; row strides multiples of 8; problem strides multiples of 8; bases 16-byte aligned.
extern "C" int ajb_gemm_bf16_batched_swiglu(const void* a, const void* b, void* gate_up, void* other, int batch, int m, int n,
                                            int k, long long lda, long long ldb, long long ld_gate_up, long long ld_other,
                                            long long a_stride, long long b_stride, long long gate_up_stride,
                                            long long other_stride, int backward, const void* valid_rows, int segment_rows,
                                            void* stream) {
  using namespace ajb;
  AJB_REQUIRE(batch > 0 && m > 0 && n > 0 && k > 0, "batched swiglu gemm: empty problem");
  AJB_REQUIRE(n % 32 == 0 && ld_gate_up % 8 == 0 && ld_other % 8 == 0 && gate_up_stride % 8 == 0 && other_stride % 8 == 0,
              "batched swiglu gemm: n must be a multiple of 32, strides multiples of 8");
  AJB_REQUIRE(other != nullptr && (backward == 0 || gate_up != nullptr), "batched swiglu gemm: missing operand");
  AJB_REQUIRE(((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(other)) & 15) == 0,
              "batched swiglu gemm: arrays must be 16-byte aligned");
  AJB_REQUIRE(valid_rows == nullptr || (segment_rows > 0 && segment_rows % gemm::BM == 0),
              "batched swiglu gemm: segment_rows must be a positive multiple of %d", gemm::BM);
  gemm::BatchSpec spec;
  spec.batch = batch; spec.a_stride = a_stride; spec.b_stride = b_stride;
  spec.valid_rows = (const int*)valid_rows; spec.segment_rows = segment_rows;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (backward) {
    spec.c_stride = other_stride; spec.c2 = gate_up; spec.ldc2 = ld_gate_up; spec.c2_stride = gate_up_stride;
    return gemm::dispatch<true>(a, b, other, m, n, k, lda, ldb, ld_other, 0, 1, gemm::kSwigluBackward, spec, s);
  }
  spec.c_stride = gate_up_stride; spec.c2 = other; spec.ldc2 = ld_other; spec.c2_stride = other_stride;
  return gemm::dispatch<true>(a, b, gate_up, m, n, k, lda, ldb, ld_gate_up, 0, 0, gemm::kStoreBf16Swiglu, spec, s);
}

// Skinny problems (few rows, e.g. decoding): C[m,n] bf16 = A[m,k] B[n,k]^T with the K range split over `split_k`
// CTAs per output tile so that all SMs stream the weights. workspace: split_k * m * n floats. c must be contiguous.
extern "C" int ajb_gemm_bf16_splitk(const void* a, const void* b, void* c, void* workspace, int m, int n, int k,
                                    long long lda, long long ldb, int split_k, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(m > 0 && n > 0 && k > 0 && split_k >= 1, "split-k gemm: bad problem");
  AJB_REQUIRE(n % 8 == 0, "split-k gemm: n must be a multiple of 8");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (split_k == 1)
    return gemm::dispatch<false>(a, b, c, m, n, k, lda, ldb, n, 0, 0, 0, gemm::BatchSpec(), s);
  gemm::BatchSpec spec;
  spec.split_k = split_k;
  spec.split_stride = (long long)m * n;
  int rc = gemm::dispatch<false>(a, b, workspace, m, n, k, lda, ldb, n, 0, 0, /*fp32 store*/ 2, spec, s);
  if (rc) return rc;
  const long long vecs = (long long)m * n / 8;
  const int blocks = (int)((vecs + 255) / 256 < (long long)sm_count() * 8 ? (vecs + 255) / 256 : (long long)sm_count() * 8);
  gemm::splitk_reduce_kernel<<<blocks, 256, 0, s>>>((const float*)workspace, (__nv_bfloat16*)c, vecs, (long long)m * n, split_k);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

// A few hundred rows (a decoding batch above 128 sequences, a short prompt chunk): out[m, n] bf16 = x[m, k] w[n, k]^T on
// CTA pairs, where every weight byte is fetched by exactly one CTA (each CTA of a pair stages half of the 256-wide
// weight tile and 128 of the rows). With few output tiles the K range is cut into slices so that one round of pairs
// covers the device; the slices add into a zeroed fp32 workspace that is small enough to stay in L2 and a small
// kernel rounds it to bf16. `split_k` = 0 lets ajb_gemm_skinny_pair_split choose. workspace: m * n floats (split_k > 1).
extern "C" int ajb_gemm_skinny_pair_split(int m, int n, int k) {
  using namespace ajb;
  const int pairs = gemm_pair::capacity();
  const int tiles = ((m + 255) / 256) * ((n + 255) / 256);
  const int k_blocks = (k + 63) / 64;
  // rough cost in units of a quarter microsecond: rounds x (k-blocks of a slice + start-up), plus what the slices'
  // reductions and the rounding kernel cost (bytes at about 4 TB/s)
  int best = 1;
  double best_cost = 1e30;
  for (int split = 1; split <= 16 && k_blocks / split >= 8; ++split) {
    if ((split - 1) * ((k_blocks + split - 1) / split) >= k_blocks) continue;      // the last slice would be empty
    const int items = tiles * split;
    const int rounds = (items + pairs - 1) / pairs;
    double cost = rounds * ((k_blocks + split - 1) / split + 3.0);
    if (split > 1) cost += 4.0 + (double)split * m * n * 4.0 / 1.0e6;
    if (cost < best_cost) { best_cost = cost; best = split; }
  }
  return best;
}

extern "C" int ajb_gemm_bf16_skinny_pair(const void* x, const void* w, void* out, void* workspace, int m, int n, int k,
                                         long long ldx, long long ldw, int split_k, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(m > 128 && n > 0 && k > 0 && n % 8 == 0, "skinny pair gemm: needs more than 128 rows and n %% 8 == 0");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (split_k <= 0) split_k = ajb_gemm_skinny_pair_split(m, n, k);
  if (split_k == 1) return gemm_pair::run(x, w, out, m, n, k, ldx, ldw, n, 0, 0, gemm::kStoreBf16, 1, s);
  const int k_blocks = (k + 63) / 64;
  AJB_REQUIRE(workspace != nullptr && (split_k - 1) * ((k_blocks + split_k - 1) / split_k) < k_blocks,
              "skinny pair gemm: K slices need a workspace and at least one k-block each");
  AJB_CUDA_OK(cudaMemsetAsync(workspace, 0, (size_t)m * n * sizeof(float), s));
  int rc = gemm_pair::run(x, w, workspace, m, n, k, ldx, ldw, n, 0, 0, gemm::kAtomicAddF32, split_k, s);
  if (rc) return rc;
  const long long vecs = (long long)m * n / 8;
  const int blocks = (int)((vecs + 255) / 256 < (long long)sm_count() * 8 ? (vecs + 255) / 256 : (long long)sm_count() * 8);
  gemm::splitk_reduce_kernel<<<blocks, 256, 0, s>>>((const float*)workspace, (__nv_bfloat16*)out, vecs, (long long)m * n, 1);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Decoding GEMM: out[rows, n] bf16 = x[rows, k] w[n, k]^T for rows <= 128, computed as (w x^T)^T: the tile's
// 128-row side is filled by weight rows, so there are n / 128 tiles times `split_k` K slices streaming the
// weights, and the partial products are rows x 128 instead of 128 x 256. workspace: split_k * rows * n floats.
extern "C" int ajb_gemm_bf16_decode(const void* x, const void* w, void* out, void* workspace, int rows, int n, int k,
                                    long long ldx, long long ldw, int split_k, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(rows > 0 && rows <= 128 && n > 0 && k > 0 && split_k >= 1, "decode gemm: bad problem");
  AJB_REQUIRE(n % 8 == 0, "decode gemm: n must be a multiple of 8");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  gemm::BatchSpec spec;
  spec.transpose_c = 1;
  if (split_k == 1) return gemm::dispatch<false>(w, x, out, n, rows, k, ldw, ldx, n, 0, 0, 0, spec, s);
  spec.split_k = split_k;
  spec.split_stride = (long long)rows * n;
  int rc = gemm::dispatch<false>(w, x, workspace, n, rows, k, ldw, ldx, n, 0, 0, /*fp32 store*/ 2, spec, s);
  if (rc) return rc;
  const long long vecs = (long long)rows * n / 8;
  const int blocks = (int)((vecs + 255) / 256 < (long long)sm_count() * 8 ? (vecs + 255) / 256 : (long long)sm_count() * 8);
  gemm::splitk_reduce_kernel<<<blocks, 256, 0, s>>>((const float*)workspace, (__nv_bfloat16*)out, vecs, (long long)rows * n, split_k);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}
