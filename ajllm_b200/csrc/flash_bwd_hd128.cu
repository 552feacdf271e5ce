// FlashAttention backward for head_dim 128 on sm_100a: one kernel, five tensor-core products per
// (128 keys x 64 queries) step, every accumulator resident in tensor memory at once.
//
// One CTA owns one (KV tile of 128 keys, KV head, batch) and walks over the query heads of its group
// and their 64-row query tiles:
//
//   S^T   = K Q^T      [128 x 64]   TMEM cols 256..319   (P^T, bf16, is written back over the first half
//                                                          of the columns each softmax group has read)
//   dP^T  = V dO^T     [128 x 64]   TMEM cols 320..383
//   dV   += P^T dO     [128 x 128]  TMEM cols 128..255   (A operand read from tensor memory)
//   dK   += dS^T Q     [128 x 128]  TMEM cols   0..127   (dS^T staged in shared memory, double buffered)
//   dQ^T  = K^T dS     [128 x 64]   TMEM cols 384..447   (lane = head-dim element, column = query)
//
// With 64-query steps nothing in tensor memory has to be aliased across products, Q/dO tiles are
// 16 KB each (three stages in flight), and the dQ^T tile of a step is small enough to be staged in
// shared memory: four drain warps copy it out of tensor memory, transpose it into [query][32
// head-dim elements] blocks and hand each 8 KB block to the TMA unit as one bulk reduce-add into an
// fp32 accumulation buffer that is laid out in exactly those blocks. That buffer is the only memory
// several CTAs add into (every KV tile contributes to every later query), so the order of the
// additions, and with it the last bits of dQ, may differ between runs; dK and dV are exact sums in
// a fixed order. A small kernel afterwards scales the buffer and writes bf16 dQ rows.
//
// 15 warps: 0 = TMA producer (+ lse / delta rows), 1 = issuer of S^T and dP^T, 2..9 = two softmax
// groups (32 query columns each, one key row per thread), 10..13 = dQ drain, 14 = issuer of dV, dK
// and dQ^T. Issuing a tcgen05.mma holds the issuing thread for about as long as the product occupies
// the tensor pipe, so a single issuer, with its waits in between, would be the critical path.
#include "common.cuh"

namespace ajb {
namespace attn {

namespace f128 {

constexpr int HD = 128;
constexpr int BKV = 128;           // keys per CTA
constexpr int BQ = 64;             // queries per step
constexpr int kStages = 3;         // Q / dO ring
constexpr int kThreads = 480;
constexpr float kLog2e = 1.4426950408889634f;

constexpr int kKvTile = BKV * HD * 2;          // 32 KB
constexpr int kQTile = BQ * HD * 2;            // 16 KB
constexpr int kDsTile = BKV * BQ * 2;          // 16 KB
constexpr int kStageBlock = BQ * 32 * 4;       // 8 KB: [64 queries][32 head-dim elements] fp32, one per drain warp
constexpr int kStatsBytes = kStages * 2 * BQ * 4;
constexpr int kSmemBytes = 2 * kKvTile + kStages * 2 * kQTile + 2 * kDsTile + 4 * kStageBlock + kStatsBytes + 256;
static_assert(kSmemBytes <= 232448, "shared memory budget");

constexpr int kDkCol = 0, kDvCol = 128, kSCol = 256, kDpCol = 320, kDqCol = 384;

struct Params {
  __nv_bfloat16* dqkv;
  const float* lse;
  const float* delta;
  float* dq_acc;          // [B, Hq, ceil(T / 64), 4, 64, 32] fp32, zeroed before the launch
  int batch, seq, heads, kv_heads;
  long long row_stride;
  int causal;
  float scale;
  DeviceStatus* status;
};

__device__ __forceinline__ void bulk_reduce_add_f32(float* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_hd128_kernel(const __grid_constant__ CUtensorMap map_kv, const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_do, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* sK = smem;
  uint8_t* sV = sK + kKvTile;
  uint8_t* sQdO = sV + kKvTile;                     // stage s: Q at sQdO + s * 2 * kQTile, dO right after
  uint8_t* sDS = sQdO + kStages * 2 * kQTile;       // two dS^T tiles
  uint8_t* sStage = sDS + 2 * kDsTile;              // four 8 KB blocks, one per drain warp
  float* sStats = reinterpret_cast<float*>(sStage + 4 * kStageBlock);   // [stage][lse * log2(e) 64 | delta 64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStats) + kStatsBytes);
  if (smem_misaligned(smem, p.status, kFlashBwdFused, reinterpret_cast<uint32_t*>(bars) + 60)) return;
  uint64_t* kv_full = bars;                    // 1
  uint64_t* qdo_full = bars + 1;               // kStages (TMA transaction + statistics rows)
  uint64_t* qdo_empty = qdo_full + kStages;    // kStages
  uint64_t* s_full = qdo_empty + kStages;      // 1
  uint64_t* dp_full = s_full + 1;              // 1
  uint64_t* p_ready = dp_full + 1;             // 1 (8 warps)
  uint64_t* ds_ready = p_ready + 1;            // 1 (8 warps)
  uint64_t* ds_free = ds_ready + 1;            // 2
  uint64_t* dq_full = ds_free + 2;             // 1
  uint64_t* dq_drained = dq_full + 1;          // 1 (4 warps)
  uint64_t* acc_done = dq_drained + 1;         // 1
  uint64_t* p_consumed = acc_done + 1;         // 1: dV of this iteration has been handed to the tensor pipe
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_consumed + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, kv_head = blockIdx.y, b = blockIdx.z;
  const int group = p.heads / p.kv_heads;
  const int k0 = kv_tile * BKV;
  const int n_q_tiles = (p.seq + BQ - 1) / BQ;
  const int first_q_tile = p.causal ? kv_tile * (BKV / BQ) : 0;
  const int per_head = n_q_tiles - first_q_tile;
  const int n_iter = per_head * group;
  const int k_col = (p.heads + kv_head) * HD;
  const int v_col = (p.heads + p.kv_heads + kv_head) * HD;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&qdo_full[i], 2);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 8);
    mbar_init(ds_ready, 8);
    mbar_init(&ds_free[0], 1);
    mbar_init(&ds_free[1], 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 4);
    mbar_init(acc_done, 1);
    mbar_init(p_consumed, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_kv);
    prefetch_tensor_map(&map_q);
    prefetch_tensor_map(&map_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer: TMA tiles + statistics rows
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * kKvTile);
#pragma unroll
      for (int i = 0; i < HD / 64; ++i) {
        tma_load_3d(sK + i * (BKV * 128), &map_kv, kv_full, k_col + 64 * i, k0, b);
        tma_load_3d(sV + i * (BKV * 128), &map_kv, kv_full, v_col + 64 * i, k0, b);
      }
    }
    int stage = 0;
    uint32_t phase = 0;
    for (int it = 0; it < n_iter; ++it) {
      const int head = kv_head * group + it / per_head;
      const int q0 = (first_q_tile + it % per_head) * BQ;
      if (!mbar_wait(&qdo_empty[stage], phase ^ 1, abort_flag, p.status, kFlashBwdFused, 1)) break;
      if (lane == 0) {
        uint8_t* sQ = sQdO + stage * 2 * kQTile;
        mbar_arrive_expect_tx(&qdo_full[stage], 2 * kQTile);
#pragma unroll
        for (int i = 0; i < HD / 64; ++i) {
          tma_load_3d(sQ + i * (BQ * 128), &map_q, &qdo_full[stage], head * HD + 64 * i, q0, b);
          tma_load_3d(sQ + kQTile + i * (BQ * 128), &map_do, &qdo_full[stage], head * HD + 64 * i, q0, b);
        }
      }
      float* st = sStats + stage * 2 * BQ;
      const size_t base = ((size_t)b * p.heads + head) * p.seq;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int q = q0 + lane * 2 + u;
        st[lane * 2 + u] = q < p.seq ? p.lse[base + q] * kLog2e : INFINITY;   // +inf -> p = 0 past the sequence end
        st[BQ + lane * 2 + u] = q < p.seq ? p.delta[base + q] : 0.0f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&qdo_full[stage]);
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- issuer A: S^T = K Q^T and dP^T = V dO^T
    constexpr uint32_t idesc_s = make_idesc(BKV, BQ, 1, false, false);
    // descriptor low words of the tiles; a k-step is a compile-time offset added to one of these
    const uint32_t k_km = desc_lo_k_major(smem_u32(sK)), v_km = desc_lo_k_major(smem_u32(sV));
    const uint32_t q_km0 = desc_lo_k_major(smem_u32(sQdO));
    constexpr uint32_t kStageStep = (2 * kQTile) >> 4, kDoStep = kQTile >> 4;
    bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kFlashBwdFused, 2);
    int stage = 0;
    uint32_t phase = 0;
    for (int it = 0; it < n_iter && ok; ++it) {
      if (!mbar_wait(&qdo_full[stage], phase, abort_flag, p.status, kFlashBwdFused, 3)) break;
      // S^T overwrites P^T of the previous iteration: its dV product must have been issued (the tensor pipe
      // executes in issue order)
      if (it > 0 && !mbar_wait(p_consumed, (uint32_t)(it - 1) & 1, abort_flag, p.status, kFlashBwdFused, 4)) break;
      tc_fence_after_sync();
      const uint32_t q_km = q_km0 + (uint32_t)stage * kStageStep, do_km = q_km + kDoStep;
      if (lane == 0) {
        umma_f16_c<false>(tmem_base + kSCol, desc_at(k_km, 0), desc_at(q_km, 0), idesc_s);
#pragma unroll
        for (int k = 1; k < HD / 16; ++k)
          umma_f16_c<true>(tmem_base + kSCol, desc_at(k_km, k_major_step(k, BKV * 128)), desc_at(q_km, k_major_step(k, BQ * 128)),
                           idesc_s);
        tc_commit(s_full);
      }
      __syncwarp();
      // dP^T of the previous iteration must have been read by the softmax warps
      if (it > 0 && !mbar_wait(ds_ready, (uint32_t)(it - 1) & 1, abort_flag, p.status, kFlashBwdFused, 5)) break;
      tc_fence_after_sync();
      if (lane == 0) {
        umma_f16_c<false>(tmem_base + kDpCol, desc_at(v_km, 0), desc_at(do_km, 0), idesc_s);
#pragma unroll
        for (int k = 1; k < HD / 16; ++k)
          umma_f16_c<true>(tmem_base + kDpCol, desc_at(v_km, k_major_step(k, BKV * 128)), desc_at(do_km, k_major_step(k, BQ * 128)),
                           idesc_s);
        tc_commit(dp_full);
      }
      __syncwarp();
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }
  } else if (warp < 10) {
    // ---------------------------------------------------------------- P^T / dS^T: thread = key row, group = 32 query columns
    const int quarter = warp & 3;
    const int wg = (warp - 2) >> 2;
    const int col_base = wg * 32;
    const int row = quarter * 32 + lane;
    const int key = k0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl = p.scale * kLog2e;
    bool ok = true;
    int stage = 0;
    uint32_t phase = 0;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int q0 = (first_q_tile + it % per_head) * BQ;
      if (!mbar_wait(&qdo_full[stage], phase, abort_flag, p.status, kFlashBwdFused, 7)) { ok = false; break; }
      if (!mbar_wait(s_full, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 8)) { ok = false; break; }
      tc_fence_after_sync();
      const float* lse2 = sStats + stage * 2 * BQ + col_base;
      const float* dlt = lse2 + BQ;
      const bool need_mask = (p.causal && q0 < k0 + BKV) || (k0 + BKV > p.seq);
      float pf[32];
      {
        uint32_t sv[32];
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(kSCol + col_base), sv);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse2 + i);
          pf[i + 0] = exp2f(fmaf(__uint_as_float(sv[i + 0]), sl, -l4.x));
          pf[i + 1] = exp2f(fmaf(__uint_as_float(sv[i + 1]), sl, -l4.y));
          pf[i + 2] = exp2f(fmaf(__uint_as_float(sv[i + 2]), sl, -l4.z));
          pf[i + 3] = exp2f(fmaf(__uint_as_float(sv[i + 3]), sl, -l4.w));
        }
        if (need_mask) {
          const int q_first = q0 + col_base;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if ((p.causal && key > q_first + i) || key >= p.seq) pf[i] = 0.0f;
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(pf[2 * i], pf[2 * i + 1]);
        tmem_st_32x16(tmem_base + lane_addr + (uint32_t)(kSCol + col_base), pk);
      }
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);

      if (!mbar_wait(dp_full, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 9)) { ok = false; break; }
      tc_fence_after_sync();
      // dS^T buffer it & 1 is free once the products of iteration it - 2 have read it
      if (!mbar_wait(&ds_free[it & 1], (((uint32_t)it >> 1) & 1) ^ 1, abort_flag, p.status, kFlashBwdFused, 10)) { ok = false; break; }
      {
        uint32_t dv[32];
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(kDpCol + col_base), dv);
        tc_wait_ld();
        uint32_t dsk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(dlt + i);
          const float a0 = pf[i + 0] * (__uint_as_float(dv[i + 0]) - d4.x);
          const float a1 = pf[i + 1] * (__uint_as_float(dv[i + 1]) - d4.y);
          const float a2 = pf[i + 2] * (__uint_as_float(dv[i + 2]) - d4.z);
          const float a3 = pf[i + 3] * (__uint_as_float(dv[i + 3]) - d4.w);
          dsk[i / 2] = pack_bf16x2(a0, a1);
          dsk[i / 2 + 1] = pack_bf16x2(a2, a3);
        }
        // K-major [128 keys x 64 queries] tile: one 128-byte row per key, 16-byte chunks swizzled by the row
        uint8_t* tile_row = sDS + (it & 1) * kDsTile + row * 128;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int chunk = wg * 4 + ch;
          *reinterpret_cast<uint4*>(tile_row + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(dsk[ch * 4], dsk[ch * 4 + 1], dsk[ch * 4 + 2], dsk[ch * 4 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }
    // epilogue: group 0 writes dK * scale, group 1 writes dV
    if (ok && n_iter > 0 && mbar_wait(acc_done, 0, abort_flag, p.status, kFlashBwdFused, 11)) {
      tc_fence_after_sync();
      const uint32_t col0 = wg == 0 ? kDkCol : kDvCol;
      const float mul = wg == 0 ? p.scale : 1.0f;
      __nv_bfloat16* dst = p.dqkv + ((size_t)b * p.seq + key) * p.row_stride + (wg == 0 ? k_col : v_col);
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_addr + col0 + (uint32_t)(c * 32), v);
        tc_wait_ld();
        if (key < p.seq) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(v[8 * i]) * mul, __uint_as_float(v[8 * i + 1]) * mul);
            q.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * mul, __uint_as_float(v[8 * i + 3]) * mul);
            q.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * mul, __uint_as_float(v[8 * i + 5]) * mul);
            q.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * mul, __uint_as_float(v[8 * i + 7]) * mul);
            reinterpret_cast<uint4*>(dst + c * 32)[i] = q;
          }
        }
      }
    }
  } else if (warp < 14) {
    // ---------------------------------------------------------------- dQ^T tiles: tensor memory -> shared memory -> bulk reduce-add
    const int quarter = warp & 3;                     // head-dim elements [32 * quarter, 32 * quarter + 32)
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float* block = reinterpret_cast<float*>(sStage + quarter * kStageBlock);   // [64 queries][32 elements]
    for (int it = 0; it < n_iter; ++it) {
      const int head = kv_head * group + it / per_head;
      const int q_tile = first_q_tile + it % per_head;
      if (!mbar_wait(dq_full, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 12)) break;
      tc_fence_after_sync();
      uint32_t v[2][32];
      tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)kDqCol, v[0]);
      tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(kDqCol + 32), v[1]);
      tc_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(dq_drained);
        bulk_wait_group_read0();          // the previous reduce of this warp has read the staging block
      }
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) block[(c * 32 + i) * 32 + lane] = __uint_as_float(v[c][i]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        float* dst = p.dq_acc + ((((size_t)b * p.heads + head) * n_q_tiles + q_tile) * 4 + quarter) * (BQ * 32);
        bulk_reduce_add_f32(dst, block, kStageBlock);
        bulk_commit_group();
      }
    }
    if (lane == 0) bulk_wait_group0();    // reductions complete before the CTA (and its shared memory) goes away
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- issuer B: dV += P^T dO, dK += dS^T Q, dQ^T = K^T dS
    constexpr uint32_t idesc_g = make_idesc(BKV, HD, 1, false, true);
    constexpr uint32_t idesc_q = make_idesc(HD, BQ, 1, true, true);
    const uint32_t k_mn = desc_lo_mn_major(smem_u32(sK), BKV * 128);
    const uint32_t q_mn0 = desc_lo_mn_major(smem_u32(sQdO), BQ * 128);
    const uint32_t ds_km0 = desc_lo_k_major(smem_u32(sDS)), ds_mn0 = desc_lo_mn_major(smem_u32(sDS), BKV * 128);
    constexpr uint32_t kStageStep = (2 * kQTile) >> 4, kDoStep = kQTile >> 4, kDsStep = kDsTile >> 4;
    bool ok = true;
    int stage = 0;
    for (int it = 0; it < n_iter && ok; ++it) {
      const uint32_t q_mn = q_mn0 + (uint32_t)stage * kStageStep, do_mn = q_mn + kDoStep;
      const uint32_t ds_km = ds_km0 + (uint32_t)(it & 1) * kDsStep, ds_mn = ds_mn0 + (uint32_t)(it & 1) * kDsStep;
      // P^T lives in tensor memory: queries 0..31 in columns [256, 272), 32..63 in [288, 304)
      if (!mbar_wait(p_ready, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 6)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        umma_f16_ts(tmem_base + kDvCol, tmem_base + kSCol, desc_at(do_mn, 0), idesc_g, it != 0);
#pragma unroll
        for (int k = 1; k < BQ / 16; ++k) {
          const uint32_t a_col = (uint32_t)(kSCol + (k < 2 ? k * 8 : 32 + (k - 2) * 8));
          umma_f16_ts_c<true>(tmem_base + kDvCol, tmem_base + a_col, desc_at(do_mn, mn_major_step(k)), idesc_g);
        }
        mbar_arrive(p_consumed);
      }
      __syncwarp();
      if (!mbar_wait(ds_ready, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 13)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        umma_f16(tmem_base + kDkCol, desc_at(ds_km, 0), desc_at(q_mn, 0), idesc_g, it != 0);
#pragma unroll
        for (int k = 1; k < BQ / 16; ++k)
          umma_f16_c<true>(tmem_base + kDkCol, desc_at(ds_km, (uint32_t)k * 32), desc_at(q_mn, mn_major_step(k)), idesc_g);
      }
      __syncwarp();
      if (it > 0 && !mbar_wait(dq_drained, (uint32_t)(it - 1) & 1, abort_flag, p.status, kFlashBwdFused, 14)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        umma_f16_c<false>(tmem_base + kDqCol, desc_at(k_mn, 0), desc_at(ds_mn, 0), idesc_q);
#pragma unroll
        for (int k = 1; k < BKV / 16; ++k)
          umma_f16_c<true>(tmem_base + kDqCol, desc_at(k_mn, mn_major_step(k)), desc_at(ds_mn, mn_major_step(k)), idesc_q);
        tc_commit(dq_full);
        tc_commit(&ds_free[it & 1]);
        tc_commit(&qdo_empty[stage]);
      }
      __syncwarp();
      if (++stage == kStages) stage = 0;
    }
    if (ok && lane == 0) tc_commit(acc_done);
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Blocked fp32 accumulation buffer -> scaled bf16 query-gradient columns of the packed rows.
__global__ void dq_store_blocked_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv, int batch,
                                        int seq, int heads, long long row_stride, float scale) {
  const int n_q_tiles = (seq + BQ - 1) / BQ;
  const long long total = (long long)batch * seq * heads * (HD / 8);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % (HD / 8));               // 8 consecutive head-dim elements
    long long r = i / (HD / 8);
    const int h = (int)(r % heads);
    r /= heads;
    const int t = (int)(r % seq);
    const int b = (int)(r / seq);
    const int d = c8 * 8;
    const float* src = acc + ((((size_t)b * heads + h) * n_q_tiles + t / BQ) * 4 + d / 32) * (BQ * 32) + (t % BQ) * 32 + d % 32;
    const float4 x = *reinterpret_cast<const float4*>(src);
    const float4 y = *reinterpret_cast<const float4*>(src + 4);
    uint4 o;
    o.x = pack_bf16x2(x.x * scale, x.y * scale);
    o.y = pack_bf16x2(x.z * scale, x.w * scale);
    o.z = pack_bf16x2(y.x * scale, y.y * scale);
    o.w = pack_bf16x2(y.z * scale, y.w * scale);
    *reinterpret_cast<uint4*>(dqkv + ((size_t)b * seq + t) * row_stride + (size_t)h * HD + d) = o;
  }
}

}  // namespace f128

// delta must already hold sum_d O * dO. dq_acc: B * Hq * ceil(T / 64) * 64 * 128 floats of scratch.
int launch_bwd_fused_hd128(const void* qkv, const void* dout, const void* lse, const void* delta, void* dqkv, void* dq_acc,
                           int batch, int seq, int heads, int kv_heads, long long row_stride, int causal, float scale,
                           cudaStream_t stream) {
  using namespace f128;
  CUtensorMap map_kv, map_q, map_do;
  int rc = make_tensor_map_3d(&map_kv, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, batch, seq, row_stride,
                              (uint64_t)seq * row_stride * 2, row_stride * 2, BKV, 64);
  if (rc) return rc;
  rc = make_tensor_map_3d(&map_q, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, batch, seq, row_stride,
                          (uint64_t)seq * row_stride * 2, row_stride * 2, BQ, 64);
  if (rc) return rc;
  const long long do_stride = (long long)heads * HD;
  rc = make_tensor_map_3d(&map_do, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, batch, seq, do_stride,
                          (uint64_t)seq * do_stride * 2, do_stride * 2, BQ, 64);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    AJB_CUDA_OK(cudaFuncSetAttribute(flash_bwd_hd128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured = true;
  }
  const int n_q_tiles = (seq + BQ - 1) / BQ;
  AJB_CUDA_OK(cudaMemsetAsync(dq_acc, 0, (size_t)batch * heads * n_q_tiles * BQ * HD * sizeof(float), stream));
  Params p;
  p.dqkv = (__nv_bfloat16*)dqkv; p.lse = (const float*)lse; p.delta = (const float*)delta; p.dq_acc = (float*)dq_acc;
  p.batch = batch; p.seq = seq; p.heads = heads; p.kv_heads = kv_heads; p.row_stride = row_stride;
  p.causal = causal; p.scale = scale; p.status = device_status_buffer();
  const int kv_tiles = (seq + BKV - 1) / BKV;
  flash_bwd_hd128_kernel<<<dim3(kv_tiles, kv_heads, batch), kThreads, kSmemBytes, stream>>>(map_kv, map_q, map_do, p);
  AJB_CUDA_OK(cudaGetLastError());
  const long long vecs = (long long)batch * seq * heads * (HD / 8);
  const int blocks = (int)min((long long)sm_count() * 8, (vecs + 255) / 256);
  dq_store_blocked_kernel<<<blocks, 256, 0, stream>>>((const float*)dq_acc, (__nv_bfloat16*)dqkv, batch, seq, heads, row_stride, scale);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace attn
}  // namespace ajb
