// FlashAttention backward for sm_100a. Three paths share this entry point:
//   * head_dim 128 with a dQ accumulation buffer: flash_bwd_hd128.cu (five products per 128 x 64 step, dQ through
//     TMA reduce-adds);
//   * other head sizes with a buffer: flash_bwd_fused_kernel below (five products per 128 x 128 step, dQ through
//     16-byte reductions);
//   * no buffer: the bit-reproducible path, two tcgen05 kernels plus a small reduction:
//
//   delta[b,h,t] = sum_d O[b,t,h,d] * dO[b,t,h,d]
//   dK/dV kernel : one CTA per (KV tile, KV head, batch); loops over the query heads of the group and
//                  their query tiles. S^T = K Q^T and dP^T = V dO^T land in tensor memory, four warps
//                  (one key row per thread) form P^T and dS^T, and dV += P^T dO, dK += dS^T Q
//                  accumulate in tensor memory over the whole loop.
//   dQ kernel    : one CTA per (query tile, head, batch); loops over KV tiles; S = Q K^T, dP = dO V^T,
//                  dS -> shared memory, dQ += dS K accumulates in tensor memory.
//
// No atomics on that path: every output element is produced by exactly one CTA.
// Gradients are written into a packed [B, T, (Hq + 2 Hkv) * hd] buffer laid out like the input.
#include "common.cuh"

namespace ajb {
namespace attn {

constexpr int BLK = 128;
constexpr int kBwdThreads = 192;
constexpr float kLog2eB = 1.4426950408889634f;

struct BwdParams {
  __nv_bfloat16* dqkv;
  const float* lse;
  const float* delta;
  float* dq_acc;          // fused kernel only: [B, T, Hq, hd] fp32, zeroed before the launch
  int batch, seq, heads, kv_heads;
  long long row_stride;
  int causal;
  float scale;
  DeviceStatus* status;
};

template <int HD>
__device__ __forceinline__ void load_tile_b(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int col, int row, int b) {
#pragma unroll
  for (int i = 0; i < HD / 64; ++i) tma_load_3d(dst + i * (BLK * 128), map, bar, col + 64 * i, row, b);
}

// Row `row` of a K-major, 128-byte-swizzled [128 x 128] bf16 operand tile: 16-byte chunk `ch` (0..15).
__device__ __forceinline__ void store_operand_chunk(uint8_t* tile, int row, int ch, uint4 val) {
  uint8_t* dst = tile + (ch >> 3) * (BLK * 128) + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
  *reinterpret_cast<uint4*>(dst) = val;
}

// ------------------------------------------------------------------------------------------ delta
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                                   float* __restrict__ delta, int batch, int seq, int heads, int head_dim) {
  // head_dim / 8 threads per (b, t, h), one 16-byte vector of O and of dO each; head_dim is 64 or 128, so a
  // group is 8 or 16 lanes of one warp
  const int group = head_dim >> 3;
  const long long thread = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long item = thread / group;
  const int part = (int)(thread % group);
  const long long total = (long long)batch * seq * heads;
  float s = 0.0f;
  if (item < total) {
    const uint4 a = reinterpret_cast<const uint4*>(out + (size_t)item * head_dim)[part];
    const uint4 g = reinterpret_cast<const uint4*>(dout + (size_t)item * head_dim)[part];
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(gh[i]);
      s += x.x * y.x + x.y * y.y;
    }
  }
  for (int off = group >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (item < total && part == 0) {
    const int h = (int)(item % heads);
    const long long bt = item / heads;
    const int b = (int)(bt / seq), t = (int)(bt % seq);
    delta[((size_t)b * heads + h) * seq + t] = s;
  }
}

// ------------------------------------------------------------------------------------------ dK / dV
template <int HD>
struct KvCfg {
  static constexpr int kTile = BLK * HD * 2;
  static constexpr int kPds = BLK * BLK * 2;
  // K, V resident; 2 stages of (Q, dO); one P/dS operand tile; per-stage lse/delta rows
  static constexpr int kSmemBytes = 2 * kTile + 4 * kTile + kPds + 2 * 2 * BLK * 4 + 256;
  static constexpr int kStCol = 0, kDptCol = 128, kDvCol = 256, kDkCol = 384;
};

template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_kv_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do,
                    const BwdParams p) {
  using Cfg = KvCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::kTile;
  uint8_t* sQdO = sV + Cfg::kTile;            // stage s: Q at sQdO + s*2*tile, dO right after
  uint8_t* sPdS = sQdO + 4 * Cfg::kTile;
  float* sStats = reinterpret_cast<float*>(sPdS + Cfg::kPds);   // [stage][lse 128 | delta 128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStats + 2 * 2 * BLK);
  if (smem_misaligned(smem, p.status, kFlashBwdKV, reinterpret_cast<uint32_t*>(bars) + 60)) return;
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // 2
  uint64_t* qdo_empty = bars + 3;    // 2
  uint64_t* s_full = bars + 5;       // 1
  uint64_t* ds_ready = bars + 6;     // 1 (count 4)
  uint64_t* dk_done = bars + 7;      // 1
  uint64_t* p_ready = bars + 8;      // 1 (count 4)
  uint64_t* dv_done = bars + 9;      // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, kv_head = blockIdx.y, b = blockIdx.z;
  const int group = p.heads / p.kv_heads;
  const int k0 = kv_tile * BLK;
  const int n_q_tiles = (p.seq + BLK - 1) / BLK;
  const int first_q_tile = p.causal ? kv_tile : 0;
  const int per_head = n_q_tiles - first_q_tile;
  const int n_iter = per_head * group;
  const int k_col = (p.heads + kv_head) * HD;
  const int v_col = (p.heads + p.kv_heads + kv_head) * HD;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1 + 4);   // TMA transaction + the four stats-loading warps
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(ds_ready, 4);
    mbar_init(dk_done, 1);
    mbar_init(p_ready, 4);
    mbar_init(dv_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_qkv);
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
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * Cfg::kTile);
      load_tile_b<HD>(sK, &map_qkv, kv_full, k_col, k0, b);
      load_tile_b<HD>(sV, &map_qkv, kv_full, v_col, k0, b);
      for (int it = 0; it < n_iter; ++it) {
        const int s = it & 1;
        const int head = kv_head * group + it / per_head;
        const int q0 = (first_q_tile + it % per_head) * BLK;
        if (!mbar_wait(&qdo_empty[s], (((uint32_t)it >> 1) & 1) ^ 1, abort_flag, p.status, kFlashBwdKV, 1)) break;
        uint8_t* sQ = sQdO + s * 2 * Cfg::kTile;
        mbar_arrive_expect_tx(&qdo_full[s], 2 * Cfg::kTile);
        load_tile_b<HD>(sQ, &map_qkv, &qdo_full[s], head * HD, q0, b);
        load_tile_b<HD>(sQ + Cfg::kTile, &map_do, &qdo_full[s], head * HD, q0, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_s = make_idesc(BLK, BLK, 1, false, false);   // K Q^T, V dO^T
    constexpr uint32_t idesc_g = make_idesc(BLK, HD, 1, false, true);     // dS^T Q, P^T dO
    const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aPdS = smem_u32(sPdS);
    bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kFlashBwdKV, 2);
    auto issue_scores = [&](int it) -> bool {
      const int s = it & 1;
      if (!mbar_wait(&qdo_full[s], ((uint32_t)it >> 1) & 1, abort_flag, p.status, kFlashBwdKV, 3)) return false;
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t aQ = smem_u32(sQdO + s * 2 * Cfg::kTile), aDO = aQ + Cfg::kTile;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t box = (uint32_t)(k / 4) * (BLK * 128), off = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kStCol, desc_k_major(aK + box, off), desc_k_major(aQ + box, off), idesc_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t box = (uint32_t)(k / 4) * (BLK * 128), off = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kDptCol, desc_k_major(aV + box, off), desc_k_major(aDO + box, off), idesc_s, k != 0);
        }
        tc_commit(s_full);
      }
      __syncwarp();
      return true;
    };
    if (ok && n_iter > 0) ok = issue_scores(0);
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const uint32_t aQ = smem_u32(sQdO + s * 2 * Cfg::kTile), aDO = aQ + Cfg::kTile;
      if (!mbar_wait(ds_ready, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdKV, 4)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k) {
          const uint32_t pbox = (uint32_t)(k / 4) * (BLK * 128), poff = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kDkCol, desc_k_major(aPdS + pbox, poff), desc_mn_major(aQ, BLK * 128, k * 16),
                   idesc_g, (it | k) != 0);
        }
        tc_commit(dk_done);
      }
      __syncwarp();
      // S^T / dP^T of this iteration have been consumed (ds_ready): start the next pair now
      if (it + 1 < n_iter) {
        ok = issue_scores(it + 1);
        if (!ok) break;
      }
      if (!mbar_wait(p_ready, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdKV, 5)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k) {
          const uint32_t pbox = (uint32_t)(k / 4) * (BLK * 128), poff = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kDvCol, desc_k_major(aPdS + pbox, poff), desc_mn_major(aDO, BLK * 128, k * 16),
                   idesc_g, (it | k) != 0);
        }
        tc_commit(dv_done);
        tc_commit(&qdo_empty[s]);
      }
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------------------- P^T / dS^T (thread = key row)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int key = k0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl = p.scale * kLog2eB;
    const int tid = threadIdx.x - 64;  // 0..127
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const int head = kv_head * group + it / per_head;
      const int q0 = (first_q_tile + it % per_head) * BLK;
      // stage the row statistics of this query tile (slot s is free: its previous user finished two iterations ago)
      {
        float* st = sStats + s * 2 * BLK;
        const int q = q0 + tid;
        const size_t idx = ((size_t)b * p.heads + head) * p.seq + q;
        st[tid] = q < p.seq ? p.lse[idx] * kLog2eB : INFINITY;   // +inf -> p = 0 for rows past the sequence end
        st[BLK + tid] = q < p.seq ? p.delta[idx] : 0.0f;
        __syncwarp();
        if (lane == 0) mbar_arrive(&qdo_full[s]);
      }
      if (!mbar_wait(&qdo_full[s], ((uint32_t)it >> 1) & 1, abort_flag, p.status, kFlashBwdKV, 6)) { ok = false; break; }
      if (!mbar_wait(s_full, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdKV, 7)) { ok = false; break; }
      tc_fence_after_sync();
      // the operand tile is free once the previous dV product has read it
      if (it > 0 && !mbar_wait(dv_done, (uint32_t)(it - 1) & 1, abort_flag, p.status, kFlashBwdKV, 8)) { ok = false; break; }
      const float* lse2 = sStats + s * 2 * BLK;
      const float* dlt = lse2 + BLK;
      const bool diag = p.causal && (q0 < k0 + BLK);   // some (key, query) pairs of this tile are masked
      uint32_t pk[64];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kStCol + c * 32), sv);
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kDptCol + c * 32), dv);
        tc_wait_ld();
        uint32_t dsk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pr[2], ds[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int qi = c * 32 + i + u;
            float pv = exp2f(fmaf(__uint_as_float(sv[i + u]), sl, -lse2[qi]));
            if ((diag && key > q0 + qi) || key >= p.seq) pv = 0.0f;
            pr[u] = pv;
            ds[u] = pv * (__uint_as_float(dv[i + u]) - dlt[qi]);
          }
          pk[c * 16 + i / 2] = pack_bf16x2(pr[0], pr[1]);
          dsk[i / 2] = pack_bf16x2(ds[0], ds[1]);
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          store_operand_chunk(sPdS, row, c * 4 + ch, make_uint4(dsk[ch * 4], dsk[ch * 4 + 1], dsk[ch * 4 + 2], dsk[ch * 4 + 3]));
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
      // dK product reads dS^T; once done, the same tile carries P^T for the dV product
      if (!mbar_wait(dk_done, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdKV, 9)) { ok = false; break; }
#pragma unroll
      for (int ch = 0; ch < 16; ++ch)
        store_operand_chunk(sPdS, row, ch, make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    // epilogue: dK * scale and dV -> packed gradient rows
    if (ok && (n_iter == 0 || mbar_wait(dv_done, (uint32_t)(n_iter - 1) & 1, abort_flag, p.status, kFlashBwdKV, 10))) {
      tc_fence_after_sync();
      const bool row_ok = key < p.seq;
      __nv_bfloat16* base = p.dqkv + ((size_t)b * p.seq + key) * p.row_stride;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t col0 = which == 0 ? Cfg::kDkCol : Cfg::kDvCol;
        const float mul = which == 0 ? p.scale : 1.0f;
        __nv_bfloat16* dst = base + (which == 0 ? k_col : v_col);
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          if (n_iter > 0) {
            tmem_ld_32x32(tmem_base + lane_addr + col0 + (uint32_t)(c * 32), v);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          if (row_ok) {
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
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------ dQ
template <int HD>
struct QCfg {
  static constexpr int kTile = BLK * HD * 2;
  static constexpr int kDs = BLK * BLK * 2;
  static constexpr int kSmemBytes = 2 * kTile + 4 * kTile + kDs + 256;
  static constexpr int kSCol = 0, kDpCol = 128, kDqCol = 256;
};

template <int HD>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_q_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do,
                   const BwdParams p) {
  using Cfg = QCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + Cfg::kTile;
  uint8_t* sKV = sDO + Cfg::kTile;           // stage s: K at sKV + s*2*tile, V right after
  uint8_t* sDS = sKV + 4 * Cfg::kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + Cfg::kDs);
  if (smem_misaligned(smem, p.status, kFlashBwdQ, reinterpret_cast<uint32_t*>(bars) + 60)) return;
  uint64_t* q_full = bars;           // 1
  uint64_t* kv_full = bars + 1;      // 2
  uint64_t* kv_empty = bars + 3;     // 2
  uint64_t* s_full = bars + 5;       // 1
  uint64_t* ds_ready = bars + 6;     // 1 (count 4)
  uint64_t* dq_done = bars + 7;      // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int head = blockIdx.y, b = blockIdx.z;
  const int kv_head = head / (p.heads / p.kv_heads);
  const int q0 = q_tile * BLK;
  const int k_col = (p.heads + kv_head) * HD;
  const int v_col = (p.heads + p.kv_heads + kv_head) * HD;
  const int kv_limit = p.causal ? min(p.seq, q0 + BLK) : p.seq;
  const int n_tiles = (kv_limit + BLK - 1) / BLK;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(ds_ready, 4);
    mbar_init(dq_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_qkv);
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
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * Cfg::kTile);
      load_tile_b<HD>(sQ, &map_qkv, q_full, head * HD, q0, b);
      load_tile_b<HD>(sDO, &map_do, q_full, head * HD, q0, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], (((uint32_t)j >> 1) & 1) ^ 1, abort_flag, p.status, kFlashBwdQ, 1)) break;
        uint8_t* sK = sKV + s * 2 * Cfg::kTile;
        mbar_arrive_expect_tx(&kv_full[s], 2 * Cfg::kTile);
        load_tile_b<HD>(sK, &map_qkv, &kv_full[s], k_col, j * BLK, b);
        load_tile_b<HD>(sK + Cfg::kTile, &map_qkv, &kv_full[s], v_col, j * BLK, b);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_s = make_idesc(BLK, BLK, 1, false, false);
    constexpr uint32_t idesc_g = make_idesc(BLK, HD, 1, false, true);
    const uint32_t aQ = smem_u32(sQ), aDO = smem_u32(sDO), aDS = smem_u32(sDS);
    bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kFlashBwdQ, 2);
    auto issue_scores = [&](int j) -> bool {
      const int s = j & 1;
      if (!mbar_wait(&kv_full[s], ((uint32_t)j >> 1) & 1, abort_flag, p.status, kFlashBwdQ, 3)) return false;
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t aK = smem_u32(sKV + s * 2 * Cfg::kTile), aV = aK + Cfg::kTile;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t box = (uint32_t)(k / 4) * (BLK * 128), off = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kSCol, desc_k_major(aQ + box, off), desc_k_major(aK + box, off), idesc_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t box = (uint32_t)(k / 4) * (BLK * 128), off = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kDpCol, desc_k_major(aDO + box, off), desc_k_major(aV + box, off), idesc_s, k != 0);
        }
        tc_commit(s_full);
      }
      __syncwarp();
      return true;
    };
    if (ok && n_tiles > 0) ok = issue_scores(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait(ds_ready, (uint32_t)j & 1, abort_flag, p.status, kFlashBwdQ, 4)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t aK = smem_u32(sKV + s * 2 * Cfg::kTile);
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k) {
          const uint32_t pbox = (uint32_t)(k / 4) * (BLK * 128), poff = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kDqCol, desc_k_major(aDS + pbox, poff), desc_mn_major(aK, BLK * 128, k * 16),
                   idesc_g, (j | k) != 0);
        }
        tc_commit(dq_done);
        tc_commit(&kv_empty[s]);
      }
      __syncwarp();
      if (j + 1 < n_tiles) {
        ok = issue_scores(j + 1);
        if (!ok) break;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int q_pos = q0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl = p.scale * kLog2eB;
    const size_t stat_idx = ((size_t)b * p.heads + head) * p.seq + q_pos;
    const float lse2 = q_pos < p.seq ? p.lse[stat_idx] * kLog2eB : INFINITY;
    const float dlt = q_pos < p.seq ? p.delta[stat_idx] : 0.0f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int k0 = j * BLK;
      if (!mbar_wait(s_full, (uint32_t)j & 1, abort_flag, p.status, kFlashBwdQ, 5)) { ok = false; break; }
      tc_fence_after_sync();
      if (j > 0 && !mbar_wait(dq_done, (uint32_t)(j - 1) & 1, abort_flag, p.status, kFlashBwdQ, 6)) { ok = false; break; }
      const bool need_mask = (p.causal && k0 + BLK > q0) || (k0 + BLK > p.seq);
      const int k_max = p.causal ? min(q_pos, p.seq - 1) : p.seq - 1;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kSCol + c * 32), sv);
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kDpCol + c * 32), dv);
        tc_wait_ld();
        uint32_t dsk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float ds[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            float pv = exp2f(fmaf(__uint_as_float(sv[i + u]), sl, -lse2));
            if (need_mask && (k0 + c * 32 + i + u > k_max)) pv = 0.0f;
            ds[u] = pv * (__uint_as_float(dv[i + u]) - dlt);
          }
          dsk[i / 2] = pack_bf16x2(ds[0], ds[1]);
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          store_operand_chunk(sDS, row, c * 4 + ch, make_uint4(dsk[ch * 4], dsk[ch * 4 + 1], dsk[ch * 4 + 2], dsk[ch * 4 + 3]));
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    if (ok && n_tiles > 0 && mbar_wait(dq_done, (uint32_t)(n_tiles - 1) & 1, abort_flag, p.status, kFlashBwdQ, 7)) {
      tc_fence_after_sync();
      const bool row_ok = q_pos < p.seq;
      __nv_bfloat16* dst = p.dqkv + ((size_t)b * p.seq + q_pos) * p.row_stride + (size_t)head * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kDqCol + c * 32), v);
        tc_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(v[8 * i]) * p.scale, __uint_as_float(v[8 * i + 1]) * p.scale);
            q.y = pack_bf16x2(__uint_as_float(v[8 * i + 2]) * p.scale, __uint_as_float(v[8 * i + 3]) * p.scale);
            q.z = pack_bf16x2(__uint_as_float(v[8 * i + 4]) * p.scale, __uint_as_float(v[8 * i + 5]) * p.scale);
            q.w = pack_bf16x2(__uint_as_float(v[8 * i + 6]) * p.scale, __uint_as_float(v[8 * i + 7]) * p.scale);
            reinterpret_cast<uint4*>(dst + c * 32)[i] = q;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}


// ------------------------------------------------------------------------------------------ fused dK / dV / dQ
// One CTA per (KV tile, KV head, batch) computes all three gradients with five tensor-core products
// per (KV tile, query tile) pair instead of the seven of the two-kernel path:
//
//   S^T  = K Q^T          -> TMEM [0, 128)      P^T (bf16, packed two per column) overwrites it in place
//   dP^T = V dO^T         -> TMEM [128, 256)    dQ_tile = dS K reuses these columns once dP^T is consumed
//   dV  += P^T dO            (A operand read from tensor memory)
//   dK  += dS^T Q            (dS^T staged once in shared memory, K-major)
//   dQ_tile = dS K           (the same dS^T tile read as an MN-major A operand)
//
// 14 warps: TMA producer (also stages the lse / delta rows), MMA issuer, two groups of four warps
// that each turn one half of the 128 query columns into P^T and dS^T (one key row per thread), and
// four warps that drain each dQ tile from tensor memory into an fp32 accumulation buffer with vector
// reductions (queries are shared by all KV tiles, so this is the one place where CTAs add into the
// same memory; the sum order, and therefore the last bits of dQ, can differ between runs).
template <int HD>
struct FusedCfg {
  static constexpr int kTile = BLK * HD * 2;
  static constexpr int kDs = BLK * BLK * 2;
  static constexpr int kSmemBytes = 2 * kTile + 4 * kTile + kDs + 2 * 2 * BLK * 4 + 256;
  static constexpr int kStCol = 0, kDptCol = 128, kDvCol = 256, kDkCol = 384;
};
constexpr int kFusedThreads = 448;

template <int HD>
__global__ void __launch_bounds__(kFusedThreads, 1)
flash_bwd_fused_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do,
                       const BwdParams p) {
  using Cfg = FusedCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::kTile;
  uint8_t* sQdO = sV + Cfg::kTile;            // stage s: Q at sQdO + s*2*tile, dO right after
  uint8_t* sDS = sQdO + 4 * Cfg::kTile;
  float* sStats = reinterpret_cast<float*>(sDS + Cfg::kDs);   // [stage][lse * log2(e) 128 | delta 128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStats + 2 * 2 * BLK);
  if (smem_misaligned(smem, p.status, kFlashBwdFused, reinterpret_cast<uint32_t*>(bars) + 60)) return;
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // 2 (TMA transaction + statistics rows)
  uint64_t* qdo_empty = bars + 3;    // 2
  uint64_t* s_full = bars + 5;       // S^T of this iteration is in tensor memory
  uint64_t* dp_full = bars + 6;      // dP^T of this iteration is in tensor memory
  uint64_t* p_ready = bars + 7;      // P^T written back to tensor memory (8 warps)
  uint64_t* ds_ready = bars + 8;     // dS^T staged in shared memory, dP^T consumed (8 warps)
  uint64_t* ds_free = bars + 9;      // the products reading dS^T have finished
  uint64_t* dq_full = bars + 10;     // dQ tile is in tensor memory
  uint64_t* dq_drained = bars + 11;  // dQ tile copied out (4 warps)
  uint64_t* acc_done = bars + 12;    // every product of this CTA has finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, kv_head = blockIdx.y, b = blockIdx.z;
  const int group = p.heads / p.kv_heads;
  const int k0 = kv_tile * BLK;
  const int n_q_tiles = (p.seq + BLK - 1) / BLK;
  const int first_q_tile = p.causal ? kv_tile : 0;
  const int per_head = n_q_tiles - first_q_tile;
  const int n_iter = per_head * group;
  const int k_col = (p.heads + kv_head) * HD;
  const int v_col = (p.heads + p.kv_heads + kv_head) * HD;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 2);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 8);
    mbar_init(ds_ready, 8);
    mbar_init(ds_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 4);
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_qkv);
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
      mbar_arrive_expect_tx(kv_full, 2 * Cfg::kTile);
      load_tile_b<HD>(sK, &map_qkv, kv_full, k_col, k0, b);
      load_tile_b<HD>(sV, &map_qkv, kv_full, v_col, k0, b);
    }
    for (int it = 0; it < n_iter; ++it) {
      const int s = it & 1;
      const int head = kv_head * group + it / per_head;
      const int q0 = (first_q_tile + it % per_head) * BLK;
      if (!mbar_wait(&qdo_empty[s], (((uint32_t)it >> 1) & 1) ^ 1, abort_flag, p.status, kFlashBwdFused, 1)) break;
      if (lane == 0) {
        uint8_t* sQ = sQdO + s * 2 * Cfg::kTile;
        mbar_arrive_expect_tx(&qdo_full[s], 2 * Cfg::kTile);
        load_tile_b<HD>(sQ, &map_qkv, &qdo_full[s], head * HD, q0, b);
        load_tile_b<HD>(sQ + Cfg::kTile, &map_do, &qdo_full[s], head * HD, q0, b);
      }
      float* st = sStats + s * 2 * BLK;
      const size_t base = ((size_t)b * p.heads + head) * p.seq;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = q0 + lane * 4 + u;
        st[lane * 4 + u] = q < p.seq ? p.lse[base + q] * kLog2eB : INFINITY;   // +inf -> p = 0 past the sequence end
        st[BLK + lane * 4 + u] = q < p.seq ? p.delta[base + q] : 0.0f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&qdo_full[s]);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_s = make_idesc(BLK, BLK, 1, false, false);   // K Q^T, V dO^T
    constexpr uint32_t idesc_g = make_idesc(BLK, HD, 1, false, true);     // P^T dO, dS^T Q
    constexpr uint32_t idesc_q = make_idesc(BLK, HD, 1, true, true);      // dS K
    const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aDS = smem_u32(sDS);
    bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kFlashBwdFused, 2);
    auto issue_s = [&](int it) -> bool {
      const int s = it & 1;
      if (!mbar_wait(&qdo_full[s], ((uint32_t)it >> 1) & 1, abort_flag, p.status, kFlashBwdFused, 3)) return false;
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t aQ = smem_u32(sQdO + s * 2 * Cfg::kTile);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t box = (uint32_t)(k / 4) * (BLK * 128), off = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kStCol, desc_k_major(aK + box, off), desc_k_major(aQ + box, off), idesc_s, k != 0);
        }
        tc_commit(s_full);
      }
      __syncwarp();
      return true;
    };
    auto issue_dp = [&](int it) {
      if (lane == 0) {
        const uint32_t aDO = smem_u32(sQdO + (it & 1) * 2 * Cfg::kTile) + Cfg::kTile;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t box = (uint32_t)(k / 4) * (BLK * 128), off = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kDptCol, desc_k_major(aV + box, off), desc_k_major(aDO + box, off), idesc_s, k != 0);
        }
        tc_commit(dp_full);
      }
      __syncwarp();
    };
    if (ok && n_iter > 0) {
      ok = issue_s(0);
      if (ok) issue_dp(0);
    }
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const uint32_t aQ = smem_u32(sQdO + s * 2 * Cfg::kTile), aDO = aQ + Cfg::kTile;
      // dV += P^T dO, with P^T read from tensor memory: query columns 0..63 live in columns [0, 32) and
      // 64..127 in [64, 96) of the S^T region (each softmax group overwrites only what it has read)
      if (!mbar_wait(p_ready, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 4)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k) {
          const uint32_t a_col = (uint32_t)(Cfg::kStCol + (k < 4 ? k * 8 : 64 + (k - 4) * 8));
          umma_f16_ts(tmem_base + Cfg::kDvCol, tmem_base + a_col, desc_mn_major(aDO, BLK * 128, k * 16), idesc_g,
                      (it | k) != 0);
        }
      }
      __syncwarp();
      // the tensor pipe executes in order, so the next S^T may overwrite P^T right behind the dV product
      if (it + 1 < n_iter) {
        ok = issue_s(it + 1);
        if (!ok) break;
      }
      if (!mbar_wait(ds_ready, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 5)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k) {
          const uint32_t pbox = (uint32_t)(k / 4) * (BLK * 128), poff = (uint32_t)(k % 4) * 32;
          umma_f16(tmem_base + Cfg::kDkCol, desc_k_major(aDS + pbox, poff), desc_mn_major(aQ, BLK * 128, k * 16),
                   idesc_g, (it | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k)
          umma_f16(tmem_base + Cfg::kDptCol, desc_mn_major(aDS, BLK * 128, k * 16), desc_mn_major(aK, BLK * 128, k * 16),
                   idesc_q, k != 0);
        tc_commit(dq_full);
        tc_commit(ds_free);
        tc_commit(&qdo_empty[s]);
      }
      __syncwarp();
      if (it + 1 < n_iter) {
        // dP^T of the next iteration lands where this dQ tile sits: wait until it has been copied out
        if (!mbar_wait(dq_drained, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 6)) { ok = false; break; }
        tc_fence_after_sync();
        issue_dp(it + 1);
      }
    }
    if (ok && lane == 0) tc_commit(acc_done);
    __syncwarp();
  } else if (warp < 10) {
    // ---------------------------------------------------------------- P^T / dS^T: thread = key row, group = 64 query columns
    const int quarter = warp & 3;
    const int wg = (warp - 2) >> 2;
    const int col_base = wg * 64;
    const int row = quarter * 32 + lane;
    const int key = k0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl = p.scale * kLog2eB;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int s = it & 1;
      const int q0 = (first_q_tile + it % per_head) * BLK;
      if (!mbar_wait(&qdo_full[s], ((uint32_t)it >> 1) & 1, abort_flag, p.status, kFlashBwdFused, 7)) { ok = false; break; }
      if (!mbar_wait(s_full, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 8)) { ok = false; break; }
      tc_fence_after_sync();
      const float* lse2 = sStats + s * 2 * BLK + col_base;
      const float* dlt = lse2 + BLK;
      const bool need_mask = (p.causal && q0 < k0 + BLK) || (k0 + BLK > p.seq);
      float pf[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32];
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kStCol + col_base + c * 32), sv);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse2 + c * 32 + i);
          pf[c * 32 + i + 0] = exp2f(fmaf(__uint_as_float(sv[i + 0]), sl, -l4.x));
          pf[c * 32 + i + 1] = exp2f(fmaf(__uint_as_float(sv[i + 1]), sl, -l4.y));
          pf[c * 32 + i + 2] = exp2f(fmaf(__uint_as_float(sv[i + 2]), sl, -l4.z));
          pf[c * 32 + i + 3] = exp2f(fmaf(__uint_as_float(sv[i + 3]), sl, -l4.w));
        }
        if (need_mask) {
          const int q_first = q0 + col_base + c * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if ((p.causal && key > q_first + i) || key >= p.seq) pf[c * 32 + i] = 0.0f;
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(pf[c * 32 + 2 * i], pf[c * 32 + 2 * i + 1]);
        tmem_st_32x16(tmem_base + lane_addr + (uint32_t)(Cfg::kStCol + col_base + c * 16), pk);
      }
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);

      if (!mbar_wait(dp_full, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 9)) { ok = false; break; }
      tc_fence_after_sync();
      // the dS^T tile is free once the products of the previous iteration have read it
      if (it > 0 && !mbar_wait(ds_free, (uint32_t)(it - 1) & 1, abort_flag, p.status, kFlashBwdFused, 10)) { ok = false; break; }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t dv[32];
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kDptCol + col_base + c * 32), dv);
        tc_wait_ld();
        uint32_t dsk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(dlt + c * 32 + i);
          const float a0 = pf[c * 32 + i + 0] * (__uint_as_float(dv[i + 0]) - d4.x);
          const float a1 = pf[c * 32 + i + 1] * (__uint_as_float(dv[i + 1]) - d4.y);
          const float a2 = pf[c * 32 + i + 2] * (__uint_as_float(dv[i + 2]) - d4.z);
          const float a3 = pf[c * 32 + i + 3] * (__uint_as_float(dv[i + 3]) - d4.w);
          dsk[i / 2] = pack_bf16x2(a0, a1);
          dsk[i / 2 + 1] = pack_bf16x2(a2, a3);
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          store_operand_chunk(sDS, row, (col_base + c * 32) / 8 + ch,
                              make_uint4(dsk[ch * 4], dsk[ch * 4 + 1], dsk[ch * 4 + 2], dsk[ch * 4 + 3]));
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    // epilogue: group 0 writes dK * scale, group 1 writes dV
    if (ok && n_iter > 0 && mbar_wait(acc_done, 0, abort_flag, p.status, kFlashBwdFused, 11)) {
      tc_fence_after_sync();
      const uint32_t col0 = wg == 0 ? Cfg::kDkCol : Cfg::kDvCol;
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
  } else {
    // ---------------------------------------------------------------- dQ tiles: tensor memory -> fp32 accumulation buffer
    const int quarter = warp & 3;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    for (int it = 0; it < n_iter; ++it) {
      const int head = kv_head * group + it / per_head;
      const int q = (first_q_tile + it % per_head) * BLK + quarter * 32 + lane;
      if (!mbar_wait(dq_full, (uint32_t)it & 1, abort_flag, p.status, kFlashBwdFused, 12)) break;
      tc_fence_after_sync();
      {
        float* dst = p.dq_acc + (((size_t)b * p.seq + q) * p.heads + head) * HD;
        // passes of 64 columns keep the register footprint at half a 128-wide tile row
#pragma unroll
        for (int half = 0; half < HD / 64; ++half) {
          uint32_t v[2][32];
          tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kDptCol + half * 64), v[0]);
          tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kDptCol + half * 64 + 32), v[1]);
          tc_wait_ld();
          if (half == HD / 64 - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(dq_drained);
          }
          if (q < p.seq) {
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                red_add_f32x4(dst + half * 64 + c * 32 + i, __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]),
                              __uint_as_float(v[c][i + 2]), __uint_as_float(v[c][i + 3]));
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// dQ accumulation buffer [B, T, Hq, hd] fp32 -> scaled bf16 rows of the packed gradient.
__global__ void flash_dq_store_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv, long long rows,
                                      int q_width, long long row_stride, float scale) {
  const int per_row = q_width / 8;
  const long long total = rows * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const float4 a = *reinterpret_cast<const float4*>(acc + r * q_width + c);
    const float4 bq = *reinterpret_cast<const float4*>(acc + r * q_width + c + 4);
    uint4 o;
    o.x = pack_bf16x2(a.x * scale, a.y * scale);
    o.y = pack_bf16x2(a.z * scale, a.w * scale);
    o.z = pack_bf16x2(bq.x * scale, bq.y * scale);
    o.w = pack_bf16x2(bq.z * scale, bq.w * scale);
    *reinterpret_cast<uint4*>(dqkv + r * row_stride + c) = o;
  }
}

// head_dim 128: five products per (128 keys x 64 queries) step, dQ through bulk reduce-adds (flash_bwd_hd128.cu)
int launch_bwd_fused_hd128(const void* qkv, const void* dout, const void* lse, const void* delta, void* dqkv, void* dq_acc,
                           int batch, int seq, int heads, int kv_heads, long long row_stride, int causal, float scale,
                           cudaStream_t stream);

template <int HD>
static int launch_bwd(const void* qkv, const void* out, const void* dout, const void* lse, void* delta, void* dqkv,
                      void* dq_acc, int batch, int seq, int heads, int kv_heads, long long row_stride, int causal,
                      float scale, cudaStream_t stream) {
  const long long items = (long long)batch * seq * heads;
  const int threads = 256;
  const long long blocks = (items * (HD / 8) + threads - 1) / threads;
  flash_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout,
                                                                (float*)delta, batch, seq, heads, HD);
  AJB_CUDA_OK(cudaGetLastError());

  CUtensorMap map_qkv, map_do;
  int rc = make_tensor_map_3d(&map_qkv, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, batch, seq, row_stride,
                              (uint64_t)seq * row_stride * 2, row_stride * 2, BLK, 64);
  if (rc) return rc;
  const long long do_stride = (long long)heads * HD;
  rc = make_tensor_map_3d(&map_do, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, batch, seq, do_stride,
                          (uint64_t)seq * do_stride * 2, do_stride * 2, BLK, 64);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    AJB_CUDA_OK(cudaFuncSetAttribute(flash_bwd_kv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     KvCfg<HD>::kSmemBytes));
    AJB_CUDA_OK(cudaFuncSetAttribute(flash_bwd_q_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     QCfg<HD>::kSmemBytes));
    AJB_CUDA_OK(cudaFuncSetAttribute(flash_bwd_fused_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     FusedCfg<HD>::kSmemBytes));
    configured = true;
  }
  BwdParams p;
  p.dqkv = (__nv_bfloat16*)dqkv; p.lse = (const float*)lse; p.delta = (const float*)delta;
  p.dq_acc = (float*)dq_acc;
  p.batch = batch; p.seq = seq; p.heads = heads; p.kv_heads = kv_heads; p.row_stride = row_stride;
  p.causal = causal; p.scale = scale; p.status = device_status_buffer();
  const int tiles = (seq + BLK - 1) / BLK;
  if (dq_acc != nullptr && HD == 128)
    return launch_bwd_fused_hd128(qkv, dout, lse, delta, dqkv, dq_acc, batch, seq, heads, kv_heads, row_stride, causal, scale,
                                  stream);
  if (dq_acc != nullptr) {
    const long long rows = (long long)batch * seq;
    const int q_width = heads * HD;
    AJB_CUDA_OK(cudaMemsetAsync(dq_acc, 0, (size_t)rows * q_width * sizeof(float), stream));
    flash_bwd_fused_kernel<HD><<<dim3(tiles, kv_heads, batch), kFusedThreads, FusedCfg<HD>::kSmemBytes, stream>>>(map_qkv, map_do, p);
    AJB_CUDA_OK(cudaGetLastError());
    const long long vecs = rows * (q_width / 8);
    const int blocks = (int)min((long long)sm_count() * 8, (vecs + 255) / 256);
    flash_dq_store_kernel<<<blocks, 256, 0, stream>>>((const float*)dq_acc, (__nv_bfloat16*)dqkv, rows, q_width, row_stride, scale);
    AJB_CUDA_OK(cudaGetLastError());
    return 0;
  }
  flash_bwd_kv_kernel<HD><<<dim3(tiles, kv_heads, batch), kBwdThreads, KvCfg<HD>::kSmemBytes, stream>>>(map_qkv, map_do, p);
  AJB_CUDA_OK(cudaGetLastError());
  flash_bwd_q_kernel<HD><<<dim3(tiles, heads, batch), kBwdThreads, QCfg<HD>::kSmemBytes, stream>>>(map_qkv, map_do, p);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace attn
}  // namespace ajb

// delta: scratch [batch, heads, seq] fp32 (written here). dqkv: packed gradient rows, same layout as qkv.
// dq_acc: fp32 scratch of batch * heads * round_up(seq, 64) * head_dim elements selects the fused single-pass
// kernels (dQ tiles are added into it with reductions); nullptr selects the two-kernel path whose results
// are bit-reproducible.
extern "C" int ajb_flash_bwd(const void* qkv, const void* out, const void* dout, const void* lse, void* delta,
                             void* dqkv, void* dq_acc, int batch, int seq, int heads, int kv_heads, int head_dim,
                             long long row_stride, int causal, float scale, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(heads % kv_heads == 0, "flash: kv_heads must divide heads");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (head_dim == 128)
    return attn::launch_bwd<128>(qkv, out, dout, lse, delta, dqkv, dq_acc, batch, seq, heads, kv_heads, row_stride, causal, scale, s);
  if (head_dim == 64)
    return attn::launch_bwd<64>(qkv, out, dout, lse, delta, dqkv, dq_acc, batch, seq, heads, kv_heads, row_stride, causal, scale, s);
  set_error("flash: head_dim %d is not supported by the tensor-core kernel (64 and 128 are)", head_dim);
  return 2;
}
