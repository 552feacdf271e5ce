// FlashAttention forward for sm_100a: S = Q K^T and O += P V run on tcgen05 with S (double
// buffered) and O resident in tensor memory; K/V tiles arrive by TMA; two groups of four softmax
// warps each own one half of the 128 key columns of a tile (one query row per thread, online max /
// sum in registers, the row maximum of the two halves exchanged through shared memory), write P as
// packed bf16 back into the tensor-memory columns of the S buffer they have just read (the P V
// product takes its A operand from tensor memory, so P never touches shared memory) and rescale O
// in tensor memory only when a row's reference maximum has to move by more than 2^8. The two
// products of a step are issued by two different warps: issuing a tcgen05.mma holds the issuing
// thread for about as long as the product occupies the tensor pipe, so one issuer doing S(j + 1),
// then waiting for P(j), then P(j) V, would itself be the critical path of the loop.
//
// Inputs are the packed projection rows [B, T, (Hq + 2 Hkv) * hd] (q heads | k heads | v heads) after
// RoPE; query head h reads KV head h / (Hq / Hkv). Outputs: O [B, T, Hq * hd] (bf16) and the row
// log-sum-exp of the scaled scores, LSE [B, Hq, T] (fp32), which the backward kernels consume.
#include "common.cuh"

namespace ajb {
namespace attn {

constexpr int BLOCK_M = 128;  // queries per CTA
constexpr int BLOCK_N = 128;  // keys per step
constexpr int kThreads = 352;   // TMA warp, S-product issuer, 2 x 4 softmax warps, P V-product issuer
constexpr float kLog2e = 1.4426950408889634f;

template <int HD>
struct FwdCfg {
  static constexpr int kTileBytes = BLOCK_N * HD * 2;       // one Q, K or V tile
  static constexpr int kStages = HD == 128 ? 3 : 4;            // K/V ring
  static constexpr int kExchangeBytes = 2 * 2 * BLOCK_M * 4;   // [parity][column half][row] partial row maxima
  static constexpr int kSmemBytes = kTileBytes /*Q*/ + kStages * 2 * kTileBytes /*(K,V) ring*/ + kExchangeBytes + 256;
  static constexpr int kTmemCols = 512;
  static constexpr int kOCol = 256;  // S0 at 0, S1 at 128, O at 256
};

struct FwdParams {
  __nv_bfloat16* out;
  float* lse;
  int batch, seq, heads, kv_heads;
  int causal;
  float scale;
  DeviceStatus* status;
};

// Loads one [128 rows x HD] tile as HD/64 boxes of [128 x 64].
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int col, int row, int b) {
#pragma unroll
  for (int i = 0; i < HD / 64; ++i) tma_load_3d(dst + i * (BLOCK_N * 128), map, bar, col + 64 * i, row, b);
}

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_qkv, const FwdParams p) {
  using Cfg = FwdCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + Cfg::kTileBytes;               // stage s: K at sKV + s*2*tile, V right after
  constexpr int kStages = Cfg::kStages;
  float* sExchange = reinterpret_cast<float*>(sKV + kStages * 2 * Cfg::kTileBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sExchange + 2 * 2 * BLOCK_M);
  if (smem_misaligned(smem, p.status, kFlashFwd, reinterpret_cast<uint32_t*>(bars) + 60)) return;
  uint64_t* q_full = bars;            // 1
  uint64_t* kv_full = bars + 1;       // kStages (<= 4)
  uint64_t* kv_empty = bars + 5;      // kStages
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* p_ready = bars + 11;      // 1
  uint64_t* pv_done = bars + 12;      // 1
  uint64_t* pair_bar = bars + 13;     // 4: the two warps that share a 32-row quarter
  uint64_t* pv_issued = bars + 17;    // 2: P V of the tile in S buffer b has been handed to the tensor pipe
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;  // heavy (late) tiles first
  const int head = blockIdx.y, b = blockIdx.z;
  const int kv_head = head / (p.heads / p.kv_heads);
  const int q0 = q_tile * BLOCK_M;
  const int q_col = head * HD;
  const int k_col = (p.heads + kv_head) * HD;
  const int v_col = (p.heads + p.kv_heads + kv_head) * HD;
  const int kv_limit = p.causal ? min(p.seq, q0 + BLOCK_M) : p.seq;
  const int n_tiles = (kv_limit + BLOCK_N - 1) / BLOCK_N;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&pv_issued[0], 1);
    mbar_init(&pv_issued[1], 1);
    for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 2);
    mbar_init(p_ready, 8);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_qkv);
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
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, Cfg::kTileBytes);
      load_tile<HD>(sQ, &map_qkv, q_full, q_col, q0, b);
      int s = 0;
      uint32_t phase = 0;
      for (int j = 0; j < n_tiles; ++j) {
        if (!mbar_wait(&kv_empty[s], phase ^ 1, abort_flag, p.status, kFlashFwd, 1)) break;
        uint8_t* sK = sKV + s * 2 * Cfg::kTileBytes;
        mbar_arrive_expect_tx(&kv_full[s], 2 * Cfg::kTileBytes);
        load_tile<HD>(sK, &map_qkv, &kv_full[s], k_col, j * BLOCK_N, b);
        load_tile<HD>(sK + Cfg::kTileBytes, &map_qkv, &kv_full[s], v_col, j * BLOCK_N, b);
        if (++s == kStages) { s = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // ---- S(j) = Q K(j)^T into S buffer j & 1
    constexpr uint32_t idesc_s = make_idesc(BLOCK_M, BLOCK_N, 1, false, false);
    // descriptor low words; a k-step is a compile-time offset added to one of these (see common.cuh)
    const uint32_t q_km = desc_lo_k_major(smem_u32(sQ));
    const uint32_t k_km0 = desc_lo_k_major(smem_u32(sKV));
    constexpr uint32_t kStageStep = (2 * Cfg::kTileBytes) >> 4;
    bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kFlashFwd, 2);
    int stage = 0;
    uint32_t phase = 0;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!mbar_wait(&kv_full[stage], phase, abort_flag, p.status, kFlashFwd, 3)) break;
      // S buffer j & 1 still holds P(j - 2) until the product P(j - 2) V has been issued: the tensor pipe
      // executes in issue order, so being issued first is enough
      if (!mbar_wait(&pv_issued[j & 1], (((uint32_t)j >> 1) & 1) ^ 1, abort_flag, p.status, kFlashFwd, 4)) break;
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t k_km = k_km0 + (uint32_t)stage * kStageStep;
        const uint32_t d = tmem_base + (uint32_t)((j & 1) * BLOCK_N);
        umma_f16_c<false>(d, desc_at(q_km, 0), desc_at(k_km, 0), idesc_s);
#pragma unroll
        for (int k = 1; k < HD / 16; ++k)
          umma_f16_c<true>(d, desc_at(q_km, k_major_step(k, BLOCK_M * 128)), desc_at(k_km, k_major_step(k, BLOCK_N * 128)), idesc_s);
        tc_commit(&s_full[j & 1]);
      }
      __syncwarp();
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }
  } else if (warp == 10) {
    // ---- O += P(j) V(j): P from tensor memory (keys 0..63 in columns [0, 32) of S buffer j & 1, 64..127 in [64, 96))
    constexpr uint32_t idesc_o = make_idesc(BLOCK_M, HD, 1, false, true);
    const uint32_t v_mn0 = desc_lo_mn_major(smem_u32(sKV) + Cfg::kTileBytes, BLOCK_N * 128);
    constexpr uint32_t kStageStep = (2 * Cfg::kTileBytes) >> 4;
    int stage = 0;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(p_ready, (uint32_t)j & 1, abort_flag, p.status, kFlashFwd, 5)) break;
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t v_mn = v_mn0 + (uint32_t)stage * kStageStep;
        const uint32_t p_base = tmem_base + (uint32_t)((j & 1) * BLOCK_N);
        umma_f16_ts(tmem_base + Cfg::kOCol, p_base, desc_at(v_mn, 0), idesc_o, j != 0);
#pragma unroll
        for (int k = 1; k < BLOCK_N / 16; ++k)
          umma_f16_ts_c<true>(tmem_base + Cfg::kOCol, p_base + (uint32_t)(k < 4 ? k * 8 : 64 + (k - 4) * 8),
                              desc_at(v_mn, mn_major_step(k)), idesc_o);
        tc_commit(pv_done);
        tc_commit(&kv_empty[stage]);
        mbar_arrive(&pv_issued[j & 1]);
      }
      __syncwarp();
      if (++stage == kStages) stage = 0;
    }
  } else {
    // ---------------------------------------------------------------- softmax / correction / epilogue
    const int quarter = warp & 3;
    const int wg = (warp - 2) >> 2;               // which half of the key columns this warp handles (warps 2..9)
    const int col_base = wg * 64;
    const int row = quarter * 32 + lane;          // row of the tile == TMEM lane
    const int q_pos = q0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl = p.scale * kLog2e;
    float m_run = -INFINITY, l_run = 0.0f;        // l_run: sum over this warp group's columns only
    bool ok = true;
    // exchange one float per row with the warp that holds the other column half (bounded, like every wait)
    auto exchange = [&](uint32_t phase, float mine, float& theirs) -> bool {
      float* slot = sExchange + (phase & 1) * 2 * BLOCK_M;
      slot[wg * BLOCK_M + row] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(&pair_bar[quarter]);
      if (!mbar_wait(&pair_bar[quarter], phase & 1, abort_flag, p.status, kFlashFwd, 9)) return false;
      theirs = slot[(wg ^ 1) * BLOCK_M + row];
      return true;
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait(&s_full[s], ((uint32_t)j >> 1) & 1, abort_flag, p.status, kFlashFwd, 6)) { ok = false; break; }
      tc_fence_after_sync();
      const int k0 = j * BLOCK_N + col_base;
      const bool need_mask = (p.causal && j * BLOCK_N + BLOCK_N > q0) || (j * BLOCK_N + BLOCK_N > p.seq);
      const int k_max = p.causal ? min(q_pos, p.seq - 1) : p.seq - 1;  // last visible key of this row
      // pass 1: row maximum over this group's 64 columns
      uint32_t sv[2][32];
      tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(s * BLOCK_N + col_base), sv[0]);
      tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(s * BLOCK_N + col_base + 32), sv[1]);
      tc_wait_ld();
      float m_loc = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float x = __uint_as_float(sv[c][i]);
            if (k0 + c * 32 + i > k_max) x = -INFINITY;
            sv[c][i] = __float_as_uint(x);
            m_loc = fmaxf(m_loc, x);
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) m_loc = fmaxf(m_loc, __uint_as_float(sv[c][i]));
        }
      }
      float m_other;
      if (!exchange((uint32_t)j, m_loc, m_other)) { ok = false; break; }
      const float m_tile = fmaxf(m_loc, m_other);
      // The reference point m_run of the exponentials only follows the true maximum when it would otherwise
      // fall behind by more than kLazyBits powers of two: exp2((s - m_run) * scale) then stays below 2^kLazyBits,
      // harmless in bf16 / fp32, and the rescaling of O in tensor memory (a round trip through registers, and
      // a wait for the previous P V product) becomes rare. The final O / l is exact either way. Both column
      // halves see the same m_tile, hence take the same decision.
      constexpr float kLazyBits = 8.0f;
      const bool moved = (m_tile - m_run) * sl > kLazyBits;       // first tile: m_run = -inf -> true
      const float m_new = moved ? m_tile : m_run;
      const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;   // fully masked row (only when q_pos >= seq)
      const float alpha = moved ? exp2f((m_run - m_safe) * sl) : 1.0f;   // m_run = -inf -> 0
      const float neg = -m_safe * sl;
      float l_tile = 0.0f;
      // pass 2: probabilities, packed to bf16
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = exp2f(fmaf(__uint_as_float(sv[c][i]), sl, neg));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[c][i + 1]), sl, neg));
          l_tile += p0 + p1;
          pk[c * 16 + i / 2] = pack_bf16x2(p0, p1);
        }
      }
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      // P(j) overwrites the first half of the S(j) columns this warp has just read (64 keys -> 32 columns)
      tmem_st_32x32(tmem_base + lane_addr + (uint32_t)(s * BLOCK_N + col_base), pk);
      // rescale O when some row of this warp moved its reference point (each group takes half of the head
      // dimension); O belongs to the previous P V product until that has completed
      if (j > 0 && __any_sync(0xffffffffu, moved)) {
        if (!mbar_wait(pv_done, (uint32_t)(j - 1) & 1, abort_flag, p.status, kFlashFwd, 7)) { ok = false; break; }
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = wg * (HD / 64); c < (wg + 1) * (HD / 64); ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kOCol + c * 32), ov);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kOCol + c * 32), ov);
        }
      }
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    // epilogue: O / l -> global (each group stores half of the head dimension), LSE
    float l_other = 0.0f;
    if (ok && n_tiles > 0) ok = exchange((uint32_t)n_tiles, l_run, l_other);
    if (ok && n_tiles > 0 && mbar_wait(pv_done, (uint32_t)(n_tiles - 1) & 1, abort_flag, p.status, kFlashFwd, 8)) {
      tc_fence_after_sync();
      const float l_all = l_run + l_other;
      const float inv_l = l_all > 0.0f ? 1.0f / l_all : 0.0f;
      const bool row_ok = q_pos < p.seq;
      __nv_bfloat16* dst = p.out + ((size_t)b * p.seq + q_pos) * ((size_t)p.heads * HD) + (size_t)head * HD;
#pragma unroll 1
      for (int c = wg * (HD / 64); c < (wg + 1) * (HD / 64); ++c) {
        uint32_t ov[32];
        tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(Cfg::kOCol + c * 32), ov);
        tc_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(ov[8 * i]) * inv_l, __uint_as_float(ov[8 * i + 1]) * inv_l);
            q.y = pack_bf16x2(__uint_as_float(ov[8 * i + 2]) * inv_l, __uint_as_float(ov[8 * i + 3]) * inv_l);
            q.z = pack_bf16x2(__uint_as_float(ov[8 * i + 4]) * inv_l, __uint_as_float(ov[8 * i + 5]) * inv_l);
            q.w = pack_bf16x2(__uint_as_float(ov[8 * i + 6]) * inv_l, __uint_as_float(ov[8 * i + 7]) * inv_l);
            reinterpret_cast<uint4*>(dst + c * 32)[i] = q;
          }
        }
      }
      if (row_ok && wg == 0) {
        p.lse[((size_t)b * p.heads + head) * p.seq + q_pos] =
            (l_all > 0.0f) ? m_run * p.scale + __logf(l_all) : -INFINITY;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int HD>
static int launch_fwd(const void* qkv, void* out, void* lse, int batch, int seq, int heads, int kv_heads,
                      long long row_stride, int causal, float scale, cudaStream_t stream) {
  using Cfg = FwdCfg<HD>;
  CUtensorMap map;
  int rc = make_tensor_map_3d(&map, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, batch, seq, row_stride,
                              (uint64_t)seq * row_stride * 2, row_stride * 2, BLOCK_N, 64);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    AJB_CUDA_OK(cudaFuncSetAttribute(flash_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  FwdParams p;
  p.out = (__nv_bfloat16*)out; p.lse = (float*)lse; p.batch = batch; p.seq = seq; p.heads = heads;
  p.kv_heads = kv_heads; p.causal = causal; p.scale = scale; p.status = device_status_buffer();
  dim3 grid((seq + BLOCK_M - 1) / BLOCK_M, heads, batch);
  flash_fwd_kernel<HD><<<grid, kThreads, Cfg::kSmemBytes, stream>>>(map, p);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace attn
}  // namespace ajb

// qkv: packed [batch, seq, row_stride] bf16 with q heads first, then k heads, then v heads.
extern "C" int ajb_flash_fwd(const void* qkv, void* out, void* lse, int batch, int seq, int heads, int kv_heads,
                             int head_dim, long long row_stride, int causal, float scale, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(heads % kv_heads == 0, "flash: kv_heads must divide heads");
  AJB_REQUIRE(row_stride % 8 == 0, "flash: row stride must be a multiple of 8 elements");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (head_dim == 128) return attn::launch_fwd<128>(qkv, out, lse, batch, seq, heads, kv_heads, row_stride, causal, scale, s);
  if (head_dim == 64) return attn::launch_fwd<64>(qkv, out, lse, batch, seq, heads, kv_heads, row_stride, causal, scale, s);
  set_error("flash: head_dim %d is not supported by the tensor-core kernel (64 and 128 are)", head_dim);
  return 2;
}
