// Paged-KV attention for decoding and speculative verification on sm_100a.
//
// One CTA serves one (sequence, KV head): the `group * q_len` query rows that share this KV head
// (group = Hq / Hkv query heads, q_len new tokens: 1 for plain decoding, k + 1 when verifying k draft
// tokens) form the top rows of a 128-row tcgen05 tile, so every K/V byte of the sequence is read once
// for all of them. K/V tiles of 64 tokens are assembled from the sequence's 16-token cache blocks by
// TMA (one box per block, addressed through the block table); S = Q K^T and O += P V run on the tensor
// cores with accumulators in tensor memory, exactly as in the training forward kernel, but only the
// softmax warps whose 32-row quarter holds real rows do any work. Row (head h, new token i) may see
// keys 0 .. context_len - q_len + i.
//
// The kernel streams the cache once and does little arithmetic per byte, so what matters is how many bytes are in
// flight per SM. A step (wait for the tile, one product, a softmax over it, a second product) is a dependent chain
// of a couple of microseconds; one CTA per SM with two 128-key stages kept about one tile in flight and reached 0.4
// of the copy bandwidth. Tiles of 64 keys halve the shared memory of a CTA (113 KB) and its tensor memory (256
// columns), so two CTAs share an SM and each one's chain hides behind the other's loads.
//
// Plain decoding has 4 to 8 real rows, all in the first quarter, and one warp would do the softmax of
// all key columns of a tile while three idle. With at most 32 rows (REPL) the query rows are therefore staged
// four times, once per 32-lane quarter: the score tile then holds four identical copies, and warp q
// works on key columns [16 q, 16 q + 16) of its own copy. The four partial row maxima (and at the end the
// partial row sums) are exchanged through shared memory; P is assembled in rows 0..31 of the operand
// tile, so only the first quarter of O is meaningful and the first warp alone rescales and stores it.
//
// Long contexts at small batch: with `splits` > 1 the tiles of a sequence are divided over `splits` CTAs (grid z).
// Each writes its un-normalised fp32 output rows and (reference maximum, row sum) to a workspace, and a second small
// kernel merges the parts with the usual log-sum-exp weights. One CTA per (sequence, KV head) walks a 4k context as
// 32 dependent tile steps while most SMs idle; eight CTAs walk four steps each.
//
// Layouts: q [tokens, Hq, hd] bf16 (rows of a sequence are contiguous, `q_start[seq]` is its first
// row); caches [num_blocks, block_size = 16, Hkv, hd] bf16; block_tables [num_seqs, max_blocks] int32;
// out like q.
#include "common.cuh"

namespace ajb {
namespace paged {

constexpr int TILE = 64;           // keys per step
constexpr int QROWS = 128;         // rows of the query / probability operand tiles (the MMA's M)
constexpr int BLOCK_TOKENS = 16;   // tokens per cache block
constexpr int kThreads = 192;
constexpr int kMaxRows = 64;       // group * q_len
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kPagedKernelId = 5;

template <int HD>
struct Cfg {
  static constexpr int kQ = QROWS * HD * 2;          // the query rows, staged once
  static constexpr int kTile = TILE * HD * 2;        // one K or V tile
  static constexpr int kP = QROWS * TILE * 2;        // probabilities of one step (A operand of P V)
  // [parity][quarter][row] partial maxima / sums of the REPL variant live in rows 64.. of the P tile: with at most 32
  // real rows those operand rows only feed accumulator rows that nobody reads
  static constexpr int kExchangeOffset = 64 * 128;
  static constexpr int kSmem = kQ + 4 * kTile /*2 x (K,V)*/ + kP + 256;
  static constexpr int kOCol = 2 * TILE;             // S0 at 0, S1 at TILE, O behind them
  static constexpr int kTmemCols = 256;              // 2 * 64 + HD <= 256: two CTAs fit the SM's 512 columns
};

struct Params {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int* block_tables;
  const int* context_lens;
  const int* q_start;
  int max_blocks;
  int heads, kv_heads, q_len;
  float scale;
  int splits;                 // CTAs per (sequence, KV head); > 1: partial results go to the workspace
  float* part_o;              // [tokens, Hq, splits, hd] fp32, un-normalised
  float2* part_ml;            // [tokens, Hq, splits] (reference maximum in log2 units, row sum); sum 0 = no keys seen
  DeviceStatus* status;
};

// 16-byte chunk `ch` of row `row` of a K-major operand tile of QROWS rows (128-byte swizzle, 64-element boxes).
__device__ __forceinline__ void store_chunk(uint8_t* tile, int row, int ch, uint4 val) {
  uint8_t* dst = tile + (ch >> 3) * (QROWS * 128) + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
  *reinterpret_cast<uint4*>(dst) = val;
}

template <int HD, bool REPL>
__global__ void __launch_bounds__(kThreads, 2)
paged_attention_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const Params p) {
  using C = Cfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + C::kQ;
  uint8_t* sP = sKV + 4 * C::kTile;
  float* sExchange = reinterpret_cast<float*>(sP + C::kExchangeOffset);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::kP);
  if (smem_misaligned(smem, p.status, kPagedKernelId, reinterpret_cast<uint32_t*>(bars) + 60)) return;
  uint64_t* kv_full = bars;        // 2
  uint64_t* kv_empty = bars + 2;   // 2
  uint64_t* s_full = bars + 4;     // 2
  uint64_t* s_free = bars + 6;     // 2
  uint64_t* p_ready = bars + 8;    // 1
  uint64_t* pv_done = bars + 9;    // 1
  uint64_t* xbar = bars + 10;      // 1 (REPL: the four softmax warps exchange partial maxima / sums)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.x, kv_head = blockIdx.y;
  const int group = p.heads / p.kv_heads;
  const int rows = group * p.q_len;                 // real rows, packed head-major: row = h_in_group * q_len + i
  const int ctx = p.context_lens[seq];
  const int all_tiles = (ctx + TILE - 1) / TILE;
  // this CTA's share of the sequence's tiles: [t0, t0 + n_tiles)
  const int per_split = (all_tiles + p.splits - 1) / p.splits;
  const int t0 = min(all_tiles, (int)blockIdx.z * per_split);
  const int n_tiles = min(all_tiles - t0, per_split);
  const int active_quarters = (rows + 31) / 32;
  const int* table = p.block_tables + (size_t)seq * p.max_blocks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
    }
    mbar_init(p_ready, 4);
    mbar_init(pv_done, 1);
    mbar_init(xbar, 4);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_k);
    prefetch_tensor_map(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  // stage Q: rows beyond `rows` are zero (their scores are never used)
  if (warp >= 2) {
    const int t = threadIdx.x - 64;                 // 0..127 == tile row
    const int qr = REPL ? (t & 31) : t;             // REPL: every quarter holds a copy of the query rows
    const bool real = qr < rows;
    const int h = real ? qr / p.q_len : 0, i = real ? qr % p.q_len : 0;
    const __nv_bfloat16* src = p.q + ((size_t)(p.q_start[seq] + i) * p.heads + kv_head * group + h) * HD;
#pragma unroll
    for (int ch = 0; ch < HD / 8; ++ch) {
      const uint4 v = real ? reinterpret_cast<const uint4*>(src)[ch] : make_uint4(0, 0, 0, 0);
      store_chunk(sQ, t, ch, v);
    }
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], (((uint32_t)j >> 1) & 1) ^ 1, abort_flag, p.status, kPagedKernelId, 1)) break;
        uint8_t* sK = sKV + s * 2 * C::kTile;
        uint8_t* sV = sK + C::kTile;
        mbar_arrive_expect_tx(&kv_full[s], 2 * C::kTile);
        const int first_block = (t0 + j) * (TILE / BLOCK_TOKENS);
        const int blocks_here = min(TILE / BLOCK_TOKENS, (ctx + BLOCK_TOKENS - 1) / BLOCK_TOKENS - first_block);
#pragma unroll 1
        for (int b = 0; b < TILE / BLOCK_TOKENS; ++b) {
          // blocks past the end of the sequence re-read the last valid block (masked later); keeps the byte count fixed
          const int id = table[first_block + min(b, blocks_here - 1)];
#pragma unroll
          for (int i = 0; i < HD / 64; ++i) {
            tma_load_3d(sK + i * (TILE * 128) + b * (BLOCK_TOKENS * 128), &map_k, &kv_full[s], kv_head * HD + 64 * i, 0, id);
            tma_load_3d(sV + i * (TILE * 128) + b * (BLOCK_TOKENS * 128), &map_v, &kv_full[s], kv_head * HD + 64 * i, 0, id);
          }
        }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_s = make_idesc(QROWS, TILE, 1, false, false);
    constexpr uint32_t idesc_o = make_idesc(QROWS, HD, 1, false, true);
    // descriptor low words; a k-step is a compile-time offset added to one of these (see common.cuh)
    const uint32_t q_km = desc_lo_k_major(smem_u32(sQ)), p_km = desc_lo_k_major(smem_u32(sP));
    const uint32_t k_km0 = desc_lo_k_major(smem_u32(sKV));
    const uint32_t v_mn0 = desc_lo_mn_major(smem_u32(sKV) + C::kTile, TILE * 128);
    constexpr uint32_t kStageStep = (2 * C::kTile) >> 4;
    bool ok = true;
    auto issue_s = [&](int j) -> bool {
      const int s = j & 1;
      const uint32_t use = (uint32_t)j >> 1;
      if (!mbar_wait(&kv_full[s], use & 1, abort_flag, p.status, kPagedKernelId, 3)) return false;
      if (!mbar_wait(&s_free[s], (use & 1) ^ 1, abort_flag, p.status, kPagedKernelId, 4)) return false;
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t k_km = k_km0 + (uint32_t)s * kStageStep;
        const uint32_t d = tmem_base + (uint32_t)(s * TILE);
        umma_f16_c<false>(d, desc_at(q_km, 0), desc_at(k_km, 0), idesc_s);
#pragma unroll
        for (int k = 1; k < HD / 16; ++k)
          umma_f16_c<true>(d, desc_at(q_km, k_major_step(k, QROWS * 128)), desc_at(k_km, k_major_step(k, TILE * 128)), idesc_s);
        tc_commit(&s_full[s]);
      }
      __syncwarp();
      return true;
    };
    if (n_tiles > 0) ok = issue_s(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (j + 1 < n_tiles) {
        ok = issue_s(j + 1);
        if (!ok) break;
      }
      if (!mbar_wait(p_ready, (uint32_t)j & 1, abort_flag, p.status, kPagedKernelId, 5)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t v_mn = v_mn0 + (uint32_t)(j & 1) * kStageStep;
        umma_f16(tmem_base + C::kOCol, desc_at(p_km, 0), desc_at(v_mn, 0), idesc_o, j != 0);
#pragma unroll
        for (int k = 1; k < TILE / 16; ++k)
          umma_f16_c<true>(tmem_base + C::kOCol, desc_at(p_km, k_major_step(k, QROWS * 128)), desc_at(v_mn, mn_major_step(k)), idesc_o);
        tc_commit(pv_done);
        tc_commit(&kv_empty[j & 1]);
      }
      __syncwarp();
    }
  } else if (REPL) {
    // ---- at most 32 query rows, copied into every quarter: warp q handles key columns [16 q, 16 q + 16)
    const int quarter = warp & 3;
    const bool real = lane < rows;
    const int h = real ? lane / p.q_len : 0, qi = real ? lane % p.q_len : 0;
    const int k_max = real ? ctx - p.q_len + qi : -1;   // last visible key
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl = p.scale * kLog2e;
    float m_run = -INFINITY, l_run = 0.0f;              // l_run: this warp's 16 columns of every tile only
    bool ok = true;
    // publishes `mine`, waits (bounded) for the other three warps, returns all four values of this row
    auto exchange = [&](uint32_t phase, float mine, float (&all)[4]) -> bool {
      float* slot = sExchange + (phase & 1) * 128;
      slot[quarter * 32 + lane] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(xbar);
      if (!mbar_wait(xbar, phase & 1, abort_flag, p.status, kPagedKernelId, 9)) return false;
#pragma unroll
      for (int q = 0; q < 4; ++q) all[q] = slot[q * 32 + lane];
      return true;
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait(&s_full[s], ((uint32_t)j >> 1) & 1, abort_flag, p.status, kPagedKernelId, 6)) { ok = false; break; }
      tc_fence_after_sync();
      const int k0 = (t0 + j) * TILE + quarter * 16;
      uint32_t sv[16];
      tmem_ld_32x16(tmem_base + lane_addr + (uint32_t)(s * TILE + quarter * 16), sv);
      tc_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[s]);
      float m_loc = -INFINITY;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float x = __uint_as_float(sv[i]);
        if (k0 + i > k_max) x = -INFINITY;
        sv[i] = __float_as_uint(x);
        m_loc = fmaxf(m_loc, x);
      }
      float part[4];
      if (!exchange((uint32_t)j, m_loc, part)) { ok = false; break; }
      const float m_tile = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
      // lazy reference maximum (see flash_fwd.cu); every warp sees the same m_tile and decides alike
      const bool moved = (m_tile - m_run) * sl > 8.0f;
      const float m_new = moved ? m_tile : m_run;
      const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = moved ? exp2f((m_run - m_safe) * sl) : 1.0f;
      const float neg = -m_safe * sl;
      float l_tile = 0.0f;
      uint32_t pk[8];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        const float p0 = exp2f(fmaf(__uint_as_float(sv[i]), sl, neg));
        const float p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), sl, neg));
        l_tile += p0 + p1;
        pk[i / 2] = pack_bf16x2(p0, p1);
      }
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      if (j > 0 && !mbar_wait(pv_done, (uint32_t)(j - 1) & 1, abort_flag, p.status, kPagedKernelId, 7)) { ok = false; break; }
      tc_fence_after_sync();
      // P row `lane`, key columns of this warp: rows 32..127 of the operand tile are never read back
#pragma unroll
      for (int ch = 0; ch < 2; ++ch)
        store_chunk(sP, lane, quarter * 2 + ch, make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]));
      if (quarter == 0 && j > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(tmem_base + (uint32_t)(C::kOCol + c * 32), ov);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st_32x32(tmem_base + (uint32_t)(C::kOCol + c * 32), ov);
        }
        tc_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    float sums[4] = {0.f, 0.f, 0.f, 0.f};
    if (ok && n_tiles > 0) ok = exchange((uint32_t)n_tiles, l_run, sums);
    const size_t out_row = (size_t)(p.q_start[seq] + qi) * p.heads + kv_head * group + h;
    if (p.splits > 1 && quarter == 0 && real && (n_tiles == 0 || !ok))
      p.part_ml[out_row * p.splits + blockIdx.z] = make_float2(0.0f, 0.0f);        // nothing to merge from this part
    if (ok && quarter == 0 && n_tiles > 0 && mbar_wait(pv_done, (uint32_t)(n_tiles - 1) & 1, abort_flag, p.status, kPagedKernelId, 8)) {
      tc_fence_after_sync();
      const float l_all = (sums[0] + sums[1]) + (sums[2] + sums[3]);
      const float inv_l = l_all > 0.0f ? 1.0f / l_all : 0.0f;
      __nv_bfloat16* dst = p.out + out_row * HD;
      if (p.splits > 1) {
        if (real) p.part_ml[out_row * p.splits + blockIdx.z] = make_float2(m_run == -INFINITY ? 0.0f : m_run * sl, l_all);
        float* part = p.part_o + (out_row * p.splits + blockIdx.z) * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(tmem_base + (uint32_t)(C::kOCol + c * 32), ov);
          tc_wait_ld();
          if (real) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<uint4*>(part + c * 32)[i] = make_uint4(ov[4 * i], ov[4 * i + 1], ov[4 * i + 2], ov[4 * i + 3]);
          }
        }
      } else
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t ov[32];
        tmem_ld_32x32(tmem_base + (uint32_t)(C::kOCol + c * 32), ov);
        tc_wait_ld();
        if (real) {
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
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const bool active = quarter < active_quarters;     // warp-uniform
    const bool real = row < rows;
    const int h = real ? row / p.q_len : 0, qi = real ? row % p.q_len : 0;
    const int k_max = real ? ctx - p.q_len + qi : -1;   // last visible key
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl = p.scale * kLog2e;
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      if (!mbar_wait(&s_full[s], ((uint32_t)j >> 1) & 1, abort_flag, p.status, kPagedKernelId, 6)) { ok = false; break; }
      tc_fence_after_sync();
      const int k0 = (t0 + j) * TILE;
      uint32_t pk[TILE / 2];
      float alpha = 1.0f;
      bool moved = false;
      if (active) {
        uint32_t sv[TILE / 32][32];
#pragma unroll
        for (int c = 0; c < TILE / 32; ++c) tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(s * TILE + c * 32), sv[c]);
        tc_wait_ld();
        float m_tile = -INFINITY;
#pragma unroll
        for (int c = 0; c < TILE / 32; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float x = __uint_as_float(sv[c][i]);
            if (k0 + c * 32 + i > k_max) x = -INFINITY;
            sv[c][i] = __float_as_uint(x);
            m_tile = fmaxf(m_tile, x);
          }
        }
        // lazy reference maximum (see flash_fwd.cu): O is rescaled only when a row would overflow 2^8
        moved = (m_tile - m_run) * sl > 8.0f;
        const float m_new = moved ? m_tile : m_run;
        const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
        alpha = moved ? exp2f((m_run - m_safe) * sl) : 1.0f;
        const float neg = -m_safe * sl;
        float l_tile = 0.0f;
#pragma unroll
        for (int c = 0; c < TILE / 32; ++c) {
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
      } else {
#pragma unroll
        for (int i = 0; i < TILE / 2; ++i) pk[i] = 0u;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[s]);
      if (j > 0 && !mbar_wait(pv_done, (uint32_t)(j - 1) & 1, abort_flag, p.status, kPagedKernelId, 7)) { ok = false; break; }
      tc_fence_after_sync();
      // inactive quarters write their (zero) rows only once: they never change
      if (active || j == 0) {
#pragma unroll
        for (int ch = 0; ch < TILE / 8; ++ch) store_chunk(sP, row, ch, make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]));
      }
      if (active && j > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(C::kOCol + c * 32), ov);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st_32x32(tmem_base + lane_addr + (uint32_t)(C::kOCol + c * 32), ov);
        }
        tc_wait_st();
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    const size_t out_row = (size_t)(p.q_start[seq] + qi) * p.heads + kv_head * group + h;
    if (p.splits > 1 && real && (n_tiles == 0 || !ok))
      p.part_ml[out_row * p.splits + blockIdx.z] = make_float2(0.0f, 0.0f);        // nothing to merge from this part
    if (ok && n_tiles > 0 && mbar_wait(pv_done, (uint32_t)(n_tiles - 1) & 1, abort_flag, p.status, kPagedKernelId, 8)) {
      tc_fence_after_sync();
      if (active && p.splits > 1) {
        if (real) p.part_ml[out_row * p.splits + blockIdx.z] = make_float2(m_run == -INFINITY ? 0.0f : m_run * sl, l_run);
        float* part = p.part_o + (out_row * p.splits + blockIdx.z) * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(C::kOCol + c * 32), ov);
          tc_wait_ld();
          if (real) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<uint4*>(part + c * 32)[i] = make_uint4(ov[4 * i], ov[4 * i + 1], ov[4 * i + 2], ov[4 * i + 3]);
          }
        }
      } else if (active) {
        const float inv_l = l_run > 0.0f ? 1.0f / l_run : 0.0f;
        __nv_bfloat16* dst = p.out + out_row * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(C::kOCol + c * 32), ov);
          tc_wait_ld();
          if (real) {
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
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// out[row, head, :] = sum_z w_z O_z / sum_z w_z l_z with w_z = 2^(m_z - max m): one warp per (row, head).
template <int HD>
__global__ void merge_splits_kernel(const float* __restrict__ part_o, const float2* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, const int* __restrict__ q_start, int q_len, int heads,
                                    int splits, long long pairs /* sequences * q_len * heads */) {
  const int lane = threadIdx.x & 31;
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (w >= pairs) return;
  const long long local_row = w / heads;
  const int head = (int)(w - local_row * heads);
  const int seq = (int)(local_row / q_len), i = (int)(local_row - (long long)seq * q_len);
  const size_t out_row = (size_t)(q_start[seq] + i) * heads + head;
  float m_max = -INFINITY;
  for (int z = 0; z < splits; ++z) {
    const float2 ml = part_ml[out_row * splits + z];
    if (ml.y > 0.0f) m_max = fmaxf(m_max, ml.x);
  }
  constexpr int kPerLane = HD / 32;
  float acc[kPerLane];
#pragma unroll
  for (int c = 0; c < kPerLane; ++c) acc[c] = 0.0f;
  float l_all = 0.0f;
  for (int z = 0; z < splits; ++z) {
    const float2 ml = part_ml[out_row * splits + z];
    if (!(ml.y > 0.0f)) continue;
    const float weight = exp2f(ml.x - m_max);
    l_all += weight * ml.y;
    const float* src = part_o + (out_row * splits + z) * HD;
#pragma unroll
    for (int c = 0; c < kPerLane; ++c) acc[c] += weight * src[c * 32 + lane];
  }
  const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
#pragma unroll
  for (int c = 0; c < kPerLane; ++c) out[out_row * HD + c * 32 + lane] = __float2bfloat16(acc[c] * inv);
}

template <int HD>
static int launch(const void* q, const void* k_cache, const void* v_cache, const void* block_tables,
                  const void* context_lens, const void* q_start, void* out, int num_seqs, int num_blocks, int max_blocks,
                  int heads, int kv_heads, int q_len, float scale, int splits, void* part_o, void* part_ml,
                  cudaStream_t stream) {
  using C = Cfg<HD>;
  CUtensorMap map_k, map_v;
  const uint64_t row_pitch = (uint64_t)kv_heads * HD * 2;
  int rc = make_tensor_map_3d(&map_k, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, num_blocks, BLOCK_TOKENS,
                              (uint64_t)kv_heads * HD, row_pitch * BLOCK_TOKENS, row_pitch, BLOCK_TOKENS, 64);
  if (rc) return rc;
  rc = make_tensor_map_3d(&map_v, v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, num_blocks, BLOCK_TOKENS,
                          (uint64_t)kv_heads * HD, row_pitch * BLOCK_TOKENS, row_pitch, BLOCK_TOKENS, 64);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    AJB_CUDA_OK(cudaFuncSetAttribute(paged_attention_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem));
    AJB_CUDA_OK(cudaFuncSetAttribute(paged_attention_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem));
    // two CTAs per SM need the whole shared-memory carve-out
    AJB_CUDA_OK(cudaFuncSetAttribute(paged_attention_kernel<HD, false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared));
    AJB_CUDA_OK(cudaFuncSetAttribute(paged_attention_kernel<HD, true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared));
    configured = true;
  }
  Params p;
  p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.block_tables = (const int*)block_tables;
  p.context_lens = (const int*)context_lens; p.q_start = (const int*)q_start; p.max_blocks = max_blocks;
  p.heads = heads; p.kv_heads = kv_heads; p.q_len = q_len; p.scale = scale; p.status = device_status_buffer();
  p.splits = splits; p.part_o = (float*)part_o; p.part_ml = (float2*)part_ml;
  if ((heads / kv_heads) * q_len <= 32)
    paged_attention_kernel<HD, true><<<dim3(num_seqs, kv_heads, splits), kThreads, C::kSmem, stream>>>(map_k, map_v, p);
  else
    paged_attention_kernel<HD, false><<<dim3(num_seqs, kv_heads, splits), kThreads, C::kSmem, stream>>>(map_k, map_v, p);
  AJB_CUDA_OK(cudaGetLastError());
  if (splits > 1) {
    const long long pairs = (long long)num_seqs * q_len * heads;
    const int threads = 128;
    const long long blocks = (pairs * 32 + threads - 1) / threads;
    merge_splits_kernel<HD><<<(unsigned)blocks, threads, 0, stream>>>((const float*)part_o, (const float2*)part_ml,
                                                                      (__nv_bfloat16*)out, (const int*)q_start, q_len, heads,
                                                                      splits, pairs);
    AJB_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

}  // namespace paged
}  // namespace ajb

// Every sequence of the launch contributes exactly q_len new rows; (heads / kv_heads) * q_len <= 64.
// splits > 1 divides every sequence's tiles over that many CTAs: part_o must hold rows * heads * splits * head_dim
// floats and part_ml rows * heads * splits * 2 floats, where rows = the total number of query rows of the batch.
extern "C" int ajb_paged_attention(const void* q, const void* k_cache, const void* v_cache, const void* block_tables,
                                   const void* context_lens, const void* q_start, void* out, int num_seqs,
                                   int num_blocks, int block_size, int max_blocks, int heads, int kv_heads,
                                   int head_dim, int q_len, float scale, int splits, void* part_o, void* part_ml,
                                   void* stream) {
  using namespace ajb;
  AJB_REQUIRE(splits >= 1 && splits <= 64 && (splits == 1 || (part_o != nullptr && part_ml != nullptr)),
              "paged attention: splits must be in [1, 64] and come with a workspace");
  AJB_REQUIRE(block_size == paged::BLOCK_TOKENS, "paged attention: cache block size must be %d", paged::BLOCK_TOKENS);
  AJB_REQUIRE(heads % kv_heads == 0 && (heads / kv_heads) * q_len <= paged::kMaxRows && q_len >= 1,
              "paged attention: (heads / kv_heads) * q_len = %d exceeds %d", (heads / kv_heads) * q_len, paged::kMaxRows);
  if (num_seqs <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (head_dim == 128)
    return paged::launch<128>(q, k_cache, v_cache, block_tables, context_lens, q_start, out, num_seqs, num_blocks,
                              max_blocks, heads, kv_heads, q_len, scale, splits, part_o, part_ml, s);
  if (head_dim == 64)
    return paged::launch<64>(q, k_cache, v_cache, block_tables, context_lens, q_start, out, num_seqs, num_blocks,
                             max_blocks, heads, kv_heads, q_len, scale, splits, part_o, part_ml, s);
  set_error("paged attention: head_dim %d is not supported (64 and 128 are)", head_dim);
  return 2;
}
