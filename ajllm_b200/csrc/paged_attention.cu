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
// In that variant the probability tile exists twice (only its first 32 rows matter, 4 KB each; the operand rows behind
// them may hold anything, they feed accumulator rows that nobody reads), so the softmax of tile j + 1 does not wait for
// the second product of tile j; and the partial maxima of tile j are exchanged while tile j + 1 is being computed:
// tile j is exponentiated against the reference maximum of the tiles before it (exact for the first tile), which is
// safe because bf16 and fp32 share the exponent range: the exponent is capped at 120, a cap that only a score jump of
// more than 80 natural units above everything seen before could reach.
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
constexpr int kReplTileBytes = 32 * 128;   // REPL variant: the 32 meaningful rows of a probability tile (64 keys x 2 bytes per row)

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
  // Q, P, the K/V ring, barriers. P sits in front of the ring: the second probability tile of the REPL variant starts
  // 4 KB into P and its (unused) operand rows reach into the ring, never past the end of the allocation
  uint8_t* sQ = smem;
  uint8_t* sP = sQ + C::kQ;
  uint8_t* sKV = sP + C::kP;
  float* sExchange = reinterpret_cast<float*>(sP + C::kExchangeOffset);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + 4 * C::kTile);
  if (smem_misaligned(smem, p.status, kPagedKernelId, reinterpret_cast<uint32_t*>(bars) + 60)) return;
  // K and V tiles have their own barriers: a K tile is free again after the first product of its step, long before
  // the V tile of the same step, and the issuing warp must never find the next K tile missing when it gets there
  uint64_t* k_full = bars;         // 2
  uint64_t* k_empty = bars + 2;    // 2
  uint64_t* v_full = bars + 4;     // 2
  uint64_t* v_empty = bars + 6;    // 2
  uint64_t* s_full = bars + 8;     // 2
  uint64_t* s_free = bars + 10;    // 2
  uint64_t* p_ready = bars + 12;   // 2 (REPL: one per probability tile; otherwise only the first)
  uint64_t* pv_done = bars + 14;   // 2 (likewise)
  uint64_t* xbar = bars + 16;      // 1 (REPL: the four softmax warps exchange partial maxima / sums)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
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
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
      mbar_init(&p_ready[i], 4);
      mbar_init(&pv_done[i], 1);
    }
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
    // Producer. The block ids of eight tiles (32 blocks) are fetched by the 32 lanes with one coalesced load, a group
    // ahead of their use, and handed to the issuing lane by shuffles: a dependent table lookup per block in front of
    // its copies would cost more than the copies themselves.
    constexpr int kBlocksPerTile = TILE / BLOCK_TOKENS;
    constexpr int kTilesPerGroup = 32 / kBlocksPerTile;
    const int last_block = (ctx + BLOCK_TOKENS - 1) / BLOCK_TOKENS - 1;
    // blocks past the end of the sequence re-read the last valid block (masked later); keeps the byte count fixed
    auto fetch_ids = [&](int group) { return table[max(0, min(last_block, (t0 + group * kTilesPerGroup) * kBlocksPerTile + lane))]; };
    int ids_next = n_tiles > 0 ? fetch_ids(0) : 0;
    bool ok = true;
    // K tiles run one step ahead of V tiles: K(j + 1) goes out as soon as the first product of step j - 1 has read
    // its slot, V(j) when the second product of step j - 2 has
    int ids_k = ids_next, ids_prev = ids_next;      // block ids of K's group of tiles and of the group before it
    int k_group = -1;
    for (int j = 0; j <= n_tiles && ok; ++j) {
      if (j < n_tiles) {
        if (j % kTilesPerGroup == 0) {
          ids_prev = ids_k;
          ids_k = ids_next;
          k_group = j / kTilesPerGroup;
          if (j + kTilesPerGroup < n_tiles) ids_next = fetch_ids(k_group + 1);
        }
        const int s = j & 1;
        int id[kBlocksPerTile];
#pragma unroll
        for (int b = 0; b < kBlocksPerTile; ++b) id[b] = __shfl_sync(0xffffffffu, ids_k, (j % kTilesPerGroup) * kBlocksPerTile + b);
        if (lane == 0) {
          ok = mbar_wait(&k_empty[s], (((uint32_t)j >> 1) & 1) ^ 1, abort_flag, p.status, kPagedKernelId, 1);
          if (ok) {
            uint8_t* sK = sKV + s * 2 * C::kTile;
            mbar_arrive_expect_tx(&k_full[s], C::kTile);
#pragma unroll
            for (int b = 0; b < kBlocksPerTile; ++b) {
#pragma unroll
              for (int i = 0; i < HD / 64; ++i)
                tma_load_3d(sK + i * (TILE * 128) + b * (BLOCK_TOKENS * 128), &map_k, &k_full[s], kv_head * HD + 64 * i, 0, id[b]);
            }
          }
        }
      }
      if (j >= 1) {
        const int jv = j - 1;
        const int ids_v = (jv / kTilesPerGroup == k_group) ? ids_k : ids_prev;     // V is one step behind K
        const int s = jv & 1;
        int id[kBlocksPerTile];
#pragma unroll
        for (int b = 0; b < kBlocksPerTile; ++b) id[b] = __shfl_sync(0xffffffffu, ids_v, (jv % kTilesPerGroup) * kBlocksPerTile + b);
        if (lane == 0 && ok) {
          ok = mbar_wait(&v_empty[s], (((uint32_t)jv >> 1) & 1) ^ 1, abort_flag, p.status, kPagedKernelId, 2);
          if (ok) {
            uint8_t* sV = sKV + s * 2 * C::kTile + C::kTile;
            mbar_arrive_expect_tx(&v_full[s], C::kTile);
#pragma unroll
            for (int b = 0; b < kBlocksPerTile; ++b) {
#pragma unroll
              for (int i = 0; i < HD / 64; ++i)
                tma_load_3d(sV + i * (TILE * 128) + b * (BLOCK_TOKENS * 128), &map_v, &v_full[s], kv_head * HD + 64 * i, 0, id[b]);
            }
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
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
      if (!mbar_wait(&k_full[s], use & 1, abort_flag, p.status, kPagedKernelId, 3)) return false;
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
        tc_commit(&k_empty[s]);
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
      // REPL: probability tile j & 1 (4 KB apart), its barriers complete every other tile
      const int pb = REPL ? (j & 1) : 0;
      const uint32_t p_phase = REPL ? (((uint32_t)j >> 1) & 1) : ((uint32_t)j & 1);
      if (!mbar_wait(&p_ready[pb], p_phase, abort_flag, p.status, kPagedKernelId, 5)) { ok = false; break; }
      if (!mbar_wait(&v_full[j & 1], ((uint32_t)j >> 1) & 1, abort_flag, p.status, kPagedKernelId, 10)) { ok = false; break; }
      tc_fence_after_sync();
      if (lane == 0) {
        const uint32_t v_mn = v_mn0 + (uint32_t)(j & 1) * kStageStep;
        const uint32_t p_lo = p_km + (uint32_t)pb * (uint32_t)(kReplTileBytes >> 4);
        umma_f16(tmem_base + C::kOCol, desc_at(p_lo, 0), desc_at(v_mn, 0), idesc_o, j != 0);
#pragma unroll
        for (int k = 1; k < TILE / 16; ++k)
          umma_f16_c<true>(tmem_base + C::kOCol, desc_at(p_lo, k_major_step(k, QROWS * 128)), desc_at(v_mn, mn_major_step(k)), idesc_o);
        tc_commit(&pv_done[pb]);
        tc_commit(&v_empty[j & 1]);
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
    // The four warps exchange a value per row through a ring of four slots: `publish` writes this warp's value of
    // exchange number `x` and arrives, `collect` waits (bounded) until all four have arrived for `x` and reads them.
    // A warp collects exchange x before it publishes x + 1, so the barrier never runs two phases ahead of a waiter,
    // and no warp can be four exchanges ahead of another (S tiles are handed back by all four warps).
    auto publish = [&](uint32_t x, float mine) {
      sExchange[(x & 3) * 128 + quarter * 32 + lane] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(xbar);
    };
    auto collect = [&](uint32_t x, float (&all)[4]) -> bool {
      if (!mbar_wait(xbar, x & 1, abort_flag, p.status, kPagedKernelId, 9)) return false;
#pragma unroll
      for (int q = 0; q < 4; ++q) all[q] = sExchange[(x & 3) * 128 + q * 32 + lane];
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
      // reference maximum: the first tile waits for its own maxima; tile j > 0 takes those of tile j - 1, which were
      // published a whole tile ago, and publishes its own for tile j + 1
      float part[4];
      if (j == 0) {
        publish(0u, m_loc);
        if (!collect(0u, part)) { ok = false; break; }
      } else {
        if (!collect((uint32_t)(j - 1), part)) { ok = false; break; }
        publish((uint32_t)j, m_loc);
      }
      const float m_seen = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
      // lazy reference maximum (see flash_fwd.cu); every warp sees the same m_seen and decides alike
      const bool moved = (m_seen - m_run) * sl > 8.0f;
      const float m_new = moved ? m_seen : m_run;
      const float m_safe = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = moved ? exp2f((m_run - m_safe) * sl) : 1.0f;
      const float neg = -m_safe * sl;
      float l_tile = 0.0f;
      uint32_t pk[8];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        // keys of this tile may exceed the reference of the tiles before it: the exponent is capped below overflow
        const float p0 = exp2f(fminf(fmaf(__uint_as_float(sv[i]), sl, neg), 120.0f));
        const float p1 = exp2f(fminf(fmaf(__uint_as_float(sv[i + 1]), sl, neg), 120.0f));
        l_tile += p0 + p1;
        pk[i / 2] = pack_bf16x2(p0, p1);
      }
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      // probability tile j & 1 was last read by the second product of tile j - 2
      const int pb = j & 1;
      if (j > 1 && !mbar_wait(&pv_done[pb], (((uint32_t)(j - 2)) >> 1) & 1, abort_flag, p.status, kPagedKernelId, 7)) { ok = false; break; }
      // P row `lane`, key columns of this warp
      uint8_t* tile_p = sP + pb * kReplTileBytes;
#pragma unroll
      for (int ch = 0; ch < 2; ++ch)
        store_chunk(tile_p, lane, quarter * 2 + ch, make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]));
      if (j > 0 && __any_sync(0xffffffffu, moved)) {
        // O changes scale: every product up to tile j - 1 must have landed first (all warps wait, so that none
        // announces its part of P before the rescaled O is in place ... the first warp rescales)
        if (!mbar_wait(&pv_done[(j - 1) & 1], (((uint32_t)(j - 1)) >> 1) & 1, abort_flag, p.status, kPagedKernelId, 7)) { ok = false; break; }
        tc_fence_after_sync();
        if (quarter == 0) {
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
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[pb]);
    }
    float sums[4] = {0.f, 0.f, 0.f, 0.f};
    if (ok && n_tiles > 0) {
      // exchange n_tiles - 1 (the last tile's maxima) is collected first to keep the order, then the sums go round
      float unused[4];
      if (n_tiles > 1) ok = collect((uint32_t)(n_tiles - 1), unused);
      if (ok) {
        publish((uint32_t)n_tiles, l_run);
        ok = collect((uint32_t)n_tiles, sums);
      }
    }
    const size_t out_row = (size_t)(p.q_start[seq] + qi) * p.heads + kv_head * group + h;
    if (p.splits > 1 && quarter == 0 && real && (n_tiles == 0 || !ok))
      p.part_ml[out_row * p.splits + blockIdx.z] = make_float2(0.0f, 0.0f);        // nothing to merge from this part
    if (ok && quarter == 0 && n_tiles > 0 &&
        mbar_wait(&pv_done[(n_tiles - 1) & 1], (((uint32_t)(n_tiles - 1)) >> 1) & 1, abort_flag, p.status, kPagedKernelId, 8)) {
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
      if (j > 0 && !mbar_wait(&pv_done[0], (uint32_t)(j - 1) & 1, abort_flag, p.status, kPagedKernelId, 7)) { ok = false; break; }
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
      if (lane == 0) mbar_arrive(&p_ready[0]);
    }
    const size_t out_row = (size_t)(p.q_start[seq] + qi) * p.heads + kv_head * group + h;
    if (p.splits > 1 && real && (n_tiles == 0 || !ok))
      p.part_ml[out_row * p.splits + blockIdx.z] = make_float2(0.0f, 0.0f);        // nothing to merge from this part
    if (ok && n_tiles > 0 && mbar_wait(&pv_done[0], (uint32_t)(n_tiles - 1) & 1, abort_flag, p.status, kPagedKernelId, 8)) {
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
