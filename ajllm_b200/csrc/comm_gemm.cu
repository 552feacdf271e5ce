// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
//
//   ag_gemm : C[M, N] = gather_rows(A_shards)[M, K] * op(B)      (column-parallel: all-gather -> GEMM)
//   gemm_rs : C_local[M/tp, N] = reduce_scatter_rows(A[M, K] * op(B))   (row-parallel: GEMM -> reduce-scatter)
//   gemm_ar : C[M, N] = sum over ranks of A[M, K] * op(B)                (row-parallel: GEMM -> all-reduce)
//   gw_gemm : C[M, N] = A[M, K] * W^T, W inside gather(flat weight shards)  (sharded weights: all-gather -> GEMM)
//
// Both are one persistent kernel per rank built on the same tcgen05 main loop as gemm_bf16.cu
// (TMA ring -> tcgen05.mma -> TMEM -> epilogue warps).
//
// The three training modes run on CTA pairs (clusters of two, tcgen05 cta_group::2, 256 x 256 tiles) whenever a
// rank's rows split into 256-row tiles: the even CTA of a pair draws the tiles and issues the products, both CTAs
// load, drain and store their 128 rows. Decoding (gemm_ar) and odd row counts use single CTAs on 128 x 256 tiles.
//
// ag_gemm: a few "copy" CTAs pull every peer's [M/tp, K] shard out of that peer's symmetric staging
// buffer with bulk asynchronous copies (peer global -> shared -> local global; every CTA fetches its own
// bytes) and publish a flag per group of pieces of a shard; the GEMM CTAs walk the output tiles shard by
// shard, starting with the shard that is already local, and their TMA producer waits for the groups that
// hold a tile's rows before touching them, so each remote byte crosses NVLink once and the transfer hides
// behind the tiles of earlier rows.
//
// gemm_rs: consecutive tiles rotate over the shards (the stores to the peers are spread over the whole
// kernel); the epilogue stores each bf16 partial tile straight into the owning rank's symmetric receive
// buffer (slot = this rank); every epilogue warp credits the tiles it stored to their owners with one
// release at the end; after its last tile every CTA waits until all partials of its own rows have arrived
// and sums them in fp32 into the local output.
//
// gemm_ar (decoding, where M is a few hundred rows at most): the same epilogue stores each partial tile
// into every rank's receive buffer (slot = this rank), and the closing reduction sums all tp slots over
// the whole [M, N] output, so the partial products cross NVLink once and no separate collective runs.
//
// gw_gemm (fully sharded parameters): the operand that is gathered is the weight. Every rank owns one
// equal slice of a unit's flat parameter buffer; the copy CTAs pull the peers' slices into the local
// full buffer exactly as in ag_gemm, and the TMA producer of a tile waits for the slices that its rows
// of W (a byte range of the flat buffer, which may straddle two slices) live in. Tiles are visited
// starting with the columns whose weights are already local, so the first products run while the rest
// of the unit, including parameters this GEMM does not use, is still arriving.
//
// Buffers that peers touch are double-buffered on the parity of the call number, and no call ends in an all-ranks
// handshake. Gathering modes: a call announces "my staging buffer holds call g" (ready), every rank tells the owners
// when it has finished reading their buffers (done = g), and call g only makes sure, before it returns, that the peers
// reported done for call g - 1, i.e. that the staging buffer the NEXT call will overwrite is no longer read. Reducing
// modes: the call number q and the arrival count that means "all partial tiles of call q are here" live in device
// memory and are advanced by the last CTA of each call (so a captured CUDA graph can replay the kernel); a rank
// stores into a peer's receive buffer of parity q & 1 only after that peer reported done for call q - 2, and reports
// its own done = q once it has summed its rows. A rank therefore waits for a peer only when it needs that peer's
// data, or a buffer that peer has not released yet.
//
// Every wait on another CTA or another GPU is bounded (see common.cuh); on expiry the kernel records a
// status word, skips the dependent work and exits through the normal teardown.
#include <string.h>

#include "common.cuh"
#include "gemm_pair.h"

#include <cstdlib>

namespace ajb {
namespace comm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kABytes = BM * BK * 2;
constexpr int kEpiRowPitch = BN * 2 + 16;               // staged output rows, padded against bank conflicts
constexpr int kEpiBytes = BM * kEpiRowPitch;            // one bf16 output tile, staged for bulk row stores
// Two variants of the kernel. Single CTAs: 128 x 256 tiles, A and the whole B tile per stage. CTA pairs (clusters
// of two, tcgen05 cta_group::2): 256 x 256 tiles, each CTA stages its 128 rows of A and half of the B tile, so a
// stage is a third smaller and the ring one slot deeper; rows per rank must then be a multiple of 256.
template <bool PAIR>
struct Cfg {
  static constexpr int kStages = PAIR ? 4 : 3;
  static constexpr int kBRows = PAIR ? BN / 2 : BN;
  static constexpr int kBBytes = kBRows * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kSmemBytes = kRingBytes + kEpiBytes + 512;
  static constexpr int kTileRows = PAIR ? 2 * BM : BM;
};
constexpr int kMaxRanks = 8;
constexpr int kGroupM = 16;
constexpr int kCopyPiece = 32768;                       // bytes per bulk copy
constexpr int kCopyBufs = 6;                            // pieces in flight per copy CTA (ring = pipeline + epilogue space)
static_assert((Cfg<false>::kRingBytes + kEpiBytes) / kCopyPiece >= kCopyBufs, "copy ring does not fit");
static_assert(kSwigluWarpBytes <= 32 * kEpiRowPitch, "the SwiGLU row buffers of a warp must fit its part of the staging tile");
static_assert((Cfg<true>::kRingBytes + kEpiBytes) / kCopyPiece >= kCopyBufs, "copy ring does not fit");
constexpr int kQueue = 4;                               // depth of the per-CTA tile queue
constexpr int kMaxGroups = 32;                          // arrival groups per shard (all-gather)
constexpr int kScratchWords = 16 + kMaxRanks * kMaxGroups;   // local scratch: flags, counters, group flags

enum Mode : int { kAllGather = 0, kReduceScatter = 1, kAllReduce = 2, kGatherWeight = 3 };

struct Params {
  int mode;
  int m, n, k;            // full problem (m = all rows)
  int tp, rank;
  int m_local;            // rows per rank
  int copy_ctas;          // all-gather: CTAs that move data instead of computing
  long long shard_bytes;  // bytes each rank contributes to the gathered buffer
  long long b_offset;     // gather-weight: byte offset of W inside the gathered buffer
  long long b_row_bytes;  // gather-weight: bytes per row of W
  // all-gather
  const void* stage_ptrs[kMaxRanks];     // each rank's symmetric [m_local, k] staging buffer (peer addresses)
  void* gathered;                        // local [m, k]
  unsigned int* shard_flags;             // local, zeroed by the host before launch, one per shard
  // all-gather: a shard arrives in up to kMaxGroups groups of `group_pieces` consecutive 32 KB pieces; every copy CTA
  // adds one to group_flags[shard * kMaxGroups + g] when its pieces of group g are in local memory, so the tiles of
  // a remote shard start as soon as their own rows are there instead of after the whole shard
  unsigned int* group_flags;
  int group_pieces;                      // pieces per group (a multiple of copy_ctas)
  int groups;                            // groups per shard
  // reduce-scatter
  void* recv_ptrs[2][kMaxRanks];         // each rank's two symmetric [tp, m_local, n] receive buffers (all-reduce: m_local = m); parity = call & 1
  unsigned int* counter_ptrs[kMaxRanks]; // each rank's symmetric arrival counters, one per source rank
  unsigned int* reduce_state;            // local: [0] reducing calls completed, [1] arrival count reached by them
  void* out_local;                       // [m_local, n] bf16 (reduce-scatter) / [m, n] bf16 (all-gather)
  long long ldc;
  // cross-rank handshakes (symmetric flag words)
  unsigned int* ready_ptrs[kMaxRanks];   // ready_ptrs[p][r] : rank r's staging buffer holds this call's data
  unsigned int* done_ptrs[kMaxRanks];    // done_ptrs[p][r]  : gathering: rank r has read rank p's staging buffer of that call;
                                         //                    reducing: rank r has summed its receive buffer of that call
  unsigned int epoch;                    // gathering modes: number of this call (host-counted)
  unsigned int* local_cta_counter;       // local, zeroed by the host before launch
  unsigned int* tile_counter;            // local, zeroed by the host before launch
  // all-gather mode only. 1: the output holds (gate, up) pairs in neighbouring columns and the epilogue also writes
  // aux[m, n / 2] = silu(gate) * up. 2: the accumulators are d_act[m, n], aux is the saved gate_up[m, 2 n] and the
  // epilogue writes d_gate_up[m, 2 n] to the output instead of the accumulators.
  int swiglu;
  void* aux;
  long long ld_aux;
  DeviceStatus* status;
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded spin until *p >= want (signed distance, so epochs may wrap). `sys` selects the scope.
__device__ __forceinline__ bool wait_ge(const unsigned int* p, unsigned int want, bool sys, volatile uint32_t* abort_flag,
                                        DeviceStatus* status, int stage) {
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    const unsigned int v = sys ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int)(v - want) >= 0) return true;
    if (abort_flag != nullptr && *abort_flag) return false;
    if ((++spins & 0xff) == 0 && global_timer_ns() - t0 > kWaitBudgetNs) {
      if (abort_flag != nullptr) *abort_flag = 1;
      if (status != nullptr && atomicCAS(&status[kCommGemm].code, 0u, (unsigned)((stage << 8) | (kCommGemm + 1))) == 0u) {
        status[kCommGemm].block = blockIdx.x;
        status[kCommGemm].detail0 = want;
        status[kCommGemm].detail1 = v;
      }
      return false;
    }
    __nanosleep(64);
  }
}

// Tile order: shard by shard (`first_shard`, then increasing modulo tp); inside a shard, groups of
// kGroupM row-blocks sweep the column blocks so a wave of CTAs shares its panels through L2.
// With `interleave` consecutive tiles rotate over the shards instead (reduce-scatter: the stores to the
// peers are then spread over the whole kernel instead of bunched at its start).
__device__ __forceinline__ void tile_coords(int tile, int tiles_m_local, int tiles_n, int tp, int first_shard,
                                            bool interleave, int& shard, int& tm, int& tn) {
  const int per_shard = tiles_m_local * tiles_n;
  const int s = interleave ? tile % tp : tile / per_shard;
  shard = (first_shard + s) % tp;
  const int within_shard = interleave ? tile / tp : tile - s * per_shard;
  const int group_span = kGroupM * tiles_n;
  const int group = within_shard / group_span;
  const int first_m = group * kGroupM;
  const int rows = min(kGroupM, tiles_m_local - first_m);
  const int within = within_shard - group * group_span;
  tm = shard * tiles_m_local + first_m + within % rows;
  tn = within / rows;
}


// One copy CTA's share of the all-gather: thread 0 streams 32 KB pieces through a shared-memory ring.
__device__ void copy_cta_all_gather(const Params& p, uint8_t* ring, uint64_t* bars, volatile uint32_t* abort_flag) {
  if (threadIdx.x != 0) return;
  const int cta = blockIdx.x, n_copy = p.copy_ctas;
  const long long shard_bytes = p.shard_bytes;
  const long long pieces = (shard_bytes + kCopyPiece - 1) / kCopyPiece;
  if (cta == 0) {
    // tell every peer that this rank's staging buffer holds the data of this call
    for (int r = 0; r < p.tp; ++r) st_release_sys(p.ready_ptrs[r] + p.rank, p.epoch);
  }
  uint32_t issued = 0, drained = 0;   // running counts over all shards (ring position / barrier phase)
  bool ok = true;
  for (int s = 1; s < p.tp && ok; ++s) {      // the local shard was placed by the host before the launch
    const int shard = (p.rank + s) % p.tp;
    ok = wait_ge(p.ready_ptrs[p.rank] + shard, p.epoch, true, abort_flag, p.status, 20);
    if (!ok) break;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.stage_ptrs[shard]);
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.gathered) + (long long)shard * shard_bytes;
    // pieces cta, cta + n_copy, ... of this shard; this CTA's j-th piece lies in group j / per_group
    long long next_load = cta, next_store = cta;
    const int per_group = p.group_pieces / n_copy;      // pieces of one CTA per group
    int stored = 0, announced = 0;                      // this CTA's stores issued / groups announced (this shard)
    auto announce_through = [&](int complete_stores) {  // the first `complete_stores` stores are in global memory
      const int upto = complete_stores / per_group;     // groups wholly covered by them
      if (upto <= announced) return;
      fence_proxy_async_all();
      __threadfence();
      for (; announced < upto && announced < p.groups; ++announced)
        red_release_gpu_add(p.group_flags + shard * kMaxGroups + announced, 1u);
    };
    auto piece_bytes = [&](long long piece) -> uint32_t {
      const long long off = piece * kCopyPiece;
      return (uint32_t)min((long long)kCopyPiece, shard_bytes - off);
    };
    while (next_store < pieces) {
      while (next_load < pieces && issued - drained < (uint32_t)kCopyBufs) {
        const int buf = issued % kCopyBufs;
        mbar_arrive_expect_tx(&bars[buf], piece_bytes(next_load));
        bulk_g2s(ring + (size_t)buf * kCopyPiece, src + next_load * kCopyPiece, piece_bytes(next_load), &bars[buf]);
        ++issued;
        next_load += n_copy;
      }
      const int buf = drained % kCopyBufs;
      if (!mbar_wait(&bars[buf], (drained / kCopyBufs) & 1, abort_flag, p.status, kCommGemm, 21)) { ok = false; break; }
      bulk_s2g(dst + next_store * kCopyPiece, ring + (size_t)buf * kCopyPiece, piece_bytes(next_store));
      bulk_commit();
      bulk_wait_read_all();      // the ring slot may be refilled once the store has read it
      ++drained;
      next_store += n_copy;
      ++stored;
      if (p.mode == kAllGather && stored >= 2 && (stored - 2) % per_group == 0 && stored - 2 > 0) {
        bulk_wait_all_but_two(); // all but the two youngest stores have landed
        announce_through(stored - 2);
      }
    }
    bulk_wait_all();             // stores of this shard are complete in global memory
    fence_proxy_async_all();
    __threadfence();
    if (p.mode == kAllGather) {
      // the remaining groups, those in which this CTA had no piece included
      for (; announced < p.groups; ++announced) red_release_gpu_add(p.group_flags + shard * kMaxGroups + announced, 1u);
    }
    red_release_gpu_add(p.shard_flags + shard, 1u);
  }
  if (!ok) {
    // loads still in flight land in this CTA's shared memory: give them a bounded moment before leaving
    const unsigned long long t0 = global_timer_ns();
    while (issued != drained && global_timer_ns() - t0 < 100000000ull) {
      if (mbar_try_wait(&bars[drained % kCopyBufs], (drained / kCopyBufs) & 1)) ++drained;
    }
  }
  // The last copy CTA to finish tells the peers that this rank no longer reads their staging buffers of this call.
  // It does not wait for the same message about this call: the staging buffers alternate, so what must be true
  // before this kernel returns is only that the peers are done with the PREVIOUS call's buffer, the one the next
  // call overwrites; they said so long ago.
  if (atomicAdd(p.local_cta_counter, 1u) == (unsigned)(n_copy - 1)) {
    __threadfence();
    for (int r = 0; r < p.tp; ++r) st_release_sys(p.done_ptrs[r] + p.rank, p.epoch);
    for (int r = 0; r < p.tp; ++r)
      if (!wait_ge(p.done_ptrs[p.rank] + r, p.epoch - 1u, true, nullptr, p.status, 22)) break;
  }
}

// Per-CTA tile queue: the TMA producer draws tile numbers from a grid-wide counter (so CTAs that spent
// the first part of the kernel copying simply join in later) and hands them to the MMA and epilogue warps.
struct TileQueue {
  int tile[kQueue];
};

// Closing reduction: out[i] = sum over the tp slots of this rank's receive buffer, fp32 accumulation, 8 bf16 per
// vector. One CTA per SM with 192 threads has to keep the whole memory system busy here, so every thread has
// TP * U independent 16-byte loads in flight before it adds anything (TP = 0: rank count known only at run time,
// U loads in flight per slot).
template <int TP, int U>
__device__ __forceinline__ void sum_slots(const Params& p, int parity) {
  const long long vec_total = (long long)p.m_local * p.n / 8;
  const uint4* base = reinterpret_cast<const uint4*>(p.recv_ptrs[parity][p.rank]);
  uint4* out = reinterpret_cast<uint4*>(p.out_local);
  const long long stride = (long long)gridDim.x * kThreads;
  const int tp = TP > 0 ? TP : p.tp;
  for (long long i0 = (long long)blockIdx.x * kThreads + threadIdx.x; i0 < vec_total; i0 += stride * U) {
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
    if (TP > 0) {
      uint4 q[TP > 0 ? TP : 1][U];
#pragma unroll
      for (int r = 0; r < (TP > 0 ? TP : 1); ++r)
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          q[r][u] = i < vec_total ? base[(long long)r * vec_total + i] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
      for (int r = 0; r < (TP > 0 ? TP : 1); ++r)
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q[r][u]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc[u][2 * j] += f.x;
            acc[u][2 * j + 1] += f.y;
          }
        }
    } else {
      for (int r = 0; r < tp; ++r) {
        uint4 q[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          q[u] = i < vec_total ? base[(long long)r * vec_total + i] : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q[u]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc[u][2 * j] += f.x;
            acc[u][2 * j + 1] += f.y;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < vec_total) {
        uint4 o;
        o.x = pack_bf16x2(acc[u][0], acc[u][1]);
        o.y = pack_bf16x2(acc[u][2], acc[u][3]);
        o.z = pack_bf16x2(acc[u][4], acc[u][5]);
        o.w = pack_bf16x2(acc[u][6], acc[u][7]);
        out[i] = o;
      }
    }
  }
}


template <bool B_MN, bool PAIR>
__device__ __forceinline__ void comm_gemm_body(const CUtensorMap& map_a, const CUtensorMap& map_b, const Params& p) {
  using C = Cfg<PAIR>;
  constexpr int kStages = C::kStages;
  constexpr int kStageBytes = C::kStageBytes;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  uint8_t* epi_base = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_base + kEpiBytes);
  if (smem_misaligned(smem, p.status, kCommGemm, reinterpret_cast<uint32_t*>(bars) + 120)) return;
  uint64_t* full = bars;                       // kStages
  uint64_t* empty = full + kStages;            // kStages
  uint64_t* acc_full = empty + kStages;        // 2
  uint64_t* acc_empty = acc_full + 2;          // 2
  uint64_t* copy_bars = acc_empty + 2;         // kCopyBufs
  uint64_t* q_full = copy_bars + kCopyBufs;    // kQueue
  uint64_t* q_empty = q_full + kQueue;         // kQueue
  TileQueue* queue = reinterpret_cast<TileQueue*>(q_empty + kQueue);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(queue + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // pair variant: the even CTA of a cluster leads (draws tiles, arms the full barriers, issues the products)
  const uint32_t pair_rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = pair_rank == 0;
  const bool gathers = p.mode == kAllGather || p.mode == kGatherWeight;
  const bool is_copy_cta = gathers && (int)blockIdx.x < p.copy_ctas;     // copy_ctas is even for pairs: whole clusters copy
  const int tiles_m_local = p.m_local / C::kTileRows;
  const int tiles_n = (p.n + BN - 1) / BN;
  const int shards = (p.mode == kAllReduce || p.mode == kGatherWeight) ? 1 : p.tp;   // one "shard" of m_local = m rows
  const int num_tiles = tiles_m_local * shards * tiles_n;
  const int num_kb = (p.k + BK - 1) / BK;
  // all-gather: the local shard is ready first. reduce-scatter: the rows this rank owns come last.
  const int first_shard = p.mode == kAllGather ? p.rank : (p.mode == kReduceScatter ? (p.rank + 1) % p.tp : 0);
  // gather-weight: start with the column block whose weight rows begin in this rank's own slice
  int tn_first = 0;
  if (p.mode == kGatherWeight) {
    const long long own = (long long)p.rank * p.shard_bytes - p.b_offset;
    if (own > 0) tn_first = (int)min((long long)tiles_n - 1, (own + (long long)BN * p.b_row_bytes - 1) / ((long long)BN * p.b_row_bytes));
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], PAIR ? 8 : 4);     // pairs: the leader's barrier collects both CTAs' epilogue warps
    }
    for (int i = 0; i < kCopyBufs; ++i) mbar_init(&copy_bars[i], 1);
    for (int i = 0; i < kQueue; ++i) {
      mbar_init(&q_full[i], 1);
      // consumers of a queue slot: MMA warp + four epilogue warps; pairs: plus the peer's producer and epilogue warps
      mbar_init(&q_empty[i], PAIR ? 10 : 5);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensor_map(&map_a);
    prefetch_tensor_map(&map_b);
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(tmem_slot, 2 * BN); tmem_relinquish_pair(); }
    else      { tmem_alloc(tmem_slot, 2 * BN); tmem_relinquish(); }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();    // the peer's barriers exist before anything is signalled across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // reducing modes: this call's number, receive-buffer parity and the arrival count that completes it (device state,
  // advanced by the last CTA of the call, after every CTA has read it)
  const bool reduces = p.mode == kReduceScatter || p.mode == kAllReduce;
  const unsigned int reduce_call = reduces ? p.reduce_state[0] + 1u : 0u;
  const unsigned int reduce_expected = reduces ? p.reduce_state[1] + (unsigned)((p.m_local / BM) * tiles_n * 4) : 0u;
  const int parity = (int)(reduce_call & 1u);

  if (is_copy_cta) {
    // phase 1 of a copy CTA: move remote shards (thread 0 drives the bulk copies), then compute like the rest
    copy_cta_all_gather(p, smem, copy_bars, abort_flag);
    __syncthreads();
  }
  // shared::cluster addresses of the barriers and the queue that live in the other CTA of the pair
  const uint32_t full_leader = PAIR ? map_to_cta(smem_u32(&full[0]), 0) : 0u;
  const uint32_t acc_empty_leader = PAIR ? map_to_cta(smem_u32(&acc_empty[0]), 0) : 0u;
  const uint32_t q_empty_leader = PAIR ? map_to_cta(smem_u32(&q_empty[0]), 0) : 0u;
  const uint32_t q_full_peer = PAIR ? map_to_cta(smem_u32(&q_full[0]), 1) : 0u;
  const uint32_t queue_peer = PAIR ? map_to_cta(smem_u32(&queue->tile[0]), 1) : 0u;
  const uint32_t empty_peer = PAIR ? map_to_cta(smem_u32(&empty[0]), 1) : 0u;
  const uint32_t acc_full_peer = PAIR ? map_to_cta(smem_u32(&acc_full[0]), 1) : 0u;
  // a consumer of queue slot `slot` is done with it
  auto release_slot = [&](int slot) {
    if (PAIR) mbar_arrive_cluster(q_empty_leader + (uint32_t)slot * 8u);
    else mbar_arrive(&q_empty[slot]);
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0, ready_shard = p.rank;
      uint32_t ready_groups = 0;        // all-gather: groups of `ready_shard` known to have arrived
      uint32_t ready_mask = 0;          // gather-weight: slices known to have arrived
      bool ok = *abort_flag == 0;
      for (uint32_t qi = 0; ok; ++qi) {
        const int slot = qi % kQueue;
        int tile;
        if (leader) {
          // pairs: half of the slot's consumers arrive from the other CTA, hence the cluster-scope acquire
          if (!(PAIR ? mbar_wait_cluster(&q_empty[slot], ((qi / kQueue) & 1) ^ 1, abort_flag, p.status, kCommGemm, 5)
                     : mbar_wait(&q_empty[slot], ((qi / kQueue) & 1) ^ 1, abort_flag, p.status, kCommGemm, 5))) { ok = false; break; }
          tile = (int)atomicAdd(p.tile_counter, 1u);
          if (tile >= num_tiles) tile = -1;
          queue->tile[slot] = tile;
          if (PAIR) {
            // the peer works on the same tile: the number goes into its queue too, then its slot is marked full
            st_shared_cluster_u32(queue_peer + (uint32_t)slot * 4u, (uint32_t)tile);
            mbar_arrive_cluster(q_full_peer + (uint32_t)slot * 8u);
          }
          mbar_arrive(&q_full[slot]);
        } else {
          if (!mbar_wait_cluster(&q_full[slot], (qi / kQueue) & 1, abort_flag, p.status, kCommGemm, 8)) { ok = false; break; }
          tile = queue->tile[slot];
          release_slot(slot);
        }
        if (tile < 0) break;
        int shard, tm, tn;
        tile_coords(tile, tiles_m_local, tiles_n, shards, first_shard, p.mode == kReduceScatter, shard, tm, tn);
        if (p.mode == kGatherWeight) {
          tn = (tn + tn_first) % tiles_n;
          // slices of the flat buffer that hold rows [tn * BN, tn * BN + BN) of W
          const long long lo = p.b_offset + (long long)tn * BN * p.b_row_bytes;
          const long long hi = p.b_offset + (long long)min(tn * BN + BN, p.n) * p.b_row_bytes - 1;
          for (int sh = (int)(lo / p.shard_bytes); sh <= (int)(hi / p.shard_bytes) && ok; ++sh) {
            if (sh == p.rank || (ready_mask >> sh) & 1u) continue;
            if (!wait_ge(p.shard_flags + sh, (unsigned)p.copy_ctas, false, abort_flag, p.status, 11)) { ok = false; break; }
            fence_proxy_async_all();
            ready_mask |= 1u << sh;
          }
          if (!ok) break;
        }
        const int m0 = tm * C::kTileRows + (int)pair_rank * BM, n0 = tn * BN + (int)pair_rank * C::kBRows;
        if (p.mode == kAllGather && shard != p.rank) {
          if (shard != ready_shard) { ready_shard = shard; ready_groups = 0; }
          // groups that hold this CTA's 128 rows of A
          const long long row_bytes = (long long)p.k * 2;
          const long long lo = (long long)(m0 - shard * p.m_local) * row_bytes;
          const long long hi = lo + (long long)BM * row_bytes - 1;
          const long long group_bytes = (long long)p.group_pieces * kCopyPiece;
          bool waited = false;
          for (int g = (int)(lo / group_bytes); g <= (int)(hi / group_bytes) && ok; ++g) {
            if ((ready_groups >> g) & 1u) continue;
            if (!wait_ge(p.group_flags + shard * kMaxGroups + g, (unsigned)p.copy_ctas, false, abort_flag, p.status, 10)) { ok = false; break; }
            ready_groups |= 1u << g;
            waited = true;
          }
          if (!ok) break;
          if (waited) fence_proxy_async_all();      // copied rows were written through the async proxy of other CTAs
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, kCommGemm, 1)) { ok = false; break; }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          const int k0 = kb * BK;
          if (PAIR) {
            // both CTAs' loads complete on the leader's barrier, which the leader arms with the bytes of both
            if (leader) mbar_arrive_expect_tx(&full[stage], 2 * kStageBytes);
            const uint32_t bar = full_leader + (uint32_t)stage * 8u;
            tma_load_2d_pair(sa, &map_a, bar, k0, m0);
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < C::kBRows / 64; ++j) tma_load_2d_pair(sb + j * (BK * 128), &map_b, bar, n0 + 64 * j, k0);
            } else {
              tma_load_2d_pair(sb, &map_b, bar, k0, n0);
            }
          } else {
            mbar_arrive_expect_tx(&full[stage], kStageBytes);
            tma_load_2d(sa, &map_a, &full[stage], k0, m0);
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * (BK * 128), &map_b, &full[stage], n0 + 64 * j, k0);
            } else {
              tma_load_2d(sb, &map_b, &full[stage], k0, n0);
            }
          }
          ++issued;
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok && leader) {
        const int pending = min(issued, kStages);
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) { s = kStages - 1; ph ^= 1; }
          const unsigned long long t0 = global_timer_ns();
          while (!mbar_try_wait(&full[s], ph) && global_timer_ns() - t0 < 100000000ull) {}
        }
      }
    }
  } else if (warp == 1 && leader) {
    constexpr uint32_t idesc = make_idesc(C::kTileRows, BN, 1, false, B_MN);
    // descriptor low words formed once; a stage is one multiply-add away, a k-step a compile-time offset
    const uint32_t a_lo0 = desc_lo_k_major(smem_u32(smem));
    const uint32_t b_lo0 = B_MN ? desc_lo_mn_major(smem_u32(smem) + kABytes, BK * 128) : desc_lo_k_major(smem_u32(smem) + kABytes);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (uint32_t qi = 0; ok; ++qi) {
      const int slot = qi % kQueue;
      if (!mbar_wait(&q_full[slot], (qi / kQueue) & 1, abort_flag, p.status, kCommGemm, 6)) break;   // filled by this CTA
      const int tile = queue->tile[slot];
      __syncwarp();
      if (lane == 0) release_slot(slot);
      if (tile < 0) break;
      const int buf = qi & 1;
      const uint32_t use = qi >> 1;
      if (!(PAIR ? mbar_wait_cluster(&acc_empty[buf], (use & 1) ^ 1, abort_flag, p.status, kCommGemm, 2)
                 : mbar_wait(&acc_empty[buf], (use & 1) ^ 1, abort_flag, p.status, kCommGemm, 2))) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kCommGemm, 3)) { ok = false; break; }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_lo = a_lo0 + (uint32_t)stage * (uint32_t)(kStageBytes >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)stage * (uint32_t)(kStageBytes >> 4);
          if (PAIR) {
            umma_pair_f16(tmem_d, desc_at(a_lo, 0), desc_at(b_lo, 0), idesc, kb != 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < BK / UMMA_K; ++k)
              umma_pair_f16_c<true>(tmem_d, desc_at(a_lo, (uint32_t)k * UMMA_K * 2),
                                    desc_at(b_lo, B_MN ? mn_major_step(k) : (uint32_t)k * UMMA_K * 2), idesc);
            // the slot is free in both CTAs once these products have read it
            tc_commit_pair(smem_u32(&empty[stage]));
            tc_commit_pair(empty_peer + (uint32_t)stage * 8u);
          } else {
            umma_f16(tmem_d, desc_at(a_lo, 0), desc_at(b_lo, 0), idesc, kb != 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < BK / UMMA_K; ++k)
              umma_f16_c<true>(tmem_d, desc_at(a_lo, (uint32_t)k * UMMA_K * 2),
                               desc_at(b_lo, B_MN ? mn_major_step(k) : (uint32_t)k * UMMA_K * 2), idesc);
            tc_commit(&empty[stage]);
          }
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (ok && lane == 0) {
        if (PAIR) {
          tc_commit_pair(smem_u32(&acc_full[buf]));
          tc_commit_pair(acc_full_peer + (uint32_t)buf * 8u);
        } else {
          tc_commit(&acc_full[buf]);
        }
      }
      __syncwarp();
    }
  } else if (warp >= 2) {
    const int quarter = warp & 3;
    uint8_t* my_row = epi_base + (quarter * 32 + lane) * kEpiRowPitch;    // this lane's staged output row
    bool ok = true;
    // The reader of a receive buffer only starts once every tile of every rank has been counted, so the
    // tiles are credited in bulk at the end of the kernel: lane r of this warp counts the tiles stored to
    // rank r and, once all stores have landed, tells rank r with one release. A release per tile would stall
    // the epilogue for longer than the tile's MMAs take.
    unsigned int stored_tiles = 0;   // lane r: tiles this warp stored into rank r's receive buffer
    if (reduces) {
      // rank `lane` must have summed (and so released) its receive buffer of this parity, last used two calls ago
      bool released = true;
      if (lane < p.tp) released = wait_ge(p.done_ptrs[p.rank] + lane, reduce_call - 2u, true, abort_flag, p.status, 32);
      ok = __all_sync(0xffffffffu, released);
    }
    for (uint32_t qi = 0; ok; ++qi) {
      const int slot = qi % kQueue;
      // pairs: the peer's slot is written and marked full by the leader, hence the cluster-scope acquire
      if (!(PAIR ? mbar_wait_cluster(&q_full[slot], (qi / kQueue) & 1, abort_flag, p.status, kCommGemm, 7)
                 : mbar_wait(&q_full[slot], (qi / kQueue) & 1, abort_flag, p.status, kCommGemm, 7))) break;
      const int tile = queue->tile[slot];
      __syncwarp();
      if (lane == 0) release_slot(slot);
      if (tile < 0) break;
      const int buf = qi & 1;
      const uint32_t use = qi >> 1;
      int shard, tm, tn;
      tile_coords(tile, tiles_m_local, tiles_n, shards, first_shard, p.mode == kReduceScatter, shard, tm, tn);
      if (p.mode == kGatherWeight) tn = (tn + tn_first) % tiles_n;
      if (!mbar_wait(&acc_full[buf], use & 1, abort_flag, p.status, kCommGemm, 4)) { ok = false; break; }
      tc_fence_after_sync();
      bulk_wait_read_all();          // the previous tile's store has read this lane's staging row
      const uint32_t taddr = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(quarter * 32) << 16);
      const int row = tm * C::kTileRows + (int)pair_rank * BM + quarter * 32 + lane;
      const int col0 = tn * BN;
      if (p.swiglu == 2) {
        // SwiGLU backward: the accumulators are d_act; they meet the saved (gate, up) words of the same positions
        // and leave as the gradient of the pairs (n is a multiple of 32: a chunk is whole or absent). The warp's
        // part of the staging tile is its row block.
        const int row0 = row - lane;
        const long long at = 2 * col0;
        swiglu_backward_rows(taddr, reinterpret_cast<const __nv_bfloat16*>(p.aux) + (long long)row0 * p.ld_aux + at, p.ld_aux,
                             reinterpret_cast<__nv_bfloat16*>(p.out_local) + (long long)row0 * p.ldc + at, p.ldc, 32,
                             min(BN, p.n - col0), epi_base + quarter * 32 * kEpiRowPitch, lane);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) mbar_arrive_cluster(acc_empty_leader + (uint32_t)buf * 8u);
          else mbar_arrive(&acc_empty[buf]);
        }
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + (uint32_t)c, v);
        tc_wait_ld();
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(my_row + c * 2 + j * 16) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        if (p.swiglu == 1 && col0 + c < p.n)
          swiglu_store_activation(w, reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.aux) +
                                                             (long long)row * p.ld_aux + ((col0 + c) >> 1)));
      }
      // the accumulator is in shared memory now: hand the TMEM buffer back before the stores
      tc_fence_before_sync();
      fence_proxy_async_smem();      // the bulk store below reads this row through the async proxy
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(acc_empty_leader + (uint32_t)buf * 8u);
        else mbar_arrive(&acc_empty[buf]);
      }
      // one bulk store per row: up to 512 contiguous bytes leave the SM without passing through registers
      const int bytes = min(BN, p.n - col0) * 2;
      if (p.mode == kAllReduce) {
        // the partial tile goes to every rank's receive buffer (own included), slot = this rank
        if (bytes > 0) {
          for (int r = 0; r < p.tp; ++r) {
            const int peer = (p.rank + r) % p.tp;
            bulk_s2g(reinterpret_cast<__nv_bfloat16*>(p.recv_ptrs[parity][peer]) + ((long long)p.rank * p.m_local + row) * p.n + col0,
                     my_row, (uint32_t)bytes);
          }
        }
      } else {
        __nv_bfloat16* dst;
        if (p.mode == kAllGather || p.mode == kGatherWeight) {
          dst = reinterpret_cast<__nv_bfloat16*>(p.out_local) + (long long)row * p.ldc + col0;
        } else {
          // partial sums of shard `shard` go to that rank's receive buffer, slot = this rank
          dst = reinterpret_cast<__nv_bfloat16*>(p.recv_ptrs[parity][shard]) +
                ((long long)p.rank * p.m_local + (row - shard * p.m_local)) * p.n + col0;
        }
        if (bytes > 0) bulk_s2g(dst, my_row, (uint32_t)bytes);
      }
      bulk_commit();
      if (p.mode == kReduceScatter) stored_tiles += lane == shard ? 1u : 0u;
      else if (p.mode == kAllReduce) stored_tiles += lane < p.tp ? 1u : 0u;
    }
    bulk_wait_all();
    __syncwarp();                    // every lane's rows are complete in (peer) memory
    if (stored_tiles != 0) red_release_sys_add(p.counter_ptrs[lane] + p.rank, stored_tiles);
  }

  tc_fence_before_sync();
  __syncthreads();
  // pairs: neither CTA frees tensor memory or moves on while the other may still read its shared memory or write
  // its accumulators (every role of both CTAs has finished, or given up after a bounded wait, before this point)
  if (PAIR) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
  }

  if (p.mode == kReduceScatter || p.mode == kAllReduce) {
    // ---- sum the tp partial copies of the rows this rank owns (all-reduce: of all rows) (fp32) into the local output
    int* arrived = reinterpret_cast<int*>(epi_base);
    if (threadIdx.x == 0) {
      bool ok = *abort_flag == 0;
      for (int r = 0; r < p.tp && ok; ++r)
        ok = wait_ge(p.counter_ptrs[p.rank] + r, reduce_expected, true, nullptr, p.status, 30);
      *arrived = ok ? 1 : 0;
    }
    __syncthreads();
    if (*arrived) {
      switch (p.tp) {
        case 2: sum_slots<2, 8>(p, parity); break;
        case 4: sum_slots<4, 4>(p, parity); break;
        case 8: sum_slots<8, 2>(p, parity); break;
        default: sum_slots<0, 4>(p, parity); break;
      }
    }
    __syncthreads();
    // The last CTA advances the device-side call state and tells the peers that this rank has summed (released) its
    // receive buffer of this call; nobody waits here: a peer checks the release when it next needs that buffer.
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(p.local_cta_counter, 1u) == gridDim.x - 1) {
        p.reduce_state[0] = reduce_call;
        p.reduce_state[1] = reduce_expected;
        __threadfence();
        for (int r = 0; r < p.tp; ++r) st_release_sys(p.done_ptrs[r] + p.rank, reduce_call);
      }
    }
  }
}

template <bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
comm_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  comm_gemm_body<B_MN, false>(map_a, map_b, p);
}

template <bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
comm_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  comm_gemm_body<B_MN, true>(map_a, map_b, p);
}

}  // namespace comm
}  // namespace ajb

// Shared argument block (all pointer tables have `tp` entries). See comm::Params for the meaning.
struct AjbCommArgs {
  int mode, m, n, k, tp, rank, b_mn_major, copy_ctas;
  long long ldb, ldc;
  const void* a;                 // reduce-scatter, all-reduce: local [m, k] activations; all-gather: unused
  const void* b;                 // local weight shard
  void* out;                     // all-gather, all-reduce: [m, n]; reduce-scatter: [m / tp, n]
  void* gathered;                // all-gather: local [m, k] buffer that receives every shard
  const void* stage_ptrs[8];     // gathering modes: every rank's staging buffer of this call's parity
  void* recv_ptrs[8];            // reducing modes: every rank's receive buffer for odd calls ...
  void* recv_ptrs_even[8];       // ... and for even calls (the kernel knows the call number, the host need not)
  unsigned int* counter_ptrs[8];
  unsigned int* ready_ptrs[8];
  unsigned int* done_ptrs[8];    // the flag words of this call's class (gathering and reducing calls count separately)
  unsigned int* shard_flags;     // local scratch of 272 words (16 + 8 ranks x 32 groups): flags, counters, group flags
  unsigned int* reduce_state;    // reducing modes: 2 local words, zero at start, owned by the kernel afterwards
  unsigned int epoch;            // gathering modes: number of this gathering call (1, 2, ...)
  int a_rows;                    // all-reduce: rows of `a` that exist (<= m; the tiles above them read zeros); 0 means m
  long long shard_elems;         // gather-weight: bf16 elements per rank slice of the flat buffer (multiple of 8)
  long long b_offset_elems;      // gather-weight: first element of W inside the gathered buffer (multiple of 8)
  int swiglu;                    // all-gather: 0 plain, 1 also write aux = silu(gate) * up, 2 out = SwiGLU gradient of aux
  void* aux;                     // swiglu 1: act [m, n / 2] (written); swiglu 2: saved gate_up [m, 2 n] (read)
  long long ld_aux;              // row stride of aux in elements (multiple of 8)
};

extern "C" int ajb_comm_gemm(const AjbCommArgs* args, void* stream) {
  using namespace ajb;
  using namespace ajb::comm;
  const AjbCommArgs& a = *args;
  AJB_REQUIRE(a.tp >= 2 && a.tp <= kMaxRanks, "comm_gemm: tp must be in [2, %d]", kMaxRanks);
  if (a.mode == kAllReduce || a.mode == kGatherWeight) {
    AJB_REQUIRE(a.m % BM == 0, "comm_gemm: rows (%d) must be a multiple of %d", a.m, BM);
    if (a.mode == kGatherWeight) {
      AJB_REQUIRE(!a.b_mn_major && a.ldb == a.k, "comm_gemm: gathered weights must be dense [n, k] rows");
      AJB_REQUIRE(a.shard_elems > 0 && a.shard_elems % 8 == 0 && a.b_offset_elems % 8 == 0,
                  "comm_gemm: slice length and weight offset must be multiples of 8 elements");
      AJB_REQUIRE(a.b_offset_elems + (long long)a.n * a.k <= a.shard_elems * a.tp, "comm_gemm: W lies outside the gathered buffer");
    }
  } else {
    AJB_REQUIRE(a.m % a.tp == 0 && (a.m / a.tp) % BM == 0, "comm_gemm: rows per rank (%d / %d) must be a multiple of %d",
                a.m, a.tp, BM);
  }
  AJB_REQUIRE(a.k % 8 == 0 && a.n % 8 == 0, "comm_gemm: n and k must be multiples of 8");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  Params p;
  memset(&p, 0, sizeof(p));
  p.mode = a.mode; p.m = a.m; p.n = a.n; p.k = a.k; p.tp = a.tp; p.rank = a.rank;
  p.m_local = (a.mode == kAllReduce || a.mode == kGatherWeight) ? a.m : a.m / a.tp;
  const bool gathers = a.mode == kAllGather || a.mode == kGatherWeight;
  // CTA pairs for the three training modes when every rank's rows split into 256-row tiles (AJB_COMM_PAIR=0: never)
  static const bool pairs_enabled = [] {
    const char* v = std::getenv("AJB_COMM_PAIR");
    return v == nullptr || v[0] != '0';
  }();
  const bool pair = pairs_enabled && a.mode != kAllReduce && p.m_local % (2 * BM) == 0;   // decoding has too few rows
  p.copy_ctas = gathers ? a.copy_ctas : 0;
  if (pair) p.copy_ctas = (p.copy_ctas + 1) / 2 * 2;      // whole clusters copy
  // every CTA of this kernel must be resident at once (copy CTAs feed compute CTAs): one CTA per SM, and for the
  // pair variant as many clusters as the device can hold at once. Under a small SM budget the pulling CTAs are at
  // most half of the launch.
  const int grid = pair ? 2 * gemm_pair::capacity() : sm_count();
  if (gathers && p.copy_ctas * 2 > grid) p.copy_ctas = pair ? (grid / 4) * 2 : grid / 2;
  p.shard_bytes = a.mode == kGatherWeight ? a.shard_elems * 2 : (long long)p.m_local * a.k * 2;
  p.b_offset = a.b_offset_elems * 2;
  p.b_row_bytes = (long long)a.k * 2;
  for (int r = 0; r < a.tp; ++r) {
    p.stage_ptrs[r] = a.stage_ptrs[r];
    p.recv_ptrs[1][r] = a.recv_ptrs[r];
    p.recv_ptrs[0][r] = a.recv_ptrs_even[r];
    p.counter_ptrs[r] = a.counter_ptrs[r];
    p.ready_ptrs[r] = a.ready_ptrs[r];
    p.done_ptrs[r] = a.done_ptrs[r];
  }
  p.gathered = a.gathered;
  p.shard_flags = a.shard_flags;
  p.local_cta_counter = a.shard_flags + 8;
  p.tile_counter = a.shard_flags + 9;
  p.group_flags = a.shard_flags + 16;
  p.group_pieces = p.copy_ctas > 0 ? p.copy_ctas : 1;
  p.groups = 1;
  if (a.mode == kAllGather) {
    // groups of at least four pieces per copy CTA (one fence per group), at most kMaxGroups of them per shard
    const long long pieces = (p.shard_bytes + kCopyPiece - 1) / kCopyPiece;
    const long long per_cta = (pieces + p.copy_ctas - 1) / p.copy_ctas;
    long long per_group = (per_cta + kMaxGroups - 1) / kMaxGroups;
    if (per_group < 4) per_group = 4;
    p.group_pieces = (int)(per_group * p.copy_ctas);
    p.groups = (int)((per_cta + per_group - 1) / per_group);
  }
  p.reduce_state = a.reduce_state;
  AJB_REQUIRE(gathers || a.reduce_state != nullptr, "comm_gemm: reducing modes need the two state words");
  p.out_local = a.out;
  p.ldc = a.ldc;
  p.swiglu = a.swiglu;
  p.aux = a.aux;
  p.ld_aux = a.ld_aux;
  if (a.swiglu != 0) {
    AJB_REQUIRE(a.mode == kAllGather && (a.swiglu == 1 || a.swiglu == 2), "comm_gemm: SwiGLU epilogues belong to the all-gather mode");
    AJB_REQUIRE(a.n % 32 == 0 && a.aux != nullptr && a.ld_aux % 8 == 0 && a.ldc % 8 == 0 &&
                    ((reinterpret_cast<uintptr_t>(a.aux) | reinterpret_cast<uintptr_t>(a.out)) & 15) == 0,
                "comm_gemm: SwiGLU epilogues need n %% 32 == 0, 16-byte aligned buffers and row strides that are multiples of 8");
  }
  p.epoch = a.epoch;
  p.status = device_status_buffer();
  AJB_CUDA_OK(cudaMemsetAsync(a.shard_flags, 0, kScratchWords * sizeof(unsigned int), s));

  const void* a_ptr = a.mode == kAllGather ? a.gathered : a.a;
  const void* b_ptr = a.mode == kGatherWeight ? static_cast<const void*>(static_cast<const uint8_t*>(a.gathered) + a.b_offset_elems * 2) : a.b;
  CUtensorMap map_a, map_b;
  const int a_rows = (a.mode == kAllReduce && a.a_rows > 0) ? a.a_rows : a.m;
  AJB_REQUIRE(a_rows <= a.m, "comm_gemm: a_rows (%d) exceeds m (%d)", a_rows, a.m);
  int rc = make_tensor_map_2d(&map_a, a_ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_rows, a.k, (uint64_t)a.k * 2, BM, 64);
  if (rc) return rc;
  if (a.b_mn_major) rc = make_tensor_map_2d(&map_b, b_ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.k, a.n, a.ldb * 2, BK, 64);
  else              rc = make_tensor_map_2d(&map_b, b_ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.n, a.k, a.ldb * 2,
                                            pair ? Cfg<true>::kBRows : BN, 64);
  if (rc) return rc;
  static bool configured[4] = {false, false, false, false};
  const int which = (a.b_mn_major ? 1 : 0) | (pair ? 2 : 0);
  if (!configured[which]) {
    const int single_bytes = Cfg<false>::kSmemBytes, pair_bytes = Cfg<true>::kSmemBytes;
    switch (which) {
      case 0: AJB_CUDA_OK(cudaFuncSetAttribute(comm_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, single_bytes)); break;
      case 1: AJB_CUDA_OK(cudaFuncSetAttribute(comm_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, single_bytes)); break;
      case 2: AJB_CUDA_OK(cudaFuncSetAttribute(comm_gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_bytes)); break;
      default: AJB_CUDA_OK(cudaFuncSetAttribute(comm_gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_bytes)); break;
    }
    configured[which] = true;
  }
  AJB_REQUIRE(p.copy_ctas < grid && (!gathers || p.copy_ctas >= 1), "comm_gemm: copy CTA count %d is out of range", p.copy_ctas);
  switch (which) {
    case 0: comm_gemm_kernel<false><<<grid, kThreads, Cfg<false>::kSmemBytes, s>>>(map_a, map_b, p); break;
    case 1: comm_gemm_kernel<true><<<grid, kThreads, Cfg<false>::kSmemBytes, s>>>(map_a, map_b, p); break;
    case 2: comm_gemm_pair_kernel<false><<<grid, kThreads, Cfg<true>::kSmemBytes, s>>>(map_a, map_b, p); break;
    default: comm_gemm_pair_kernel<true><<<grid, kThreads, Cfg<true>::kSmemBytes, s>>>(map_a, map_b, p); break;
  }
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}
