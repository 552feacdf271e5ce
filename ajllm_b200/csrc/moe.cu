// Mixture-of-experts routing and token movement for sm_100a.
//
//   route_fwd     : softmax over the experts, top-k, optional renormalisation -> (experts, gates); one warp per token.
//   assign_slots  : deterministic capacity assignment. One CTA per expert scans the (token, choice) list in
//                   order; assignment number j of expert e gets slot e * stride + j, or -1 once j >= capacity.
//   push_rows     : expert-parallel dispatch. Every kept (token, choice) row is written straight into the owning
//                   rank's expert-major symmetric buffer over NVLink (peer stores), together with the per-(expert,
//                   source) row counts the grouped GEMM uses to skip padding; the kernel ends with a cross-rank
//                   handshake so that, when it returns, every row addressed to this rank has arrived.
//   pull_rows     : combine. Every token reads its k expert output rows from the ranks that computed them (peer
//                   loads), forms the gate-weighted sum in fp32, and optionally the k dot products with an upstream
//                   gradient (the gate gradients); a closing handshake tells the owners when their buffer is free.
//
// Slot layout on the destination rank: row ((local_expert * ep + source_rank) * stride + position).
// All cross-rank waits are bounded (common.cuh).
#include "common.cuh"

namespace ajb {
namespace moe {

constexpr int kMoeKernelId = 7;
constexpr int kMaxRanks = 8;
constexpr int kMaxTopK = 8;

// ------------------------------------------------------------------------------------------ routing
__global__ void route_fwd_kernel(const float* __restrict__ logits, int tokens, int experts, int top_k, int normalize,
                                 int* __restrict__ out_experts, float* __restrict__ out_gates,
                                 float* __restrict__ out_probs /* optional [tokens, experts] */) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  const float* row = logits + (size_t)warp * experts;
  // up to 256 experts: 8 values per lane
  float v[8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < experts ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = (lane + 32 * i) < experts ? __expf(v[i] - mx) : 0.0f;
    sum += v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.0f / sum;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] *= inv;
    if (out_probs != nullptr && lane + 32 * i < experts) out_probs[(size_t)warp * experts + lane + 32 * i] = v[i];
  }
  float gate_sum = 0.0f;
  float picked_gate[kMaxTopK];
  int picked_expert[kMaxTopK];
  for (int j = 0; j < top_k; ++j) {
    float best = -1.0f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    picked_gate[j] = best;
    picked_expert[j] = best_e;
    gate_sum += best;
    if ((best_e & 31) == lane) v[best_e >> 5] = -2.0f;   // remove from the next rounds
  }
  if (lane == 0) {
    const float scale = normalize ? 1.0f / gate_sum : 1.0f;
    for (int j = 0; j < top_k; ++j) {
      out_experts[(size_t)warp * top_k + j] = picked_expert[j];
      out_gates[(size_t)warp * top_k + j] = picked_gate[j] * scale;
    }
  }
}

// One CTA per expert. experts_of: [assignments] (token-major, choice-minor). slots: [assignments].
// counts[e] = kept assignments of expert e.
__global__ void __launch_bounds__(1024)
assign_slots_kernel(const int* __restrict__ experts_of, long long assignments, int capacity, int stride,
                    int* __restrict__ slots, int* __restrict__ counts) {
  __shared__ int warp_totals[32];
  __shared__ int base_shared;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base_shared = 0;
  __syncthreads();
  for (long long start = 0; start < assignments; start += blockDim.x) {
    const long long i = start + threadIdx.x;
    const bool mine = i < assignments && experts_of[i] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    const int before_in_warp = __popc(ballot & ((1u << lane) - 1));
    if (lane == 0) warp_totals[warp] = __popc(ballot);
    __syncthreads();
    int before_warps = 0, total = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
      const int t = warp_totals[w];
      if (w < warp) before_warps += t;
      total += t;
    }
    const int base = base_shared;
    if (mine) {
      const int pos = base + before_warps + before_in_warp;
      slots[i] = pos < capacity ? e * stride + pos : -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) base_shared = base + total;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = min(base_shared, capacity);
}

// ------------------------------------------------------------------------------------------ cross-rank helpers
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ bool wait_flag(const unsigned int* p, unsigned int want, DeviceStatus* status, int stage) {
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    const unsigned int v = ld_acquire_sys(p);
    if ((int)(v - want) >= 0) return true;
    if ((++spins & 0xff) == 0 && global_timer_ns() - t0 > kWaitBudgetNs) {
      if (status != nullptr && atomicCAS(&status[kMoeKernelId].code, 0u, (unsigned)((stage << 8) | (kMoeKernelId + 1))) == 0u) {
        status[kMoeKernelId].block = blockIdx.x;
        status[kMoeKernelId].detail0 = want;
        status[kMoeKernelId].detail1 = v;
      }
      return false;
    }
    __nanosleep(64);
  }
}

struct ExchangeParams {
  int tokens, top_k, dim;            // dim in bf16 elements (multiple of 8)
  int ep, rank, local_experts, stride;
  const int* slots;                  // [tokens, top_k], e * stride + pos or -1 (e = global expert id)
  void* peer_buffers[kMaxRanks];     // symmetric expert-major buffers [local_experts * ep * stride, dim]
  unsigned int* flag_ptrs[kMaxRanks];// symmetric flag words: [0:8] arrival, [8:16] release, [16:24] ready
  int* peer_counts[kMaxRanks];       // symmetric [local_experts, ep] int32 (dispatch only)
  const int* counts;                 // local [experts] kept rows per global expert (dispatch only)
  unsigned int epoch;
  unsigned int* local_counter;       // zeroed by the host before the launch
  DeviceStatus* status;
};

__device__ __forceinline__ long long dest_row(const ExchangeParams& p, int slot, int& dest_rank) {
  const int e = slot / p.stride, pos = slot - e * p.stride;
  dest_rank = e / p.local_experts;
  const int le = e - dest_rank * p.local_experts;
  return ((long long)le * p.ep + p.rank) * p.stride + pos;
}

// The last CTA to finish publishes `epoch` in slot `which` (0 = arrival, 8 = release) of every peer and waits
// until every peer has done the same here.
__device__ void closing_handshake(const ExchangeParams& p, int which) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(p.local_counter, 1u) == gridDim.x - 1) {
      for (int r = 0; r < p.ep; ++r) st_release_sys(p.flag_ptrs[r] + which + p.rank, p.epoch);
      for (int r = 0; r < p.ep; ++r)
        if (!wait_flag(p.flag_ptrs[p.rank] + which + r, p.epoch, p.status, 1 + which)) break;
    }
  }
}

// rows: [tokens, dim] bf16 source rows; scale (optional) [tokens, top_k] multiplies the row before it is sent.
__global__ void push_rows_kernel(const __nv_bfloat16* __restrict__ rows, const float* __restrict__ scale, ExchangeParams p) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long total = (long long)p.tokens * p.top_k;
  const int vecs = p.dim >> 3;
  if (blockIdx.x == 0 && p.counts != nullptr) {
    // row counts per (local expert on the destination, this source rank)
    for (int e = threadIdx.x; e < p.ep * p.local_experts; e += blockDim.x) {
      const int r = e / p.local_experts, le = e - r * p.local_experts;
      p.peer_counts[r][le * p.ep + p.rank] = p.counts[e];
    }
  }
  for (long long a = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; a < total; a += warps) {
    const int slot = p.slots[a];
    if (slot < 0) continue;
    int r;
    const long long row = dest_row(p, slot, r);
    const uint4* src = reinterpret_cast<const uint4*>(rows + (a / p.top_k) * p.dim);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.peer_buffers[r]) + row * p.dim);
    const float s = scale != nullptr ? scale[a] : 1.0f;
    for (int v = lane; v < vecs; v += 32) {
      uint4 q = src[v];
      if (scale != nullptr) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          h[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
      }
      dst[v] = q;
    }
  }
  closing_handshake(p, 0);
}

// out[t] = sum_j w[t, j] * row(t, j)   (w optional -> 1);  dots[t, j] = <upstream[t], row(t, j)> (optional).
__global__ void pull_rows_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ weights,
                                 const __nv_bfloat16* __restrict__ upstream, float* __restrict__ dots, ExchangeParams p) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int vecs = p.dim >> 3;
  // opening handshake: a peer's buffer may be read once that peer has announced this call (its buffer was
  // filled earlier on its own stream)
  __shared__ int peers_ready;
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0)
      for (int r = 0; r < p.ep; ++r) st_release_sys(p.flag_ptrs[r] + 16 + p.rank, p.epoch);
    bool ok = true;
    for (int r = 0; r < p.ep && ok; ++r) ok = wait_flag(p.flag_ptrs[p.rank] + 16 + r, p.epoch, p.status, 20);
    peers_ready = ok ? 1 : 0;
  }
  __syncthreads();
  for (long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; t < p.tokens && peers_ready; t += warps) {
    for (int v0 = 0; v0 < vecs; v0 += 32) {
      const int v = v0 + lane;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      float up[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (upstream != nullptr && v < vecs) {
        const uint4 q = reinterpret_cast<const uint4*>(upstream + t * p.dim)[v];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); up[2 * j] = f.x; up[2 * j + 1] = f.y; }
      }
      for (int j = 0; j < p.top_k; ++j) {
        const int slot = p.slots[t * p.top_k + j];
        float dot = 0.0f;
        if (slot >= 0 && v < vecs) {
          int r;
          const long long row = dest_row(p, slot, r);
          const uint4 q = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.peer_buffers[r]) + row * p.dim)[v];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
          const float w = weights != nullptr ? weights[t * p.top_k + j] : 1.0f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            acc[2 * i] += w * f.x;
            acc[2 * i + 1] += w * f.y;
            dot += up[2 * i] * f.x + up[2 * i + 1] * f.y;
          }
        }
        if (dots != nullptr) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          if (lane == 0) {
            if (v0 == 0) dots[t * p.top_k + j] = dot;
            else dots[t * p.top_k + j] += dot;
          }
        }
      }
      if (out != nullptr && v < vecs) {
        uint4 q;
        q.x = pack_bf16x2(acc[0], acc[1]);
        q.y = pack_bf16x2(acc[2], acc[3]);
        q.z = pack_bf16x2(acc[4], acc[5]);
        q.w = pack_bf16x2(acc[6], acc[7]);
        reinterpret_cast<uint4*>(out + t * p.dim)[v] = q;
      }
    }
  }
  closing_handshake(p, 8);
}

}  // namespace moe
}  // namespace ajb

extern "C" int ajb_moe_route_fwd(const void* logits, int tokens, int experts, int top_k, int normalize, void* out_experts,
                                 void* out_gates, void* out_probs, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(experts <= 256 && top_k >= 1 && top_k <= moe::kMaxTopK && top_k <= experts,
              "moe route: supports up to 256 experts and top-%d", moe::kMaxTopK);
  if (tokens <= 0) return 0;
  const int threads = 256;
  const long long blocks = ((long long)tokens * 32 + threads - 1) / threads;
  moe::route_fwd_kernel<<<(unsigned)blocks, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const float*)logits, tokens, experts, top_k, normalize, (int*)out_experts, (float*)out_gates, (float*)out_probs);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_moe_assign_slots(const void* experts_of, long long assignments, int num_experts, int capacity,
                                    int stride, void* slots, void* counts, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(stride >= capacity && capacity >= 1, "moe slots: stride must be >= capacity >= 1");
  if (assignments <= 0) return 0;
  moe::assign_slots_kernel<<<num_experts, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const int*)experts_of, assignments, capacity, stride, (int*)slots, (int*)counts);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

struct AjbMoeExchangeArgs {
  int tokens, top_k, dim, ep, rank, local_experts, stride, pad;
  const void* slots;
  void* peer_buffers[8];
  void* flag_ptrs[8];
  void* peer_counts[8];
  const void* counts;
  unsigned int epoch;
  unsigned int pad2;
  void* local_counter;
};

static void fill_params(const AjbMoeExchangeArgs& a, ajb::moe::ExchangeParams& p) {
  p.tokens = a.tokens; p.top_k = a.top_k; p.dim = a.dim; p.ep = a.ep; p.rank = a.rank;
  p.local_experts = a.local_experts; p.stride = a.stride; p.slots = (const int*)a.slots;
  for (int r = 0; r < 8; ++r) {
    p.peer_buffers[r] = a.peer_buffers[r];
    p.flag_ptrs[r] = (unsigned int*)a.flag_ptrs[r];
    p.peer_counts[r] = (int*)a.peer_counts[r];
  }
  p.counts = (const int*)a.counts;
  p.epoch = a.epoch;
  p.local_counter = (unsigned int*)a.local_counter;
  p.status = ajb::device_status_buffer();
}

// Dispatch: rows [tokens, dim] bf16 -> peers' expert-major buffers; scale may be null.
extern "C" int ajb_moe_push_rows(const AjbMoeExchangeArgs* args, const void* rows, const void* scale, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(args->dim % 8 == 0 && args->ep >= 1 && args->ep <= 8, "moe push: dim must be a multiple of 8, ep <= 8");
  moe::ExchangeParams p;
  fill_params(*args, p);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  AJB_CUDA_OK(cudaMemsetAsync(args->local_counter, 0, sizeof(unsigned int), s));
  const int grid = sm_count() * 4;
  moe::push_rows_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)rows, (const float*)scale, p);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Combine: out [tokens, dim] (may be null), weights [tokens, top_k] (may be null), upstream / dots (may be null).
extern "C" int ajb_moe_pull_rows(const AjbMoeExchangeArgs* args, void* out, const void* weights, const void* upstream,
                                 void* dots, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(args->dim % 8 == 0 && args->ep >= 1 && args->ep <= 8, "moe pull: dim must be a multiple of 8, ep <= 8");
  moe::ExchangeParams p;
  fill_params(*args, p);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  AJB_CUDA_OK(cudaMemsetAsync(args->local_counter, 0, sizeof(unsigned int), s));
  const int grid = sm_count() * 4;
  moe::pull_rows_kernel<<<grid, 256, 0, s>>>((__nv_bfloat16*)out, (const float*)weights, (const __nv_bfloat16*)upstream,
                                             (float*)dots, p);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}
