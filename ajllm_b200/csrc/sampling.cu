// Token selection on the GPU: batched temperature / top-p / greedy sampling and the speculative
// decoding accept-reject step. One CTA per row (sampler) or per sequence (verify); the vocabulary row
// is streamed from global memory (L2-resident between passes), nothing is sorted.
//
// Sampler semantics (same distribution as ajllm/generation/sampling.py:8-22): temperature <= 0 picks
// the argmax; otherwise p = softmax(logits / T); with top_p < 1 the kept set is the shortest prefix
// of the tokens in decreasing-probability order whose preceding mass is still below top_p, found here
// by bisection on the probability threshold; one token is drawn from the kept, renormalised mass.
// Random numbers are a counter-based hash of (seed, draw index), so a request's stream does not depend
// on which other requests share its batch.
//
// Verify semantics: draft token d_i is accepted with probability min(1, p_i(d_i) / q_i(d_i)); the first
// rejected position is re-drawn from normalise(max(0, p_i - q_i)); when all k are accepted a bonus token
// is drawn from p_k. With temperature 0 this is "accept while d_i equals the target argmax".
#include "common.cuh"

namespace ajb {
namespace sampling {

constexpr int kThreads = 512;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.0f;
  return warp_sum(t);
}
__device__ float block_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : -INFINITY;
  return warp_max(t);
}

// uniform in [0, 1) from (seed, counter)
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long counter) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (counter + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

struct RowStats {
  float max_logit;
  float sum_exp;   // sum of exp((x - max) * inv_t)
  int argmax;
};

// Pass 1 for small batches: `chunks` CTAs per row each find the maximum (and its first index) of one slice of the
// vocabulary, so that a handful of rows over a 128k vocabulary are read by a hundred CTAs instead of a handful.
// part[(row * chunks + c) * 2] = {max as float bits, index}.
__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float* __restrict__ logits, long long row_pitch, int vocab, int chunks, int* __restrict__ part) {
  __shared__ float red[32];
  __shared__ int red_i[32];
  const int r = blockIdx.y, c = blockIdx.x;
  const float* row = logits + (size_t)r * row_pitch;
  const int per = ((vocab + chunks - 1) / chunks + 3) & ~3;
  const int lo = c * per, hi = min(vocab, lo + per);
  float mx = -INFINITY;
  int arg = 0x7fffffff;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  if (vec) {
    const int hi4 = lo + ((hi - lo) & ~3);
    for (int i = lo + 4 * (int)threadIdx.x; i < hi4; i += 4 * (int)blockDim.x) {
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      if (v.x > mx) { mx = v.x; arg = i; }
      if (v.y > mx) { mx = v.y; arg = i + 1; }
      if (v.z > mx) { mx = v.z; arg = i + 2; }
      if (v.w > mx) { mx = v.w; arg = i + 3; }
    }
    for (int i = hi4 + (int)threadIdx.x; i < hi; i += (int)blockDim.x) {
      const float x = row[i];
      if (x > mx) { mx = x; arg = i; }
    }
  } else {
    for (int i = lo + (int)threadIdx.x; i < hi; i += (int)blockDim.x) {
      const float x = row[i];
      if (x > mx) { mx = x; arg = i; }
    }
  }
  const float gmax = block_max(mx, red);
  int cand = (mx == gmax && lo < hi) ? arg : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red_i[threadIdx.x >> 5] = cand;
  __syncthreads();
  if (threadIdx.x == 0) {
    int best = 0x7fffffff;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) best = min(best, red_i[w]);
    part[((size_t)r * chunks + c) * 2] = __float_as_int(gmax);
    part[((size_t)r * chunks + c) * 2 + 1] = best;
  }
}

// Greedy rows (`need_sum` false) only need the argmax, i.e. one pass over the row. Rows that start on a 16-byte
// boundary with a vocabulary that is a multiple of 4 are read as float4.
// With `part` (pass 1 done by argmax_chunks_kernel) the maximum comes from the `chunks` partial results.
__device__ RowStats row_stats(const float* __restrict__ row, int vocab, float inv_t, bool need_sum, float* red, int* red_i,
                              const int* __restrict__ part = nullptr, int chunks = 0) {
  float mx = -INFINITY;
  int arg = 0;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0 && (vocab & 3) == 0;
  if (part != nullptr) {
    // chunks are in index order, so a strict comparison keeps the smallest index among equal maxima
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
      const float v = __int_as_float(part[2 * c]);
      if (v > mx) { mx = v; arg = part[2 * c + 1]; }
    }
  } else if (vec) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int i = threadIdx.x; i < (vocab >> 2); i += blockDim.x) {
      const float4 v = row4[i];
      // increasing index and a strict comparison keep the smallest index among equal values
      if (v.x > mx) { mx = v.x; arg = 4 * i; }
      if (v.y > mx) { mx = v.y; arg = 4 * i + 1; }
      if (v.z > mx) { mx = v.z; arg = 4 * i + 2; }
      if (v.w > mx) { mx = v.w; arg = 4 * i + 3; }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float x = row[i];
      if (x > mx) { mx = x; arg = i; }
    }
  }
  const float gmax = block_max(mx, red);
  // smallest index among the maxima
  int cand = (mx == gmax) ? arg : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red_i[threadIdx.x >> 5] = cand;
  __syncthreads();
  int best = 0x7fffffff;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) best = min(best, red_i[w]);
  RowStats out;
  out.max_logit = gmax;
  out.argmax = best;
  out.sum_exp = 1.0f;
  if (need_sum) {
    float s = 0.0f;
    if (vec) {
      const float4* row4 = reinterpret_cast<const float4*>(row);
      for (int i = threadIdx.x; i < (vocab >> 2); i += blockDim.x) {
        const float4 v = row4[i];
        s += __expf((v.x - gmax) * inv_t) + __expf((v.y - gmax) * inv_t) + __expf((v.z - gmax) * inv_t) +
             __expf((v.w - gmax) * inv_t);
      }
    } else {
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) s += __expf((row[i] - gmax) * inv_t);
    }
    out.sum_exp = block_sum(s, red);
  }
  return out;
}

// Index of the first element (vocabulary order) at which the running sum of weight(i) exceeds `target`.
template <class Weight>
__device__ int pick_by_mass(int vocab, float target, Weight weight, float* red, int* red_i) {
  // pass 1: per-thread contiguous chunk sums; pass 2: locate inside the owning chunk
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * per, hi = min(vocab, lo + per);
  float mine = 0.0f;
  for (int i = lo; i < hi; ++i) mine += weight(i);
  __shared__ float chunk[kThreads];
  chunk[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.0f;
    int owner = blockDim.x - 1;
    float before = 0.0f;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      if (run + chunk[t] > target) { owner = t; before = run; break; }
      run += chunk[t];
      before = run;
    }
    // if rounding pushed the target past the total, fall back to the last non-empty chunk
    if (owner == (int)blockDim.x - 1 && run + chunk[owner] <= target) {
      while (owner > 0 && chunk[owner] <= 0.0f) --owner;
      before = 0.0f;
      for (int t = 0; t < owner; ++t) before += chunk[t];
    }
    red_i[0] = owner;
    red[0] = before;
  }
  __syncthreads();
  const int owner = red_i[0];
  const float before = red[0];
  __syncthreads();
  if ((int)threadIdx.x == owner) {
    float run = before;
    int found = -1, last_positive = -1;
    for (int i = lo; i < hi; ++i) {
      const float w = weight(i);
      if (w > 0.0f) last_positive = i;
      run += w;
      if (run > target) { found = i; break; }
    }
    red_i[1] = found >= 0 ? found : max(last_positive, lo < vocab ? lo : vocab - 1);
  }
  __syncthreads();
  return red_i[1];
}

__global__ void __launch_bounds__(kThreads)
sample_rows_kernel(const float* __restrict__ logits, long long row_pitch, int vocab, const float* __restrict__ temperature,
                   const float* __restrict__ top_p, const unsigned long long* __restrict__ seeds,
                   const unsigned long long* __restrict__ counters, int* __restrict__ out_tokens,
                   const int* __restrict__ part, int chunks) {
  __shared__ float red[32];
  __shared__ int red_i[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_pitch;
  const float temp = temperature[r];
  const float inv_t = temp > 0.0f ? 1.0f / temp : 1.0f;
  const RowStats st = row_stats(row, vocab, inv_t, temp > 0.0f, red, red_i,
                                part != nullptr ? part + (size_t)r * chunks * 2 : nullptr, chunks);
  if (temp <= 0.0f) {
    if (threadIdx.x == 0) out_tokens[r] = st.argmax;
    return;
  }
  const float inv_sum = 1.0f / st.sum_exp;
  const float gmax = st.max_logit;
  auto prob = [&](int i) { return __expf((row[i] - gmax) * inv_t) * inv_sum; };
  float threshold = 0.0f;
  const float want = top_p ? top_p[r] : 1.0f;
  float kept_mass = 1.0f;
  if (want < 1.0f) {
    // largest t with mass(p >= t) >= want
    float lo = 0.0f, hi = inv_sum;       // the largest probability is exp(0) / sum
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (lo + hi);
      float m = 0.0f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float pr = prob(i);
        m += pr >= mid ? pr : 0.0f;
      }
      m = block_sum(m, red);
      if (m >= want) lo = mid; else hi = mid;
    }
    threshold = lo;
    float m = 0.0f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float pr = prob(i);
      m += pr >= threshold ? pr : 0.0f;
    }
    kept_mass = block_sum(m, red);
  }
  const float u = uniform01(seeds[r], counters[r]) * kept_mass;
  const int token = pick_by_mass(vocab, u, [&](int i) { const float pr = prob(i); return pr >= threshold ? pr : 0.0f; }, red, red_i);
  if (threadIdx.x == 0) out_tokens[r] = token;
}

// One CTA per sequence. target_logits [seqs, k + 1, vocab], draft_logits [seqs, k, vocab], draft_tokens [seqs, k].
// result[seq] = {accepted, next_token}.
__global__ void __launch_bounds__(kThreads)
spec_verify_kernel(const float* __restrict__ target_logits, const float* __restrict__ draft_logits,
                   const int* __restrict__ draft_tokens, int k, int vocab, const float* __restrict__ temperature,
                   const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
                   int* __restrict__ result) {
  __shared__ float red[32];
  __shared__ int red_i[32];
  const int s = blockIdx.x;
  const float temp = temperature[s];
  const float* trow = target_logits + (size_t)s * (k + 1) * vocab;
  const float* drow = draft_logits + (size_t)s * k * vocab;
  const int* tokens = draft_tokens + (size_t)s * k;
  const float inv_t = temp > 0.0f ? 1.0f / temp : 1.0f;
  int accepted = 0;
  int next_token = -1;
  for (int i = 0; i < k; ++i) {
    const RowStats ts = row_stats(trow + (size_t)i * vocab, vocab, inv_t, temp > 0.0f, red, red_i);
    const int d = tokens[i];
    if (temp <= 0.0f) {
      if (d == ts.argmax) { ++accepted; continue; }
      next_token = ts.argmax;
      break;
    }
    const RowStats ds = row_stats(drow + (size_t)i * vocab, vocab, inv_t, true, red, red_i);
    const float* tr = trow + (size_t)i * vocab;
    const float* dr = drow + (size_t)i * vocab;
    const float p = __expf((tr[d] - ts.max_logit) * inv_t) / ts.sum_exp;
    const float q = __expf((dr[d] - ds.max_logit) * inv_t) / ds.sum_exp;
    const float u = uniform01(seeds[s], counters[s] + 2 * i);
    if (q > 0.0f && u * q <= p) { ++accepted; continue; }
    // rejected: draw from the normalised positive part of p - q
    const float ti = 1.0f / ts.sum_exp, di = 1.0f / ds.sum_exp;
    const float tmax = ts.max_logit, dmax = ds.max_logit;
    auto residual = [&](int j) {
      return fmaxf(0.0f, __expf((tr[j] - tmax) * inv_t) * ti - __expf((dr[j] - dmax) * inv_t) * di);
    };
    float m = 0.0f;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) m += residual(j);
    m = block_sum(m, red);
    const float u2 = uniform01(seeds[s], counters[s] + 2 * i + 1);
    if (m > 0.0f) {
      next_token = pick_by_mass(vocab, u2 * m, residual, red, red_i);
    } else {   // p == q everywhere: a draw from p is a valid correction
      next_token = pick_by_mass(vocab, u2, [&](int j) { return __expf((tr[j] - tmax) * inv_t) * ti; }, red, red_i);
    }
    break;
  }
  if (next_token < 0) {   // every draft token accepted: bonus token from the last target row
    const float* tr = trow + (size_t)k * vocab;
    const RowStats ts = row_stats(tr, vocab, inv_t, temp > 0.0f, red, red_i);
    if (temp <= 0.0f) {
      next_token = ts.argmax;
    } else {
      const float ti = 1.0f / ts.sum_exp, tmax = ts.max_logit;
      const float u = uniform01(seeds[s], counters[s] + 2 * k);
      next_token = pick_by_mass(vocab, u, [&](int j) { return __expf((tr[j] - tmax) * inv_t) * ti; }, red, red_i);
    }
  }
  if (threadIdx.x == 0) {
    result[2 * s] = accepted;
    result[2 * s + 1] = next_token;
  }
}

}  // namespace sampling
}  // namespace ajb

// chunks > 1 (with `workspace` of rows * chunks * 2 ints): the row maxima are found by rows * chunks CTAs first, and
// greedy rows then only combine `chunks` partial results.
extern "C" int ajb_sample_rows(const void* logits, long long row_pitch, int rows, int vocab, const void* temperature,
                               const void* top_p, const void* seeds, const void* counters, void* out_tokens,
                               int chunks, void* workspace, void* stream) {
  using namespace ajb;
  if (rows <= 0) return 0;
  AJB_REQUIRE(chunks >= 1 && chunks <= 512 && (chunks == 1 || workspace != nullptr),
              "sample_rows: chunks must be in [1, 512] and come with a workspace");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int* part = nullptr;
  if (chunks > 1) {
    sampling::argmax_chunks_kernel<<<dim3(chunks, rows), 256, 0, s>>>((const float*)logits, row_pitch, vocab, chunks,
                                                                      (int*)workspace);
    AJB_CUDA_OK(cudaGetLastError());
    part = (const int*)workspace;
  }
  sampling::sample_rows_kernel<<<rows, sampling::kThreads, 0, s>>>(
      (const float*)logits, row_pitch, vocab, (const float*)temperature, (const float*)top_p,
      (const unsigned long long*)seeds, (const unsigned long long*)counters, (int*)out_tokens, part, chunks);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_spec_verify(const void* target_logits, const void* draft_logits, const void* draft_tokens, int seqs,
                               int k, int vocab, const void* temperature, const void* seeds, const void* counters,
                               void* result, void* stream) {
  using namespace ajb;
  AJB_REQUIRE(k >= 1, "spec verify: k must be positive");
  if (seqs <= 0) return 0;
  sampling::spec_verify_kernel<<<seqs, sampling::kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const float*)target_logits, (const float*)draft_logits, (const int*)draft_tokens, k, vocab,
      (const float*)temperature, (const unsigned long long*)seeds, (const unsigned long long*)counters, (int*)result);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}
