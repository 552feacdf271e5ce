// Bandwidth-bound kernels of the training path: fused residual-add + RMSNorm (fwd/bwd), interleaved
// RoPE on packed q|k|v rows, SwiGLU on interleaved gate/up columns, row-wise softmax cross-entropy
// that overwrites logits with their gradient, embedding gather / scatter-add, squared-norm
// reduction and the flat AdamW update. All activations are bf16, statistics and optimizer state fp32;
// every kernel moves 16 bytes per thread per access.
#include "common.cuh"

namespace ajb {
namespace pw {

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const Bf16x8& in, float (&out)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(in.v[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ Bf16x8 pack8(const float (&in)[8]) {
  Bf16x8 out;
#pragma unroll
  for (int i = 0; i < 4; ++i) out.v[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
  return out;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

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
// Sum over the block; every thread receives the result. `red` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nwarps ? red[lane] : 0.0f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nwarps ? red[lane] : -INFINITY;
  return warp_max(t);
}

// ------------------------------------------------------------------------------------------ RMSNorm
constexpr int kNormThreads = 256;
constexpr int kNormVecLimit = 4;  // row cached in registers up to 256*4*8 = 8192 features (template: 1, 2 or 4 vectors per thread)

// h = x (+ delta); y = h * rsqrt(mean(h^2) + eps) * gain. Writes h only when delta is given.
template <int kNormMaxVec>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                   const __nv_bfloat16* __restrict__ gain, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int rows, int dim, float eps) {
  __shared__ float red[32];
  const int nvec = dim >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + (size_t)row * dim);
    const Bf16x8* dr = delta ? reinterpret_cast<const Bf16x8*>(delta + (size_t)row * dim) : nullptr;
    float cache[kNormMaxVec][8];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        unpack8(xr[v], cache[i]);
        if (dr) {
          float d[8];
          unpack8(dr[v], d);
#pragma unroll
          for (int j = 0; j < 8; ++j) cache[i][j] += d[j];
          // the residual stream is stored in bf16: normalise exactly what later layers will read
          Bf16x8 hq = pack8(cache[i]);
          reinterpret_cast<Bf16x8*>(h_out + (size_t)row * dim)[v] = hq;
          unpack8(hq, cache[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += cache[i][j] * cache[i][j];
      }
    }
    const float total = block_sum(ss, red);
    const float rstd = rsqrtf(total / (float)dim + eps);
    if (threadIdx.x == 0) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float g[8], o[8];
        unpack8(reinterpret_cast<const Bf16x8*>(gain)[v], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = cache[i][j] * rstd * g[j];
        reinterpret_cast<Bf16x8*>(y + (size_t)row * dim)[v] = pack8(o);
      }
    }
  }
}

// dx = rstd * (gain*dy - xhat * mean(gain*dy*xhat)) (+ dh), xhat = h * rstd.
// Block b accumulates sum_rows dy*xhat for its rows into partial[b, :].
template <int kNormMaxVec>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ gain, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dh, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ partial, int rows, int dim) {
  __shared__ float red[32];
  const int nvec = dim >> 3;
  float gacc[kNormMaxVec][8];
  float g[kNormMaxVec][8];
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) gacc[i][j] = 0.0f;
    if (v < nvec) unpack8(reinterpret_cast<const Bf16x8*>(gain)[v], g[i]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float xh[kNormMaxVec][8], gy[kNormMaxVec][8];
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float hv[8], dyv[8];
        unpack8(reinterpret_cast<const Bf16x8*>(h + (size_t)row * dim)[v], hv);
        unpack8(reinterpret_cast<const Bf16x8*>(dy + (size_t)row * dim)[v], dyv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = hv[j] * rstd;
          gacc[i][j] += dyv[j] * xh[i][j];
          gy[i][j] = dyv[j] * g[i][j];
          dot += gy[i][j] * xh[i][j];
        }
      }
    }
    const float mean_dot = block_sum(dot, red) / (float)dim;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (gy[i][j] - xh[i][j] * mean_dot);
        if (dh) {
          float r[8];
          unpack8(reinterpret_cast<const Bf16x8*>(dh + (size_t)row * dim)[v], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        reinterpret_cast<Bf16x8*>(dx + (size_t)row * dim)[v] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kNormMaxVec; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
      float* dst = partial + (size_t)blockIdx.x * dim + v * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(gacc[i][0], gacc[i][1], gacc[i][2], gacc[i][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(gacc[i][4], gacc[i][5], gacc[i][6], gacc[i][7]);
    }
  }
}

// out[c] (+)= sum_r in[r, c]. One CTA owns 32 columns; its 8 warps take every 8th row (a warp reads 128
// contiguous bytes per row) and their partial sums meet in shared memory in a fixed order. Accumulation is one
// atomic add per column, so two launches on different streams (two micro-batches in flight) may target the same
// gradient buffer.
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ in, float* __restrict__ out, int rows,
                                                     int cols, int accumulate) {
  __shared__ float part[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s0 = 0.0f, s1 = 0.0f;
  if (c < cols) {
    int r = warp;
    for (; r + 8 < rows; r += 16) {
      s0 += in[(size_t)r * cols + c];
      s1 += in[(size_t)(r + 8) * cols + c];
    }
    if (r < rows) s0 += in[(size_t)r * cols + c];
  }
  part[warp][lane] = s0 + s1;
  __syncthreads();
  if (warp == 0 && c < cols) {
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += part[w][lane];
    if (accumulate) atomicAdd(out + c, s);
    else out[c] = s;
  }
}

// ------------------------------------------------------------------------------------------ RoPE
// Rotates pairs (x[2i], x[2i+1]) of every q and k head of each packed row in place.
__global__ void rope_qk_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                               const float* __restrict__ sin_t, const int* __restrict__ positions, int rows, int seq,
                               int rot_heads, int head_dim, long long row_stride, float sin_sign) {
  const int vec_per_head = head_dim >> 3;
  const int vec_per_row = rot_heads * vec_per_head;
  const long long total = (long long)rows * vec_per_row;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(idx / vec_per_row);
    const int rem = (int)(idx - (long long)row * vec_per_row);
    const int head = rem / vec_per_head;
    const int v = rem - head * vec_per_head;
    const int pos = positions ? positions[row] : row % seq;
    Bf16x8* ptr = reinterpret_cast<Bf16x8*>(qkv + (size_t)row * row_stride + head * head_dim) + v;
    float x[8], o[8];
    unpack8(*ptr, x);
    const float4 c = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * (head_dim >> 1) + v * 4);
    const float4 s = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * (head_dim >> 1) + v * 4);
    const float cc[4] = {c.x, c.y, c.z, c.w};
    const float ss[4] = {s.x * sin_sign, s.y * sin_sign, s.z * sin_sign, s.w * sin_sign};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] = x[2 * i] * cc[i] - x[2 * i + 1] * ss[i];
      o[2 * i + 1] = x[2 * i] * ss[i] + x[2 * i + 1] * cc[i];
    }
    *ptr = pack8(o);
  }
}

// ------------------------------------------------------------------------------------------ SwiGLU
// One thread per 16-byte vector of the interleaved (gate, up) columns: neighbouring threads touch neighbouring
// 16 bytes of the wide tensor and neighbouring 8 bytes of the narrow one, so every sector that moves is used whole.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ act,
                                  long long total_vec /* rows * F / 4: vectors of four (gate, up) pairs */) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_vec;
       idx += (long long)gridDim.x * blockDim.x) {
    float a[8];
    unpack8(reinterpret_cast<const Bf16x8*>(gate_up)[idx], a);
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float g = a[2 * i], u = a[2 * i + 1];
      o[i] = g / (1.0f + __expf(-g)) * u;
    }
    uint2 packed;
    packed.x = pack2(o[0], o[1]);
    packed.y = pack2(o[2], o[3]);
    reinterpret_cast<uint2*>(act)[idx] = packed;
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gate_up, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dgate_up, long long total_vec) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_vec;
       idx += (long long)gridDim.x * blockDim.x) {
    float a[8], oa[8];
    unpack8(reinterpret_cast<const Bf16x8*>(gate_up)[idx], a);
    const uint2 dv = reinterpret_cast<const uint2*>(dact)[idx];
    const float2 d01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.x));
    const float2 d23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.y));
    const float d[4] = {d01.x, d01.y, d23.x, d23.y};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float g = a[2 * i], u = a[2 * i + 1], sig = 1.0f / (1.0f + __expf(-g));
      oa[2 * i] = d[i] * u * sig * (1.0f + g * (1.0f - sig));
      oa[2 * i + 1] = d[i] * g * sig;
    }
    reinterpret_cast<Bf16x8*>(dgate_up)[idx] = pack8(oa);
  }
}

// Head repacking: rows of `heads` heads of `src_hd` elements each -> rows of `heads` heads of `dst_hd` elements. A wider
// destination head is zero-filled behind the copied part, a narrower one keeps the leading part. The attention kernels
// are built for 64- and 128-wide heads; other head sizes (the reference's own flagship has 32) run on them through
// this zero padding, which changes neither the scores (zeros add nothing to q . k) nor the kept output columns.
__global__ void repack_heads_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows,
                                    int heads, int src_hd, int dst_hd, long long src_stride, long long dst_stride) {
  const int dst_vec = dst_hd >> 3, src_vec = src_hd >> 3;
  const long long per_row = (long long)heads * dst_vec;
  const long long total = rows * per_row;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long row = idx / per_row;
    const int rem = (int)(idx - row * per_row);
    const int head = rem / dst_vec, v = rem - head * dst_vec;
    uint4 q = make_uint4(0u, 0u, 0u, 0u);
    if (v < src_vec) q = reinterpret_cast<const uint4*>(src + row * src_stride + (long long)head * src_hd)[v];
    reinterpret_cast<uint4*>(dst + row * dst_stride + (long long)head * dst_hd)[v] = q;
  }
}

// SiLU feed-forward activation (the reference's non-gated option): y = x * sigmoid(x); with `dy` the derivative
// dy * sigmoid(x) * (1 + x * (1 - sigmoid(x))) is written instead.
__global__ void silu_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                            __nv_bfloat16* __restrict__ out, long long total_vec) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_vec;
       idx += (long long)gridDim.x * blockDim.x) {
    float a[8], d[8], o[8];
    unpack8(reinterpret_cast<const Bf16x8*>(x)[idx], a);
    if (dy != nullptr) unpack8(reinterpret_cast<const Bf16x8*>(dy)[idx], d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sig = 1.0f / (1.0f + __expf(-a[i]));
      o[i] = dy != nullptr ? d[i] * sig * (1.0f + a[i] * (1.0f - sig)) : a[i] * sig;
    }
    reinterpret_cast<Bf16x8*>(out)[idx] = pack8(o);
  }
}

// ------------------------------------------------------------------------------------------ cross-entropy
// One block per row: online (max, sum-exp) over the vocabulary, loss += lse - logit[target];
// optionally overwrite the row with (softmax - onehot) * grad_scale.
constexpr int kCeThreads = 512;
__global__ void __launch_bounds__(kCeThreads)
ce_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ loss_sum,
          int rows, int vocab, long long ld, float grad_scale, int write_grad) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  __nv_bfloat16* lr = logits + (size_t)row * ld;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(lr) & 15) == 0);
  const int nvec = vec_ok ? (vocab >> 3) : 0;
  float mx = -INFINITY, sum = 0.0f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float x[8];
    unpack8(reinterpret_cast<const Bf16x8*>(lr)[v], x);
    float local = x[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) local = fmaxf(local, x[j]);
    if (local > mx) {
      sum *= __expf(mx - local);
      mx = local;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += __expf(x[j] - mx);
  }
  for (int c = nvec * 8 + threadIdx.x; c < vocab; c += blockDim.x) {
    const float x = __bfloat162float(lr[c]);
    if (x > mx) {
      sum *= __expf(mx - x);
      mx = x;
    }
    sum += __expf(x - mx);
  }
  const float gmax = block_max(mx, red);
  const float gsum = block_sum(mx == -INFINITY ? 0.0f : sum * __expf(mx - gmax), red);
  const float lse = gmax + __logf(gsum);
  const long long target = targets[row];
  if (threadIdx.x == 0) {
    const float picked = (target >= 0 && target < vocab) ? __bfloat162float(lr[target]) : lse;
    atomicAdd(loss_sum, lse - picked);
  }
  if (!write_grad) return;
  __syncthreads();  // thread 0 has read the target logit
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float x[8];
    unpack8(reinterpret_cast<const Bf16x8*>(lr)[v], x);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float pr = __expf(x[j] - lse);
      x[j] = (pr - ((long long)(v * 8 + j) == target ? 1.0f : 0.0f)) * grad_scale;
    }
    reinterpret_cast<Bf16x8*>(lr)[v] = pack8(x);
  }
  for (int c = nvec * 8 + threadIdx.x; c < vocab; c += blockDim.x) {
    const float pr = __expf(__bfloat162float(lr[c]) - lse);
    lr[c] = __float2bfloat16((pr - ((long long)c == target ? 1.0f : 0.0f)) * grad_scale);
  }
}

// ------------------------------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int tokens, int dim, int vocab) {
  const int nvec = dim >> 3;
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    long long id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const Bf16x8* src = reinterpret_cast<const Bf16x8*>(table + (size_t)id * dim);
    Bf16x8* dst = reinterpret_cast<Bf16x8*>(out + (size_t)t * dim);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = src[v];
  }
}

__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ grad,
                                     float* __restrict__ table_grad, int tokens, int dim, int vocab) {
  const int nvec = dim >> 3;
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    const long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    const Bf16x8* src = reinterpret_cast<const Bf16x8*>(grad + (size_t)t * dim);
    float* dst = table_grad + (size_t)id * dim;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float g[8];
      unpack8(src[v], g);
      atomicAdd(reinterpret_cast<float4*>(dst + v * 8), make_float4(g[0], g[1], g[2], g[3]));
      atomicAdd(reinterpret_cast<float4*>(dst + v * 8 + 4), make_float4(g[4], g[5], g[6], g[7]));
    }
  }
}

// ------------------------------------------------------------------------------------------ norm + AdamW
constexpr int kSumsqBlocks = 1024;
constexpr int kSumsqThreads = 256;

// Stage 1: partial[b] = sum of squares of block b's grid-stride slice (fixed order -> deterministic).
__global__ void __launch_bounds__(kSumsqThreads)
sumsq_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.0f;
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long long i = nvec * 4 + threadIdx.x; i < n; i += blockDim.x) s += x[i] * x[i];
  const float total = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = total;
}
// Stage 2: out[0] = sum(partial[0..count)).
__global__ void __launch_bounds__(kSumsqThreads)
sumsq_final_kernel(const float* __restrict__ partial, int count, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.0f;
  for (int i = threadIdx.x; i < count; i += blockDim.x) s += partial[i];
  const float total = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = total;
}

// master/m/v fp32, grad fp32; clip = min(1, max_norm / (sqrt(*sumsq) + 1e-6)) when sumsq != null.
__global__ void adamw_flat_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m,
                                  float* __restrict__ v, __nv_bfloat16* __restrict__ working, long long n,
                                  float step_size, float beta1, float beta2, float eps, float decay,
                                  const float* __restrict__ sumsq, float max_norm) {
  float clip = 1.0f;
  if (sumsq != nullptr && max_norm > 0.0f) {
    const float norm = sqrtf(*sumsq);
    if (norm > max_norm) clip = max_norm / (norm + 1e-6f);
  }
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(master)[i];
    const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float pp[4] = {p.x, p.y, p.z, p.w};
    const float gg[4] = {g4.x * clip, g4.y * clip, g4.z * clip, g4.w * clip};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mm[j] = beta1 * mm[j] + (1.0f - beta1) * gg[j];
      vv[j] = beta2 * vv[j] + (1.0f - beta2) * gg[j] * gg[j];
      pp[j] = (pp[j] - step_size * mm[j] / (sqrtf(vv[j]) + eps)) * decay;
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (working != nullptr) {
      uint2 w;
      w.x = pack_bf16x2(pp[0], pp[1]);
      w.y = pack_bf16x2(pp[2], pp[3]);
      reinterpret_cast<uint2*>(working)[i] = w;
    }
  }
  if (blockIdx.x == 0) {
    for (long long i = nvec * 4 + threadIdx.x; i < n; i += blockDim.x) {
      const float g = grad[i] * clip;
      const float mi = beta1 * m[i] + (1.0f - beta1) * g;
      const float vi = beta2 * v[i] + (1.0f - beta2) * g * g;
      const float pi = (master[i] - step_size * mi / (sqrtf(vi) + eps)) * decay;
      m[i] = mi; v[i] = vi; master[i] = pi;
      if (working != nullptr) working[i] = __float2bfloat16(pi);
    }
  }
}

__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    unpack8(reinterpret_cast<const Bf16x8*>(a)[i], x);
    unpack8(reinterpret_cast<const Bf16x8*>(b)[i], y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    reinterpret_cast<Bf16x8*>(out)[i] = pack8(x);
  }
}

static inline int grid_for(long long work_items, int threads, int per_sm = 8) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = (long long)sm_count() * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace pw
}  // namespace ajb

using namespace ajb;
using namespace ajb::pw;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
typedef __nv_bfloat16 bf16;

extern "C" int ajb_rmsnorm_fwd(const void* x, const void* delta, const void* gain, void* y, void* h_out, void* rstd,
                               int rows, int dim, float eps, void* stream) {
  AJB_REQUIRE(dim % 8 == 0 && dim <= kNormThreads * kNormVecLimit * 8, "rmsnorm: dim %d must be a multiple of 8 and <= %d",
              dim, kNormThreads * kNormVecLimit * 8);
  AJB_REQUIRE(delta == nullptr || h_out != nullptr, "rmsnorm: h_out is required when delta is given");
  if (rows <= 0) return 0;
  const int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
  const int vecs = (dim / 8 + kNormThreads - 1) / kNormThreads;
#define AJB_NORM_FWD(V) rmsnorm_fwd_kernel<V><<<grid, kNormThreads, 0, STREAM(stream)>>>( \
      (const bf16*)x, (const bf16*)delta, (const bf16*)gain, (bf16*)y, (bf16*)h_out, (float*)rstd, rows, dim, eps)
  if (vecs <= 1) AJB_NORM_FWD(1); else if (vecs == 2) AJB_NORM_FWD(2); else AJB_NORM_FWD(4);
#undef AJB_NORM_FWD
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

// partial must hold nparts * dim floats; the launch uses exactly nparts blocks.
extern "C" int ajb_rmsnorm_bwd(const void* dy, const void* h, const void* gain, const void* rstd, const void* dh,
                               void* dx, void* partial, int rows, int dim, int nparts, void* stream) {
  AJB_REQUIRE(dim % 8 == 0 && dim <= kNormThreads * kNormVecLimit * 8, "rmsnorm_bwd: unsupported dim %d", dim);
  AJB_REQUIRE(nparts >= 1, "rmsnorm_bwd: nparts must be positive");
  if (rows <= 0) return 0;
  const int vecs = (dim / 8 + kNormThreads - 1) / kNormThreads;
#define AJB_NORM_BWD(V) rmsnorm_bwd_kernel<V><<<nparts, kNormThreads, 0, STREAM(stream)>>>( \
      (const bf16*)dy, (const bf16*)h, (const bf16*)gain, (const float*)rstd, (const bf16*)dh, (bf16*)dx, (float*)partial, rows, dim)
  if (vecs <= 1) AJB_NORM_BWD(1); else if (vecs == 2) AJB_NORM_BWD(2); else AJB_NORM_BWD(4);
#undef AJB_NORM_BWD
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_colsum_f32(const void* in, void* out, int rows, int cols, int accumulate, void* stream) {
  colsum_kernel<<<(cols + 31) / 32, 256, 0, STREAM(stream)>>>((const float*)in, (float*)out, rows, cols, accumulate);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Rotates the first (num_heads + num_kv_heads) heads of each packed row. inverse != 0 applies the
// transposed rotation (the gradient of the forward rotation).
extern "C" int ajb_rope_qk(void* qkv, const void* cos_t, const void* sin_t, const void* positions, int rows, int seq,
                           int num_heads, int num_kv_heads, int head_dim, long long row_stride, int inverse,
                           void* stream) {
  AJB_REQUIRE(head_dim % 8 == 0 && row_stride % 8 == 0, "rope: head_dim and row stride must be multiples of 8");
  const int rot_heads = num_heads + num_kv_heads;
  const long long total = (long long)rows * rot_heads * (head_dim / 8);
  if (total <= 0) return 0;
  rope_qk_kernel<<<grid_for(total, 256), 256, 0, STREAM(stream)>>>((bf16*)qkv, (const float*)cos_t, (const float*)sin_t,
                                                                    (const int*)positions, rows, seq, rot_heads,
                                                                    head_dim, row_stride, inverse ? -1.0f : 1.0f);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_swiglu_fwd(const void* gate_up, void* act, long long rows, int ff, void* stream) {
  AJB_REQUIRE(ff % 8 == 0, "swiglu: width %d must be a multiple of 8", ff);
  const long long total = rows * (ff / 4);
  if (total <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for(total, 256), 256, 0, STREAM(stream)>>>((const bf16*)gate_up, (bf16*)act, total);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_swiglu_bwd(const void* gate_up, const void* dact, void* dgate_up, long long rows, int ff,
                              void* stream) {
  AJB_REQUIRE(ff % 8 == 0, "swiglu: width %d must be a multiple of 8", ff);
  const long long total = rows * (ff / 4);
  if (total <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for(total, 256), 256, 0, STREAM(stream)>>>((const bf16*)gate_up, (const bf16*)dact,
                                                                       (bf16*)dgate_up, total);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_repack_heads(const void* src, void* dst, long long rows, int heads, int src_hd, int dst_hd,
                                long long src_stride, long long dst_stride, void* stream) {
  AJB_REQUIRE(src_hd % 8 == 0 && dst_hd % 8 == 0 && src_stride % 8 == 0 && dst_stride % 8 == 0,
              "repack_heads: head sizes and row strides must be multiples of 8 elements");
  const long long total = rows * heads * (dst_hd / 8);
  if (total <= 0) return 0;
  repack_heads_kernel<<<grid_for(total, 256), 256, 0, STREAM(stream)>>>((const bf16*)src, (bf16*)dst, rows, heads, src_hd,
                                                                        dst_hd, src_stride, dst_stride);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

// out = silu(x) (dy == nullptr) or dy * silu'(x); n elements, a multiple of 8.
extern "C" int ajb_silu(const void* x, const void* dy, void* out, long long n, void* stream) {
  AJB_REQUIRE(n % 8 == 0, "silu: element count must be a multiple of 8");
  if (n <= 0) return 0;
  silu_kernel<<<grid_for(n / 8, 256), 256, 0, STREAM(stream)>>>((const bf16*)x, (const bf16*)dy, (bf16*)out, n / 8);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_ce_fwd_bwd(void* logits, const void* targets, void* loss_sum, int rows, int vocab, long long ld,
                              float grad_scale, int write_grad, void* stream) {
  if (rows <= 0) return 0;
  ce_kernel<<<rows, kCeThreads, 0, STREAM(stream)>>>((bf16*)logits, (const long long*)targets, (float*)loss_sum, rows,
                                                     vocab, ld, grad_scale, write_grad);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_embedding_fwd(const void* ids, const void* table, void* out, int tokens, int dim, int vocab,
                                 void* stream) {
  AJB_REQUIRE(dim % 8 == 0, "embedding: dim %d must be a multiple of 8", dim);
  if (tokens <= 0) return 0;
  const int grid = tokens < sm_count() * 16 ? tokens : sm_count() * 16;
  embedding_fwd_kernel<<<grid, 128, 0, STREAM(stream)>>>((const long long*)ids, (const bf16*)table, (bf16*)out, tokens,
                                                         dim, vocab);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_embedding_bwd(const void* ids, const void* grad, void* table_grad, int tokens, int dim, int vocab,
                                 void* stream) {
  AJB_REQUIRE(dim % 8 == 0, "embedding: dim %d must be a multiple of 8", dim);
  if (tokens <= 0) return 0;
  const int grid = tokens < sm_count() * 16 ? tokens : sm_count() * 16;
  embedding_bwd_kernel<<<grid, 128, 0, STREAM(stream)>>>((const long long*)ids, (const bf16*)grad, (float*)table_grad,
                                                         tokens, dim, vocab);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Two-stage deterministic reduction. `scratch` must hold ajb_sumsq_scratch_floats() floats.
extern "C" int ajb_sumsq_scratch_floats() { return kSumsqBlocks; }

extern "C" int ajb_sumsq_f32(const void* x, long long n, void* scratch, void* out, void* stream) {
  AJB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, "sumsq: input must be 16-byte aligned");
  AJB_REQUIRE(scratch != nullptr && out != nullptr, "sumsq: scratch and out are required");
  long long blocks = ((n >> 2) + kSumsqThreads - 1) / kSumsqThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > kSumsqBlocks) blocks = kSumsqBlocks;
  sumsq_partial_kernel<<<(int)blocks, kSumsqThreads, 0, STREAM(stream)>>>((const float*)x, n, (float*)scratch);
  AJB_CUDA_OK(cudaGetLastError());
  sumsq_final_kernel<<<1, kSumsqThreads, 0, STREAM(stream)>>>((const float*)scratch, (int)blocks, (float*)out);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_adamw_flat(void* master, const void* grad, void* m, void* v, void* working, long long n,
                              float step_size, float beta1, float beta2, float eps, float decay, const void* sumsq,
                              float max_norm, void* stream) {
  if (n <= 0) return 0;
  AJB_REQUIRE(((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(m) |
                reinterpret_cast<uintptr_t>(v)) & 15) == 0 && (reinterpret_cast<uintptr_t>(working) & 7) == 0,
              "adamw: buffers must be 16-byte aligned");
  adamw_flat_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, STREAM(stream)>>>(
      (float*)master, (const float*)grad, (float*)m, (float*)v, (bf16*)working, n, step_size, beta1, beta2, eps, decay,
      (const float*)sumsq, max_norm);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int ajb_add_bf16(const void* a, const void* b, void* out, long long n, void* stream) {
  AJB_REQUIRE(n % 8 == 0, "add: element count must be a multiple of 8");
  if (n <= 0) return 0;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, STREAM(stream)>>>((const bf16*)a, (const bf16*)b, (bf16*)out, n / 8);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of ajb_sumsq_f32 (declared in ajllm_b200.h; no counterpart in the reference).
//
// Who needs it: code that runs where device memory cannot be requested. Examples are an inference
// plug-in whose enqueue hook is forbidden to allocate, a host thread working inside a region in which
// the process has frozen its memory pool, or a tool that was handed a fixed memory budget up front
// and owns no allocator at all. Such callers can still pass their input and a 4-byte output, but they
// have nowhere to get the partial-sum buffer that the two-stage reduction needs between its kernels.
//
// The partial sums therefore live in a file-scope device array that is part of the loaded module:
// every GPU that loads this library holds these 4 KB until the process exits. The array is shared by
// every call. Stage one overwrites exactly the entries stage two reads, so nothing has to be cleared
// between calls, but two calls that are in flight on the GPU at the same time (different streams)
// would write the same entries and corrupt each other's result: callers must serialise them.
//
// A host function cannot use the array's name as a pointer (on the host the name is only a handle),
// so the device address is looked up with cudaGetSymbolAddress once per device, with that device
// current, on the first call made for that device. That first call should be made before any stream
// capture begins, because the lookup is not a stream operation.
constexpr long long kSumsqStaticMaxElements = 1ll << 32;   // 16 GiB of fp32 input
static __device__ __align__(256) float g_sumsq_static_partials[ajb::pw::kSumsqBlocks];
static float* g_sumsq_static_address[16] = {nullptr};

extern "C" long long ajb_sumsq_f32_static_max_elements() { return kSumsqStaticMaxElements; }

extern "C" int ajb_sumsq_f32_static(const void* x, long long n, void* out, void* stream) {
  AJB_REQUIRE(out != nullptr, "sumsq_static: the output pointer is required");
  // an empty input may come with a null pointer (an empty tensor has none): the kernels then read nothing and write 0
  AJB_REQUIRE(x != nullptr || n == 0, "sumsq_static: the input pointer is required when n > 0");
  AJB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, "sumsq_static: input must be 16-byte aligned");
  AJB_REQUIRE(n >= 0 && n <= kSumsqStaticMaxElements,
              "sumsq_static: %lld elements is outside the supported range [0, %lld]; use ajb_sumsq_f32 with a "
              "caller-provided scratch buffer for larger inputs", n, kSumsqStaticMaxElements);
  int device = -1;
  AJB_CUDA_OK(cudaGetDevice(&device));
  AJB_REQUIRE(device >= 0 && device < 16, "sumsq_static: device index %d is not supported", device);
  // The address belongs to the current device: `stream` must be a stream of that device. Two host threads making
  // the first call for one device at the same time both look the address up and store the same value.
  if (g_sumsq_static_address[device] == nullptr) {
    float* address = nullptr;
    AJB_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_sumsq_static_partials));
    AJB_REQUIRE(address != nullptr, "sumsq_static: the scratch symbol has no device address");
    g_sumsq_static_address[device] = address;
  }
  float* partials = g_sumsq_static_address[device];
  long long blocks = ((n >> 2) + kSumsqThreads - 1) / kSumsqThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > kSumsqBlocks) blocks = kSumsqBlocks;
  sumsq_partial_kernel<<<(int)blocks, kSumsqThreads, 0, STREAM(stream)>>>((const float*)x, n, partials);
  AJB_CUDA_OK(cudaGetLastError());
  sumsq_final_kernel<<<1, kSumsqThreads, 0, STREAM(stream)>>>(partials, (int)blocks, (float*)out);
  AJB_CUDA_OK(cudaGetLastError());
  return 0;
}
