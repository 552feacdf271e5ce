// Entry points of the CTA-pair GEMM (gemm_bf16_pair.cu) for the dispatcher in gemm_bf16.cu.
#pragma once
#include <cuda_runtime.h>

namespace ajb {
namespace gemm_pair {

// Pairs of CTAs that can be resident at once on this device (at most half the SM count).
int capacity();

// C (+)= op(A) op(B) on 256 x 256 pair tiles; same operand conventions as ajb_gemm_bf16. `split_k` > 1 needs the
// fp32 add epilogue (3) and at least that many 64-wide k-blocks per slice.
int run(const void* a, const void* b, void* c, int m, int n, int k, long long lda, long long ldb, long long ldc,
        int a_mn_major, int b_mn_major, int epilogue, int split_k, cudaStream_t stream);

}  // namespace gemm_pair
}  // namespace ajb
