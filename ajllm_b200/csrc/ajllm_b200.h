/* C interface of libajllm_b200.so (sm_100a). Every function returns 0 on success; on failure
 * ajb_last_error() describes what was wrong. Pointers are device pointers unless stated otherwise,
 * `stream` is a cudaStream_t passed as void*. */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

const char* ajb_last_error(void);
int ajb_check_status(void);

/* Sum of squares of `n` fp32 values into out[0]. `scratch` must hold ajb_sumsq_scratch_floats()
 * floats; the reduction order is fixed, so equal inputs give bit-equal results. */
int ajb_sumsq_scratch_floats(void);
int ajb_sumsq_f32(const void* x, long long n, void* scratch, void* out, void* stream);

/* Same result as ajb_sumsq_f32 for callers that cannot allocate device memory (an allocation-free
 * plug-in hook, a thread running while the process memory pool is frozen, a tool given a fixed memory
 * budget): the scratch is a 4 KB array built into the library instead of a caller buffer. This entry
 * point exists only in this library; the reference project has nothing like it.
 *   - allocates nothing, on the host or on the device;
 *   - accepts 0 <= n <= ajb_sumsq_f32_static_max_elements() and fails with a message otherwise; with n == 0 the
 *     input pointer may be null and out[0] becomes 0;
 *   - `stream` must belong to the device that is current when the call is made (the scratch address is looked
 *     up for the current device);
 *   - the first call on each device looks up the array's device address: make that call before any
 *     stream capture starts on that device; concurrent first calls from several host threads are harmless
 *     (each stores the same address);
 *   - all calls share the array: do not let two of them overlap on the GPU. */
long long ajb_sumsq_f32_static_max_elements(void);
int ajb_sumsq_f32_static(const void* x, long long n, void* out, void* stream);

int ajb_gemm_bf16(const void* a, const void* b, void* c, int m, int n, int k, long long lda, long long ldb,
                  long long ldc, int a_mn_major, int b_mn_major, int epilogue, void* stream);

#ifdef __cplusplus
}
#endif
