/* Allocation-free entry point of libb200_kernels.so.
 *
 * This entry point has no counterpart in the reference engine; it exists for callers of this
 * library that are not allowed to allocate device memory at the moment they need a GEMM: code
 * running inside a region where cudaMalloc / cudaFree are forbidden or would synchronise the
 * device (a latency-critical serving loop that must never touch the allocator, a host application
 * that hands this library a fixed memory budget up front, a plug-in loaded into a process whose
 * allocator the plug-in must not disturb). The normal entry point, b200_gemm, needs a
 * caller-provided zero-initialised scratch buffer for its split-K path; the function below uses
 * a scratch array that lives inside the library image instead.
 */
#ifndef B200_NOALLOC_H_
#define B200_NOALLOC_H_

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Largest token count (rows of x) the allocation-free GEMM accepts. */
#define B200_NOALLOC_MAX_TOKENS 128
/* Size of the library-resident scratch array. Every GPU on which the library is loaded keeps this
 * much device memory until the process exits. */
#define B200_NOALLOC_SCRATCH_BYTES (10 * 1024 * 1024)

/* out[m][n] (bf16, leading dimension ldc) = x[m][k] * w[n][k]^T (+ bias[n]) (+ residual[m][n])
 *   dtype 0: x, w are bf16.
 *   dtype 1: x, w are e4m3 bytes with fp32 scales x_scale [m][k/128] and w_scale [ceil(n/128)][k/128];
 *            k must then be a multiple of 128.
 *   dtype 2: x, w are e4m3 bytes with power-of-two (UE8M0) scales applied by the tensor core. The two
 *            scale arguments then point (through the same `const float*` parameters) at blocked
 *            scale-factor arrays of 32-bit words: [row tiles of 128][ceil(k/512)][128 words]; row r of
 *            a tile sits at word (r % 32) * 4 + r / 32, and byte (kb % 4) of the word is the biased
 *            exponent of 128-wide K block kb. Weight rows of one 128-row block share their scale, so
 *            its tile repeats one byte per K block. k must be a multiple of 16; bytes of K blocks
 *            past the end of k must hold a finite exponent (127).
 * Same arithmetic and the same kernel as b200_gemm; only the scratch memory differs.
 *
 * The caller passes inputs and outputs (device pointers, 16-byte aligned rows); nothing is
 * allocated or freed by this call, and no allocating library routine is used.
 *
 * Limits and rules:
 *   - m must be <= B200_NOALLOC_MAX_TOKENS; larger problems return B200_NOALLOC_ERR_TOO_LARGE
 *     (-8) and launch nothing. Use b200_gemm with your own scratch buffer for those.
 *   - The first call on each device resolves the device address of the scratch array (once per
 *     device, with that device current). Make that first call outside any CUDA stream capture.
 *   - All calls on a device share the one scratch array, which keeps whatever the previous call
 *     left in it. The part that has to start at zero (the tile arrival counters) is cleared on
 *     `stream` at the start of every call. Two calls that can overlap on the GPU (different
 *     streams without an ordering between them) race on the array and give wrong results:
 *     serialise them.
 *   - Fully split small GEMMs are reduced by a second kernel launched by the same call (the
 *     library default; b200_gemm_set_cluster_reduce / b200_gemm_set_external_reduce change it
 *     for every entry point of the process, this one included).
 *   - The kernel's internal waits are bounded, but this entry point takes no status word: a wait
 *     that ran out cannot be reported here. Callers that need that report use b200_gemm, which
 *     accepts a 16-byte status record.
 * Returns 0 on success, a negative code otherwise (argument / launch errors as b200_gemm). */
#define B200_NOALLOC_ERR_TOO_LARGE (-8)
#define B200_NOALLOC_ERR_SETUP (-9)
int b200_gemm_noalloc(const void* x, const void* w, void* out, int m, int n, int k, long long ldx,
                      long long ldw, long long ldc, int dtype, const float* x_scale,
                      const float* w_scale, const void* bias, const void* residual,
                      cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
