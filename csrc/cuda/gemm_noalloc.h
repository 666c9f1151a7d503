/* Allocation-free split-K GEMM entry point.
 *
 * This entry point has no counterpart in the reference project; it exists for callers of this
 * library that are not allowed to allocate device memory at the moment they need a GEMM:
 * a serving process that has already handed every free byte of HBM to weights and KV pages (a
 * cudaMalloc there either fails or forces an eviction), a latency-critical decode thread for
 * which the implicit device synchronisation of cudaMalloc/cudaFree is unacceptable, or a host
 * application that owns the allocator and forbids foreign allocations.
 *
 *   y[M, N] (bf16) = x[M, K] (bf16) * w[N, K]^T (bf16),   1 <= M <= 128, split over `splits` K ranges
 *
 * The fp32 partial sums and the per-tile arrival counters of the split-K kernel live in one
 * file-scope device array of fixed size (PLOW_NOALLOC_SCRATCH_BYTES, 8 MiB + 64 KiB) that every GPU
 * loading the library holds until the process exits.  The function calls no cudaMalloc, cudaFree
 * or any allocating library routine.
 *
 * Rules for callers:
 *   - The first call on a device resolves the array's device address (cudaGetSymbolAddress, with
 *     that device current) and sets the kernel's shared-memory attribute.  Make that first call
 *     outside any stream capture.
 *   - A problem whose partials do not fit (ceil(N/128) * splits * 128 * BN * 4 bytes, BN = 32/64/128
 *     covering M, more than 8 MiB; or more than 128 output tiles) is rejected with
 *     PLOW_NOALLOC_E_TOO_LARGE before anything is launched.
 *   - All calls on a device share the one array, and it keeps the previous call's contents; the
 *     counters are cleared on the caller's stream at the start of every call.  Two calls that
 *     overlap on the GPU (different streams, no ordering between them) race on it.
 */
#ifndef PLOW_GEMM_NOALLOC_H
#define PLOW_GEMM_NOALLOC_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define PLOW_NOALLOC_SCRATCH_BYTES ((8u << 20) + (64u << 10))
#define PLOW_NOALLOC_E_ARG (-1)         /* null pointer, M outside [1,128], misaligned operand */
#define PLOW_NOALLOC_E_TOO_LARGE (-2)   /* partials exceed the static scratch */
#define PLOW_NOALLOC_E_SYMBOL (-3)      /* cudaGetSymbolAddress failed */

/* x, w, y: device pointers (16-byte aligned, K a multiple of 8).  status: one device int32 the
 * kernel writes a non-zero code into if one of its bounded waits expires.  stream: cudaStream_t.
 * Returns 0 on a successful launch, a PLOW_NOALLOC_E_* code, or a positive launcher code. */
int plow_gemm_splitk_noalloc(const void* x, const void* w, void* y, int32_t M, int32_t N, int32_t K,
                             int32_t splits, int32_t* status, void* stream);

/* Human-readable text for the negative codes above. */
const char* plow_gemm_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif
