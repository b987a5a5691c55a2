/* Allocation-free entry point of libtesseract_b200_cuda.so.
 *
 * This entry point has no counterpart in the reference project; it exists for callers of this library
 * that are not allowed to allocate device memory at the moment they need attention to run: code executing
 * inside a region where the memory pool is frozen (a serving loop that pre-sized every buffer at start-up
 * and treats a late cudaMalloc as a bug), plugins loaded into a host application that owns the allocator,
 * and real-time paths where the implicit device synchronisation of cudaMalloc / cudaFree is not acceptable.
 *
 * tsb_paged_decode_static() computes exactly what tsb_paged_decode() computes (split-K attention of one new
 * query token per request over a paged KV pool, bf16 / fp16, optional INT8 KV) but takes no scratch pointer:
 * the split partials go to a fixed array that is part of the library image
 * (TSB_STATIC_DECODE_SCRATCH_FLOATS fp32 elements = 8 MiB). Every GPU whose context loads the library holds
 * its own copy of that array until the process exits.
 *
 * Rules for callers
 *   - The caller still passes every input and the output buffer; nothing is allocated or freed by the call,
 *     by the CUDA runtime on its behalf, or by any library it calls.
 *   - The first call on each device resolves the device address of the array (cudaGetSymbolAddress with that
 *     device current) and caches it. Make that first call during start-up, outside any stream capture.
 *   - A problem whose partials do not fit (requests x query heads x key splits x (head_dim + 2) floats larger
 *     than the array) is refused with TSB_ERR_STATIC_SCRATCH_TOO_SMALL and nothing is launched; use
 *     tsb_paged_decode() with caller-owned scratch for such sizes. A problem that needs a single key split
 *     uses no scratch at all and always fits.
 *   - All calls on one device share the one array and it keeps whatever the previous call left there. The
 *     kernels overwrite every element they later read, so nothing needs clearing between calls, but two calls
 *     whose kernels can overlap on the GPU (different streams without an ordering between them) race on it.
 *     Serialise them on one stream or order them with events.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define TSB_STATIC_DECODE_SCRATCH_FLOATS (2 * 1024 * 1024)
#define TSB_ERR_STATIC_SCRATCH_TOO_SMALL (-4)

/* Arguments as tsb_paged_decode() minus `scratch`. Returns 0, a cudaError_t, -2 (bad argument) or
 * TSB_ERR_STATIC_SCRATCH_TOO_SMALL. */
int tsb_paged_decode_static(const void* q, const void* k_pool, const void* v_pool, const float* k_scale,
                            const float* v_scale, const int* tables, const int* lens, void* out, int A, int H,
                            int Hkv, int D, int bs, int nb, int max_logical, float scale, int max_len, int dtype,
                            void* stream);

/* Capacity of the built-in array in fp32 elements. */
long long tsb_paged_decode_static_capacity_floats(void);

/* Host-only helper: fp32 elements of scratch that the split plan of this problem needs on the current device
 * (0 when a single key split is used). The call above refuses exactly when this exceeds the capacity. With the
 * present split plan (at most 8 CTAs' worth of splits per SM) the need stays below the capacity on a 148-SM GPU
 * for every problem, so the refusal is a guard for other devices and future plans rather than a path callers
 * meet today. */
long long tsb_paged_decode_static_need_floats(int A, int H, int Hkv, int D, int max_len, int kv_int8);

#ifdef __cplusplus
}
#endif
