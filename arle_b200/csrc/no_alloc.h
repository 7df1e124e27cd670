/* arle_sample_static: next-token sampling without any device allocation.
 *
 * This entry point has no counterpart in cklxx/arle (its sampler always takes a
 * scratch buffer that the Rust side allocates, crates/cuda-kernels/csrc/misc/
 * sampling.cu:327-338).  It exists for callers of this library that are not
 * allowed to allocate device memory at the moment they need a token: code
 * running where cudaMalloc is forbidden or would deadlock (inside another
 * framework's allocator callback, under a memory-budget harness that has handed
 * out every byte, in a process whose device memory is fully reserved up front),
 * and thin C or FFI clients that have no allocator of their own and only own
 * the input and output buffers they were given.
 *
 *   int arle_sample_static(const float* logits, int ld, int rows, int vocab,
 *                          const float* temperature, const int* top_k,
 *                          const float* top_p, const float* min_p,
 *                          const float* uniform, int* out, cudaStream_t stream);
 *
 * Same arithmetic and same results as arle_sample (see sampling.cu): for every
 * row, argmax when temperature <= 0 or top_k == 1 (or when temperature is NULL:
 * all rows greedy), else softmax(logits / temperature), min_p, top_k, top_p and
 * the inverse CDF at uniform[row].  All pointers are device pointers supplied by
 * the caller; `out` gets one int per row.  Returns 0, a positive cudaError_t, or
 * a negative ARLE_E_* code; arle_no_alloc_error_string(code) gives the words.
 *
 * What replaces the caller's scratch: a float array of
 * ARLE_SAMPLE_STATIC_MAX_FLOATS elements (4 MiB) that is part of the library's
 * device image.  Every GPU that loads the library holds those 4 MiB until the
 * process exits, used or not.  A call with rows * vocab beyond that maximum is
 * refused with ARLE_E_TOO_LARGE and launches nothing (4 rows of a 262,144-entry
 * vocabulary fit, or 6 rows of Qwen3's 151,936).  The limit applies only when
 * temperatures are given: with temperature == NULL every row is an argmax, the
 * array is not used, and any number of rows is taken.
 *
 * Rules for callers:
 *  - The function calls no cudaMalloc, cudaFree or other allocating routine, and
 *    launches exactly one kernel on `stream`.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and remembers it.  Make
 *    that first call outside any stream capture.
 *  - The array is shared by all calls and keeps whatever the last call left in
 *    it.  The kernel needs none of it zeroed (it writes each probability before
 *    reading it), so nothing is cleared between calls.
 *  - Because the array is shared, two calls that can overlap on the GPU (on
 *    different streams, or from different threads on one device) race on it and
 *    give wrong tokens.  Issue calls on one stream, or order them with events.
 */
#ifndef ARLE_B200_NO_ALLOC_H
#define ARLE_B200_NO_ALLOC_H

#include <cuda_runtime.h>

#define ARLE_SAMPLE_STATIC_MAX_FLOATS (1 << 20)
#define ARLE_E_TOO_LARGE (-4)

#ifdef __cplusplus
extern "C" {
#endif

int arle_sample_static(const float* logits, int ld, int rows, int vocab, const float* temperature,
                       const int* top_k, const float* top_p, const float* min_p, const float* uniform, int* out,
                       cudaStream_t stream);
long long arle_sample_static_max_floats(void);
const char* arle_no_alloc_error_string(int code);

#ifdef __cplusplus
}
#endif
#endif
