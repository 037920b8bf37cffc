/* Column sums without any allocation: C entry point for callers that cannot allocate.
 *
 * This entry point has no counterpart in the reference; it exists for embedding this library
 * into hosts where device allocation is off limits at call time.
 *
 * Who needs it. Code that runs inside a region where `cudaMalloc` is forbidden or must not
 * happen: a plugin called from another framework's allocator-owned section, a real-time loop
 * that pre-reserved all device memory, a process whose memory pool is owned by a parent
 * runtime, or a C / ctypes caller that has no tensor library to lend it a workspace. The
 * regular `colsum` launcher asks its caller for a workspace of `colsum_parts(rows) * cols`
 * floats; such callers have nowhere to get one.
 *
 * What it does. `out[c] (+)= sum over rows of x[r, c]`, same kernels and same results as the
 * regular launcher, but the partial sums live in a fixed array inside the library
 * (`static __device__`, 4 MiB, resident on every GPU that loads the library until the process
 * exits). The caller passes only the input and the output.
 *
 * Limits and rules.
 *   - cols <= ETHB_COLSUM_NOALLOC_MAX_COLS and cols % 8 == 0; larger problems are rejected with
 *     ETHB_NOALLOC_TOO_LARGE (nothing is launched).
 *   - The first call on each device looks up the device address of the internal array (no
 *     allocation, but a runtime query): make that first call outside any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents. Nothing in it
 *     needs clearing: every partial sum that a call reads is first written by that same call.
 *     Two calls that overlap on the GPU (different streams, no ordering) race on the array;
 *     order them on one stream or with events.
 *   - No cudaMalloc / cudaFree / allocating library routine is called, on any path.
 *
 *   - `x` must start on a 16-byte boundary (the kernel uses 16-byte loads); `out` has no alignment
 *     requirement beyond its element type. A misaligned `x` is rejected with ETHB_NOALLOC_BAD_ARGUMENT.
 * dtype codes: 0 = float32, 1 = float16, 2 = bfloat16 (x uses `dtype`, out uses `out_dtype`).
 * Returns 0 on success, a negative ETHB_NOALLOC_* code for rejected arguments, or a positive
 * cudaError_t value if the runtime reported an error. `ethb_noalloc_strerror` describes any of
 * them.
 */
#ifndef ETHB_NO_ALLOC_H_
#define ETHB_NO_ALLOC_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ETHB_COLSUM_NOALLOC_MAX_COLS 16384
#define ETHB_COLSUM_NOALLOC_MAX_PARTS 64
#define ETHB_NOALLOC_BAD_ARGUMENT (-1)
#define ETHB_NOALLOC_TOO_LARGE (-2)

int ethb_colsum_noalloc(const void* x, void* out, int64_t rows, int32_t cols, int32_t dtype, int32_t out_dtype,
                        int32_t accumulate, void* cuda_stream);

const char* ethb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* ETHB_NO_ALLOC_H_ */
