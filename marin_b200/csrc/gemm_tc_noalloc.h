// mb_gemm_tc_noalloc: the tensor-core matrix product for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (Kayleexx/marin allocates its scratch with the
// cache, crates/cuda/src/kv.rs:22-24); it exists for users of this library.
//
// Who needs it.  Some programs that link these kernels cannot call cudaMalloc where the product runs:
// a serving process that handed the whole device to its own arena at start-up and treats any later
// driver allocation as a bug; a latency-critical loop in which cudaMalloc's device-wide
// synchronisation would stall every other stream; a plug-in loaded into a host whose memory budget
// is accounted by someone else.  The ordinary entry point (mb_gemm_tc) takes its split-K scratch
// (partial tiles, tile counters, error flag) from the caller, who has to allocate it.  This one
// carries the scratch inside the library instead.
//
// What it costs.  The scratch is a file-scope `static __device__` array of MB_NOALLOC_SCRATCH_BYTES
// (8 MiB + 64 KiB): every GPU on which the library is loaded holds that much until the process
// exits, used or not.
//
// Limits and rules.
//  * A call whose K slices need more than MB_NOALLOC_MAX_PARTIALS floats of partial tiles
//    (slices * T * N), or more than MB_NOALLOC_MAX_TILES tiles, is refused with
//    MB_ERR_NOALLOC_TOO_LARGE before anything is launched; mb_gemm_tc_noalloc_last_error() says
//    which limit and by how much.  (With one K slice no scratch is used and any size is accepted.)
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and the device's SM count.  Make that first call outside any stream
//    capture, and from one thread: nothing guards the per-device set-up against two first calls
//    at the same time (both would store the same values).
//  * All calls share the one array, and it keeps what the last call left.  The tile counters are
//    cleared on the call's stream before each launch.  Two calls that overlap on the GPU (different
//    streams without an ordering between them) race on the scratch and give wrong results: order them.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define MB_NOALLOC_MAX_PARTIALS (2 * 1024 * 1024)          /* floats: 8 MiB */
#define MB_NOALLOC_MAX_TILES 4096                          /* ints */
#define MB_NOALLOC_SCRATCH_BYTES (MB_NOALLOC_MAX_PARTIALS * 4 + 64 * 1024)
#define MB_ERR_NOALLOC_TOO_LARGE (-5)
#define MB_ERR_NOALLOC_SETUP (-6)

#ifdef __cplusplus
extern "C" {
#endif

// out[t, n] (+)= sum_k x[t, k] * w[n, k];  x [T, K] and w [N, K] bfloat16, K a multiple of 8, both 16-byte
// aligned; out [T, N] is bfloat16 (mode 0), float32 (mode 1) or float32 accumulated into (mode 2).
// Returns 0, a cudaError_t (> 0), or a negative MB_ERR_* code.
int mb_gemm_tc_noalloc(const void* x, const void* w, void* out, int mode, int T, int N, int K, cudaStream_t stream);

// Text for the last MB_ERR_NOALLOC_* code this thread got ("" if none).
const char* mb_gemm_tc_noalloc_last_error(void);

// Non-zero if a kernel launched through mb_gemm_tc_noalloc on the current device gave up a wait since the
// last call of this function; -1 if the device could not be asked.  It waits for ALL work on the device
// (cudaDeviceSynchronize), whatever streams the products ran on, reads the flag and clears it; do not
// call it while other threads launch products on the same device.
int mb_gemm_tc_noalloc_device_error(void);

#ifdef __cplusplus
}
#endif
