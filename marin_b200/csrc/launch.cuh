// Launching with programmatic dependent launch (PDL): a kernel may be scheduled while the kernel before it in the
// stream is still running, so that its start-up (and, for the matrix product, the first weight tiles, which no
// earlier kernel writes) overlaps the predecessor's tail.  Rules every kernel of this package follows:
//   * nothing that an earlier kernel may write is read, and no global memory is written, before pdl_wait(); pointers
//     to such data are renewed with pdl_fresh() after the wait, so that the compiler cannot move their loads up;
//   * pdl_wait() returns once every earlier kernel in the stream has finished and its writes are visible.
// Without the launch attribute both instructions do nothing.  MARIN_B200_PDL=0 in the environment turns it off;
// MARIN_B200_PDL_OFF=gemm_tc,sampling turns it off for the launches of some libraries (each source file names its
// library in MB_LIB before it includes this header): a tool for finding which kernel a race between neighbours is in.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>

#ifndef MB_LIB
#define MB_LIB ""
#endif

// -DMB_TRACE: every kernel's first block leaves a mark in a buffer the host owns (pinned memory: it outlives a fault of
// the context): buffer[0] counts the marks, mark i is at buffer[1 + i % 1023] = library id << 20 | source line of the
// kernel's entry.  A tool for finding which kernels were running when a launch failed; nothing is built with it by default.
#ifdef MB_TRACE
#ifndef MB_LIB_ID
#define MB_LIB_ID 0
#endif
__device__ int* mb_trace_buf;
extern "C" __attribute__((visibility("default"))) int mb_set_trace(int* p) { return (int)cudaMemcpyToSymbol(mb_trace_buf, &p, sizeof p); }
#define MB_TRACE_MARK()                                                                                      \
    do {                                                                                                     \
        if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && mb_trace_buf != nullptr) { \
            const int mark_at = atomicAdd_system(mb_trace_buf, 1);                                           \
            mb_trace_buf[1 + mark_at % 1023] = (MB_LIB_ID << 20) | __LINE__;                                 \
            __threadfence_system();                                                                          \
        }                                                                                                    \
    } while (0)
#else
#define MB_TRACE_MARK() do { } while (0)
#endif

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A pointer to what a kernel ahead in the stream has written goes through this after the wait, before anything is
// loaded through it.  A load through a `const __restrict__` pointer is an invariant load to the compiler, which a
// memory clobber does not hold in place: it may be moved above the wait, and was, once (decode attention read its
// queries before the kernel ahead had written them).  The empty volatile asm makes the pointer's value, and with
// it every load through it, come after the wait.
template <typename T>
__device__ __forceinline__ T* pdl_fresh(T* p) {
    asm volatile("" : "+l"(p) : : "memory");
    return p;
}

// The start of a kernel that needs nothing before its inputs.  PDL_ENTER() lets the kernels behind it be scheduled
// once its own inputs are there; PDL_ENTER_EARLY() lets them be scheduled at once, so that their CTAs sit on the
// SMs, set up and waiting, while this kernel runs.  Measured on B200: early scheduling gains 3 % on a prompt of 2,048
// tokens when the long kernels (the persistent matrix product, prefill attention) do it, and loses 5 % in decode
// steps when the short kernels do it too.  -DPDL_WAIT_FIRST or -DPDL_LAUNCH_FIRST force one order everywhere.
#define PDL_ENTER_LATE() do { MB_TRACE_MARK(); pdl_wait(); pdl_launch_dependents(); } while (0)
#define PDL_ENTER_AT_ONCE() do { MB_TRACE_MARK(); pdl_launch_dependents(); pdl_wait(); } while (0)
#if defined(PDL_WAIT_FIRST)
#define PDL_ENTER() PDL_ENTER_LATE()
#define PDL_ENTER_EARLY() PDL_ENTER_LATE()
#elif defined(PDL_LAUNCH_FIRST)
#define PDL_ENTER() PDL_ENTER_AT_ONCE()
#define PDL_ENTER_EARLY() PDL_ENTER_AT_ONCE()
#else
#define PDL_ENTER() PDL_ENTER_LATE()
#define PDL_ENTER_EARLY() PDL_ENTER_AT_ONCE()
#endif

static inline bool pdl_enabled() {
    static int state = -1;
    if (state < 0) {
        const char* v = getenv("MARIN_B200_PDL");
        state = (v != nullptr && v[0] == '0') ? 0 : 1;
        const char* off = getenv("MARIN_B200_PDL_OFF");
        if (off != nullptr && MB_LIB[0] != 0 && strstr(off, MB_LIB) != nullptr) state = 0;
    }
    return state == 1;
}

// cluster_z > 1 launches thread-block clusters of (1, 1, cluster_z); cluster_z < -1 clusters of (-cluster_z, 1, 1).
template <typename... KArgs, typename... Args>
static inline int launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_z,
                                Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1 || cluster_z < -1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_z < 0 ? (unsigned)(-cluster_z) : 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = cluster_z > 0 ? (unsigned)cluster_z : 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
