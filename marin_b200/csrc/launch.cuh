// Launching with programmatic dependent launch (PDL): a kernel may be scheduled while the kernel before it in the
// stream is still running, so that its start-up (and, for the matrix product, the first weight tiles, which no
// earlier kernel writes) overlaps the predecessor's tail.  Rules every kernel of this package follows:
//   * nothing that an earlier kernel may write is read, and no global memory is written, before pdl_wait();
//   * pdl_wait() returns once every earlier kernel in the stream has finished and its writes are visible.
// Without the launch attribute both instructions do nothing.  MARIN_B200_PDL=0 in the environment turns it off.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool pdl_enabled() {
    static int state = -1;
    if (state < 0) {
        const char* v = getenv("MARIN_B200_PDL");
        state = (v != nullptr && v[0] == '0') ? 0 : 1;
    }
    return state == 1;
}

// cluster_z > 1 launches thread-block clusters of (1, 1, cluster_z).
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
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = (unsigned)cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
