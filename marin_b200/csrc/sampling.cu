// Sampling on the device.  arg-max: the largest logit among the first `usable`, the lowest id among
// equals (the reference's greedy rule, crates/sampler/src/lib.rs:40-48); one block per row.
#include "common.cuh"
#include "launch.cuh"

#define AM_THREADS 512

__global__ void __launch_bounds__(AM_THREADS) argmax_kernel(const float* __restrict__ logits, int vocab, int usable,
                                                            int* __restrict__ out) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float best_v[AM_THREADS / 32];
    __shared__ int best_i[AM_THREADS / 32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < usable; i += AM_THREADS) {
        const float x = row[i];
        if (x > v || (x == v && i < idx)) { v = x; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = lane < AM_THREADS / 32 ? best_v[lane] : -INFINITY;
        idx = lane < AM_THREADS / 32 ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

MB_API int mb_argmax(const float* logits, int rows, int vocab, int usable, int* out, cudaStream_t s) {
    if (rows <= 0) return 0;
    if (usable <= 0 || usable > vocab) return MB_ERR_BAD_SIZE;
    return launch_kernel(argmax_kernel, rows, AM_THREADS, 0, s, 0, logits, vocab, usable, out);
}
