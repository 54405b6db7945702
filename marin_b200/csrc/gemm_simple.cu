// Plain tiled matrix product on the CUDA cores: out[t, n] = sum_k x[t, k] * w[n, k], float32 accumulate,
// k summed in increasing order in every thread, so a row's result does not depend on how many other
// rows the batch holds.  This is the whole 32-bit path's matrix product (no tensor cores, no reduced-
// precision mode) and the plain twin the tensor-core kernel is tested against.  The reference's
// counterpart is its warp-per-row kernel (crates/cuda/src/kernels.cu:73-116).
#define MB_LIB "gemm_simple"
#define MB_LIB_ID 6
#include "common.cuh"
#include "launch.cuh"

#define GS_TILE 64
#define GS_BK 16

template <typename TX, typename TW, typename TO, bool ACC>
__global__ void __launch_bounds__(256) gemm_simple_kernel(const TX* __restrict__ x, const TW* __restrict__ w,
                                                          TO* __restrict__ out, int T, int N, int K) {
    PDL_ENTER();
    x = pdl_fresh(x);
    __shared__ float sx[GS_BK][GS_TILE + 1];
    __shared__ float sw[GS_BK][GS_TILE + 1];
    const int t0 = blockIdx.y * GS_TILE, n0 = blockIdx.x * GS_TILE;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // tx: n direction, ty: t direction
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += GS_BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = threadIdx.x + r * 256;
            const int row = e >> 4, kk = e & 15;
            const int k = k0 + kk;
            const int t = t0 + row, n = n0 + row;
            sx[kk][row] = (t < T && k < K) ? to_f32(x[(size_t)t * K + k]) : 0.0f;
            sw[kk][row] = (n < N && k < K) ? to_f32(w[(size_t)n * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GS_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sx[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = sw[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const size_t at = (size_t)t * N + n;
            if (ACC) out[at] = from_f32<TO>(to_f32(out[at]) + acc[i][j]);
            else out[at] = from_f32<TO>(acc[i][j]);
        }
    }
}

template <typename TX, typename TW, typename TO>
static int launch(const void* x, const void* w, void* out, int T, int N, int K, int accumulate, cudaStream_t s) {
    dim3 grid((N + GS_TILE - 1) / GS_TILE, (T + GS_TILE - 1) / GS_TILE);
    if (accumulate) return launch_kernel(gemm_simple_kernel<TX, TW, TO, true>, grid, 256, 0, s, 0, (const TX*)x, (const TW*)w, (TO*)out, T, N, K);
    return launch_kernel(gemm_simple_kernel<TX, TW, TO, false>, grid, 256, 0, s, 0, (const TX*)x, (const TW*)w, (TO*)out, T, N, K);
}

// x [T, K] (x_dtype), w [N, K] (w_dtype), out [T, N] (out_dtype); accumulate: out += (float32 out only).
MB_API int mb_gemm_simple(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                          int T, int N, int K, int accumulate, cudaStream_t s) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0) return MB_ERR_BAD_SIZE;
    if (accumulate && out_dtype != MB_F32) return MB_ERR_BAD_DTYPE;
    if (x_dtype == MB_F32 && w_dtype == MB_F32 && out_dtype == MB_F32) return launch<float, float, float>(x, w, out, T, N, K, accumulate, s);
    if (x_dtype == MB_BF16 && w_dtype == MB_BF16 && out_dtype == MB_BF16) return launch<bf16, bf16, bf16>(x, w, out, T, N, K, accumulate, s);
    if (x_dtype == MB_BF16 && w_dtype == MB_BF16 && out_dtype == MB_F32) return launch<bf16, bf16, float>(x, w, out, T, N, K, accumulate, s);
    return MB_ERR_BAD_DTYPE;
}
