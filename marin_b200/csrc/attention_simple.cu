// Plain causal grouped-query attention over the paged cache: one block per (token, query head), keys
// in chunks of 128 with an online softmax in float32.  It serves prompt portions and decoded tokens
// alike, any head size, with or without a window.  It is the 32-bit path's attention and the plain twin
// of the fast kernels (the reference's generic kernel has the same shape, crates/cuda/src/attention.cu:6-96).
// Page layout: [page][kv_head][offset in page][d].
#define MB_LIB "attention_simple"
#define MB_LIB_ID 7
#include "common.cuh"
#include "launch.cuh"

#define AS_THREADS 128
#define AS_MAX_D_PER_THREAD 4

template <typename T>
__global__ void __launch_bounds__(AS_THREADS) attention_simple_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ req_index,
    const int* __restrict__ positions, int H, int K, int d, int page_size, float scale, int window) {
    PDL_ENTER();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache);
    extern __shared__ float smem[];
    float* qs = smem;                 // [d]
    float* ps = smem + d;             // [AS_THREADS]
    float* scratch = ps + AS_THREADS; // [32]
    const int t = blockIdx.x, head = blockIdx.y;
    const int kh = head / (H / K);
    const int req = req_index[t];
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)req * max_pages;
    const T* qrow = q + ((size_t)t * H + head) * d;
    for (int i = threadIdx.x; i < d; i += AS_THREADS) qs[i] = to_f32(qrow[i]);
    __syncthreads();

    float m = -INFINITY, l = 0.0f;
    float acc[AS_MAX_D_PER_THREAD];
#pragma unroll
    for (int r = 0; r < AS_MAX_D_PER_THREAD; ++r) acc[r] = 0.0f;

    for (int base = lo; base <= pos; base += AS_THREADS) {
        const int key = base + threadIdx.x;
        float s = -INFINITY;
        if (key <= pos) {
            const size_t page = (size_t)table[key / page_size];
            const T* krow = k_cache + ((page * K + kh) * page_size + (size_t)(key % page_size)) * d;
            float dot = 0.0f;
            for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(krow[i]), dot);
            s = dot * scale;
        }
        const float chunk_max = block_max(s, scratch);
        const float m_new = fmaxf(m, chunk_max);
        const float corr = expf(m - m_new);   // exp(-inf) = 0 on the first chunk
        const float p = key <= pos ? expf(s - m_new) : 0.0f;
        __syncthreads();
        ps[threadIdx.x] = p;
        const float chunk_sum = block_sum(p, scratch);  // has the barriers that publish ps
        l = l * corr + chunk_sum;
        m = m_new;
        const int count = min(AS_THREADS, pos - base + 1);
#pragma unroll
        for (int r = 0; r < AS_MAX_D_PER_THREAD; ++r) {
            const int dd = threadIdx.x + r * AS_THREADS;
            if (dd < d) {
                float a = acc[r] * corr;
                for (int j = 0; j < count; ++j) {
                    const int kj = base + j;
                    const size_t page = (size_t)table[kj / page_size];
                    const T* vrow = v_cache + ((page * K + kh) * page_size + (size_t)(kj % page_size)) * d;
                    a = fmaf(ps[j], to_f32(vrow[dd]), a);
                }
                acc[r] = a;
            }
        }
        __syncthreads();
    }
    T* orow = out + ((size_t)t * H + head) * d;
#pragma unroll
    for (int r = 0; r < AS_MAX_D_PER_THREAD; ++r) {
        const int dd = threadIdx.x + r * AS_THREADS;
        if (dd < d) orow[dd] = from_f32<T>(acc[r] / l);
    }
}

MB_API int mb_attention_simple(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype,
                               const int* block_table, int max_pages, const int* req_index, const int* positions,
                               int tokens, int H, int K, int d, int page_size, float scale, int window,
                               cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (d <= 0 || d > AS_THREADS * AS_MAX_D_PER_THREAD || K <= 0 || H % K != 0) return MB_ERR_BAD_SIZE;
    dim3 grid(tokens, H);
    const size_t smem = (size_t)(d + AS_THREADS + 32) * sizeof(float);
    if (dtype == MB_F32)
        return launch_kernel(attention_simple_kernel<float>, grid, AS_THREADS, smem, s, 0,
            (const float*)q, (const float*)k_cache, (const float*)v_cache, (float*)out, block_table, max_pages,
            req_index, positions, H, K, d, page_size, scale, window);
    else if (dtype == MB_BF16)
        return launch_kernel(attention_simple_kernel<bf16>, grid, AS_THREADS, smem, s, 0,
            (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, block_table, max_pages,
            req_index, positions, H, K, d, page_size, scale, window);
    else return MB_ERR_BAD_DTYPE;
    return mb_last_error();
}
