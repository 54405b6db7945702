// What the tcgen05 matrix-product kernels share besides tc_common.cuh: tile sizes, output modes, the ways a finished
// accumulator is written out, and the couplings of a product with the norms and heads around it.
#pragma once
#include "tc_common.cuh"

#define TC_BM 128          // weight rows per CTA (the MMA's M)
#define TC_BK 64           // k per pipeline stage: 64 bf16 = one 128-byte swizzle row

#define TC_OUT_BF16 0
#define TC_OUT_F32 1
#define TC_OUT_F32_ACC 2
#define TC_OUT_SWIGLU 3       // w holds gate and up rows interleaved in blocks of 16; out [T, N/2] bf16 = silu(gate) * up

template <int BN>
struct TcSmem {
    static constexpr int A_BYTES = TC_BM * TC_BK * 2;
    static constexpr int B_BYTES = BN * TC_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
};

__device__ __forceinline__ void store_out(void* out, int mode, size_t at, float v) {
    if (mode == TC_OUT_BF16) ((bf16*)out)[at] = __float2bfloat16_rn(v);
    else if (mode == TC_OUT_F32) ((float*)out)[at] = v;
    else ((float*)out)[at] += v;
}

// Sixteen consecutive tokens of one weight row: out[t_first + j, n] for j < 16, tokens below T only.  For "+=" all
// sixteen old values are asked for before any is written back, so that their latencies overlap.
__device__ __forceinline__ void store_chunk(void* out, int mode, int t_first, int n, int T, int N, const float* v) {
    if (mode == TC_OUT_F32_ACC) {
        float* o = (float*)out;
        float old[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) old[j] = (t_first + j < T) ? o[(size_t)(t_first + j) * N + n] : 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (t_first + j < T) o[(size_t)(t_first + j) * N + n] = old[j] + v[j];
    } else if (mode == TC_OUT_BF16) {
        bf16* o = (bf16*)out;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (t_first + j < T) o[(size_t)(t_first + j) * N + n] = __float2bfloat16_rn(v[j]);
    } else {
        float* o = (float*)out;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (t_first + j < T) o[(size_t)(t_first + j) * N + n] = v[j];
    }
}

// SwiGLU in the epilogue.  The weight rows of a warp's 32 accumulator lanes are 16 gate rows followed by the 16 up
// rows of the same intermediate indices, so lane l < 16 holds gate(i) and lane l + 16 holds up(i): one shuffle brings
// them together and out[t, i] = g / (1 + exp(-g)) * u is written in bf16 (crates/tensor/src/silu.rs:18; the fast
// exponential and division are accurate to a few float32 ulps, far inside the bf16 rounding of the result).  All 32
// lanes must call this; n_base is the warp's first weight row (a multiple of 32).
__device__ __forceinline__ void store_chunk_swiglu(void* out, int t_first, int n_base, int lane, int T, int N, const float* v) {
    bf16* o = (bf16*)out;
    const int half = N >> 1;
    const int i = (n_base >> 1) + (lane & 15);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float u = __shfl_down_sync(0xffffffffu, v[j], 16);
        const float g = v[j];
        if (lane < 16 && t_first + j < T && i < half)
            o[(size_t)(t_first + j) * half + i] = __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * u);
    }
}

// Two optional couplings of a product with the RMS norm next to it, so that the norm needs no kernel of its own
// (y = norm(h) W^T = rstd(h) * ((h * g) W^T): the per-token factor commutes with the product).
//   TcNormOut, on a "+=" into the residual stream h: the updated rows times the norm's weight g are also written in
//   bf16, and the sums of their squares over each group of at most 32 weight rows go to sumsq[slot][T]
//   (slot = tile * max(4, splits) + group, written without atomics: the sum over slots has a fixed order).
//   TcRowScale, on the product that consumes those rows: the accumulator of token t is multiplied by
//   1 / sqrt(sum_slots sumsq[slot][t] / dim + eps) in float32 before it is written (crates/tensor/src/norm.rs:16-22).
struct TcNormOut {
    const float* weight;      // [N]; nullptr: none of this
    bf16* scaled;             // [T, N]
    float* sumsq;             // [slots][T]
    int unit_offset;          // 1: the factor is 1 + weight
};
struct TcRowScale {
    const float* sumsq;       // [slots][T]; nullptr: no scaling
    int slots;
    int dim;
    float eps;
};

// A third coupling, for the product that makes queries, keys and values with heads of 128 = one tile of weight rows:
// instead of writing q|k|v rows, each head is finished where its sums are (per-head RMS norm with weight, half-split
// rotation by the token's position, crates/model/src/qwen3/layer.rs:59-75) and goes straight to the query buffer or
// into the paged caches.  Head h < H is a query head, the next K are key heads, the last K value heads (stored as is).
struct TcHeadsOut {
    bf16* q_out;              // [T, H * 128]; nullptr: none of this
    bf16* k_cache;            // [page][K][page_size][128]
    bf16* v_cache;
    const float* q_weight;    // [128] or nullptr: no norm
    const float* k_weight;
    const int* positions;     // [T]
    const float* inv_freq;    // [64] or nullptr: no rotation
    const int* slot_mapping;  // [T]: page * page_size + offset, negative: a padded token, nothing is stored
    float eps;
    int H, K, page_size;
};

__device__ __forceinline__ float group_sum(float v, int width) {       // over aligned groups of `width` lanes (<= 32)
    for (int o = width >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// "+=" of sixteen tokens of weight row n with the norm's side outputs; all 32 lanes call it (valid: n < N).
__device__ __forceinline__ void store_chunk_norm(void* out, int t_first, int n, bool valid, int T, int N, const float* v,
                                                 const TcNormOut& norm, float* sumsq_slot, int lane) {
    float* o = (float*)out;
    float nv[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) nv[j] = (valid && t_first + j < T) ? o[(size_t)(t_first + j) * N + n] : 0.0f;
    float g = valid ? norm.weight[n] : 0.0f;
    if (norm.unit_offset) g += 1.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        nv[j] = (valid && t_first + j < T) ? nv[j] + v[j] : 0.0f;
        if (valid && t_first + j < T) {
            o[(size_t)(t_first + j) * N + n] = nv[j];
            norm.scaled[(size_t)(t_first + j) * N + n] = __float2bfloat16_rn(nv[j] * g);
        }
        const float sq = group_sum(nv[j] * nv[j], 32);
        if (lane == 0 && t_first + j < T) sumsq_slot[t_first + j] = sq;
    }
}


// ---- host side ----
// A [rows, K] bf16 row-major matrix seen as tiles of box_rows x 64 elements with 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiled enc = encode_tiled();
    if (enc == nullptr) return MB_ERR_BAD_SIZE;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

