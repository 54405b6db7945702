// Embedding, RMSNorm, fused q/k-norm + rotation + paged cache write, SwiGLU, row gather, arg-max.
// Each kernel takes its sizes as arguments; sums, norms and angles are float32 whatever the
// activation dtype.  The formulas are the reference's (crates/cuda/src/kernels.cu:43-67,147-175,
// crates/cuda/src/kv_format.cu:48-72); the fusion and the page layout are this engine's own.
#define MB_LIB "elementwise"
#define MB_LIB_ID 1
#include "common.cuh"
#include "launch.cuh"

// ---- embedding: out[t, :] = float(table[ids[t], :]) -------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table, float* __restrict__ out, int h) {
    PDL_ENTER();
    const int t = blockIdx.x;
    const TW* row = table + (size_t)ids[t] * h;
    float* dst = out + (size_t)t * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) dst[i] = to_f32(row[i]);
}

MB_API int mb_embed(const int* ids, const void* table, int table_dtype, float* out, int tokens, int h, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (table_dtype == MB_F32) return launch_kernel(embed_kernel<float>, tokens, 256, 0, s, 0, ids, (const float*)table, out, h);
    else if (table_dtype == MB_BF16) return launch_kernel(embed_kernel<bf16>, tokens, 256, 0, s, 0, ids, (const bf16*)table, out, h);
    else return MB_ERR_BAD_DTYPE;
    return mb_last_error();
}

// ---- RMSNorm over rows of a float32 matrix ---------------------------------------------------------
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, int unit_offset,
                               TO* __restrict__ out, int n) {
    PDL_ENTER();
    x = pdl_fresh(x);
    __shared__ float scratch[32];
    const float* row = x + (size_t)blockIdx.x * n;
    TO* dst = out + (size_t)blockIdx.x * n;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { float v = row[i]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float wi = unit_offset ? 1.0f + w[i] : w[i];
        dst[i] = from_f32<TO>(row[i] * scale * wi);
    }
}

// The same with the row held in registers: 16-byte loads, one pass over memory.  n is a multiple of 4, at most
// 1024 * R (R float4 per thread).
template <typename TO, int R>
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                                                          int unit_offset, TO* __restrict__ out, int n) {
    PDL_ENTER();
    x = pdl_fresh(x);
    __shared__ float scratch[32];
    const float4* row = reinterpret_cast<const float4*>(x + (size_t)blockIdx.x * n);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const int n4 = n >> 2;
    float4 v[R];
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = threadIdx.x + r * 256;
        v[r] = i < n4 ? row[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += v[r].x * v[r].x + v[r].y * v[r].y + v[r].z * v[r].z + v[r].w * v[r].w;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    TO* dst = out + (size_t)blockIdx.x * n;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = threadIdx.x + r * 256;
        if (i < n4) {
            float4 g = w4[i];
            if (unit_offset) { g.x += 1.0f; g.y += 1.0f; g.z += 1.0f; g.w += 1.0f; }
            const float a = v[r].x * scale * g.x, b = v[r].y * scale * g.y, c = v[r].z * scale * g.z, d = v[r].w * scale * g.w;
            if (sizeof(TO) == 4) {
                reinterpret_cast<float4*>(dst)[i] = make_float4(a, b, c, d);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(dst)[i] = packed;
            }
        }
    }
}

MB_API int mb_rmsnorm(const float* x, const float* w, float eps, int unit_offset, void* out, int out_dtype,
                      int rows, int n, cudaStream_t s) {
    if (rows <= 0) return 0;
    if (out_dtype != MB_F32 && out_dtype != MB_BF16) return MB_ERR_BAD_DTYPE;
    const bool vec = n % 4 == 0 && n <= 8192 && n >= 512 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0;
    if (vec && n <= 4096) {
        if (out_dtype == MB_F32) return launch_kernel(rmsnorm_vec_kernel<float, 4>, rows, 256, 0, s, 0, x, w, eps, unit_offset, (float*)out, n);
        return launch_kernel(rmsnorm_vec_kernel<bf16, 4>, rows, 256, 0, s, 0, x, w, eps, unit_offset, (bf16*)out, n);
    }
    if (vec) {
        if (out_dtype == MB_F32) return launch_kernel(rmsnorm_vec_kernel<float, 8>, rows, 256, 0, s, 0, x, w, eps, unit_offset, (float*)out, n);
        return launch_kernel(rmsnorm_vec_kernel<bf16, 8>, rows, 256, 0, s, 0, x, w, eps, unit_offset, (bf16*)out, n);
    }
    const int threads = n >= 1024 ? 256 : 128;
    if (out_dtype == MB_F32) return launch_kernel(rmsnorm_kernel<float>, rows, threads, 0, s, 0, x, w, eps, unit_offset, (float*)out, n);
    return launch_kernel(rmsnorm_kernel<bf16>, rows, threads, 0, s, 0, x, w, eps, unit_offset, (bf16*)out, n);
}

// ---- per-head RMSNorm of q and k, rotation of q and k, k and v into their pages ---------------------
// One warp per (token, head).  Heads 0..H-1 are queries, H..H+K-1 keys, H+K..H+2K-1 values, as they
// lie in a row of the fused projection.  Page layout: [page][kv_head][offset in page][d].
template <typename T>
__global__ void qk_norm_rope_write_kernel(const T* __restrict__ qkv, int row_stride, T* __restrict__ q_out,
                                          const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                          const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                          int rotary_dim, int interleaved, const int* __restrict__ slot_mapping,
                                          T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int K, int d,
                                          int page_size, int heads_total, int heads_per_warp) {
    PDL_ENTER();
    qkv = pdl_fresh(qkv);
    extern __shared__ float smem[];
    const int warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int half = rotary_dim >> 1;
    float* cs_tab = smem;                                  // [half] cosines then [half] sines of this token's angles
    float* buf = smem + 2 * half + (size_t)warp * d;
    if (inv_freq != nullptr) {
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            cs_tab[i] = cs;
            cs_tab[half + i] = sn;
        }
    }
    __syncthreads();
    const int first = (blockIdx.y * warps + warp) * heads_per_warp;
    for (int head = first; head < min(heads_total, first + heads_per_warp); ++head) {
        const T* src = qkv + (size_t)t * row_stride + (size_t)head * d;
        const bool is_q = head < H, is_k = !is_q && head < H + K;
        float ss = 0.0f;
        for (int i = lane; i < d; i += 32) { float v = to_f32(src[i]); buf[i] = v; ss += v * v; }
        const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
        if (w != nullptr) {
            ss = warp_sum(ss);
            const float scale = 1.0f / sqrtf(ss / (float)d + eps);
            __syncwarp();
            for (int i = lane; i < d; i += 32) buf[i] = buf[i] * scale * w[i];
        }
        __syncwarp();
        if ((is_q || is_k) && inv_freq != nullptr) {
            for (int i = lane; i < half; i += 32) {
                const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
                const float cs = cs_tab[i], sn = cs_tab[half + i];
                const float a = buf[ia], b = buf[ib];
                buf[ia] = a * cs - b * sn;
                buf[ib] = b * cs + a * sn;
            }
            __syncwarp();
        }
        T* dst = nullptr;
        if (is_q) {
            dst = q_out + ((size_t)t * H + head) * d;
        } else {
            const int slot = slot_mapping[t];
            if (slot >= 0) {
                const int kh = is_k ? head - H : head - H - K;
                const size_t page = (size_t)(slot / page_size), off = (size_t)(slot % page_size);
                dst = (is_k ? k_cache : v_cache) + ((page * K + kh) * page_size + off) * d;
            }
        }
        if (dst != nullptr)
            for (int i = lane; i < d; i += 32) dst[i] = from_f32<T>(buf[i]);
        __syncwarp();
    }
}

// The same for bf16 heads of 64, 128 or 256 elements with the rotation over the whole head (half-split pairs): a
// head is LPH = d/8 consecutive lanes holding 8 elements each in registers (one 16-byte load, one 16-byte store);
// the sum of squares and the rotation partner (element i +- d/2 lies LPH/2 lanes away) travel by shuffle; all heads
// of a token are in flight at once.
template <int LPH>
__global__ void __launch_bounds__(256) qk_norm_rope_write_fast_kernel(
    const bf16* __restrict__ qkv, int row_stride, bf16* __restrict__ q_out, const float* __restrict__ q_w,
    const float* __restrict__ k_w, float eps, const int* __restrict__ positions, const float* __restrict__ inv_freq,
    const int* __restrict__ slot_mapping, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int H, int K, int page_size,
    int heads_total) {
    PDL_ENTER();
    qkv = pdl_fresh(qkv);
    constexpr int d = LPH * 8, half = d / 2;
    __shared__ float cs_tab[half], sn_tab[half];
    const int t = blockIdx.x;
    if (inv_freq != nullptr) {
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += 256) sincosf(pos * inv_freq[i], &sn_tab[i], &cs_tab[i]);
    }
    __syncthreads();
    const int sub = threadIdx.x % LPH;
    const int slot = slot_mapping[t];
    for (int base = 0; base < heads_total; base += 256 / LPH) {
        const int head = base + threadIdx.x / LPH;
        const bool valid = head < heads_total;
        const int hh = valid ? head : heads_total - 1;
        const bool is_q = hh < H, is_k = !is_q && hh < H + K;
        const uint4 raw = *reinterpret_cast<const uint4*>(qkv + (size_t)t * row_stride + (size_t)hh * d + sub * 8);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h2[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
        const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (w != nullptr) {
            const float scale = 1.0f / sqrtf(ss / (float)d + eps);
            const float4 w0 = *reinterpret_cast<const float4*>(w + sub * 8), w1 = *reinterpret_cast<const float4*>(w + sub * 8 + 4);
            v[0] = v[0] * scale * w0.x; v[1] = v[1] * scale * w0.y; v[2] = v[2] * scale * w0.z; v[3] = v[3] * scale * w0.w;
            v[4] = v[4] * scale * w1.x; v[5] = v[5] * scale * w1.y; v[6] = v[6] * scale * w1.z; v[7] = v[7] * scale * w1.w;
        }
        const bool rotate = (is_q || is_k) && inv_freq != nullptr;
        const bool first_half = sub < LPH / 2;
        const int idx0 = (first_half ? sub : sub - LPH / 2) * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, v[e], LPH / 2);
            if (rotate) {
                const float cs = cs_tab[idx0 + e], sn = sn_tab[idx0 + e];
                v[e] = first_half ? v[e] * cs - other * sn : v[e] * cs + other * sn;
            }
        }
        bf16* dst = nullptr;
        if (valid) {
            if (is_q) dst = q_out + ((size_t)t * H + hh) * d;
            else if (slot >= 0) {
                const int kh = is_k ? hh - H : hh - H - K;
                dst = (is_k ? k_cache : v_cache) + (((size_t)(slot / page_size) * K + kh) * page_size + (size_t)(slot % page_size)) * d;
            }
        }
        if (dst != nullptr) {
            uint4 packed;
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
            for (int i = 0; i < 4; ++i) p2[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            *reinterpret_cast<uint4*>(dst + sub * 8) = packed;
        }
    }
}

MB_API int mb_qk_norm_rope_write(const void* qkv, int dtype, void* q_out, const float* q_w, const float* k_w, float eps,
                                 const int* positions, const float* inv_freq, int rotary_dim, int interleaved,
                                 const int* slot_mapping, void* k_cache, void* v_cache, int tokens, int H, int K, int d,
                                 int page_size, int write_kv, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (d <= 0 || rotary_dim > d || (rotary_dim & 1)) return MB_ERR_BAD_SIZE;
    const int heads_total = write_kv ? H + 2 * K : H;
    const int row_stride = heads_total * d;
    if (dtype == MB_BF16 && (d == 64 || d == 128 || d == 256) && !interleaved && (inv_freq == nullptr || rotary_dim == d) &&
        ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 &&
        ((uintptr_t)q_w & 15) == 0 && ((uintptr_t)k_w & 15) == 0) {
        if (d == 64)
            return launch_kernel(qk_norm_rope_write_fast_kernel<8>, tokens, 256, 0, s, 0, (const bf16*)qkv, row_stride, (bf16*)q_out, q_w, k_w,
                                 eps, positions, inv_freq, slot_mapping, (bf16*)k_cache, (bf16*)v_cache, H, K, page_size, heads_total);
        if (d == 128)
            return launch_kernel(qk_norm_rope_write_fast_kernel<16>, tokens, 256, 0, s, 0, (const bf16*)qkv, row_stride, (bf16*)q_out, q_w, k_w,
                                 eps, positions, inv_freq, slot_mapping, (bf16*)k_cache, (bf16*)v_cache, H, K, page_size, heads_total);
        return launch_kernel(qk_norm_rope_write_fast_kernel<32>, tokens, 256, 0, s, 0, (const bf16*)qkv, row_stride, (bf16*)q_out, q_w, k_w,
                             eps, positions, inv_freq, slot_mapping, (bf16*)k_cache, (bf16*)v_cache, H, K, page_size, heads_total);
    }
    const int warps = 4;
    // few tokens: a warp per head, the heads spread over CTAs; many tokens: one CTA per token walks all heads and
    // the token's sines and cosines are computed once
    const int heads_per_warp = tokens >= 256 ? (heads_total + warps - 1) / warps : 1;
    dim3 grid(tokens, (heads_total + warps * heads_per_warp - 1) / (warps * heads_per_warp));
    const size_t smem = (size_t)(warps * d + rotary_dim) * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32)
        return launch_kernel(qk_norm_rope_write_kernel<float>, grid, warps * 32, smem, s, 0,
            (const float*)qkv, row_stride, (float*)q_out, q_w, k_w, eps, positions, inv_freq, rotary_dim, interleaved,
            slot_mapping, (float*)k_cache, (float*)v_cache, H, K, d, page_size, heads_total, heads_per_warp);
    else if (dtype == MB_BF16)
        return launch_kernel(qk_norm_rope_write_kernel<bf16>, grid, warps * 32, smem, s, 0,
            (const bf16*)qkv, row_stride, (bf16*)q_out, q_w, k_w, eps, positions, inv_freq, rotary_dim, interleaved,
            slot_mapping, (bf16*)k_cache, (bf16*)v_cache, H, K, d, page_size, heads_total, heads_per_warp);
    return MB_ERR_BAD_DTYPE;
}

// ---- SwiGLU: out[t, i] = g / (1 + exp(-g)) * u with g = gu[t, i], u = gu[t, I + i]; or, interleaved, with gate and
// up in alternating blocks of 16 columns: g = gu[t, 32 (i / 16) + i % 16], u = 16 columns further -----------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total, int interleaved) {
    PDL_ENTER();
    gu = pdl_fresh(gu);
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const size_t t = idx / I, i = idx % I;
        const size_t gi = interleaved ? (i >> 4) * 32 + (i & 15) : i;
        const size_t ui = interleaved ? gi + 16 : I + i;
        const float g = to_f32(gu[t * 2 * I + gi]), u = to_f32(gu[t * 2 * I + ui]);
        out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

// cos and sin of position * inv_freq for every token of a step, made once per step for the kernels that rotate heads
// inside a matrix product's epilogue: out[t][0 .. half) = cos, out[t][half .. 2 half) = sin (float32 angles, sincosf).
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int half, float* __restrict__ out, int T) {
    PDL_ENTER();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx - t * half;
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
    out[(size_t)t * 2 * half + i] = cs;
    out[(size_t)t * 2 * half + half + i] = sn;
}

MB_API int mb_rope_table(const int* positions, const float* inv_freq, int half, float* out, int T, cudaStream_t s) {
    if (T <= 0 || half <= 0) return 0;
    const int total = T * half;
    return launch_kernel(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, s, 0, positions, inv_freq, half, out, T);
}

MB_API int mb_swiglu(const void* gate_up, void* out, int dtype, int tokens, int I, int interleaved, cudaStream_t s) {
    const size_t total = (size_t)tokens * I;
    if (total == 0) return 0;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == MB_F32) return launch_kernel(swiglu_kernel<float>, blocks, threads, 0, s, 0, (const float*)gate_up, (float*)out, I, total, interleaved);
    else if (dtype == MB_BF16) return launch_kernel(swiglu_kernel<bf16>, blocks, threads, 0, s, 0, (const bf16*)gate_up, (bf16*)out, I, total, interleaved);
    else return MB_ERR_BAD_DTYPE;
    return mb_last_error();
}

// ---- rows of the residual stream whose logits are wanted ----------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ src, const int* __restrict__ rows, float* __restrict__ out, int h) {
    PDL_ENTER();
    src = pdl_fresh(src);
    const float* row = src + (size_t)rows[blockIdx.x] * h;
    float* dst = out + (size_t)blockIdx.x * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) dst[i] = row[i];
}

MB_API int mb_gather_rows(const float* src, const int* rows, float* out, int count, int h, cudaStream_t s) {
    if (count <= 0) return 0;
    return launch_kernel(gather_rows_kernel, count, 256, 0, s, 0, src, rows, out, h);
}

// ---- y += x (float32 residual, x in the activation dtype) ---------------------------------------------
template <typename T>
__global__ void add_into_kernel(float* __restrict__ y, const T* __restrict__ x, size_t total) {
    PDL_ENTER();
    x = pdl_fresh(x);
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) y[idx] += to_f32(x[idx]);
}

MB_API int mb_add_into(float* y, const void* x, int dtype, size_t total, cudaStream_t s) {
    if (total == 0) return 0;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == MB_F32) return launch_kernel(add_into_kernel<float>, blocks, threads, 0, s, 0, y, (const float*)x, total);
    else if (dtype == MB_BF16) return launch_kernel(add_into_kernel<bf16>, blocks, threads, 0, s, 0, y, (const bf16*)x, total);
    else return MB_ERR_BAD_DTYPE;
    return mb_last_error();
}
