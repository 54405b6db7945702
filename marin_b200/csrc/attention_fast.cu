// Fast bf16 attention over the paged cache, compiled for one head size and one group size
// (-DHEAD_DIM=.. -DGROUP=..: what the model at hand needs, built at first use).
//
//  * decode: one new token per request.  A CTA takes one kv head of one request and one chunk of 128 keys
//    (fixed by absolute position, so the arithmetic does not depend on the batch or on the number of SMs);
//    all GROUP query heads that share the kv head are served from one pass over K and one over V; the
//    partial (max, sum, accumulator) of every chunk goes to scratch and the CTA that finishes last combines them.
//    The reference splits decode attention the same way but sizes chunks by SM count
//    (crates/cuda/src/attention.rs:23-30, attention.cu:224-351,481-494).
//  * prefill: a CTA takes 64 consecutive query tokens of one request and one query head, walks the keys in
//    blocks of 64 with an online softmax in float32; Q K^T and P V run on mma.sync.m16n8k16 (bf16 in,
//    float32 accumulate).  Portions of prompts at any cached length, causal inside the portion.
//    (The reference's counterpart: crates/cuda/src/attention_mma.cu:43-180, f16, whole prompts.)
//
// Page layout: [page][kv_head][offset in page][HEAD_DIM]; block_table[request][logical page] -> page.
#define MB_LIB "attention_fast"
#define MB_LIB_ID 3
#include "tc_common.cuh"
#include "launch.cuh"
#include <type_traits>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 16, at most 128>"
#endif
#ifndef GROUP
#error "compile with -DGROUP=<query heads per kv head, at most 8>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 128, "head size must be a multiple of 16 up to 128");
static_assert(GROUP >= 1 && GROUP <= 8, "1 to 8 query heads per kv head");

#define D HEAD_DIM

// 2^x for x <= 0 (softmax numerators): one MUFU instruction, a couple of ulps off, flushes denormals to zero;
// exp2f proper costs several more instructions per element and the probabilities are rounded to bf16 anyway.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
#ifndef DEC_WARPS
#define DEC_WARPS 4
#endif
#define DPL (D / 8)                   // dims per lane: 8 lanes share one key
#define VW (DPL % 8 == 0 ? 8 : (DPL % 4 == 0 ? 4 : 2))   // elements per vector load
#define NV (DPL / VW)                 // vector loads per lane and key

// Loads this lane's DPL elements of one row: vector v covers dims v * (8 * VW) + sub * VW ..
__device__ __forceinline__ void load_slice(const bf16* row, int sub, float* dst) {
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const bf16* p = row + v * (8 * VW) + sub * VW;
        if (VW == 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(p);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); dst[v * VW + 2 * i] = f.x; dst[v * VW + 2 * i + 1] = f.y; }
        } else if (VW == 4) {
            const uint2 raw = *reinterpret_cast<const uint2*>(p);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 2; ++i) { const float2 f = __bfloat1622float2(h[i]); dst[v * VW + 2 * i] = f.x; dst[v * VW + 2 * i + 1] = f.y; }
        } else {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
            dst[v * VW] = f.x; dst[v * VW + 1] = f.y;
        }
    }
}

// The dim a lane's element e stands for.
__device__ __forceinline__ int slice_dim(int sub, int e) { return (e / VW) * (8 * VW) + sub * VW + (e % VW); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// 16 bytes from global to shared memory without passing through registers.
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A float from the shared memory of CTA `rank` of this cluster, at the address `addr` has in this CTA.
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr, int rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

#define LDP (D + 8)                   // padded row of a tile in shared memory (elements): ldmatrix without bank conflicts
#ifndef DEC_STAGES
#define DEC_STAGES 3                  // per-warp ring of 16-key stages
#endif
#define DEC_STAGE_KEYS 16
#ifndef DEC_MAX_CLUSTER
#define DEC_MAX_CLUSTER 16            // most chunks of one sequence that merge as one thread-block cluster (more than 8 is
                                      // a non-portable size: the launcher asks for it and the caller falls back if refused)
#endif
#define DEC_Q_BYTES (16 * LDP * 2)
#define DEC_STAGE_BYTES (2 * DEC_STAGE_KEYS * LDP * 2)          // keys then values
#define DEC_WARP_BYTES (DEC_STAGES * DEC_STAGE_BYTES)
#define DEC_SMEM (DEC_Q_BYTES + DEC_WARPS * DEC_WARP_BYTES)
static_assert(GROUP * D * 4 <= DEC_WARP_BYTES, "a warp's accumulators are written over its stage buffers");
// With TMA a stage is dense: per 64 dims one tile of 16 rows x 128 bytes in the 128-byte swizzle (keys, then values).
#define DEC_TMA (D % 64 == 0)
#define DEC_TMA_STAGE_BYTES (2 * DEC_STAGE_KEYS * D * 2)
#define DEC_TMA_SMEM (DEC_Q_BYTES + DEC_WARPS * DEC_STAGES * DEC_TMA_STAGE_BYTES + 1024)
static_assert(!DEC_TMA || GROUP * D * 4 <= DEC_STAGES * DEC_TMA_STAGE_BYTES, "a warp's accumulators are written over its stage buffers");

// Decode.  A CTA takes `split_keys` consecutive keys (by absolute position) of one kv head of one request; each of
// its four warps takes a quarter of them and walks it in stages of 16 keys through its own ring of buffers
// (three stages in flight per warp, no block-wide barrier in the loop).  The GROUP query heads are rows
// 0..GROUP-1 of a 16-row tile (the other rows are zero); S = Q K^T and O = P V are mma.sync.m16n8k16, the
// softmax runs online in float32 in the exp2 domain.  Partial (m, l, acc) per CTA: m is in log2 units.
// TMA = true (heads of 64 or 128, pages of at least 16 positions): a stage lies inside one page and one lane
// fetches it with two or four tensor copies onto the warp's mbarrier, instead of sixteen cp.async per lane.
template <bool TMA>
__global__ void __launch_bounds__(DEC_WARPS * 32) attn_decode_split_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_lens, int K, int page_shift,
    float scale, int window, float* __restrict__ part_acc, float* __restrict__ part_ml, int max_chunks, int split_keys,
    int* __restrict__ counters, bf16* __restrict__ out, int* __restrict__ error_flag, int cluster_merge) {
    // The dependency wait comes later: sequence lengths and block tables were copied before the step began, and every
    // key and value but the newest token's was written by earlier steps, so most of the cache may be asked for while
    // the kernels ahead are still running.
    extern __shared__ __align__(16) uint8_t dec_smem_raw[];
    constexpr int STAGE_BYTES = TMA ? DEC_TMA_STAGE_BYTES : DEC_STAGE_BYTES;
    constexpr int WARP_BYTES = DEC_STAGES * STAGE_BYTES;
    uint8_t* dec_smem = TMA ? (uint8_t*)(((uintptr_t)dec_smem_raw + 1023) & ~(uintptr_t)1023) : dec_smem_raw;
    __shared__ float s_m[DEC_WARPS][8], s_l[DEC_WARPS][8];
    __shared__ int s_last;
    __shared__ uint64_t s_full[DEC_WARPS][DEC_STAGES];
    __shared__ float c_m[8], c_l[8];                   // this CTA's (max, sum) per query head, for its cluster
    const int chunk = blockIdx.x, kh = blockIdx.y, r = blockIdx.z;
    const int H = K * GROUP;
    const int len = seq_lens[r];
    const int pos = len - 1;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int c_begin = chunk * split_keys, c_end = min(len, c_begin + split_keys);
    const bool has_work = c_begin < len && c_end > lo;
    if (!has_work && !cluster_merge) { PDL_ENTER(); return; }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = block_table + (size_t)r * max_pages;
    uint8_t* ring = dec_smem + (size_t)warp * WARP_BYTES;
    bf16* sQ = reinterpret_cast<bf16*>(dec_smem + (size_t)DEC_WARPS * WARP_BYTES);
    float* c_acc = reinterpret_cast<float*>(sQ);       // [GROUP][D] for the cluster, once the query tile is in registers
    static_assert(GROUP * D * 4 <= DEC_Q_BYTES, "the CTA's partial result is written over the query tile");
    if (has_work) {
    const int kpw = split_keys / DEC_WARPS;
    const int w_begin = c_begin + warp * kpw, w_stop = min(len, w_begin + kpw);
    const int first = max(w_begin, (lo / DEC_STAGE_KEYS) * DEC_STAGE_KEYS);
    const int n_it = w_stop > first ? (w_stop - first + DEC_STAGE_KEYS - 1) / DEC_STAGE_KEYS : 0;
    constexpr int PIECES = D / 8;
    if (TMA) {
        if (lane == 0) {
            for (int st = 0; st < DEC_STAGES; ++st) mbar_init(&s_full[warp][st], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
    }

    // stage i: keys first + 16 i .. + 16, K rows then V rows; rows outside [lo, len) are zero
    const int page_mask = (1 << page_shift) - 1;
    const size_t head_rows = (size_t)kh << page_shift;             // rows before this kv head inside a page
    const size_t page_rows = (size_t)K << page_shift;              // rows of a whole page
    // Where this lane's pieces of a stage lie: piece p of row r (rows 0..15 keys, 16..31 values) for idx = lane + 32 j.
    auto issue = [&](int i) {
        if (TMA) {
            // the whole stage lies in one page (pages hold at least 16 positions); rows outside [lo, len) come along
            // and are masked (keys) or cleared (values) when the stage is used
            if (i < n_it && lane == 0) {
                uint8_t* dst = ring + (size_t)(i % DEC_STAGES) * STAGE_BYTES;
                uint64_t* bar = &s_full[warp][i % DEC_STAGES];
                const int key_base = first + i * DEC_STAGE_KEYS;
                const int row0 = (int)(((size_t)table[key_base >> page_shift] * K + kh) << page_shift) + (key_base & page_mask);
                mbar_expect_tx(bar, STAGE_BYTES);
#pragma unroll
                for (int hf = 0; hf < D / 64; ++hf) {
                    tma_load_2d(dst + hf * 2048, &map_k, hf * 64, row0, bar);
                    tma_load_2d(dst + STAGE_BYTES / 2 + hf * 2048, &map_v, hf * 64, row0, bar);
                }
            }
            return;
        }
        if (i < n_it) {
            bf16* dst = reinterpret_cast<bf16*>(ring + (size_t)(i % DEC_STAGES) * DEC_STAGE_BYTES);
            const int key_base = first + i * DEC_STAGE_KEYS;
            if (page_shift >= 4 && key_base >= lo && key_base + DEC_STAGE_KEYS <= len) {
                // the whole stage is valid and lies in one page: one block-table lookup, then constant strides
                const size_t row0 = (size_t)table[key_base >> page_shift] * page_rows + head_rows + (size_t)(key_base & page_mask);
                const bf16* ksrc = k_cache + row0 * D;
                const bf16* vsrc = v_cache + row0 * D;
#pragma unroll
                for (int idx = lane; idx < DEC_STAGE_KEYS * PIECES; idx += 32) {
                    const int row = idx / PIECES, piece = idx % PIECES;
                    cp_async16(dst + row * LDP + piece * 8, ksrc + row * D + piece * 8);
                    cp_async16(dst + (DEC_STAGE_KEYS + row) * LDP + piece * 8, vsrc + row * D + piece * 8);
                }
            } else {
#pragma unroll
                for (int idx = lane; idx < 2 * DEC_STAGE_KEYS * PIECES; idx += 32) {
                    const int row = idx / PIECES, piece = idx % PIECES;           // rows 0..15 keys, 16..31 values
                    const int key = key_base + (row & (DEC_STAGE_KEYS - 1));
                    bf16* d = dst + row * LDP + piece * 8;
                    if (key < len && key >= lo) {
                        const bf16* cache = row < DEC_STAGE_KEYS ? k_cache : v_cache;
                        const size_t at = (size_t)table[key >> page_shift] * page_rows + head_rows + (size_t)(key & page_mask);
                        cp_async16(d, cache + at * D + piece * 8);
                    } else {
                        *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
                    }
                }
            }
        }
        cp_async_commit();
    };
    // only the stage that holds the newest position (written by the kernel just ahead) has to wait for that kernel
    bool waited = false;
#pragma unroll
    for (int i = 0; i < DEC_STAGES; ++i) {
        const int key_base = first + i * DEC_STAGE_KEYS;
        if (!waited && i < n_it && key_base + DEC_STAGE_KEYS > pos) { PDL_ENTER(); waited = true; }
        issue(i);
    }
    if (!waited) PDL_ENTER();

    // The query tile, GROUP heads in rows 0..GROUP-1 of 16 (the rest zero), straight into the MMA's A fragments: lane l
    // holds row l / 4, columns 2 (l % 4) + {0, 1} and + 8 of every 16-column step; rows 8..15 (a1, a3) are zero since at
    // most 8 heads share a kv head.  Every warp loads its own copy: no shared memory, no block-wide barrier.
    uint32_t qa[D / 16][4];
    {
        const int qrow = lane >> 2;
        // (the queries were written by the kernel just ahead: see pdl_fresh)
        const bf16* qsrc = pdl_fresh(q) + ((size_t)r * H + kh * GROUP + (qrow < GROUP ? qrow : 0)) * D + 2 * (lane & 3);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            qa[kk][0] = qrow < GROUP ? *reinterpret_cast<const uint32_t*>(qsrc + kk * 16) : 0u;
            qa[kk][2] = qrow < GROUP ? *reinterpret_cast<const uint32_t*>(qsrc + kk * 16 + 8) : 0u;
            qa[kk][1] = 0u;
            qa[kk][3] = 0u;
        }
    }

    const float sl2 = scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.0f;              // of this thread's row (= query head lane / 4)
    float o[D / 8][4];                                 // [2] and [3] are rows 8..15 of the tile: they stay zero
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }

    // where this lane's ldmatrix rows lie in a swizzled tile: 16-byte chunk c of row r is at r * 128 + ((c ^ (r & 7)) << 4)
    uint32_t offk[4], offv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        offk[j] = (uint32_t)(((((lane >> 3) & 1) + 2 * j) ^ (lane & 7)) << 4);
        offv[j] = (uint32_t)((((lane >> 4) + 2 * j) ^ (lane & 7)) << 4);
    }
    for (int it = 0; it < n_it; ++it) {
        const int key_base = first + it * DEC_STAGE_KEYS;
        const uint8_t* stage = ring + (size_t)(it % DEC_STAGES) * STAGE_BYTES;
        if (TMA) {
            const bool arrived = mbar_wait(&s_full[warp][it % DEC_STAGES], (uint32_t)(it / DEC_STAGES) & 1u);
            if (!__all_sync(0xffffffffu, arrived)) {
                if (lane == 0) atomicExch(error_flag, 31);
                break;
            }
            if (key_base < lo || key_base + DEC_STAGE_KEYS > len) {
                // values of positions outside [lo, len) may be anything (0 * NaN is NaN): clear their rows
                for (int idx = lane; idx < DEC_STAGE_KEYS * PIECES; idx += 32) {
                    const int row = idx / PIECES, c = idx % PIECES;
                    const int key = key_base + row;
                    if (!(key < len && key >= lo))
                        *reinterpret_cast<uint4*>(const_cast<uint8_t*>(stage) + STAGE_BYTES / 2 + (c >> 3) * 2048 + row * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
            }
        } else {
            cp_async_wait<DEC_STAGES - 1>();
            __syncwarp();
        }
        const bf16* sK = reinterpret_cast<const bf16*>(stage);
        const bf16* sV = sK + DEC_STAGE_KEYS * LDP;
        float sc[2][4];
        sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.0f;
        const uint32_t k_addr = TMA ? smem_u32(stage) + (uint32_t)(((lane & 7) + (lane >> 4) * 8) * 128)
                                    : (uint32_t)__cvta_generic_to_shared(sK + ((lane & 7) + (lane >> 4) * 8) * LDP + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(TMA ? k_addr + (uint32_t)((kk >> 2) * 2048) + offk[kk & 3] : k_addr + kk * 32, b0, b1, b2, b3);
            mma_bf16_16816(sc[0], qa[kk], b0, b1);
            mma_bf16_16816(sc[1], qa[kk], b2, b3);
        }
        if (key_base < lo || key_base + DEC_STAGE_KEYS > len) {            // only the ends of the range need masking
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int key = key_base + 2 * (lane & 3) + j * 8;
                if (!(key < len && key >= lo)) sc[j][0] = -INFINITY;
                if (!(key + 1 < len && key + 1 >= lo)) sc[j][1] = -INFINITY;
            }
        }
        float mx = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx * sl2);                        // log2 units; the scale is positive
        const float base = m_new == -INFINITY ? 0.0f : m_new;
        const float corr = fast_exp2(m_run - base);
        m_run = m_new;
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            sc[j][0] = fast_exp2(fmaf(sc[j][0], sl2, -base));
            sc[j][1] = fast_exp2(fmaf(sc[j][1], sl2, -base));
            sum += sc[j][0] + sc[j][1];
        }
        l_run = l_run * corr + sum;
        uint32_t pa[4];
        pa[0] = pack_bf16(sc[0][0], sc[0][1]);
        pa[1] = 0u;
        pa[2] = pack_bf16(sc[1][0], sc[1][1]);
        pa[3] = 0u;
        const uint32_t v_addr = TMA ? smem_u32(stage) + (uint32_t)(STAGE_BYTES / 2 + ((lane & 7) + ((lane >> 3) & 1) * 8) * 128)
                                    : (uint32_t)__cvta_generic_to_shared(sV + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDP + (lane >> 4) * 8);
#pragma unroll
        for (int dt = 0; dt < D / 8; dt += 2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(TMA ? v_addr + (uint32_t)((dt >> 3) * 2048) + offv[(dt >> 1) & 3] : v_addr + dt * 16, b0, b1, b2, b3);
            o[dt][0] *= corr; o[dt][1] *= corr; o[dt + 1][0] *= corr; o[dt + 1][1] *= corr;
            mma_bf16_16816(o[dt], pa, b0, b1);
            mma_bf16_16816(o[dt + 1], pa, b2, b3);
        }
        __syncwarp();                                   // the stage is free: refill it
        issue(it + DEC_STAGES);
    }
    if (!TMA) cp_async_wait<0>();
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

    // each warp leaves (m, l, acc) of its keys in shared memory (over its ring), then the CTA adds the warps
    float* s_acc = reinterpret_cast<float*>(ring);
    __syncwarp();
    const int g_row = lane >> 2;
    if (g_row < GROUP) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            s_acc[g_row * D + i * 8 + 2 * (lane & 3)] = o[i][0];
            s_acc[g_row * D + i * 8 + 2 * (lane & 3) + 1] = o[i][1];
        }
        if ((lane & 3) == 0) { s_m[warp][g_row] = m_run; s_l[warp][g_row] = l_run; }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < GROUP * D; idx += DEC_WARPS * 32) {
        const int g = idx / D, dd = idx % D;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, s_m[w][g]);
        float a = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = s_m[w][g] == -INFINITY ? 0.0f : exp2f(s_m[w][g] - mm);
            const float* wacc = reinterpret_cast<const float*>(dec_smem + (size_t)w * WARP_BYTES);
            a = fmaf(wacc[g * D + dd], f, a);
            ll = fmaf(s_l[w][g], f, ll);
        }
        if (cluster_merge) {
            c_acc[idx] = a;
            if (dd == 0) { c_m[g] = mm; c_l[g] = ll; }
        } else {
            const size_t at = ((size_t)r * H + kh * GROUP + g) * max_chunks + chunk;
            part_acc[at * D + dd] = a;
            if (dd == 0) { part_ml[at * 2] = mm; part_ml[at * 2 + 1] = ll; }
        }
    }
    } else {
        PDL_ENTER();                                   // it still writes its share of the outputs below
        if (threadIdx.x < 8) {
            c_m[threadIdx.x] = -INFINITY;              // a chunk outside the sequence (or the window) adds nothing
            c_l[threadIdx.x] = 0.0f;
        }
    }
    if (cluster_merge) {
        // The chunks of this (request, kv head) are the CTAs of one cluster: after a cluster barrier every CTA combines
        // its share of the outputs from all partial results, read through distributed shared memory, chunks in
        // increasing order: out = sum_c acc_c 2^(m_c - M) / sum_c l_c 2^(m_c - M).
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        const int ranks = gridDim.x;
        const int per = (GROUP * D + ranks - 1) / ranks;
        const int i_end = min(GROUP * D, (chunk + 1) * per);
        const uint32_t a_acc = smem_u32(c_acc), a_m = smem_u32(c_m), a_l = smem_u32(c_l);
        // the chunks' weights 2^(m_c - M) and the inverse of the total sum, once per head (ranks <= MC), then every
        // output is one weighted sum over the chunks
        __shared__ float wgt[8 * DEC_MAX_CLUSTER], inv_total[8];     // [head][chunk], [head]
        // (written for 8 and for 16 chunks: the loops are unrolled, and the common small clusters do not pay for the wide ones)
        auto merge = [&](auto width) {
            constexpr int MC = decltype(width)::value;
            if (threadIdx.x < GROUP) {
                const int g = threadIdx.x;
                float mc[MC], mm = -INFINITY;
#pragma unroll
                for (int c = 0; c < MC; ++c) { mc[c] = c < ranks ? ld_cluster_f32(a_m + g * 4, c) : -INFINITY; mm = fmaxf(mm, mc[c]); }
                float ll = 0.0f;
#pragma unroll
                for (int c = 0; c < MC; ++c) {
                    const float f = mc[c] == -INFINITY ? 0.0f : exp2f(mc[c] - mm);
                    wgt[g * MC + c] = f;
                    if (c < ranks && f != 0.0f) ll = fmaf(ld_cluster_f32(a_l + g * 4, c), f, ll);
                }
                inv_total[g] = 1.0f / ll;
            }
            __syncthreads();
            for (int idx = chunk * per + threadIdx.x; idx < i_end; idx += DEC_WARPS * 32) {
                const int g = idx / D;
                float part[MC];
#pragma unroll
                for (int c = 0; c < MC; ++c) part[c] = (c < ranks && wgt[g * MC + c] != 0.0f) ? ld_cluster_f32(a_acc + idx * 4, c) : 0.0f;
                float a = 0.0f;
#pragma unroll
                for (int c = 0; c < MC; ++c) a = fmaf(part[c], wgt[g * MC + c], a);
                out[((size_t)r * H + kh * GROUP) * D + idx] = __float2bfloat16_rn(a * inv_total[g]);
            }
        };
        if (DEC_MAX_CLUSTER <= 8 || ranks <= 8) merge(std::integral_constant<int, DEC_MAX_CLUSTER < 8 ? DEC_MAX_CLUSTER : 8>{});
        else merge(std::integral_constant<int, DEC_MAX_CLUSTER>{});
        // nobody leaves while a peer may still read its partial result (nothing is published: a relaxed arrival)
        asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        return;
    }
    // The CTA that finishes last among the chunks of this (request, kv head) combines them:
    // out = sum_c acc_c 2^(m_c - M) / sum_c l_c 2^(m_c - M), chunks in increasing order.  The counter goes back to zero.
    const int c_first = lo / split_keys, c_last = pos / split_keys;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int arrived = atomicAdd(&counters[r * K + kh], 1);
        s_last = arrived == c_last - c_first;
        if (s_last) counters[r * K + kh] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // weights of the chunks first (one warp per head, lanes over chunks), then every thread sums its outputs
    const int n_c = c_last - c_first + 1;
    float* wgt = reinterpret_cast<float*>(dec_smem);               // [GROUP][n_c]; the rings are free now
    float* s_total = reinterpret_cast<float*>(s_m);                // [GROUP] sums of l_c * weight
    const bool fits = (size_t)GROUP * n_c * sizeof(float) <= (size_t)DEC_WARPS * WARP_BYTES;
    for (int g = warp; g < GROUP && fits; g += DEC_WARPS) {
        const size_t base = ((size_t)r * H + kh * GROUP + g) * max_chunks + c_first;
        float mm = -INFINITY;
        for (int c = lane; c < n_c; c += 32) mm = fmaxf(mm, __ldcg(&part_ml[(base + c) * 2]));
        mm = warp_max(mm);
        float ll = 0.0f;
        for (int c = lane; c < n_c; c += 32) {
            const float mc = __ldcg(&part_ml[(base + c) * 2]);
            const float f = mc == -INFINITY ? 0.0f : exp2f(mc - mm);
            wgt[g * n_c + c] = f;
            ll = fmaf(__ldcg(&part_ml[(base + c) * 2 + 1]), f, ll);
        }
        ll = warp_sum(ll);
        if (lane == 0) s_total[g] = ll;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < GROUP * D; idx += DEC_WARPS * 32) {
        const int g = idx / D, dd = idx % D;
        const size_t base = ((size_t)r * H + kh * GROUP + g) * max_chunks + c_first;
        float a = 0.0f, ll;
        if (fits) {
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
            int c = 0;
            for (; c + 4 <= n_c; c += 4) {
                a0 = fmaf(__ldcg(&part_acc[(base + c) * D + dd]), wgt[g * n_c + c], a0);
                a1 = fmaf(__ldcg(&part_acc[(base + c + 1) * D + dd]), wgt[g * n_c + c + 1], a1);
                a2 = fmaf(__ldcg(&part_acc[(base + c + 2) * D + dd]), wgt[g * n_c + c + 2], a2);
                a3 = fmaf(__ldcg(&part_acc[(base + c + 3) * D + dd]), wgt[g * n_c + c + 3], a3);
            }
            for (; c < n_c; ++c) a0 = fmaf(__ldcg(&part_acc[(base + c) * D + dd]), wgt[g * n_c + c], a0);
            a = (a0 + a1) + (a2 + a3);
            ll = s_total[g];
        } else {                                                   // more chunks than shared memory holds weights for
            float mm = -INFINITY;
            for (int c = 0; c < n_c; ++c) mm = fmaxf(mm, __ldcg(&part_ml[(base + c) * 2]));
            ll = 0.0f;
            for (int c = 0; c < n_c; ++c) {
                const float mc = __ldcg(&part_ml[(base + c) * 2]);
                const float f = mc == -INFINITY ? 0.0f : exp2f(mc - mm);
                a = fmaf(__ldcg(&part_acc[(base + c) * D + dd]), f, a);
                ll = fmaf(__ldcg(&part_ml[(base + c) * 2 + 1]), f, ll);
            }
        }
        out[((size_t)r * H + kh * GROUP + g) * D + dd] = __float2bfloat16_rn(a / ll);
    }
}

// ---- prefill ------------------------------------------------------------------------------------------------------
#define PF_BM 64
#define PF_BN 64
#define PF_LD LDP
#ifndef PF_BUFFERS
#define PF_BUFFERS 1                  // 1: one buffer for keys and values (more CTAs per SM); 2: the next block is prefetched
#endif
#ifndef PF_MIN_CTAS
#define PF_MIN_CTAS 3
#endif
#define PF_SMEM ((1 + 2 * PF_BUFFERS) * PF_BM * PF_LD * 2)

// Asks for the rows of one 64-key block of K and of V (cp.async); keys past `k_last` are zero (their pages may not
// exist).  One address computation per row serves both caches.
__device__ __forceinline__ void load_kv_tile(bf16* dst_k, bf16* dst_v, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                                             const int* __restrict__ table, int K, int kh, int page_shift, int key0, int k_last) {
    constexpr int CHUNKS = D / 8;
    const int page_mask = (1 << page_shift) - 1;
#pragma unroll
    for (int idx = threadIdx.x; idx < PF_BN * CHUNKS; idx += 128) {
        const int row = idx / CHUNKS, c = idx % CHUNKS;
        const int key = key0 + row;
        const int off = row * PF_LD + c * 8;
        if (key <= k_last) {
            const size_t at = ((((size_t)table[key >> page_shift] * K + kh) << page_shift) + (size_t)(key & page_mask)) * D + c * 8;
            cp_async16(dst_k + off, k_cache + at);
            cp_async16(dst_v + off, v_cache + at);
        } else {
            *reinterpret_cast<uint4*>(dst_k + off) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dst_v + off) = make_uint4(0, 0, 0, 0);
        }
    }
}

__global__ void __launch_bounds__(128, PF_MIN_CTAS) attn_prefill_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, bf16* __restrict__ out,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ cu_tokens, const int* __restrict__ seq_lens,
    int first_req, int K, int page_shift, float scale, int window) {
    PDL_ENTER_EARLY();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache);
    extern __shared__ __align__(16) uint8_t pf_smem[];
    bf16* sQ = reinterpret_cast<bf16*>(pf_smem);
    bf16* sKV = sQ + PF_BM * PF_LD;                  // [2 buffers][K then V][64][PF_LD]
    const int H = K * GROUP;
    const int r = first_req + blockIdx.z, h = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;   // long tiles first
    const int tok0 = cu_tokens[r], n = cu_tokens[r + 1] - tok0;
    if (qt * PF_BM >= n) return;
    const int len = seq_lens[r], pos0 = len - n;
    const int rows = min(PF_BM, n - qt * PF_BM);
    const int q_first = pos0 + qt * PF_BM, q_last = q_first + rows - 1;
    const int k_lo = window > 0 ? max(0, q_first - window + 1) : 0;
    const int kh = h / GROUP;
    const int* table = block_table + (size_t)r * max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int kb_first = k_lo / PF_BN, kb_last = q_last / PF_BN;
    {   // the query tile (rows past the request's tokens are zero) and the first block of keys and values
        constexpr int CHUNKS = D / 8;
        for (int idx = threadIdx.x; idx < PF_BM * CHUNKS; idx += 128) {
            const int row = idx / CHUNKS, c = idx % CHUNKS;
            bf16* d = sQ + row * PF_LD + c * 8;
            if (row < rows) cp_async16(d, q + ((size_t)(tok0 + qt * PF_BM + row) * H + h) * D + c * 8);
            else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
        load_kv_tile(sKV, sKV + PF_BN * PF_LD, k_cache, v_cache, table, K, kh, page_shift, kb_first * PF_BN, q_last);
        cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();
    const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PF_LD + (lane >> 4) * 8);

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const float sl2 = scale * 1.4426950408889634f;
    const int row0 = warp * 16 + (lane >> 2);                 // this thread's rows: row0 and row0 + 8
    const int qp0 = q_first + row0, qp1 = qp0 + 8;
    const int lo0 = window > 0 ? max(0, qp0 - window + 1) : 0, lo1 = window > 0 ? max(0, qp1 - window + 1) : 0;

    for (int kb = kb_first; kb <= kb_last; ++kb) {
        const int key0 = kb * PF_BN;
#if PF_BUFFERS == 2
        const int buf = (kb - kb_first) & 1;
        bf16* sK = sKV + (size_t)buf * 2 * PF_BN * PF_LD;
        bf16* sV = sK + PF_BN * PF_LD;
        if (kb < kb_last) {                                    // ask for the next block while this one is used
            bf16* nK = sKV + (size_t)(buf ^ 1) * 2 * PF_BN * PF_LD;
            load_kv_tile(nK, nK + PF_BN * PF_LD, k_cache, v_cache, table, K, kh, page_shift, key0 + PF_BN, q_last);
        }
        cp_async_commit();
        if (kb > kb_first) {
            cp_async_wait<1>();                                // this block has arrived (the next may still be on its way)
            __syncthreads();
        }
#else
        bf16* sK = sKV;
        bf16* sV = sK + PF_BN * PF_LD;
        if (kb > kb_first) {                                   // the barrier at the end of the last block freed the buffer
            load_kv_tile(sK, sV, k_cache, v_cache, table, K, kh, page_shift, key0, q_last);
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
        }
#endif

        float s[PF_BN / 8][4];
#pragma unroll
        for (int j = 0; j < PF_BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
        const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(sK + ((lane & 7) + (lane >> 4) * 8) * PF_LD + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t qa[4];
            ldsm_x4(q_addr + kk * 32, qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
            for (int j = 0; j < PF_BN / 8; j += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(k_addr + (uint32_t)(j * 8 * PF_LD * 2 + kk * 32), b0, b1, b2, b3);
                mma_bf16_16816(s[j], qa, b0, b1);
                mma_bf16_16816(s[j + 1], qa, b2, b3);
            }
        }
        // mask, online softmax
        float mx0 = -INFINITY, mx1 = -INFINITY;
        // a block needs masking only if it reaches past the tile's first query or starts before the last query's window
        const bool interior = key0 + PF_BN - 1 <= q_first && (window <= 0 || key0 >= q_last - window + 1);
        if (!interior) {
#pragma unroll
            for (int j = 0; j < PF_BN / 8; ++j) {
                const int key = key0 + j * 8 + 2 * (lane & 3);
                if (!(key <= qp0 && key >= lo0)) s[j][0] = -INFINITY;
                if (!(key + 1 <= qp0 && key + 1 >= lo0)) s[j][1] = -INFINITY;
                if (!(key <= qp1 && key >= lo1)) s[j][2] = -INFINITY;
                if (!(key + 1 <= qp1 && key + 1 >= lo1)) s[j][3] = -INFINITY;
            }
        }
#pragma unroll
        for (int j = 0; j < PF_BN / 8; ++j) {
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // running maxima are kept in log2 units (raw score * scale * log2 e); the scale is positive
        const float mn0 = fmaxf(m_run[0], mx0 * sl2), mn1 = fmaxf(m_run[1], mx1 * sl2);
        const float base0 = mn0 == -INFINITY ? 0.0f : mn0, base1 = mn1 == -INFINITY ? 0.0f : mn1;
        const float corr0 = fast_exp2(m_run[0] - base0), corr1 = fast_exp2(m_run[1] - base1);
        m_run[0] = mn0; m_run[1] = mn1;
        float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
        for (int j = 0; j < PF_BN / 8; ++j) {
            s[j][0] = fast_exp2(fmaf(s[j][0], sl2, -base0)); s[j][1] = fast_exp2(fmaf(s[j][1], sl2, -base0));
            s[j][2] = fast_exp2(fmaf(s[j][2], sl2, -base1)); s[j][3] = fast_exp2(fmaf(s[j][3], sl2, -base1));
            sum0 += s[j][0] + s[j][1];
            sum1 += s[j][2] + s[j][3];
        }
        l_run[0] = l_run[0] * corr0 + sum0;
        l_run[1] = l_run[1] * corr1 + sum1;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr0; o[i][1] *= corr0; o[i][2] *= corr1; o[i][3] *= corr1; }
        // O += P V
        const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(sV + ((lane & 7) + ((lane >> 3) & 1) * 8) * PF_LD + (lane >> 4) * 8);
#pragma unroll
        for (int ks = 0; ks < PF_BN / 16; ++ks) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
            pa[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            pa[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            pa[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int dt = 0; dt < D / 8; dt += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(v_addr + (uint32_t)(ks * 16 * PF_LD * 2 + dt * 16), b0, b1, b2, b3);
                mma_bf16_16816(o[dt], pa, b0, b1);
                mma_bf16_16816(o[dt + 1], pa, b2, b3);
            }
        }
        __syncthreads();                                       // everyone is done with this block's buffers
    }
    cp_async_wait<0>();
    // row sums live in four lanes each
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    const float inv0 = 1.0f / l_run[0], inv1 = 1.0f / l_run[1];
    const int col = 2 * (lane & 3);
    if (row0 < rows) {
        bf16* dst = out + ((size_t)(tok0 + qt * PF_BM + row0) * H + h) * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8 + col) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
    }
    if (row0 + 8 < rows) {
        bf16* dst = out + ((size_t)(tok0 + qt * PF_BM + row0 + 8) * H + h) * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8 + col) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------

// Pages hold a power-of-two number of positions: the kernels shift and mask instead of dividing.
static int page_shift_of(int page_size) {
    for (int s = 0; s < 16; ++s)
        if ((1 << s) == page_size) return s;
    return -1;
}

MB_API int mb_attn_head_dim() { return D; }
MB_API int mb_attn_group() { return GROUP; }
// Decode: q/out rows 0..requests-1 are the single new tokens of requests 0..requests-1.  A CTA takes split_keys
// keys (a multiple of 64); part_acc holds requests*H*max_chunks*HEAD_DIM floats and part_ml requests*H*max_chunks*2,
// with max_chunks >= ceil(longest/split_keys); counters holds requests*K ints that are zero between launches;
// cache_pages pages in each cache; error_flag receives a code if a wait on a copy gives up.
static int decode_map(CUtensorMap* map, const void* base, uint64_t rows) {
    EncodeTiled enc = encode_tiled();
    if (enc == nullptr) return MB_ERR_BAD_SIZE;
    cuuint64_t dims[2] = {(cuuint64_t)D, rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, DEC_STAGE_KEYS};
    cuuint32_t elem[2] = {1, 1};
    CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : 1000 + (int)rc;
}

// Clusters of more than 8 CTAs are a non-portable size: the kernels are allowed it once, and whether the device can
// place such a cluster at all (16 CTAs with this kernel's shared memory inside one GPC) is asked, not assumed.
template <bool TMA>
static bool decode_wide_clusters() {
    static int state = -1;
    if (state < 0) {
        state = 0;
        const int smem = TMA ? DEC_TMA_SMEM : DEC_SMEM;
        if (DEC_MAX_CLUSTER > 8 &&
            cudaFuncSetAttribute(attn_decode_split_kernel<TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
            cudaFuncSetAttribute(attn_decode_split_kernel<TMA>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(DEC_MAX_CLUSTER, 1, 1);
            cfg.blockDim = dim3(DEC_WARPS * 32);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = DEC_MAX_CLUSTER;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, attn_decode_split_kernel<TMA>, &cfg) == cudaSuccess && clusters >= 1) state = 1;
            else (void)cudaGetLastError();
        }
    }
    return state == 1;
}

// The most chunks of a sequence that the decode kernel merges as one cluster on this device (8 or DEC_MAX_CLUSTER).
MB_API int mb_attn_decode_max_cluster() {
    return (DEC_TMA ? decode_wide_clusters<true>() : decode_wide_clusters<false>()) ? DEC_MAX_CLUSTER : (DEC_MAX_CLUSTER < 8 ? DEC_MAX_CLUSTER : 8);
}

MB_API int mb_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                          int max_pages, const int* seq_lens, int requests, int K, int page_size, long long cache_pages,
                          float scale, int window, float* part_acc, float* part_ml, int* counters, int max_chunks,
                          int split_keys, int* error_flag, cudaStream_t s) {
    if (requests <= 0) return 0;
    if (max_chunks <= 0 || K <= 0 || split_keys < 16 * DEC_WARPS || split_keys % (16 * DEC_WARPS) != 0) return MB_ERR_BAD_SIZE;
    const int page_shift = page_shift_of(page_size);
    if (page_shift < 0) return MB_ERR_BAD_SIZE;
    dim3 grid(max_chunks, K, requests);
    const uint64_t rows = (uint64_t)cache_pages * K * page_size;
    const bool tma = DEC_TMA && page_shift >= 4 && error_flag != nullptr && rows > 0 && rows < (1ull << 31) &&
                     ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0;
    // a few chunks (up to 8, or 16 where the device places such clusters): they are one cluster and merge through
    // distributed shared memory, without scratch
    const int widest = max_chunks <= 8 ? 8 : ((tma ? decode_wide_clusters<true>() : decode_wide_clusters<false>()) ? DEC_MAX_CLUSTER : 8);
    const int cluster_merge = (max_chunks >= 2 && max_chunks <= widest) ? 1 : 0;
    const int cluster = cluster_merge ? -max_chunks : 0;
    CUtensorMap mk = {}, mv = {};
    if (tma) {
        int rc = decode_map(&mk, k_cache, rows);
        if (rc) return rc;
        rc = decode_map(&mv, v_cache, rows);
        if (rc) return rc;
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(attn_decode_split_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_TMA_SMEM);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        return launch_kernel(attn_decode_split_kernel<true>, grid, DEC_WARPS * 32, DEC_TMA_SMEM, s, cluster, mk, mv, (const bf16*)q,
                             (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_pages, seq_lens, K, page_shift, scale,
                             window, part_acc, part_ml, max_chunks, split_keys, counters, (bf16*)out, error_flag, cluster_merge);
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_split_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return launch_kernel(attn_decode_split_kernel<false>, grid, DEC_WARPS * 32, DEC_SMEM, s, cluster, mk, mv, (const bf16*)q,
                         (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_pages, seq_lens, K, page_shift, scale, window,
                         part_acc, part_ml, max_chunks, split_keys, counters, (bf16*)out, error_flag, cluster_merge);
}

// Prefill: requests first_req .. first_req+requests-1 of the step, each with its tokens cu_tokens[r]..cu_tokens[r+1].
MB_API int mb_attn_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                           int max_pages, const int* cu_tokens, const int* seq_lens, int first_req, int requests,
                           int max_query_len, int K, int page_size, float scale, int window, cudaStream_t s) {
    if (requests <= 0 || max_query_len <= 0) return 0;
    const int page_shift = page_shift_of(page_size);
    if (page_shift < 0) return MB_ERR_BAD_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((max_query_len + PF_BM - 1) / PF_BM, K * GROUP, requests);
    return launch_kernel(attn_prefill_kernel, grid, 128, PF_SMEM, s, 0, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                         (bf16*)out, block_table, max_pages, cu_tokens, seq_lens, first_req, K, page_shift, scale, window);
}
