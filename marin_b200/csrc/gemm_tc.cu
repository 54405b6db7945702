// bf16 matrix product on the 5th-generation tensor cores: out[t, n] (+)= sum_k x[t, k] * w[n, k].
//
// The weight matrix is the M operand of tcgen05.mma (128 rows of w per CTA) and the tokens are the N operand
// (BN = 16..256 tokens per CTA), so that a decode step with a handful of tokens still fills the 128-row
// datapath and streams every weight exactly once.  Both operands are K-major in global memory (w is
// [N, K], x is [T, K]) and are brought into shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle,
// no multicast) through a ring of STAGES buffers guarded by mbarriers; one thread issues the MMAs (two, into two
// accumulators that the epilogue adds, with up to 64 tokens), whose float32 accumulator lives in tensor memory; four
// warps read it back with tcgen05.ld and write out[t, n] (32 consecutive n per warp and token: coalesced).
//
// Split-K: with few tokens and few weight rows there are fewer tiles than SMs, so blockIdx.z cuts K into
// slices.  The slices of a tile are the CTAs of one thread-block cluster and add their partial tiles through
// distributed shared memory, in slice order (gemm_tc_kernel with cluster_reduce); without clusters each slice writes
// its float32 partial tile to scratch memory and the CTA that arrives last at the tile's counter adds them, again in
// slice order, and leaves the counter at zero for the next launch.
//
// Many tokens: gemm_tc_persistent_kernel, one CTA per SM walking over tiles, or over equal runs of k-blocks
// (stream-K in groups, see TcStreamK).
//
// Every wait on an mbarrier has a time limit; a wait that gives up records a code in *error_flag and the
// kernel winds down (tensor memory is freed on every path).  The reference's counterpart is its mma.sync
// kernel with hi/lo-split activations (crates/cuda/src/mma.cu:52-141).
#define MB_LIB "gemm_tc"
#define MB_LIB_ID 2
#include "tc_epilogue.cuh"
#include "launch.cuh"

#ifndef TC_ROWS4
#define TC_ROWS4 1             // the cluster's reduction four rows per thread (0: row by row)
#endif

// The cluster's reduction of a split-K tile, four weight rows of one token per thread (N a multiple of 4): every peer's
// slice of the partial tile comes through distributed shared memory in 16-byte loads, all of a thread's loads (up to
// U items x S slices) asked for before any is used; the slices are added in slice order, whatever S or the batch
// is, so the sums are the same bits as row by row.  Then what follows the product: "+=" into the residual stream with
// the norm's side outputs, the per-token factor of a norm ahead, or the plain store.
template <int S, int U>
__device__ __forceinline__ void cluster_reduce_rows4(uint32_t red_addr, void* out, int mode, int T, int N, int n0, int t0, int t_count,
                                                     const TcNormOut& norm, const TcRowScale& scale, const float* s_scale) {
    constexpr int rows_per = TC_BM / S, per_token = rows_per / 4;
    constexpr int group = rows_per < 32 ? rows_per : 32;              // rows whose squares are added into one slot
    constexpr int slots_per_tile = S < 4 ? 4 : S;
    const int row_first = blockIdx.z * rows_per;
    const int total = t_count * per_token;
    const bool acc_mode = mode == TC_OUT_F32_ACC;
    for (int base = 0; base < total; base += 128 * U) {               // every thread makes every trip (shuffles below)
        float4 old[U], gain[U], pv[U][S];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = base + u * 128 + threadIdx.x;
            const int tt = idx / per_token, row = row_first + 4 * (idx % per_token);
            const bool valid = idx < total && n0 + row < N;
            old[u] = (acc_mode && valid) ? *reinterpret_cast<const float4*>((const float*)out + (size_t)(t0 + tt) * N + n0 + row) : make_float4(0.f, 0.f, 0.f, 0.f);
            gain[u] = (norm.weight != nullptr && valid) ? *reinterpret_cast<const float4*>(norm.weight + n0 + row) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int z = 0; z < S; ++z) {
                pv[u][z] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (idx < total) {
                    uint32_t remote;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(red_addr + (uint32_t)(tt * TC_BM + row) * 4u), "r"(z));
                    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(pv[u][z].x), "=f"(pv[u][z].y), "=f"(pv[u][z].z), "=f"(pv[u][z].w) : "r"(remote) : "memory");
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (base + u * 128 >= total) break;                       // the same for every thread
            const int idx = base + u * 128 + threadIdx.x;
            const bool active = idx < total;
            const int tt = idx / per_token, in_slice = 4 * (idx % per_token), row = row_first + in_slice;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int z = 0; z < S; ++z) { sum[0] += pv[u][z].x; sum[1] += pv[u][z].y; sum[2] += pv[u][z].z; sum[3] += pv[u][z].w; }
            if (scale.sumsq != nullptr && active) {
                const float f = s_scale[tt];
#pragma unroll
                for (int e = 0; e < 4; ++e) sum[e] *= f;
            }
            const bool valid = active && n0 + row < N;
            const size_t at = (size_t)(t0 + tt) * N + n0 + row;
            float nv[4] = {0.f, 0.f, 0.f, 0.f};
            if (valid) {
                if (acc_mode) {
                    nv[0] = old[u].x + sum[0]; nv[1] = old[u].y + sum[1]; nv[2] = old[u].z + sum[2]; nv[3] = old[u].w + sum[3];
                    *reinterpret_cast<float4*>((float*)out + at) = make_float4(nv[0], nv[1], nv[2], nv[3]);
                    if (norm.weight != nullptr) {
                        const float o1 = norm.unit_offset ? 1.0f : 0.0f;
                        uint2 packed;
                        *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(nv[0] * (gain[u].x + o1), nv[1] * (gain[u].y + o1));
                        *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(nv[2] * (gain[u].z + o1), nv[3] * (gain[u].w + o1));
                        *reinterpret_cast<uint2*>(norm.scaled + at) = packed;
                    }
                } else if (mode == TC_OUT_BF16) {
                    uint2 packed;
                    *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(sum[0], sum[1]);
                    *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(sum[2], sum[3]);
                    *reinterpret_cast<uint2*>((bf16*)out + at) = packed;
                } else {
                    *reinterpret_cast<float4*>((float*)out + at) = make_float4(sum[0], sum[1], sum[2], sum[3]);
                }
            }
            if (norm.weight != nullptr) {
                // the squares of a group of rows: this thread's four, then the group's threads in a fixed tree
                const float sq = group_sum(((nv[0] * nv[0] + nv[1] * nv[1]) + nv[2] * nv[2]) + nv[3] * nv[3], group / 4);
                if (active && in_slice % group == 0) {
                    const int slot = blockIdx.x * slots_per_tile + blockIdx.z * (slots_per_tile / S) + in_slice / group;
                    norm.sumsq[(size_t)slot * T + t0 + tt] = sq;
                }
            }
        }
    }
}

// The same meeting of the cluster where the tile is one head of 128 elements (TcHeadsOut): CTA z finishes tokens z,
// z + S, ...; half a warp takes one token, a lane elements 4l..4l+3 and 64+4l..64+4l+3 (a rotation pair each), so the
// head's sum of squares needs four shuffles and the rotation none; eight tokens of a CTA are in flight at a time.
// All threads make every trip.
template <int S>
__device__ __forceinline__ void cluster_reduce_heads(uint32_t red_addr, int T, int t0, int t_count, const TcHeadsOut& heads,
                                                     const TcRowScale& scale, const float* s_scale) {
    const int head = blockIdx.x, lane = threadIdx.x & 31, hl = lane & 15, sub = threadIdx.x >> 4;
    const bool is_q = head < heads.H, is_k = !is_q && head < heads.H + heads.K;
    const float* hw = is_q ? heads.q_weight : (is_k ? heads.k_weight : nullptr);
    const bool rotate = (is_q || is_k) && heads.inv_freq != nullptr;
    float4 w_lo = make_float4(1.f, 1.f, 1.f, 1.f), w_hi = w_lo, freq = make_float4(0.f, 0.f, 0.f, 0.f);
    if (hw != nullptr) {
        w_lo = *reinterpret_cast<const float4*>(hw + 4 * hl);
        w_hi = *reinterpret_cast<const float4*>(hw + 64 + 4 * hl);
    }
    if (rotate) freq = *reinterpret_cast<const float4*>(heads.inv_freq + 4 * hl);
    const int mine = t_count > (int)blockIdx.z ? (t_count - (int)blockIdx.z + S - 1) / S : 0;
    for (int k0 = 0; k0 < mine; k0 += 8) {
        const int k = k0 + sub;
        const bool active = k < mine;
        const int tt = (int)blockIdx.z + S * k, t = t0 + tt;
        float4 lo[S], hi[S];
#pragma unroll
        for (int z = 0; z < S; ++z) {
            lo[z] = hi[z] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (active) {
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(red_addr + (uint32_t)(tt * TC_BM + 4 * hl) * 4u), "r"(z));
                asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(lo[z].x), "=f"(lo[z].y), "=f"(lo[z].z), "=f"(lo[z].w) : "r"(remote) : "memory");
                asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(hi[z].x), "=f"(hi[z].y), "=f"(hi[z].z), "=f"(hi[z].w) : "r"(remote + 256u) : "memory");
            }
        }
        int pos = 0, slot = -1;
        if (active) {
            if (rotate) pos = heads.positions[t];
            if (!is_q) slot = heads.slot_mapping[t];
        }
        float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int z = 0; z < S; ++z) {                                  // in slice order
            a[0] += lo[z].x; a[1] += lo[z].y; a[2] += lo[z].z; a[3] += lo[z].w;
            b[0] += hi[z].x; b[1] += hi[z].y; b[2] += hi[z].z; b[3] += hi[z].w;
        }
        const float f = (scale.sumsq != nullptr && active) ? s_scale[tt] : 1.0f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            // rounded to bf16 here, as the q|k|v rows are when they are written out and normed by a second kernel
            a[e] = __bfloat162float(__float2bfloat16_rn(a[e] * f));
            b[e] = __bfloat162float(__float2bfloat16_rn(b[e] * f));
        }
        if (hw != nullptr) {
            float ss = 0.0f;
#pragma unroll
            for (int e = 0; e < 4; ++e) ss += a[e] * a[e] + b[e] * b[e];
            ss = group_sum(ss, 16);
            const float rstd = 1.0f / sqrtf(ss / (float)TC_BM + heads.eps);
            const float wl[4] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w}, wh[4] = {w_hi.x, w_hi.y, w_hi.z, w_hi.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) { a[e] = a[e] * rstd * wl[e]; b[e] = b[e] * rstd * wh[e]; }
        }
        if (!active) continue;
        if (rotate) {
            const float fr[4] = {freq.x, freq.y, freq.z, freq.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sn, cs;
                sincosf((float)pos * fr[e], &sn, &cs);
                const float x = a[e], y = b[e];
                a[e] = x * cs - y * sn;
                b[e] = y * cs + x * sn;
            }
        }
        bf16* dst = nullptr;
        if (is_q) {
            dst = heads.q_out + ((size_t)t * heads.H + head) * TC_BM;
        } else if (slot >= 0) {
            const int kh = is_k ? head - heads.H : head - heads.H - heads.K;
            dst = (is_k ? heads.k_cache : heads.v_cache) +
                  (((size_t)(slot / heads.page_size) * heads.K + kh) * heads.page_size + (size_t)(slot % heads.page_size)) * TC_BM;
        }
        if (dst != nullptr) {
            uint2 out_lo, out_hi;
            *reinterpret_cast<__nv_bfloat162*>(&out_lo.x) = __floats2bfloat162_rn(a[0], a[1]);
            *reinterpret_cast<__nv_bfloat162*>(&out_lo.y) = __floats2bfloat162_rn(a[2], a[3]);
            *reinterpret_cast<__nv_bfloat162*>(&out_hi.x) = __floats2bfloat162_rn(b[0], b[1]);
            *reinterpret_cast<__nv_bfloat162*>(&out_hi.y) = __floats2bfloat162_rn(b[2], b[3]);
            *reinterpret_cast<uint2*>(dst + 4 * hl) = out_lo;
            *reinterpret_cast<uint2*>(dst + 64 + 4 * hl) = out_hi;
        }
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(128) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                      const __grid_constant__ CUtensorMap map_x, void* __restrict__ out,
                                                      int mode, int T, int N, int K, int kb_per_split,
                                                      float* __restrict__ partials, int* __restrict__ counters,
                                                      int* __restrict__ error_flag, int cluster_reduce,
                                                      const TcNormOut norm, const TcRowScale scale, const TcHeadsOut heads) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ float s_scale[BN];
    __shared__ float s_head[TC_BM], s_part[4];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    using L = TcSmem<BN>;
    uint64_t* full = (uint64_t*)(smem + STAGES * L::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accum + 1);
    int* last_slot = (int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TC_BM, t0 = blockIdx.y * BN;
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    const int kb_begin = blockIdx.z * kb_per_split;
    const int kb_end = min(total_kb, kb_begin + kb_per_split);
    const int nkb = kb_end - kb_begin;
    // Starting an MMA costs the issuing thread on the order of a hundred cycles, whatever its size, and with few tokens
    // that, not the data, sets the pace once the weights have landed: up to 64 tokens two threads issue, even k-blocks
    // into one accumulator and odd ones into a second, and the epilogue adds the two.
    constexpr bool DUAL = BN <= 64;
    // With two issuers the ring must have an even number of stages: a stage then belongs to one issuer for good.  With
    // an odd number the issuers take turns on a stage, and an issuer's first wait on it can be for the barrier's
    // second phase: a parity wait cannot tell "the second phase is over" from "the first has not ended yet", so the
    // issuer that is ahead would run MMAs on a stage that is still being filled and give it back once too often
    // (seen with five stages at 32 tokens: a launch failure once in a few hundred steps).
    static_assert(!DUAL || STAGES % 2 == 0, "two MMA issuers need an even number of stages");
    constexpr int NSC = DUAL ? 32 : 64;                               // threads that work out the per-token factors
    constexpr uint32_t TMEM_COLS = (DUAL ? 2 * BN : BN) < 32 ? 32 : (DUAL ? 2 * BN : BN);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(accum, DUAL ? 2 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    MB_TRACE_MARK();
    pdl_launch_dependents();
    if (warp == 0 && lane == 0) {
        // ---- producer: TMA loads into the ring.  The weights are written by no kernel, so the first tiles of w
        // are asked for before the wait on the kernels ahead in the stream; x is read only after it. ----
        const int early = min(nkb, STAGES);
        for (int i = 0; i < early; ++i) {
            mbar_expect_tx(&full[i], L::STAGE_BYTES);
            tma_load_2d(smem + i * L::STAGE_BYTES, &map_w, (kb_begin + i) * TC_BK, n0, &full[i]);
        }
        pdl_wait();
        for (int i = 0; i < early; ++i)
            tma_load_2d(smem + i * L::STAGE_BYTES + L::A_BYTES, &map_x, (kb_begin + i) * TC_BK, t0, &full[i]);
        for (int i = early; i < nkb; ++i) {
            const int s = i % STAGES;
            const uint32_t phase = (i / STAGES) & 1;
            if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(error_flag, 1); break; }
            mbar_expect_tx(&full[s], L::STAGE_BYTES);
            uint8_t* a = smem + s * L::STAGE_BYTES;
            const int k = (kb_begin + i) * TC_BK;
            tma_load_2d(a, &map_w, k, n0, &full[s]);
            tma_load_2d(a + L::A_BYTES, &map_x, k, t0, &full[s]);
        }
    } else if ((warp == 1 || (DUAL && warp == 3)) && lane == 0) {
        // ---- MMA issuers: thread `which` takes the k-blocks i = which, which + step, ... into accumulator `which` ----
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
        const int which = warp == 1 ? 0 : 1, step = DUAL ? 2 : 1;
        const uint32_t tmem_d = tmem_base + (uint32_t)(which * BN);
        bool ok = true;
        for (int i = which; i < nkb && ok; i += step) {
            const int s = i % STAGES;
            const uint32_t phase = (i / STAGES) & 1;
            if (!mbar_wait(&full[s], phase)) { atomicExch(error_flag, 2); ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a = smem_u32(smem + s * L::STAGE_BYTES);
            const uint64_t adesc = umma_desc(a), bdesc = umma_desc(a + L::A_BYTES);
#pragma unroll
            for (int kk = 0; kk < TC_BK / 16; ++kk)
                umma_bf16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (i > which || kk > 0) ? 1u : 0u);
            if (i + STAGES < nkb) umma_commit(&empty[s]);             // only a stage that is filled again needs to be given back
        }
        umma_commit(accum);
    } else if ((DUAL ? warp == 2 : warp >= 2) && scale.sumsq != nullptr) {
        // ---- the per-token factors of the norm ahead of this product: warp 2 (and 3, with one issuer) adds the slots, in slot order ----
        pdl_wait();
        // warps 2 and 3: `tpt` threads per token (a power of two, at most 32), each adds its share of the slots in
        // slot order, up to 24 loads in flight at a time; then the shares are added in a fixed tree
        const int here = min(BN, T - t0);
        int tpt = 32;
        while (tpt * here > NSC && tpt > 1) tpt >>= 1;
        const int local = threadIdx.x - 64, part = local % tpt;
        const int per = (scale.slots + tpt - 1) / tpt;
        const int trips = (BN * tpt + NSC - 1) / NSC;                 // the same for every thread: shuffles below
        for (int trip = 0; trip < trips; ++trip) {
            const int tt = trip * (NSC / tpt) + local / tpt;
            const int t = t0 + tt;
            float sum = 0.0f;
            if (tt < BN && t < T) {
                const int s_end = min(scale.slots, (part + 1) * per);
                for (int s0 = part * per; s0 < s_end; s0 += 24) {
                    float v[24];
#pragma unroll
                    for (int i = 0; i < 24; ++i) v[i] = s0 + i < s_end ? __ldcg(&scale.sumsq[(size_t)(s0 + i) * T + t]) : 0.0f;
#pragma unroll
                    for (int i = 0; i < 24; ++i) sum += v[i];
                }
            }
            sum = group_sum(sum, tpt);
            if (part == 0 && tt < BN) s_scale[tt] = t < T ? 1.0f / sqrtf(sum / (float)scale.dim + scale.eps) : 0.0f;
        }
    }
    __syncwarp();
    if (scale.sumsq != nullptr) __syncthreads();

    // ---- epilogue: every warp reads its 32 lanes of the accumulator ----
    pdl_wait();                                   // out may be read (+=) and is written: only after the kernels ahead
    bool have = nkb > 0;
    if (have) {
        if (!mbar_wait(accum, 0)) { if (lane == 0) atomicExch(error_flag, 3); have = false; }
    }
    have = __all_sync(0xffffffffu, have);     // tcgen05.ld below is warp-wide: the whole warp takes one path
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int n = n0 + warp * 32 + lane;
    const int splits = gridDim.z;
    const bool direct = splits == 1;
    if (cluster_reduce && !direct) {
        // ---- split-K inside a thread-block cluster: the K slices of one tile are the CTAs of one cluster.  Each
        // leaves its float32 partial tile in its own shared memory (the pipeline buffers are free now); after a
        // cluster barrier CTA z adds rows [z*128/S, (z+1)*128/S) of all S partials, in slice order, reading its
        // peers' tiles through distributed shared memory, and writes that part of the output.
        float* red = reinterpret_cast<float*>(smem);                 // [BN][128]: red[t][row]
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
            float v[16];
            if (have) {
                tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
                if (DUAL && nkb >= 2) {                               // the odd k-blocks' accumulator
                    float v2[16];
                    tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(BN + c0), v2);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] += v2[j];
                }
            }
            else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) red[(c0 + j) * TC_BM + warp * 32 + lane] = v[j];
        }
        // this CTA's tile is in place: say so to the cluster now, and wait for the peers only when their tiles are needed
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        const int rows_per = TC_BM / splits;                         // splits is 2, 4 or 8
        const int row_first = blockIdx.z * rows_per;
        const int t_count = min(BN, T - t0);
        if (heads.q_out != nullptr) {
            if (BN <= 16) {
                // few tokens: all 128 threads on one token at a time (one angle each) is the shorter chain
                // ---- this tile is one head: CTA z finishes tokens z, z + splits, ...; a thread is one element of the head
                const int head = blockIdx.x, i = threadIdx.x;
                const bool is_q = head < heads.H, is_k = !is_q && head < heads.H + heads.K;
                const float* hw = is_q ? heads.q_weight : (is_k ? heads.k_weight : nullptr);
                const float wi = hw != nullptr ? hw[i] : 1.0f;
                const bool rotate = (is_q || is_k) && heads.inv_freq != nullptr;
                const float freq = rotate ? heads.inv_freq[i & 63] : 0.0f;
                asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
                const uint32_t red_addr = smem_u32(red);
                for (int tt = blockIdx.z; tt < t_count; tt += splits) {
                    const int t = t0 + tt;
                    float sum = 0.0f;
                    for (int z = 0; z < splits; ++z) {
                        uint32_t remote;
                        float pv;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(red_addr + (uint32_t)(tt * TC_BM + i) * 4u), "r"(z));
                        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv) : "r"(remote) : "memory");
                        sum += pv;
                    }
                    if (scale.sumsq != nullptr) sum *= s_scale[tt];
                    // rounded to bf16 here, as the q|k|v rows are when they are written out and normed by a second kernel
                    float v = __bfloat162float(__float2bfloat16_rn(sum));
                    if (hw != nullptr) {
                        const float ss = group_sum(v * v, 32);
                        if (lane == 0) s_part[warp] = ss;
                        __syncthreads();
                        const float total = ((s_part[0] + s_part[1]) + s_part[2]) + s_part[3];
                        v = v * (1.0f / sqrtf(total / (float)TC_BM + heads.eps)) * wi;
                    }
                    if (rotate) {
                        s_head[i] = v;
                        __syncthreads();
                        const float other = s_head[i ^ 64];
                        float sn, cs;
                        sincosf((float)heads.positions[t] * freq, &sn, &cs);
                        v = i < 64 ? v * cs - other * sn : v * cs + other * sn;
                    }
                    if (is_q) {
                        heads.q_out[((size_t)t * heads.H + head) * TC_BM + i] = __float2bfloat16_rn(v);
                    } else {
                        const int slot = heads.slot_mapping[t];
                        if (slot >= 0) {
                            const int kh = is_k ? head - heads.H : head - heads.H - heads.K;
                            bf16* cache = is_k ? heads.k_cache : heads.v_cache;
                            cache[(((size_t)(slot / heads.page_size) * heads.K + kh) * heads.page_size + (size_t)(slot % heads.page_size)) * TC_BM + i] =
                                __float2bfloat16_rn(v);
                        }
                    }
                    __syncthreads();                                      // s_part and s_head are used again
                }
                asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
            } else {
                // ---- this tile is one head ----
                asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
                const uint32_t red_addr = smem_u32(red);
                if (splits == 8) cluster_reduce_heads<8>(red_addr, T, t0, t_count, heads, scale, s_scale);
                else if (splits == 4) cluster_reduce_heads<4>(red_addr, T, t0, t_count, heads, scale, s_scale);
                else cluster_reduce_heads<2>(red_addr, T, t0, t_count, heads, scale, s_scale);
                asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
            }
        } else if (TC_ROWS4 && N % 4 == 0) {
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
            const uint32_t red_addr = smem_u32(red);
            // items of a thread in flight at a time: all of them where the registers allow
            constexpr int U8 = BN >= 32 ? 2 : 1, U4 = BN >= 64 ? 4 : (BN >= 32 ? 2 : 1), U2 = BN >= 32 ? 4 : (BN >= 16 ? 2 : 1);
            if (splits == 8) cluster_reduce_rows4<8, U8>(red_addr, out, mode, T, N, n0, t0, t_count, norm, scale, s_scale);
            else if (splits == 4) cluster_reduce_rows4<4, U4>(red_addr, out, mode, T, N, n0, t0, t_count, norm, scale, s_scale);
            else cluster_reduce_rows4<2, U2>(red_addr, out, mode, T, N, n0, t0, t_count, norm, scale, s_scale);
            asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        } else {
        // Trips of 128 (token, row) pairs, four at a time: all loads of the four (the old values from global memory,
        // then the slices from the peers' shared memory) are asked for before any is used, so their latencies overlap.
        // What the first four need from global memory is asked for before the cluster meets.
        constexpr int U = BN >= 64 ? 4 : (BN >= 32 ? 2 : 1);
        const int total = t_count * rows_per;
        const bool acc_mode = mode == TC_OUT_F32_ACC;
        float old[U], gain[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = u * 128 + threadIdx.x;
            const int tt = idx / rows_per, row = row_first + idx % rows_per;
            const bool valid = idx < total && n0 + row < N;
            old[u] = (acc_mode && valid) ? ((const float*)out)[(size_t)(t0 + tt) * N + n0 + row] : 0.0f;
            gain[u] = (norm.weight != nullptr && valid) ? norm.weight[n0 + row] : 0.0f;
        }
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        const uint32_t red_addr = smem_u32(red);
        const int group = rows_per < 32 ? rows_per : 32;             // rows whose squares are added into one slot
        const int slots_per_tile = splits < 4 ? 4 : splits;
        for (int base = 0; base < total; base += 128 * U) {           // every thread makes every trip (shuffles below)
            if (base > 0) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int idx = base + u * 128 + threadIdx.x;
                    const int tt = idx / rows_per, row = row_first + idx % rows_per;
                    const bool valid = idx < total && n0 + row < N;
                    old[u] = (acc_mode && valid) ? ((const float*)out)[(size_t)(t0 + tt) * N + n0 + row] : 0.0f;
                    gain[u] = (norm.weight != nullptr && valid) ? norm.weight[n0 + row] : 0.0f;
                }
            }
            float pv[U][8];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = base + u * 128 + threadIdx.x;
                const int tt = idx / rows_per, row = row_first + idx % rows_per;
#pragma unroll
                for (int z = 0; z < 8; ++z) {
                    pv[u][z] = 0.0f;
                    if (z < splits && idx < total) {
                        uint32_t remote;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(red_addr + (uint32_t)(tt * TC_BM + row) * 4u), "r"(z));
                        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv[u][z]) : "r"(remote) : "memory");
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (base + u * 128 >= total) break;                   // the same for every thread
                const int idx = base + u * 128 + threadIdx.x;
                const bool active = idx < total;
                const int tt = idx / rows_per, in_slice = idx % rows_per, row = row_first + in_slice;
                float sum = 0.0f;
#pragma unroll
                for (int z = 0; z < 8; ++z) sum += pv[u][z];          // slices beyond `splits` are zero
                if (scale.sumsq != nullptr && active) sum *= s_scale[tt];
                const bool valid = active && n0 + row < N;
                const size_t at = (size_t)(t0 + tt) * N + n0 + row;
                float nv = 0.0f;
                if (valid) {
                    if (acc_mode) {
                        nv = old[u] + sum;
                        ((float*)out)[at] = nv;
                        if (norm.weight != nullptr) norm.scaled[at] = __float2bfloat16_rn(nv * (norm.unit_offset ? gain[u] + 1.0f : gain[u]));
                    } else {
                        store_out(out, mode, at, sum);
                    }
                }
                if (norm.weight != nullptr) {
                    const float sq = group_sum(nv * nv, group);
                    if (active && in_slice % group == 0) {
                        const int slot = blockIdx.x * slots_per_tile + blockIdx.z * (slots_per_tile / splits) + in_slice / group;
                        norm.sumsq[(size_t)slot * T + t0 + tt] = sq;
                    }
                }
            }
        }
        // nobody leaves while a peer may still read its tile (nothing is published here: a relaxed arrival does not wait
        // for this CTA's own stores to drain)
        asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        }
    } else {
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16];
        if (have) {
            tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
            if (DUAL && nkb >= 2) {                                   // the odd k-blocks' accumulator
                float v2[16];
                tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(BN + c0), v2);
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += v2[j];
            }
        }
        else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
        }
        if (direct && scale.sumsq != nullptr) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] *= s_scale[c0 + j];
        }
        if (direct && norm.weight != nullptr) {
            store_chunk_norm(out, t0 + c0, n, n < N, T, N, v, norm, norm.sumsq + (size_t)(blockIdx.x * 4 + warp) * T, lane);
        } else if (direct && mode == TC_OUT_SWIGLU) {
            if (n0 + warp * 32 < N) store_chunk_swiglu(out, t0 + c0, n0 + warp * 32, lane, T, N, v);
        } else if (n < N) {
            if (direct) store_chunk(out, mode, t0 + c0, n, T, N, v);
            else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int t = t0 + c0 + j;
                    if (t < T) partials[((size_t)blockIdx.z * T + t) * N + n] = v[j];
                }
            }
        }
    }
    if (!direct) {
        // ---- split-K through global scratch: the CTA that arrives last adds the slices in order ----
        __threadfence();
        __syncthreads();
        const int tile = blockIdx.y * gridDim.x + blockIdx.x;
        if (threadIdx.x == 0) {
            const int old = atomicAdd(&counters[tile], 1);
            *last_slot = old == splits - 1;
            if (old == splits - 1) counters[tile] = 0;
        }
        __syncthreads();
        if (*last_slot) {
            __threadfence();
            if (n < N) {
                const int t_end = min(T, t0 + BN);
                for (int t = t0; t < t_end; ++t) {
                    float sum = 0.0f;
                    for (int z = 0; z < splits; ++z) sum += __ldcg(&partials[((size_t)z * T + t) * N + n]);
                    store_out(out, mode, (size_t)t * N + n, sum);
                }
            }
        }
    }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- the persistent kernel for many tokens -------------------------------------------------------------------------
// One CTA per SM walks over output tiles (128 weight rows x BN tokens).  Warp 0 feeds the shared-memory ring with
// TMA and runs ahead into the next tile; warp 1 issues the MMAs into one of two accumulators in tensor memory;
// warps 2..9 drain the other accumulator (tcgen05.ld, convert, store; two warps per 32-lane quarter) meanwhile, so the tensor cores do not wait
// for the epilogue.
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// The order of tiles.  CTAs that run at the same time take consecutive tiles, so what is fastest decides what they
// share: with TC_TOKENS_FASTEST (the default) a wave holds few weight tiles, each under all token tiles, and the
// weight matrix comes from HBM once (x, much smaller, stays in L2); the other order streams all of w once per
// token tile.
#ifndef TC_WEIGHTS_FASTEST
__device__ __forceinline__ int tile_rows(int tile, int tiles_n, int tiles_t) { return tile / tiles_t; }
__device__ __forceinline__ int tile_tokens(int tile, int tiles_n, int tiles_t) { return tile % tiles_t; }
#else
__device__ __forceinline__ int tile_rows(int tile, int tiles_n, int tiles_t) { return tile % tiles_n; }
__device__ __forceinline__ int tile_tokens(int tile, int tiles_n, int tiles_t) { return tile / tiles_n; }
#endif

// What a CTA of the persistent kernel works on, piece by piece.  Tile by tile (units_per_group = 0): tiles blockIdx.x,
// blockIdx.x + gridDim.x, ... each over all of k.  Stream-K (units_per_group > 0): the CTAs form groups of tiles_t,
// one CTA for each token tile; the weight-row tiles laid end to end are tiles_n * nkb k-blocks, and group g takes
// k-blocks [g * units_per_group, (g + 1) * units_per_group) of them, whatever row tiles they fall into.  Every SM
// gets the same amount of work however many tiles there are, and the CTAs of a group walk the same weight k-blocks
// at the same time (one copy from HBM, the others from L2), which dealing k-blocks to single CTAs would lose.  With
// units_per_group >= nkb (the launcher sees to it) a tile is shared by two CTAs at most: CTA c + tiles_t starts with
// the tile's last k-blocks (its first piece), CTA c ends with the tile's first k-blocks (its last piece).
struct TcStreamK {
    float* partials;        // [ctas][BN][128] float32: the piece a CTA began with, if it began inside a tile
    int* flags;             // [ctas][8]: one per epilogue warp; 1 while that warp's part of the piece is there
    int units_per_group;
};

struct TcWalk {
    int nkb, limit, step, at, token_tile, tiles_t;
    bool streamk;
    __device__ TcWalk(const TcStreamK& sk, bool streamk_, int tiles_n, int tiles_t_, int nkb_) : nkb(nkb_), tiles_t(tiles_t_), streamk(streamk_) {
        if (streamk) {
            const int group = blockIdx.x / tiles_t_;
            token_tile = blockIdx.x - group * tiles_t_;
            const long long total = (long long)tiles_n * nkb_;
            const long long from = (long long)group * sk.units_per_group, to = from + sk.units_per_group;
            at = (int)(from < total ? from : total);
            limit = (int)(to < total ? to : total);
            step = 0;
        } else {
            at = blockIdx.x; limit = tiles_n * tiles_t_; step = gridDim.x; token_tile = 0;
        }
    }
    // the next piece: k-blocks [kb0, kb1) of `tile` (numbered with the token tiles fastest)
    __device__ bool next(int& tile, int& kb0, int& kb1) {
        if (at >= limit) return false;
        if (!streamk) { tile = at; kb0 = 0; kb1 = nkb; at += step; return true; }
        const int row = at / nkb;
        tile = row * tiles_t + token_tile;
        kb0 = at - row * nkb;
        kb1 = kb0 + (limit - at) < nkb ? kb0 + (limit - at) : nkb;
        at += kb1 - kb0;
        return true;
    }
};

#ifdef TC_PROBE
// Where the roles of the persistent kernel spend their time (a build for measuring only, -DTC_PROBE): per CTA, clock
// ticks of [0] the producer waiting for a free stage, [1] the producer issuing, [2] the MMA thread waiting for a full
// stage, [3] the MMA thread waiting for a free accumulator, [4] the MMA thread in all.
__device__ long long tc_probe[148 * 8];
MB_API int mb_gemm_tc_probe_read(long long* host) { return (int)cudaMemcpyFromSymbol(host, tc_probe, sizeof(tc_probe)); }
#define PROBE_DECL(name) long long name = 0
#define PROBE_T() clock64()
#define PROBE_ADD(name, since) name += clock64() - (since)
#define PROBE_OUT(slot, name) if (blockIdx.x < 148) tc_probe[blockIdx.x * 8 + (slot)] = name
#else
#define PROBE_DECL(name)
#define PROBE_T() 0
#define PROBE_ADD(name, since) (void)(since)
#define PROBE_OUT(slot, name)
#endif

template <int BN, int STAGES, bool SK>
__global__ void __launch_bounds__(320) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                 const __grid_constant__ CUtensorMap map_x,
                                                                 void* __restrict__ out, int mode, int T, int N, int K,
                                                                 int* __restrict__ error_flag, const TcNormOut norm,
                                                                 const TcRowScale scale, const TcStreamK sk, const TcHeadsOut heads,
                                                                 const float* __restrict__ rope,
                                                                 const __grid_constant__ CUtensorMap map_out, int reduce_out) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ float s_pscale[2][BN];          // the per-token factors of a coupled norm, for the tile in each accumulator
    // heads finished in the epilogue: per half of the columns (its four warps), two staging buffers of sixteen tokens
    __shared__ __align__(128) bf16 s_hx[2][2][16 * TC_BM];     // (also, as floats, the staging of a "+=" by TMA reduction: 8 KB per half)
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    using L = TcSmem<BN>;
    uint64_t* full = (uint64_t*)(smem + STAGES * L::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;       // [2]
    uint64_t* acc_empty = acc_full + 2;        // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (N + TC_BM - 1) / TC_BM, tiles_t = (T + BN - 1) / BN;
    const int nkb = (K + TC_BK - 1) / TC_BK;
    constexpr uint32_t TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    PDL_ENTER_EARLY();

    if (warp == 0 && lane == 0) {
        int it = 0;                                                   // k-blocks issued so far, over all tiles
        bool ok = true;
        PROBE_DECL(p_wait); PROBE_DECL(p_issue);
        TcWalk walk(sk, SK, tiles_n, tiles_t, nkb);
        for (int tile, kb0, kb1; ok && walk.next(tile, kb0, kb1);) {
            const int n0 = tile_rows(tile, tiles_n, tiles_t) * TC_BM, t0 = tile_tokens(tile, tiles_n, tiles_t) * BN;
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t phase = (it / STAGES) & 1;
                const long long pt0 = PROBE_T();
                if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(error_flag, 11); ok = false; break; }
                PROBE_ADD(p_wait, pt0);
                const long long pt1 = PROBE_T();
                mbar_expect_tx(&full[s], L::STAGE_BYTES);
                uint8_t* a = smem + s * L::STAGE_BYTES;
                tma_load_2d(a, &map_w, kb * TC_BK, n0, &full[s]);
                tma_load_2d(a + L::A_BYTES, &map_x, kb * TC_BK, t0, &full[s]);
                PROBE_ADD(p_issue, pt1);
            }
        }
        PROBE_OUT(0, p_wait); PROBE_OUT(1, p_issue);
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
        int it = 0, local = 0;
        bool ok = true;
        PROBE_DECL(m_full); PROBE_DECL(m_acc); PROBE_DECL(m_all);
        const long long mt_start = PROBE_T();
        TcWalk walk(sk, SK, tiles_n, tiles_t, nkb);
        for (int tile, kb0, kb1; ok && walk.next(tile, kb0, kb1); ++local) {
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            const long long mt0 = PROBE_T();
            if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1)) { atomicExch(error_flag, 12); ok = false; break; }
            PROBE_ADD(m_acc, mt0);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t phase = (it / STAGES) & 1;
                const long long mt1 = PROBE_T();
                if (!mbar_wait(&full[s], phase)) { atomicExch(error_flag, 13); ok = false; break; }
                PROBE_ADD(m_full, mt1);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a = smem_u32(smem + s * L::STAGE_BYTES);
                const uint64_t adesc = umma_desc(a), bdesc = umma_desc(a + L::A_BYTES);
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)
                    umma_bf16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            umma_commit(&acc_full[buf]);
        }
        PROBE_ADD(m_all, mt_start);
        PROBE_OUT(2, m_full); PROBE_OUT(3, m_acc); PROBE_OUT(4, m_all);
    } else if (warp >= 2) {
        const int quarter = warp & 3;                                 // the 32 TMEM lanes this warp may read
        const int col_half = (warp - 2) >> 2;                         // two warps share a quarter: each takes half the columns
        constexpr int HALF_COLS = ((BN / 16 + 1) / 2) * 16;
        int local = 0;
        int heads_chunk = 0;                                          // chunks this warp has staged (TcHeadsOut): picks the buffer
        bool ok = true;
        TcWalk walk(sk, SK, tiles_n, tiles_t, nkb);
        for (int tile, kb0, kb1; walk.next(tile, kb0, kb1); ++local) {
            const bool is_tail = SK && kb0 > 0;    // the tile's last k-blocks: parked for the CTA that has its first ones
            const bool is_head = SK && kb1 < nkb;  // the tile's first k-blocks: the next CTA's parked piece is added
            const int tile_row = tile_rows(tile, tiles_n, tiles_t);
            const int n0 = tile_row * TC_BM, t0 = tile_tokens(tile, tiles_n, tiles_t) * BN;
            const int buf = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            if (scale.sumsq != nullptr) {
                // while the MMAs of this tile run: each of the 256 epilogue threads adds the slots of one token, in slot
                // order, up to 24 loads in flight; the eight warps then meet at a barrier of their own
                for (int e = (warp - 2) * 32 + lane; e < BN; e += 256) {
                    const int t = t0 + e;
                    float sum = 0.0f;
                    if (t < T) {
                        for (int s0 = 0; s0 < scale.slots; s0 += 24) {
                            float part[24];
#pragma unroll
                            for (int i = 0; i < 24; ++i) part[i] = s0 + i < scale.slots ? __ldcg(&scale.sumsq[(size_t)(s0 + i) * T + t]) : 0.0f;
#pragma unroll
                            for (int i = 0; i < 24; ++i) sum += part[i];
                        }
                    }
                    s_pscale[buf][e] = t < T ? 1.0f / sqrtf(sum / (float)scale.dim + scale.eps) : 0.0f;
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
            }
            const int c_begin = col_half * HALF_COLS, c_end = col_half == 0 ? HALF_COLS : BN;
            const int n = n0 + quarter * 32 + lane;
            float4 rope_c[2], rope_s[2];
            int kv_slot[2];
            // TcHeadsOut: the angles and the cache slot of the two tokens this lane finishes in a chunk come from global
            // memory, an L2 round trip that nothing in the chunk could hide: they are asked for one chunk ahead
            auto heads_fetch = [&](int c0) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int t = t0 + c0 + r * 8 + quarter * 2 + (lane >> 4);
                    const bool is_q = tile_row < heads.H;
                    const bool there = t < T && c0 < c_end;
                    if (there && rope != nullptr && tile_row < heads.H + heads.K) {
                        rope_c[r] = __ldg(reinterpret_cast<const float4*>(rope + (size_t)t * TC_BM) + (lane & 15));
                        rope_s[r] = __ldg(reinterpret_cast<const float4*>(rope + (size_t)t * TC_BM + 64) + (lane & 15));
                    }
                    kv_slot[r] = (there && !is_q) ? __ldg(heads.slot_mapping + t) : -1;
                }
            };
            if (!SK && heads.q_out != nullptr) heads_fetch(c_begin);
            // the four warps that share a half of the columns meet at barriers inside some epilogues' chunks (ids 2 and
            // 3): there they go on together or not at all
            auto half_agrees = [&](bool mine) {
                uint32_t all_ok;
                asm volatile("{ .reg .pred p, q; setp.ne.u32 p, %1, 0; bar.red.and.pred q, %2, 128, p; selp.u32 %0, 1, 0, q; }"
                             : "=r"(all_ok) : "r"((uint32_t)mine), "r"(2 + col_half) : "memory");
                return all_ok != 0;
            };
            // what happens to 16 finished columns of this thread's row
            auto finish_chunk = [&](float* v, int c0) {
                if (!SK && heads.q_out != nullptr) {
                    // This tile is one head (128 rows) of sixteen tokens here.  The four warps that share this half of
                    // the columns lay their values, rounded to bf16 as a stored row would be, token by token into a
                    // staging buffer and meet at a barrier of their own (id 2 or 3; every one of them makes every
                    // trip).  Then half a warp takes one token: a lane holds elements 4l..4l+3 and 64+4l..64+4l+3,
                    // a rotation pair each, so the per-head RMS norm needs four shuffles and the rotation none, and the
                    // head leaves as 128 contiguous bytes twice: to the query rows or into the paged cache, as the
                    // kernel of few tokens does it (TcHeadsOut).  Two buffers in turn: a warp reaches the next
                    // chunk's barrier only after it has read this chunk's buffer, so one barrier a chunk is enough.
                    const int head = tile_row;
                    const bool is_q = head < heads.H, is_k = !is_q && head < heads.H + heads.K;
                    const float* hw = is_q ? heads.q_weight : (is_k ? heads.k_weight : nullptr);
                    const bool rotate = (is_q || is_k) && rope != nullptr;
                    bf16* stage = s_hx[col_half][heads_chunk & 1];
                    ++heads_chunk;
                    const int row = quarter * 32 + lane;
#pragma unroll
                    for (int j = 0; j < 16; ++j) stage[j * TC_BM + row] = __float2bfloat16_rn(v[j]);
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + col_half) : "memory");
                    const int hl = lane & 15;
                    float4 w_lo = make_float4(1.0f, 1.0f, 1.0f, 1.0f), w_hi = w_lo;
                    if (hw != nullptr) {
                        w_lo = __ldg(reinterpret_cast<const float4*>(hw) + hl);
                        w_hi = __ldg(reinterpret_cast<const float4*>(hw + 64) + hl);
                    }
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const int j = r * 8 + quarter * 2 + (lane >> 4);
                        const int t = t0 + c0 + j;
                        const uint2 raw_lo = *reinterpret_cast<const uint2*>(stage + j * TC_BM + 4 * hl);
                        const uint2 raw_hi = *reinterpret_cast<const uint2*>(stage + j * TC_BM + 64 + 4 * hl);
                        float a[4], b[4];
                        {
                            const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw_lo.x));
                            const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw_lo.y));
                            const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw_hi.x));
                            const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw_hi.y));
                            a[0] = a0.x; a[1] = a0.y; a[2] = a1.x; a[3] = a1.y;
                            b[0] = b0.x; b[1] = b0.y; b[2] = b1.x; b[3] = b1.y;
                        }
                        if (hw != nullptr) {
                            float ss = 0.0f;
#pragma unroll
                            for (int e = 0; e < 4; ++e) ss += a[e] * a[e] + b[e] * b[e];
                            ss = group_sum(ss, 16);
                            const float rstd = 1.0f / sqrtf(ss / (float)TC_BM + heads.eps);
                            const float wl[4] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w}, wh[4] = {w_hi.x, w_hi.y, w_hi.z, w_hi.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) { a[e] = a[e] * rstd * wl[e]; b[e] = b[e] * rstd * wh[e]; }
                        }
                        if (t >= T) continue;
                        if (rotate) {
                            const float4 c4 = rope_c[r], s4 = rope_s[r];
                            const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float x = a[e], y = b[e];
                                a[e] = x * cs[e] - y * sn[e];
                                b[e] = y * cs[e] + x * sn[e];
                            }
                        }
                        bf16* dst = nullptr;
                        if (is_q) {
                            dst = heads.q_out + ((size_t)t * heads.H + head) * TC_BM;
                        } else {
                            const int slot = kv_slot[r];
                            if (slot >= 0) {
                                const int kh = is_k ? head - heads.H : head - heads.H - heads.K;
                                dst = (is_k ? heads.k_cache : heads.v_cache) +
                                      (((size_t)(slot / heads.page_size) * heads.K + kh) * heads.page_size + (size_t)(slot % heads.page_size)) * TC_BM;
                            }
                        }
                        if (dst != nullptr) {
                            uint2 out_lo, out_hi;
                            *reinterpret_cast<__nv_bfloat162*>(&out_lo.x) = __floats2bfloat162_rn(a[0], a[1]);
                            *reinterpret_cast<__nv_bfloat162*>(&out_lo.y) = __floats2bfloat162_rn(a[2], a[3]);
                            *reinterpret_cast<__nv_bfloat162*>(&out_hi.x) = __floats2bfloat162_rn(b[0], b[1]);
                            *reinterpret_cast<__nv_bfloat162*>(&out_hi.y) = __floats2bfloat162_rn(b[2], b[3]);
                            *reinterpret_cast<uint2*>(dst + 4 * hl) = out_lo;
                            *reinterpret_cast<uint2*>(dst + 64 + 4 * hl) = out_hi;
                        }
                    }
                    heads_fetch(c0 + 16);
                    return;
                }
                if (scale.sumsq != nullptr) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] *= s_pscale[buf][c0 + j];
                }
                if (norm.weight != nullptr) {
                    store_chunk_norm(out, t0 + c0, n, n < N, T, N, v, norm, norm.sumsq + (size_t)(tile_row * 4 + quarter) * T, lane);
                } else if (mode == TC_OUT_SWIGLU) {
                    if (n0 + quarter * 32 < N) store_chunk_swiglu(out, t0 + c0, n0 + quarter * 32, lane, T, N, v);
                } else if (reduce_out) {
                    // "+=" into float32 without reading the old values: the four warps that share this half of the columns
                    // lay sixteen tokens of the tile into shared memory and one thread hands them to a TMA reduction
                    // (an add in L2; rows and tokens past the matrix are clipped).  One add per element and launch: the
                    // same bits every time.  The buffer is used again once the reduction before has read it.
                    float* stage = reinterpret_cast<float*>(&s_hx[col_half][0][0]);
                    const bool issuer = quarter == 0 && lane == 0;
                    if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + col_half) : "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) stage[j * TC_BM + quarter * 32 + lane] = v[j];
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + col_half) : "memory");
                    if (issuer) {
                        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                                     ::"l"(&map_out), "r"(smem_u32(stage)), "r"(n0), "r"(t0 + c0) : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (n < N) store_chunk(out, mode, t0 + c0, n, T, N, v);
            };
            // the parked piece: [BN columns][128 rows], so that a warp's 32 lanes store and load 128 contiguous bytes;
            // this warp reads exactly what the warp of the same number wrote in the other CTA
            float* parked = SK ? sk.partials + (size_t)(blockIdx.x + (is_head ? tiles_t : 0)) * BN * TC_BM + quarter * 32 + lane : nullptr;
            int* parked_flag = SK ? sk.flags + (blockIdx.x + (is_head ? tiles_t : 0)) * 8 + (warp - 2) : nullptr;
            if (SK && is_head) {
                // The other CTA parked its piece first thing and this is our last piece: the wait is short or none.
                // The piece comes from L2 a microsecond after it is asked for, and nothing runs beside this last
                // epilogue: its first chunks are asked for here, while the MMAs of the piece still run, and each
                // later chunk as soon as a register set is free.
                constexpr int AHEAD = 4;
                float pre[AHEAD][16];
                bool there = false;
                if (ok && lane == 0) {
                    for (int spin = 0; spin < (1 << 22) && !there; ++spin) {
                        int seen;
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(parked_flag) : "memory");
                        there = seen == 1;
                        if (!there) __nanosleep(64);
                    }
                    if (!there) atomicExch(error_flag, 15);
                }
                there = __shfl_sync(0xffffffffu, there, 0);
                __syncwarp();
                if (!there) ok = false;
                if (ok) {
#pragma unroll
                    for (int c = 0; c < AHEAD; ++c) {
                        if (c_begin + c * 16 < c_end) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) pre[c][j] = __ldcg(parked + (size_t)(c_begin + c * 16 + j) * TC_BM);
                        }
                    }
                }
                if (ok && !mbar_wait(&acc_full[buf], acc_phase)) { if (lane == 0) atomicExch(error_flag, 14); ok = false; }
                ok = __all_sync(0xffffffffu, ok);
                if (reduce_out) ok = half_agrees(ok);
                if (!ok) continue;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (int cg = c_begin; cg < c_end; cg += AHEAD * 16) {
#pragma unroll
                    for (int c = 0; c < AHEAD; ++c) {
                        const int c0 = cg + c * 16;
                        if (c0 >= c_end) break;
                        float v[16];
                        tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), v);
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] += pre[c][j];
                        if (c0 + AHEAD * 16 < c_end) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) pre[c][j] = __ldcg(parked + (size_t)(c0 + AHEAD * 16 + j) * TC_BM);
                        }
                        finish_chunk(v, c0);
                    }
                }
            } else {
                // a warp whose wait gave up keeps walking the tiles (the barrier above counts on it) but touches nothing
                if (ok && !mbar_wait(&acc_full[buf], acc_phase)) { if (lane == 0) atomicExch(error_flag, 14); ok = false; }
                ok = __all_sync(0xffffffffu, ok);
                if ((!SK && heads.q_out != nullptr) || reduce_out) ok = half_agrees(ok);
                if (!ok) continue;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                for (int c0 = c_begin; c0 < c_end; c0 += 16) {
                    float v[16];
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0), v);
                    if (SK && is_tail) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) __stcg(parked + (size_t)(c0 + j) * TC_BM, v[j]);
                    } else {
                        finish_chunk(v, c0);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (is_tail) __threadfence();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&acc_empty[buf]);
                if (is_tail) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(parked_flag), "r"(1) : "memory");
                if (is_head) asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(parked_flag), "r"(0) : "memory");   // for the next launch
            }
        }
        // the reductions this thread handed to TMA are done before the kernel ends
        if (reduce_out && quarter == 0 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ----------------------------------------------------------------------------------------------

#ifndef TC_STAGES16
#define TC_STAGES16 6          // ring depth with up to 16 tokens per CTA
#endif

template <int BN, int STAGES>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int mode, int T, int N, int K, int splits,
                     int kb_per_split, float* partials, int* counters, int* error_flag, int cluster_reduce,
                     const TcNormOut& norm, const TcRowScale& scale, const TcHeadsOut& heads, cudaStream_t s) {
    constexpr int smem = STAGES * TcSmem<BN>::STAGE_BYTES + 1024 + 256;
    static_assert(STAGES * TcSmem<BN>::STAGE_BYTES >= BN * TC_BM * 4, "the cluster reduction reuses the pipeline buffers");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const bool clustered = cluster_reduce && splits > 1;
    return launch_kernel(gemm_tc_kernel<BN, STAGES>, dim3((N + TC_BM - 1) / TC_BM, (T + BN - 1) / BN, splits), dim3(128), smem, s,
                         clustered ? splits : 0, mw, mx, out, mode, T, N, K, kb_per_split, partials, counters, error_flag,
                         clustered ? 1 : 0, norm, scale, heads);
}

// Tiles a launch with `bn` tokens per CTA would have (for the caller's choice of split).
MB_API int mb_gemm_tc_tiles(int T, int N, int bn) { return ((N + TC_BM - 1) / TC_BM) * ((T + bn - 1) / bn); }

// MARIN_B200_TMA_REDUCE=0 in the environment: the "+=" epilogue of the persistent kernel reads and writes instead.
static bool tc_reduce_out() {
    static int state = -1;
    if (state < 0) {
        const char* v = getenv("MARIN_B200_TMA_REDUCE");
        state = (v != nullptr && v[0] == '0') ? 0 : 1;
    }
    return state == 1;
}

template <int BN, int STAGES, bool SK>
static int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int mode, int T, int N, int K, int ctas,
                             int* error_flag, const TcNormOut& norm, const TcRowScale& scale, TcStreamK sk, cudaStream_t s,
                             const TcHeadsOut& heads = TcHeadsOut{}, const float* rope = nullptr) {
    // "+=" into float32 with nothing riding on it: by TMA reduction, if the rows of out can be a tensor map's
    CUtensorMap mo = mw;
    int reduce_out = 0;
    if (mode == TC_OUT_F32_ACC && norm.weight == nullptr && tc_reduce_out() && N % 4 == 0 && ((uintptr_t)out & 15) == 0) {
        EncodeTiled enc = encode_tiled();
        cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)T};
        cuuint64_t strides[1] = {(cuuint64_t)N * 4};
        cuuint32_t box[2] = {TC_BM, 16};
        cuuint32_t elem[2] = {1, 1};
        if (enc != nullptr && enc(&mo, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, out, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
            reduce_out = 1;
    }
    constexpr int smem = STAGES * TcSmem<BN>::STAGE_BYTES + 1024 + 256;
    static_assert(smem <= 227 * 1024, "the ring does not fit shared memory");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, STAGES, SK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles_n = (N + TC_BM - 1) / TC_BM, tiles_t = (T + BN - 1) / BN, tiles = tiles_n * tiles_t;
    int grid = tiles < ctas ? tiles : ctas;
    if (SK) {
        // every group the same number of k-blocks; at least a tile's worth each, so that a tile has two owners at most
        const int groups = ctas / tiles_t;
        const long long units = (long long)tiles_n * ((K + TC_BK - 1) / TC_BK);
        sk.units_per_group = (int)((units + groups - 1) / groups);
        grid = groups * tiles_t;
    }
    return launch_kernel(gemm_tc_persistent_kernel<BN, STAGES, SK>, dim3(grid), dim3(320), smem, s, 0, mw, mx, out, mode, T, N, K,
                         error_flag, norm, scale, sk, heads, rope, mo, reduce_out);
}

static int persistent_dispatch(const void* x, const void* w, void* out, int mode, int T, int N, int K, int bn, int ctas,
                               int* error_flag, const TcNormOut& norm, const TcRowScale& scale, const TcStreamK& sk, cudaStream_t s,
                               const TcHeadsOut& heads = TcHeadsOut{}, const float* rope = nullptr) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ctas <= 0) return MB_ERR_BAD_SIZE;
    if (mode < 0 || mode > 3 || (mode == 3 && N % 32 != 0)) return MB_ERR_BAD_DTYPE;
    if (norm.weight != nullptr && (mode != TC_OUT_F32_ACC || norm.scaled == nullptr || norm.sumsq == nullptr)) return MB_ERR_BAD_DTYPE;
    if (scale.sumsq != nullptr && (scale.slots <= 0 || scale.dim <= 0)) return MB_ERR_BAD_SIZE;
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, N, K, TC_BM);
    if (rc) return rc;
    rc = make_map(&mx, x, T, K, bn);
    if (rc) return rc;
    if (sk.partials != nullptr) {
        switch (bn) {                                   // stream-K: three widths
            case 128: return launch_persistent<128, 6, true>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s);
            case 192: return launch_persistent<192, 5, true>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s);
            case 256: return launch_persistent<256, 4, true>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s);
            default: return MB_ERR_BAD_SIZE;
        }
    }
    switch (bn) {
        case 128: return launch_persistent<128, 6, false>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s, heads, rope);
        case 144: return launch_persistent<144, 6, false>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s, heads, rope);
        case 160: return launch_persistent<160, 5, false>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s, heads, rope);
        case 176: return launch_persistent<176, 5, false>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s, heads, rope);
        case 192: return launch_persistent<192, 5, false>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s, heads, rope);
        case 208: return launch_persistent<208, 4, false>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s, heads, rope);
        case 224: return launch_persistent<224, 4, false>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s, heads, rope);
        case 240: return launch_persistent<240, 4, false>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s, heads, rope);
        case 256: return launch_persistent<256, 4, false>(mw, mx, out, mode, T, N, K, ctas, error_flag, norm, scale, sk, s, heads, rope);
        default: return MB_ERR_BAD_SIZE;
    }
}

// The number of SMs of the device that is current, asked once per device.
static int sm_count_of_current_device() {
    static int known[64];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    if (known[device] == 0) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
        known[device] = sms;
    }
    return known[device];
}

// The persistent kernel: bn tokens per tile (a multiple of 16 from 128 to 256), `ctas` CTAs (one per SM).
MB_API int mb_gemm_tc_persistent(const void* x, const void* w, void* out, int mode, int T, int N, int K, int bn, int ctas,
                                 int* error_flag, cudaStream_t s) {
    return persistent_dispatch(x, w, out, mode, T, N, K, bn, ctas, error_flag, TcNormOut{}, TcRowScale{}, TcStreamK{}, s);
}

// The same with the k-blocks dealt out evenly (stream-K, see TcStreamK): no last round of tiles that fills a part of
// the SMs.  bn is 128, 192 or 256.  ctas must not exceed the SMs of the device (a CTA may wait for its neighbour's
// piece); there must be no more token tiles than CTAs and at least as many weight-row tiles as groups (ctas / token tiles).  partials:
// ctas * bn * 128 floats; flags: ctas * 8 ints, zero before the first call (the kernel leaves them at zero).  Two
// launches that share them must not overlap.
MB_API int mb_gemm_tc_persistent_streamk(const void* x, const void* w, void* out, int mode, int T, int N, int K, int bn, int ctas,
                                         float* partials, long long partials_floats, int* flags, int* error_flag, cudaStream_t s) {
    if (T <= 0 || N <= 0) return 0;
    if (partials == nullptr || flags == nullptr || bn <= 0 || ctas <= 0) return MB_ERR_BAD_SIZE;
    const int sms = sm_count_of_current_device();                  // a CTA may wait for its neighbour: all must be resident
    if (sms <= 0) return MB_ERR_BAD_SIZE;
    const int tiles_n = (N + TC_BM - 1) / TC_BM, tiles_t = (T + bn - 1) / bn;
    if (ctas > sms || tiles_t > ctas || tiles_n < ctas / tiles_t || partials_floats < (long long)ctas * bn * TC_BM) return MB_ERR_BAD_SIZE;
    return persistent_dispatch(x, w, out, mode, T, N, K, bn, ctas, error_flag, TcNormOut{}, TcRowScale{}, TcStreamK{partials, flags, 0}, s);
}

// The same coupled with the RMS norms around it (see mb_gemm_tc_coupled; the slots are mb_gemm_tc_norm_slots(N, 1)).
MB_API int mb_gemm_tc_persistent_coupled(const void* x, const void* w, void* out, int mode, int T, int N, int K, int bn, int ctas,
                                         const float* norm_weight, int norm_unit_offset, void* scaled_out, float* sumsq_out,
                                         const float* scale_sumsq, int scale_slots, int scale_dim, float scale_eps,
                                         int* error_flag, cudaStream_t s) {
    TcNormOut norm{norm_weight, (bf16*)scaled_out, sumsq_out, norm_unit_offset};
    TcRowScale scale{scale_sumsq, scale_slots, scale_dim, scale_eps};
    return persistent_dispatch(x, w, out, mode, T, N, K, bn, ctas, error_flag, norm, scale, TcStreamK{}, s);
}

// The q|k|v product of many tokens with heads of 128 elements, each head finished in the persistent kernel's epilogue
// (see TcHeadsOut; mb_gemm_tc_heads is the same for at most 16 tokens).  rope: [T][128] float32, cos of the 64 angles
// then sin (mb_rope_table), or null for no rotation.
MB_API int mb_gemm_tc_persistent_heads(const void* x, const void* w, int T, int N, int K, int bn, int ctas, void* q_out, void* k_cache,
                                       void* v_cache, const float* q_weight, const float* k_weight, float eps, const float* rope,
                                       const int* slot_mapping, int H, int KV, int page_size, int* error_flag, cudaStream_t s) {
    if (q_out == nullptr || H <= 0 || KV < 0 || (N != H * TC_BM && N != (H + 2 * KV) * TC_BM)) return MB_ERR_BAD_SIZE;
    if (N != H * TC_BM && (k_cache == nullptr || v_cache == nullptr || slot_mapping == nullptr || page_size <= 0)) return MB_ERR_BAD_SIZE;
    TcHeadsOut heads{(bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, q_weight, k_weight, nullptr, nullptr, slot_mapping, eps, H, KV, page_size};
    return persistent_dispatch(x, w, q_out, TC_OUT_BF16, T, N, K, bn, ctas, error_flag, TcNormOut{}, TcRowScale{}, TcStreamK{}, s, heads, rope);
}

// x [T, K] bf16, w [N, K] bf16, out [T, N]: bf16 (mode 0), float32 (1), float32 += (2).  K must be a multiple
// of 8 and both pointers 16-byte aligned (TMA).  splits > 1 needs partials (splits*T*N floats) and counters
// (one zeroed int per tile).  bn in {16, 32, 64, 128, 256}.
static int gemm_tc_dispatch(const void* x, const void* w, void* out, int mode, int T, int N, int K, int bn, int splits,
                            float* partials, int* counters, int* error_flag, int cluster_reduce, const TcNormOut& norm,
                            const TcRowScale& scale, const TcHeadsOut& heads, cudaStream_t s) {
    if (T <= 0 || N <= 0) return 0;
    // heads are finished only where the K slices of a tile meet as a cluster
    if (heads.q_out != nullptr && (!cluster_reduce || splits < 2 || N % TC_BM != 0 || bn > 128 || T > bn)) return MB_ERR_BAD_SIZE;
    // the norm's side outputs exist for "+=" without global split-K scratch
    if (norm.weight != nullptr && (mode != TC_OUT_F32_ACC || norm.scaled == nullptr || norm.sumsq == nullptr)) return MB_ERR_BAD_DTYPE;
    if (norm.weight != nullptr && !cluster_reduce && splits > 1) return MB_ERR_BAD_SIZE;
    if (scale.sumsq != nullptr && (scale.slots <= 0 || scale.dim <= 0 || (!cluster_reduce && splits > 1))) return MB_ERR_BAD_SIZE;
    if (K <= 0 || K % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return MB_ERR_BAD_SIZE;
    if (mode < 0 || mode > 3 || (mode == 3 && (splits > 1 || N % 32 != 0))) return MB_ERR_BAD_DTYPE;
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    if (splits < 1) splits = 1;
    if (splits > total_kb) splits = total_kb;
    int kb_per_split = (total_kb + splits - 1) / splits;
    if (cluster_reduce) {
        // the cluster is the K slices: 2, 4 or 8 of them, none empty
        if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return MB_ERR_BAD_SIZE;
        if ((splits - 1) * kb_per_split >= total_kb) return MB_ERR_BAD_SIZE;
    } else {
        splits = (total_kb + kb_per_split - 1) / kb_per_split;
        if (splits > 1 && (partials == nullptr || counters == nullptr)) return MB_ERR_BAD_SIZE;
    }
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, N, K, TC_BM);
    if (rc) return rc;
    rc = make_map(&mx, x, T, K, bn);
    if (rc) return rc;
    switch (bn) {
        case 16: return launch_tc<16, TC_STAGES16>(mw, mx, out, mode, T, N, K, splits, kb_per_split, partials, counters, error_flag, cluster_reduce, norm, scale, heads, s);
        case 32: return launch_tc<32, 4>(mw, mx, out, mode, T, N, K, splits, kb_per_split, partials, counters, error_flag, cluster_reduce, norm, scale, heads, s);
        case 64: return launch_tc<64, 4>(mw, mx, out, mode, T, N, K, splits, kb_per_split, partials, counters, error_flag, cluster_reduce, norm, scale, heads, s);
        case 128: return launch_tc<128, 3>(mw, mx, out, mode, T, N, K, splits, kb_per_split, partials, counters, error_flag, cluster_reduce, norm, scale, heads, s);
        case 256: return launch_tc<256, 4>(mw, mx, out, mode, T, N, K, splits, kb_per_split, partials, counters, error_flag, cluster_reduce, norm, scale, heads, s);
        default: return MB_ERR_BAD_SIZE;
    }
}

// x [T, K] bf16, w [N, K] bf16, out [T, N]: bf16 (mode 0), float32 (1), float32 += (2).  K must be a multiple
// of 8 and both pointers 16-byte aligned (TMA).  splits > 1 needs partials (splits*T*N floats) and counters
// (one zeroed int per tile).  bn in {16, 32, 64, 128, 256}.
MB_API int mb_gemm_tc(const void* x, const void* w, void* out, int mode, int T, int N, int K, int bn, int splits,
                      float* partials, int* counters, int* error_flag, cudaStream_t s) {
    return gemm_tc_dispatch(x, w, out, mode, T, N, K, bn, splits, partials, counters, error_flag, 0, TcNormOut{}, TcRowScale{}, TcHeadsOut{}, s);
}

// The same product with the K slices of a tile as one thread-block cluster (splits in {1, 2, 4, 8}): the slices
// are added through distributed shared memory, no global scratch is touched.
MB_API int mb_gemm_tc_cluster(const void* x, const void* w, void* out, int mode, int T, int N, int K, int bn, int splits,
                              int* error_flag, cudaStream_t s) {
    return gemm_tc_dispatch(x, w, out, mode, T, N, K, bn, splits, nullptr, nullptr, error_flag, 1, TcNormOut{}, TcRowScale{}, TcHeadsOut{}, s);
}

// Slots of sums of squares per token that a "+=" product over N weight rows with `splits` K slices writes.
MB_API int mb_gemm_tc_norm_slots(int N, int splits) { return ((N + TC_BM - 1) / TC_BM) * (splits < 4 ? 4 : splits); }

// mb_gemm_tc_cluster coupled with the RMS norms around it (either coupling may be absent: null pointers).
//   norm_weight [N] float32, scaled_out [T, N] bf16, sumsq_out [mb_gemm_tc_norm_slots(N, splits)][T] float32: with
//   mode 2, the updated rows times the norm weight (1 + weight with unit_offset) and their sums of squares.
//   scale_sumsq [scale_slots][T]: token t of the product is multiplied by 1 / sqrt(sum of its slots / scale_dim + eps).
MB_API int mb_gemm_tc_coupled(const void* x, const void* w, void* out, int mode, int T, int N, int K, int bn, int splits,
                              const float* norm_weight, int norm_unit_offset, void* scaled_out, float* sumsq_out,
                              const float* scale_sumsq, int scale_slots, int scale_dim, float scale_eps, int* error_flag,
                              cudaStream_t s) {
    TcNormOut norm{norm_weight, (bf16*)scaled_out, sumsq_out, norm_unit_offset};
    TcRowScale scale{scale_sumsq, scale_slots, scale_dim, scale_eps};
    return gemm_tc_dispatch(x, w, out, mode, T, N, K, bn, splits, nullptr, nullptr, error_flag, 1, norm, scale, TcHeadsOut{}, s);
}

// The q|k|v product of at most bn tokens (16, 32, 64 or 128) with heads of 128 elements, each head finished in the
// epilogue (see TcHeadsOut): w is [(H + 2 K) * 128, Kdim] (or [H * 128, Kdim]: queries only, when k_cache is null); splits >= 2.
// q_weight / k_weight null: no norm; inv_freq null: no rotation.  scale_*: as for mb_gemm_tc_coupled.
MB_API int mb_gemm_tc_heads(const void* x, const void* w, int T, int N, int K, int bn, int splits, void* q_out, void* k_cache, void* v_cache,
                            const float* q_weight, const float* k_weight, float eps, const int* positions, const float* inv_freq,
                            const int* slot_mapping, int H, int KV, int page_size, const float* scale_sumsq, int scale_slots,
                            int scale_dim, float scale_eps, int* error_flag, cudaStream_t s) {
    if (q_out == nullptr || H <= 0 || KV < 0 || (N != H * TC_BM && N != (H + 2 * KV) * TC_BM)) return MB_ERR_BAD_SIZE;
    if (N != H * TC_BM && (k_cache == nullptr || v_cache == nullptr || slot_mapping == nullptr || page_size <= 0)) return MB_ERR_BAD_SIZE;
    if (inv_freq != nullptr && positions == nullptr) return MB_ERR_BAD_SIZE;
    TcHeadsOut heads{(bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, q_weight, k_weight, positions, inv_freq, slot_mapping, eps, H, KV, page_size};
    TcRowScale scale{scale_sumsq, scale_slots, scale_dim, scale_eps};
    return gemm_tc_dispatch(x, w, nullptr, TC_OUT_BF16, T, N, K, bn, splits, nullptr, nullptr, error_flag, 1, TcNormOut{}, scale, heads, s);
}

// ---- the entry point that allocates nothing (see gemm_tc_noalloc.h) --------------------------------------------
#include <stdio.h>

#include "gemm_tc_noalloc.h"

// Split-K scratch for mb_gemm_tc_noalloc: partial tiles, then tile counters, then the error flag.  In host
// code this name is only a handle for the runtime; its device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char mb_noalloc_scratch[MB_NOALLOC_SCRATCH_BYTES];

#define MB_NOALLOC_MAX_DEVICES 64
// Per device, filled at its first call.  Nothing guards these: two threads that make a device's first call at the same
// time both write the same values, which is harmless, but the header asks callers to make that first call alone.
static unsigned char* noalloc_base[MB_NOALLOC_MAX_DEVICES];
static int noalloc_sms[MB_NOALLOC_MAX_DEVICES];
static thread_local char noalloc_message[256] = "";

static int noalloc_setup(unsigned char** base, int* sms = nullptr) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MB_NOALLOC_MAX_DEVICES) {
        snprintf(noalloc_message, sizeof noalloc_message, "device index %d is outside 0..%d", device, MB_NOALLOC_MAX_DEVICES - 1);
        return MB_ERR_NOALLOC_SETUP;
    }
    if (noalloc_base[device] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, mb_noalloc_scratch);       // the address on the device that is current now
        if (e != cudaSuccess || p == nullptr) {
            snprintf(noalloc_message, sizeof noalloc_message, "cudaGetSymbolAddress failed on device %d: %s", device,
                     cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : MB_ERR_NOALLOC_SETUP;
        }
        int count = 0;
        e = cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess || count <= 0) {
            snprintf(noalloc_message, sizeof noalloc_message, "the SM count of device %d could not be read: %s", device, cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : MB_ERR_NOALLOC_SETUP;
        }
        noalloc_sms[device] = count;
        noalloc_base[device] = (unsigned char*)p;
    }
    *base = noalloc_base[device];
    if (sms != nullptr) *sms = noalloc_sms[device];
    return 0;
}

MB_API const char* mb_gemm_tc_noalloc_last_error(void) { return noalloc_message; }

MB_API int mb_gemm_tc_noalloc_device_error(void) {
    unsigned char* base = nullptr;
    if (noalloc_setup(&base) != 0) return -1;
    int* flag = (int*)(base + (size_t)MB_NOALLOC_MAX_PARTIALS * 4 + (size_t)MB_NOALLOC_MAX_TILES * 4);
    // Wait for the whole device, not for the legacy default stream alone: a copy on that stream does not wait for
    // kernels on streams created as non-blocking, which is what most callers' streams are.
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    int value = 0;
    if (cudaMemcpy(&value, flag, sizeof value, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (value != 0 && cudaMemset(flag, 0, sizeof value) != cudaSuccess) return -1;   // the device is idle: nothing races with this
    return value;
}

MB_API int mb_gemm_tc_noalloc(const void* x, const void* w, void* out, int mode, int T, int N, int K, cudaStream_t stream) {
    noalloc_message[0] = 0;
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0) return MB_ERR_BAD_SIZE;
    unsigned char* base = nullptr;
    int sms = 0;
    int rc = noalloc_setup(&base, &sms);
    if (rc != 0) return rc;
    // A plan of this entry point's own (the Python wrapper plans for clusters of 2, 4 or 8 CTAs that reduce through
    // shared memory; here the slices reduce through the built-in scratch, so up to 16 are taken): tokens per CTA by
    // the number of tokens, then K slices while there are fewer tiles than SMs, about two CTAs per SM in all, each
    // slice at least four k-blocks long.
    const int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128;
    const long long tiles = (long long)((N + TC_BM - 1) / TC_BM) * ((T + bn - 1) / bn);
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    int splits = 1;
    if (tiles < sms) {
        splits = (int)(2 * sms / tiles);
        if (splits > total_kb / 4) splits = total_kb / 4;
        if (splits > 16) splits = 16;
        if (splits < 1) splits = 1;
    }
    if (splits > 1) {
        const long long need = (long long)splits * T * N;
        if (need > MB_NOALLOC_MAX_PARTIALS) {
            snprintf(noalloc_message, sizeof noalloc_message,
                     "T=%d N=%d K=%d needs %lld floats of split-K scratch (%d slices); the built-in scratch holds %d",
                     T, N, K, need, splits, MB_NOALLOC_MAX_PARTIALS);
            return MB_ERR_NOALLOC_TOO_LARGE;
        }
        if (tiles > MB_NOALLOC_MAX_TILES) {
            snprintf(noalloc_message, sizeof noalloc_message, "%lld tiles need counters; the built-in scratch holds %d",
                     tiles, MB_NOALLOC_MAX_TILES);
            return MB_ERR_NOALLOC_TOO_LARGE;
        }
    }
    float* partials = (float*)base;
    int* counters = (int*)(base + (size_t)MB_NOALLOC_MAX_PARTIALS * 4);
    int* error_flag = counters + MB_NOALLOC_MAX_TILES;
    if (splits > 1) {
        // the counters must start at zero; an earlier call that was cut short may have left them otherwise
        cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)tiles * sizeof(int), stream);
        if (e != cudaSuccess) return (int)e;
    }
    return mb_gemm_tc(x, w, out, mode, T, N, K, bn, splits, partials, counters, error_flag, stream);
}
