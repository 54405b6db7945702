// Sampling on the device.  arg-max: the largest logit among the first `usable`, the lowest id among
// equals (the reference's greedy rule, crates/sampler/src/lib.rs:40-48).  A row is shared by several blocks; each
// folds its best (value, id) into one 64-bit key per row with atomicMax, and the block that arrives last writes
// the id and clears the row's key and counter for the next launch.
//
// A logit that is NaN or infinite among the usable ones is an error, as in the reference (crates/sampler/src/lib.rs:
// 135-137): both kernels write the id -1 for such a row.  report[0] receives the code another kernel left in
// `error_flag` when one of its bounded waits gave up (untouched otherwise), so that the host learns of both with the
// ids it reads anyway; the host clears it after it has seen a non-zero value.
//
// arg-max can leave its ids in two more places (ArgmaxAlso).  `feed`: where the NEXT step reads its token ids, so that a
// step launched before the host has seen these ids is fed on the device.  `mirror`: memory of the host that the device
// can write (pinned): row *which of [rows of `mirror_stride` ints] receives the error code, three zeros and the ids,
// and the host reads them there once an event behind the kernel has completed, with no copy of its own in the
// stream.  Two rows in turn (the host says which, in device memory, before each step): the step that runs must not
// overwrite what the host still reads of the step before.
#define MB_LIB "sampling"
#define MB_LIB_ID 5
#include "common.cuh"
#include "launch.cuh"
#include <limits.h>

#define AM_THREADS 512

__device__ __forceinline__ bool not_finite(float x) { return !(fabsf(x) <= 3.402823466e+38f); }

#define AM_BAD_ROW 0xffffffffffffffffull      // no key of a value that can win looks like this (its high word would be a NaN's)

// Larger value first, then lower id: the value's bits made monotonic in the high word, the inverted id in the low.
__device__ __forceinline__ unsigned long long am_key(float v, int idx) {
    v += 0.0f;                                               // -0 and +0 are equal: one key for both
    unsigned int b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (unsigned long long)(0xffffffffu - (unsigned int)idx);
}

struct ArgmaxAlso {
    int* feed;                 // [rows] or null
    int* mirror;               // host memory the device can write, [2][mirror_stride], or null
    int mirror_stride;
    const int* which;          // device int: 0 or 1, the mirror's row for this launch
    int row0;                  // first row of this launch among the caller's rows
};

// keys, count: one entry per row of this launch, zero between launches (the caller's scratch memory).
__global__ void __launch_bounds__(AM_THREADS) argmax_kernel(const float* __restrict__ logits, int vocab, int usable,
                                                            int per_block, int* __restrict__ out, unsigned long long* keys,
                                                            int* count, int* report, const int* error_flag, const ArgmaxAlso also) {
    PDL_ENTER();
    logits = pdl_fresh(logits);
    __shared__ float best_v[AM_THREADS / 32];
    __shared__ int best_i[AM_THREADS / 32];
    const int r = blockIdx.y;
    const float* row = logits + (size_t)r * vocab;
    const int begin = blockIdx.x * per_block, end = min(usable, begin + per_block);
    float v = -INFINITY;
    int idx = 0x7fffffff;
    bool bad = false;
    for (int i = begin + threadIdx.x; i < end; i += AM_THREADS) {
        const float x = row[i];
        bad |= not_finite(x);
        if (x > v || (x == v && i < idx)) { v = x; idx = i; }
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicMax(&keys[r], AM_BAD_ROW);
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && report != nullptr && error_flag != nullptr) {
        const int code = *(const volatile int*)error_flag;   // every earlier kernel of the stream has ended
        if (code != 0) report[0] = code;
        if (also.mirror != nullptr && also.row0 == 0) {
            int* head = also.mirror + (size_t)(*also.which & 1) * also.mirror_stride;
            head[0] = code != 0 ? code : report[0];
            head[1] = head[2] = head[3] = 0;
        }
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
        if (lane == 0) {
            if (idx != 0x7fffffff) atomicMax(&keys[r], am_key(v, idx));
            __threadfence();
            if (atomicAdd(&count[r], 1) == (int)gridDim.x - 1) {
                __threadfence();
                const unsigned long long key = atomicExch(&keys[r], 0ull);
                count[r] = 0;
                const int id = key == AM_BAD_ROW ? -1 : key == 0ull ? 0 : (int)(0xffffffffu - (unsigned int)(key & 0xffffffffull));
                out[r] = id;
                if (also.feed != nullptr) also.feed[also.row0 + r] = id < 0 ? 0 : id;
                if (also.mirror != nullptr) also.mirror[(size_t)(*also.which & 1) * also.mirror_stride + 4 + also.row0 + r] = id;
            }
        }
    }
}

// keys/count hold `key_rows` entries; `blocks_wanted` is about how many blocks the launch should have in all (the
// caller knows the device: two per SM).  report and error_flag may be null.
MB_API int mb_argmax(const float* logits, int rows, int vocab, int usable, int* out, unsigned long long* keys, int* count,
                     int key_rows, int blocks_wanted, int* report, const int* error_flag, int* feed, int* mirror, int mirror_stride,
                     const int* mirror_which, cudaStream_t s) {
    if (rows <= 0) return 0;
    if (usable <= 0 || usable > vocab || key_rows <= 0 || keys == nullptr || count == nullptr) return MB_ERR_BAD_SIZE;
    if (mirror != nullptr && (mirror_which == nullptr || report == nullptr || error_flag == nullptr || mirror_stride < 4 + rows)) return MB_ERR_BAD_SIZE;
    if (blocks_wanted <= 0) blocks_wanted = 1;
    for (int r0 = 0; r0 < rows; r0 += key_rows) {
        const int n = rows - r0 < key_rows ? rows - r0 : key_rows;
        int blocks = (blocks_wanted + n - 1) / n;
        const int most = (usable + 4 * AM_THREADS - 1) / (4 * AM_THREADS);  // at least four values per thread
        if (blocks > most) blocks = most;
        const int per_block = (usable + blocks - 1) / blocks;
        blocks = (usable + per_block - 1) / per_block;
        const int rc = launch_kernel(argmax_kernel, dim3(blocks, n), AM_THREADS, 0, s, 0, logits + (size_t)r0 * vocab, vocab, usable,
                                     per_block, out + r0, keys, count, report, error_flag, ArgmaxAlso{feed, mirror, mirror_stride, mirror_which, r0});
        if (rc) return rc;
    }
    return 0;
}

// ---- temperature / top-k / top-p sampling on the device ---------------------------------------------------------------
// One block per row.  The kept set is the reference's (crates/sampler/src/lib.rs:122-193): tokens ranked by (logit
// descending, id ascending), the best top_k of them (0 = all), weights exp((l - max) / temperature), then the
// shortest prefix of that ranking whose share of the weight reaches top_p.  Ranking is never materialised: the
// k-th largest logit and the logit at which the nucleus closes are found by bisection on the logits' bit patterns
// (which order like the values), and ties at either threshold are kept in id order, as many as the rule admits.
// A token is then drawn from the kept set with probability proportional to its weight by walking the ids in
// increasing order until the running weight passes u * total, u in [0, 1) coming from the request's own
// splitmix64 stream on the host.  (The reference walks in rank order: the distribution is the same, the token a
// given u selects is not.)  temperature 0 picks the largest logit, the lowest id among equals.
#define SP_THREADS 1024

__device__ __forceinline__ int order_key(float v) {           // monotone map float -> int (IEEE total order)
    const int b = __float_as_int(v);
    return b ^ ((b >> 31) & 0x7fffffff);
}

// Sum over the block, the same tree whatever the data; every thread gets the result.
__device__ __forceinline__ float sp_block_sum(float v, float* scratch) { return block_sum(v, scratch); }

__device__ __forceinline__ int sp_block_sum_int(int v, int* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    int total = lane < SP_THREADS / 32 ? scratch[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    return total;
}

// Exclusive prefix of v over the block (thread order), and the block total.
__device__ __forceinline__ float sp_block_scan(float v, float* scratch, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float n = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += n; }
    __syncthreads();
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    float w = lane < SP_THREADS / 32 ? scratch[lane] : 0.0f;
    float winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float n = __shfl_up_sync(0xffffffffu, winc, o); if (lane >= o) winc += n; }
    const float before = __shfl_sync(0xffffffffu, winc - w, warp);
    *total = __shfl_sync(0xffffffffu, winc, 31);
    return before + inc - v;
}

__global__ void __launch_bounds__(SP_THREADS) sample_kernel(const float* __restrict__ logits, int vocab, const int* __restrict__ usable_of,
                                                            const float* __restrict__ temperature, const int* __restrict__ top_k,
                                                            const float* __restrict__ top_p, const float* __restrict__ uniform,
                                                            int* __restrict__ out, int* report, const int* error_flag) {
    PDL_ENTER();
    logits = pdl_fresh(logits);
    __shared__ float fs[32];
    __shared__ int is[32];
    __shared__ int s_found;
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int n = usable_of[blockIdx.x];
    const float temp = temperature[blockIdx.x];
    int k = top_k[blockIdx.x];
    float p = top_p[blockIdx.x];
    if (temp == 0.0f) { k = 1; p = 1.0f; }
    const float inv_t = temp == 0.0f ? 1.0f : 1.0f / temp;

    // the largest logit; a row with a value that is not finite gets the id -1
    float m = -INFINITY;
    bool bad = false;
    for (int i = threadIdx.x; i < n; i += SP_THREADS) {
        const float x = row[i];
        bad |= not_finite(x);
        m = fmaxf(m, x);
    }
    m = block_max(m, fs);
    if (blockIdx.x == 0 && threadIdx.x == 0 && report != nullptr && error_flag != nullptr) {
        const int code = *(const volatile int*)error_flag;
        if (code != 0) report[0] = code;
    }
    if (__syncthreads_or(bad)) {
        if (threadIdx.x == 0) out[blockIdx.x] = -1;
        return;
    }

    // top-k: the k-th largest key, how many lie above it, how many of its ties are kept
    int tk = INT_MIN, ties_k = INT_MAX;                       // keep key > tk, and the first ties_k ids with key == tk
    if (k > 0 && k < n) {
        long long lo = INT_MIN, hi = order_key(m);            // largest t with count(key >= t) >= k
        while (lo < hi) {
            const long long mid = lo + (hi - lo + 1) / 2;
            int c = 0;
            for (int i = threadIdx.x; i < n; i += SP_THREADS) c += order_key(row[i]) >= (int)mid;
            c = sp_block_sum_int(c, is);
            if (c >= k) lo = mid; else hi = mid - 1;
        }
        tk = (int)lo;
        int above = 0;
        for (int i = threadIdx.x; i < n; i += SP_THREADS) above += order_key(row[i]) > tk;
        above = sp_block_sum_int(above, is);
        ties_k = k - above;
    }
    // membership in the top-k set needs the rank of a tie among the ties, in id order: the ordered walks below carry
    // a running count of ties seen so far.

    // total weight of the top-k set
    float z = 0.0f;
    {
        int seen = 0;
        for (int base = 0; base < n; base += SP_THREADS) {
            const int i = base + threadIdx.x;
            const int key = i < n ? order_key(row[i]) : INT_MIN;
            const int tie = i < n && key == tk && ties_k != INT_MAX;
            float tot;
            const int rank = seen + (int)sp_block_scan((float)tie, fs, &tot);
            seen += (int)tot;
            const bool member = i < n && (key > tk || (tie && rank < ties_k) || (ties_k == INT_MAX));
            z += member ? expf((row[i] - m) * inv_t) : 0.0f;
        }
        z = sp_block_sum(z, fs);
    }

    // top-p: the key at which the ranked prefix reaches p * z, and how many of its ties are kept
    int tp = INT_MIN, ties_p = INT_MAX;
    if (p < 1.0f) {
        const float need = p * z;
        long long lo = tk == INT_MIN ? (long long)INT_MIN : (long long)tk, hi = order_key(m);   // largest t with mass(key >= t) >= need
        while (lo < hi) {
            const long long mid = lo + (hi - lo + 1) / 2;
            float mass = 0.0f;
            for (int i = threadIdx.x; i < n; i += SP_THREADS) {
                const int key = order_key(row[i]);
                mass += key >= (int)mid ? expf((row[i] - m) * inv_t) : 0.0f;        // above tk every token is a member
            }
            mass = sp_block_sum(mass, fs);
            if (mass >= need) lo = mid; else hi = mid - 1;
        }
        tp = (int)lo;
        if (tp > tk) {
            float above = 0.0f;
            int ties = 0;
            float w_tie = 0.0f;
            for (int i = threadIdx.x; i < n; i += SP_THREADS) {
                const int key = order_key(row[i]);
                if (key > tp) above += expf((row[i] - m) * inv_t);
                else if (key == tp) { ties += 1; w_tie = expf((row[i] - m) * inv_t); }
            }
            above = sp_block_sum(above, fs);
            ties = sp_block_sum_int(ties, is);
            w_tie = block_max(w_tie, fs);
            int keep = (int)ceilf((need - above) / w_tie);
            ties_p = min(max(keep, 1), ties);
        } else {
            tp = INT_MIN;                                      // the nucleus takes the whole top-k set
        }
    }

    // the final set: key > T, plus the first `ties` ids with key == T, where (T, ties) is the tighter of the two rules
    int T = tk, ties = ties_k;
    if (tp != INT_MIN) { T = tp; ties = ties_p; }
    const bool all = T == INT_MIN && ties == INT_MAX;
    float zk = 0.0f;
    {
        int seen = 0;
        for (int base = 0; base < n; base += SP_THREADS) {
            const int i = base + threadIdx.x;
            const int key = i < n ? order_key(row[i]) : INT_MIN;
            const int tie = !all && i < n && key == T;
            float tot;
            const int rank = seen + (int)sp_block_scan((float)tie, fs, &tot);
            seen += (int)tot;
            const bool member = i < n && (all || key > T || (tie && rank < ties));
            zk += member ? expf((row[i] - m) * inv_t) : 0.0f;
        }
        zk = sp_block_sum(zk, fs);
    }
    const float target = uniform[blockIdx.x] * zk;
    if (threadIdx.x == 0) s_found = INT_MAX;
    __syncthreads();
    float run = 0.0f;
    int seen = 0, last_member = -1;
    for (int base = 0; base < n; base += SP_THREADS) {
        const int i = base + threadIdx.x;
        const int key = i < n ? order_key(row[i]) : INT_MIN;
        const int tie = !all && i < n && key == T;
        float tot;
        const int rank = seen + (int)sp_block_scan((float)tie, fs, &tot);
        seen += (int)tot;
        const bool member = i < n && (all || key > T || (tie && rank < ties));
        const float w = member ? expf((row[i] - m) * inv_t) : 0.0f;
        float wtot;
        const float before = run + sp_block_scan(w, fs, &wtot);
        if (member && before <= target && target < before + w) atomicMin(&s_found, i);   // at most one thread; min for safety
        if (member) last_member = i;
        run += wtot;
        __syncthreads();
        if (s_found != INT_MAX) break;
    }
    // rounding may leave target at or past the total: the last member then
    int lm = last_member;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lm = max(lm, __shfl_xor_sync(0xffffffffu, lm, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) is[threadIdx.x >> 5] = lm;
    __syncthreads();
    if (threadIdx.x == 0) {
        int best = -1;
        for (int w = 0; w < SP_THREADS / 32; ++w) best = max(best, is[w]);
        out[blockIdx.x] = s_found != INT_MAX ? s_found : max(best, 0);
    }
}

MB_API int mb_sample(const float* logits, int rows, int vocab, const int* usable, const float* temperature, const int* top_k,
                     const float* top_p, const float* uniform, int* out, int* report, const int* error_flag, cudaStream_t s) {
    if (rows <= 0) return 0;
    return launch_kernel(sample_kernel, rows, SP_THREADS, 0, s, 0, logits, vocab, usable, temperature, top_k, top_p, uniform, out,
                         report, error_flag);
}
