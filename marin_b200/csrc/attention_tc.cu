// Prefill attention on the 5th-generation tensor cores (tcgen05 / TMEM), compiled per head size (-DHEAD_DIM=64|128)
// and group size (-DGROUP).  A CTA takes 128 consecutive query tokens of one request and one query head and
// walks the keys in blocks of 64:
//   S = Q K^T      tcgen05.mma, M = 128 queries, N = 64 keys, K = HEAD_DIM; Q and K tiles in shared memory (TMA,
//                  128-byte swizzle, K-major); the accumulator S is 64 columns of tensor memory;
//   softmax        thread t owns query row t (TMEM lane t): it reads its 64 scores with tcgen05.ld, masks, keeps the
//                  running maximum and sum in float32 (exp2 domain) — no shuffles — and writes its row of P in bf16
//                  back into tensor memory, over the first half of its own scores (tcgen05.st);
//   PV             tcgen05.mma with P as the A operand straight from tensor memory, M = 128, N = HEAD_DIM, K = 64
//                  keys; V stays as it lies in the cache ([key][d], d
//                  contiguous), i.e. an MN-major B operand; the product accumulates in HEAD_DIM more TMEM columns.  The
//                  running maximum a row's O is scaled by is only raised when the true maximum has moved by more than
//                  8 (a factor 256, harmless in float32): then the row's O is read, rescaled and written back
//                  (tcgen05.ld/st); otherwise O is never touched until the end.
// K and V blocks arrive by TMA straight from the paged cache (one 16-key box per page piece and 64-column half) into
// two buffers each.  S (and with it P) has two buffers as well; the MMAs run in the order they are issued, so S of
// block i + 2 may follow P V of block i without a barrier.  Every barrier used once per block exists per buffer parity,
// since the rows may run a block ahead of the MMA warp.
// Eight warps: four own the 128 query rows (softmax, output), one issues S, one P V, one asks for keys and one for values.
// (A cycle-stamped timeline of one CTA showed that asking for a block of K or V, or issuing a block's MMAs, takes a
// warp 700 to 900 cycles each; one warp doing all four jobs set the pace of the kernel at 3,400 cycles a block, a warp
// for each brings it to 1,500, which is the rows' softmax: a -DTA_PROBE build counts where the rows and the issuers
// wait.  The rows read a block's 64 scores twice, each time with one load of 64 columns; keeping them in registers
// instead takes the thread to 128 registers with spills and is slower, and two threads per row, each with half of
// the keys, meet at a barrier every block and are slower too: 1,800 cycles.)
// Two CTAs fit an SM: one's softmax overlaps the other's MMAs.  Needs pages of at least 16 positions.  Waits are
// bounded and record a code in *error_flag.
// The mma.sync kernel in attention_fast.cu is the fallback and the plain twin (the reference's counterpart:
// crates/cuda/src/attention_mma.cu:43-180).
#define MB_LIB "attention_tc"
#define MB_LIB_ID 4
#include "tc_common.cuh"
#include "launch.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=64 or 128"
#endif
#ifndef GROUP
#error "compile with -DGROUP=<query heads per kv head>"
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "the tcgen05 attention kernel takes heads of 64 or 128");

#define D HEAD_DIM
#define NH (D / 64)                    // 64-column halves of a head: one 128-byte swizzle row each
#define TA_BM 128
#define TA_BN 64
#define TA_Q_BYTES (NH * TA_BM * 128)
#define TA_KV_BYTES (NH * TA_BN * 128)  // one of K or V, one buffer
#define TA_PAGE_CACHE 1024            // page ids of a tile's keys kept in shared memory (more are read from global memory)
#define TA_SMEM (TA_Q_BYTES + 4 * TA_KV_BYTES + 256)
#define TA_TMEM_COLS 256               // two S buffers of 64 columns, then O: HEAD_DIM columns
#define TA_O_COL (2 * TA_BN)

__device__ __forceinline__ float ta_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// MN-major B operand (V: rows are keys, 64 head columns contiguous per 128-byte swizzled row): 8-key groups 1024 bytes
// apart (stride offset), 64-column halves `half_bytes` apart (leading offset).
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t half_bytes) {
    const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | ((half_bytes >> 4) << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 64 columns of this thread's lane in one instruction and one wait (two loads of 32 cost two round trips to tensor
// memory, about 200 cycles each, that nothing in the thread can hide).
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float* v) {
    uint32_t r[64];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

// Waits for a phase; gives up at once if another thread of the CTA already gave up (`*abort`), and says so itself when
// its own time limit passes.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort, int* error_flag, int code) {
    const uint32_t addr = smem_u32(bar);
    const long long start = clock64();
    unsigned polls = 0;
    for (;;) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((++polls & 31) == 0) {
            if (*abort) return false;
            if (clock64() - start > TC_WAIT_LIMIT) { *abort = 1; atomicExch(error_flag, code); return false; }
        }
    }
}

// Has the phase with this parity completed?  Does not block.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

__device__ __forceinline__ void mbar_arrive_one(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// The MMA with its A operand in tensor memory (row m in lane m, two bf16 per 32-bit column) and B in shared memory.
__device__ __forceinline__ void umma_bf16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 256 threads: warps 0..3 own the 128 query rows (softmax, output); warp 4 issues S, warp 7 P V; warp 5 asks for keys, warp 6 for values.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st32_bits(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
          "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]),
          "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
          "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

#ifdef TA_PROBE
// Where the roles wait (a build for measuring only, -DTA_PROBE): per CTA (x + gridDim.x * y of request 0), clock ticks
// of [0] row 0 waiting for S, [1] row 0 waiting for O before a rescale, [2] row 0's loop in all, [3] the MMA thread
// finding nothing to issue, [4] the MMA thread's loop in all, [5] the key blocks.
__device__ long long ta_probe[4096 * 8];
MB_API int mb_attn_prefill_tc_probe_read(long long* host) { return (int)cudaMemcpyFromSymbol(host, ta_probe, sizeof(ta_probe)); }
#define TA_T() clock64()
#define TA_OUT(slot, v) do { const int cta_ = blockIdx.x + gridDim.x * blockIdx.y; if (blockIdx.z == 0 && cta_ < 4096) ta_probe[cta_ * 8 + (slot)] = (v); } while (0)
#else
#define TA_T() 0LL
#define TA_OUT(slot, v) do { (void)(v); } while (0)
#endif

__global__ void __launch_bounds__(256, 2) attn_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
    bf16* __restrict__ out, const int* __restrict__ block_table, int max_pages, const int* __restrict__ cu_tokens,
    const int* __restrict__ seq_lens, int first_req, int K, int page_shift, float scale, int window, int* __restrict__ error_flag,
    int box_rows) {
    extern __shared__ __align__(1024) uint8_t smem[];     // the swizzled tiles need 1024-byte alignment (checked below)
    uint8_t* sQ = smem;
    uint8_t* sKV = sQ + TA_Q_BYTES;                       // [buffer][K then V][half][64 rows][128 B]
    uint64_t* bars = (uint64_t*)(sKV + 4 * TA_KV_BYTES);
    uint64_t* q_full = bars;              // Q tile has landed
    uint64_t* k_full = bars + 1;          // [2] a block of K has landed
    uint64_t* v_full = bars + 3;          // [2] a block of V has landed
    uint64_t* v_free = bars + 5;          // [2] the P V product that read the V buffer is done
    uint64_t* s_done = bars + 7;          // [2] S = Q K^T is in its tensor-memory buffer (and its K buffer is free again)
    uint64_t* p_ready = bars + 9;         // [2] P is in tensor memory, over the first half of its S buffer (4 warps arrive)
    // Every barrier that is used once per key block exists twice, one per buffer parity: a waiter may be a block behind
    // or ahead of the other side, and a single barrier's phase parity would then be taken for the wrong block.
    // v_free[b] also tells the rows that O += P V of a block with parity b has been added.
    uint32_t* tmem_slot = (uint32_t*)(bars + 13);
    volatile int* abort = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    PDL_ENTER_EARLY();
    const int H = K * GROUP;
    const int r = first_req + blockIdx.z, h = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;   // long tiles first
    const int tok0 = cu_tokens[r], n = cu_tokens[r + 1] - tok0;
    if (qt * TA_BM >= n) return;                           // nothing to do here (before any tensor memory is taken)
    if ((smem_u32(smem) & 1023u) != 0) { if (threadIdx.x == 0) atomicExch(error_flag, 20); return; }
    const int len = seq_lens[r], pos0 = len - n;
    const int rows = min(TA_BM, n - qt * TA_BM);
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int b = 0; b < 2; ++b) { mbar_init(&k_full[b], 1); mbar_init(&v_full[b], 1); mbar_init(&v_free[b], 1); }
        for (int b = 0; b < 2; ++b) mbar_init(&s_done[b], 1);
        mbar_init(&p_ready[0], 4); mbar_init(&p_ready[1], 4);
        *abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TA_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    const int q_first = pos0 + qt * TA_BM, q_last = q_first + rows - 1;
    const int k_lo = window > 0 ? max(0, q_first - window + 1) : 0;
    const int kh = h / GROUP;
    const int kb_first = k_lo / TA_BN, kb_last = q_last / TA_BN;
    const int nblk = kb_last - kb_first + 1;
    // the page ids of this tile's keys, copied once: the issuer must not wait for global memory between two MMAs
    __shared__ int s_pages[TA_PAGE_CACHE];
    const int page_first = (kb_first * TA_BN) >> page_shift;
    {
        const int* table = block_table + (size_t)r * max_pages;
        const int count = min(TA_PAGE_CACHE, (((kb_last + 1) * TA_BN - 1) >> page_shift) - page_first + 1);
        for (int i = threadIdx.x; i < count; i += blockDim.x) s_pages[i] = table[min(page_first + i, max_pages - 1)];
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // The online softmax does not care about the order of the key blocks.  Every CTA starts at another block, so that
    // the many CTAs that read the same keys and values (the query tiles of a request, the heads of a group) do not
    // all ask the L2 for the same lines at the same moment.
    const int rot = (int)(((unsigned)(h * gridDim.x + qt) * 37u) % (unsigned)nblk);
    auto block_of = [&](int i) { const int j = i + rot; return kb_first + (j >= nblk ? j - nblk : j); };

    if (warp == 5 || warp == 6) {
        // ---- the loader warps: warp 5 asks for Q once and then for every block of K, warp 6 for every block of V, each
        // as soon as the block's buffer is free.  Lanes 0..3 each ask for one box of a block, so that one instruction
        // starts four TMA copies.  (Measured with cycle stamps: asking for a block takes a warp about 900 cycles, issuing
        // a block's MMAs about as long; one warp doing all of it set the pace of the whole kernel.) ----
        const bool keys = warp == 5;
        const int* table = block_table + (size_t)r * max_pages;
        const int page_mask = (1 << page_shift) - 1;
        const CUtensorMap* map = keys ? &map_k : &map_v;
        // One block of keys, or of values: 16-key boxes, one per page piece and 64-column half.  Where a block's boxes
        // lie in the cache is worked out one block ahead (row_of), while the warp waits for the buffer anyway: once
        // the buffer is free only the copies themselves remain to be started.
        const int g = lane * box_rows;                      // box_rows keys per box: 16, 32 or 64 (at most a page)
        auto row_of = [&](int j) {
            if (g >= TA_BN || j >= nblk) return 0;
            const int key = block_of(j) * TA_BN + g;
            const int pg = (key >> page_shift) - page_first;
            const int page_id = pg < TA_PAGE_CACHE ? s_pages[pg] : table[min(key >> page_shift, max_pages - 1)];
            return (int)((((size_t)page_id * K + kh) << page_shift) + (size_t)(key & page_mask));
        };
        auto load_block = [&](int j, int row) {
            uint8_t* dst = sKV + (size_t)(j & 1) * 2 * TA_KV_BYTES + (keys ? 0 : TA_KV_BYTES);
            uint64_t* bar = keys ? &k_full[j & 1] : &v_full[j & 1];
            if (lane == 0) mbar_expect_tx(bar, TA_KV_BYTES);
            __syncwarp();
            if (g < TA_BN) {
#pragma unroll
                for (int hf = 0; hf < NH; ++hf) tma_load_2d(dst + hf * (TA_BN * 128) + g * 128, map, hf * 64, row, bar);
            }
        };
        if (keys && lane == 0) {
            mbar_expect_tx(q_full, TA_Q_BYTES);
#pragma unroll
            for (int hf = 0; hf < NH; ++hf) tma_load_2d(sQ + hf * (TA_BM * 128), &map_q, h * D + hf * 64, tok0 + qt * TA_BM, q_full);
        }
        load_block(0, row_of(0));
        // the K buffer of block j is free once S of block j - 2 is done, the V buffer once P V of block j - 2 is
        uint64_t* freed = keys ? s_done : v_free;
        bool ok = true;
        unsigned idle = 0;
        const long long start = clock64();
        int row_next = row_of(1);
        for (int next = 1; ok && next < nblk;) {
            if (__shfl_sync(0xffffffffu, (int)(next < 2 || mbar_test(&freed[next & 1], ((next - 2) >> 1) & 1)), 0)) {
                load_block(next, row_next);
                ++next;
                row_next = row_of(next);
            } else if ((++idle & 63) == 0) {
                if (*abort) ok = false;
                else if (clock64() - start > 8 * TC_WAIT_LIMIT) { *abort = 1; atomicExch(error_flag, 28); ok = false; }
                ok = __all_sync(0xffffffffu, ok);
            }
        }
    } else if (warp == 4) {
        // ---- the issuer of S: one lane issues S(i) = Q K(i)^T as soon as the block's keys have landed and P V of block
        // i - 2 is done (S(i) goes where P(i - 2) lies).  Issuing an MMA costs the thread over a hundred cycles, and a
        // block has twelve: one thread for all of them set the kernel's pace (1,600 of a block's 1,620 cycles busy), so
        // S and P V have an issuer each. ----
        if (lane == 0) {
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TA_BN >> 3) << 17) | ((uint32_t)(TA_BM >> 4) << 24);
            const uint32_t sq = smem_u32(sQ);
            uint64_t qdesc[D / 16], kdesc[2][D / 16];
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                qdesc[kk] = umma_desc(sq + (kk / 4) * (TA_BM * 128)) + 2 * (kk % 4);
#pragma unroll
                for (int b = 0; b < 2; ++b)
                    kdesc[b][kk] = umma_desc(smem_u32(sKV + (size_t)b * 2 * TA_KV_BYTES) + (kk / 4) * (TA_BN * 128)) + 2 * (kk % 4);
            }
            bool ok = wait_or_abort(q_full, 0, abort, error_flag, 21);
            const long long start = TA_T();
            long long m_idle = 0;
            for (int i = 0; ok && i < nblk; ++i) {
                const long long m_t0 = TA_T();
                ok = wait_or_abort(&k_full[i & 1], (i >> 1) & 1, abort, error_flag, 29);
                if (ok && i >= 2) ok = wait_or_abort(&v_free[i & 1], ((i - 2) >> 1) & 1, abort, error_flag, 29);
                m_idle += TA_T() - m_t0;
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (i & 1) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) umma_bf16(tmem_base + (uint32_t)TA_BN, qdesc[kk], kdesc[1][kk], idesc_s, kk > 0 ? 1u : 0u);
                } else {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) umma_bf16(tmem_base, qdesc[kk], kdesc[0][kk], idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_done[i & 1]);
            }
            TA_OUT(3, m_idle); TA_OUT(4, TA_T() - start); TA_OUT(5, (long long)nblk);
        }
    } else if (warp == 7) {
        // ---- the issuer of P V: O += P(i) V(i) once the rows have put P(i) into tensor memory and the values have landed
        // (any rescaling of O by the rows happened before they arrived) ----
        if (lane == 0) {
            constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(TA_BM >> 4) << 24);
            uint64_t vdesc[2][TA_BN / 16];
#pragma unroll
            for (int kk = 0; kk < TA_BN / 16; ++kk)
#pragma unroll
                for (int b = 0; b < 2; ++b)
                    vdesc[b][kk] = umma_desc_mn(smem_u32(sKV + (size_t)b * 2 * TA_KV_BYTES) + TA_KV_BYTES + kk * 2048, TA_BN * 128);
            bool ok = true;
            const long long start = TA_T();
            long long m_idle = 0;
            for (int i = 0; ok && i < nblk; ++i) {
                const int buf = i & 1;
                const long long m_t0 = TA_T();
                ok = wait_or_abort(&p_ready[buf], (i >> 1) & 1, abort, error_flag, 29);
                if (ok) ok = wait_or_abort(&v_full[buf], (i >> 1) & 1, abort, error_flag, 29);
                m_idle += TA_T() - m_t0;
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // P is the A operand straight from tensor memory: row = lane, two bf16 per 32-bit column
                const uint32_t tp = tmem_base + (uint32_t)(buf * TA_BN);
                if (buf) {
#pragma unroll
                    for (int kk = 0; kk < TA_BN / 16; ++kk)
                        umma_bf16_tmem_a(tmem_base + TA_O_COL, tp + (uint32_t)(kk * 8), vdesc[1][kk], idesc_pv, (i > 0 || kk > 0) ? 1u : 0u);
                } else {
#pragma unroll
                    for (int kk = 0; kk < TA_BN / 16; ++kk)
                        umma_bf16_tmem_a(tmem_base + TA_O_COL, tp + (uint32_t)(kk * 8), vdesc[0][kk], idesc_pv, (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&v_free[buf]);
            }
            TA_OUT(6, m_idle); TA_OUT(7, TA_T() - start);
        }
    } else {
        // ---- the rows: thread t owns query row t ----
        const int row_t = threadIdx.x;
        const int qp = q_first + row_t;
        const int lo_t = window > 0 ? max(0, qp - window + 1) : 0;
        const float sl2 = scale * 1.4426950408889634f;
        const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
        float m_used = -INFINITY, l_run = 0.0f;           // the maximum O and l are currently scaled by (log2 units)
        bool ok = true;
        long long r_s = 0, r_o = 0;
        const long long r_start = TA_T();
        for (int i = 0; i < nblk; ++i) {
            const int key0 = block_of(i) * TA_BN;
            const uint32_t s_col = lane_base + (uint32_t)((i & 1) * TA_BN);
            const long long r_t0 = TA_T();
            ok = ok && wait_or_abort(&s_done[i & 1], (i >> 1) & 1, abort, error_flag, 23);
            r_s += TA_T() - r_t0;
            ok = __all_sync(0xffffffffu, ok);              // tcgen05.ld is warp-wide: the warp takes one path
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // two passes over the 64 scores, 32 at a time (tensor memory is cheap to read twice; registers are not):
            // the row maximum first, then the probabilities
            const bool interior = key0 + TA_BN - 1 <= q_first && (window <= 0 || key0 >= q_last - window + 1);
            float mx = -INFINITY;
            {
                float s[64];
                tmem_ld64(s_col, s);
                if (!interior) {
#pragma unroll
                    for (int j = 0; j < 64; ++j)
                        if (!(key0 + j <= qp && key0 + j >= lo_t)) s[j] = -INFINITY;
                }
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 64; j += 4) {
                    m4[0] = fmaxf(m4[0], s[j]); m4[1] = fmaxf(m4[1], s[j + 1]); m4[2] = fmaxf(m4[2], s[j + 2]); m4[3] = fmaxf(m4[3], s[j + 3]);
                }
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            }
            // raise the scaling maximum only when the true one has moved by more than 8 (or from -inf)
            const float m_true = fmaxf(m_used, mx * sl2);
            const bool raise = m_true > m_used + 8.0f || (m_used == -INFINITY && m_true != -INFINITY);
            const float m_new = raise ? m_true : m_used;
            const float corr = raise ? ta_exp2(m_used - m_new) : 1.0f;      // exp2(-inf) = 0 on the first raise
            if (__any_sync(0xffffffffu, raise) && i >= 1) {
                // O is being added to by the MMAs of block i - 1 until they are done (blocks up to i - 2 are: S(i) came after them)
                const long long r_t1 = TA_T();
                ok = wait_or_abort(&v_free[(i - 1) & 1], ((i - 1) >> 1) & 1, abort, error_flag, 24);
                r_o += TA_T() - r_t1;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    float ov[32];
                    tmem_ld32(lane_base + TA_O_COL + c * 32, ov);
#pragma unroll
                    for (int j = 0; j < 32; ++j) ov[j] *= corr;
                    tmem_st32(lane_base + TA_O_COL + c * 32, ov);
                }
            }
            m_used = m_new;
            const float base = m_used == -INFINITY ? 0.0f : m_used;
            float sum = 0.0f;
            uint4 packed[TA_BN / 8];                           // the row of P, kept until the last block's P has been consumed
            {
                float s[64];
                tmem_ld64(s_col, s);
                if (!interior) {
#pragma unroll
                    for (int j = 0; j < 64; ++j)
                        if (!(key0 + j <= qp && key0 + j >= lo_t)) s[j] = -INFINITY;
                }
                float sum2[2] = {0.0f, 0.0f};
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    float p[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) { p[e] = ta_exp2(fmaf(s[c * 8 + e], sl2, -base)); sum2[e & 1] += p[e]; }
                    __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&packed[c]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) p2[e] = __floats2bfloat162_rn(p[2 * e], p[2 * e + 1]);
                }
                sum = sum2[0] + sum2[1];
            }
            l_run = l_run * corr + sum;
            // the row of P goes over the first 32 columns of its own scores (all 64 are in registers by now)
            tmem_st32_bits(s_col, reinterpret_cast<const uint32_t*>(packed));
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_one(&p_ready[i & 1]);
        }
        if (threadIdx.x == 0) { TA_OUT(0, r_s); TA_OUT(1, r_o); TA_OUT(2, TA_T() - r_start); }
        if (ok) {
            ok = wait_or_abort(&v_free[(nblk - 1) & 1], ((nblk - 1) >> 1) & 1, abort, error_flag, 24);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = 1.0f / l_run;
            bf16* dst = out + ((size_t)(tok0 + qt * TA_BM + row_t) * H + h) * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                float ov[32];
                tmem_ld32(lane_base + TA_O_COL + c * 32, ov);
                if (row_t < rows) {
#pragma unroll
                    for (int q8 = 0; q8 < 4; ++q8) {
                        uint4 packed;
                        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                        for (int e = 0; e < 4; ++e) p2[e] = __floats2bfloat162_rn(ov[q8 * 8 + 2 * e] * inv, ov[q8 * 8 + 2 * e + 1] * inv);
                        reinterpret_cast<uint4*>(dst)[c * 4 + q8] = packed;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TA_TMEM_COLS) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
static int map_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiled enc = encode_tiled();
    if (enc == nullptr) return MB_ERR_BAD_SIZE;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS ? 0 : 1000 + (int)rc;
}

// Prefill attention of requests first_req .. first_req+requests-1 (tokens cu_tokens[r]..cu_tokens[r+1], all `tokens`
// rows of q and out belong to the step); cache_pages pages of page_size (>= 16) positions.
MB_API int mb_attn_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                              int max_pages, const int* cu_tokens, const int* seq_lens, int first_req, int requests,
                              int max_query_len, int tokens, int K, int page_size, long long cache_pages, float scale,
                              int window, int* error_flag, cudaStream_t s) {
    if (requests <= 0 || max_query_len <= 0) return 0;
    int page_shift = -1;
    for (int b = 4; b < 16; ++b)
        if ((1 << b) == page_size) page_shift = b;
    if (page_shift < 0) return MB_ERR_BAD_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return MB_ERR_BAD_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    CUtensorMap mq, mk, mv;
    int rc = map_2d(&mq, q, (uint64_t)tokens, (uint64_t)K * GROUP * D, TA_BM);
    if (rc) return rc;
    const uint64_t cache_rows = (uint64_t)cache_pages * K * page_size;
    const int box_rows = page_size < TA_BN ? page_size : TA_BN;
    rc = map_2d(&mk, k_cache, cache_rows, D, box_rows);
    if (rc) return rc;
    rc = map_2d(&mv, v_cache, cache_rows, D, box_rows);
    if (rc) return rc;
    dim3 grid((max_query_len + TA_BM - 1) / TA_BM, K * GROUP, requests);
    return launch_kernel(attn_prefill_tc_kernel, grid, 256, TA_SMEM, s, 0, mq, mk, mv, (bf16*)out, block_table, max_pages, cu_tokens,
                         seq_lens, first_req, K, page_shift, scale, window, error_flag, box_rows);
}
