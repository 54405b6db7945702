// Host side of the cache manager, in C++: page pools, per-request block tables and state slots, and the packing
// of a step's requests into the one int32 buffer the kernels read.  No device memory is touched here; the Python
// classes in marin_b200/cache keep the tensors and call in through the C functions at the end of this file.
//
// Layers whose mixers need the same thing of the cache form a group with a pool of its own; a request holds one
// block table per group.  Pages go back to their pool when the request ends or when a group's window has passed
// them, and are handed out again, last freed first.  (The reference keeps one private LIFO pool per sequence:
// crates/cuda/src/pages.rs:20-65, crates/cuda/src/kv.rs:214-270; the shared pool is this engine's own design.)
#include "cache_core.h"

using namespace mbh;

namespace {

void put_message(const std::string& why, char* msg, int cap) {
    if (msg != nullptr && cap > 0) {
        std::snprintf(msg, (size_t)cap, "%s", why.c_str());
    }
}

}  // namespace

// ---- a pool alone (the Python PagePool and SlotPool) ----------------------------------------------------------------
MBH_API void* mbh_pool_create(int n) { return n > 0 ? new PagePool(n) : nullptr; }
MBH_API void mbh_pool_destroy(void* p) { delete static_cast<PagePool*>(p); }
MBH_API int mbh_pool_num_free(void* p) { return static_cast<PagePool*>(p)->num_free(); }
MBH_API int mbh_pool_num_held(void* p) { return static_cast<PagePool*>(p)->num_held(); }
MBH_API int mbh_pool_alloc(void* p, int count, int* out) {
    std::vector<int> got;
    const int rc = static_cast<PagePool*>(p)->alloc(count, &got);
    if (rc == MBH_OK) std::copy(got.begin(), got.end(), out);
    return rc;
}
MBH_API int mbh_pool_free(void* p, int page) { return static_cast<PagePool*>(p)->free_page(page); }
MBH_API int mbh_pool_check(void* p, char* msg, int cap) {
    std::string why;
    const int rc = static_cast<PagePool*>(p)->check(&why);
    put_message(why, msg, cap);
    return rc;
}

// ---- the cache manager ----------------------------------------------------------------------------------------------
// windows[g] < 0: group g keeps all keys.
MBH_API void* mbh_cache_create(int page_size, int num_pages, int max_requests, int n_groups, const int* windows) {
    if (page_size <= 0 || num_pages <= 0 || max_requests <= 0 || n_groups < 0) return nullptr;
    return new Cache(page_size, num_pages, max_requests, n_groups, windows);
}
MBH_API void mbh_cache_destroy(void* c) { delete static_cast<Cache*>(c); }
MBH_API int mbh_admit(void* c, int64_t* handle, int* slot) { return static_cast<Cache*>(c)->admit(handle, slot); }
MBH_API int mbh_length(void* c, int64_t h) {
    Request* r = static_cast<Cache*>(c)->find(h);
    return r == nullptr ? -1 : r->length;
}
MBH_API int mbh_pages_missing(void* c, int64_t h, int new_len, int* out) {
    Cache* cache = static_cast<Cache*>(c);
    Request* r = cache->find(h);
    if (r == nullptr) return MBH_UNKNOWN_REQUEST;
    cache->missing(*r, new_len, out);
    return MBH_OK;
}
// Whether all of (handle, new_len) could be reserved together: 1 yes, 0 no, negative: an unknown request.
MBH_API int mbh_can_reserve(void* c, int n, const int64_t* handles, const int* new_lens) {
    Cache* cache = static_cast<Cache*>(c);
    std::vector<int> need(cache->groups(), 0), one(cache->groups(), 0);
    for (int i = 0; i < n; ++i) {
        Request* r = cache->find(handles[i]);
        if (r == nullptr) return -MBH_UNKNOWN_REQUEST;
        cache->missing(*r, new_lens[i], one.data());
        for (int g = 0; g < cache->groups(); ++g) need[g] += one[g];
    }
    for (int g = 0; g < cache->groups(); ++g)
        if (need[g] > cache->pool(g).num_free()) return 0;
    return 1;
}
MBH_API int mbh_reserve(void* c, int64_t h, int new_len) {
    Cache* cache = static_cast<Cache*>(c);
    Request* r = cache->find(h);
    return r == nullptr ? MBH_UNKNOWN_REQUEST : cache->reserve(*r, new_len);
}
MBH_API int mbh_commit(void* c, int64_t h, int new_len) {
    Cache* cache = static_cast<Cache*>(c);
    Request* r = cache->find(h);
    return r == nullptr ? MBH_UNKNOWN_REQUEST : cache->commit(*r, new_len);
}
MBH_API int mbh_release(void* c, int64_t h) { return static_cast<Cache*>(c)->release(h); }
// The request's block table of one group (DROPPED = -1 where a window gave the page back): returns its length, or
// a negative code; copies at most `cap` entries.
MBH_API int mbh_block_table(void* c, int64_t h, int group, int* out, int cap) {
    Cache* cache = static_cast<Cache*>(c);
    Request* r = cache->find(h);
    if (r == nullptr) return -MBH_UNKNOWN_REQUEST;
    if (group < 0 || group >= cache->groups()) return -MBH_BAD_ARG;
    const std::vector<int>& t = r->pages[group];
    std::copy(t.begin(), t.begin() + std::min((size_t)std::max(cap, 0), t.size()), out);
    return (int)t.size();
}
MBH_API int mbh_group_free(void* c, int group) { return static_cast<Cache*>(c)->pool(group).num_free(); }
MBH_API int mbh_group_held(void* c, int group) { return static_cast<Cache*>(c)->pool(group).num_held(); }
MBH_API int mbh_group_check(void* c, int group, char* msg, int cap) {
    std::string why;
    const int rc = static_cast<Cache*>(c)->pool(group).check(&why);
    put_message(why, msg, cap);
    return rc;
}
MBH_API int mbh_slots_free(void* c) { return static_cast<Cache*>(c)->slots().num_free(); }
MBH_API int mbh_slots_held(void* c) { return static_cast<Cache*>(c)->slots().num_held(); }
MBH_API int mbh_slots_check(void* c, char* msg, int cap) {
    std::string why;
    const int rc = static_cast<Cache*>(c)->slots().check(&why);
    put_message(why, msg, cap);
    return rc;
}
MBH_API int mbh_check(void* c, char* msg, int cap) {
    std::string why;
    const int rc = static_cast<Cache*>(c)->check(&why);
    put_message(why, msg, cap);
    return rc;
}

// ---- a whole step's accounting in one call each -----------------------------------------------------------------------
// Before the step: every entry (handle, number of new tokens) must stay within max_seq_len positions and all of them
// together must find their pages, which are then taken; otherwise nothing is taken.  info[0] names the entry at fault
// (-1 for MBH_OUT_OF_PAGES: the step as a whole does not fit), info[1] receives the longest sequence after the step.
MBH_API int mbh_step_reserve(void* c, int n, const int64_t* handles, const int* counts, int max_seq_len, int* info) {
    Cache* cache = static_cast<Cache*>(c);
    std::vector<Request*> reqs(n);
    std::vector<int> need(cache->groups(), 0), one(cache->groups(), 0);
    info[0] = -1;
    info[1] = 0;
    for (int i = 0; i < n; ++i) {
        reqs[i] = cache->find(handles[i]);
        info[0] = i;
        if (reqs[i] == nullptr) return MBH_UNKNOWN_REQUEST;
        if (counts[i] <= 0) return MBH_BAD_ARG;
        if (reqs[i]->length + counts[i] > max_seq_len) return MBH_CONTEXT_FULL;
        info[1] = std::max(info[1], reqs[i]->length + counts[i]);
        cache->missing(*reqs[i], reqs[i]->length + counts[i], one.data());
        for (int g = 0; g < cache->groups(); ++g) need[g] += one[g];
    }
    info[0] = -1;
    for (int g = 0; g < cache->groups(); ++g)
        if (need[g] > cache->pool(g).num_free()) return MBH_OUT_OF_PAGES;
    for (int i = 0; i < n; ++i) {
        const int rc = cache->reserve(*reqs[i], reqs[i]->length + counts[i]);
        if (rc != MBH_OK) return rc;          // cannot happen: the sum was checked above
    }
    return MBH_OK;
}
// After the step: every entry's request now holds its new tokens.
MBH_API int mbh_step_commit(void* c, int n, const int64_t* handles, const int* counts) {
    Cache* cache = static_cast<Cache*>(c);
    for (int i = 0; i < n; ++i) {
        Request* r = cache->find(handles[i]);
        if (r == nullptr) return MBH_UNKNOWN_REQUEST;
        const int rc = cache->commit(*r, r->length + counts[i]);
        if (rc != MBH_OK) return rc;
    }
    return MBH_OK;
}

// ---- packing a step ---------------------------------------------------------------------------------------------------
// The step's n entries (request handle, its next tokens, the places among them whose logits are wanted) become the
// arrays the kernels read, in one int32 buffer in this order:
//   token ids [T], positions [T], request row of each token [T], first token of each row [R + 1], lengths after the
//   step [R], state slots [R], rows whose logits are wanted [W], block tables [G][R][max_pages], and for each group
//   where each new token is written [G][T] (page * page_size + offset, -1: nowhere).
// Entries with a single token come first (the decode kernels take rows 0 .. num_decode - 1), otherwise in the order
// given.  pad_to > 0 (single-token steps only) pads to pad_to rows that stand for empty requests (length 0, state slot
// max_requests: a spare slot no request ever holds), so that a captured graph sees one shape.  info receives T, R, W, the number of single-token rows, the longest entry and the longest
// sequence; spans[row] = (entry, first token, count, first position, slot).  Returns the number of ints written or a
// negative code.
MBH_API int mbh_pack_step(void* c, int n, const int64_t* handles, const int* counts, const int* tokens, const int* want_counts,
                          const int* wants, int pad_to, int max_pages, int32_t* out, int out_cap, int32_t* info, int32_t* spans) {
    Cache* cache = static_cast<Cache*>(c);
    const int G = cache->groups(), page = cache->page_size();
    if (n <= 0 || max_pages <= 0) return -MBH_BAD_ARG;
    std::vector<int> order;
    order.reserve(n);
    int real_T = 0, num_decode = 0, max_query = 0;
    for (int i = 0; i < n; ++i) {
        if (counts[i] <= 0) return -MBH_BAD_ARG;
        if (counts[i] == 1) { order.push_back(i); ++num_decode; }
        real_T += counts[i];
        max_query = std::max(max_query, counts[i]);
    }
    for (int i = 0; i < n; ++i)
        if (counts[i] != 1) order.push_back(i);
    if (pad_to > 0 && (num_decode != n || pad_to < n)) return -MBH_BAD_ARG;
    const int R = pad_to > 0 ? pad_to : n, T = pad_to > 0 ? pad_to : real_T;
    int W = 0;
    if (pad_to > 0) W = pad_to;
    else
        for (int i = 0; i < n; ++i) W += want_counts[i];
    const long long total = 3LL * T + (R + 1) + 2LL * R + W + (long long)G * R * max_pages + (long long)G * T;
    if (total > out_cap) return -MBH_TOO_SMALL;
    int32_t* tok = out;
    int32_t* pos = tok + T;
    int32_t* req = pos + T;
    int32_t* cu = req + T;
    int32_t* lens = cu + R + 1;
    int32_t* slots = lens + R;
    int32_t* rows = slots + R;
    int32_t* tables = rows + W;
    int32_t* maps = tables + (size_t)G * R * max_pages;
    std::fill(out, out + total, 0);
    std::fill(maps, maps + (size_t)G * T, -1);
    if (pad_to > 0) {
        for (int t = 0; t < T; ++t) req[t] = t;
        for (int r = 0; r <= R; ++r) cu[r] = r;
        for (int r = 0; r < W; ++r) rows[r] = r;
    }
    // where each entry's tokens and wants start in the flat inputs
    std::vector<int> tok_at(n + 1, 0), want_at(n + 1, 0), flat_start(n, 0);
    for (int i = 0; i < n; ++i) {
        tok_at[i + 1] = tok_at[i] + counts[i];
        want_at[i + 1] = want_at[i] + (want_counts != nullptr ? want_counts[i] : 0);
    }
    int at = 0, max_seq = 0;
    for (int row = 0; row < n; ++row) {
        const int i = order[row];
        Request* r = cache->find(handles[i]);
        if (r == nullptr) return -MBH_UNKNOWN_REQUEST;
        const int cnt = counts[i];
        flat_start[i] = at;
        for (int j = 0; j < cnt; ++j) {
            tok[at + j] = tokens[tok_at[i] + j];
            pos[at + j] = r->length + j;
            req[at + j] = row;
        }
        cu[row + 1] = at + cnt;
        lens[row] = r->length + cnt;
        max_seq = std::max(max_seq, r->length + cnt);
        slots[row] = r->slot;
        for (int g = 0; g < G; ++g) {
            const std::vector<int>& t = r->pages[g];
            if ((int)t.size() > max_pages) return -MBH_TOO_SMALL;
            int32_t* dst = tables + ((size_t)g * R + row) * max_pages;
            for (size_t k = 0; k < t.size(); ++k) dst[k] = std::max(t[k], 0);
            for (int j = 0; j < cnt; ++j) {
                const int p = r->length + j;
                if (p / page >= (int)t.size()) return -MBH_BAD_ARG;            // the position has no page: reserve first
                maps[(size_t)g * T + at + j] = std::max(t[p / page], 0) * page + p % page;
            }
        }
        spans[row * 5 + 0] = i;
        spans[row * 5 + 1] = at;
        spans[row * 5 + 2] = cnt;
        spans[row * 5 + 3] = r->length;
        spans[row * 5 + 4] = r->slot;
        at += cnt;
    }
    // rows that pad a captured batch stand for empty requests: length 0, and the spare state slot behind the real ones
    for (int row = n; row < R; ++row) slots[row] = cache->slots().size();
    if (pad_to <= 0) {
        int w = 0;
        for (int i = 0; i < n; ++i)
            for (int k = 0; k < want_counts[i]; ++k) rows[w++] = flat_start[i] + wants[want_at[i] + k];
    }
    info[0] = T;
    info[1] = R;
    info[2] = W;
    info[3] = num_decode;
    info[4] = max_query;
    info[5] = max_seq;
    return (int)total;
}
