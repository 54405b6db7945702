// Host side of the cache manager, in C++: page pools, per-request block tables and state slots, and the packing
// of a step's requests into the one int32 buffer the kernels read.  No device memory is touched here; the Python
// classes in marin_b200/cache keep the tensors and call in through the C functions at the end of this file.
//
// Layers whose mixers need the same thing of the cache form a group with a pool of its own; a request holds one
// block table per group.  Pages go back to their pool when the request ends or when a group's window has passed
// them, and are handed out again, last freed first.  (The reference keeps one private LIFO pool per sequence:
// crates/cuda/src/pages.rs:20-65, crates/cuda/src/kv.rs:214-270; the shared pool is this engine's own design.)
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#define MBH_API extern "C" __attribute__((visibility("default")))

enum {
    MBH_OK = 0,
    MBH_OUT_OF_PAGES = 1,       // nothing was taken
    MBH_NOT_HELD = 2,           // a page freed twice or never handed out
    MBH_BAD_ARG = 3,
    MBH_UNKNOWN_REQUEST = 4,
    MBH_NO_SLOT = 5,
    MBH_INCONSISTENT = 6,       // check() found a page lost or held twice
    MBH_TOO_SMALL = 7,          // the caller's buffer is too small
    MBH_CONTEXT_FULL = 8,       // a request would grow past the context capacity
};

static const int DROPPED = -1;  // a block-table entry whose page a window has given back

namespace {

class PagePool {
  public:
    explicit PagePool(int n) : n_(n), held_(n, 0), held_count_(0) {
        free_.reserve(n);
        for (int p = n - 1; p >= 0; --p) free_.push_back(p);
    }
    int size() const { return n_; }
    int num_free() const { return (int)free_.size(); }
    int num_held() const { return held_count_; }
    // All of `count` pages or none.
    int alloc(int count, std::vector<int>* out) {
        if (count < 0) return MBH_BAD_ARG;
        if (count > (int)free_.size()) return MBH_OUT_OF_PAGES;
        for (int i = 0; i < count; ++i) {
            const int p = free_.back();
            free_.pop_back();
            held_[p] = 1;
            ++held_count_;
            out->push_back(p);
        }
        return MBH_OK;
    }
    int free_page(int page) {
        if (page < 0 || page >= n_ || !held_[page]) return MBH_NOT_HELD;
        held_[page] = 0;
        --held_count_;
        free_.push_back(page);
        return MBH_OK;
    }
    bool is_held(int page) const { return page >= 0 && page < n_ && held_[page]; }
    // Every page is either free or held, exactly once.
    int check(std::string* why) const {
        std::vector<char> seen(n_, 0);
        for (int p : free_) {
            if (p < 0 || p >= n_) { *why = "a page id outside the pool is on the free list"; return MBH_INCONSISTENT; }
            if (seen[p]) { *why = "a page is on the free list twice"; return MBH_INCONSISTENT; }
            if (held_[p]) { *why = "page " + std::to_string(p) + " is both free and held"; return MBH_INCONSISTENT; }
            seen[p] = 1;
        }
        if ((int)free_.size() + held_count_ != n_) { *why = "a page was lost"; return MBH_INCONSISTENT; }
        return MBH_OK;
    }

  private:
    int n_;
    std::vector<int> free_;
    std::vector<char> held_;
    int held_count_;
};

struct Request {
    int slot = 0;
    int length = 0;
    int dropped = 0;                          // pages that windows have given back so far
    std::vector<std::vector<int>> pages;      // per group: logical page -> page id or DROPPED
};

class Cache {
  public:
    Cache(int page_size, int num_pages, int max_requests, int n_groups, const int* windows)
        : page_size_(page_size), slots_(max_requests) {
        for (int g = 0; g < n_groups; ++g) {
            windows_.push_back(windows[g]);
            pools_.emplace_back(num_pages);
        }
    }
    int groups() const { return (int)pools_.size(); }
    int page_size() const { return page_size_; }
    PagePool& pool(int g) { return pools_[g]; }
    PagePool& slots() { return slots_; }
    Request* find(int64_t h) {
        auto it = reqs_.find(h);
        return it == reqs_.end() ? nullptr : &it->second;
    }
    size_t live() const { return reqs_.size(); }

    int admit(int64_t* handle, int* slot) {
        std::vector<int> got;
        if (slots_.alloc(1, &got) != MBH_OK) return MBH_NO_SLOT;
        Request r;
        r.slot = got[0];
        r.pages.resize(pools_.size());
        *handle = next_++;
        *slot = r.slot;
        reqs_.emplace(*handle, std::move(r));
        return MBH_OK;
    }
    void missing(const Request& r, int new_len, int* out) const {
        const int total = (new_len + page_size_ - 1) / page_size_;
        for (size_t g = 0; g < pools_.size(); ++g) out[g] = std::max(0, total - (int)r.pages[g].size());
    }
    // Pages so that positions < new_len have a place, in every group, or MBH_OUT_OF_PAGES with nothing taken.
    int reserve(Request& r, int new_len) {
        std::vector<int> need(pools_.size());
        missing(r, new_len, need.data());
        for (size_t g = 0; g < pools_.size(); ++g)
            if (need[g] > pools_[g].num_free()) return MBH_OUT_OF_PAGES;
        for (size_t g = 0; g < pools_.size(); ++g) pools_[g].alloc(need[g], &r.pages[g]);
        return MBH_OK;
    }
    // The step succeeded: the request holds new_len positions; pages a window has passed go back to their pool.
    int commit(Request& r, int new_len) {
        if (new_len < r.length) return MBH_BAD_ARG;
        r.length = new_len;
        for (size_t g = 0; g < pools_.size(); ++g) {
            if (windows_[g] < 0) continue;
            const int first = std::max(0, new_len - windows_[g] + 1) / page_size_;   // the next token's first needed page
            std::vector<int>& table = r.pages[g];
            for (int logical = 0; logical < std::min(first, (int)table.size()); ++logical) {
                if (table[logical] != DROPPED) {
                    const int rc = pools_[g].free_page(table[logical]);
                    if (rc != MBH_OK) return rc;
                    table[logical] = DROPPED;
                    ++r.dropped;
                }
            }
        }
        return MBH_OK;
    }
    int release(int64_t h) {
        auto it = reqs_.find(h);
        if (it == reqs_.end()) return MBH_UNKNOWN_REQUEST;
        int rc = MBH_OK;
        for (size_t g = 0; g < pools_.size(); ++g)
            for (int p : it->second.pages[g])
                if (p != DROPPED) {
                    const int e = pools_[g].free_page(p);
                    if (e != MBH_OK) rc = e;
                }
        const int e = slots_.free_page(it->second.slot);
        if (e != MBH_OK) rc = e;
        reqs_.erase(it);
        return rc;
    }
    // No page lost, held twice or freed twice: the pools agree with the block tables.
    int check(std::string* why) {
        for (size_t g = 0; g < pools_.size(); ++g) {
            const int rc = pools_[g].check(why);
            if (rc != MBH_OK) return rc;
            std::vector<char> seen(pools_[g].size(), 0);
            int count = 0;
            for (auto& kv : reqs_)
                for (int p : kv.second.pages[g]) {
                    if (p == DROPPED) continue;
                    if (!pools_[g].is_held(p)) { *why = "a block table names page " + std::to_string(p) + " that is not held"; return MBH_INCONSISTENT; }
                    if (seen[p]) { *why = "page " + std::to_string(p) + " of group " + std::to_string(g) + " is in two block tables"; return MBH_INCONSISTENT; }
                    seen[p] = 1;
                    ++count;
                }
            if (count != pools_[g].num_held()) {
                *why = "group " + std::to_string(g) + ": " + std::to_string(pools_[g].num_held()) + " pages held, " + std::to_string(count) + " in block tables";
                return MBH_INCONSISTENT;
            }
        }
        const int rc = slots_.check(why);
        if (rc != MBH_OK) return rc;
        if (slots_.num_held() != (int)reqs_.size()) { *why = "slots held and live requests differ"; return MBH_INCONSISTENT; }
        return MBH_OK;
    }

  private:
    int page_size_;
    std::vector<int> windows_;               // per group, -1: all keys are kept
    std::vector<PagePool> pools_;
    PagePool slots_;
    std::unordered_map<int64_t, Request> reqs_;
    int64_t next_ = 1;
};

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
// together must find their pages, which are then taken; otherwise nothing is taken and *bad names the entry at fault
// (for MBH_OUT_OF_PAGES: -1, the step as a whole does not fit).
MBH_API int mbh_step_reserve(void* c, int n, const int64_t* handles, const int* counts, int max_seq_len, int* bad) {
    Cache* cache = static_cast<Cache*>(c);
    std::vector<Request*> reqs(n);
    std::vector<int> need(cache->groups(), 0), one(cache->groups(), 0);
    *bad = -1;
    for (int i = 0; i < n; ++i) {
        reqs[i] = cache->find(handles[i]);
        *bad = i;
        if (reqs[i] == nullptr) return MBH_UNKNOWN_REQUEST;
        if (counts[i] <= 0) return MBH_BAD_ARG;
        if (reqs[i]->length + counts[i] > max_seq_len) return MBH_CONTEXT_FULL;
        cache->missing(*reqs[i], reqs[i]->length + counts[i], one.data());
        for (int g = 0; g < cache->groups(); ++g) need[g] += one[g];
    }
    *bad = -1;
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
// given.  pad_to > 0 (single-token steps only) pads to pad_to rows that stand for empty requests, so that a captured
// graph sees one shape.  info receives T, R, W, the number of single-token rows, the longest entry and the longest
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
