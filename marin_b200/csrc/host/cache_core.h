// Classes of the host side of the cache manager (see cache_core.cpp): page pools, requests with their block tables,
// and the cache that owns them.  Shared by the C functions of cache_core.cpp and by the scheduler (scheduler.cpp).
#pragma once
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

namespace mbh {

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

}  // namespace mbh
