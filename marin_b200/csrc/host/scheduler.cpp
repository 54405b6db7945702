// The scheduler, host side, in C++: which requests run in the next step, and with how many tokens.
//
// Policy.  Each step has a token budget.  Running requests come first, oldest first: one that is decoding takes one
// token, one that is still reading its prompt takes min(rest of the prompt, budget left) tokens, down to one.  What
// is left of the budget goes to newly admitted requests, first come first served, while fewer than max_batch run
// and the first portion's pages are free.  When pages run out for a request that is already running, the most
// recently admitted running request that is not yet part of the step is preempted: its pages go back, it returns to
// the front of the waiting queue and later recomputes its prompt plus the tokens it had generated.  A request that
// does not fit the pool even when it runs alone ends with OUT_OF_PAGES.  (The reference never runs two Qwen3 requests
// at once and makes a starved request wait for another to finish, crates/cli/src/server/sched.rs:30-51,150-162; its
// stop reasons are crates/runtime/src/generate.rs:38-44.)
#include <deque>

#include "cache_core.h"

using namespace mbh;

namespace {

enum Stop { STOP_NONE = -1, STOP_MAX_TOKENS = 0, STOP_END_OF_TEXT = 1, STOP_CONTEXT_FULL = 2, STOP_CANCELLED = 3, STOP_OUT_OF_PAGES = 4,
            STOP_NON_FINITE = 5 };
enum Where { WAITING = 0, RUNNING = 1, FINISHED = 2 };
enum { MBS_EMPTY_PROMPT = 20, MBS_PROMPT_TOO_LONG = 21, MBS_UNKNOWN = 22 };

struct SReq {
    int64_t id = 0;
    std::vector<int> prompt, output, stop_tokens;
    int max_tokens = 0;
    int computed = 0;            // tokens of prompt + output whose keys and values are in the cache
    int stop = STOP_NONE;
    int preemptions = 0;
    int admitted_at = -1;
    int where = WAITING;
    int64_t handle = 0;          // in the cache, while running
    int slot = -1;
    int num_tokens() const { return (int)(prompt.size() + output.size()); }
    int token_at(int i) const { return i < (int)prompt.size() ? prompt[i] : output[i - (int)prompt.size()]; }
};

struct PlanItem {
    int64_t id;
    int start, count, sample;
    std::vector<int> missing;    // pages per cache group this portion still needs
};

class Scheduler {
  public:
    Scheduler(Cache* cache, int max_batch, int budget, int max_seq_len)
        : cache_(cache), max_batch_(max_batch), budget_(budget), max_seq_len_(max_seq_len) {}

    int add(const int* prompt, int n, int max_tokens, const int* stop_tokens, int n_stop, int64_t* id) {
        if (n <= 0) return MBS_EMPTY_PROMPT;
        if (n > max_seq_len_) return MBS_PROMPT_TOO_LONG;
        SReq r;
        r.id = next_++;
        r.prompt.assign(prompt, prompt + n);
        r.stop_tokens.assign(stop_tokens, stop_tokens + n_stop);
        r.max_tokens = max_tokens;
        *id = r.id;
        if (max_tokens == 0) {
            r.stop = STOP_MAX_TOKENS;
            r.where = FINISHED;
            finished_.push_back(r.id);
        } else {
            waiting_.push_back(r.id);
        }
        reqs_.emplace(r.id, std::move(r));
        return MBH_OK;
    }
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    SReq* find(int64_t id) {
        auto it = reqs_.find(id);
        return it == reqs_.end() ? nullptr : &it->second;
    }
    int forget(int64_t id) {
        SReq* r = find(id);
        if (r == nullptr) return MBS_UNKNOWN;
        if (r->where != FINISHED) return MBH_BAD_ARG;
        finished_.erase(std::remove(finished_.begin(), finished_.end(), id), finished_.end());
        reqs_.erase(id);
        return MBH_OK;
    }
    int cancel(int64_t id) {
        SReq* r = find(id);
        if (r == nullptr) return MBS_UNKNOWN;
        if (r->where == RUNNING) finish(*r, STOP_CANCELLED);
        else if (r->where == WAITING) {
            waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
            r->stop = STOP_CANCELLED;
            r->where = FINISHED;
            finished_.push_back(id);
        }
        return MBH_OK;
    }

    // ---- one step's plan ----------------------------------------------------------------------------------------
    const std::vector<PlanItem>& schedule() {
        plan_.clear();
        membership_changed_ = false;
        int budget = budget_;
        // 1. running requests, oldest first
        std::vector<int64_t> order = running_;
        std::sort(order.begin(), order.end(), [this](int64_t a, int64_t b) { return reqs_[a].admitted_at < reqs_[b].admitted_at; });
        for (int64_t id : order) {
            SReq& r = reqs_[id];
            if (r.where != RUNNING) continue;            // preempted while making room for an older one
            if (budget == 0) break;
            PlanItem item = portion(r, budget);
            while (!fits(item, r)) {
                SReq* victim = nullptr;
                for (int64_t vid : running_) {
                    SReq& v = reqs_[vid];
                    if (vid == id || planned(vid)) continue;
                    if (victim == nullptr || v.admitted_at > victim->admitted_at) victim = &v;
                }
                if (victim == nullptr) break;
                preempt(*victim);
            }
            if (!fits(item, r)) {
                if (plan_.empty() && running_.size() == 1) finish(r, STOP_OUT_OF_PAGES);
                continue;
            }
            item.missing.assign(cache_->groups(), 0);
            cache_->missing(*cache_->find(r.handle), r.computed + item.count, item.missing.data());
            budget -= item.count;
            plan_.push_back(std::move(item));
        }
        // 2. admit waiting requests while there is room
        while (!waiting_.empty() && budget > 0 && (int)running_.size() < max_batch_) {
            SReq& r = reqs_[waiting_.front()];
            PlanItem item = portion(r, budget);
            if (cache_->admit(&r.handle, &r.slot) != MBH_OK) break;        // no state slot: wait
            if (!fits(item, r)) {
                cache_->release(r.handle);
                r.handle = 0;
                if (running_.empty()) {
                    // alone and still too large for the pool: it can never run
                    waiting_.pop_front();
                    r.stop = STOP_OUT_OF_PAGES;
                    r.where = FINISHED;
                    finished_.push_back(r.id);
                    membership_changed_ = true;
                    continue;
                }
                break;
            }
            waiting_.pop_front();
            r.admitted_at = ++clock_;
            r.where = RUNNING;
            running_.push_back(r.id);
            membership_changed_ = true;
            item.missing.assign(cache_->groups(), 0);
            cache_->missing(*cache_->find(r.handle), r.computed + item.count, item.missing.data());
            budget -= item.count;
            plan_.push_back(std::move(item));
        }
        return plan_;
    }

    // The plan of a step that is ALREADY RUNNING: the engine launched it before it knew the tokens of the step before,
    // supposing that the same requests go on with one token each (their pages were taken then).  Requests that have
    // ended or been cancelled since are left out; nobody is admitted or preempted, and nothing is planned for a
    // request that has more than its one next token to read.  Returns false (and an empty plan) if a request of the
    // plan would need a page: such a step must not have been launched.
    bool schedule_decode_only() {
        plan_.clear();
        membership_changed_ = false;
        std::vector<int64_t> order = running_;
        std::sort(order.begin(), order.end(), [this](int64_t a, int64_t b) { return reqs_[a].admitted_at < reqs_[b].admitted_at; });
        for (int64_t id : order) {
            SReq& r = reqs_[id];
            if (r.num_tokens() - r.computed != 1) continue;
            PlanItem item = portion(r, 1);
            item.missing.assign(cache_->groups(), 0);
            Request* rc = cache_->find(r.handle);
            if (rc == nullptr) continue;
            cache_->missing(*rc, r.computed + 1, item.missing.data());
            for (int m : item.missing)
                if (m != 0) { plan_.clear(); return false; }
            plan_.push_back(std::move(item));
        }
        return true;
    }

    // ---- after the step -------------------------------------------------------------------------------------------
    // tokens[k] is the token sampled for the k-th plan item that asked for one (negative: its logits were not finite, the
    // request ends with STOP_NON_FINITE and emits nothing); emitted receives (id, token) pairs.
    int update(const int* tokens, int n_tokens, int64_t* emitted_ids, int* emitted_tokens) {
        membership_changed_ = false;
        int k = 0, out = 0;
        for (const PlanItem& item : plan_) {
            SReq* r = find(item.id);
            const bool live = r != nullptr && r->where == RUNNING;      // not cancelled since the plan was made
            if (live) r->computed += item.count;
            if (!item.sample) continue;
            if (k >= n_tokens) return -MBH_BAD_ARG;
            const int token = tokens[k++];
            if (!live) continue;
            if (token < 0) {                                        // the sampler refused the row: its logits were not finite
                finish(*r, STOP_NON_FINITE);
                continue;
            }
            if (std::find(r->stop_tokens.begin(), r->stop_tokens.end(), token) != r->stop_tokens.end()) {
                finish(*r, STOP_END_OF_TEXT);                       // the stop token is not emitted
                continue;
            }
            r->output.push_back(token);
            emitted_ids[out] = r->id;
            emitted_tokens[out++] = token;
            if ((int)r->output.size() >= r->max_tokens) finish(*r, STOP_MAX_TOKENS);
            else if (r->computed >= max_seq_len_) finish(*r, STOP_CONTEXT_FULL);   // the token just emitted cannot be fed (generate.rs:217-221)
        }
        plan_.clear();
        return out;
    }

    const std::vector<PlanItem>& plan() const { return plan_; }
    const std::deque<int64_t>& waiting() const { return waiting_; }
    const std::vector<int64_t>& running() const { return running_; }
    const std::vector<int64_t>& finished() const { return finished_; }
    bool membership_changed() const { return membership_changed_; }

  private:
    PlanItem portion(const SReq& r, int budget) const {
        const int rest = r.num_tokens() - r.computed;
        PlanItem item;
        item.id = r.id;
        item.start = r.computed;
        item.count = std::min(rest, budget);
        item.sample = rest <= budget ? 1 : 0;
        return item;
    }
    bool planned(int64_t id) const {
        for (const PlanItem& p : plan_)
            if (p.id == id) return true;
        return false;
    }
    // Whether the pages the planned portions and this one need are free, in every group.
    bool fits(const PlanItem& item, const SReq& r) {
        const int G = cache_->groups();
        std::vector<int> need(G, 0), one(G, 0);
        for (const PlanItem& p : plan_)
            for (int g = 0; g < G; ++g) need[g] += p.missing[g];
        Request* rc = cache_->find(r.handle);
        if (rc == nullptr) return false;
        cache_->missing(*rc, r.computed + item.count, one.data());
        for (int g = 0; g < G; ++g)
            if (need[g] + one[g] > cache_->pool(g).num_free()) return false;
        return true;
    }
    void preempt(SReq& v) {
        cache_->release(v.handle);
        v.handle = 0;
        running_.erase(std::remove(running_.begin(), running_.end(), v.id), running_.end());
        v.computed = 0;
        ++v.preemptions;
        v.where = WAITING;
        waiting_.push_front(v.id);
        membership_changed_ = true;
    }
    void finish(SReq& r, int reason) {
        r.stop = reason;
        membership_changed_ = true;
        if (r.where == RUNNING) {
            running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
            cache_->release(r.handle);
            r.handle = 0;
        }
        r.where = FINISHED;
        finished_.push_back(r.id);
    }

    Cache* cache_;
    int max_batch_, budget_, max_seq_len_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_, finished_;
    std::unordered_map<int64_t, SReq> reqs_;
    std::vector<PlanItem> plan_;
    int clock_ = 0;
    int64_t next_ = 1;
    bool membership_changed_ = false;
};

}  // namespace

// ---- C functions ------------------------------------------------------------------------------------------------------
MBH_API void* mbs_create(void* cache, int max_batch, int token_budget, int max_seq_len) {
    if (cache == nullptr || max_batch < 1 || token_budget < 1) return nullptr;
    return new Scheduler(static_cast<Cache*>(cache), max_batch, token_budget, max_seq_len);
}
MBH_API void mbs_destroy(void* s) { delete static_cast<Scheduler*>(s); }
// Returns 0 and the request's id, or 20 (empty prompt) / 21 (prompt longer than the context).
MBH_API int mbs_add(void* s, const int* prompt, int n, int max_tokens, const int* stop_tokens, int n_stop, int64_t* id) {
    return static_cast<Scheduler*>(s)->add(prompt, n, max_tokens, stop_tokens, n_stop, id);
}
MBH_API int mbs_cancel(void* s, int64_t id) { return static_cast<Scheduler*>(s)->cancel(id); }
MBH_API int mbs_forget(void* s, int64_t id) { return static_cast<Scheduler*>(s)->forget(id); }
MBH_API int mbs_has_work(void* s) { return static_cast<Scheduler*>(s)->has_work() ? 1 : 0; }
// Plans the next step.  items receives up to cap rows of (id, first token, count, sample, cache handle, slot); the
// step's tokens, in the same order, go to tokens (up to token_cap).  Returns the number of rows, or a negative code.
// *changed is set when requests were admitted, preempted or ended while planning.
static int mbs_write_plan(Scheduler* sched, const std::vector<PlanItem>& plan, int64_t* items, int cap, int* tokens, int token_cap);

MBH_API int mbs_schedule(void* s, int64_t* items, int cap, int* tokens, int token_cap, int* changed) {
    Scheduler* sched = static_cast<Scheduler*>(s);
    const std::vector<PlanItem>& plan = sched->schedule();
    *changed = sched->membership_changed() ? 1 : 0;
    return mbs_write_plan(sched, plan, items, cap, tokens, token_cap);
}
// The plan of a step that is already running (see Scheduler::schedule_decode_only): rows as mbs_schedule, or -MBH_BAD_ARG
// if that step needed pages it does not have.
MBH_API int mbs_schedule_running(void* s, int64_t* items, int cap, int* tokens, int token_cap) {
    Scheduler* sched = static_cast<Scheduler*>(s);
    if (!sched->schedule_decode_only()) return -MBH_BAD_ARG;
    return mbs_write_plan(sched, sched->plan(), items, cap, tokens, token_cap);
}
static int mbs_write_plan(Scheduler* sched, const std::vector<PlanItem>& plan, int64_t* items, int cap, int* tokens, int token_cap) {
    if ((int)plan.size() > cap) return -MBH_TOO_SMALL;
    int at = 0;
    for (size_t k = 0; k < plan.size(); ++k) {
        const SReq* r = sched->find(plan[k].id);
        items[k * 6 + 0] = plan[k].id;
        items[k * 6 + 1] = plan[k].start;
        items[k * 6 + 2] = plan[k].count;
        items[k * 6 + 3] = plan[k].sample;
        items[k * 6 + 4] = r->handle;
        items[k * 6 + 5] = r->slot;
        if (at + plan[k].count > token_cap) return -MBH_TOO_SMALL;
        for (int j = 0; j < plan[k].count; ++j) tokens[at++] = r->token_at(plan[k].start + j);
    }
    return (int)plan.size();
}
// Records the step that was planned last: tokens[k] for the k-th planned request that asked for a token.  Returns the
// number of (id, token) pairs emitted; *changed is set when requests ended.
MBH_API int mbs_update(void* s, const int* tokens, int n_tokens, int64_t* emitted_ids, int* emitted_tokens, int* changed) {
    Scheduler* sched = static_cast<Scheduler*>(s);
    const int n = sched->update(tokens, n_tokens, emitted_ids, emitted_tokens);
    *changed = sched->membership_changed() ? 1 : 0;
    return n;
}
// out = (computed, tokens generated, stop reason or -1, preemptions, admitted_at, where: 0 waiting 1 running 2 finished,
// cache handle (low 32 bits are enough for tests: the full value comes with mbs_schedule), slot) for each id.
MBH_API int mbs_states(void* s, int n, const int64_t* ids, int64_t* out) {
    Scheduler* sched = static_cast<Scheduler*>(s);
    for (int i = 0; i < n; ++i) {
        const SReq* r = sched->find(ids[i]);
        if (r == nullptr) return MBS_UNKNOWN;
        int64_t* o = out + (size_t)i * 8;
        o[0] = r->computed;
        o[1] = (int64_t)r->output.size();
        o[2] = r->stop;
        o[3] = r->preemptions;
        o[4] = r->admitted_at;
        o[5] = r->where;
        o[6] = r->handle;
        o[7] = r->slot;
    }
    return MBH_OK;
}
// The generated tokens of one request: returns their number, copies at most cap.
MBH_API int mbs_output(void* s, int64_t id, int* out, int cap) {
    const SReq* r = static_cast<Scheduler*>(s)->find(id);
    if (r == nullptr) return -MBS_UNKNOWN;
    std::copy(r->output.begin(), r->output.begin() + std::min((size_t)std::max(cap, 0), r->output.size()), out);
    return (int)r->output.size();
}
// which: 0 waiting (front first), 1 running (in admission order of the list), 2 finished (in the order they ended).
MBH_API int mbs_list(void* s, int which, int64_t* out, int cap) {
    Scheduler* sched = static_cast<Scheduler*>(s);
    std::vector<int64_t> ids;
    if (which == WAITING) ids.assign(sched->waiting().begin(), sched->waiting().end());
    else if (which == RUNNING) ids = sched->running();
    else ids = sched->finished();
    std::copy(ids.begin(), ids.begin() + std::min((size_t)std::max(cap, 0), ids.size()), out);
    return (int)ids.size();
}
