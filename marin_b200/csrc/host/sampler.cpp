// Token sampling on the host with the reference's semantics (crates/sampler/src/lib.rs), in C++.
//
// Order of operations (lib.rs:122-193): only the first `usable` logits are candidates; a NaN or infinity is an error;
// temperature 0 picks the largest logit, the lowest id among equals; otherwise tokens are ranked by (logit descending,
// id ascending), the best top_k are kept (0 = all), weights exp((l - l_max) / temperature) are normalised, the shortest
// prefix whose mass reaches top_p is kept (the crossing token included) and renormalised.  A draw u in [0, 1) from
// splitmix64 (top 24 bits, lib.rs:196-203) selects the first token whose cumulative probability exceeds it, else the
// last (lib.rs:101-118).  Sums are float32 and sequential.  The reference's two shortcuts (bounded top-k scan, the FAR
// cutoff) give the same tokens as this plain algorithm by construction and are not repeated here.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#define MBH_API extern "C" __attribute__((visibility("default")))

enum { MBP_BAD_USABLE = 1, MBP_NOT_FINITE = 2, MBP_TOO_SMALL = 3 };

namespace {

// Keys that order float32 values the way IEEE total order does (-0.0 below +0.0).
inline int32_t total_order_key(float v) {
    int32_t bits;
    std::memcpy(&bits, &v, 4);
    return bits ^ ((bits >> 31) & 0x7FFFFFFF);
}

int best_index(const float* v, int n) {
    int best = 0;
    int32_t best_key = total_order_key(v[0]);
    for (int i = 1; i < n; ++i) {
        const int32_t k = total_order_key(v[i]);
        if (k > best_key) { best_key = k; best = i; }         // the lowest id among equals stays
    }
    return best;
}

// The kept set in rank order with its probabilities; returns its size or a negative code.
int distribution(const float* logits, int n, int usable, float temperature, int top_k, float top_p, std::vector<int>* ids,
                 std::vector<float>* probs) {
    if (usable <= 0 || usable > n) return -MBP_BAD_USABLE;
    for (int i = 0; i < usable; ++i)
        if (!std::isfinite(logits[i])) return -MBP_NOT_FINITE;
    ids->clear();
    probs->clear();
    if (temperature == 0.0f) {
        ids->push_back(best_index(logits, usable));
        probs->push_back(1.0f);
        return 1;
    }
    std::vector<int> order(usable);
    std::iota(order.begin(), order.end(), 0);
    auto before = [logits](int a, int b) {
        const int32_t ka = total_order_key(logits[a]), kb = total_order_key(logits[b]);
        return ka != kb ? ka > kb : a < b;                     // logit descending, id ascending among equals
    };
    int keep_k = usable;
    if (top_k > 0 && top_k < usable) {
        std::partial_sort(order.begin(), order.begin() + top_k, order.end(), before);
        keep_k = top_k;
    } else {
        std::sort(order.begin(), order.end(), before);
    }
    std::vector<float> weights(keep_k);
    const float top = logits[order[0]];
    float total = 0.0f;
    for (int r = 0; r < keep_k; ++r) {
        weights[r] = std::exp((logits[order[r]] - top) / temperature);
        total += weights[r];
    }
    float mass = 0.0f;
    int keep = keep_k;
    for (int r = 0; r < keep_k; ++r) {
        weights[r] = weights[r] / total;
        mass += weights[r];
        if (mass >= top_p) { keep = r + 1; break; }
    }
    float kept_mass = 0.0f;
    for (int r = 0; r < keep; ++r) kept_mass += weights[r];
    for (int r = 0; r < keep; ++r) {
        ids->push_back(order[r]);
        probs->push_back(weights[r] / kept_mass);
    }
    return keep;
}

float next_unit(uint64_t* state) {
    *state += 0x9E3779B97F4A7C15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) / 16777216.0f;
}

}  // namespace

MBH_API int mbp_best_index(const float* values, int n) { return n > 0 ? best_index(values, n) : -MBP_BAD_USABLE; }

// ids/probs receive the kept set in rank order (at most cap entries are copied); returns its size or a negative code.
MBH_API int mbp_distribution(const float* logits, int n, int usable, float temperature, int top_k, float top_p, int* ids,
                             float* probs, int cap) {
    std::vector<int> i;
    std::vector<float> p;
    const int kept = distribution(logits, n, usable, temperature, top_k, top_p, &i, &p);
    if (kept < 0) return kept;
    const int copy = std::min(kept, std::max(cap, 0));
    std::copy(i.begin(), i.begin() + copy, ids);
    std::copy(p.begin(), p.begin() + copy, probs);
    return kept;
}

MBH_API float mbp_next_unit(uint64_t* state) { return next_unit(state); }

// One token for one row of logits; the generator's state advances only when a draw is needed.
MBH_API int mbp_sample(const float* logits, int n, int usable, float temperature, int top_k, float top_p, uint64_t* state) {
    std::vector<int> ids;
    std::vector<float> probs;
    const int kept = distribution(logits, n, usable, temperature, top_k, top_p, &ids, &probs);
    if (kept < 0) return kept;
    if (temperature == 0.0f) return ids[0];
    const float draw = next_unit(state);
    float cumulative = 0.0f;
    for (int r = 0; r < kept; ++r) {
        cumulative += probs[r];
        if (draw < cumulative) return ids[r];
    }
    return ids[kept - 1];
}
