// Host sampler: repetition / presence / frequency penalties, greedy, temperature with top-k / top-p /
// min-p truncation, reported log-probabilities and top-k logprobs.  It is the exact reference the GPU
// sampler is tested against and the fallback when a row's GPU candidates do not settle a draw
// (semantics of the reference's src/session/sampling.cpp:20-140,263-273: weights exp((L - max)/T),
// tokens more than 30 nats below the maximum weigh 0, ties by lower index, top-p keeps the smallest
// prefix whose mass reaches p, min-p is relative to the most likely kept token).
#pragma once
#include <algorithm>
#include <numeric>
#include <random>
#include <unordered_map>
#include <vector>

#include "common.hpp"

namespace qwh {

struct SamplingParams {
    float temperature = 0.f, top_p = 1.f;
    int32_t top_k = 0;
    float min_p = 0.f, presence_penalty = 0.f, frequency_penalty = 0.f, repetition_penalty = 1.f;
    uint64_t seed = 0;
};

// test switch: 1 = every truncation sorts all candidates (the straightforward form the shortcuts are checked against)
inline int &sampler_full_sort_flag() { static int f = 0; return f; }
inline bool sampler_full_sort() { return sampler_full_sort_flag() != 0; }

inline float log_sum_exp(const float *l, int V) {
    const float mx = *std::max_element(l, l + V);
    double z = 0;
    for (int i = 0; i < V; ++i) z += std::exp(double(l[i] - mx));
    return mx + float(std::log(z));
}

// hist[0..n_hist): the sequence so far (prompt + generated); tokens from prompt_end on count for
// presence / frequency, all of them for repetition.  Returns the token; *logprob = raw log-probability.
inline int32_t sample_token(const float *raw, int V, const SamplingParams &p, const int32_t *hist, size_t n_hist,
                            size_t prompt_end, std::mt19937_64 &rng, float *logprob) {
    const bool pen = p.presence_penalty != 0.f || p.frequency_penalty != 0.f || p.repetition_penalty != 1.f;
    std::vector<float> tmp;
    const float *L = raw;
    if (pen) {
        tmp.assign(raw, raw + V);
        if (p.repetition_penalty != 1.f) {
            std::vector<char> seen(size_t(V), 0);
            for (size_t i = 0; i < n_hist; ++i) if (hist[i] >= 0 && hist[i] < V) seen[size_t(hist[i])] = 1;
            for (int i = 0; i < V; ++i)
                if (seen[size_t(i)]) tmp[size_t(i)] = tmp[size_t(i)] > 0 ? tmp[size_t(i)] / p.repetition_penalty : tmp[size_t(i)] * p.repetition_penalty;
        }
        std::unordered_map<int32_t, int> counts;
        for (size_t i = prompt_end; i < n_hist; ++i) if (hist[i] >= 0 && hist[i] < V) ++counts[hist[i]];
        for (auto &kv : counts) tmp[size_t(kv.first)] -= p.presence_penalty + p.frequency_penalty * float(kv.second);
        L = tmp.data();
    }
    auto finish = [&](int32_t tok) {
        if (logprob) *logprob = raw[tok] - log_sum_exp(raw, V);
        return tok;
    };
    const int32_t best = int32_t(std::max_element(L, L + V) - L);
    if (p.temperature <= 0.f) return finish(best);
    std::mt19937_64 seeded(p.seed + n_hist);
    std::mt19937_64 &g = p.seed ? seeded : rng;
    const float lmax = L[best], inv_t = 1.f / p.temperature;
    std::vector<int32_t> idx;
    std::vector<double> w;
    double z_all = 0;
    for (int i = 0; i < V; ++i) {
        const float z = (L[i] - lmax) * inv_t;
        if (z < -30.f) continue;
        idx.push_back(i);
        w.push_back(std::exp(double(z)));
        z_all += w.back();
    }
    std::vector<size_t> order(idx.size());
    std::iota(order.begin(), order.end(), size_t(0));
    auto by_logit = [&](size_t a, size_t b) { return L[idx[a]] > L[idx[b]] || (L[idx[a]] == L[idx[b]] && idx[a] < idx[b]); };
    const size_t n = order.size();
    size_t K = n;
    if (p.top_k > 0 && size_t(p.top_k) < K) K = size_t(p.top_k);
    // Only as much of the order as the truncation looks at is ever sorted (by_logit is a strict total order, so the first m
    // entries of a partial sort are the first m of the full sort): a vocabulary of 250k candidates costs a few
    // milliseconds instead of fifty.  sampler_full_sort() switches the shortcut off (the tests compare the two).
    auto sort_first = [&](size_t m) {
        if (m >= n / 2 || sampler_full_sort()) {
            std::sort(order.begin(), order.end(), by_logit);
        } else if (m <= 64) {
            std::partial_sort(order.begin(), order.begin() + ptrdiff_t(m), order.end(), by_logit);
        } else {                                              // select the m first (linear), then order them
            std::nth_element(order.begin(), order.begin() + ptrdiff_t(m), order.end(), by_logit);
            std::sort(order.begin(), order.begin() + ptrdiff_t(m), by_logit);
        }
    };
    const bool truncating = p.top_p < 1.f || p.top_k > 0 || p.min_p > 0.f;
    size_t keep = K;
    const bool k_sorted = truncating && (K < n || p.top_k > 0);          // top-k: its K entries are sorted up front
    if (k_sorted) {
        sort_first(K);
    } else if (truncating && p.top_p >= 1.f) {
        // min-p alone: the kept tokens are exactly those that weigh at least min_p times the heaviest (weight 1)
        size_t heavy = 0;
        for (size_t i = 0; i < n; ++i) heavy += w[i] >= double(p.min_p) ? 1 : 0;
        sort_first(std::max<size_t>(heavy, 1));
    }
    double z = 0;
    if (p.top_k > 0) for (size_t i = 0; i < K; ++i) z += w[order[i]];
    const double norm = p.top_k > 0 ? z : z_all;
    if (p.top_p < 1.f) {
        // top-p: the shortest prefix whose mass reaches p; without top-k the sorted part is widened until it holds that prefix
        size_t sorted = k_sorted ? K : 0;
        for (;;) {
            if (sorted < K) {
                sorted = std::min(K, std::max<size_t>(1024, sorted * 8));
                sort_first(sorted);
                if (sampler_full_sort()) sorted = K;
            }
            double acc = 0;
            bool found = false;
            for (size_t i = 0; i < sorted; ++i) {
                acc += w[order[i]] / norm;
                if (acc >= p.top_p) { keep = i + 1; found = true; break; }
            }
            if (found || sorted >= K) break;
        }
    }
    if (p.min_p > 0.f) {
        const double thr = double(p.min_p) * w[order[0]];
        size_t k = 0;
        while (k < keep && w[order[k]] >= thr) ++k;
        keep = std::max<size_t>(k, 1);
    }
    double tot = 0;
    for (size_t i = 0; i < keep; ++i) tot += w[order[i]];
    double r = std::uniform_real_distribution<double>(0, tot)(g);
    for (size_t i = 0; i < keep; ++i) {
        r -= w[order[i]];
        if (r <= 0) return finish(idx[order[i]]);
    }
    return finish(idx[order[keep - 1]]);
}

inline int top_logprobs(const float *raw, int V, int k, int32_t *ids, float *lps) {
    k = std::min(k, V);
    std::vector<int32_t> order(static_cast<size_t>(V), 0);
    std::iota(order.begin(), order.end(), 0);
    std::partial_sort(order.begin(), order.begin() + k, order.end(), [&](int32_t a, int32_t b) { return raw[a] > raw[b] || (raw[a] == raw[b] && a < b); });
    const float lse = log_sum_exp(raw, V);
    for (int i = 0; i < k; ++i) { ids[i] = order[size_t(i)]; lps[i] = raw[order[size_t(i)]] - lse; }
    return k;
}

}  // namespace qwh
