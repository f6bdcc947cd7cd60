// TEST INFRASTRUCTURE — not part of the product.
//
// The part of the CPU checkers that is the same whichever engine produces the candidate list: row pre-processing
// (bias, mask), the draw with a caller-supplied uniform, draft verification, general p/q rejection sampling and the
// threaded timing loop. An Engine provides:
//     Engine(const orc_params&, uint32_t n_vocab, uint64_t seed);
//     void accept(int32_t token);
//     bool greedy() const;
//     const std::vector<std::pair<float, int32_t>>& distribution(const float* logits);   // (q, id), draw order
//     int32_t sample_own_rng(const float* logits);                                        // unmodified sample()
// sampler_port.cpp supplies a restated engine, ref_shim.cpp one backed by the reference's own Sampler.
#pragma once

#include "oracle_api.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <random>
#include <thread>
#include <utility>
#include <vector>

namespace orc {

using Cand = std::pair<float, int32_t>;

// Bias then mask, on a copy of the row (the order the kernels use too). Returns the pointer the engine should read.
inline const float* preprocess(const orc_row& row, std::vector<float>& tmp)
{
    if (row.n_bias == 0 && row.mask == nullptr)
        return row.logits;
    tmp.assign(row.logits, row.logits + row.n_vocab);
    for (uint32_t j = 0; j < row.n_bias; ++j) {
        const int32_t id = row.bias_ids[j];
        if (id >= 0 && uint32_t(id) < row.n_vocab)
            tmp[size_t(id)] = tmp[size_t(id)] + row.bias_vals[j];
    }
    if (row.mask != nullptr) {
        const float ninf = -std::numeric_limits<float>::infinity();
        for (uint32_t i = 0; i < row.n_vocab; ++i)
            if (((row.mask[i >> 5] >> (i & 31)) & 1u) == 0)
                tmp[i] = ninf;
    }
    return tmp.data();
}

// Greedy: first maximum of the row the sampler is handed (sampler.cpp:77-78); penalties play no part.
inline int32_t first_argmax(const float* l, uint32_t n)
{
    return int32_t(std::max_element(l, l + n) - l);
}

// Left-to-right float sum of the candidates in stored order (sampler.cpp:80-82).
inline float float_total(const std::vector<Cand>& c)
{
    float total = 0;
    for (const Cand& x : c)
        total += x.first;
    return total;
}

// The walk of sampler.cpp:64-73 with r = u * total supplied from outside. Returns the position in c.
inline size_t walk(const std::vector<Cand>& c, float r)
{
    for (size_t i = 0; i < c.size(); ++i) {
        if (r < c[i].first)
            return i;
        r -= c[i].first;
    }
    return c.size() - 1;
}

// 1 when r = u*total lies within 1e-6*total of the CDF boundary below or above the chosen candidate.
inline uint32_t near_cdf_boundary(const std::vector<Cand>& c, float r0, float total, size_t chosen)
{
    float r = r0;
    for (size_t i = 0; i < chosen; ++i)
        r -= c[i].first;
    const float eps = 1e-6f * total;
    const bool low = chosen > 0 && r < eps;
    const bool high = chosen + 1 < c.size() && (c[chosen].first - r) < eps;
    return (low || high) ? 1u : 0u;
}

template <class Engine> struct Driver {
    static void load_history(Engine& e, const orc_row& row)
    {
        for (uint32_t j = 0; j < row.n_history; ++j)
            e.accept(row.history[j]);
    }

    static int sample(const orc_params* p, const orc_row* row, float u, int32_t* token, float* prob, uint32_t* n_cand,
                      int32_t* cand_ids, float* cand_q, uint32_t cap, uint32_t* near_boundary)
    {
        if (!p || !row || row->n_vocab == 0)
            return -1;
        Engine e(*p, row->n_vocab, 0);
        load_history(e, *row);
        std::vector<float> tmp;
        const float* l = preprocess(*row, tmp);
        if (near_boundary)
            *near_boundary = 0;
        if (e.greedy()) {
            const int32_t t = first_argmax(l, row->n_vocab);
            if (token) *token = t;
            if (prob) *prob = 1.0f;
            if (n_cand) *n_cand = 1;
            if (cap > 0 && cand_ids) cand_ids[0] = t;
            if (cap > 0 && cand_q) cand_q[0] = 1.0f;
            return 0;
        }
        const std::vector<Cand>& c = e.distribution(l);
        const float total = float_total(c);
        const float r = u * total;
        const size_t k = walk(c, r);
        if (token) *token = c[k].second;
        if (prob) *prob = c[k].first / total;
        if (n_cand) *n_cand = uint32_t(c.size());
        for (size_t i = 0; i < c.size() && i < cap; ++i) {
            if (cand_ids) cand_ids[i] = c[i].second;
            if (cand_q) cand_q[i] = c[i].first;
        }
        if (near_boundary)
            *near_boundary = near_cdf_boundary(c, r, total, k);
        return 0;
    }

    // sampler.cpp:86-107 with both uniforms supplied.
    static int verify(const orc_params* p, const orc_row* row, int32_t draft, float u1, float u2, int32_t* token,
                      int32_t* accepted)
    {
        if (!p || !row || row->n_vocab == 0)
            return -1;
        Engine e(*p, row->n_vocab, 0);
        load_history(e, *row);
        std::vector<float> tmp;
        const float* l = preprocess(*row, tmp);
        if (e.greedy()) {
            const int32_t t = first_argmax(l, row->n_vocab);
            *accepted = t == draft;
            *token = t;
            return 0;
        }
        std::vector<Cand> c = e.distribution(l);
        float total = 0, q_draft = 0;
        for (const Cand& x : c) {
            total += x.first;
            if (x.second == draft)
                q_draft = x.first;
        }
        *accepted = (u1 * total) < q_draft;
        if (*accepted) {
            *token = draft;
            return 0;
        }
        c.erase(std::remove_if(c.begin(), c.end(), [&](const Cand& x) { return x.second == draft; }), c.end());
        if (c.empty()) {
            *token = draft;
            return 0;
        }
        const float rest = total - q_draft;
        *token = c[walk(c, u2 * rest)].second;
        return 0;
    }

    static int verify_pq(const orc_params* p, const orc_row* target, const orc_row* drafter, float u_draft,
                         float u_accept, float u_resample, int32_t* draft_token, int32_t* accepted, int32_t* token)
    {
        if (!p || !target || !drafter || target->n_vocab == 0 || drafter->n_vocab != target->n_vocab)
            return -1;
        std::vector<float> tmp;
        Engine eq(*p, drafter->n_vocab, 0);
        load_history(eq, *drafter);
        const float* lq = preprocess(*drafter, tmp);
        if (eq.greedy()) { // both distributions are one-hot: the draft is kept iff it is the target's argmax
            const int32_t d = first_argmax(lq, drafter->n_vocab);
            std::vector<float> tmp2;
            const float* lp = preprocess(*target, tmp2);
            const int32_t t = first_argmax(lp, target->n_vocab);
            *draft_token = d;
            *accepted = t == d;
            *token = t;
            return 0;
        }
        std::vector<Cand> cq = eq.distribution(lq);
        const float total_q = float_total(cq);
        const size_t kd = walk(cq, u_draft * total_q);
        const int32_t d = cq[kd].second;
        const float qd = cq[kd].first / total_q;

        Engine ep(*p, target->n_vocab, 0);
        load_history(ep, *target);
        const float* lp = preprocess(*target, tmp);
        std::vector<Cand> cp = ep.distribution(lp);
        const float total_p = float_total(cp);
        float pd = 0;
        for (const Cand& x : cp)
            if (x.second == d)
                pd = x.first / total_p;
        *draft_token = d;
        *accepted = (u_accept * qd) < pd;
        if (*accepted) {
            *token = d;
            return 0;
        }
        // Residual over the union, ascending id.
        auto by_id = [](const Cand& a, const Cand& b) { return a.second < b.second; };
        std::sort(cp.begin(), cp.end(), by_id);
        std::sort(cq.begin(), cq.end(), by_id);
        std::vector<Cand> res;
        size_t i = 0, j = 0;
        while (i < cp.size() || j < cq.size()) {
            int32_t id;
            float pn = 0, qn = 0;
            if (j >= cq.size() || (i < cp.size() && cp[i].second < cq[j].second)) {
                id = cp[i].second;
                pn = cp[i].first / total_p;
                ++i;
            } else if (i >= cp.size() || cq[j].second < cp[i].second) {
                id = cq[j].second;
                qn = cq[j].first / total_q;
                ++j;
            } else {
                id = cp[i].second;
                pn = cp[i].first / total_p;
                qn = cq[j].first / total_q;
                ++i;
                ++j;
            }
            const float r = pn - qn;
            if (r > 0.0f)
                res.emplace_back(r, id);
        }
        if (res.empty()) {
            *token = d;
            return 0;
        }
        const float total_r = float_total(res);
        *token = res[walk(res, u_resample * total_r)].second;
        return 0;
    }

    static int sample_rng(const orc_params* p, const orc_row* row, uint64_t seed, uint32_t n_draws, int32_t* tokens)
    {
        if (!p || !row || row->n_vocab == 0)
            return -1;
        Engine e(*p, row->n_vocab, seed);
        load_history(e, *row);
        std::vector<float> tmp;
        const float* l = preprocess(*row, tmp);
        for (uint32_t i = 0; i < n_draws; ++i)
            tokens[i] = e.sample_own_rng(l);
        return 0;
    }

    static double time_batch(const orc_params* p, uint32_t batch, uint32_t n_vocab, const float* logits, uint64_t ld,
                             const int32_t* history, uint32_t n_history, const uint32_t* mask, uint64_t mask_ld,
                             const int32_t* bias_ids, const float* bias_vals, uint32_t n_bias, const float* u,
                             uint32_t n_threads, int32_t* tokens)
    {
        if (!p || n_vocab == 0 || batch == 0 || !logits || !u || !tokens)
            return -1.0;
        n_threads = std::max(1u, std::min(n_threads, batch));
        std::vector<Engine> engines;
        engines.reserve(batch);
        for (uint32_t b = 0; b < batch; ++b) {
            engines.emplace_back(*p, n_vocab, 0);
            for (uint32_t j = 0; j < n_history; ++j)
                engines.back().accept(history[size_t(b) * n_history + j]);
        }
        auto work = [&](uint32_t t) {
            std::vector<float> tmp;
            for (uint32_t b = t; b < batch; b += n_threads) {
                orc_row row{n_vocab,
                            logits + size_t(b) * ld,
                            nullptr,
                            0,
                            mask ? mask + size_t(b) * mask_ld : nullptr,
                            n_bias ? bias_ids + size_t(b) * n_bias : nullptr,
                            n_bias ? bias_vals + size_t(b) * n_bias : nullptr,
                            n_bias};
                const float* l = preprocess(row, tmp);
                Engine& e = engines[b];
                if (e.greedy()) {
                    tokens[b] = first_argmax(l, n_vocab);
                    continue;
                }
                const std::vector<Cand>& c = e.distribution(l);
                const float total = float_total(c);
                tokens[b] = c[walk(c, u[b] * total)].second;
            }
        };
        auto pass = [&]() {
            if (n_threads == 1) {
                work(0);
            } else {
                std::vector<std::thread> pool;
                for (uint32_t t = 0; t < n_threads; ++t)
                    pool.emplace_back(work, t);
                for (auto& th : pool)
                    th.join();
            }
        };
        // One untimed pass first: a sampler's work and candidate vectors are allocated by its first call, which a
        // long-lived reference Sampler pays once per request, not once per token. The timed pass is the steady state.
        pass();
        const auto t0 = std::chrono::steady_clock::now();
        pass();
        return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    }
};

} // namespace orc

#define ORC_EXPORT_API(ENGINE, KIND)                                                                                   \
    extern "C" {                                                                                                       \
    const char* orc_kind(void) { return KIND; }                                                                        \
    int orc_sample(const orc_params* p, const orc_row* row, float u, int32_t* token, float* prob, uint32_t* n_cand,    \
                   int32_t* cand_ids, float* cand_q, uint32_t cap, uint32_t* nb)                                       \
    {                                                                                                                  \
        return orc::Driver<ENGINE>::sample(p, row, u, token, prob, n_cand, cand_ids, cand_q, cap, nb);                 \
    }                                                                                                                  \
    int orc_verify(const orc_params* p, const orc_row* row, int32_t draft, float u1, float u2, int32_t* token,         \
                   int32_t* accepted)                                                                                  \
    {                                                                                                                  \
        return orc::Driver<ENGINE>::verify(p, row, draft, u1, u2, token, accepted);                                    \
    }                                                                                                                  \
    int orc_verify_pq(const orc_params* p, const orc_row* t, const orc_row* d, float ud, float ua, float ur,           \
                      int32_t* draft_token, int32_t* accepted, int32_t* token)                                         \
    {                                                                                                                  \
        return orc::Driver<ENGINE>::verify_pq(p, t, d, ud, ua, ur, draft_token, accepted, token);                      \
    }                                                                                                                  \
    int orc_sample_rng(const orc_params* p, const orc_row* row, uint64_t seed, uint32_t n, int32_t* tokens)            \
    {                                                                                                                  \
        return orc::Driver<ENGINE>::sample_rng(p, row, seed, n, tokens);                                               \
    }                                                                                                                  \
    void orc_uniforms(uint64_t seed, uint32_t n, float* out)                                                           \
    {                                                                                                                  \
        std::mt19937_64 g(seed);                                                                                       \
        for (uint32_t i = 0; i < n; ++i)                                                                               \
            out[i] = std::generate_canonical<float, std::numeric_limits<float>::digits>(g);                            \
    }                                                                                                                  \
    double orc_time_sample_batch(const orc_params* p, uint32_t batch, uint32_t n_vocab, const float* logits,           \
                                 uint64_t ld, const int32_t* history, uint32_t n_history, const uint32_t* mask,        \
                                 uint64_t mask_ld, const int32_t* bias_ids, const float* bias_vals, uint32_t n_bias,   \
                                 const float* u, uint32_t n_threads, int32_t* tokens)                                  \
    {                                                                                                                  \
        return orc::Driver<ENGINE>::time_batch(p, batch, n_vocab, logits, ld, history, n_history, mask, mask_ld,       \
                                               bias_ids, bias_vals, n_bias, u, n_threads, tokens);                     \
    }                                                                                                                  \
    }
