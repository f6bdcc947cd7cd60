// TEST INFRASTRUCTURE — not part of the product.
//
// CPU restatement ("port") of the reference token sampler, written from its behaviour and used as the parity
// checker where the reference sources are not present. Each step cites the reference lines it follows
// (src/gen/sampler.cpp). The float/double mix and the operation order are part of the contract: the ids drawn
// depend on them. Parity of this restatement with the reference itself is pinned by tests that compare it, call
// for call, with oracle/_ref (the reference's own sampler.cpp compiled unmodified) and by the committed golden
// vectors generated from that library.
//
// Build: g++ -std=c++20 -O2 -ffp-contract=off (no -ffast-math, no -march=native), see oracle/Makefile.
#include "driver.hpp"

#include <map>
#include <random>
#include <stdexcept>

namespace {

class PortEngine {
public:
    // sampler.cpp:9-13
    PortEngine(const orc_params& p, uint32_t n_vocab, uint64_t seed) : p_(p), n_vocab_(n_vocab), gen_(seed)
    {
        if (n_vocab == 0)
            throw std::invalid_argument("sampler: empty vocabulary");
    }

    // sampler.cpp:15-18 — the history is a multiset: id -> number of times generated.
    void accept(int32_t token) { seen_[token] += 1u; }

    // sampler.hpp:26
    bool greedy() const { return p_.temperature <= 0.0f; }

    const std::vector<orc::Cand>& distribution(const float* logits)
    {
        // sampler.cpp:22-28 — penalties on a working copy, once per distinct generated id with its count n:
        // repetition first (divide a positive logit, multiply otherwise), then presence + frequency*n as one
        // float sum subtracted in one step.
        row_.assign(logits, logits + n_vocab_);
        const float rep = p_.repetition_penalty;
        for (const auto& kv : seen_) {
            float v = row_[size_t(kv.first)];
            if (rep != 1.0f)
                v = (v > 0.0f) ? (v / rep) : (v * rep);
            const float step = p_.presence_penalty + p_.frequency_penalty * float(kv.second);
            row_[size_t(kv.first)] = v - step;
        }
        // sampler.cpp:29 — reciprocal temperature and the row maximum (first maximum under operator<).
        const float inv_t = 1.0f / p_.temperature;
        const float top = *std::max_element(row_.begin(), row_.end());
        // sampler.cpp:30-36 — unnormalised weight q = expf((l - max) * inv_t); keep q >= min(min_p, 1) and q > 0,
        // ascending id.
        const float floor_q = std::min(p_.min_p, 1.0f);
        cand_.clear();
        for (uint32_t i = 0; i < n_vocab_; ++i) {
            const float q = expf((row_[i] - top) * inv_t);
            if (q >= floor_q && q > 0.0f)
                cand_.emplace_back(q, int32_t(i));
        }
        // sampler.cpp:37-38 — nothing finite left: the first maximum alone with weight 1.
        if (cand_.empty())
            cand_.emplace_back(1.0f, int32_t(std::max_element(row_.begin(), row_.end()) - row_.begin()));
        auto better = [](const orc::Cand& a, const orc::Cand& b) {
            return a.first > b.first || (a.first == b.first && a.second < b.second);
        };
        // sampler.cpp:39-43 — top_k keeps the k best under (q desc, id asc). The reference leaves them in
        // nth_element's order; here they are left sorted (the set is the same).
        const bool cut_k = p_.top_k > 0 && size_t(p_.top_k) < cand_.size();
        if (cut_k) {
            std::sort(cand_.begin(), cand_.end(), better);
            cand_.resize(p_.top_k);
        }
        // sampler.cpp:44-61 — top_p: double total over the current candidates, want = top_p * total, shortest
        // sorted prefix whose double running sum reaches want, at least one.
        if (p_.top_p < 1.0f) {
            double total = 0.0;
            for (const orc::Cand& c : cand_)
                total += double(c.first);
            const double want = double(p_.top_p) * total;
            if (!cut_k)
                std::sort(cand_.begin(), cand_.end(), better);
            double run = 0.0;
            size_t n = 0;
            while (n < cand_.size() && run < want)
                run += double(cand_[n++].first);
            cand_.resize(std::max<size_t>(n, 1));
        }
        return cand_;
    }

    // sampler.cpp:64-84 with the generator draw of libstdc++: uniform_real_distribution<float>(0,total) is
    // generate_canonical<float,24>(gen) * total, one 64-bit draw.
    int32_t sample_own_rng(const float* logits)
    {
        if (greedy())
            return orc::first_argmax(logits, n_vocab_);
        const std::vector<orc::Cand>& c = distribution(logits);
        const float total = orc::float_total(c);
        const float u = std::generate_canonical<float, std::numeric_limits<float>::digits>(gen_);
        return c[orc::walk(c, u * total)].second;
    }

private:
    orc_params p_;
    uint32_t n_vocab_;
    std::mt19937_64 gen_;
    std::map<int32_t, uint32_t> seen_;
    std::vector<float> row_;
    std::vector<orc::Cand> cand_;
};

// Driver<>::sample sorts nothing itself; the engine's list is already in draw order (sorted whenever a
// truncation sorted it, ascending id otherwise).

} // namespace

ORC_EXPORT_API(PortEngine, "port")
