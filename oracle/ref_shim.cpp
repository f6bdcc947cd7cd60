// TEST INFRASTRUCTURE — not part of the product.
//
// Driver around the reference's own sampler: this file is compiled together with the reference's
// src/gen/sampler.cpp, taken unmodified from where the reference checkout lies (see oracle/Makefile), into
// oracle/_ref/. No reference source is copied. The reference class keeps distribution() and its candidate list
// private, so the header is included with `private` opened up — in this translation unit only; sampler.cpp itself
// is compiled as it is, and the class layout does not depend on access specifiers.
#include "driver.hpp"

#include <random>
#include <unordered_map>

#define private public
#include "gen/sampler.hpp"
#undef private

namespace {

class RefEngine {
public:
    RefEngine(const orc_params& p, uint32_t n_vocab, uint64_t seed)
        : top_k_only_(p.top_k > 0 && !(p.top_p < 1.0f)),
          s_(mako::gen::SamplingParams{p.temperature, p.top_k, p.top_p, p.min_p, p.presence_penalty,
                                       p.frequency_penalty, p.repetition_penalty},
             n_vocab, seed)
    {
    }
    void accept(int32_t token) { s_.accept(token); }
    bool greedy() const { return s_.greedy(); }
    const std::vector<orc::Cand>& distribution(const float* logits)
    {
        s_.distribution(logits);
        // top_k without top_p leaves nth_element's order (src/gen/sampler.cpp:41): canonical order is sorted.
        if (top_k_only_)
            std::sort(s_.cand_.begin(), s_.cand_.end(), [](const orc::Cand& a, const orc::Cand& b) {
                return a.first > b.first || (a.first == b.first && a.second < b.second);
            });
        return s_.cand_;
    }
    int32_t sample_own_rng(const float* logits) { return s_.sample(logits); }

private:
    bool top_k_only_;
    mako::gen::Sampler s_;
};

} // namespace

ORC_EXPORT_API(RefEngine, "reference")
