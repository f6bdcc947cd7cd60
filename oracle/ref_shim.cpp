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
        // top_k without top_p, when it truncates, leaves nth_element's order (src/gen/sampler.cpp:41): canonical order
        // is sorted. When no more than top_k candidates exist nothing is reordered there (ascending id, :30-36) and
        // nothing is here. A list of exactly top_k entries may be either: the candidates are counted again from the
        // sampler's own edited logits, with its expressions (:29-35).
        if (top_k_only_ && s_.cand_.size() == size_t(s_.p_.top_k)) {
            const float inv_t = 1.0f / s_.p_.temperature, m = *std::max_element(s_.work_.begin(), s_.work_.end());
            size_t n_before = 0;
            for (const float l : s_.work_) {
                const float q = std::exp((l - m) * inv_t);
                if (q >= std::min(s_.p_.min_p, 1.0f) && q > 0.0f)
                    ++n_before;
            }
            if (n_before > s_.cand_.size())
                std::sort(s_.cand_.begin(), s_.cand_.end(), [](const orc::Cand& a, const orc::Cand& b) {
                    return a.first > b.first || (a.first == b.first && a.second < b.second);
                });
        }
        return s_.cand_;
    }
    int32_t sample_own_rng(const float* logits) { return s_.sample(logits); }

private:
    bool top_k_only_;
    mako::gen::Sampler s_;
};

} // namespace

ORC_EXPORT_API(RefEngine, "reference")
