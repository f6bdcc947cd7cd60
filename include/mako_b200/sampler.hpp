// C++ face of the library with the reference's own signatures: a replacement for mako::gen::SamplingParams and
// mako::gen::Sampler (src/gen/sampler.hpp:12-45). Header-only over the C ABI in mako_b200.h; link libmako_b200.so.
//
//   reference                                  here
//   Sampler(params, n_vocab, seed)             same; throws std::invalid_argument for n_vocab == 0 (sampler.cpp:11-12)
//   bool greedy() const                        same
//   int32_t sample(const float* logits)        same; `logits` may be a host pointer (as in the reference: the engine's
//                                              std::vector<float>) or a device pointer (read in place, no copy)
//   int32_t verify(logits, draft, accepted)    same
//   void accept(int32_t token)                 same
//
// State, threading and generator follow the reference: one object per request, not thread-safe, a std::mt19937_64
// seeded with `seed` that yields one uniform per sample(), one per verify() plus one more after a rejection, none
// when greedy — so a session that swaps this class in draws the same tokens as before for the same seed. The one
// exception is top_k truncating (more candidates than top_k) with top_p >= 1: the reference then walks its candidates
// in whatever order std::nth_element left them (sampler.cpp:41, 64-73), this class in sorted order (weight
// descending, id ascending).
// Candidate set and probabilities are identical; the seeded token stream is not.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>

#include "../mako_b200.h"

namespace mako_b200::gen {

// Applied in this order: penalties, temperature, min_p, top_k, top_p (src/gen/sampler.hpp:11).
struct SamplingParams {
    float temperature = 1.0f; // <= 0: greedy
    uint32_t top_k = 0;       // 0: no limit
    float top_p = 1.0f;
    float min_p = 0.0f;
    float presence_penalty = 0.0f, frequency_penalty = 0.0f;
    float repetition_penalty = 1.0f;
};

class Sampler {
public:
    Sampler(const SamplingParams& p, uint32_t n_vocab, uint64_t seed, int device = 0) : p_(p)
    {
        if (n_vocab == 0)
            throw std::invalid_argument("sampler: empty vocabulary");
        const mk_sampling_params c{p.temperature,      p.top_k,           p.top_p,           p.min_p,
                                   p.presence_penalty, p.frequency_penalty, p.repetition_penalty};
        const int rc = mk_row_sampler_create(&h_, &c, n_vocab, seed, device);
        if (rc == MK_ERR_INVALID_ARGUMENT)
            throw std::invalid_argument(mk_last_error());
        if (rc != MK_OK)
            throw std::runtime_error(std::string("mako_b200: ") + mk_last_error());
    }
    ~Sampler() { mk_row_sampler_destroy(h_); }
    Sampler(const Sampler&) = delete;
    Sampler& operator=(const Sampler&) = delete;
    Sampler(Sampler&& o) noexcept : p_(o.p_), h_(o.h_) { o.h_ = nullptr; }

    bool greedy() const { return p_.temperature <= 0.0f; }

    int32_t sample(const float* logits)
    {
        int32_t token = -1;
        check(mk_row_sampler_sample(h_, logits, &token));
        return token;
    }

    int32_t verify(const float* logits, int32_t draft, bool& accepted)
    {
        int32_t token = -1, acc = 0;
        check(mk_row_sampler_verify(h_, logits, draft, &acc, &token));
        accepted = acc != 0;
        return token;
    }

    void accept(int32_t token) { check(mk_row_sampler_accept(h_, token)); }

private:
    static void check(int rc)
    {
        if (rc != MK_OK)
            throw std::runtime_error(std::string("mako_b200: ") + mk_last_error());
    }
    SamplingParams p_;
    mk_row_sampler* h_ = nullptr;
};

} // namespace mako_b200::gen
