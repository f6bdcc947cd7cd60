/*
 * TEST INFRASTRUCTURE — not part of the product.
 *
 * C interface shared by the two CPU checkers of the token-sampling path:
 *   - sampler_port.cpp : a CPU restatement of the reference sampler (kind "port"), builds anywhere;
 *   - ref_shim.cpp     : a thin driver around the reference's own, unmodified src/gen/sampler.cpp
 *                        (kind "reference"), built only where the reference sources are present.
 * Both export exactly these symbols, so a test can load either and compare them call for call.
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may load these libraries.
 *
 * Semantics every function follows (reference: src/gen/sampler.cpp:20-107):
 *   row pre-processing (absent from the reference, defined here): logit += bias for each (id, value) pair,
 *   then logit = -inf where the packed mask bit (bit id%32 of word id/32) is 0; the result is what the
 *   reference sampler is handed. History ids are replayed through accept() (sampler.cpp:15-18).
 *   A caller-supplied uniform u in [0,1) replaces the reference's own generator draw: the reference computes
 *   r = uniform_real_distribution<float>(0,total)(rng) = u * total (sampler.cpp:66,100), here u is given.
 *   With top_k active and top_p >= 1 the reference's candidate order, when top_k truncates, is whatever
 *   nth_element leaves (sampler.cpp:41); both checkers sort that case by (q descending, id ascending) before
 *   drawing. When no more than top_k candidates exist the list stays in ascending id, as in the reference.
 */
#ifndef MAKO_ORACLE_API_H
#define MAKO_ORACLE_API_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Field for field the reference's SamplingParams (src/gen/sampler.hpp:12-20). */
typedef struct orc_params {
    float temperature;
    uint32_t top_k;
    float top_p;
    float min_p;
    float presence_penalty;
    float frequency_penalty;
    float repetition_penalty;
} orc_params;

/* One row of input. Pointers may be NULL when the matching count is 0 / the mask is absent. */
typedef struct orc_row {
    uint32_t n_vocab;
    const float* logits;
    const int32_t* history;
    uint32_t n_history;
    const uint32_t* mask;
    const int32_t* bias_ids;
    const float* bias_vals;
    uint32_t n_bias;
} orc_row;

/* "port" or "reference". */
const char* orc_kind(void);

/* sample(): token, its probability q/total, and the surviving candidates in draw order (up to cap).
 * near_boundary (nullable) is set to 1 when u*total lies within 1e-6*total of a CDF boundary next to the
 * chosen candidate. Returns 0, or -1 on a bad argument (n_vocab == 0). */
int orc_sample(const orc_params* p, const orc_row* row, float u, int32_t* token, float* prob, uint32_t* n_cand,
               int32_t* cand_ids, float* cand_q, uint32_t cap, uint32_t* near_boundary);

/* verify() of a deterministic draft (sampler.cpp:86-107): u1 decides acceptance, u2 the redraw. */
int orc_verify(const orc_params* p, const orc_row* row, int32_t draft, float u1, float u2, int32_t* token,
               int32_t* accepted);

/* General rejection sampling against a drafter distribution (no counterpart in the reference; built from two
 * distribution() calls): the draft token is drawn from the drafter row with u_draft, accepted iff
 * u_accept * q(d) < p(d) on the normalised probabilities, else redrawn from max(0, p - q) over the union of both
 * candidate sets in ascending id with u_resample (the draft itself if that residual is all zero). */
int orc_verify_pq(const orc_params* p, const orc_row* target, const orc_row* drafter, float u_draft, float u_accept,
                  float u_resample, int32_t* draft_token, int32_t* accepted, int32_t* token);

/* The reference's own generator path: n draws of sample() from one sampler seeded with `seed`
 * (std::mt19937_64, one 64-bit draw per call). Used to pin the u-driven path to the unmodified one. */
int orc_sample_rng(const orc_params* p, const orc_row* row, uint64_t seed, uint32_t n_draws, int32_t* tokens);

/* The uniforms libstdc++'s uniform_real_distribution<float> takes from std::mt19937_64(seed), one 64-bit draw
 * each: what the reference multiplies `total` with (sampler.cpp:66). */
void orc_uniforms(uint64_t seed, uint32_t n, float* out);

/* Times sample() over a batch of rows spread over n_threads host threads; sampler construction, the history
 * replay and one untimed pass over the batch (which sizes each sampler's work vectors, as the first token of a
 * request does) are outside the timed region, bias/mask pre-processing is inside. Rows share params; row b reads
 * logits + b*ld, history + b*n_history, mask + b*mask_ld, bias + b*n_bias, u[b]. Returns seconds, <0 on error. */
double orc_time_sample_batch(const orc_params* p, uint32_t batch, uint32_t n_vocab, const float* logits, uint64_t ld,
                             const int32_t* history, uint32_t n_history, const uint32_t* mask, uint64_t mask_ld,
                             const int32_t* bias_ids, const float* bias_vals, uint32_t n_bias, const float* u,
                             uint32_t n_threads, int32_t* tokens);

#ifdef __cplusplus
}
#endif
#endif
