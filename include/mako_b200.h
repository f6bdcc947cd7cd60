/*
 * mako_b200 — C ABI of the B200 (sm_100a) token sampler.
 *
 * A drop-in for the token-sampling path of jhanssen/mako: what the reference does one row at a time on the host in
 * mako::gen::Sampler (src/gen/sampler.hpp:22-45, src/gen/sampler.cpp:9-107) is done here for a batch of rows on the
 * GPU, with results (candidate sets, token ids) identical to the reference on the same logits, history and
 * uniforms. Plain C types only; every pointer documented as "device" is a CUDA device pointer of the handle's
 * device, `stream` is a cudaStream_t passed as void*. No function throws; each returns an mk_status and leaves a
 * message for mk_last_error() (thread-local) on failure.
 *
 * Order of operations on a row (reference: src/gen/sampler.hpp:11, sampler.cpp:20-62):
 *   logit bias (+=)  ->  allowed-token mask (-inf)  ->  repetition / presence / frequency penalties over the
 *   token history  ->  temperature  ->  min_p  ->  top_k  ->  top_p  ->  draw by inverse CDF with the caller's u.
 * Bias and mask have no counterpart in the reference; they act on the logits before the reference pipeline sees
 * them. A masked token stays excluded whatever the penalties do to it.
 */
#ifndef MAKO_B200_H
#define MAKO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mk_status {
    MK_OK = 0,
    MK_ERR_INVALID_ARGUMENT = 1, /* the reference throws std::invalid_argument (sampler.cpp:11-12) */
    MK_ERR_CUDA = 2,
    MK_ERR_UNSUPPORTED = 3,
    MK_ERR_NO_DEVICE = 4
} mk_status;

/* Per-row result flags (bit set). */
#define MK_FLAG_NEAR_CDF_BOUNDARY 0x001u /* u*total within 1e-6*total of a CDF boundary beside the chosen token */
#define MK_FLAG_GUARD_BAND        0x002u /* a keep/drop decision fell inside the numeric guard band */
#define MK_FLAG_NO_CANDIDATE      0x004u /* nothing finite survived: first argmax returned (sampler.cpp:37-38) */
#define MK_FLAG_ALL_MASKED        0x008u /* the mask allowed no token of this row */
#define MK_FLAG_OVERFLOW          0x010u /* more candidates than the handle's capacity: token = -1 */
#define MK_FLAG_VP_TRUNCATED      0x020u /* vocab-parallel: the nucleus may reach past a shard's top-k list */
#define MK_FLAG_TIMEOUT           0x040u /* a bounded device-side wait ran out: token = -1 */
#define MK_FLAG_HISTORY_FULL      0x100u /* mk_decode_commit: the row's history buffer is full, the token was not appended;
                                           sampling: history_len[b] exceeded min(history_ld, 65535) and was clamped to it */

/* Field for field mako::gen::SamplingParams (src/gen/sampler.hpp:12-20). temperature <= 0 selects greedy. */
typedef struct mk_sampling_params {
    float temperature;
    uint32_t top_k;
    float top_p;
    float min_p;
    float presence_penalty;
    float frequency_penalty;
    float repetition_penalty;
} mk_sampling_params;

/* Sparse logit bias entry; id < 0 marks an unused slot. Ids of one row must be distinct. */
typedef struct mk_bias {
    int32_t id;
    float value;
} mk_bias;

/* A batch of rows. Row b reads logits + b*ld (n_vocab floats), history + b*history_ld, mask + b*mask_ld (words),
 * bias + b*n_bias. The fast (bulk-copy) path needs logits 16-byte aligned and ld % 4 == 0; other layouts take a
 * slower path with identical results (about ten times the time per row: pad the rows to a multiple of four columns
 * and keep the buffer 16-byte aligned). */
typedef struct mk_rows {
    const float* logits;         /* device [batch][ld] fp32 — the row Sampler::sample is handed (sampler.hpp:27) */
    uint64_t ld;
    uint32_t batch;
    uint32_t n_vocab;            /* columns held here (the whole vocabulary, or one shard of it) */
    int32_t id_offset;           /* token id of column 0 (vocab-parallel shards), else 0 */
    uint32_t n_history;          /* history entries per row when history_len == NULL; <= 65535 */
    const int32_t* history;      /* device [batch][history_ld] generated-token ids = accept() calls (sampler.cpp:15-18) */
    uint64_t history_ld;
    const int32_t* history_len;  /* device [batch] or NULL; a value above min(history_ld, 65535) is clamped to it
                                    and reported as MK_FLAG_HISTORY_FULL */
    const uint32_t* mask;        /* device [batch][mask_ld]; bit id%32 of word id/32 set = allowed; NULL = all */
    uint64_t mask_ld;
    const mk_bias* bias;         /* device [batch][n_bias] or NULL */
    uint32_t n_bias;
    const mk_sampling_params* params_dev; /* device [batch] per-row parameters, or NULL to use `params` */
    mk_sampling_params params;
} mk_rows;

/* Per-row outputs (device). Only token is mandatory. cand_* receive the surviving candidates in draw order. */
typedef struct mk_sample_out {
    int32_t* token;     /* [batch] */
    float* prob;        /* [batch] probability of the chosen token = q / total (float) */
    uint32_t* flags;    /* [batch] MK_FLAG_* */
    uint32_t* n_cand;   /* [batch] number of surviving candidates */
    int32_t* cand_ids;  /* [batch][cand_cap] */
    float* cand_q;      /* [batch][cand_cap] unnormalised weights q (sampler.cpp:33) */
    uint32_t cand_cap;
} mk_sample_out;

typedef struct mk_sampler mk_sampler;

/* Library / build information: "mako_b200 <version> sm_100a". */
const char* mk_version(void);
/* Message of the last failure on this thread. */
const char* mk_last_error(void);

/* Replaces Sampler::Sampler(params, n_vocab, seed) (sampler.cpp:9-13) for a batch: allocates the handle's scratch
 * for up to max_batch rows of at most n_vocab columns on `device` — candidate lists of 16 * n_vocab bytes a row,
 * twice (the two row sets of mk_sampler_verify_pq_batch run side by side), and 64 KB of candidate lists a row for
 * that call's two distributions: about 5 MB a row at 151,552 columns. n_vocab == 0 is MK_ERR_INVALID_ARGUMENT, as the
 * reference throws. Nothing is allocated after this call. */
int mk_sampler_create(mk_sampler** out, int device, uint32_t n_vocab, uint32_t max_batch);
void mk_sampler_destroy(mk_sampler* s);

/* The same checks the reference applies upstream of the sampler (src/server/openai.cpp:316-328): all finite,
 * temperature 0 or >= 1e-3, repetition_penalty in (0, 100], |presence|, |frequency| <= 100. */
int mk_check_sampling(const mk_sampling_params* p);

/* No counterpart in the reference (its sampler runs on the host, between two engine steps). How the row kernel of
 * this handle's sample / verify calls is launched behind the kernel that precedes it in the stream:
 *   MK_OVERLAP_OFF                 plain stream order (the default);
 *   MK_OVERLAP_LAUNCH              programmatic dependent launch: the kernel's CTAs may be scheduled while the
 *                                  previous kernel drains, and wait for its completion before they touch any memory.
 *                                  Always safe; hides the launch gap;
 *   MK_OVERLAP_STABLE_SIDE_INPUTS  the same, and the caller promises that the previous kernel in the stream writes
 *                                  none of params_dev, history, history_len and bias of the call: the kernel then
 *                                  builds its per-row history tables before it waits, so that only streaming the
 *                                  logits is left once the previous kernel (the one that produces the logits, or the
 *                                  previous sample call) has finished. Logits, mask, uniforms and drafts are read,
 *                                  and everything is written, after the wait. */
#define MK_OVERLAP_OFF 0
#define MK_OVERLAP_LAUNCH 1
#define MK_OVERLAP_STABLE_SIDE_INPUTS 2
int mk_sampler_set_overlap(mk_sampler* s, int mode);

/* No counterpart in the reference. A sample call of at most 8 rows with one shared parameter set that draws
 * (temperature > 0) under 1 <= top_k <= 64 leaves the device idle as one CTA per row, so by default it runs as three
 * launches instead: every row's columns split over up to 64 CTAs that each write the record of a vocabulary shard,
 * the merge of mk_sampler_vp_merge over the records, and a launch of the one-CTA-per-row kernel that returns at once
 * for every row except those the merge flagged MK_FLAG_VP_TRUNCATED. Same tokens, probabilities and candidate lists
 * as the plain path. on = 0 makes every batch run as one CTA per row. */
int mk_sampler_set_split(mk_sampler* s, int on);

/* Replaces Sampler::sample (sampler.cpp:75-84) for rows->batch rows: u[b] in [0,1) is the uniform the reference
 * would draw from its generator (r = u * total, sampler.cpp:66). One kernel, one pass over the logits. */
int mk_sampler_sample_batch(mk_sampler* s, const mk_rows* rows, const float* u, const mk_sample_out* out,
                            void* stream);

/* No counterpart in the reference. mk_sampler_sample_batch for callers that must not allocate device memory — code
 * that runs inside someone else's memory plan (an inference server that hands every byte out at start-up, a plugin
 * loaded into a process whose allocator it may not touch) or at a point where cudaMalloc is off limits — and so
 * cannot create an mk_sampler, whose scratch is cudaMalloc'ed. Same inputs, same outputs, same results; the kernel's
 * candidate scratch is a fixed array inside the library instead (about 20 MiB on each GPU that loads the library,
 * kept until the process exits). Limits: at most MK_STATIC_MAX_ROWS rows per call and MK_STATIC_MAX_VOCAB columns;
 * larger arguments return MK_ERR_INVALID_ARGUMENT. The call itself allocates nothing. The first call on a device
 * also looks up the array's device address; make that first call before any stream capture begins. All calls on a
 * device share the one array: two calls that overlap on the GPU (different streams, or different host threads)
 * race on it — run them one after the other. */
#define MK_STATIC_MAX_ROWS 8u
#define MK_STATIC_MAX_VOCAB 163840u
int mk_sample_rows_static(int device, const mk_rows* rows, const float* u, const mk_sample_out* out, void* stream);

/* Replaces Sampler::verify (sampler.cpp:86-107) for rows->batch (sequence, position) rows with deterministic
 * drafts: draft[b] is accepted iff u_accept[b]*total < q(draft); else the draft is removed and a token is drawn
 * with u_redraw[b]. accepted[b] is 0/1, out->token[b] the returned token. */
int mk_sampler_verify_batch(mk_sampler* s, const mk_rows* rows, const int32_t* draft, const float* u_accept,
                            const float* u_redraw, const mk_sample_out* out, int32_t* accepted, void* stream);

/* Rejection sampling against a drafter distribution (generalises Sampler::verify, which is the one-hot case):
 * rows describe the target logits p; draft_logits [batch][draft_ld] the drafter's q (same history, mask, bias and
 * parameters). The draft token is drawn from q with u_draft, accepted iff u_accept*q(d) < p(d), else redrawn from
 * max(0, p - q) with u_resample. */
int mk_sampler_verify_pq_batch(mk_sampler* s, const mk_rows* rows, const float* draft_logits, uint64_t draft_ld,
                               const float* u_draft, const float* u_accept, const float* u_resample,
                               int32_t* draft_token, int32_t* accepted, int32_t* token, uint32_t* flags,
                               void* stream);

/* The acceptance loop of the reference's speculative round (src/gen/session.cpp:481-496,505) over per-position
 * results laid out [n_seq][n_pos] (n_pos - 1 drafted positions then the bonus position): n_kept[s] = drafts kept
 * up to the first rejection, next_token[s] = the replacement at the first rejection, or the bonus position's token
 * if every draft was kept. */
int mk_spec_resolve(mk_sampler* s, uint32_t n_seq, uint32_t n_pos, const int32_t* accepted, const int32_t* token,
                    int32_t* n_kept, int32_t* next_token, void* stream);

/* One whole speculative round of the reference (src/gen/session.cpp:451-506) for rows->batch / n_pos sequences in
 * one launch. rows->logits holds n_pos rows per sequence — row s*n_pos + j is the distribution after the round's
 * token and drafts 0..j-1 (what Model::verify returns, src/gen/model.hpp:84-88) — while rows->history / history_len
 * are per SEQUENCE (row s): the tokens accept()ed so far, the round's first token included. Position j < n_pos - 1
 * verifies drafts[s][j] exactly as Sampler::verify would after the drafts before it were accepted: its penalties
 * count history + drafts[s][0..j-1] (each kept draft is emit()ted before the next row is looked at, :491). The last
 * position is the bonus row and is sampled (:505). forced[s][j] >= 0 (optional array) is the caller's forced token for
 * that position: it takes the sampler's place without drawing, and a draft is kept only if it equals it (:481-484).
 * u[s][0..n_pos] is the sequence's stream of uniforms in the order the reference's generator would produce them: a
 * position takes the next one for its acceptance test (or its draw, for the bonus row) and the one after it for the
 * redraw after a rejection; forced positions take none. Outputs: accepted / out->token per position as
 * mk_sampler_verify_batch gives them, n_kept[s] = drafts kept up to the first rejection, next_token[s] = the
 * replacement there, or the bonus row's token when every draft was kept — what Session::run carries into its next
 * round. Positions after the first rejection are computed too and ignored, as positions of one launch must be. */
int mk_sampler_spec_round(mk_sampler* s, const mk_rows* rows, uint32_t n_pos, const int32_t* drafts,
                          const int32_t* forced, const float* u, const mk_sample_out* out, int32_t* accepted,
                          int32_t* n_kept, int32_t* next_token, void* stream);

/* The round's bookkeeping on the device: the kept drafts and then next_token[s] are appended to the sequence's
 * history (the accept() calls of :420 for each emit(), the last one made at the top of the reference's next round),
 * history_len[s] grows by n_kept[s] + 1, next_input[s] (optional) receives next_token[s]. A sequence whose round
 * failed (next_token < 0) is left alone; a full history sets MK_FLAG_HISTORY_FULL in flags[s] (optional). */
int mk_spec_commit(mk_sampler* s, uint32_t n_seq, uint32_t n_pos, const int32_t* drafts, const int32_t* n_kept,
                   const int32_t* next_token, int32_t* history, uint64_t history_ld, uint32_t history_cap,
                   int32_t* history_len, int32_t* next_input, uint32_t* flags, void* stream);

/* One step of the reference's drafter pick (ds_markov + ds_draft_pick, src/kernels/dsv41.metal:664-742; host loop
 * src/dsv41/engine.cpp:1474-1497) for up to 8 sequences that share the drafter: per sequence b,
 * score[v] = logits[b][v] + head[v] . embed[prev[b]] (head [n_vocab][rank], 16-byte aligned; embed [n_embed][rank]; rank a multiple of 4, <= 256),
 * draft[b] = argmax_v score[v], the lowest id on ties (id 0 when no score is above -inf), and
 * conf[b] = 1 / (1 + exp(-([x[b], embed[prev[b]]] . w))) with x [n_seq][x_ld] (dim used) and w [dim + rank].
 * prev[b] is the previous draft of the chain (or the last sampled token at step 0); the caller runs the chain's steps
 * one call after the other, as the reference does. The scores are not written anywhere. Floating point: dot products
 * are summed in another order than the reference's simdgroup reduction — scores agree to about 1e-6 relative, so
 * the argmax is the reference's unless the two best scores are that close. All pointers are device pointers. Calls on
 * one handle must not overlap (they share the handle's maxima and ticket counter); use one handle per stream. */
int mk_draft_pick(mk_sampler* s, const float* logits, uint64_t ld, const float* head, const float* embed, const float* x,
                  uint64_t x_ld, const float* w, const int32_t* prev, uint32_t n_seq, uint32_t n_vocab, uint32_t rank,
                  uint32_t dim, uint32_t n_embed, int32_t* draft, float* conf, void* stream);

/* The reference's other drafter pick (hy4_draft_pick, src/kernels/hy4f.metal:352-397), per sequence b:
 * draft[b] = index of the largest logit (the lowest index on ties; 0 when nothing is above -inf), also written to
 * next_prev[b] (optional: the next step's embedding index), conf[b] = 1 / (1 + exp(-(conf_w . h[b] + conf_bias)))
 * over `width` floats. logits [n_seq][ld], h [n_seq][h_ld]. All pointers are device pointers. */
int mk_draft_pick_plain(mk_sampler* s, const float* logits, uint64_t ld, uint32_t n_seq, uint32_t n_vocab, const float* h,
                        uint64_t h_ld, const float* conf_w, uint32_t width, float conf_bias, int32_t* draft, float* conf,
                        int32_t* next_prev, void* stream);

/* The logit test of the reference's reasoning budget (ReasoningBudget::forced, src/server/openai.cpp:596-603): in
 * the budget's last stretch the closing token is forced as soon as it is among the k = 3 largest raw logits. Per row
 * b: above[b] = number of logits[b][i] strictly greater than logits[b][token[b]] (NaN never counts), forced[b] =
 * token[b] if above[b] < k, else -1; a token[b] outside [0, n_vocab) forces nothing (forced -1, above 0xffffffff).
 * `forced` feeds mk_decode_commit directly; either output may be NULL. The budget's counters (which rows are in the
 * last stretch) stay with the caller: rows not in it pass token -1. All pointers are device pointers; one streaming
 * pass over the rows (4 bytes per column). */
int mk_rank_force(mk_sampler* s, const float* logits, uint64_t ld, uint32_t batch, uint32_t n_vocab,
                  const int32_t* token, uint32_t k, int32_t* forced, uint32_t* above, void* stream);

/* The bookkeeping of the reference's decode loop (src/gen/session.cpp:416-444) on the device, so that a step needs
 * no host round trip between the sampler and the next forward pass. Per row b: token = forced[b] if `forced` is given
 * and forced[b] >= 0 (the reference bypasses the sampler for a forced token — tool_choice, the reasoning budget,
 * src/gen/session.hpp:43-45 — without drawing, but still accept()s it), else sampled[b]. The token is written to
 * committed[b] and next_input[b] (both optional: the next step's input id) and appended to the row's history,
 * history[b][history_len[b]++] — what Sampler::accept does (sampler.cpp:15-18); the next sample call reads the same
 * buffers through mk_rows.history / history_len. A row whose history is full keeps its length and gets
 * MK_FLAG_HISTORY_FULL or-ed into flags[b] (optional); a sampled token < 0 (a failed row) is not committed.
 * history_cap is at most 65535 (the sampler counts a token's occurrences in 16 bits). All pointers are device
 * pointers. */
int mk_decode_commit(mk_sampler* s, uint32_t batch, const int32_t* sampled, const int32_t* forced, int32_t* history,
                     uint64_t history_ld, uint32_t history_cap, int32_t* history_len, int32_t* next_input,
                     int32_t* committed, uint32_t* flags, void* stream);

/* Vocab-parallel sampling, step 1 of 2 (no counterpart in the reference, which runs on one device): each shard
 * writes one record per row — its maximum, its sum of exp((l - max)/T) and its `k` best candidates (<= 64) — of
 * mk_vp_record_bytes(k) bytes. The caller all-gathers the records of all shards ([n_shards][batch] records,
 * e.g. ncclAllGather) and calls mk_sampler_vp_merge on every rank (or one). */
uint32_t mk_vp_record_bytes(uint32_t k);
int mk_sampler_vp_local(mk_sampler* s, const mk_rows* shard_rows, uint32_t k, void* records, void* stream);
/* Shard g of the gathered records must hold columns that all lie below shard g+1's (any widths, equal or not);
 * n_vocab_total <= 2^26. */
int mk_sampler_vp_merge(mk_sampler* s, const void* gathered, uint32_t n_shards, uint32_t batch, uint32_t k,
                        uint32_t n_vocab_total, const mk_sampling_params* params, const float* u,
                        const mk_sample_out* out, void* stream);

/* Host-buffer form of mk_sampler_sample_batch — what the reference's caller has (Sampler::sample takes a host
 * row, sampler.hpp:27): every pointer in rows/u/out is a HOST pointer (pinned memory overlaps best); the call
 * copies inputs to device staging owned by the handle, runs the kernel, copies results back and synchronises. */
int mk_sampler_sample_host(mk_sampler* s, const mk_rows* host_rows, const float* u, const mk_sample_out* host_out);

/* The reference's own object, one row at a time with its own state: replaces mako::gen::Sampler
 * (src/gen/sampler.hpp:22-45) call for call. Keeps the parameters, the generated-token history (accept,
 * sampler.cpp:15-18) and a std::mt19937_64 seeded like the reference's, from which it takes the same uniforms in
 * the same order: one per sample(), one per verify() plus one more after a rejection, none when greedy. With the
 * same seed the token stream is the reference's, with one exception: top_k truncating (more candidates than top_k)
 * and top_p >= 1. There the reference
 * walks its candidates in the order std::nth_element happened to leave them (sampler.cpp:41, 64-73), which no
 * specification fixes; this library walks them sorted by (weight descending, id ascending). The candidate set and
 * every probability are the same, the draw order is not, so the streams differ in that one case. `logits`
 * may be a host pointer (copied, as the reference's callers hold host rows) or a device pointer (read in place).
 * include/mako_b200/sampler.hpp wraps these five calls in a C++ class with the reference's signatures. */
typedef struct mk_row_sampler mk_row_sampler;
int mk_row_sampler_create(mk_row_sampler** out, const mk_sampling_params* p, uint32_t n_vocab, uint64_t seed,
                          int device);
void mk_row_sampler_destroy(mk_row_sampler* r);
int mk_row_sampler_greedy(const mk_row_sampler* r);
int mk_row_sampler_accept(mk_row_sampler* r, int32_t token);
int mk_row_sampler_sample(mk_row_sampler* r, const float* logits, int32_t* token);
int mk_row_sampler_verify(mk_row_sampler* r, const float* logits, int32_t draft, int32_t* accepted, int32_t* token);

/* Test hook: y[i] = the device's float exponential of x[i] (device pointers), which must equal the host C
 * library's expf bit for bit (the reference calls std::exp(float), sampler.cpp:33). */
int mk_debug_expf(const float* x_dev, float* y_dev, uint64_t n, void* stream);

/* Profiling hook: when timing_dev (device, [max_batch][64] uint64) is non-NULL, each row's CTA of the following
 * sample/verify launches stores %globaltimer nanosecond stamps: [0] start, [1] set-up done, [2] last tile requested,
 * [3] end; inside the set-up [6] memory cleared, [7] bitmap, [8] ranks, [4] counts, [5] first tiles landed; inside
 * the finish [11] candidates filtered ([9] collected, [10] kept: counts, not times), [12] ordered, [13] top_p done. */
int mk_debug_set_timing(mk_sampler* s, unsigned long long* timing_dev);

/* Test hook for the bounded waits: the following sample / verify launches of this handle never request the copy of
 * tile `tile` (4096 columns each) of any row, and a wait for a tile gives up after `wait_probes` probes of up to
 * 20 us each instead of after seconds. Every wait in the kernel is bounded: the waits for the missing tile run out,
 * the row's CTA leaves in good order and the row reports token -1 with MK_FLAG_TIMEOUT — no trap, no hang, the
 * context stays usable. tile < 0 switches the hook off (and wait_probes 0 restores the default limit). */
int mk_debug_withhold_tile(mk_sampler* s, int tile, uint32_t wait_probes);

/* Bytes the roofline counts for one row: logits once + history + mask + bias + uniforms + outputs. */
uint64_t mk_row_bytes(uint32_t n_vocab, uint32_t n_history, int has_mask, uint32_t n_bias, uint32_t n_uniforms);

#ifdef __cplusplus
}
#endif
#endif
