// Host-visible declarations of the row pipeline kernels (internal to the library; the public surface is
// include/mako_b200.h).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/mako_b200.h"

namespace mk {

enum RowMode : int {
    kModeSample = 0,   // Sampler::sample
    kModeVerify = 1,   // Sampler::verify with a deterministic draft
    kModeDistOnly = 2, // candidate list only (target side of p/q verification)
    kModeVpLocal = 3   // vocab-parallel shard record
};

struct RowKernelArgs {
    // inputs
    const float* logits;
    uint64_t ld;
    uint32_t n_vocab;
    int32_t id_offset;
    const int32_t* history;
    uint64_t history_ld;
    const int32_t* history_len;
    uint32_t n_history;
    const uint32_t* mask;
    uint64_t mask_ld;
    const mk_bias* bias;
    uint32_t n_bias;
    const mk_sampling_params* params_dev;
    mk_sampling_params params;
    const float* u;        // sample: draw; verify: acceptance
    const float* u2;       // verify: redraw
    const int32_t* draft;  // verify
    // outputs
    int32_t* token;
    float* prob;
    uint32_t* flags;
    uint32_t* n_cand;
    int32_t* cand_ids;
    float* cand_q;
    uint32_t cand_cap;
    int32_t* accepted;     // verify
    float* total_out;      // optional [batch]: float total of the final list
    // vocab-parallel
    void* vp_records;
    uint32_t vp_k;
    // scratch owned by the handle
    uint32_t* scratch;     // [batch][row_scratch_words(scratch_cap)]: raw candidates (logit bits, column), then a sort buffer / a float per column
    uint32_t scratch_cap;
    unsigned long long* timing; // optional [batch][64] ns timestamps (slots: see mk_debug_set_timing)
    int mode;
    int pass;              // 0: first launch; 1: second pass, only the rows that asked for it (set by launch_row_kernel)
    int use_bulk_copy;     // 1: TMA bulk staging (aligned rows); 0: plain loads
    int overlap;           // MK_OVERLAP_*: launch behind the previous kernel of the stream programmatically
    // a speculative round: row = sequence * spec_n_pos + position (0: off); history and history_len are per sequence
    uint32_t spec_n_pos;
    const int32_t* spec_drafts; // [n_seq][spec_n_pos - 1]
    const int32_t* spec_forced; // [n_seq][spec_n_pos] forced token or -1, or NULL
    // split launch (shard records only): every row's columns in shards of split_w columns, one CTA per (row, shard);
    // records laid out [n_shards][batch]. 0: off
    uint32_t split_w;
    // follow-up launch: only rows whose flags (written by an earlier step) have one of these bits set are processed
    const uint32_t* only_flagged;
    uint32_t only_flagged_mask;
    uint32_t debug_skip_tile;   // test hook: the copy of this tile is never requested (0xffffffff: none)
    uint32_t debug_wait_probes; // test hook: probes a wait for a tile makes before it gives up (0: the default)
};

// Words of handle scratch per row: 4 per column of capacity, then 4 of per-row state (word 0: the row asks for the
// second pass).
__host__ __device__ inline size_t row_scratch_words(uint32_t cap) { return 4ull * cap + 4ull; }

size_t row_kernel_smem_bytes();
cudaError_t launch_row_kernel(const RowKernelArgs& a, uint32_t batch, cudaStream_t stream);

struct VpMergeArgs {
    const unsigned char* gathered; // [n_shards][batch] records
    uint32_t n_shards, batch, k, n_vocab_total;
    const mk_sampling_params* params_dev;
    mk_sampling_params params;
    const float* u;
    int32_t* token;
    float* prob;
    uint32_t* flags;
    uint32_t* n_cand;
    int32_t* cand_ids;
    float* cand_q;
    uint32_t cand_cap;
};
cudaError_t launch_vp_merge(const VpMergeArgs& a, cudaStream_t stream);

struct PqResolveArgs {
    uint32_t batch, cap;
    const int32_t* p_ids; const float* p_q; const uint32_t* p_n; const uint32_t* p_flags;
    const int32_t* q_ids; const float* q_q; const uint32_t* q_n; const uint32_t* q_flags;
    const float* p_total; const float* q_total; // float totals of the two lists (draw order)
    const float* q_prob;        // probability of the draft token under q
    const int32_t* draft_token; // drawn from q by the sample launch
    const float* u_accept; const float* u_resample;
    int32_t* accepted; int32_t* token; uint32_t* flags;
    uint32_t n_vocab; int32_t id_offset; // ids are id_offset .. id_offset + n_vocab - 1
};
cudaError_t launch_pq_resolve(const PqResolveArgs& a, cudaStream_t stream);

cudaError_t launch_spec_resolve(uint32_t n_seq, uint32_t n_pos, const int32_t* accepted, const int32_t* token,
                                int32_t* n_kept, int32_t* next_token, cudaStream_t stream);

cudaError_t launch_spec_commit(uint32_t n_seq, uint32_t n_pos, const int32_t* drafts, const int32_t* n_kept,
                               const int32_t* next_token, int32_t* history, uint64_t history_ld, uint32_t history_cap,
                               int32_t* history_len, int32_t* next_input, uint32_t* flags, cudaStream_t stream);

constexpr uint32_t kDraftPickMaxSeq = 8, kDraftPickMaxRank = 256;
cudaError_t launch_draft_pick(const float* logits, uint64_t ld, const float* head, const float* embed, const float* x,
                              uint64_t x_ld, const float* w, const int32_t* prev, uint32_t n_seq, uint32_t n_vocab,
                              uint32_t rank, uint32_t dim, uint32_t n_embed, unsigned long long* best, int32_t* draft,
                              float* conf, cudaStream_t stream);

cudaError_t launch_draft_pick_plain(const float* logits, uint64_t ld, uint32_t n_seq, uint32_t n_vocab, const float* h,
                                    uint64_t h_ld, const float* conf_w, uint32_t width, float conf_bias, int32_t* draft,
                                    float* conf, int32_t* next_prev, cudaStream_t stream);

cudaError_t launch_rank_force(const float* logits, uint64_t ld, uint32_t batch, uint32_t n_vocab, const int32_t* token,
                              uint32_t k, int32_t* forced, uint32_t* above, cudaStream_t stream);

cudaError_t launch_decode_commit(uint32_t batch, const int32_t* sampled, const int32_t* forced, int32_t* history,
                                 uint64_t history_ld, uint32_t history_cap, int32_t* history_len, int32_t* next_input,
                                 int32_t* committed, uint32_t* flags, cudaStream_t stream);

// Test hook: y[i] = expf_host_exact(x[i]).
cudaError_t launch_expf_probe(const float* x, float* y, uint64_t n, cudaStream_t stream);

constexpr uint32_t kVpMaxK = 64;
constexpr uint32_t kVpHeaderBytes = 16;
__host__ __device__ inline uint32_t vp_record_bytes(uint32_t k) { return kVpHeaderBytes + 8u * k; }

} // namespace mk
