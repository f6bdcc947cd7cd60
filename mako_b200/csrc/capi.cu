// C ABI of the library (declared in include/mako_b200.h): argument checks, scratch ownership, kernel launches.
// No allocation happens after mk_sampler_create, except the host-buffer entry point, which sizes its device staging on
// first use. There is no CPU fallback anywhere: without a CUDA device every entry point fails.
#include "row_pipeline.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <random>
#include <vector>

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what)
{
    return fail(MK_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define MK_CUDA(call)                                                                                                  \
    do {                                                                                                               \
        cudaError_t e__ = (call);                                                                                      \
        if (e__ != cudaSuccess)                                                                                        \
            return cuda_fail(e__, #call);                                                                              \
    } while (0)

// Entries of raw-candidate scratch per row: the vocabulary rounded up to a multiple of 4, so that every row's
// 16*cap-byte block starts on a 16-byte boundary (the raw candidates are read and written as 8-byte pairs).
inline uint32_t scratch_cap(uint32_t n_vocab) { return (n_vocab + 3u) & ~3u; }

constexpr uint32_t kPqCap = 4096;      // candidates per list in p/q verification
constexpr uint32_t kSplitMaxBatch = 8, kSplitMaxShards = 64, kSplitKeys = 1024;
constexpr uint32_t kMaxTiles = 512, kTile = 4096;

} // namespace

struct mk_sampler {
    int device = 0;
    uint32_t n_vocab = 0, max_batch = 0;
    uint32_t* scratch = nullptr; // [max_batch][4*n_vocab] words: raw candidates (a row can never overflow it) + sort buffer / a float per column
    uint32_t* scratch_pq = nullptr; // the same again: p/q verification runs its two row sets side by side
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    // p/q verification lists
    int32_t *p_ids = nullptr, *q_ids = nullptr;
    float *p_q = nullptr, *q_q = nullptr, *p_total = nullptr, *q_total = nullptr, *q_prob = nullptr;
    uint32_t *p_n = nullptr, *q_n = nullptr, *p_flags = nullptr, *q_flags = nullptr;
    int32_t* p_tok = nullptr;
    // host-buffer staging (sized on first use)
    cudaStream_t own_stream = nullptr;
    int overlap = MK_OVERLAP_OFF;         // how the row kernel is launched behind its predecessor in the stream
    unsigned long long* timing = nullptr; // debug: per-row phase timestamps of the next launches
    uint32_t skip_tile = 0xffffffffu, wait_probes = 0; // debug: withhold one tile's copy; probes before a wait gives up
    unsigned long long* pick_best = nullptr; // mk_draft_pick: one packed (score, id) maximum per sequence
    unsigned char* stage = nullptr;
    size_t stage_bytes = 0;
    // small batches under a top_k: every row split over many CTAs (shard records, then the merge)
    unsigned char* split_records = nullptr; // [kSplitMaxShards][kSplitMaxBatch] records of kVpMaxK entries
    uint32_t* split_flags = nullptr;        // [kSplitMaxBatch], when the caller asks for no flags
    int split = 1;                          // 0: every batch runs as one CTA per row
};

namespace {

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev)
    {
        if (cudaGetDevice(&prev) != cudaSuccess)
            ok = false;
        else if (prev != dev && cudaSetDevice(dev) != cudaSuccess)
            ok = false;
    }
    ~DeviceGuard()
    {
        if (prev >= 0)
            cudaSetDevice(prev);
    }
};

int check_rows(const mk_sampler* s, const mk_rows* r)
{
    if (!s)
        return fail(MK_ERR_INVALID_ARGUMENT, "null sampler handle");
    if (!r)
        return fail(MK_ERR_INVALID_ARGUMENT, "null rows");
    if (r->n_vocab == 0)
        return fail(MK_ERR_INVALID_ARGUMENT, "sampler: empty vocabulary");
    if (r->n_vocab > s->n_vocab)
        return fail(MK_ERR_INVALID_ARGUMENT, "n_vocab %u exceeds the handle's %u", r->n_vocab, s->n_vocab);
    if ((r->n_vocab + kTile - 1) / kTile > kMaxTiles)
        return fail(MK_ERR_INVALID_ARGUMENT, "n_vocab %u above the supported %u", r->n_vocab, kMaxTiles * kTile);
    if (r->batch > s->max_batch)
        return fail(MK_ERR_INVALID_ARGUMENT, "batch %u exceeds the handle's max_batch %u", r->batch, s->max_batch);
    if (r->batch > 0 && !r->logits)
        return fail(MK_ERR_INVALID_ARGUMENT, "null logits");
    if (r->ld < r->n_vocab)
        return fail(MK_ERR_INVALID_ARGUMENT, "ld %llu smaller than n_vocab %u", (unsigned long long)r->ld, r->n_vocab);
    if (r->history) {
        if (!r->history_len && r->n_history > 65535u)
            return fail(MK_ERR_INVALID_ARGUMENT, "n_history %u above 65535", r->n_history);
        if (r->history_ld < r->n_history && !r->history_len)
            return fail(MK_ERR_INVALID_ARGUMENT, "history_ld smaller than n_history");
    }
    if (r->mask && r->mask_ld < (uint64_t)(r->n_vocab + 31) / 32)
        return fail(MK_ERR_INVALID_ARGUMENT, "mask_ld %llu smaller than ceil(n_vocab/32)", (unsigned long long)r->mask_ld);
    return MK_OK;
}

void fill_common(mk::RowKernelArgs& a, const mk_sampler* s, const mk_rows* r)
{
    std::memset(&a, 0, sizeof a);
    a.logits = r->logits;
    a.ld = r->ld;
    a.n_vocab = r->n_vocab;
    a.id_offset = r->id_offset;
    a.history = (r->history && (r->history_len || r->n_history)) ? r->history : nullptr;
    a.history_ld = r->history_ld;
    a.history_len = r->history_len;
    a.n_history = r->n_history;
    a.mask = r->mask;
    a.mask_ld = r->mask_ld;
    a.bias = r->n_bias ? r->bias : nullptr;
    a.n_bias = r->bias ? r->n_bias : 0;
    a.params_dev = r->params_dev;
    a.params = r->params;
    a.scratch = s->scratch;
    a.scratch_cap = scratch_cap(s->n_vocab);
    a.timing = s->timing;
    a.overlap = s->overlap;
    a.debug_skip_tile = s->skip_tile;
    a.debug_wait_probes = s->wait_probes;
    a.use_bulk_copy = ((reinterpret_cast<uintptr_t>(r->logits) & 15u) == 0 && (r->ld % 4u) == 0) ? 1 : 0;
}

void fill_out(mk::RowKernelArgs& a, const mk_sample_out* o)
{
    a.token = o->token;
    a.prob = o->prob;
    a.flags = o->flags;
    a.n_cand = o->n_cand;
    a.cand_ids = o->cand_cap ? o->cand_ids : nullptr;
    a.cand_q = o->cand_cap ? o->cand_q : nullptr;
    a.cand_cap = o->cand_cap;
}

bool all_greedy(const mk_rows* r)
{
    return !r->params_dev && r->params.temperature <= 0.0f;
}

// A handful of rows under a top_k leaves most of the device idle when each row is one CTA, and the top_k bound costs
// that CTA a histogram update per element. Such a batch is split instead: every row's columns go to many CTAs, each
// writing the record a vocabulary shard writes (maximum, partial sum, its best entries); the merge draws from the
// records. A row the merge cannot prove complete (VP_TRUNCATED: one shard's whole list inside the deciding set) is
// run again as one CTA by a follow-up launch that skips every other row, so the results are those of the plain path.
bool split_eligible(const mk_sampler* s, const mk_rows* r, const mk::RowKernelArgs& a)
{
    if (!s->split || r->batch == 0 || r->batch > kSplitMaxBatch || r->params_dev || !a.use_bulk_copy)
        return false;
    const mk_sampling_params& p = r->params;
    if (!(p.temperature > 0.0f) || p.top_k == 0 || p.top_k > mk::kVpMaxK)
        return false;
    if (r->n_vocab < 4u * kTile || r->id_offset < 0 || (uint64_t)r->id_offset + r->n_vocab > (1u << 26))
        return false;
    return s->timing == nullptr && s->skip_tile == 0xffffffffu;
}

int sample_split(mk_sampler* s, const mk_rows* rows, mk::RowKernelArgs a, const mk_sample_out* out, cudaStream_t stream)
{
    (void)out;
    const uint32_t n_tiles = (rows->n_vocab + kTile - 1) / kTile;
    const uint32_t per = (n_tiles + kSplitMaxShards - 1) / kSplitMaxShards; // tiles per shard
    const uint32_t n_shards = (n_tiles + per - 1) / per;
    uint32_t k = kSplitKeys / n_shards;
    k = k > mk::kVpMaxK ? mk::kVpMaxK : (k < 8u ? 8u : k);
    mk::RowKernelArgs first = a;
    first.mode = mk::kModeVpLocal;
    first.split_w = per * kTile;
    first.vp_records = s->split_records;
    first.vp_k = k;
    first.token = nullptr;
    first.prob = nullptr;
    first.flags = nullptr;
    first.n_cand = nullptr;
    first.cand_ids = nullptr;
    first.cand_q = nullptr;
    MK_CUDA(mk::launch_row_kernel(first, rows->batch, stream));
    mk::VpMergeArgs m;
    std::memset(&m, 0, sizeof m);
    m.gathered = s->split_records;
    m.n_shards = n_shards;
    m.batch = rows->batch;
    m.k = k;
    m.n_vocab_total = rows->n_vocab;
    m.params = rows->params;
    m.u = a.u;
    m.token = a.token;
    m.prob = a.prob;
    m.flags = a.flags ? a.flags : s->split_flags;
    m.n_cand = a.n_cand;
    m.cand_ids = a.cand_ids;
    m.cand_q = a.cand_q;
    m.cand_cap = a.cand_cap;
    MK_CUDA(mk::launch_vp_merge(m, stream));
    // the rows the merge reported incomplete, as one CTA each; this launch reads the flags the merge wrote, so it is
    // never started ahead of it
    a.overlap = MK_OVERLAP_OFF;
    a.only_flagged = m.flags;
    a.only_flagged_mask = MK_FLAG_VP_TRUNCATED;
    a.flags = m.flags;
    MK_CUDA(mk::launch_row_kernel(a, rows->batch, stream));
    return MK_OK;
}

} // namespace

extern "C" {

const char* mk_version(void)
{
    return "mako_b200 0.1 sm_100a";
}

const char* mk_last_error(void)
{
    return g_err;
}

uint64_t mk_row_bytes(uint32_t n_vocab, uint32_t n_history, int has_mask, uint32_t n_bias, uint32_t n_uniforms)
{
    return 4ull * n_vocab + 4ull * n_history + (has_mask ? 4ull * ((n_vocab + 31) / 32) : 0ull) + 8ull * n_bias +
           4ull * n_uniforms + 8ull;
}

int mk_check_sampling(const mk_sampling_params* p)
{
    if (!p)
        return fail(MK_ERR_INVALID_ARGUMENT, "null params");
    const float v[6] = {p->temperature, p->top_p, p->min_p, p->presence_penalty, p->frequency_penalty,
                        p->repetition_penalty};
    for (float x : v)
        if (!std::isfinite(x))
            return fail(MK_ERR_INVALID_ARGUMENT, "sampling parameters must be finite");
    if (p->temperature > 0 && p->temperature < 1e-3f)
        return fail(MK_ERR_INVALID_ARGUMENT, "temperature must be 0 (greedy) or at least 0.001");
    if (p->repetition_penalty <= 0 || p->repetition_penalty > 100)
        return fail(MK_ERR_INVALID_ARGUMENT, "repetition_penalty must be in (0, 100]");
    if (std::fabs(p->presence_penalty) > 100 || std::fabs(p->frequency_penalty) > 100)
        return fail(MK_ERR_INVALID_ARGUMENT, "presence_penalty and frequency_penalty must be within -100..100");
    return MK_OK;
}

int mk_sampler_create(mk_sampler** out, int device, uint32_t n_vocab, uint32_t max_batch)
{
    if (!out)
        return fail(MK_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    if (n_vocab == 0)
        return fail(MK_ERR_INVALID_ARGUMENT, "sampler: empty vocabulary");
    if (max_batch == 0)
        return fail(MK_ERR_INVALID_ARGUMENT, "max_batch must be at least 1");
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
        cudaGetLastError();
        return fail(MK_ERR_NO_DEVICE, "no CUDA device: this library has no CPU path");
    }
    if (device < 0 || device >= n_dev)
        return fail(MK_ERR_INVALID_ARGUMENT, "device %d out of range (%d devices)", device, n_dev);
    DeviceGuard g(device);
    if (!g.ok)
        return fail(MK_ERR_CUDA, "cannot select device %d", device);
    cudaDeviceProp prop;
    MK_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10)
        return fail(MK_ERR_UNSUPPORTED, "device %d is sm_%d%d; the kernels are built for sm_100a only", device,
                    prop.major, prop.minor);
    mk_sampler* s = new (std::nothrow) mk_sampler();
    if (!s)
        return fail(MK_ERR_INVALID_ARGUMENT, "out of host memory");
    s->device = device;
    s->n_vocab = n_vocab;
    s->max_batch = max_batch;
    const size_t b = max_batch;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) {
        if (e == cudaSuccess)
            e = cudaMalloc(p, bytes);
    };
    alloc((void**)&s->scratch, b * mk::row_scratch_words(scratch_cap(n_vocab)) * 4);
    alloc((void**)&s->scratch_pq, b * mk::row_scratch_words(scratch_cap(n_vocab)) * 4);
    alloc((void**)&s->p_ids, b * kPqCap * 4);
    alloc((void**)&s->q_ids, b * kPqCap * 4);
    alloc((void**)&s->p_q, b * kPqCap * 4);
    alloc((void**)&s->q_q, b * kPqCap * 4);
    alloc((void**)&s->p_total, b * 4);
    alloc((void**)&s->q_total, b * 4);
    alloc((void**)&s->q_prob, b * 4);
    alloc((void**)&s->p_n, b * 4);
    alloc((void**)&s->q_n, b * 4);
    alloc((void**)&s->p_flags, b * 4);
    alloc((void**)&s->q_flags, b * 4);
    alloc((void**)&s->p_tok, b * 4);
    alloc((void**)&s->pick_best, (mk::kDraftPickMaxSeq + 1) * sizeof(unsigned long long)); // maxima + ticket counter
    alloc((void**)&s->split_records, (size_t)kSplitMaxShards * kSplitMaxBatch * mk::vp_record_bytes(mk::kVpMaxK));
    alloc((void**)&s->split_flags, kSplitMaxBatch * 4);
    if (e == cudaSuccess)
        e = cudaMemset(s->pick_best, 0, (mk::kDraftPickMaxSeq + 1) * sizeof(unsigned long long));
    if (e == cudaSuccess)
        e = cudaStreamCreateWithFlags(&s->own_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess)
        e = cudaEventCreateWithFlags(&s->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess)
        e = cudaEventCreateWithFlags(&s->ev_join, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        mk_sampler_destroy(s);
        return cuda_fail(e, "allocating the handle's scratch");
    }
    *out = s;
    return MK_OK;
}

void mk_sampler_destroy(mk_sampler* s)
{
    if (!s)
        return;
    DeviceGuard g(s->device);
    void* ptrs[] = {s->scratch, s->p_ids, s->q_ids, s->p_q, s->q_q, s->p_total, s->q_total, s->q_prob,
                    s->p_n,     s->q_n,   s->p_flags, s->q_flags, s->p_tok, s->stage, s->pick_best,
                    s->split_records, s->split_flags, s->scratch_pq};
    for (void* p : ptrs)
        if (p)
            cudaFree(p);
    if (s->ev_fork)
        cudaEventDestroy(s->ev_fork);
    if (s->ev_join)
        cudaEventDestroy(s->ev_join);
    if (s->own_stream)
        cudaStreamDestroy(s->own_stream);
    delete s;
}

int mk_sampler_sample_batch(mk_sampler* s, const mk_rows* rows, const float* u, const mk_sample_out* out, void* stream)
{
    if (int rc = check_rows(s, rows))
        return rc;
    if (!out || !out->token)
        return fail(MK_ERR_INVALID_ARGUMENT, "out->token is required");
    if (!u && !all_greedy(rows))
        return fail(MK_ERR_INVALID_ARGUMENT, "uniforms are required unless every row is greedy");
    DeviceGuard g(s->device);
    mk::RowKernelArgs a;
    fill_common(a, s, rows);
    fill_out(a, out);
    a.u = u;
    a.mode = mk::kModeSample;
    if (split_eligible(s, rows, a))
        return sample_split(s, rows, a, out, (cudaStream_t)stream);
    MK_CUDA(mk::launch_row_kernel(a, rows->batch, (cudaStream_t)stream));
    return MK_OK;
}

// ---- sampling without any allocation --------------------------------------------------------------------------------
// The row kernel parks its raw candidate list in global memory. For callers that cannot allocate, that list lives
// in this file-scope device array instead of a handle's buffer: MK_STATIC_MAX_ROWS rows of 16 bytes per column
// for vocabularies up to MK_STATIC_MAX_VOCAB, about 20 MiB on every GPU that loads the library, held until the
// process exits. The symbol is a host-side stand-in here; the address the kernel needs is asked for once per device.
static __device__ __align__(256) uint32_t g_static_scratch[(size_t)MK_STATIC_MAX_ROWS * (4u * MK_STATIC_MAX_VOCAB + 4u)];
static uint32_t* g_static_scratch_ptr[64] = {};

int mk_sample_rows_static(int device, const mk_rows* rows, const float* u, const mk_sample_out* out, void* stream)
{
    if (device < 0 || device >= 64)
        return fail(MK_ERR_INVALID_ARGUMENT, "device %d out of range", device);
    if (!rows)
        return fail(MK_ERR_INVALID_ARGUMENT, "null rows");
    if (rows->batch > MK_STATIC_MAX_ROWS)
        return fail(MK_ERR_INVALID_ARGUMENT, "batch %u above the static limit of %u rows", rows->batch,
                    (unsigned)MK_STATIC_MAX_ROWS);
    if (rows->n_vocab > MK_STATIC_MAX_VOCAB)
        return fail(MK_ERR_INVALID_ARGUMENT, "n_vocab %u above the static limit of %u columns", rows->n_vocab,
                    (unsigned)MK_STATIC_MAX_VOCAB);
    mk_sampler tmp; // a view for the shared argument checks; owns nothing
    tmp.device = device;
    tmp.n_vocab = MK_STATIC_MAX_VOCAB;
    tmp.max_batch = MK_STATIC_MAX_ROWS;
    if (int rc = check_rows(&tmp, rows))
        return rc;
    if (!out || !out->token)
        return fail(MK_ERR_INVALID_ARGUMENT, "out->token is required");
    if (!u && !all_greedy(rows))
        return fail(MK_ERR_INVALID_ARGUMENT, "uniforms are required unless every row is greedy");
    DeviceGuard g(device);
    if (!g.ok)
        return fail(MK_ERR_CUDA, "cannot select device %d", device);
    if (!g_static_scratch_ptr[device]) { // first call on this device: resolve the symbol with the device current
        void* p = nullptr;
        MK_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        g_static_scratch_ptr[device] = static_cast<uint32_t*>(p);
    }
    tmp.scratch = g_static_scratch_ptr[device];
    mk::RowKernelArgs a;
    fill_common(a, &tmp, rows);
    fill_out(a, out);
    a.u = u;
    a.mode = mk::kModeSample;
    MK_CUDA(mk::launch_row_kernel(a, rows->batch, (cudaStream_t)stream));
    return MK_OK;
}

int mk_sampler_verify_batch(mk_sampler* s, const mk_rows* rows, const int32_t* draft, const float* u_accept,
                            const float* u_redraw, const mk_sample_out* out, int32_t* accepted, void* stream)
{
    if (int rc = check_rows(s, rows))
        return rc;
    if (!out || !out->token || !accepted || !draft)
        return fail(MK_ERR_INVALID_ARGUMENT, "draft, accepted and out->token are required");
    if ((!u_accept || !u_redraw) && !all_greedy(rows))
        return fail(MK_ERR_INVALID_ARGUMENT, "both uniforms are required unless every row is greedy");
    DeviceGuard g(s->device);
    mk::RowKernelArgs a;
    fill_common(a, s, rows);
    fill_out(a, out);
    a.u = u_accept;
    a.u2 = u_redraw;
    a.draft = draft;
    a.accepted = accepted;
    a.mode = mk::kModeVerify;
    MK_CUDA(mk::launch_row_kernel(a, rows->batch, (cudaStream_t)stream));
    return MK_OK;
}

int mk_sampler_verify_pq_batch(mk_sampler* s, const mk_rows* rows, const float* draft_logits, uint64_t draft_ld,
                               const float* u_draft, const float* u_accept, const float* u_resample,
                               int32_t* draft_token, int32_t* accepted, int32_t* token, uint32_t* flags, void* stream)
{
    if (int rc = check_rows(s, rows))
        return rc;
    if (!draft_logits || draft_ld < rows->n_vocab)
        return fail(MK_ERR_INVALID_ARGUMENT, "draft_logits / draft_ld invalid");
    if (!draft_token || !accepted || !token)
        return fail(MK_ERR_INVALID_ARGUMENT, "draft_token, accepted and token are required");
    if ((!u_draft || !u_accept || !u_resample))
        return fail(MK_ERR_INVALID_ARGUMENT, "three uniforms per row are required");
    DeviceGuard g(s->device);
    cudaStream_t st = (cudaStream_t)stream;
    // The drafter's rows and the target's rows are independent until the resolve: the target's launches go to the
    // handle's own stream, forked from and joined back into the caller's (a stream capture follows both arms), so the
    // few long rows of one set's second launch do not leave the device idle and the two first launches fill it as
    // one. Each arm has its own candidate scratch.
    MK_CUDA(cudaEventRecord(s->ev_fork, st));
    MK_CUDA(cudaStreamWaitEvent(s->own_stream, s->ev_fork, 0));
    // drafter rows: draw the draft token and keep q's list
    mk_rows qrows = *rows;
    qrows.logits = draft_logits;
    qrows.ld = draft_ld;
    mk::RowKernelArgs a;
    fill_common(a, s, &qrows);
    a.u = u_draft;
    a.token = draft_token;
    a.prob = s->q_prob;
    a.flags = s->q_flags;
    a.n_cand = s->q_n;
    a.cand_ids = s->q_ids;
    a.cand_q = s->q_q;
    a.cand_cap = kPqCap;
    a.total_out = s->q_total;
    a.mode = mk::kModeSample;
    MK_CUDA(mk::launch_row_kernel(a, rows->batch, st));
    // target rows: p's list
    fill_common(a, s, rows);
    a.token = s->p_tok;
    a.flags = s->p_flags;
    a.n_cand = s->p_n;
    a.cand_ids = s->p_ids;
    a.cand_q = s->p_q;
    a.cand_cap = kPqCap;
    a.total_out = s->p_total;
    a.mode = mk::kModeDistOnly;
    a.scratch = s->scratch_pq;
    a.overlap = MK_OVERLAP_OFF; // nothing precedes it in that stream but the fork
    MK_CUDA(mk::launch_row_kernel(a, rows->batch, s->own_stream));
    MK_CUDA(cudaEventRecord(s->ev_join, s->own_stream));
    MK_CUDA(cudaStreamWaitEvent(st, s->ev_join, 0));
    mk::PqResolveArgs r;
    std::memset(&r, 0, sizeof r);
    r.batch = rows->batch;
    r.cap = kPqCap;
    r.p_ids = s->p_ids; r.p_q = s->p_q; r.p_n = s->p_n; r.p_flags = s->p_flags;
    r.q_ids = s->q_ids; r.q_q = s->q_q; r.q_n = s->q_n; r.q_flags = s->q_flags;
    r.p_total = s->p_total; r.q_total = s->q_total; r.q_prob = s->q_prob;
    r.draft_token = draft_token;
    r.u_accept = u_accept; r.u_resample = u_resample;
    r.accepted = accepted; r.token = token; r.flags = flags;
    r.n_vocab = rows->n_vocab; r.id_offset = rows->id_offset;
    MK_CUDA(mk::launch_pq_resolve(r, st));
    return MK_OK;
}

int mk_draft_pick(mk_sampler* s, const float* logits, uint64_t ld, const float* head, const float* embed, const float* x,
                  uint64_t x_ld, const float* w, const int32_t* prev, uint32_t n_seq, uint32_t n_vocab, uint32_t rank,
                  uint32_t dim, uint32_t n_embed, int32_t* draft, float* conf, void* stream)
{
    if (!s || !logits || !head || !embed || !x || !w || !prev || !draft || !conf)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_draft_pick: null argument");
    if (n_seq > mk::kDraftPickMaxSeq || rank == 0 || rank > mk::kDraftPickMaxRank || (rank & 3u) != 0 ||
        (reinterpret_cast<uintptr_t>(head) & 15u) != 0 || n_vocab == 0 || ld < n_vocab ||
        x_ld < dim)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_draft_pick: n_seq %u (max %u), rank %u (a multiple of 4, max %u; head 16-byte aligned), n_vocab %u, ld %llu",
                    n_seq, mk::kDraftPickMaxSeq, rank, mk::kDraftPickMaxRank, n_vocab, (unsigned long long)ld);
    DeviceGuard g(s->device);
    MK_CUDA(mk::launch_draft_pick(logits, ld, head, embed, x, x_ld, w, prev, n_seq, n_vocab, rank, dim, n_embed,
                                  s->pick_best, draft, conf, (cudaStream_t)stream));
    return MK_OK;
}

int mk_draft_pick_plain(mk_sampler* s, const float* logits, uint64_t ld, uint32_t n_seq, uint32_t n_vocab, const float* h,
                        uint64_t h_ld, const float* conf_w, uint32_t width, float conf_bias, int32_t* draft, float* conf,
                        int32_t* next_prev, void* stream)
{
    if (!s || !logits || !h || !conf_w || !draft || !conf)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_draft_pick_plain: null argument");
    if (n_vocab == 0 || ld < n_vocab || h_ld < width)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_draft_pick_plain: n_vocab %u, ld %llu, width %u, h_ld %llu", n_vocab,
                    (unsigned long long)ld, width, (unsigned long long)h_ld);
    DeviceGuard g(s->device);
    MK_CUDA(mk::launch_draft_pick_plain(logits, ld, n_seq, n_vocab, h, h_ld, conf_w, width, conf_bias, draft, conf,
                                        next_prev, (cudaStream_t)stream));
    return MK_OK;
}

int mk_rank_force(mk_sampler* s, const float* logits, uint64_t ld, uint32_t batch, uint32_t n_vocab,
                  const int32_t* token, uint32_t k, int32_t* forced, uint32_t* above, void* stream)
{
    if (!s || !logits || !token || (!forced && !above))
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_rank_force: logits, token and one output are required");
    if (n_vocab == 0 || ld < n_vocab)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_rank_force: n_vocab %u, ld %llu", n_vocab, (unsigned long long)ld);
    DeviceGuard g(s->device);
    MK_CUDA(mk::launch_rank_force(logits, ld, batch, n_vocab, token, k, forced, above, (cudaStream_t)stream));
    return MK_OK;
}

int mk_decode_commit(mk_sampler* s, uint32_t batch, const int32_t* sampled, const int32_t* forced, int32_t* history,
                     uint64_t history_ld, uint32_t history_cap, int32_t* history_len, int32_t* next_input,
                     int32_t* committed, uint32_t* flags, void* stream)
{
    if (!s || !sampled || !history || !history_len)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_decode_commit: sampled, history and history_len are required");
    if (history_ld < history_cap)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_decode_commit: history_ld %llu below history_cap %u",
                    (unsigned long long)history_ld, history_cap);
    if (history_cap > 65535u)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_decode_commit: history_cap %u above 65535 (the sampler counts a "
                                             "token's occurrences in 16 bits)", history_cap);
    DeviceGuard g(s->device);
    MK_CUDA(mk::launch_decode_commit(batch, sampled, forced, history, history_ld, history_cap, history_len, next_input,
                                     committed, flags, (cudaStream_t)stream));
    return MK_OK;
}

int mk_spec_resolve(mk_sampler* s, uint32_t n_seq, uint32_t n_pos, const int32_t* accepted, const int32_t* token,
                    int32_t* n_kept, int32_t* next_token, void* stream)
{
    if (!s || !accepted || !token || !n_kept || !next_token || n_pos == 0)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_spec_resolve: null argument or n_pos == 0");
    DeviceGuard g(s->device);
    MK_CUDA(mk::launch_spec_resolve(n_seq, n_pos, accepted, token, n_kept, next_token, (cudaStream_t)stream));
    return MK_OK;
}

int mk_sampler_spec_round(mk_sampler* s, const mk_rows* rows, uint32_t n_pos, const int32_t* drafts,
                          const int32_t* forced, const float* u, const mk_sample_out* out, int32_t* accepted,
                          int32_t* n_kept, int32_t* next_token, void* stream)
{
    if (int rc = check_rows(s, rows))
        return rc;
    if (n_pos == 0 || rows->batch % n_pos != 0)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_sampler_spec_round: batch %u is not a multiple of n_pos %u",
                    rows->batch, n_pos);
    if (!out || !out->token || !accepted || !n_kept || !next_token || (n_pos > 1 && !drafts))
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_sampler_spec_round: drafts, accepted, n_kept, next_token and "
                                             "out->token are required");
    if (!u && !all_greedy(rows))
        return fail(MK_ERR_INVALID_ARGUMENT, "uniforms are required unless every row is greedy");
    DeviceGuard g(s->device);
    mk::RowKernelArgs a;
    fill_common(a, s, rows);
    fill_out(a, out);
    a.u = u;
    a.accepted = accepted;
    a.mode = mk::kModeVerify; // per row: the last position of a sequence is sampled, the others are verified
    a.spec_n_pos = n_pos;
    a.spec_drafts = drafts;
    a.spec_forced = forced;
    MK_CUDA(mk::launch_row_kernel(a, rows->batch, (cudaStream_t)stream));
    MK_CUDA(mk::launch_spec_resolve(rows->batch / n_pos, n_pos, accepted, out->token, n_kept, next_token,
                                    (cudaStream_t)stream));
    return MK_OK;
}

int mk_spec_commit(mk_sampler* s, uint32_t n_seq, uint32_t n_pos, const int32_t* drafts, const int32_t* n_kept,
                   const int32_t* next_token, int32_t* history, uint64_t history_ld, uint32_t history_cap,
                   int32_t* history_len, int32_t* next_input, uint32_t* flags, void* stream)
{
    if (!s || !n_kept || !next_token || !history || !history_len || n_pos == 0 || (n_pos > 1 && !drafts))
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_spec_commit: null argument or n_pos == 0");
    if (history_ld < history_cap || history_cap > 65535u)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_spec_commit: history_ld %llu, history_cap %u (at most 65535)",
                    (unsigned long long)history_ld, history_cap);
    DeviceGuard g(s->device);
    MK_CUDA(mk::launch_spec_commit(n_seq, n_pos, drafts, n_kept, next_token, history, history_ld, history_cap,
                                   history_len, next_input, flags, (cudaStream_t)stream));
    return MK_OK;
}

uint32_t mk_vp_record_bytes(uint32_t k)
{
    return mk::vp_record_bytes(k);
}

int mk_sampler_vp_local(mk_sampler* s, const mk_rows* shard_rows, uint32_t k, void* records, void* stream)
{
    if (int rc = check_rows(s, shard_rows))
        return rc;
    if (!records || k == 0 || k > mk::kVpMaxK)
        return fail(MK_ERR_INVALID_ARGUMENT, "records required and 1 <= k <= %u", mk::kVpMaxK);
    DeviceGuard g(s->device);
    mk::RowKernelArgs a;
    fill_common(a, s, shard_rows);
    a.vp_records = records;
    a.vp_k = k;
    a.mode = mk::kModeVpLocal;
    MK_CUDA(mk::launch_row_kernel(a, shard_rows->batch, (cudaStream_t)stream));
    return MK_OK;
}

int mk_sampler_vp_merge(mk_sampler* s, const void* gathered, uint32_t n_shards, uint32_t batch, uint32_t k,
                        uint32_t n_vocab_total, const mk_sampling_params* params, const float* u,
                        const mk_sample_out* out, void* stream)
{
    if (!s || !gathered || !params || !out || !out->token)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_sampler_vp_merge: null argument");
    if (n_shards == 0 || n_shards > 64 || k == 0 || k > mk::kVpMaxK || n_shards * k > 2048)
        return fail(MK_ERR_INVALID_ARGUMENT, "n_shards in 1..64, k in 1..%u, n_shards*k <= 2048", mk::kVpMaxK);
    if (!u && params->temperature > 0.0f)
        return fail(MK_ERR_INVALID_ARGUMENT, "uniforms are required unless greedy");
    if (n_vocab_total > (1u << 26))
        return fail(MK_ERR_INVALID_ARGUMENT, "n_vocab_total %u above 2^26 (the merge keeps the shard beside the id)",
                    n_vocab_total);
    DeviceGuard g(s->device);
    mk::VpMergeArgs a;
    std::memset(&a, 0, sizeof a);
    a.gathered = static_cast<const unsigned char*>(gathered);
    a.n_shards = n_shards;
    a.batch = batch;
    a.k = k;
    a.n_vocab_total = n_vocab_total;
    a.params = *params;
    a.u = u;
    a.token = out->token;
    a.prob = out->prob;
    a.flags = out->flags;
    a.n_cand = out->n_cand;
    a.cand_ids = out->cand_cap ? out->cand_ids : nullptr;
    a.cand_q = out->cand_cap ? out->cand_q : nullptr;
    a.cand_cap = out->cand_cap;
    MK_CUDA(mk::launch_vp_merge(a, (cudaStream_t)stream));
    return MK_OK;
}

int mk_sampler_sample_host(mk_sampler* s, const mk_rows* hr, const float* u, const mk_sample_out* ho)
{
    if (!s || !hr || !ho || !ho->token)
        return fail(MK_ERR_INVALID_ARGUMENT, "mk_sampler_sample_host: null argument");
    if (hr->params_dev)
        return fail(MK_ERR_INVALID_ARGUMENT, "host form takes shared params only");
    if (hr->history_len)
        return fail(MK_ERR_INVALID_ARGUMENT, "host form takes one history length for all rows (n_history); "
                                             "history_len must be NULL");
    if (int rc = check_rows(s, hr)) // strides, sizes and limits, before any of them sizes the staging buffer
        return rc;
    if (!u && !all_greedy(hr))
        return fail(MK_ERR_INVALID_ARGUMENT, "uniforms are required unless every row is greedy");
    DeviceGuard g(s->device);
    const size_t B = hr->batch, V = hr->n_vocab;
    const size_t ldd = (V + 3) & ~size_t(3);
    const size_t mask_w = (V + 31) / 32, mask_ld = (mask_w + 3) & ~size_t(3);
    const bool has_hist = hr->history && hr->n_history;
    auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
    size_t off = 0;
    const size_t o_logits = off; off += up(B * ldd * 4);
    const size_t o_hist = off;   off += up(has_hist ? B * hr->n_history * 4 : 0);
    const size_t o_mask = off;   off += up(hr->mask ? B * mask_ld * 4 : 0);
    const size_t o_bias = off;   off += up(hr->bias ? B * hr->n_bias * sizeof(mk_bias) : 0);
    const size_t o_u = off;      off += up(B * 4);
    const size_t o_tok = off;    off += up(B * 4);
    const size_t o_prob = off;   off += up(B * 4);
    const size_t o_flags = off;  off += up(B * 4);
    const size_t o_n = off;      off += up(B * 4);
    if (off > s->stage_bytes) {
        if (s->stage)
            cudaFree(s->stage);
        s->stage = nullptr;
        s->stage_bytes = 0;
        MK_CUDA(cudaMalloc((void**)&s->stage, off));
        s->stage_bytes = off;
    }
    unsigned char* d = s->stage;
    cudaStream_t st = s->own_stream;
    if (B == 0)
        return MK_OK;
    MK_CUDA(cudaMemcpy2DAsync(d + o_logits, ldd * 4, hr->logits, hr->ld * 4, V * 4, B, cudaMemcpyHostToDevice, st));
    if (has_hist)
        MK_CUDA(cudaMemcpy2DAsync(d + o_hist, hr->n_history * 4, hr->history, hr->history_ld * 4, hr->n_history * 4, B,
                                  cudaMemcpyHostToDevice, st));
    if (hr->mask)
        MK_CUDA(cudaMemcpy2DAsync(d + o_mask, mask_ld * 4, hr->mask, hr->mask_ld * 4, mask_w * 4, B,
                                  cudaMemcpyHostToDevice, st));
    if (hr->bias && hr->n_bias)
        MK_CUDA(cudaMemcpyAsync(d + o_bias, hr->bias, B * hr->n_bias * sizeof(mk_bias), cudaMemcpyHostToDevice, st));
    if (u)
        MK_CUDA(cudaMemcpyAsync(d + o_u, u, B * 4, cudaMemcpyHostToDevice, st));
    mk_rows dr = *hr;
    dr.logits = reinterpret_cast<const float*>(d + o_logits);
    dr.ld = ldd;
    dr.history = has_hist ? reinterpret_cast<const int32_t*>(d + o_hist) : nullptr;
    dr.history_ld = hr->n_history;
    dr.history_len = nullptr;
    dr.mask = hr->mask ? reinterpret_cast<const uint32_t*>(d + o_mask) : nullptr;
    dr.mask_ld = mask_ld;
    dr.bias = (hr->bias && hr->n_bias) ? reinterpret_cast<const mk_bias*>(d + o_bias) : nullptr;
    mk_sample_out dout;
    std::memset(&dout, 0, sizeof dout);
    dout.token = reinterpret_cast<int32_t*>(d + o_tok);
    dout.prob = reinterpret_cast<float*>(d + o_prob);
    dout.flags = reinterpret_cast<uint32_t*>(d + o_flags);
    dout.n_cand = reinterpret_cast<uint32_t*>(d + o_n);
    if (int rc = mk_sampler_sample_batch(s, &dr, u ? reinterpret_cast<const float*>(d + o_u) : nullptr, &dout, st))
        return rc;
    MK_CUDA(cudaMemcpyAsync(ho->token, dout.token, B * 4, cudaMemcpyDeviceToHost, st));
    if (ho->prob)
        MK_CUDA(cudaMemcpyAsync(ho->prob, dout.prob, B * 4, cudaMemcpyDeviceToHost, st));
    if (ho->flags)
        MK_CUDA(cudaMemcpyAsync(ho->flags, dout.flags, B * 4, cudaMemcpyDeviceToHost, st));
    if (ho->n_cand)
        MK_CUDA(cudaMemcpyAsync(ho->n_cand, dout.n_cand, B * 4, cudaMemcpyDeviceToHost, st));
    MK_CUDA(cudaStreamSynchronize(st));
    return MK_OK;
}


int mk_sampler_set_overlap(mk_sampler* s, int mode)
{
    if (!s)
        return fail(MK_ERR_INVALID_ARGUMENT, "null sampler handle");
    if (mode != MK_OVERLAP_OFF && mode != MK_OVERLAP_LAUNCH && mode != MK_OVERLAP_STABLE_SIDE_INPUTS)
        return fail(MK_ERR_INVALID_ARGUMENT, "overlap mode %d is none of MK_OVERLAP_*", mode);
    s->overlap = mode;
    return MK_OK;
}

int mk_sampler_set_split(mk_sampler* s, int on)
{
    if (!s)
        return fail(MK_ERR_INVALID_ARGUMENT, "null sampler handle");
    s->split = on ? 1 : 0;
    return MK_OK;
}

int mk_debug_withhold_tile(mk_sampler* s, int tile, uint32_t wait_probes)
{
    if (!s)
        return fail(MK_ERR_INVALID_ARGUMENT, "null sampler handle");
    s->skip_tile = tile < 0 ? 0xffffffffu : (uint32_t)tile;
    s->wait_probes = wait_probes;
    return MK_OK;
}

int mk_debug_set_timing(mk_sampler* s, unsigned long long* timing_dev)
{
    if (!s)
        return fail(MK_ERR_INVALID_ARGUMENT, "null sampler handle");
    s->timing = timing_dev;
    return MK_OK;
}

/* test hook, not declared in the public header's main section */
int mk_debug_expf(const float* x_dev, float* y_dev, uint64_t n, void* stream)
{
    MK_CUDA(mk::launch_expf_probe(x_dev, y_dev, n, (cudaStream_t)stream));
    return MK_OK;
}

} // extern "C"
