// The reference's one-row, stateful sampler object behind the C ABI: mako::gen::Sampler (src/gen/sampler.hpp:22-45)
// keeps the sampling parameters, the multiset of generated tokens and a std::mt19937_64; so does this handle, with
// the history mirrored in device memory and the uniforms produced on the host exactly as libstdc++'s
// uniform_real_distribution<float> produces them from that generator (one 64-bit draw per uniform), so that the
// same seed gives the reference's token stream. The arithmetic runs in the row pipeline kernel.
#include "row_pipeline.h"

#include <limits>
#include <new>
#include <random>
#include <vector>

extern "C" const char* mk_last_error(void);

struct mk_row_sampler {
    mk_sampler* core = nullptr;
    mk_sampling_params params{};
    uint32_t n_vocab = 0;
    int device = 0;
    std::mt19937_64 rng;
    std::vector<int32_t> history;
    int32_t* d_history = nullptr;
    size_t d_history_cap = 0;
    float* d_row = nullptr;     // staging for a host logits row
    float* d_u = nullptr;       // [2]
    int32_t* d_io = nullptr;    // [0] token, [1] accepted, [2] draft
    cudaStream_t stream = nullptr;
};

namespace {

float next_uniform(std::mt19937_64& g)
{
    // what uniform_real_distribution<float>(0, total) multiplies total with (sampler.cpp:66,100)
    return std::generate_canonical<float, std::numeric_limits<float>::digits>(g);
}

int ensure_history(mk_row_sampler* r)
{
    if (r->history.size() <= r->d_history_cap)
        return MK_OK;
    size_t cap = r->d_history_cap ? r->d_history_cap * 2 : 4096;
    while (cap < r->history.size())
        cap *= 2;
    int32_t* p = nullptr;
    if (cudaMalloc((void**)&p, cap * 4) != cudaSuccess)
        return MK_ERR_CUDA;
    if (r->d_history) {
        cudaMemcpyAsync(p, r->d_history, r->d_history_cap * 4, cudaMemcpyDeviceToDevice, r->stream);
        cudaStreamSynchronize(r->stream);
        cudaFree(r->d_history);
    }
    r->d_history = p;
    r->d_history_cap = cap;
    return MK_OK;
}

const float* device_row(mk_row_sampler* r, const float* logits)
{
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, logits) == cudaSuccess &&
        (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged))
        return logits;
    cudaGetLastError();
    cudaMemcpyAsync(r->d_row, logits, (size_t)r->n_vocab * 4, cudaMemcpyHostToDevice, r->stream);
    return r->d_row;
}

void fill_rows(mk_row_sampler* r, const float* dev_logits, mk_rows& rows)
{
    rows = mk_rows{};
    rows.logits = dev_logits;
    rows.ld = r->n_vocab;
    rows.batch = 1;
    rows.n_vocab = r->n_vocab;
    // the reference counts every accepted token; a history longer than the kernel's 16-bit counters allow would
    // need the long form of the penalty pass
    rows.n_history = (uint32_t)r->history.size();
    rows.history = r->history.empty() ? nullptr : r->d_history;
    rows.history_ld = r->history.size();
    rows.params = r->params;
}

} // namespace

extern "C" {

int mk_row_sampler_create(mk_row_sampler** out, const mk_sampling_params* p, uint32_t n_vocab, uint64_t seed, int device)
{
    if (!out || !p)
        return MK_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    mk_sampler* core = nullptr;
    if (int rc = mk_sampler_create(&core, device, n_vocab, 1))
        return rc;
    mk_row_sampler* r = new (std::nothrow) mk_row_sampler();
    if (!r) {
        mk_sampler_destroy(core);
        return MK_ERR_INVALID_ARGUMENT;
    }
    r->core = core;
    r->params = *p;
    r->n_vocab = n_vocab;
    r->device = device;
    r->rng.seed(seed);
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(device);
    bool ok = cudaMalloc((void**)&r->d_row, (size_t)n_vocab * 4) == cudaSuccess &&
              cudaMalloc((void**)&r->d_u, 8) == cudaSuccess && cudaMalloc((void**)&r->d_io, 12) == cudaSuccess &&
              cudaStreamCreateWithFlags(&r->stream, cudaStreamNonBlocking) == cudaSuccess;
    cudaSetDevice(prev);
    if (!ok) {
        mk_row_sampler_destroy(r);
        return MK_ERR_CUDA;
    }
    *out = r;
    return MK_OK;
}

void mk_row_sampler_destroy(mk_row_sampler* r)
{
    if (!r)
        return;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(r->device);
    if (r->d_history) cudaFree(r->d_history);
    if (r->d_row) cudaFree(r->d_row);
    if (r->d_u) cudaFree(r->d_u);
    if (r->d_io) cudaFree(r->d_io);
    if (r->stream) cudaStreamDestroy(r->stream);
    cudaSetDevice(prev);
    mk_sampler_destroy(r->core);
    delete r;
}

int mk_row_sampler_greedy(const mk_row_sampler* r)
{
    return r && r->params.temperature <= 0.0f;
}

// Sampler::accept (sampler.cpp:15-18)
int mk_row_sampler_accept(mk_row_sampler* r, int32_t token)
{
    if (!r)
        return MK_ERR_INVALID_ARGUMENT;
    if (r->history.size() >= 65535)
        return MK_ERR_UNSUPPORTED;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(r->device);
    r->history.push_back(token);
    int rc = ensure_history(r);
    if (rc == MK_OK &&
        cudaMemcpyAsync(r->d_history + (r->history.size() - 1), &r->history.back(), 4, cudaMemcpyHostToDevice,
                        r->stream) != cudaSuccess)
        rc = MK_ERR_CUDA;
    cudaSetDevice(prev);
    return rc;
}

// Sampler::sample (sampler.cpp:75-84). logits: host or device pointer to n_vocab floats.
int mk_row_sampler_sample(mk_row_sampler* r, const float* logits, int32_t* token)
{
    if (!r || !logits || !token)
        return MK_ERR_INVALID_ARGUMENT;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(r->device);
    const bool greedy = mk_row_sampler_greedy(r);
    float u[2] = {0.0f, 0.0f};
    if (!greedy) { // greedy draws nothing from the generator
        u[0] = next_uniform(r->rng);
        cudaMemcpyAsync(r->d_u, u, 4, cudaMemcpyHostToDevice, r->stream);
    }
    mk_rows rows;
    fill_rows(r, device_row(r, logits), rows);
    mk_sample_out out{};
    out.token = r->d_io;
    int rc = mk_sampler_sample_batch(r->core, &rows, r->d_u, &out, r->stream);
    if (rc == MK_OK) {
        if (cudaMemcpyAsync(token, r->d_io, 4, cudaMemcpyDeviceToHost, r->stream) != cudaSuccess ||
            cudaStreamSynchronize(r->stream) != cudaSuccess)
            rc = MK_ERR_CUDA;
    }
    cudaSetDevice(prev);
    return rc;
}

// Sampler::verify (sampler.cpp:86-107): one generator draw for the acceptance, one more only after a rejection.
int mk_row_sampler_verify(mk_row_sampler* r, const float* logits, int32_t draft, int32_t* accepted, int32_t* token)
{
    if (!r || !logits || !token || !accepted)
        return MK_ERR_INVALID_ARGUMENT;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(r->device);
    const bool greedy = mk_row_sampler_greedy(r);
    float u[2] = {0.0f, 0.0f};
    std::mt19937_64 after_first = r->rng;
    if (!greedy) {
        u[0] = next_uniform(r->rng);
        after_first = r->rng;
        u[1] = next_uniform(r->rng);
        cudaMemcpyAsync(r->d_u, u, 8, cudaMemcpyHostToDevice, r->stream);
    }
    int32_t io[3] = {0, 0, draft};
    cudaMemcpyAsync(r->d_io + 2, &io[2], 4, cudaMemcpyHostToDevice, r->stream);
    mk_rows rows;
    fill_rows(r, device_row(r, logits), rows);
    mk_sample_out out{};
    out.token = r->d_io;
    int rc = mk_sampler_verify_batch(r->core, &rows, r->d_io + 2, r->d_u, r->d_u + 1, &out, r->d_io + 1, r->stream);
    if (rc == MK_OK) {
        if (cudaMemcpyAsync(io, r->d_io, 8, cudaMemcpyDeviceToHost, r->stream) != cudaSuccess ||
            cudaStreamSynchronize(r->stream) != cudaSuccess)
            rc = MK_ERR_CUDA;
    }
    if (rc == MK_OK) {
        *token = io[0];
        *accepted = io[1];
        if (!greedy && io[1])
            r->rng = after_first; // the second draw was not consumed
    }
    cudaSetDevice(prev);
    return rc;
}

} // extern "C"
