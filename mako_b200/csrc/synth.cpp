// Deterministic synthetic inputs for the token-sampling path: logits, token histories, allowed-token masks, sparse
// biases and uniforms, all from counter-addressed PCG-XSH-RR 64/32 streams so that any (seed, stream, row) can be
// regenerated independently on any host thread. No dataset is involved: the distributions below are the
// definition of the benchmark and test inputs.
//
//   logits   : i.i.d. N(0, sigma^2) by Box-Muller, plus n_spikes "spike" tokens per row at distinct uniformly
//              random ids with value U(spike_lo, spike_hi)
//   history  : ids = rank-1 with rank ~ Zipf(s) over [1, V] (inverse CDF on a double cumulative table)
//   mask     : packed uint32 words, bit id%32 of word id/32; about `fraction` of the ids allowed, half of them in
//              4 random contiguous blocks and half scattered; each spike id allowed with probability 0.5
//   bias     : n_bias pairs per row with distinct ids and value U(lo, hi)
//   uniforms : u = (x >> 8) * 2^-24 in [0, 1)
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

struct Pcg32 {
    uint64_t state, inc;
    Pcg32(uint64_t seed, uint64_t seq)
    {
        state = 0;
        inc = (seq << 1) | 1u;
        next();
        state += seed;
        next();
    }
    uint32_t next()
    {
        const uint64_t old = state;
        state = old * 6364136223846793005ULL + inc;
        const uint32_t xs = uint32_t(((old >> 18) ^ old) >> 27);
        const uint32_t rot = uint32_t(old >> 59);
        return (xs >> rot) | (xs << ((32 - rot) & 31));
    }
    float uniform() { return float(next() >> 8) * (1.0f / 16777216.0f); }
    double uniform_open() { return (double(next() >> 8) + 1.0) * (1.0 / 16777216.0); } // (0, 1]
    uint32_t below(uint32_t n) { return uint32_t((uint64_t(next()) * n) >> 32); }
};

// One stream id per (purpose, row): purposes keep logits, history, mask, bias and uniforms of a row independent.
inline uint64_t stream_id(uint32_t purpose, uint64_t step, uint64_t row)
{
    return (uint64_t(purpose) << 56) ^ (step << 24) ^ row;
}

template <class F> void parallel_rows(uint32_t rows, uint32_t n_threads, F&& f)
{
    n_threads = std::max(1u, std::min(n_threads, rows));
    if (n_threads == 1) {
        for (uint32_t r = 0; r < rows; ++r)
            f(r);
        return;
    }
    std::vector<std::thread> pool;
    for (uint32_t t = 0; t < n_threads; ++t)
        pool.emplace_back([&, t] {
            for (uint32_t r = t; r < rows; r += n_threads)
                f(r);
        });
    for (auto& th : pool)
        th.join();
}

} // namespace

extern "C" {

// out[b*ld + i], b < rows; spike_ids (nullable) receives rows*n_spikes ids. row0 offsets the stream so that a
// shard of a larger batch generates exactly its own rows.
void mk_synth_logits(uint64_t seed, uint64_t step, uint32_t row0, uint32_t rows, uint32_t n_vocab, uint64_t ld,
                     float sigma, uint32_t n_spikes, float spike_lo, float spike_hi, float* out, int32_t* spike_ids,
                     uint32_t n_threads)
{
    parallel_rows(rows, n_threads, [&](uint32_t b) {
        Pcg32 g(seed, stream_id(1, step, uint64_t(row0) + b));
        float* o = out + size_t(b) * ld;
        for (uint32_t i = 0; i < n_vocab; i += 2) {
            const double u1 = g.uniform_open(), u2 = double(g.uniform());
            const double rad = std::sqrt(-2.0 * std::log(u1)), ang = 6.283185307179586476925 * u2;
            o[i] = float(double(sigma) * rad * std::cos(ang));
            if (i + 1 < n_vocab)
                o[i + 1] = float(double(sigma) * rad * std::sin(ang));
        }
        std::vector<int32_t> picked;
        while (picked.size() < n_spikes && picked.size() < n_vocab) {
            const int32_t id = int32_t(g.below(n_vocab));
            if (std::find(picked.begin(), picked.end(), id) != picked.end())
                continue;
            picked.push_back(id);
            o[id] = spike_lo + (spike_hi - spike_lo) * g.uniform();
        }
        if (spike_ids)
            for (uint32_t k = 0; k < n_spikes; ++k)
                spike_ids[size_t(b) * n_spikes + k] = k < picked.size() ? picked[k] : -1;
    });
}

void mk_synth_history_zipf(uint64_t seed, uint64_t step, uint32_t row0, uint32_t rows, uint32_t n_vocab,
                           uint32_t n_history, double s, int32_t* out, uint32_t n_threads)
{
    std::vector<double> cdf(n_vocab);
    double acc = 0;
    for (uint32_t r = 0; r < n_vocab; ++r) {
        acc += std::pow(double(r) + 1.0, -s);
        cdf[r] = acc;
    }
    parallel_rows(rows, n_threads, [&](uint32_t b) {
        Pcg32 g(seed, stream_id(2, step, uint64_t(row0) + b));
        for (uint32_t j = 0; j < n_history; ++j) {
            const double x = double(g.uniform()) * acc;
            const uint32_t r = uint32_t(std::upper_bound(cdf.begin(), cdf.end(), x) - cdf.begin());
            out[size_t(b) * n_history + j] = int32_t(std::min(r, n_vocab - 1));
        }
    });
}

// mask_ld = words per row (>= ceil(V/32)); words beyond the vocabulary stay 0.
void mk_synth_mask(uint64_t seed, uint64_t step, uint32_t row0, uint32_t rows, uint32_t n_vocab, uint64_t mask_ld,
                   double fraction, const int32_t* spike_ids, uint32_t n_spikes, uint32_t* out, uint32_t n_threads)
{
    parallel_rows(rows, n_threads, [&](uint32_t b) {
        Pcg32 g(seed, stream_id(3, step, uint64_t(row0) + b));
        uint32_t* m = out + size_t(b) * mask_ld;
        std::memset(m, 0, size_t(mask_ld) * 4);
        auto set = [&](uint32_t id) { m[id >> 5] |= 1u << (id & 31); };
        auto clear = [&](uint32_t id) { m[id >> 5] &= ~(1u << (id & 31)); };
        const uint32_t want = std::max<uint32_t>(1, uint32_t(fraction * n_vocab));
        const uint32_t block = std::max<uint32_t>(1, want / 8);
        for (int k = 0; k < 4; ++k) {
            const uint32_t start = g.below(n_vocab > block ? n_vocab - block : 1);
            for (uint32_t i = 0; i < block && start + i < n_vocab; ++i)
                set(start + i);
        }
        for (uint32_t k = 0; k < want / 2; ++k)
            set(g.below(n_vocab));
        if (spike_ids)
            for (uint32_t k = 0; k < n_spikes; ++k) {
                const int32_t id = spike_ids[size_t(b) * n_spikes + k];
                if (id < 0)
                    continue;
                if (g.next() & 1u)
                    set(uint32_t(id));
                else
                    clear(uint32_t(id));
            }
    });
}

void mk_synth_bias(uint64_t seed, uint64_t step, uint32_t row0, uint32_t rows, uint32_t n_vocab, uint32_t n_bias,
                   float lo, float hi, int32_t* ids, float* vals, uint32_t n_threads)
{
    parallel_rows(rows, n_threads, [&](uint32_t b) {
        Pcg32 g(seed, stream_id(4, step, uint64_t(row0) + b));
        int32_t* id = ids + size_t(b) * n_bias;
        float* v = vals + size_t(b) * n_bias;
        uint32_t n = 0;
        while (n < n_bias) {
            const int32_t c = int32_t(g.below(n_vocab));
            if (n_bias <= n_vocab && std::find(id, id + n, c) != id + n)
                continue;
            id[n] = c;
            v[n] = lo + (hi - lo) * g.uniform();
            ++n;
        }
    });
}

void mk_synth_uniforms(uint64_t seed, uint64_t step, uint32_t purpose, uint32_t row0, uint32_t n, float* out)
{
    for (uint32_t b = 0; b < n; ++b) {
        Pcg32 g(seed, stream_id(8 + purpose, step, uint64_t(row0) + b));
        out[b] = g.uniform();
    }
}

// N(0, sigma^2) noise added in place (drafter logits = target logits + noise).
void mk_synth_add_noise(uint64_t seed, uint64_t step, uint32_t row0, uint32_t rows, uint32_t n_vocab, uint64_t ld,
                        float sigma, float* inout, uint32_t n_threads)
{
    parallel_rows(rows, n_threads, [&](uint32_t b) {
        Pcg32 g(seed, stream_id(5, step, uint64_t(row0) + b));
        float* o = inout + size_t(b) * ld;
        for (uint32_t i = 0; i < n_vocab; i += 2) {
            const double u1 = g.uniform_open(), u2 = double(g.uniform());
            const double rad = std::sqrt(-2.0 * std::log(u1)), ang = 6.283185307179586476925 * u2;
            o[i] += float(double(sigma) * rad * std::cos(ang));
            if (i + 1 < n_vocab)
                o[i + 1] += float(double(sigma) * rad * std::sin(ang));
        }
    });
}

} // extern "C"
