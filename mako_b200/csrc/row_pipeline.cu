// The fused row pipeline of the token sampler for sm_100a: one CTA per row, one pass over the row in HBM.
//
// What it replaces: mako::gen::Sampler::distribution / draw / sample / verify (src/gen/sampler.cpp:20-107), which
// the reference runs on the host, one row at a time, over a copy of the logits.
//
// Shape of the kernel (352 threads = 11 warps, 113 KB shared memory laid out per row, two CTAs per SM):
//   warp 0        producer: streams the row through a ring of 16 KB tiles — five stages beside a history's tables,
//                 seven without — with untiled bulk asynchronous copies (TMA, cp.async.bulk, no multicast, L2
//                 evict-first), completion on an mbarrier per stage; the first stages are requested before the
//                 set-up so that they fly meanwhile.
//   set-up        all warps: the token history becomes a bitmap of generated columns, the rank of each bitmap
//                 word's first set bit (prefix popcount) and, by rank, the count of each generated column — the
//                 multiset the reference keeps in an unordered_map (sampler.cpp:15-18). The history entry that set
//                 a column's bit owns the column; owners apply the penalties to the tiles that have landed by then
//                 (the dense head of the history).
//   warps 1-2     fix-up: each owns every other tile; once it has landed, apply the sparse edits in shared memory —
//                 logit bias, then the repetition / presence / frequency penalties of the tile's generated columns,
//                 each once with its count (sampler.cpp:23-28), found by rank (binary search over the word ranks,
//                 then the n-th set bit of the word) — and release it to the readers.
//   warps 3-10    readers: 128-bit shared loads, allowed-token mask, running row maximum (warp shuffles), and
//                 collection of every element that can still become a candidate: the keep thresholds of min_p,
//                 top_k and top_p are all lower-bounded by a function of the running maximum (or, for top_k, of a
//                 histogram of the reader threads' maxima) that only rises while the row streams, so filtering with
//                 the current bound keeps a superset of the final candidates. The loop exists in five variants.
//   finish        exact weights q = expf((l - max) * inv_t) for the few collected elements with the host library's
//                 float exponential (device_expf.cuh), min_p, top_k, top_p, and the sequential float total and walk
//                 of the draw — in the reference's precision and order, because token ids depend on both. Up to 64
//                 candidates: one warp, in registers. Steps only unusual rows need (long lists) live in functions of
//                 their own.
//   second pass   top_p alone: the first launch keeps the 24 largest elements; a row whose nucleus that does not
//                 settle marks itself, and a second launch of this kernel streams the marked rows again.
//   split launch  a few rows under a top_k: a second grid dimension over column shards, each CTA writing a shard
//                 record for the merge kernel (also the local step of vocab-parallel sampling).
//
// Numeric contract (what makes ids bit-exact): IEEE division and no FMA contraction in the penalties and in
// (l - max) * inv_t; q through expf_host_exact; top_p sums in double; total and the walk in float, left to right.
#include "row_pipeline.h"

#include "device_expf.cuh"
#include "ptx.cuh"

#include <cfloat>
#include <type_traits>

namespace mk {

namespace {

constexpr int kTile = 4096;     // floats per tile
constexpr int kMaxStages = 7;  // ring stages that fit when a row needs no tables
constexpr int kProducerThreads = 32;
constexpr int kFixers = 64;
constexpr int kReaders = 256;
constexpr int kThreads = kProducerThreads + kFixers + kReaders;
constexpr int kReaderWarps = kReaders / 32;
constexpr int kVec = kTile / (kReaders * 4); // 128-bit loads per reader thread per tile
constexpr int kEl = kVec * 4;
static_assert(kVec * kReaders * 4 == kTile, "a tile is a whole number of 128-bit loads per reader thread");
constexpr int kHistCap = 4096;  // history entries de-duplicated in shared memory; longer histories scan global memory
constexpr int kBmWords = 5120;  // history bitmap: one bit per column, vocabularies up to 163840 columns
constexpr uint32_t kMaxBitmapVocab = kBmWords * 32u;
constexpr int kSortCap = 8192;  // 64-bit sort keys: they take the ring (64 KB) once the streaming is over
constexpr uint32_t kBarSort = 3;         // named barrier of the sorting warps
constexpr uint32_t kNucleusGuess = 24;  // top_p alone, first launch: the largest elements kept (the one-warp finish takes 32 candidates)
#ifndef MK_PREFIX_TILES
#define MK_PREFIX_TILES 4
#endif
constexpr int kPrefixTiles = MK_PREFIX_TILES;  // tiles all warps edit before the stream starts (their columns fit 16 bits)
constexpr int kBins = 2048;     // bins of the top_k histogram (see hist_bin)

// Shared memory of a CTA: this fixed head, then kDynBytes laid out per row. While the row streams: the tables the
// row needs (generated-column bitmap, per-word ranks, counts; the top_k histogram) and, in all that is left, the
// tile ring — five stages beside a history's tables, seven without. Once the streaming is over the same bytes hold
// the finish's sort keys and its own bitmap, ranks and order list.
struct __align__(128) Smem {
    double warp_sum[kThreads / 32];
    uint64_t full[kMaxStages], ready[kMaxStages], empty[kMaxStages];
    unsigned long long best_key;    // (order key of the row maximum << 32) | ~column: first argmax wins
    uint32_t m_key;                 // running maximum, as order key
    uint32_t thr_topk_key;          // top_k lower bound, as order key (only ever raised)
    uint32_t ncand;                 // raw candidates appended
    uint32_t nsurv;                 // candidates surviving the exact filter
    uint32_t abort_flag;
    uint32_t nan0;                  // column 0 (token id 0) is NaN: the reference's max_element keeps it
    uint32_t hi_group;              // highest non-empty group of 32 histogram bins
    uint32_t first_tile_warps;      // reader warps whose first-tile maxima are in the histogram
    uint32_t n_final;
    uint32_t flags;
    uint32_t n_distinct;            // distinct special columns (generated or biased)
    uint32_t n_own;                 // generated columns within the first tiles (edited by all warps)
};
constexpr uint32_t kSmemBytes = 115712; // two CTAs per SM: (228 KB - 2 x 1 KB reserved) / 2
constexpr uint32_t kHeadBytes = (sizeof(Smem) + 127u) & ~127u;
constexpr uint32_t kDynBytes = kSmemBytes - kHeadBytes;
// finish-phase layout inside the dynamic part
constexpr uint32_t kOffKeys = 0;                                  // kSortCap 64-bit keys
constexpr uint32_t kOffFinBitmap = kSortCap * 8u;                 // kBmWords words (also: the mass histogram)
constexpr uint32_t kOffFinWpre = kOffFinBitmap + kBmWords * 4u;   // kBmWords 16-bit ranks
constexpr uint32_t kOffFinOrd = kOffFinWpre + kBmWords * 2u;      // kSortCap 16-bit slots
static_assert(kOffFinOrd + kSortCap * 2u <= kDynBytes, "finish layout fits");
static_assert(kBins * 4u <= kBmWords * 4u, "mass histogram fits the finish bitmap area");

// Bins of the histogram that bounds the k-th largest element of a row: monotone in the float order, fine where
// logits live — 32 bins per octave for magnitudes from 2^-10 to 2^8 (a bin is 2.2 % wide), everything smaller or
// larger folded into the end bins of its sign — so that the bin in which the count from the top reaches k holds few
// elements beyond the k wanted. Positive values take bins 1024.., negative ones mirror them below; NaN takes bin 0.
__device__ __forceinline__ uint32_t hist_bin(float v)
{
    if (v != v)
        return 0u;
    const uint32_t u = __float_as_uint(v), mag = u & 0x7fffffffu;
    const int e = (int)(mag >> 23) - 117;
    uint32_t p; // 0..575
    if (e < 0)
        p = 0u;
    else if (e > 17)
        p = 575u;
    else
        p = (uint32_t)e * 32u + ((mag >> 18) & 31u);
    return (u >> 31) ? 1023u - p : 1024u + p;
}

// A float no element of bin b is smaller than (a bound from below; b >= 1).
__device__ __forceinline__ float hist_bin_floor(uint32_t b)
{
    if (b >= 1024u) {
        const uint32_t p = min(b - 1024u, 575u);
        return p == 0u ? 0.0f : __uint_as_float((((p >> 5) + 117u) << 23) | ((p & 31u) << 18));
    }
    const uint32_t p = 1023u - b; // magnitudes of this bin lie below the next bin's start
    if (p >= 575u)
        return -__int_as_float(0x7f800000);
    const uint32_t q = p + 1u;
    return -__uint_as_float((((q >> 5) + 117u) << 23) | ((q & 31u) << 18));
}

struct RowCfg {
    float temperature, inv_t, minp_eff, top_p;
    uint32_t top_k;
    uint32_t hist_k;    // the histogram bound keeps the hist_k largest elements
    float rep, presence, frequency;
    bool greedy, hist_mode, need_sum, use_topp, pen_active, optimistic;
    float delta_w;      // keep elements with l >= running max - delta_w
    bool force_none;    // inv_t is inf/NaN: no finite weight can exist
};

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ RowCfg make_cfg(const mk_sampling_params& p, uint32_t n_vocab, int mode, uint32_t vp_k, int pass)
{
    RowCfg c;
    c.temperature = p.temperature;
    c.greedy = p.temperature <= 0.0f;                       // sampler.hpp:26
    c.inv_t = __fdiv_rn(1.0f, p.temperature);               // sampler.cpp:29
    c.minp_eff = (1.0f < p.min_p) ? 1.0f : p.min_p;         // std::min(min_p, 1.0f), sampler.cpp:34
    c.top_p = p.top_p;
    c.top_k = p.top_k;
    c.rep = p.repetition_penalty;
    c.presence = p.presence_penalty;
    c.frequency = p.frequency_penalty;
    c.pen_active = !(c.rep == 1.0f && c.presence == 0.0f && c.frequency == 0.0f);
    c.use_topp = p.top_p < 1.0f;
    c.hist_mode = !c.greedy && p.top_k > 0 && p.top_k < n_vocab;
    // One more than top_k is kept, so that "more candidates than top_k" (which decides whether the reference
    // truncates, and with it the order of the list, sampler.cpp:39) can be told from the kept elements alone.
    c.hist_k = p.top_k + 1u;
    const bool minp_on = c.minp_eff > 0.0f;
    // The float total over "all candidates" is only needed when top_p is the only truncation.
    c.need_sum = !c.greedy && c.use_topp && !minp_on && !c.hist_mode;
    c.force_none = !c.greedy && (!(c.inv_t < __int_as_float(0x7f800000)) || !(c.inv_t == c.inv_t));
    // top_p alone: the first launch bets that the nucleus lies within the kNucleusGuess largest elements and keeps
    // only those (the top_k histogram bound, with no top_k cut afterwards); a row whose nucleus does not close within
    // what was kept asks for the second pass, which keeps everything the mass bound allows.
    c.optimistic = c.need_sum && pass == 0 && mode != kModeVpLocal && kNucleusGuess < n_vocab;
    if (c.optimistic) {
        c.hist_mode = true;
        c.hist_k = kNucleusGuess;
    }
    if (mode == kModeVpLocal) {
        c.hist_mode = vp_k < n_vocab;
        c.top_k = vp_k;
        c.hist_k = vp_k;
        c.need_sum = true;
        c.use_topp = false;
        c.minp_eff = 0.0f;
    }
    // Distance below the row maximum, in units of (l - max) * inv_t, past which an element cannot be kept:
    //   q == 0 below about -103.98 (float underflow of expf);
    //   q < min_p below ln(min_p);
    //   with top_p alone, an element with q < (1 - top_p) / n_vocab is outside the nucleus, because all such
    //   elements together weigh less than (1 - top_p) * total (total >= 1: the maximum itself has q = 1).
    float d = 104.2f;
    if (mode != kModeVpLocal) {
        if (minp_on)
            d = fminf(d, -logf(c.minp_eff));
        if (c.need_sum) {
            float a = (1.0f - c.top_p) / (float)n_vocab;
            a = fminf(a, 1.0f);
            if (a > 0.0f)
                d = fminf(d, -logf(a));
        }
    }
    d = d * 1.001f + 1e-3f;
    c.delta_w = d * fmaxf(c.temperature, 0.0f);
    if (!(c.delta_w == c.delta_w))
        c.delta_w = __int_as_float(0x7f800000);
    return c;
}

// Threshold on the (edited) logit for the current running maximum; never -inf, so masked elements never pass.
__device__ __forceinline__ float keep_threshold(const RowCfg& c, float m_run)
{
    if (c.force_none || !(m_run < __int_as_float(0x7f800000)))
        return __int_as_float(0x7f800000); // no finite weight can exist (an infinite maximum makes l - max NaN or -inf)
    const float t = m_run - c.delta_w - fabsf(m_run) * 1e-6f;
    return fmaxf(t, -FLT_MAX);
}

// Penalties of one generated token with count n, exactly as sampler.cpp:24-27.
__device__ __forceinline__ float penalise(float l, uint32_t n, const RowCfg& c)
{
    if (c.rep != 1.0f)
        l = (l > 0.0f) ? __fdiv_rn(l, c.rep) : __fmul_rn(l, c.rep);
    const float step = __fadd_rn(c.presence, __fmul_rn(c.frequency, (float)n));
    return __fsub_rn(l, step);
}

__device__ __forceinline__ unsigned long long pack_by_weight(float q, uint32_t col)
{
    // ascending key order = (q descending, column ascending); q > 0 so its bit pattern is monotone
    return ((unsigned long long)(~__float_as_uint(q)) << 32) | col;
}
__device__ __forceinline__ unsigned long long pack_by_column(float q, uint32_t col)
{
    return ((unsigned long long)col << 32) | __float_as_uint(q);
}

// Position of the n-th set bit (n = 0: the lowest) of a word that has more than n bits set: five halvings by
// popcount (the library's find-n-th-set is a loop over the bits).
__device__ __forceinline__ uint32_t nth_set_bit(uint32_t w, uint32_t n)
{
    uint32_t pos = 0;
#pragma unroll
    for (uint32_t width = 16; width > 0; width >>= 1) {
        const uint32_t c = (uint32_t)__popc(w & ((1u << width) - 1u));
        if (n >= c) {
            n -= c;
            pos += width;
            w >>= width;
        }
    }
    return pos;
}

// Penalties (sampler.cpp:23-28) for the generated columns with ranks [r_lo, r_hi) — the ones whose bitmap words lie
// in [w_lo, w_hi) — spread evenly over n_thr threads (this one is `thr`): a rank is turned back into its column by a
// binary search over the per-word ranks and a find-n-th-set-bit in the word, and indexes the count directly. Every
// column is touched by exactly one thread. `tile` points at column `col0` of the row in shared memory.
__device__ __forceinline__ void fix_hits(const uint32_t* bitmap, const uint16_t* wpre, const uint32_t* counts,
                                         float* tile, uint32_t col0, uint32_t w_lo, uint32_t w_hi, uint32_t r_lo,
                                         uint32_t r_hi, uint32_t thr, uint32_t n_thr, const RowCfg& cfg)
{
    for (uint32_t r = r_lo + thr; r < r_hi; r += n_thr) {
        uint32_t lo = w_lo, hi = w_hi; // largest word in [lo, hi) whose rank is <= r
        while (hi - lo > 1u) {
            const uint32_t mid = (lo + hi) >> 1;
            if ((uint32_t)wpre[mid] <= r)
                lo = mid;
            else
                hi = mid;
        }
        const uint32_t bit = nth_set_bit(bitmap[lo], r - (uint32_t)wpre[lo]);
        const uint32_t n = (counts[r >> 1] >> ((r & 1u) * 16u)) & 0xffffu;
        const uint32_t loc = (lo << 5) + bit - col0;
        tile[loc] = penalise(tile[loc], n, cfg);
    }
}

// Exclusive prefix of the per-word popcounts of bitmap[0, bm_words) into wpre, total into s.n_distinct: a set
// bit's rank among all set bits is then wpre[word] + popcount of the lower bits of its word. Whole CTA; the caller
// synchronises before (bitmap complete) and after (wpre complete). Each thread takes a contiguous run of words; the
// run length is odd, so that the lanes of a warp, one run apart, read 32 different banks.
__device__ __forceinline__ void word_ranks(Smem& s, const uint32_t* bitmap, uint16_t* wpre, uint32_t bm_words)
{
    constexpr int kWordsPerThread = ((kBmWords + kThreads - 1) / kThreads) | 1;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t per = ((bm_words + kThreads - 1) / kThreads) | 1u;
    const uint32_t w0 = min(tid * per, bm_words);
    uint32_t pc[kWordsPerThread]; // popcounts of this thread's words: all loads in flight together
    uint32_t mine = 0;
#pragma unroll
    for (int i = 0; i < kWordsPerThread; ++i) {
        const uint32_t w = w0 + (uint32_t)i;
        pc[i] = ((uint32_t)i < per && w < bm_words) ? (uint32_t)__popc(bitmap[w]) : 0u;
        mine += pc[i];
    }
    uint32_t inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, inc, o);
        if ((int)lane >= o)
            inc += y;
    }
    uint32_t* wtot = reinterpret_cast<uint32_t*>(s.warp_sum); // 22 words of scratch
    if (lane == 31)
        wtot[warp] = inc;
    __syncthreads();
    uint32_t before = inc - mine;
    for (uint32_t w = 0; w < warp; ++w)
        before += wtot[w];
#pragma unroll
    for (int i = 0; i < kWordsPerThread; ++i) {
        const uint32_t w = w0 + (uint32_t)i;
        if ((uint32_t)i < per && w < bm_words)
            wpre[w] = (uint16_t)before;
        before += pc[i];
    }
    if (tid == kThreads - 1)
        s.n_distinct = before; // every word lies at or before the last thread's run
}

// Bitonic sort of n2 (power of two) 64-bit keys in shared memory. Called by the whole CTA; only as many warps as
// have a compare-exchange to do per step take part (a short list is sorted by a few warps over a cheap named barrier
// instead of by 352 threads over the CTA's), the others wait at the end.
__device__ void block_sort(unsigned long long* keys, uint32_t n2)
{
    const uint32_t nthr = min((uint32_t)kThreads, max(32u, ((n2 >> 1) + 31u) & ~31u));
    if (threadIdx.x < nthr) {
        for (uint32_t k = 2; k <= n2; k <<= 1) {
            for (uint32_t j = k >> 1; j > 0; j >>= 1) {
                for (uint32_t c = threadIdx.x; c < (n2 >> 1); c += nthr) {
                    // the c-th pair of this step: i has bit j clear
                    const uint32_t i = ((c & ~(j - 1u)) << 1) | (c & (j - 1u)), l = i | j;
                    const unsigned long long a = keys[i], b = keys[l];
                    if ((a > b) == ((i & k) == 0)) {
                        keys[i] = b;
                        keys[l] = a;
                    }
                }
                if (nthr == 32u)
                    __syncwarp();
                else
                    named_barrier(kBarSort, nthr);
            }
        }
    }
    __syncthreads();
}

// One pass of a merge sort over n 64-bit keys in global memory: runs of w sorted keys in `src` are merged pairwise
// into `dst`. Every key finds its place by a binary search in the partner run — the lower bound for a key of the left
// run, the upper bound for one of the right run, so equal keys would still land in distinct slots. Four searches
// per thread are interleaved to overlap their memory latencies.
__device__ void merge_pass(const unsigned long long* src, unsigned long long* dst,
                           uint32_t n, uint32_t w)
{
    for (uint32_t i0 = threadIdx.x * 4u; i0 < n; i0 += kThreads * 4u) {
        unsigned long long key[4];
        uint32_t lo[4], hi[4], own[4], base[4];
        bool right[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t i = i0 + (uint32_t)k;
            lo[k] = hi[k] = own[k] = base[k] = 0;
            right[k] = false;
            key[k] = 0;
            if (i < n) {
                key[k] = src[i];
                const uint32_t pair = i / (2u * w), in_pair = i - pair * 2u * w;
                const uint32_t l0 = pair * 2u * w, l1 = min(l0 + w, n), r1 = min(l0 + 2u * w, n);
                const bool left = in_pair < w;
                right[k] = !left;
                own[k] = left ? (i - l0) : (i - l1);
                base[k] = l0;
                lo[k] = left ? l1 : l0;      // partner run [lo, hi)
                hi[k] = left ? r1 : l1;
            }
        }
        uint32_t a[4], b[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            a[k] = lo[k];
            b[k] = hi[k];
        }
        bool busy = true;
        while (busy) { // four searches in step
            busy = false;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (a[k] < b[k]) {
                    const uint32_t mid = (a[k] + b[k]) >> 1;
                    const unsigned long long v = src[mid];
                    if (v < key[k] || (right[k] && v == key[k]))
                        a[k] = mid + 1;
                    else
                        b[k] = mid;
                    busy = true;
                }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (i0 + (uint32_t)k < n)
                dst[base[k] + own[k] + (a[k] - lo[k])] = key[k];
    }
}

// Where a row's results go (the output pointers of the launch), for the steps that live out of line.
struct RowOut {
    int32_t* token;
    float* prob;
    uint32_t* flags;
    uint32_t* n_cand;
    int32_t* accepted;
    float* total_out;
    int32_t* cand_ids;
    float* cand_q;
    uint32_t cand_cap;
    int32_t id_offset;
    unsigned long long* timing;
    int mode;
};

// More candidates than the shared-memory sort holds, and no truncation orders them: the draw walks them in ascending
// id (sampler.cpp:64-73). The exact weights are laid out by column in scratch (`qrow`) and one thread adds and walks
// them in the reference's order and precision; the other threads stage tiles for it (`stage`: two tiles of shared
// memory). Writes the row's results. Whole CTA.
__device__ __noinline__ void wide_id_ordered(Smem& s, float* stage, const uint2* scratch, float* qrow, uint32_t n_raw,
                                             uint32_t n, uint32_t V, float thr_final, float m, float inv_t, float minp_eff,
                                             uint32_t row, uint32_t flags, float u_row, float u2_row, int32_t draft_row,
                                             const RowOut o)
{
    const uint32_t tid = threadIdx.x;
    for (uint32_t i = tid; i < V; i += kThreads)
        qrow[i] = 0.0f;
    __syncthreads();
    for (uint32_t i = tid; i < n_raw; i += kThreads) {
        const uint2 c = scratch[i];
        if (!(__uint_as_float(c.x) >= thr_final))
            continue;
        const float q = expf_host_exact(__fmul_rn(__fsub_rn(__uint_as_float(c.x), m), inv_t));
        if (q >= minp_eff && q > 0.0f)
            qrow[c.y] = q;
    }
    __threadfence_block();
    __syncthreads();
    const int32_t draft_col = (o.mode == kModeVerify) ? (draft_row - o.id_offset) : -1;
    float total = 0.0f, q_draft = 0.0f;
    // pass 0: float total (and the draft's weight); pass 1: the walk
    float r = 0.0f, walk_total = 0.0f, eps = 0.0f;
    int32_t tok = -1, last = -1, acc = 0;
    float prob = 0.0f, last_q = 0.0f;
    bool first = true, done = false, skip_draft = false;
    uint32_t emitted = 0;
    for (int pass = 0; pass < 2 && !done; ++pass) {
        for (uint32_t t = 0; t * kTile < V && !done; ++t) {
            const uint32_t base = t * kTile, n_t = min((uint32_t)kTile, V - base);
            float* buf = stage + (t & 1) * kTile;
            for (uint32_t e = tid; e < n_t; e += kThreads)
                buf[e] = qrow[base + e];
            __syncthreads();
            if (tid == 0) {
                if (pass == 0) {
                    for (uint32_t e = 0; e < n_t; ++e) {
                        const float q = buf[e];
                        if (q > 0.0f) {
                            total = __fadd_rn(total, q);
                            if ((int32_t)(base + e) == draft_col)
                                q_draft = q;
                            if (emitted < o.cand_cap) {
                                if (o.cand_ids) o.cand_ids[(size_t)row * o.cand_cap + emitted] = (int32_t)(base + e) + o.id_offset;
                                if (o.cand_q) o.cand_q[(size_t)row * o.cand_cap + emitted] = q;
                            }
                            ++emitted;
                        }
                    }
                } else {
                    for (uint32_t e = 0; e < n_t && !done; ++e) {
                        const float q = buf[e];
                        if (!(q > 0.0f) || (skip_draft && (int32_t)(base + e) == draft_col))
                            continue;
                        last = (int32_t)(base + e);
                        last_q = q;
                        if (r < q) {
                            tok = last;
                            prob = __fdiv_rn(q, walk_total);
                            if ((!first && r < eps) || __fsub_rn(q, r) < eps)
                                s.flags = 1; // upper boundary: cleared below if this was the last candidate
                            s.n_final = (!first && r < eps) ? 2u : 0u;
                            done = true;
                        } else {
                            r = __fsub_rn(r, q);
                            first = false;
                        }
                    }
                }
            }
            __syncthreads();
            if (pass == 1) {
                // the walking thread publishes "done" through shared memory
                if (tid == 0)
                    s.nsurv = done ? 0xffffffffu : n;
                __syncthreads();
                done = s.nsurv == 0xffffffffu;
            }
        }
        if (pass == 0) {
            // decide what the walk does (sampler.cpp:100-106 for verify)
            if (tid == 0) {
                walk_total = total;
                if (o.mode == kModeVerify) {
                    acc = __fmul_rn(u_row, total) < q_draft;
                    if (acc) {
                        tok = draft_col + o.id_offset;
                        prob = __fdiv_rn(q_draft, total);
                    } else {
                        skip_draft = true;
                        walk_total = __fsub_rn(total, q_draft);
                    }
                }
                const float uu = (o.mode == kModeVerify) ? u2_row : u_row;
                r = __fmul_rn(uu, walk_total);
                eps = 1e-6f * walk_total;
                s.n_final = 0;
                s.flags = 0;
                s.nsurv = (o.mode == kModeDistOnly || acc) ? 0xffffffffu : n;
            }
            __syncthreads();
            done = s.nsurv == 0xffffffffu;
        }
    }
    if (tid == 0) {
        if (o.mode == kModeDistOnly) {
            tok = -1;
        } else if (tok < 0) { // rounding: the last candidate
            tok = last;
            prob = __fdiv_rn(last_q, walk_total);
        } else if (!acc && o.mode != kModeDistOnly) {
            // near-boundary report: lower boundary always counts; the upper one only if a candidate follows
            bool more = false;
            for (uint32_t c = (uint32_t)tok + 1; c < V && !more; ++c)
                if (qrow[c] > 0.0f && !(skip_draft && (int32_t)c == draft_col))
                    more = true;
            if (s.n_final == 2u || (s.flags && more))
                flags |= MK_FLAG_NEAR_CDF_BOUNDARY;
        }
        if (o.token) o.token[row] = (tok >= 0 && !(acc)) ? tok + o.id_offset : tok;
        if (o.prob) o.prob[row] = prob;
        if (o.flags) o.flags[row] = flags;
        if (o.n_cand) o.n_cand[row] = n;
        if (o.accepted) o.accepted[row] = acc;
        if (o.total_out) o.total_out[row] = total;
        if (o.timing) o.timing[(size_t)row * 64 + 3] = global_ns();
    }
}

// sampler.cpp:44-61 for a list longer than one warp walks: the shortest prefix of the sorted list whose double sum
// reaches top_p * total. The sums are taken by the whole CTA (each thread a contiguous run of the list, then a scan
// over threads); their rounding differs from the reference's left-to-right sum by far less than the margin inside
// which a decision is reported. Returns the prefix length; bit 31 set: the list ended before the nucleus did
// (`need_sum` rows), or the decision lies within the margin. `total_need`/`band_need`: the row total and its margin
// when the total covers more than the list (`use_row_total`).
__device__ __noinline__ uint32_t wide_top_p(Smem& s, const unsigned long long* ksrc, uint32_t n, float top_p, bool need_sum,
                                            bool use_row_total, double total_need, double band_need)
{
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t per = (n + kThreads - 1) / kThreads;
    const uint32_t r0 = min(tid * per, n), r1 = min(r0 + per, n);
    double mine = 0.0;
    for (uint32_t r = r0; r < r1; ++r)
        mine += (double)__uint_as_float(~(uint32_t)(ksrc[r] >> 32));
    double inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double y = __shfl_up_sync(0xffffffffu, inc, o);
        if ((int)lane >= o)
            inc += y;
    }
    __syncthreads(); // warp_sum may still be read
    if (lane == 31)
        s.warp_sum[warp] = inc;
    if (tid == 0)
        s.n_final = n;
    __syncthreads();
    double before = inc - mine, list_total = 0.0;
    for (uint32_t w = 0; w < (uint32_t)(kThreads / 32); ++w) {
        if (w < warp)
            before += s.warp_sum[w];
        list_total += s.warp_sum[w];
    }
    double total, band;
    if (use_row_total) {
        total = total_need;
        band = band_need + 0x1p-36 * total;
    } else {
        total = list_total;
        band = 0x1p-36 * total;
    }
    const double want = (double)top_p * total;
    {
        double run = before;
        for (uint32_t r = r0; r < r1; ++r) {
            run += (double)__uint_as_float(~(uint32_t)(ksrc[r] >> 32));
            if (!(run < want)) {
                atomicMin(&s.n_final, r + 1u);
                break;
            }
        }
    }
    __syncthreads();
    const uint32_t k = s.n_final; // candidates taken: the first count whose sum is not below `want`, else all
    __syncthreads();
    {
        double run = before;
        for (uint32_t r = r0; r < r1; ++r) {
            const double prev = run;
            run += (double)__uint_as_float(~(uint32_t)(ksrc[r] >> 32));
            if (r + 1u == k) {
                s.warp_sum[0] = run;
                s.warp_sum[1] = prev;
            }
        }
    }
    __syncthreads();
    const double run = s.warp_sum[0], prev = s.warp_sum[1];
    const bool unsure = (need_sum && run < want) ||
                        (k >= 1 && (fabs(run - want) <= band || (k >= 2 && fabs(prev - want) <= band)));
    return k | (unsure ? 0x80000000u : 0u);
}

// A sweep of the whole CTA over a row's collected (logit, column) pairs in global memory, two pairs per 16-byte load
// and eight loads of every thread in flight: such a list is read at the pace of its loads' latency, so the bytes in
// flight are what counts. `f(logit bits, column)` is called once per pair, in no particular order.
template <class F>
__device__ __forceinline__ void for_each_collected(const uint2* scratch, uint32_t n_raw, F&& f)
{
    const uint4* const s4 = reinterpret_cast<const uint4*>(scratch); // a row's scratch starts on a 16-byte boundary
    const uint32_t n_pairs = (n_raw + 1u) >> 1;
    for (uint32_t p0 = threadIdx.x; p0 < n_pairs; p0 += 8u * kThreads) {
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t p = p0 + (uint32_t)k * kThreads;
            v[k] = (p < n_pairs) ? s4[p] : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t p = p0 + (uint32_t)k * kThreads;
            if (p < n_pairs) {
                f(v[k].x, v[k].y);
                if (2u * p + 1u < n_raw)
                    f(v[k].z, v[k].w);
            }
        }
    }
}

// top_p alone, a long collected list: the nucleus leaves out a tail of mass (1 - top_p) * total. Everything that was
// not collected belongs to that tail; collected elements can join it from the bottom for as long as the tail stays
// within the budget. Approximate weights decide the cut (with margins) and raise s.thr_topk_key; the nucleus itself
// is then computed from exact weights, and a cut that turns out too tight is reported. Whole CTA. (Out of line, like
// the other steps few rows need: what the common row runs stays short and contiguous.)
//
// The cut is found in one sweep over the collected logits that sorts their approximate weights into kCutBins equal
// steps of the logit between the bound in force and the row maximum (a step is a fraction of a logit: what a finer
// cut would still drop is a few per cent of the list; the loop below would refine it, and one sweep of a long list
// costs more than that). Every thread keeps its own bins (`ph`, kCutBins x kThreads floats, the thread index innermost: no two lanes
// share a bank), so nothing is atomic; the bins are summed over the threads afterwards. A logit below the value
// lo + c * width has a bin index of at most c (the index is monotone in the logit), so "everything below that value"
// weighs no more than the mass below `lo` plus bins 0..c: the largest c for which that fits the budget is taken.
constexpr int kCutBins = 64;
static_assert((uint32_t)kCutBins * kThreads * 4u + (uint32_t)kCutBins * 8u <= kDynBytes, "the cut's bins fit");
__device__ __noinline__ void mass_cut(Smem& s, unsigned char* dyn, const uint2* scratch, uint32_t n_raw, float thr_final,
                                      float m, float inv_t, float top_p, double total_approx)
{
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    float* const ph = reinterpret_cast<float*>(dyn);
    double* const bin_total = reinterpret_cast<double*>(dyn + (size_t)kCutBins * kThreads * 4u);
    const float c2 = inv_t * 1.4426950408889634f;
    float lo = thr_final, hi = m;
    double budget = 0.0;
    for (int sweep = 0; sweep < 1; ++sweep) {
        if (!(hi > lo)) // also false for NaN
            break;
        const float width = (hi - lo) * (1.0f / (float)kCutBins);
        const float scale = (float)kCutBins / (hi - lo);
        if (!(width > 0.0f) || !(scale < __int_as_float(0x7f800000)))
            break;
        for (int b = 0; b < kCutBins; ++b)
            ph[b * kThreads + tid] = 0.0f;
        if (tid == 0)
            s.warp_sum[0] = s.warp_sum[1] = 0.0;
        __syncthreads();
        double all = 0.0, low = 0.0; // every collected element; those below `lo`
        float all_f = 0.0f, low_f = 0.0f; // a thread's share: at most a few hundred terms each
        for_each_collected(scratch, n_raw, [&](uint32_t bits, uint32_t) {
            const float w = __uint_as_float(bits);
            const float qa = ex2_approx((w - m) * c2);
            all_f += qa;
            if (w < lo) {
                low_f += qa;
            } else if (w < hi) {
                const int b = min(kCutBins - 1, (int)((w - lo) * scale));
                ph[b * kThreads + tid] += qa;
            }
        });
        all = (double)all_f;
        low = (double)low_f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            all += __shfl_xor_sync(0xffffffffu, all, o);
            low += __shfl_xor_sync(0xffffffffu, low, o);
        }
        if (lane == 0) {
            atomicAdd(&s.warp_sum[0], all);
            atomicAdd(&s.warp_sum[1], low);
        }
        __syncthreads();
        for (int b = (int)warp; b < kCutBins; b += kThreads / 32) { // a warp per bin: the threads' shares, summed
            double t = 0.0;
            for (uint32_t j = lane; j < (uint32_t)kThreads; j += 32u)
                t += (double)ph[b * kThreads + j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0)
                bin_total[b] = t;
        }
        __syncthreads();
        if (sweep == 0) {
            const double collected = s.warp_sum[0];
            const double total_est = collected + total_approx; // total_approx: what was never collected
            budget = (1.0 - (double)top_p) * total_est * 0.999 - (total_approx + 1e-5 * total_est);
        }
        // every thread walks the 64 bin totals itself (the same values, the same result)
        double upto = s.warp_sum[1];
        int cut = -1; // the largest c whose bins 0..c, with everything below `lo`, fit the budget
        for (int b = 0; b < kCutBins; ++b) {
            upto += bin_total[b];
            if (upto <= budget)
                cut = b;
            else
                break;
        }
        __syncthreads(); // bin_total, warp_sum and ph are written again by the next sweep and the caller
        if (!(budget > 0.0) || cut < 0)
            break; // nothing more can be left out at this resolution
        const float new_lo = lo + (float)cut * width;
        hi = fminf(hi, lo + (float)(cut + 2) * width);
        lo = new_lo;
        if (tid == 0 && lo > thr_final)
            s.thr_topk_key = max(s.thr_topk_key, order_key(lo));
    }
    __syncthreads();
}

// More candidates than the shared-memory sort holds, in an order that matters: the survivors (exact weight, min_p) are
// compacted into the second half of the row's scratch as sort keys, sorted as kSortCap-key runs in shared memory,
// then merged pairwise between the two halves. Returns where the sorted list of n keys ends up. Whole CTA.
__device__ __noinline__ const unsigned long long* long_sort(Smem& s, unsigned long long* keys, uint2* scratch, uint32_t cap,
                                                            uint32_t n_raw, uint32_t n, float thr2, float m, float inv_t,
                                                            float minp_eff)
{
    const uint32_t tid = threadIdx.x;
    unsigned long long* KA = reinterpret_cast<unsigned long long*>(scratch) + cap; // second half
    unsigned long long* KB = reinterpret_cast<unsigned long long*>(scratch);                 // over the raw list
    if (tid == 0)
        s.nsurv = 0;
    __syncthreads();
    for (uint32_t i0 = tid; i0 < n_raw; i0 += 4u * kThreads) { // survivors, compacted, as sort keys
        uint2 cv[4]; // four loads in flight
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t i = i0 + (uint32_t)k * kThreads;
            cv[k] = (i < n_raw) ? scratch[i] : make_uint2(0xff800000u, 0u); // filler: -inf, below any bound
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint2 c = cv[k];
            if (__uint_as_float(c.x) >= thr2) {
                const float q = expf_host_exact(__fmul_rn(__fsub_rn(__uint_as_float(c.x), m), inv_t));
                if (q >= minp_eff && q > 0.0f)
                    KA[atomicAdd(&s.nsurv, 1u)] = pack_by_weight(q, c.y);
            }
        }
    }
    __syncthreads();
    for (uint32_t r0 = 0; r0 < n; r0 += (uint32_t)kSortCap) {
        for (uint32_t i = tid; i < (uint32_t)kSortCap; i += kThreads)
            keys[i] = (r0 + i < n) ? KA[r0 + i] : ~0ull;
        __syncthreads();
        block_sort(keys, (uint32_t)kSortCap);
        for (uint32_t i = tid; i < (uint32_t)kSortCap; i += kThreads)
            if (r0 + i < n)
                KA[r0 + i] = keys[i];
        __syncthreads();
    }
    const unsigned long long* P = KA;
    {
        unsigned long long *src = KA, *dst = KB;
        for (uint32_t w = (uint32_t)kSortCap; w < n; w <<= 1) {
            merge_pass(src, dst, n, w);
            __syncthreads();
            unsigned long long* t = src;
            src = dst;
            dst = t;
        }
        P = src;
    }
    return P;
}

constexpr uint32_t kWideCand = 64;
// The one-warp finish of row_pipeline_kernel for 33 to 64 candidates (a top_k of 40 or 50): the same steps with two
// candidates a lane — a 64-key network, its last level between a lane's own two keys — and chains that take candidate
// j from register j / 32 of lane j % 32 (sampler.cpp:39-73, 86-107). Called by warp 0 with the candidates' (weight,
// column) pairs in `fkeys`. Out of line: the rows it does not serve run the code they always ran.
__device__ __noinline__ void wide_finish(Smem& s, const unsigned long long* fkeys, uint32_t n, uint32_t top_k, bool use_topp,
                                         float top_p, float inv_t, float m, uint32_t flags, int32_t draft_row, float u_row,
                                         float u2_row, uint32_t row, RowOut o)
{
    const uint32_t full = 0xffffffffu, lane = threadIdx.x & 31u;
    const int mode = o.mode;
    const int32_t id_off = o.id_offset;
    uint32_t fl = flags;
    const bool cut_k = top_k > 0 && top_k < n; // sampler.cpp:39
    const bool sorted = cut_k || use_topp;         // else ascending id
    unsigned long long key[2];
#pragma unroll
    for (uint32_t r = 0; r < 2; ++r) {
        key[r] = ~0ull;
        if (r * 32u + lane < n) {
            const unsigned long long raw = fkeys[r * 32u + lane];
            const float q = __uint_as_float((uint32_t)(raw >> 32));
            const uint32_t col = (uint32_t)(raw & 0xffffffffull);
            key[r] = sorted ? pack_by_weight(q, col) : pack_by_column(q, col);
        }
    }
    for (uint32_t k = 2; k <= 64u; k <<= 1)
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            if (j == 32u) { // k == 64: element `lane` against element `lane + 32`, ascending
                const unsigned long long lo = min(key[0], key[1]), hi = max(key[0], key[1]);
                key[0] = lo;
                key[1] = hi;
            } else {
#pragma unroll
                for (uint32_t r = 0; r < 2; ++r) {
                    const uint32_t i = r * 32u + lane;
                    const unsigned long long other = __shfl_xor_sync(full, key[r], j);
                    const bool keep_small = ((i & j) == 0) == ((i & k) == 0);
                    key[r] = (keep_small == (key[r] < other)) ? key[r] : other;
                }
            }
        }
    float q[2];
    uint32_t col[2];
#pragma unroll
    for (uint32_t r = 0; r < 2; ++r) {
        if (sorted) {
            q[r] = __uint_as_float(~(uint32_t)(key[r] >> 32));
            col[r] = (uint32_t)(key[r] & 0xffffffffull);
        } else {
            q[r] = __uint_as_float((uint32_t)(key[r] & 0xffffffffull));
            col[r] = (uint32_t)(key[r] >> 32);
        }
        if (r * 32u + lane >= n)
            q[r] = 0.0f;
    }
    auto q_at = [&](uint32_t j) -> float { return __shfl_sync(full, j < 32u ? q[0] : q[1], (int)(j & 31u)); };
    auto col_at = [&](uint32_t j) -> uint32_t { return __shfl_sync(full, j < 32u ? col[0] : col[1], (int)(j & 31u)); };
    if (cut_k) { // sampler.cpp:40-42; the tie rule is the general finish's
        const float qk = q_at(top_k - 1u);
        const uint32_t edge_key = s.thr_topk_key;
        const float below = key_to_float(edge_key - 1u);
        if (edge_key > order_key(-FLT_MAX) && expf_host_exact(__fmul_rn(__fsub_rn(below, m), inv_t)) >= qk)
            fl |= MK_FLAG_GUARD_BAND;
        n = top_k;
    }
    if (use_topp) { // sampler.cpp:44-61, sequentially
        double total_d = 0.0;
        for (uint32_t j = 0; j < n; ++j)
            total_d += (double)q_at(j);
        const double band = 0x1p-40 * total_d, want = (double)top_p * total_d;
        double run = 0.0, prev = 0.0;
        uint32_t k = 0;
        for (uint32_t j = 0; j < n && run < want; ++j) {
            prev = run;
            run += (double)q_at(j);
            k = j + 1u;
        }
        if (k >= 1 && (fabs(run - want) <= band || (k >= 2 && fabs(prev - want) <= band)))
            fl |= MK_FLAG_GUARD_BAND;
        n = max(k, 1u);
    }
#pragma unroll
    for (uint32_t r = 0; r < 2; ++r)
        if (r * 32u + lane >= n)
            q[r] = 0.0f;
    float total = 0.0f;
    for (uint32_t j = 0; j < n; ++j)
        total = __fadd_rn(total, q_at(j));
    const int32_t draft = (mode == kModeVerify) ? draft_row : -1;
    const uint32_t dm0 = __ballot_sync(full, draft >= 0 && lane < n && (int32_t)col[0] + id_off == draft);
    const uint32_t dm1 = __ballot_sync(full, draft >= 0 && 32u + lane < n && (int32_t)col[1] + id_off == draft);
    const uint32_t draft_idx = dm0 ? (uint32_t)__ffs((int)dm0) - 1u : (dm1 ? 31u + (uint32_t)__ffs((int)dm1) : 0xffffffffu);
    const float q_draft = (dm0 | dm1) ? q_at(draft_idx) : 0.0f;
    int32_t tok = -1, acc = 0;
    float prob = 0.0f;
    if (mode == kModeDistOnly) {
        tok = (int32_t)col_at(0) + id_off;
        prob = __fdiv_rn(q_at(0), total);
    } else {
        uint32_t skip_idx = 0xffffffffu;
        float walk_total = total;
        if (mode == kModeVerify) { // sampler.cpp:100-106
            acc = __fmul_rn(u_row, total) < q_draft;
            if (acc) {
                tok = draft;
                prob = __fdiv_rn(q_draft, total);
            } else {
                skip_idx = draft_idx;
                walk_total = __fsub_rn(total, q_draft);
                if (n == 1 && draft_idx == 0u) { // nothing but the rejected draft
                    tok = draft;
                    prob = 1.0f;
                }
            }
        }
        if (tok < 0) {
            float r = __fmul_rn((mode == kModeVerify) ? u2_row : u_row, walk_total);
            const float eps = 1e-6f * walk_total;
            const uint32_t first_valid = (skip_idx == 0u) ? 1u : 0u;
            const uint32_t last_valid = (skip_idx == n - 1u) ? n - 2u : n - 1u;
            if (lane == skip_idx)
                q[0] = 0.0f; // the skipped draft never wins
            if (32u + lane == skip_idx)
                q[1] = 0.0f;
            uint32_t hit = last_valid; // rounding: the last candidate (sampler.cpp:72)
            float q_hit = q_at(last_valid);
            bool found = false;
            for (uint32_t j = 0; j < n && !found; ++j) {
                const float qj = q_at(j);
                if (r < qj) {
                    found = true;
                    hit = j;
                    q_hit = qj;
                    // boundary below (not for the first candidate) or above (not for the last)
                    if ((j != first_valid && r < eps) || (j < last_valid && __fsub_rn(qj, r) < eps))
                        fl |= MK_FLAG_NEAR_CDF_BOUNDARY;
                } else {
                    r = __fsub_rn(r, qj);
                }
            }
            tok = (int32_t)col_at(hit) + id_off;
            prob = __fdiv_rn(q_hit, walk_total);
        }
    }
    if (lane == 0) {
        if (o.token) o.token[row] = tok;
        if (o.prob) o.prob[row] = prob;
        if (o.flags) o.flags[row] = fl;
        if (o.n_cand) o.n_cand[row] = n;
        if (o.accepted) o.accepted[row] = acc;
        if (o.total_out) o.total_out[row] = total;
        if (o.timing)
            o.timing[(size_t)row * 64 + 3] = global_ns();
    }
    // the candidate list as the chains saw it, except that a rejected draft keeps its weight there
#pragma unroll
    for (uint32_t r = 0; r < 2; ++r) {
        const uint32_t i = r * 32u + lane;
        if (i < min(n, o.cand_cap)) {
            const float qo = sorted ? __uint_as_float(~(uint32_t)(key[r] >> 32)) : __uint_as_float((uint32_t)(key[r] & 0xffffffffull));
            if (o.cand_ids) o.cand_ids[(size_t)row * o.cand_cap + i] = (int32_t)col[r] + id_off;
            if (o.cand_q) o.cand_q[(size_t)row * o.cand_cap + i] = qo;
        }
    }
}

} // namespace

// kSpec: the rows of a speculative round (row = sequence * n_pos + position); compiled apart, so that the plain
// kernel carries none of its bookkeeping.
// kSplit: a launch whose grid has a second dimension over column shards of every row (shard records of a few rows
// split over many CTAs: the single-row latency path).
template <bool kSpec, bool kSplit>
__global__ void __launch_bounds__(kThreads, 2) row_pipeline_kernel(const RowKernelArgs a)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>(smem_raw);

    const uint32_t row = blockIdx.x;
    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31;
    // a split launch: CTA (row, g) takes columns [g * split_w, ...) of the row, and that share of the row's scratch
    const uint32_t col0 = kSplit ? blockIdx.y * a.split_w : 0u;
    const uint32_t V = kSplit ? min(a.split_w, a.n_vocab - col0) : a.n_vocab;
    const int32_t id_off = kSplit ? a.id_offset + (int32_t)col0 : a.id_offset;
    const uint32_t scratch_cap = kSplit ? min(a.split_w, a.scratch_cap - col0) : a.scratch_cap;
    const uint32_t n_tiles = (V + kTile - 1) / kTile;
    const float* __restrict__ lrow = a.logits + (size_t)row * a.ld + col0;
    // A speculative round (src/gen/session.cpp:451-506): row = sequence * n_pos + position. Position j < n_pos - 1
    // verifies draft j, the last one is the bonus row and is sampled; the penalties of position j count the sequence's
    // history plus drafts 0..j-1 (each accepted draft is emit()ted before the next row is looked at, :491); a forced
    // token takes the place of the sampler and draws nothing (:481-484), so the position's uniforms are found by
    // counting the positions before it that are not forced.
    constexpr bool spec = kSpec;
    const uint32_t seq = spec ? row / a.spec_n_pos : row, pos = spec ? row - seq * a.spec_n_pos : 0u;
    const int mode = spec ? ((pos + 1u == a.spec_n_pos) ? (int)kModeSample : (int)kModeVerify) : a.mode;
    const int32_t* __restrict__ extra = spec ? a.spec_drafts + (size_t)seq * (a.spec_n_pos - 1u) : nullptr;
    const uint32_t n_extra = spec ? pos : 0u;
    // Launched programmatically behind the previous kernel of the stream, this grid may start while that one still
    // runs. Nothing that kernel may have written is touched before griddep_wait() — which comes first thing, unless
    // the caller has declared the side inputs (parameters, histories, biases) stable: then the whole set-up runs
    // ahead and only the logits, the mask, the uniforms and every write to global memory wait. The second pass reads
    // a word the first pass wrote: it always waits first.
    const bool early = a.overlap == MK_OVERLAP_STABLE_SIDE_INPUTS && a.pass == 0;
    // Probes a wait for a tile makes before it gives up (each parks the thread for up to 20 us): seconds normally, a
    // few milliseconds with the test hook that withholds a tile.
    const uint32_t wait_probes = a.debug_wait_probes ? a.debug_wait_probes : (1u << 17);
    if (!early)
        griddep_wait();
    const mk_sampling_params prm = a.params_dev ? a.params_dev[row] : a.params;
    // Whether the history matters is known from three comparisons; its loads (the first thing the set-up waits for)
    // are issued before the rest of the parameters is worked out.
    // A per-row length read from device memory is clamped to what the row's buffer holds and to the 16-bit counters
    // of the long-history path; a clamp that bites is reported in the row's flags (MK_FLAG_HISTORY_FULL).
    const uint32_t hlen_cap = (uint32_t)min((uint64_t)65535u, a.history_ld);
    const uint32_t hlen_dev = (a.history && a.history_len) ? (uint32_t)max(a.history_len[seq], 0) : 0u;
    const bool hlen_clamped = hlen_dev > hlen_cap;
    const uint32_t hlen_base = a.history ? (a.history_len ? min(hlen_dev, hlen_cap) : a.n_history) : 0u;
    const uint32_t hlen_all = hlen_base + n_extra;
    const bool has_hist = !(prm.temperature <= 0.0f) && hlen_all > 0 &&
                          !(prm.repetition_penalty == 1.0f && prm.presence_penalty == 0.0f && prm.frequency_penalty == 0.0f);
    const uint32_t hlen = has_hist ? hlen_all : 0u;
    const int32_t* __restrict__ hrow = a.history ? a.history + (size_t)seq * a.history_ld : nullptr;
    auto hist_at = [&](uint32_t j) -> int32_t {
        if constexpr (kSpec)
            return j < hlen_base ? __ldg(hrow + j) : __ldg(extra + (j - hlen_base));
        else
            return __ldg(hrow + j);
    };
    const uint32_t nb = a.bias ? a.n_bias : 0u;
    const mk_bias* __restrict__ brow = a.bias ? a.bias + (size_t)row * a.n_bias : nullptr;
    // Columns whose value is not the one in memory — biased tokens and generated tokens (penalties) — are edited by
    // two fix-up warps in every tile in shared memory before the readers see it. While the history is short (the
    // usual case) a bitmap names the generated columns, with rank-indexed counts behind it, and a tile's columns are
    // spread over the lanes by rank; a longer history, or a vocabulary beyond the bitmap, takes the slower path where
    // one warp matches the whole history against every tile. The few bias entries are matched against each tile.
    const bool has_special = has_hist || nb > 0;
    const bool use_table = has_hist && hlen <= (uint32_t)kHistCap && V <= kMaxBitmapVocab;
    const bool long_history = has_hist && !use_table;
    // The history is read into registers first thing, all loads in flight together, so that their latency
    // overlaps the barrier set-up instead of being paid once per loop trip.
    constexpr int kHistPerThread = (kHistCap + kThreads - 1) / kThreads;
    uint32_t hc[kHistPerThread]; // the entries as columns of this row (ids outside it: 0xffffffff, as past-the-end)
    if (use_table) {
#pragma unroll
        for (int i = 0; i < kHistPerThread; ++i) {
            const uint32_t j = (uint32_t)i * kThreads + tid;
            hc[i] = (j < hlen) ? (uint32_t)hist_at(j) - (uint32_t)id_off : 0xffffffffu;
        }
    }
    const RowCfg cfg = make_cfg(prm, V, mode, a.vp_k, a.pass);
    const uint32_t* __restrict__ mrow = a.mask ? a.mask + (size_t)row * a.mask_ld + (col0 >> 5) : nullptr;
    // Per-row scratch, 16 bytes per column: scratch_cap raw candidates (logit bits, column) — sorted in place as
    // 64-bit keys by the large sorted-list path — then as much again: the merge sort's second buffer, or (large
    // unsorted lists) one float per column.
    uint32_t* const row_scratch = a.scratch + (size_t)row * row_scratch_words(a.scratch_cap) + 4ull * col0;
    uint2* __restrict__ scratch = reinterpret_cast<uint2*>(row_scratch);
    float* __restrict__ qrow = reinterpret_cast<float*>(row_scratch + 2u * scratch_cap);
    uint32_t* const again = row_scratch + 4u * scratch_cap; // set by the first launch: this row wants the second pass
    if (spec && a.spec_forced) {
        const int32_t f = __ldg(a.spec_forced + row);
        if (f >= 0) { // the sampler is bypassed: the token is the forced one, a draft is kept only if it matches
            if (early)
                griddep_wait();
            if (tid == 0 && a.pass == 0) {
                if (a.token) a.token[row] = f;
                if (a.prob) a.prob[row] = 1.0f;
                if (a.flags) a.flags[row] = 0u;
                if (a.n_cand) a.n_cand[row] = 0u;
                if (a.accepted) a.accepted[row] = (mode == kModeVerify && f == __ldg(extra + pos)) ? 1 : 0;
            }
            return;
        }
    }
    if (a.pass == 1 && again[0] == 0u)
        return;
    if (a.only_flagged && !(a.only_flagged[row] & a.only_flagged_mask))
        return; // a follow-up launch for the rows an earlier step reported: the others are done
    // ---- shared-memory layout of the streaming phase ---------------------------------------------------------------
    const uint32_t bm_words = (V + 31u) / 32u;
    unsigned char* const dyn = smem_raw + kHeadBytes;
    uint32_t off = 0;
    uint32_t* const bitmap = reinterpret_cast<uint32_t*>(dyn + off); // long histories: per-tile id counters instead
    off += use_table ? ((bm_words * 4u + 15u) & ~15u) : (long_history ? (uint32_t)kTile * 2u : 0u);
    uint16_t* const wpre = reinterpret_cast<uint16_t*>(dyn + off); // rank of each bitmap word's first set bit
    off += use_table ? ((bm_words * 2u + 15u) & ~15u) : 0u;
    uint32_t* const counts = reinterpret_cast<uint32_t*>(dyn + off); // by rank: occurrences, two per word
    off += use_table ? (uint32_t)kHistCap * 2u : 0u;
    uint32_t* const hist = reinterpret_cast<uint32_t*>(dyn + off);
    off += cfg.hist_mode ? (uint32_t)kBins * 4u : 0u;
    off = (off + 127u) & ~127u;
    float* const ring = reinterpret_cast<float*>(dyn + off);
    const uint32_t n_stages = min((uint32_t)kMaxStages, (kDynBytes - off) / ((uint32_t)kTile * 4u)); // >= 4
    // ---- set-up -------------------------------------------------------------------------------------------------
    if (a.timing && tid == 0 && !early)
        a.timing[(size_t)row * 64 + 0] = global_ns();
    const unsigned long long t_begin = (a.timing && tid == 0 && early) ? global_ns() : 0ull;
    if (tid == 0) {
        for (int i = 0; i < kMaxStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.ready[i], 1);
            mbar_init(&s.empty[i], kReaderWarps);
        }
        s.best_key = 0ull;
        s.m_key = order_key(-__int_as_float(0x7f800000));
        s.thr_topk_key = order_key(-FLT_MAX);
        s.ncand = 0;
        s.nsurv = 0;
        s.abort_flag = 0;
        s.nan0 = 0;
        s.hi_group = 0;
        s.first_tile_warps = 0;
        s.n_final = 0;
        s.flags = 0;
        s.n_distinct = 0;
        s.n_own = 0;
        fence_barrier_init();
    }
    uint32_t* const cnt = bitmap; // long histories: per-tile id counters (two 16-bit counters per word)
    if (long_history)
        for (uint32_t i = tid; i < kTile / 2; i += kThreads)
            cnt[i] = 0;
    if (cfg.hist_mode)
        for (uint32_t i = tid; i < kBins; i += kThreads)
            hist[i] = 0;
    if (use_table) { // bitmap, ranks and counts are contiguous and 16-byte aligned: cleared with 128-bit stores
        uint4* const z = reinterpret_cast<uint4*>(bitmap);
        const uint32_t nz = (uint32_t)(reinterpret_cast<unsigned char*>(counts + kHistCap / 2) -
                                       reinterpret_cast<unsigned char*>(bitmap)) / 16u;
        for (uint32_t i = tid; i < nz; i += kThreads)
            z[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    if (a.timing && tid == 0 && !early)
        a.timing[(size_t)row * 64 + 6] = global_ns();
    // The producer fills the ring before anything else, so that the copies fly during the set-up (unless the set-up
    // runs ahead of the previous kernel: then the logits come after the wait below). With a history the last stage
    // first serves the set-up as a list (see below) and is requested once that list has been used.
    const uint32_t tiles_issued = a.use_bulk_copy ? min(n_stages, n_tiles) : 0u;
    const bool list_owners = use_table && has_hist && tiles_issued > 0;
    const uint32_t tiles_early = (list_owners && tiles_issued == n_stages) ? n_stages - 1u : tiles_issued;
    auto fill_ring = [&](uint32_t t0, uint32_t t1) {
        for (uint32_t t = t0; t < t1; ++t) {
            if (t == a.debug_skip_tile)
                continue; // test hook: this tile's copy is never requested, so that the waits for it run out
            const uint32_t n_t = min((uint32_t)kTile, V - t * kTile);
            const uint32_t bytes = (n_t * 4u) & ~15u;
            const float* src = lrow + (size_t)t * kTile;
            for (uint32_t e = bytes / 4; e < n_t; ++e)
                ring[t * kTile + e] = src[e];
            if (bytes > 0) {
                mbar_arrive_expect_tx(&s.full[t], bytes);
                bulk_load(ring + t * kTile, src, bytes, &s.full[t]);
            } else {
                mbar_arrive(&s.full[t]);
            }
        }
    };
    if (!early && tid == 0)
        fill_ring(0, tiles_early);
    // The first tiles hold the most frequent token ids, by far the largest share of a history: all warps edit
    // their generated columns together before the stream starts. The columns to edit are listed while the bitmap is
    // built — by the history entry that sets a column's bit, so each column once — in the last ring stage.
    const uint32_t prefixed = list_owners ? min((uint32_t)kPrefixTiles, tiles_early) : 0u;
    const uint32_t span = min(prefixed * (uint32_t)kTile, V);
    uint16_t* const own_list = reinterpret_cast<uint16_t*>(ring + (n_stages - 1u) * kTile); // <= kHistCap entries
    if (use_table) {
        // The special columns as a bitmap: all the readers need in order to set them aside. The rest of what the
        // reference keeps about the generated tokens (a multiset id -> count, sampler.cpp:15-18) is built by the
        // side warps while the row already streams.
#pragma unroll
        for (int hi = 0; hi < kHistPerThread; ++hi) {
            bool mine = false;
            if (hc[hi] < V) { // unsigned: an id below the row's first column wraps past V
                const uint32_t col = hc[hi], bit = 1u << (col & 31u);
                if (!(*(volatile uint32_t*)&bitmap[col >> 5] & bit)) // skip the atomic once the bit is visible
                    if (!(atomicOr(&bitmap[col >> 5], bit) & bit))
                        mine = col < span; // exactly one entry per distinct column sees its bit go from 0 to 1
            }
            const uint32_t bal = __ballot_sync(0xffffffffu, mine);
            if (bal) { // one slot range per warp and round
                uint32_t at = 0;
                if (lane == 0)
                    at = atomicAdd(&s.n_own, (uint32_t)__popc(bal));
                at = __shfl_sync(0xffffffffu, at, 0) + (uint32_t)__popc(bal & ((1u << lane) - 1u));
                if (mine)
                    own_list[at] = (uint16_t)hc[hi];
            }
        }
        __syncthreads();
        if (a.timing && tid == 0 && !early)
            a.timing[(size_t)row * 64 + 7] = global_ns();
        // The rest of what the reference keeps about the generated tokens (a multiset id -> count,
        // sampler.cpp:15-18) in a form that needs no search: the number of set bits before each bitmap word (so a
        // column's rank among the special ones is one popcount away) and, by rank, how often the token occurs and
        // its bias.
        word_ranks(s, bitmap, wpre, bm_words);
        __syncthreads();
        if (a.timing && tid == 0 && !early)
            a.timing[(size_t)row * 64 + 8] = global_ns();
        // (ranks of all of a thread's entries first, so that their look-ups are in flight together; then the adds)
        {
            uint32_t rk[kHistPerThread];
#pragma unroll
            for (int hi = 0; hi < kHistPerThread; ++hi) {
                const uint32_t col = hc[hi] < V ? hc[hi] : 0u;
                rk[hi] = wpre[col >> 5] + __popc(bitmap[col >> 5] & ((1u << (col & 31u)) - 1u));
            }
#pragma unroll
            for (int hi = 0; hi < kHistPerThread; ++hi)
                if (hc[hi] < V)
                    atomicAdd(&counts[rk[hi] >> 1], 1u << ((rk[hi] & 1u) * 16u));
        }
        __syncthreads();
        if (a.timing && tid == 0 && !early)
            a.timing[(size_t)row * 64 + 4] = global_ns();
    }
    if (early) {
        griddep_wait();
        if (tid == 0)
            fill_ring(0, tiles_early);
        if (a.timing && tid == 0) {
            a.timing[(size_t)row * 64 + 0] = t_begin;
            a.timing[(size_t)row * 64 + 7] = global_ns();
        }
    }
    griddep_launch_dependents();
    if (a.pass == 0 && tid == 0 && !kSplit)
        again[0] = 0u;
    float u_row = a.u ? __ldg(a.u + (spec ? 0u : row)) : 0.0f;
    float u2_row = a.u2 ? __ldg(a.u2 + row) : 0.0f;
    int32_t draft_row = a.draft ? __ldg(a.draft + row) : -1;
    if constexpr (kSpec) {
        uint32_t drawn = 0; // uniforms the positions before this one consume when every draft before it is kept
        for (uint32_t i = 0; i < pos; ++i)
            drawn += (a.spec_forced && __ldg(a.spec_forced + (size_t)seq * a.spec_n_pos + i) >= 0) ? 0u : 1u;
        const float* useq = a.u + (size_t)seq * (a.spec_n_pos + 1u);
        u_row = __ldg(useq + drawn);
        u2_row = __ldg(useq + drawn + 1u);
        draft_row = (mode == kModeVerify) ? __ldg(extra + pos) : -1;
    }
    if (prefixed > 0) {
        // requested before the set-up, the first tiles have landed by now (requested after the wait, they are
        // waited for here)
        bool ok = true;
        for (uint32_t t = 0; t < prefixed; ++t)
            ok = mbar_wait(&s.full[t], 0, wait_probes) && ok;
        if (!ok)
            atomicExch(&s.abort_flag, 1u);
        if (a.timing && tid == 0)
            a.timing[(size_t)row * 64 + 5] = global_ns();
        if (nb > 0) {
            for (uint32_t j = tid; j < nb; j += kThreads) {
                const mk_bias be = brow[j];
                const int64_t loc = (int64_t)be.id - id_off;
                if (be.id >= 0 && loc >= 0 && loc < (int64_t)span)
                    ring[loc] = __fadd_rn(ring[loc], be.value); // stages 0.. are contiguous
            }
            __syncthreads();
        }
        // no search: the list names the column, its rank is one popcount away and indexes the count
        const uint32_t n_own = s.n_own;
#pragma unroll 2
        for (uint32_t i = tid; i < n_own; i += kThreads) {
            const uint32_t c = own_list[i];
            const uint32_t rank = wpre[c >> 5] + __popc(bitmap[c >> 5] & ((1u << (c & 31u)) - 1u));
            const uint32_t n = (counts[rank >> 1] >> ((rank & 1u) * 16u)) & 0xffffu;
            ring[c] = penalise(ring[c], n, cfg);
        }
        __syncthreads();
    }
    if (tid == 0 && tiles_issued > tiles_early) {
        fence_proxy_async(); // the stage was written as plain shared memory until here
        fill_ring(tiles_early, tiles_issued);
    }
    // ---- streaming ----------------------------------------------------------------------------------------------
    if (a.timing && tid == 0)
        a.timing[(size_t)row * 64 + 1] = global_ns();
    float best = -__int_as_float(0x7f800000);
    int32_t best_col = -1;
    double sum_acc = 0.0; // need_sum: sum of exp2((l - best) * c2) over this thread's uncollected elements

    if (warp == 0) {
        // producer
        // tile t lives in stage t % n_stages, k = t / n_stages; the loop starts at 0 or, after a full prologue, at n_stages
        uint32_t st = (tiles_issued == n_stages) ? 0u : tiles_issued, k = (tiles_issued == n_stages) ? 1u : 0u;
        for (uint32_t t = tiles_issued; t < n_tiles; ++t, ++st) {
            if (st == n_stages) {
                st = 0;
                ++k;
            }
            float* dst = ring + st * kTile;
            const uint32_t n_t = min((uint32_t)kTile, V - t * kTile);
            const float* src = lrow + (size_t)t * kTile;
            if (k > 0) {
                bool ok = true;
                if (lane == 0) // polling: this lane's reaction time is on every stage's round trip
                    ok = mbar_wait_poll(&s.empty[st], (k - 1) & 1);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0)
                        atomicExch(&s.abort_flag, 1u);
                    break;
                }
            }
            if (*(volatile uint32_t*)&s.abort_flag)
                break;
            if (t == a.debug_skip_tile)
                continue;
            if (a.use_bulk_copy) {
                if (lane == 0) {
                    fence_proxy_async();
                    const uint32_t bytes = (n_t * 4u) & ~15u;
                    for (uint32_t e = bytes / 4; e < n_t; ++e)
                        dst[e] = src[e];
                    if (bytes > 0) {
                        mbar_arrive_expect_tx(&s.full[st], bytes);
                        bulk_load(dst, src, bytes, &s.full[st]);
                    } else {
                        mbar_arrive(&s.full[st]);
                    }
                }
            } else {
                for (uint32_t e = lane; e < n_t; e += 32)
                    dst[e] = src[e];
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&s.full[st]);
            }
        }
    } else if (warp <= kFixers / 32) {
        // fix-up: each of the two warps owns every other tile of those that follow the ones edited above (a long
        // history: warp 0 owns them all, because its per-tile counters are shared), so two tiles are edited at a time
        // and nothing synchronises across warps
        if (has_special) {
            const uint32_t fw = warp - 1;
            if (fw == 0 && lane == 0)
                for (uint32_t t = 0; t < prefixed; ++t) // edited by all warps above
                    mbar_arrive(&s.ready[t]);
            const uint32_t t_step = long_history ? 1u : (uint32_t)(kFixers / 32);
            uint32_t t_first = prefixed;
            if (!long_history)
                t_first += (fw + (kFixers / 32) - (prefixed % (kFixers / 32))) % (kFixers / 32); // t % 2 == fw
            const bool idle = long_history && fw != 0;
            uint32_t st = t_first % n_stages, k = t_first / n_stages;
            for (uint32_t t = t_first; t < n_tiles && !idle; t += t_step, st += t_step) {
                if (st >= n_stages) {
                    st -= n_stages;
                    ++k;
                }
                float* tp = ring + st * kTile;
                const uint32_t base = t * kTile;
                const uint32_t n_t = min((uint32_t)kTile, V - base);
                if (!mbar_wait(&s.full[st], k & 1, (*(volatile uint32_t*)&s.abort_flag) ? 1u : wait_probes))
                    atomicExch(&s.abort_flag, 1u);
                if (nb > 0) {
                    for (uint32_t j = lane; j < nb; j += 32) {
                        const mk_bias be = brow[j];
                        const int64_t loc = (int64_t)be.id - id_off - (int64_t)base;
                        if (be.id >= 0 && loc >= 0 && loc < (int64_t)n_t)
                            tp[loc] = __fadd_rn(tp[loc], be.value);
                    }
                    __syncwarp();
                }
                if (use_table) {
                    // the tile's generated columns, spread evenly over the lanes by rank (sampler.cpp:23-28)
                    const uint32_t w_lo = base >> 5, w_hi = min((base + n_t + 31u) >> 5, bm_words);
                    fix_hits(bitmap, wpre, counts, tp, base, w_lo, w_hi, (uint32_t)wpre[w_lo],
                             (w_hi < bm_words) ? (uint32_t)wpre[w_hi] : s.n_distinct, lane, 32u, cfg);
                } else if (has_hist) {
                    // long history: count the tile's ids in 16-bit counters, then the first lane to clear a
                    // counter owns that id and applies the penalties with its count
                    for (uint32_t j = lane; j < hlen; j += 32) {
                        const int64_t loc = (int64_t)hist_at(j) - id_off - (int64_t)base;
                        if (loc >= 0 && loc < (int64_t)n_t)
                            atomicAdd(&cnt[(uint32_t)loc >> 1], 1u << (((uint32_t)loc & 1u) * 16u));
                    }
                    __syncwarp();
                    for (uint32_t j = lane; j < hlen; j += 32) {
                        const int64_t loc64 = (int64_t)hist_at(j) - id_off - (int64_t)base;
                        if (loc64 >= 0 && loc64 < (int64_t)n_t) {
                            const uint32_t loc = (uint32_t)loc64, sh = (loc & 1u) * 16u;
                            const uint32_t old = atomicAnd(&cnt[loc >> 1], ~(0xffffu << sh));
                            const uint32_t n = (old >> sh) & 0xffffu;
                            if (n)
                                tp[loc] = penalise(tp[loc], n, cfg);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&s.ready[st]);
            }
        }
    } else {
        // readers
        const uint32_t rt = tid - kProducerThreads - kFixers;
        const uint32_t rwarp = rt >> 5;
        uint64_t* const avail = has_special ? s.ready : s.full;
        const float c2 = cfg.inv_t * 1.4426950408889634f;
        const float ninf = -__int_as_float(0x7f800000);
        const bool collect = !cfg.greedy || mode == kModeVpLocal;
        const bool sum_all = mode == kModeVpLocal;
        float warp_pub = ninf;
        // The loop over the tiles is compiled four times, with the mask, the top_k histogram and the streamed sum
        // compiled in or out: a row runs a variant that holds little beyond its own work. (One loop with all
        // three as run-time branches costs the common penalised row 12 % of its launch time, and all eight
        // combinations cost it 3 % again: the size of the code matters, executed or not.)
        auto read_tiles = [&](auto has_mask, auto has_hist, auto has_sum, auto aggregate) {
            constexpr bool kMask = decltype(has_mask)::value, kHist = decltype(has_hist)::value,
                           kSum = decltype(has_sum)::value, kAgg = decltype(aggregate)::value;
            uint32_t mw_next[kVec];
#pragma unroll
            for (int j = 0; j < kVec; ++j) {
                const uint32_t i0 = j * 1024 + rt * 4;
                mw_next[j] = (kMask && mrow) ? ((i0 < V) ? __ldg(mrow + (i0 >> 5)) : 0u) : 0xffffffffu;
            }
            uint32_t st = 0, k = 0;
            for (uint32_t t = 0; t < n_tiles; ++t, ++st) {
                if (st == n_stages) {
                    st = 0;
                    ++k;
                }
                const uint32_t base = t * kTile;
                uint32_t mw[kVec]; // this tile's mask words were requested a tile ago
#pragma unroll
                for (int j = 0; j < kVec; ++j)
                    mw[j] = mw_next[j];
                if (kMask && mrow) {
#pragma unroll
                    for (int j = 0; j < kVec; ++j) {
                        const uint32_t i0 = base + kTile + j * 1024 + rt * 4;
                        mw_next[j] = (i0 < V) ? __ldg(mrow + (i0 >> 5)) : 0u;
                    }
                }
                if (!mbar_wait(&avail[st], k & 1, (*(volatile uint32_t*)&s.abort_flag) ? 1u : wait_probes))
                    atomicExch(&s.abort_flag, 1u); // keep walking: the named barriers below must stay matched
                float w[kEl];
                const float4* tp4 = reinterpret_cast<const float4*>(ring + st * kTile);
#pragma unroll
                for (int j = 0; j < kVec; ++j) {
                    const float4 v = tp4[j * 256 + rt];
                    w[4 * j + 0] = v.x;
                    w[4 * j + 1] = v.y;
                    w[4 * j + 2] = v.z;
                    w[4 * j + 3] = v.w;
                }
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&s.empty[st]);

                if (kMask && mrow) {
#pragma unroll
                    for (int j = 0; j < kVec; ++j) {
                        const uint32_t bits = mw[j] >> ((rt * 4) & 31);
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (!((bits >> c) & 1u))
                                w[4 * j + c] = ninf;
                    }
                }
                if (base + kTile > V) {
#pragma unroll
                    for (int j = 0; j < kVec; ++j)
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (base + j * 1024 + rt * 4 + c >= V)
                                w[4 * j + c] = ninf;
                }
                if (t == 0 && rt == 0 && w[0] != w[0])
                    s.nan0 = 1;

                float tm = ninf;
#pragma unroll
                for (int e = 0; e < kEl; ++e)
                    tm = fmaxf(tm, w[e]);
                const float old_best = best;
                if (tm > best) {
                    best = tm;
#pragma unroll
                    for (int e = kEl - 1; e >= 0; --e)
                        if (w[e] == tm)
                            best_col = (int32_t)(base + (e >> 2) * 1024 + rt * 4 + (e & 3));
                }
                if (__any_sync(0xffffffffu, tm > warp_pub)) {
                    const float wm = warp_max(tm);
                    if (wm > warp_pub) {
                        warp_pub = wm;
                        if (lane == 0)
                            atomicMax(&s.m_key, order_key(wm));
                    }
                }
                float thr = keep_threshold(cfg, key_to_float(*(volatile uint32_t*)&s.m_key));
                if (kHist && cfg.hist_mode) {
                    // top_k bound. Every thread enters the largest of its 16 elements of the tile, if that is still at
                    // or above the bound in force, into a histogram of the value range: the maxima of different
                    // threads and tiles are different elements, so the bin in which the count from the top reaches k
                    // bounds the k-th largest element of the row from below — one histogram update for 16 elements,
                    // and a bound nearly as tight as a histogram of every element gives (the k largest rarely share
                    // a thread's 16 columns).
                    thr = fmaxf(thr, key_to_float(*(volatile uint32_t*)&s.thr_topk_key));
                    if (tm >= thr) {
                        const uint32_t bin = hist_bin(tm);
                        atomicAdd(&hist[bin], 1u);
                        if ((bin >> 5) > *(volatile uint32_t*)&s.hi_group)
                            atomicMax(&s.hi_group, bin >> 5);
                    }
                    __syncwarp();
                    // The first tile would be kept whole (no bound exists while it is read), so its 256 thread maxima
                    // give a first bound before anything is kept: the warps wait for one another's maxima — a bounded
                    // wait; a warp that gives up merely keeps more than it had to — and every warp reads the bound off.
                    if (t == 0) {
                        __threadfence_block();
                        if (lane == 0) {
                            atomicAdd(&s.first_tile_warps, 1u);
                            for (uint32_t probe = 0; probe < (1u << 12); ++probe)
                                if (*(volatile uint32_t*)&s.first_tile_warps >= (uint32_t)(kReaders / 32))
                                    break;
                        }
                        __syncwarp();
                    }
                    // One reader warp per tile rescans the histogram and raises the bound; nobody waits for it. Counts
                    // only grow and every count is an element at or above its bin's edge, so a bound read from a
                    // histogram that other warps are still adding to has its k elements all the same.
                    if (t == 0 || rwarp == (t % (kReaders / 32))) {
                        uint32_t cum = 0;
                        int found = -1;
                        for (int g = (int)*(volatile uint32_t*)&s.hi_group; g >= 0 && found < 0; --g) {
                            const uint32_t cbin = ((volatile uint32_t*)hist)[g * 32 + lane];
                            uint32_t suf = cbin; // suffix sum over lanes >= lane
#pragma unroll
                            for (int o = 1; o < 32; o <<= 1) {
                                const uint32_t y = __shfl_down_sync(0xffffffffu, suf, o);
                                if ((int)lane + o < 32)
                                    suf += y;
                            }
                            const uint32_t hit = __ballot_sync(0xffffffffu, cum + suf >= cfg.hist_k);
                            if (hit)
                                found = g * 32 + (31 - __clz(hit));
                            cum += __shfl_sync(0xffffffffu, suf, 0);
                        }
                        // the lowest key of a bin is its smallest float; bin 0 (NaN keys) is never a bound
                        if (lane == 0 && found > 0)
                            atomicMax(&s.thr_topk_key, order_key(hist_bin_floor((uint32_t)found)));
                        if (t == 0) {
                            __syncwarp();
                            thr = fmaxf(thr, key_to_float(*(volatile uint32_t*)&s.thr_topk_key));
                        }
                    }
                    if (collect && tm >= thr) {
#pragma unroll
                        for (int e = 0; e < kEl; ++e)
                            if (w[e] >= thr) {
                                const uint32_t slot = atomicAdd(&s.ncand, 1u);
                                if (slot < scratch_cap)
                                    scratch[slot] = make_uint2(__float_as_uint(w[e]), base + (e >> 2) * 1024 + rt * 4 + (e & 3));
                            }
                    }
                }
                if (kSum && cfg.need_sum && best > ninf) {
                    // Approximate weight of what is NOT collected (`thr` is the bound the collection used; a shard record
                    // sums everything): the collected
                    // elements get exact weights in the finish, so only the far tail carries the approximation.
                    if (best > old_best)
                        sum_acc *= (double)exp2f((old_best - best) * c2);
                    float p = 0.0f;
#pragma unroll
                    for (int e = 0; e < kEl; ++e)
                        p += (sum_all || w[e] < thr) ? ex2_approx((w[e] - best) * c2) : 0.0f;
                    sum_acc += (double)p;
                }
                if (!(kHist && cfg.hist_mode) && collect) {
                    const bool some = tm >= thr;
                    const uint32_t lanes = kAgg ? __ballot_sync(0xffffffffu, some) : 0u;
                    if (kAgg && __popc(lanes) >= 8) {
                        // Many lanes have something to keep (a flat row, or the first tiles of any row, before the
                        // maximum is known): one slot range per warp — a prefix sum over the lanes' counts and one
                        // atomic — instead of one atomic per element on the same shared-memory word.
                        uint32_t mine = 0;
#pragma unroll
                        for (int e = 0; e < kEl; ++e)
                            mine += (w[e] >= thr) ? 1u : 0u;
                        uint32_t inc = mine;
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) {
                            const uint32_t y = __shfl_up_sync(0xffffffffu, inc, o);
                            if ((int)lane >= o)
                                inc += y;
                        }
                        uint32_t slot = 0;
                        if (lane == 31)
                            slot = atomicAdd(&s.ncand, inc);
                        slot = __shfl_sync(0xffffffffu, slot, 31) + inc - mine;
                        if (some) {
#pragma unroll
                            for (int e = 0; e < kEl; ++e)
                                if (w[e] >= thr) {
                                    if (slot < scratch_cap)
                                        scratch[slot] = make_uint2(__float_as_uint(w[e]),
                                                                   base + (e >> 2) * 1024 + rt * 4 + (e & 3));
                                    ++slot;
                                }
                        }
                    } else if (some) {
#pragma unroll
                        for (int e = 0; e < kEl; ++e)
                            if (w[e] >= thr) {
                                const uint32_t slot = atomicAdd(&s.ncand, 1u);
                                const uint2 c = make_uint2(__float_as_uint(w[e]), base + (e >> 2) * 1024 + rt * 4 + (e & 3));
                                if (slot < scratch_cap)
                                    scratch[slot] = c;
                            }
                    }
                }
            }
        };
        using T = std::true_type;
        using F = std::false_type;
        if (!mrow && !cfg.hist_mode && !cfg.need_sum)
            read_tiles(F{}, F{}, F{}, F{}); // penalties, min_p, greedy: nothing but maximum and bound
        else if (!mrow && !cfg.need_sum)
            read_tiles(F{}, T{}, F{}, F{}); // top_k
        else if (!mrow && a.pass == 1)
            read_tiles(F{}, F{}, T{}, T{}); // top_p alone, second pass: a third of a flat row is kept
        else if (!mrow)
            read_tiles(F{}, T{}, T{}, F{}); // top_p alone (with its first-launch histogram), shard records
        else
            read_tiles(T{}, T{}, T{}, F{}); // masked rows: everything, chosen at run time
        if (best_col >= 0)
            atomicMax(&s.best_key,
                      ((unsigned long long)order_key(best) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)best_col));
    }
    __syncthreads();

    // ---- finish -------------------------------------------------------------------------------------------------
    if (a.timing && tid == 0)
        a.timing[(size_t)row * 64 + 2] = global_ns();
    if (s.abort_flag) {
        // A bounded wait ran out. Give copies still in flight time to land before the CTA's shared memory is
        // released, then report.
        for (int i = 0; i < 64; ++i)
            __nanosleep(1000);
        if (tid == 0) {
            if (a.token) a.token[row] = -1;
            if (a.flags) a.flags[row] = MK_FLAG_TIMEOUT;
            if (a.n_cand) a.n_cand[row] = 0;
            if (a.accepted) a.accepted[row] = 0;
        }
        return;
    }

    const bool any_finite = s.best_key != 0ull;
    float m = any_finite ? key_to_float((uint32_t)(s.best_key >> 32)) : -__int_as_float(0x7f800000);
    uint32_t arg_col = any_finite ? (0xffffffffu - (uint32_t)(s.best_key & 0xffffffffull)) : 0u;
    if (s.nan0) { // max_element keeps a NaN in front: every weight is NaN, the first column is returned
        m = __int_as_float(0x7fc00000);
        arg_col = 0;
    }
    uint32_t flags = hlen_clamped ? MK_FLAG_HISTORY_FULL : 0u;
    if (mrow && !any_finite && !s.nan0)
        flags |= MK_FLAG_ALL_MASKED;

    // need_sum: weight of the uncollected tail (the whole row for a shard record), relative to the row maximum:
    // sum over reader threads of sum_acc * exp2((best - m) * c2), fixed order
    double total_approx = 0.0;
    if (cfg.need_sum) {
        double part = 0.0;
        if (warp > kFixers / 32) {
            const float c2 = cfg.inv_t * 1.4426950408889634f;
            if (best > -__int_as_float(0x7f800000) && sum_acc > 0.0)
                part += sum_acc * exp2((double)(best - m) * (double)c2);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                part += __shfl_xor_sync(0xffffffffu, part, o);
            if (lane == 0)
                s.warp_sum[warp] = part;
        } else {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                part += __shfl_xor_sync(0xffffffffu, part, o);
            if (lane == 0)
                s.warp_sum[warp] = part;
        }
        __syncthreads();
        for (int i = 0; i < kThreads / 32; ++i)
            total_approx += s.warp_sum[i];
        __syncthreads(); // warp_sum is written again below
    }

    // ---- the short finish: what nearly every row takes ---------------------------------------------------------
    // Few collected elements, at most 32 of them candidates, no row total beyond their own: one warp does it all in
    // registers — exact weights, a 32-key sorting network over the lanes, top_k / top_p / total / draw as sequential
    // chains fed by shuffles, in the reference's order and precision (sampler.cpp:33-73, 86-107) — while the other
    // warps wait at one barrier. A one-shot phase waits for its instructions more than for anything else, so this path
    // is short and contiguous; every other row falls through to the general finish below, which recomputes from the
    // collected elements.
    constexpr uint32_t kFastRaw = 256;
    if (mode != kModeVpLocal && !cfg.greedy && !s.nan0 && s.ncand <= 2u * kFastRaw && s.ncand <= scratch_cap) {
        // Compiled twice: rows whose total is the candidates' own (nearly all) run code that knows nothing of the
        // row total of top_p alone.
        auto short_finish = [&](auto row_total_tag) {
            constexpr bool kRowTotal = decltype(row_total_tag)::value;
            const uint32_t full = 0xffffffffu;
            const uint32_t n_raw = s.ncand;
            const float thr_final = fmaxf(keep_threshold(cfg, m), key_to_float(s.thr_topk_key));
            unsigned long long* const fkeys = reinterpret_cast<unsigned long long*>(dyn + kOffKeys);
            uint32_t n = 0;
            double sum_kept = 0.0, sum_rest = 0.0; // top_p alone: exact weights at or above the bound, the others
            for (uint32_t r0 = 0; r0 < n_raw && n <= kWideCand; r0 += kFastRaw) { // once, for nearly every row
                uint2 craw[kFastRaw / 32]; // all requested at once: one trip to memory under load, not one per chunk
#pragma unroll
                for (uint32_t i = 0; i < kFastRaw / 32; ++i)
                    craw[i] = (r0 + i * 32u + lane < n_raw) ? scratch[r0 + i * 32u + lane] : make_uint2(0xff800000u, 0u);
#pragma unroll
                for (uint32_t i = 0; i < kFastRaw / 32; ++i) {
                    if (r0 + i * 32u >= n_raw || n > kWideCand)
                        break;
                    const uint2 c = craw[i];
                    float q = 0.0f;
                    if (__uint_as_float(c.x) >= thr_final) {
                        q = expf_host_exact(__fmul_rn(__fsub_rn(__uint_as_float(c.x), m), cfg.inv_t));
                        if (kRowTotal && q == q)
                            sum_kept += (double)q;
                    } else if (kRowTotal) {
                        // collected while the bound was lower: part of the row total, never a candidate
                        sum_rest += (double)ex2_approx((__uint_as_float(c.x) - m) * (cfg.inv_t * 1.4426950408889634f));
                    }
                    const bool ok = q >= cfg.minp_eff && q > 0.0f; // false for NaN
                    const uint32_t bal = __ballot_sync(full, ok);
                    const uint32_t pos = n + (uint32_t)__popc(bal & ((1u << lane) - 1u));
                    if (ok && pos < kWideCand)
                        fkeys[pos] = ((unsigned long long)__float_as_uint(q) << 32) | c.y;
                    n += (uint32_t)__popc(bal);
                }
            }
            __syncwarp();
            bool done = n <= 32u;
            if (!kRowTotal && n > 32u && n <= kWideCand) {
                const RowOut o = {a.token, a.prob, a.flags, a.n_cand, a.accepted, a.total_out, a.cand_ids, a.cand_q,
                                  a.cand_cap, id_off, a.timing, mode};
                wide_finish(s, fkeys, n, cfg.top_k, cfg.use_topp, cfg.top_p, cfg.inv_t, m, flags, draft_row, u_row, u2_row, row, o);
                done = true;
            }
            if (n <= 32u) {
                uint32_t fl = flags;
                bool retry = false;
                if (n == 0) { // sampler.cpp:37-38
                    fl |= MK_FLAG_NO_CANDIDATE;
                    if (lane == 0)
                        fkeys[0] = ((unsigned long long)__float_as_uint(1.0f) << 32) | arg_col;
                    n = 1;
                    __syncwarp();
                }
                const bool cut_k = cfg.top_k > 0 && cfg.top_k < n; // sampler.cpp:39
                const bool sorted = cut_k || cfg.use_topp;         // else ascending id
                unsigned long long key = ~0ull;
                if (lane < n) {
                    const unsigned long long raw = fkeys[lane];
                    const float q = __uint_as_float((uint32_t)(raw >> 32));
                    const uint32_t col = (uint32_t)(raw & 0xffffffffull);
                    key = sorted ? pack_by_weight(q, col) : pack_by_column(q, col);
                }
                for (uint32_t k = 2; k <= 32u; k <<= 1) // bitonic network over the 32 lanes
                    for (uint32_t j = k >> 1; j > 0; j >>= 1) {
                        const unsigned long long other = __shfl_xor_sync(full, key, j);
                        const bool keep_small = ((lane & j) == 0) == ((lane & k) == 0);
                        key = (keep_small == (key < other)) ? key : other;
                    }
                float q;
                uint32_t col;
                if (sorted) {
                    q = __uint_as_float(~(uint32_t)(key >> 32));
                    col = (uint32_t)(key & 0xffffffffull);
                } else {
                    q = __uint_as_float((uint32_t)(key & 0xffffffffull));
                    col = (uint32_t)(key >> 32);
                }
                if (lane >= n)
                    q = 0.0f;
                if (cut_k) { // sampler.cpp:40-42; the tie rule is the general finish's
                    const float qk = __shfl_sync(full, q, (int)cfg.top_k - 1);
                    const uint32_t edge_key = s.thr_topk_key;
                    const float below = key_to_float(edge_key - 1u);
                    if (edge_key > order_key(-FLT_MAX) &&
                        expf_host_exact(__fmul_rn(__fsub_rn(below, m), cfg.inv_t)) >= qk)
                        fl |= MK_FLAG_GUARD_BAND;
                    n = cfg.top_k;
                }
                if (cfg.use_topp) { // sampler.cpp:44-61, sequentially
                    double total_d = 0.0, band;
                    // top_p alone: the total covers every column — exact weights of what was kept, the streamed sum
                    // and the approximations above for the rest — and carries the margin of the approximate part
                    const bool row_total = kRowTotal && !(fl & MK_FLAG_NO_CANDIDATE);
                    if (row_total) {
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) {
                            sum_kept += __shfl_xor_sync(full, sum_kept, o);
                            sum_rest += __shfl_xor_sync(full, sum_rest, o);
                        }
                        const double rest = total_approx + sum_rest;
                        total_d = sum_kept + rest;
                        band = 1e-5 * rest + 0x1p-40 * total_d;
                    } else {
                        for (uint32_t j = 0; j < n; ++j)
                            total_d += (double)__shfl_sync(full, q, (int)j);
                        band = 0x1p-40 * total_d;
                    }
                    const double want = (double)cfg.top_p * total_d;
                    double run = 0.0, prev = 0.0;
                    uint32_t k = 0;
                    for (uint32_t j = 0; j < n && run < want; ++j) {
                        prev = run;
                        run += (double)__shfl_sync(full, q, (int)j);
                        k = j + 1u;
                    }
                    if ((row_total && run < want) ||
                        (k >= 1 && (fabs(run - want) <= band || (k >= 2 && fabs(prev - want) <= band)))) {
                        if (cfg.optimistic)
                            retry = true; // what was kept does not settle the nucleus: the second pass will
                        else
                            fl |= MK_FLAG_GUARD_BAND;
                    }
                    n = max(k, 1u);
                }
                if (lane >= n)
                    q = 0.0f;
                float total = 0.0f;
                for (uint32_t j = 0; j < n; ++j)
                    total = __fadd_rn(total, __shfl_sync(full, q, (int)j));
                const int32_t draft = (mode == kModeVerify) ? draft_row : -1;
                const uint32_t dm = __ballot_sync(full, draft >= 0 && lane < n && (int32_t)col + id_off == draft);
                const uint32_t draft_idx = dm ? (uint32_t)__ffs((int)dm) - 1u : 0xffffffffu;
                const float q_draft = dm ? __shfl_sync(full, q, (int)draft_idx) : 0.0f;
                int32_t tok = -1, acc = 0;
                float prob = 0.0f;
                if (mode == kModeDistOnly) {
                    tok = (int32_t)__shfl_sync(full, col, 0) + id_off;
                    prob = __fdiv_rn(__shfl_sync(full, q, 0), total);
                } else {
                    uint32_t skip_idx = 0xffffffffu;
                    float walk_total = total;
                    if (mode == kModeVerify) { // sampler.cpp:100-106
                        acc = __fmul_rn(u_row, total) < q_draft;
                        if (acc) {
                            tok = draft;
                            prob = __fdiv_rn(q_draft, total);
                        } else {
                            skip_idx = draft_idx;
                            walk_total = __fsub_rn(total, q_draft);
                            if (n == 1 && draft_idx == 0u) { // nothing but the rejected draft
                                tok = draft;
                                prob = 1.0f;
                            }
                        }
                    }
                    if (tok < 0) {
                        float r = __fmul_rn((mode == kModeVerify) ? u2_row : u_row, walk_total);
                        const float eps = 1e-6f * walk_total;
                        const uint32_t first_valid = (skip_idx == 0u) ? 1u : 0u;
                        const uint32_t last_valid = (skip_idx == n - 1u) ? n - 2u : n - 1u;
                        const float qw = (lane == skip_idx) ? 0.0f : q; // the skipped draft never wins
                        uint32_t hit = last_valid; // rounding: the last candidate (sampler.cpp:72)
                        float q_hit = __shfl_sync(full, qw, (int)last_valid);
                        bool found = false;
                        for (uint32_t j = 0; j < n && !found; ++j) {
                            const float qj = __shfl_sync(full, qw, (int)j);
                            if (r < qj) {
                                found = true;
                                hit = j;
                                q_hit = qj;
                                // boundary below (not for the first candidate) or above (not for the last)
                                if ((j != first_valid && r < eps) || (j < last_valid && __fsub_rn(qj, r) < eps))
                                    fl |= MK_FLAG_NEAR_CDF_BOUNDARY;
                            } else {
                                r = __fsub_rn(r, qj);
                            }
                        }
                        tok = (int32_t)__shfl_sync(full, col, (int)hit) + id_off;
                        prob = __fdiv_rn(q_hit, walk_total);
                    }
                }
                if (lane == 0) {
                    if (retry)
                        again[0] = 1u; // every output of this row is written again by the second pass
                    if (a.token) a.token[row] = retry ? -1 : tok;
                    if (a.prob) a.prob[row] = prob;
                    if (a.flags) a.flags[row] = fl;
                    if (a.n_cand) a.n_cand[row] = n;
                    if (a.accepted) a.accepted[row] = acc;
                    if (a.total_out) a.total_out[row] = total;
                    if (a.timing)
                        a.timing[(size_t)row * 64 + 3] = global_ns();
                }
                if (lane < min(n, a.cand_cap)) {
                    if (a.cand_ids) a.cand_ids[(size_t)row * a.cand_cap + lane] = (int32_t)col + id_off;
                    if (a.cand_q) a.cand_q[(size_t)row * a.cand_cap + lane] = q;
                }
            }
            if (lane == 0)
                s.n_final = done ? 1u : 0u; // 1: the row is done
        };
        if (warp == 0) {
            if (cfg.need_sum)
                short_finish(std::true_type{});
            else
                short_finish(std::false_type{});
        }
        __syncthreads();
        if (s.n_final)
            return;
        __syncthreads(); // n_final is written again below
        if (tid == 0)
            s.n_final = 0;
    }

    if (mode == kModeVpLocal) {
        // Shard record: header {max, n, sum} then the k best (logit, global id), by (logit desc, id asc).
        unsigned long long* keys = reinterpret_cast<unsigned long long*>(dyn + kOffKeys);
        const uint32_t n_all = min(s.ncand, scratch_cap);
        const float thr_final = fmaxf(keep_threshold(cfg, m), key_to_float(s.thr_topk_key));
        for (uint32_t i = tid; i < n_all; i += kThreads) {
            const uint2 c = scratch[i];
            if (__uint_as_float(c.x) >= thr_final) {
                const uint32_t slot = atomicAdd(&s.nsurv, 1u);
                if (slot < (uint32_t)kSortCap)
                    keys[slot] = ((unsigned long long)(~order_key(__uint_as_float(c.x))) << 32) | c.y;
            }
        }
        __syncthreads();
        const uint32_t n_raw = min(s.nsurv, (uint32_t)kSortCap);
        const bool over = s.nsurv > (uint32_t)kSortCap || s.ncand > scratch_cap;
        uint32_t n2 = 2;
        while (n2 < n_raw)
            n2 <<= 1;
        for (uint32_t i = n_raw + tid; i < n2; i += kThreads)
            keys[i] = ~0ull;
        __syncthreads();
        block_sort(keys, n2);
        unsigned char* rec = reinterpret_cast<unsigned char*>(a.vp_records) +
                             ((size_t)(kSplit ? blockIdx.y * gridDim.x : 0u) + row) * vp_record_bytes(a.vp_k);
        const uint32_t n_out = min(n_raw, a.vp_k);
        if (tid == 0) {
            float* hf = reinterpret_cast<float*>(rec);
            uint32_t* hu = reinterpret_cast<uint32_t*>(rec);
            hf[0] = m;
            hu[1] = n_out | (over ? 0x80000000u : 0u) | ((V > a.vp_k) ? 0x40000000u : 0u);
            *reinterpret_cast<double*>(rec + 8) = total_approx;
        }
        for (uint32_t i = tid; i < a.vp_k; i += kThreads) {
            uint2 o = make_uint2(__float_as_uint(-__int_as_float(0x7f800000)), 0xffffffffu);
            if (i < n_out) {
                const unsigned long long key = keys[i];
                const uint32_t ok = ~(uint32_t)(key >> 32);
                o.x = __float_as_uint(key_to_float(ok));
                o.y = (uint32_t)((int32_t)(uint32_t)(key & 0xffffffffull) + id_off);
            }
            reinterpret_cast<uint2*>(rec + kVpHeaderBytes)[i] = o;
        }
        return;
    }

    if (cfg.greedy) {
        // sampler.cpp:77-78, 88-91: first maximum of the row as handed over (bias and mask applied, no penalties)
        if (tid == 0) {
            const int32_t t = (int32_t)arg_col + id_off;
            if (a.token) a.token[row] = t;
            if (a.prob) a.prob[row] = 1.0f;
            if (a.n_cand) a.n_cand[row] = 1;
            if (a.flags) a.flags[row] = flags;
            if (a.cand_ids && a.cand_cap) a.cand_ids[(size_t)row * a.cand_cap] = t;
            if (a.cand_q && a.cand_cap) a.cand_q[(size_t)row * a.cand_cap] = 1.0f;
            if (a.total_out) a.total_out[row] = 1.0f;
            if (mode == kModeVerify && a.accepted)
                a.accepted[row] = (draft_row == t) ? 1 : 0;
        }
        return;
    }

    // exact weights of the collected elements, min_p filter (sampler.cpp:33-35)
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(dyn + kOffKeys);
    const uint32_t n_raw = min(s.ncand, scratch_cap);
    bool overflow = s.ncand > scratch_cap;
    double total_need = 0.0, band_need = 0.0; // need_sum: the row total that top_p scales, and its margin
    if (!s.nan0) {
        // Elements collected while the running maximum was still low are dropped by the final bound first.
        float thr_final = fmaxf(keep_threshold(cfg, m), key_to_float(s.thr_topk_key));
        // A long list under top_p alone: the bound is raised first, and the elements it leaves out get approximate
        // weights (they join the part of the row total that carries the 1e-5 margin); exact weights only above it.
        bool approx_below = false;
        if (cfg.need_sum && n_raw > 4096u) {
            mass_cut(s, dyn, scratch, n_raw, thr_final, m, cfg.inv_t, cfg.top_p, total_approx);
            thr_final = fmaxf(thr_final, key_to_float(s.thr_topk_key));
            approx_below = true;
        }
        double below = 0.0, exact = 0.0;
        const float c2w = cfg.inv_t * 1.4426950408889634f;
        for (uint32_t i0 = tid; i0 < n_raw; i0 += 4u * kThreads) {
            uint2 cv[4]; // four loads in flight
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t i = i0 + (uint32_t)k * kThreads;
                cv[k] = (i < n_raw) ? scratch[i] : make_uint2(0xff800000u, 0u); // filler: -inf
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint2 c = cv[k];
                const bool in = __uint_as_float(c.x) >= thr_final;
                if (!in && (!cfg.need_sum || i0 + (uint32_t)k * kThreads >= n_raw))
                    continue;
                if (!in && approx_below) {
                    below += (double)ex2_approx((__uint_as_float(c.x) - m) * c2w);
                    continue;
                }
                const float x = __fmul_rn(__fsub_rn(__uint_as_float(c.x), m), cfg.inv_t);
                const float q = expf_host_exact(x);
                if (q == q)
                    exact += (double)q;
                if (in && q >= cfg.minp_eff && q > 0.0f) {
                    const uint32_t slot = atomicAdd(&s.nsurv, 1u);
                    if (slot < (uint32_t)kSortCap)
                        keys[slot] = ((unsigned long long)__float_as_uint(q) << 32) | c.y;
                }
            }
        }
        if (cfg.need_sum) {
            // top_p's total (sampler.cpp:45-47) covers every column: exact weights for all that was collected, the
            // approximate sum for the rest. The margin that goes with it is 1e-5 of the approximate part plus the
            // rounding of a double sum taken in another order than the reference's.
            __syncthreads();
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                exact += __shfl_xor_sync(0xffffffffu, exact, o);
                below += __shfl_xor_sync(0xffffffffu, below, o);
            }
            if (lane == 0)
                s.warp_sum[warp] = exact;
            __syncthreads();
            double sum = 0.0;
            for (int i = 0; i < kThreads / 32; ++i)
                sum += s.warp_sum[i];
            __syncthreads();
            if (lane == 0)
                s.warp_sum[warp] = below;
            __syncthreads();
            for (int i = 0; i < kThreads / 32; ++i)
                total_approx += s.warp_sum[i];
            total_need = sum + total_approx;
            band_need = 1e-5 * total_approx + 0x1p-40 * total_need;
        }
    }
    __syncthreads();
    uint32_t n = s.nsurv;
    if (a.timing && tid == 0) {
        a.timing[(size_t)row * 64 + 9] = n_raw;
        a.timing[(size_t)row * 64 + 10] = n;
        a.timing[(size_t)row * 64 + 11] = global_ns();
    }
    if (!overflow && n > (uint32_t)kSortCap && !cfg.use_topp && !(cfg.top_k > 0 && cfg.top_k < n)) {
        const RowOut o = {a.token, a.prob, a.flags, a.n_cand, a.accepted, a.total_out, a.cand_ids, a.cand_q,
                          a.cand_cap, id_off, a.timing, mode};
        wide_id_ordered(s, reinterpret_cast<float*>(dyn + kOffKeys), scratch, qrow, n_raw, n, V,
                        fmaxf(keep_threshold(cfg, m), key_to_float(s.thr_topk_key)), m, cfg.inv_t, cfg.minp_eff, row,
                        flags, u_row, u2_row, draft_row, o);
        return;
    }
    const unsigned long long* ksrc = keys; // the ordered list: shared memory, or the row's scratch for a long one
    bool pre_sorted = false;
    if (!overflow && n > (uint32_t)kSortCap && mode != kModeDistOnly) {
        // More candidates than the shared-memory sort holds, and a truncation that orders them (the unordered case
        // returned above): a flat row under top_p, or a very large top_k. The candidates are sorted in global
        // memory — 8192-key runs in shared memory, then merge passes between the two halves of the row's scratch —
        // and the steps below read the list from there.
        const unsigned long long* P = long_sort(s, keys, scratch, scratch_cap, n_raw, n,
                                                fmaxf(keep_threshold(cfg, m), key_to_float(s.thr_topk_key)), m, cfg.inv_t,
                                                cfg.minp_eff);
        ksrc = P;
        pre_sorted = true;
        // The float total and the walk below are sequential chains that take 32 candidates per step: fed from global
        // memory they run at the pace of its latency, so a list that fits is staged in shared memory first.
        if (n <= kDynBytes / 8u) {
            unsigned long long* const staged = reinterpret_cast<unsigned long long*>(dyn);
            for (uint32_t i = tid; i < n; i += kThreads)
                staged[i] = P[i];
            __syncthreads();
            ksrc = staged;
        }
    }
    if (!pre_sorted && n > (uint32_t)kSortCap)
        overflow = true;
    if (overflow) {
        if (tid == 0) {
            if (a.token) a.token[row] = -1;
            if (a.prob) a.prob[row] = 0.0f;
            if (a.flags) a.flags[row] = flags | MK_FLAG_OVERFLOW;
            if (a.n_cand) a.n_cand[row] = s.ncand;
            if (a.accepted) a.accepted[row] = 0;
            if (a.total_out) a.total_out[row] = 0.0f;
        }
        return;
    }
    if (n == 0) { // sampler.cpp:37-38
        flags |= MK_FLAG_NO_CANDIDATE;
        if (tid == 0)
            keys[0] = ((unsigned long long)__float_as_uint(1.0f) << 32) | arg_col;
        n = 1;
        __syncthreads();
    }
    const bool cut_k = cfg.top_k > 0 && cfg.top_k < n;       // sampler.cpp:39
    const bool sorted = cut_k || cfg.use_topp;               // else ascending id
    // Ascending id needs no sort: a bitmap of the candidates' columns ranks them, and `ord` lists the candidates'
    // slots by rank. (Vocabularies beyond the bitmap, and lists too short to be worth it, sort by column.)
    const bool by_rank = !pre_sorted && !sorted && V <= kMaxBitmapVocab && n > 64u;
    uint32_t* const fbitmap = reinterpret_cast<uint32_t*>(dyn + kOffFinBitmap);
    uint16_t* const fwpre = reinterpret_cast<uint16_t*>(dyn + kOffFinWpre);
    uint16_t* const ord = reinterpret_cast<uint16_t*>(dyn + kOffFinOrd);
    if (pre_sorted) {
        // ordered above
    } else if (by_rank) {
        const uint32_t words = (V + 31u) >> 5;
        for (uint32_t w = tid; w < words; w += kThreads)
            fbitmap[w] = 0u;
        __syncthreads();
        for (uint32_t i = tid; i < n; i += kThreads) {
            const uint32_t col = (uint32_t)(keys[i] & 0xffffffffull);
            atomicOr(&fbitmap[col >> 5], 1u << (col & 31u));
        }
        __syncthreads();
        word_ranks(s, fbitmap, fwpre, words);
        __syncthreads();
        for (uint32_t i = tid; i < n; i += kThreads) {
            const uint32_t col = (uint32_t)(keys[i] & 0xffffffffull);
            ord[fwpre[col >> 5] + __popc(fbitmap[col >> 5] & ((1u << (col & 31u)) - 1u))] = (uint16_t)i;
        }
        __syncthreads();
    } else {
        uint32_t n2 = 2;
        while (n2 < n)
            n2 <<= 1;
        for (uint32_t i = tid; i < n2; i += kThreads) {
            unsigned long long key = ~0ull;
            if (i < n) {
                const unsigned long long raw = keys[i];
                const float q = __uint_as_float((uint32_t)(raw >> 32));
                const uint32_t col = (uint32_t)(raw & 0xffffffffull);
                key = sorted ? pack_by_weight(q, col) : pack_by_column(q, col);
            }
            keys[i] = key;
        }
        __syncthreads();
        if (n > 1)
            block_sort(keys, n2);
    }
    if (a.timing && tid == 0)
        a.timing[(size_t)row * 64 + 12] = global_ns();
    // the r-th candidate of the list in the reference's order
    auto fetch = [&](uint32_t r, float& q, uint32_t& col) {
        if (sorted) {
            const unsigned long long key = ksrc[r];
            q = __uint_as_float(~(uint32_t)(key >> 32));
            col = (uint32_t)(key & 0xffffffffull);
        } else if (by_rank) {
            const unsigned long long key = keys[ord[r]];
            q = __uint_as_float((uint32_t)(key >> 32));
            col = (uint32_t)(key & 0xffffffffull);
        } else {
            const unsigned long long key = keys[r];
            q = __uint_as_float((uint32_t)(key & 0xffffffffull));
            col = (uint32_t)(key >> 32);
        }
    };
    auto q_of = [&](uint32_t r) -> float {
        float q;
        uint32_t col;
        fetch(r, q, col);
        return q;
    };

    if (cut_k) {
        // sampler.cpp:40-42. Ties in q with the k-th weight are ordered by id among ALL elements with that weight;
        // elements below the histogram bound were not collected, so the largest value below the bound must map to a
        // strictly smaller weight than the k-th (weights are monotone in the logit).
        const float qk = q_of(cfg.top_k - 1);
        const uint32_t edge_key = s.thr_topk_key;
        const float below = key_to_float(edge_key - 1u);
        if (edge_key > order_key(-FLT_MAX) && expf_host_exact(__fmul_rn(__fsub_rn(below, m), cfg.inv_t)) >= qk)
            flags |= MK_FLAG_GUARD_BAND;
        n = cfg.top_k;
    }
    const bool short_list = n <= 128u; // one warp does it all, in the reference's own order, without CTA barriers
    bool retry = false; // first launch, top_p alone: what was kept does not settle the nucleus; the second pass will
    if (cfg.use_topp && !short_list) {
        const uint32_t kk = wide_top_p(s, ksrc, n, cfg.top_p, cfg.need_sum, cfg.need_sum && !(flags & MK_FLAG_NO_CANDIDATE),
                                       total_need, band_need);
        if (kk & 0x80000000u) {
            if (cfg.optimistic)
                retry = true;
            else
                flags |= MK_FLAG_GUARD_BAND;
        }
        n = max(kk & 0x7fffffffu, 1u);
    }

    if (a.timing && tid == 0)
        a.timing[(size_t)row * 64 + 13] = global_ns();
    // Float total and the walk, left to right in the reference's order and precision (sampler.cpp:64-73, 80-83,
    // 100-106), by one warp: every lane loads one candidate, the values go round by shuffle and every lane runs
    // the same sequential chain, so the chain never waits for memory.
    if (warp == 0) {
        const uint32_t full = 0xffffffffu;
        const int32_t draft = (mode == kModeVerify) ? draft_row : -1;
        if (cfg.use_topp && short_list) { // sampler.cpp:44-61, sequentially
            double total_d = 0.0, band;
            if (cfg.need_sum && !(flags & MK_FLAG_NO_CANDIDATE)) {
                total_d = total_need;
                band = band_need;
            } else {
                for (uint32_t base = 0; base < n; base += 32u) {
                    const float q = (base + lane < n) ? q_of(base + lane) : 0.0f;
                    const int cnt = (int)min(32u, n - base);
#pragma unroll 4
                    for (int j = 0; j < cnt; ++j)
                        total_d += (double)__shfl_sync(full, q, j);
                }
                band = 0x1p-40 * total_d;
            }
            const double want = (double)cfg.top_p * total_d;
            double run = 0.0, prev = 0.0;
            uint32_t k = 0;
            bool open = true;
            for (uint32_t base = 0; base < n && open; base += 32u) {
                const float q = (base + lane < n) ? q_of(base + lane) : 0.0f;
                const int cnt = (int)min(32u, n - base);
#pragma unroll 4
                for (int j = 0; j < cnt; ++j) {
                    const double qj = (double)__shfl_sync(full, q, j);
                    open = open && run < want;
                    if (open) {
                        prev = run;
                        run += qj;
                        k = base + (uint32_t)j + 1u;
                    }
                }
            }
            if ((cfg.need_sum && run < want) ||
                (k >= 1 && (fabs(run - want) <= band || (k >= 2 && fabs(prev - want) <= band)))) {
                if (cfg.optimistic)
                    retry = true;
                else
                    flags |= MK_FLAG_GUARD_BAND;
            }
            n = max(k, 1u);
        }
        float total = 0.0f, q_draft = 0.0f;
        uint32_t draft_idx = 0xffffffffu;
        float q_next = 0.0f; // the next 32 candidates are fetched while this chain runs (long lists sit in global memory)
        uint32_t col_next = 0xffffffffu;
        if (lane < n)
            fetch(lane, q_next, col_next);
        for (uint32_t base = 0; base < n; base += 32u) {
            const float q = q_next;
            const uint32_t col = col_next;
            q_next = 0.0f;
            col_next = 0xffffffffu;
            if (base + 32u + lane < n)
                fetch(base + 32u + lane, q_next, col_next);
            const uint32_t dm = __ballot_sync(full, draft >= 0 && base + lane < n && (int32_t)col + id_off == draft);
            if (dm) {
                q_draft = __shfl_sync(full, q, __ffs(dm) - 1);
                draft_idx = base + (uint32_t)__ffs(dm) - 1u;
            }
            const int cnt = (int)min(32u, n - base);
            if (cnt == 32) {
                // a full step unrolled whole: the 32 shuffles do not depend on the sum, so they all issue ahead of
                // the chain of additions, which then runs at the adder's latency
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    total = __fadd_rn(total, __shfl_sync(full, q, j));
            } else {
#pragma unroll 8
                for (int j = 0; j < cnt; ++j)
                    total = __fadd_rn(total, __shfl_sync(full, q, j));
            }
        }
        int32_t tok = -1, acc = 0;
        float prob = 0.0f;
        if (mode == kModeDistOnly) {
            float q0;
            uint32_t c0;
            fetch(0, q0, c0);
            tok = (int32_t)c0 + id_off;
            prob = __fdiv_rn(q0, total);
        } else {
            uint32_t skip_idx = 0xffffffffu;
            float walk_total = total;
            if (mode == kModeVerify) { // sampler.cpp:100-106
                acc = __fmul_rn(u_row, total) < q_draft;
                if (acc) {
                    tok = draft;
                    prob = __fdiv_rn(q_draft, total);
                } else {
                    skip_idx = draft_idx;
                    walk_total = __fsub_rn(total, q_draft);
                    if (n == 1 && draft_idx == 0u) { // nothing but the rejected draft
                        tok = draft;
                        prob = 1.0f;
                    }
                }
            }
            if (tok < 0) {
                float r = __fmul_rn((mode == kModeVerify) ? u2_row : u_row, walk_total);
                const float eps = 1e-6f * walk_total;
                const uint32_t first_valid = (skip_idx == 0u) ? 1u : 0u;
                const uint32_t last_valid = (skip_idx == n - 1u) ? n - 2u : n - 1u;
                bool found = false;
                uint32_t hit = 0;
                float r_hit = 0.0f, q_hit = 0.0f;
                float qn = (lane < n && lane != skip_idx) ? q_of(lane) : 0.0f;
                for (uint32_t base = 0; base < n && !found; base += 32u) {
                    const float q = qn; // the skipped draft has weight 0: it never wins and changes nothing
                    qn = (base + 32u + lane < n && base + 32u + lane != skip_idx) ? q_of(base + 32u + lane) : 0.0f;
                    const int cnt = (int)min(32u, n - base);
                    if (cnt == 32) {
                        // a full step: the chain of subtractions alone, noting which candidates the draw fell short
                        // of; the first of them is the hit, and the remainder in front of it is subtracted again
                        uint32_t short_of = 0u;
                        float rr = r;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float qj = __shfl_sync(full, q, j);
                            short_of |= (rr < qj) ? (1u << j) : 0u;
                            rr = __fsub_rn(rr, qj);
                        }
                        if (short_of) {
                            const int jh = __ffs((int)short_of) - 1;
                            for (int j = 0; j < jh; ++j)
                                r = __fsub_rn(r, __shfl_sync(full, q, j));
                            found = true;
                            hit = base + (uint32_t)jh;
                            r_hit = r;
                            q_hit = __shfl_sync(full, q, jh);
                        } else {
                            r = rr;
                        }
                    } else {
#pragma unroll 8
                        for (int j = 0; j < cnt; ++j) {
                            const float qj = __shfl_sync(full, q, j);
                            if (!found && r < qj) {
                                found = true;
                                hit = base + (uint32_t)j;
                                r_hit = r;
                                q_hit = qj;
                            }
                            r = __fsub_rn(r, qj);
                        }
                    }
                }
                float qx;
                uint32_t cx;
                if (found) {
                    fetch(hit, qx, cx);
                    tok = (int32_t)cx + id_off;
                    prob = __fdiv_rn(q_hit, walk_total);
                    // boundary below (not for the first candidate) or above (not for the last)
                    if ((hit != first_valid && r_hit < eps) || (hit < last_valid && __fsub_rn(q_hit, r_hit) < eps))
                        flags |= MK_FLAG_NEAR_CDF_BOUNDARY;
                } else { // rounding: the last candidate (sampler.cpp:72)
                    fetch(last_valid, qx, cx);
                    tok = (int32_t)cx + id_off;
                    prob = __fdiv_rn(qx, walk_total);
                }
            }
        }
        if (lane == 0) {
            if (retry)
                again[0] = 1u; // every output of this row is written again by the second pass
            if (a.token) a.token[row] = retry ? -1 : tok;
            if (a.prob) a.prob[row] = prob;
            if (a.flags) a.flags[row] = flags;
            if (a.n_cand) a.n_cand[row] = n;
            if (a.accepted) a.accepted[row] = acc;
            if (a.total_out) a.total_out[row] = total;
            s.n_final = n;
            if (a.timing)
                a.timing[(size_t)row * 64 + 3] = global_ns();
        }
    }
    if (a.cand_ids || a.cand_q) {
        __syncthreads();
        const uint32_t nf = min(s.n_final, a.cand_cap);
        for (uint32_t i = tid; i < nf; i += kThreads) {
            float q;
            uint32_t col;
            fetch(i, q, col);
            if (a.cand_ids) a.cand_ids[(size_t)row * a.cand_cap + i] = (int32_t)col + id_off;
            if (a.cand_q) a.cand_q[(size_t)row * a.cand_cap + i] = q;
        }
    }
}

size_t row_kernel_smem_bytes()
{
    return kSmemBytes;
}

cudaError_t launch_row_kernel(const RowKernelArgs& a, uint32_t batch, cudaStream_t stream)
{
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return e;
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(row_pipeline_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess)
            return e;
        e = cudaFuncSetAttribute(row_pipeline_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess)
            return e;
        e = cudaFuncSetAttribute(row_pipeline_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess)
            return e;
        configured[dev] = true;
    }
    if (batch == 0)
        return cudaSuccess;
    // With an overlap mode the launch carries the programmatic-serialization attribute: the grid may be scheduled
    // while the previous kernel of the stream drains, and synchronises with it by griddep_wait() in the kernel.
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(batch);
    lc.blockDim = dim3(kThreads);
    lc.dynamicSmemBytes = kSmemBytes;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = a.overlap != MK_OVERLAP_OFF ? 1u : 0u;
    RowKernelArgs first = a;
    first.pass = 0;
    const bool spec = a.spec_n_pos != 0u;
    if (a.split_w != 0u) { // shard records of every row, one CTA per (row, column shard)
        lc.gridDim = dim3(batch, (a.n_vocab + a.split_w - 1u) / a.split_w);
        return cudaLaunchKernelEx(&lc, row_pipeline_kernel<false, true>, first);
    }
    e = spec ? cudaLaunchKernelEx(&lc, row_pipeline_kernel<true, false>, first)
             : cudaLaunchKernelEx(&lc, row_pipeline_kernel<false, false>, first);
    if (e != cudaSuccess)
        return e;
    // top_p alone (make_cfg: need_sum): rows whose nucleus the first launch could not settle are streamed again
    // with the loose bound. With per-row parameters on the device any row may be one; CTAs of other rows return at once.
    const mk_sampling_params& p = a.params;
    const float minp_eff = (1.0f < p.min_p) ? 1.0f : p.min_p;
    const bool host_need_sum = !(p.temperature <= 0.0f) && p.top_p < 1.0f && !(minp_eff > 0.0f) &&
                               !(p.top_k > 0 && p.top_k < a.n_vocab);
    if (a.mode != kModeVpLocal && kNucleusGuess < a.n_vocab && (a.params_dev || host_need_sum)) {
        RowKernelArgs second = a;
        second.pass = 1;
        e = spec ? cudaLaunchKernelEx(&lc, row_pipeline_kernel<true, false>, second)
                 : cudaLaunchKernelEx(&lc, row_pipeline_kernel<false, false>, second);
    }
    return e;
}

// ---- test hook --------------------------------------------------------------------------------------------------
__global__ void expf_probe_kernel(const float* x, float* y, uint64_t n)
{
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n)
        y[i] = expf_host_exact(x[i]);
}

cudaError_t launch_expf_probe(const float* x, float* y, uint64_t n, cudaStream_t stream)
{
    if (n == 0)
        return cudaSuccess;
    expf_probe_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(x, y, n);
    return cudaGetLastError();
}

} // namespace mk
