// Small kernels around the row pipeline: the merge step of vocab-parallel sampling, the resolution of p/q
// rejection sampling from two candidate lists, and the acceptance loop of a speculative round.
#include "row_pipeline.h"

#include "device_expf.cuh"
#include "ptx.cuh"

#include <cfloat>

namespace mk {

namespace {

constexpr int kMergeThreads = 128;    // a CTA per row of a large batch
constexpr int kMergeThreadsFew = 512; // a handful of rows: the sort is what takes the time, so more threads on it
constexpr int kMergeCap = 2048; // n_shards * k
constexpr uint32_t kShardShift = 26, kIdMask = (1u << kShardShift) - 1u; // sort keys: shard above the token id

__device__ void sort_keys(unsigned long long* keys, uint32_t n2, uint32_t n_threads)
{
    for (uint32_t k = 2; k <= n2; k <<= 1) {
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            for (uint32_t i = threadIdx.x; i < n2; i += n_threads) {
                const uint32_t l = i ^ j;
                if (l > i) {
                    const unsigned long long a = keys[i], b = keys[l];
                    const bool up = (i & k) == 0;
                    if ((a > b) == up) {
                        keys[i] = b;
                        keys[l] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
}

} // namespace

// One CTA per row. Input: for each shard a record {float max; uint32 n|flags; double sum; (float logit, int32 id) x k}
// where sum = sum over the shard of exp((l - max) * inv_t) (approximate) and the list holds the shard's k best
// edited logits by (logit desc, id asc). The merge recomputes exact weights against the global maximum, so a
// candidate's q is the same float the single-device pipeline computes; only the row total that top_p needs when no
// other truncation is active comes from the rescaled partial sums, and decisions within 1e-5 of it are flagged.
__global__ void __launch_bounds__(kMergeThreadsFew) vp_merge_kernel(const VpMergeArgs a)
{
    __shared__ unsigned long long keys[kMergeCap];
    __shared__ uint32_t s_n, s_nfinal;
    __shared__ uint32_t s_shard_in[64];  // entries of each shard that are in the deciding set
    const uint32_t row = blockIdx.x, tid = threadIdx.x, n_thr = blockDim.x;
    const uint32_t rb = vp_record_bytes(a.k);
    const mk_sampling_params prm = a.params_dev ? a.params_dev[row] : a.params;
    const float inv_t = __fdiv_rn(1.0f, prm.temperature);
    const bool greedy = prm.temperature <= 0.0f;
    const float minp_eff = (1.0f < prm.min_p) ? 1.0f : prm.min_p;
    const float ninf = -__int_as_float(0x7f800000);

    auto rec = [&](uint32_t g) { return a.gathered + ((size_t)g * a.batch + row) * rb; };

    // the shards' headers and best entries, fetched side by side (one thread per shard): every thread walks them below
    __shared__ float s_max[64];
    __shared__ uint32_t s_hdr[64], s_first[64];
    __shared__ double s_sum[64];
    if (tid < a.n_shards) {
        s_max[tid] = *reinterpret_cast<const float*>(rec(tid));
        s_hdr[tid] = *reinterpret_cast<const uint32_t*>(rec(tid) + 4);
        s_sum[tid] = *reinterpret_cast<const double*>(rec(tid) + 8);
        s_first[tid] = reinterpret_cast<const uint2*>(rec(tid) + kVpHeaderBytes)->y;
    }
    __syncthreads();

    // global maximum and first argmax
    float m = ninf;
    uint32_t arg_id = 0, arg_shard = 0;
    bool any = false, nan0 = false;
    for (uint32_t g = 0; g < a.n_shards; ++g) {
        const float mg = s_max[g];
        const uint32_t ng = s_hdr[g] & 0xffffu;
        if (mg != mg) {
            nan0 = true;
            continue;
        }
        if (ng > 0 && mg > ninf) {
            if (!any || mg > m) { // shards ascend in id, so the first shard holding the maximum wins ties
                m = mg;
                arg_id = s_first[g];
                arg_shard = g;
                any = true;
            }
        }
    }
    if (nan0) {
        m = __int_as_float(0x7fc00000);
        arg_id = 0;
        arg_shard = 0;
    }
    if (tid == 0) {
        s_n = 0;
        s_nfinal = 0;
    }
    if (tid < 64)
        s_shard_in[tid] = 0;
    __syncthreads();

    uint32_t flags = 0;
    if (greedy) {
        if (tid == 0) {
            if (a.token) a.token[row] = (int32_t)arg_id;
            if (a.prob) a.prob[row] = 1.0f;
            if (a.flags) a.flags[row] = 0;
            if (a.n_cand) a.n_cand[row] = 1;
            if (a.cand_ids && a.cand_cap) a.cand_ids[(size_t)row * a.cand_cap] = (int32_t)arg_id;
            if (a.cand_q && a.cand_cap) a.cand_q[(size_t)row * a.cand_cap] = 1.0f;
        }
        return;
    }

    // exact weights. The id field of a key carries the shard the candidate came from in its top six bits (ids stay
    // below 2^26, checked by the caller): shards ascend in id, so the order by id is unchanged, and the count of a
    // shard's members in the deciding set below needs no knowledge of how the columns were split.
    if (!nan0) {
        for (uint32_t e = tid; e < a.n_shards * a.k; e += n_thr) {
            const uint32_t g = e / a.k, i = e % a.k;
            const uint32_t ng = s_hdr[g] & 0xffffu;
            if (i >= ng)
                continue;
            const uint2 c = reinterpret_cast<const uint2*>(rec(g) + kVpHeaderBytes)[i];
            const float x = __fmul_rn(__fsub_rn(__uint_as_float(c.x), m), inv_t);
            const float q = expf_host_exact(x);
            if (q >= minp_eff && q > 0.0f) {
                const uint32_t slot = atomicAdd(&s_n, 1u);
                keys[slot] = ((unsigned long long)__float_as_uint(q) << 32) | (g << kShardShift) | c.y;
            }
        }
    }
    __syncthreads();
    uint32_t n = s_n;
    if (n == 0) {
        flags |= MK_FLAG_NO_CANDIDATE;
        if (tid == 0)
            keys[0] = ((unsigned long long)__float_as_uint(1.0f) << 32) | arg_shard << kShardShift | arg_id;
        n = 1;
        __syncthreads();
    }
    const bool minp_on = minp_eff > 0.0f;
    const bool cut_k = prm.top_k > 0 && prm.top_k < n;
    const bool use_topp = prm.top_p < 1.0f;
    const bool sorted = cut_k || use_topp;
    const bool need_sum = use_topp && !minp_on && !(prm.top_k > 0 && prm.top_k < a.n_vocab_total);
    uint32_t n2 = 2;
    while (n2 < n)
        n2 <<= 1;
    for (uint32_t i = tid; i < n2; i += n_thr) {
        unsigned long long key = ~0ull;
        if (i < n) {
            const unsigned long long raw = keys[i];
            const uint32_t qb = (uint32_t)(raw >> 32), id = (uint32_t)(raw & 0xffffffffull);
            key = sorted ? (((unsigned long long)(~qb) << 32) | id) : (((unsigned long long)id << 32) | qb);
        }
        keys[i] = key;
    }
    __syncthreads();
    if (n > 1)
        sort_keys(keys, n2, n_thr);

    // The rest is sequential by the reference's definition (double sums for top_p, a float total, the walk) or tiny:
    // one warp runs it, the candidates handed round 32 at a time by shuffles so that no chain waits for a load.
    if (tid < 32) {
        const uint32_t lane = tid, full = 0xffffffffu;
        auto q_at = [&](uint32_t i) -> float {
            const unsigned long long key = keys[i];
            return sorted ? __uint_as_float(~(uint32_t)(key >> 32)) : __uint_as_float((uint32_t)(key & 0xffffffffull));
        };
        auto tag_at = [&](uint32_t i) -> uint32_t { // shard << kShardShift | token id
            const unsigned long long key = keys[i];
            return sorted ? (uint32_t)(key & 0xffffffffull) : (uint32_t)(key >> 32);
        };
        // A shard whose whole list is inside the deciding set may hold further members the merge cannot see.
        uint32_t n_decide = n; // the set whose completeness matters: all candidates when the total is their sum
        if (cut_k)
            n = prm.top_k;
        if (use_topp) {
            double total = 0.0, band;
            if (need_sum && !(flags & MK_FLAG_NO_CANDIDATE)) {
                const double c2 = (double)inv_t * 1.4426950408889634;
                for (uint32_t g0 = 0; g0 < a.n_shards; g0 += 32u) { // the shards' rescaled sums, added in shard order
                    const uint32_t g = g0 + lane;
                    double term = 0.0;
                    if (g < a.n_shards && s_max[g] > ninf && s_sum[g] > 0.0)
                        term = s_sum[g] * exp2((double)(s_max[g] - m) * c2);
                    const int cnt = (int)min(32u, a.n_shards - g0);
                    for (int j = 0; j < cnt; ++j)
                        total += __shfl_sync(full, term, j);
                }
                band = 1e-5 * total;
            } else {
                for (uint32_t base = 0; base < n; base += 32u) {
                    const float q = (base + lane < n) ? q_at(base + lane) : 0.0f;
                    const int cnt = (int)min(32u, n - base);
                    for (int j = 0; j < cnt; ++j)
                        total += (double)__shfl_sync(full, q, j);
                }
                band = 0x1p-40 * total;
            }
            const double want = (double)prm.top_p * total;
            double run = 0.0, prev = 0.0;
            uint32_t k = 0;
            bool open = true;
            for (uint32_t base = 0; base < n && open; base += 32u) {
                const float q = (base + lane < n) ? q_at(base + lane) : 0.0f;
                const int cnt = (int)min(32u, n - base);
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
            if (need_sum && run < want)
                flags |= MK_FLAG_VP_TRUNCATED;
            if (k >= 1 && (fabs(run - want) <= band || (k >= 2 && fabs(prev - want) <= band)))
                flags |= MK_FLAG_GUARD_BAND;
            n = max(k, 1u);
            if (need_sum)
                n_decide = n;
        }
        if (cut_k && !use_topp)
            n_decide = n;
        else if (cut_k)
            n_decide = min(n_decide, prm.top_k);
        // count members per shard among the deciding set
        for (uint32_t i = lane; i < n_decide; i += 32u)
            atomicAdd(&s_shard_in[tag_at(i) >> kShardShift], 1u);
        __syncwarp();
        bool cut_short = false;
        for (uint32_t g = lane; g < a.n_shards && g < 64u; g += 32u) {
            const uint32_t hdr = s_hdr[g];
            const uint32_t ng = hdr & 0xffffu;
            const bool more = (hdr & 0x40000000u) != 0;
            cut_short = cut_short || (hdr & 0x80000000u) || (more && ng > 0 && s_shard_in[g] >= ng);
        }
        if (__any_sync(full, cut_short))
            flags |= MK_FLAG_VP_TRUNCATED;
        float total = 0.0f;
        for (uint32_t base = 0; base < n; base += 32u) {
            const float q = (base + lane < n) ? q_at(base + lane) : 0.0f;
            const int cnt = (int)min(32u, n - base);
            for (int j = 0; j < cnt; ++j)
                total = __fadd_rn(total, __shfl_sync(full, q, j));
        }
        float r = __fmul_rn(a.u[row], total);
        const float eps = 1e-6f * total;
        uint32_t hit = n - 1u;
        float q_hit = q_at(n - 1u);
        bool found = false;
        for (uint32_t base = 0; base < n && !found; base += 32u) {
            const float q = (base + lane < n) ? q_at(base + lane) : 0.0f;
            const int cnt = (int)min(32u, n - base);
            for (int j = 0; j < cnt && !found; ++j) {
                const float qj = __shfl_sync(full, q, j);
                const uint32_t i = base + (uint32_t)j;
                if (r < qj) {
                    found = true;
                    hit = i;
                    q_hit = qj;
                    if ((i > 0 && r < eps) || (i + 1 < n && __fsub_rn(qj, r) < eps))
                        flags |= MK_FLAG_NEAR_CDF_BOUNDARY;
                } else {
                    r = __fsub_rn(r, qj);
                }
            }
        }
        if (lane == 0) {
            if (a.token) a.token[row] = (int32_t)(tag_at(hit) & kIdMask);
            if (a.prob) a.prob[row] = __fdiv_rn(q_hit, total);
            if (a.flags) a.flags[row] = flags;
            if (a.n_cand) a.n_cand[row] = n;
            s_nfinal = n;
        }
    }
    __syncthreads();
    if (a.cand_ids || a.cand_q) {
        const uint32_t nf = min(s_nfinal, a.cand_cap);
        for (uint32_t i = tid; i < nf; i += n_thr) {
            const unsigned long long key = keys[i];
            const uint32_t id = (sorted ? (uint32_t)(key & 0xffffffffull) : (uint32_t)(key >> 32)) & kIdMask;
            const float q = sorted ? __uint_as_float(~(uint32_t)(key >> 32)) : __uint_as_float((uint32_t)(key & 0xffffffffull));
            if (a.cand_ids) a.cand_ids[(size_t)row * a.cand_cap + i] = (int32_t)id;
            if (a.cand_q) a.cand_q[(size_t)row * a.cand_cap + i] = q;
        }
    }
}

cudaError_t launch_vp_merge(const VpMergeArgs& a, cudaStream_t stream)
{
    if (a.batch == 0)
        return cudaSuccess;
    vp_merge_kernel<<<a.batch, a.batch <= 16u ? kMergeThreadsFew : kMergeThreads, 0, stream>>>(a);
    return cudaGetLastError();
}

// ---- p/q rejection sampling from two candidate lists ---------------------------------------------------------------
// One CTA per position. p_* / q_* are the final candidate lists (draw order) of the target and drafter rows with
// their float totals; draft_token was drawn from q. Accept iff u_accept * q(d) < p(d) on normalised probabilities;
// otherwise walk max(0, p - q) over the union in ascending id with u_resample.
namespace {
constexpr int kPqThreads = 512; // the sort of two long lists (a flat row: thousands of candidates each) is what takes the time
}

// The rejected position's resample when a list runs to hundreds or thousands of entries: no sort. Each list marks its
// ids in a bitmap of the vocabulary; the number of marked ids before each word (a prefix popcount) makes an id's place
// in ascending order one popcount away. The drafter's weights are laid out by that rank, every target entry looks its
// id up in the drafter's bitmap and leaves max-able residual p/P - q/Q at its own rank, and one warp adds and walks the
// residuals in ascending id as the restated rule demands. Shared memory: two bitmaps, two rank arrays, two float
// arrays by rank.
constexpr uint32_t kPqBitmapVocab = 163840, kPqBmWords = kPqBitmapVocab / 32, kPqRankMin = 256;
constexpr size_t kPqRankSmem = 2 * (kPqBmWords * 4 + kPqBmWords * 2) + 2 * 4096 * 4;
__device__ __noinline__ void pq_resolve_by_rank(const PqResolveArgs& a, uint32_t row, uint32_t np, uint32_t nq, float total_p,
                                                float total_q, int32_t d, uint32_t fl)
{
    extern __shared__ unsigned long long pq_keys[];
    __shared__ uint32_t s_wtot[2][kPqThreads / 32];
    unsigned char* const base = reinterpret_cast<unsigned char*>(pq_keys);
    uint32_t* const bm_p = reinterpret_cast<uint32_t*>(base);
    uint32_t* const bm_q = bm_p + kPqBmWords;
    uint16_t* const wp_p = reinterpret_cast<uint16_t*>(bm_q + kPqBmWords);
    uint16_t* const wp_q = wp_p + kPqBmWords;
    float* const res = reinterpret_cast<float*>(wp_q + kPqBmWords); // residuals of the target's entries, by rank
    float* const qv = res + a.cap;                                    // the drafter's weights, by rank
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t words = (a.n_vocab + 31u) >> 5;
    __syncthreads(); // the lists staged for the sort path are dead from here
    for (uint32_t w = tid; w < 2u * kPqBmWords; w += kPqThreads)
        bm_p[w] = 0u;
    __syncthreads();
    const int32_t* const pid = a.p_ids + (size_t)row * a.cap;
    const int32_t* const qid = a.q_ids + (size_t)row * a.cap;
    const float* const pw = a.p_q + (size_t)row * a.cap;
    const float* const qw = a.q_q + (size_t)row * a.cap;
    for (uint32_t i = tid; i < np; i += kPqThreads) {
        const uint32_t c = (uint32_t)(pid[i] - a.id_offset);
        atomicOr(&bm_p[c >> 5], 1u << (c & 31u));
    }
    for (uint32_t i = tid; i < nq; i += kPqThreads) {
        const uint32_t c = (uint32_t)(qid[i] - a.id_offset);
        atomicOr(&bm_q[c >> 5], 1u << (c & 31u));
    }
    __syncthreads();
    // prefix popcounts of both bitmaps: each thread a run of words, a scan over the threads' sums
    const uint32_t per = (words + kPqThreads - 1u) / kPqThreads, w0 = min(tid * per, words), w1 = min(w0 + per, words);
    uint32_t mine_p = 0, mine_q = 0;
    for (uint32_t w = w0; w < w1; ++w) {
        mine_p += (uint32_t)__popc(bm_p[w]);
        mine_q += (uint32_t)__popc(bm_q[w]);
    }
    uint32_t inc_p = mine_p, inc_q = mine_q;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t yp = __shfl_up_sync(0xffffffffu, inc_p, o), yq = __shfl_up_sync(0xffffffffu, inc_q, o);
        if ((int)lane >= o) {
            inc_p += yp;
            inc_q += yq;
        }
    }
    if (lane == 31) {
        s_wtot[0][warp] = inc_p;
        s_wtot[1][warp] = inc_q;
    }
    __syncthreads();
    uint32_t before_p = inc_p - mine_p, before_q = inc_q - mine_q;
    for (uint32_t w = 0; w < warp; ++w) {
        before_p += s_wtot[0][w];
        before_q += s_wtot[1][w];
    }
    for (uint32_t w = w0; w < w1; ++w) {
        wp_p[w] = (uint16_t)before_p;
        wp_q[w] = (uint16_t)before_q;
        before_p += (uint32_t)__popc(bm_p[w]);
        before_q += (uint32_t)__popc(bm_q[w]);
    }
    __syncthreads();
    for (uint32_t i = tid; i < nq; i += kPqThreads) {
        const uint32_t c = (uint32_t)(qid[i] - a.id_offset);
        qv[wp_q[c >> 5] + __popc(bm_q[c >> 5] & ((1u << (c & 31u)) - 1u))] = qw[i];
    }
    __syncthreads();
    for (uint32_t i = tid; i < np; i += kPqThreads) {
        const uint32_t c = (uint32_t)(pid[i] - a.id_offset), bit = 1u << (c & 31u);
        const float pn = __fdiv_rn(pw[i], total_p);
        float qn = 0.0f;
        if (bm_q[c >> 5] & bit)
            qn = __fdiv_rn(qv[wp_q[c >> 5] + __popc(bm_q[c >> 5] & (bit - 1u))], total_q);
        res[wp_p[c >> 5] + __popc(bm_p[c >> 5] & (bit - 1u))] = __fsub_rn(pn, qn);
    }
    __syncthreads();
    if (tid < 32) {
        const uint32_t full = 0xffffffffu;
        float total_r = 0.0f;
        uint32_t n_res = 0;
        for (uint32_t base_i = 0; base_i < np; base_i += 32u) {
            const float r_l = (base_i + lane < np) ? res[base_i + lane] : 0.0f;
            const int cnt = (int)min(32u, np - base_i);
            for (int j = 0; j < cnt; ++j) {
                const float rj = __shfl_sync(full, r_l, j);
                if (rj > 0.0f) {
                    total_r = __fadd_rn(total_r, rj);
                    ++n_res;
                }
            }
        }
        float r = __fmul_rn(a.u_resample[row], total_r);
        uint32_t hit = 0xffffffffu, last = 0xffffffffu; // ranks
        bool done = false;
        for (uint32_t base_i = 0; base_i < np && !done; base_i += 32u) {
            const float r_l = (base_i + lane < np) ? res[base_i + lane] : 0.0f;
            const int cnt = (int)min(32u, np - base_i);
            for (int j = 0; j < cnt && !done; ++j) {
                const float rj = __shfl_sync(full, r_l, j);
                if (rj > 0.0f) {
                    last = base_i + (uint32_t)j;
                    if (r < rj) {
                        hit = last;
                        done = true;
                    } else {
                        r = __fsub_rn(r, rj);
                    }
                }
            }
        }
        if (!done)
            hit = last;
        if (lane == 0) {
            int32_t tok = d;
            if (n_res && hit != 0xffffffffu) {
                // the id of rank `hit`: the last word whose prefix does not exceed it, then its (hit - prefix)-th bit
                uint32_t lo = 0, hi = words;
                while (hi - lo > 1u) {
                    const uint32_t mid = (lo + hi) >> 1;
                    if ((uint32_t)wp_p[mid] <= hit)
                        lo = mid;
                    else
                        hi = mid;
                }
                uint32_t bits = bm_p[lo];
                for (uint32_t k = hit - wp_p[lo]; k > 0u; --k)
                    bits &= bits - 1u;
                tok = (int32_t)(lo * 32u + (uint32_t)(__ffs((int)bits) - 1)) + a.id_offset;
            }
            a.accepted[row] = 0;
            a.token[row] = tok;
            if (a.flags) a.flags[row] = fl;
        }
    }
}

__global__ void __launch_bounds__(kPqThreads) pq_resolve_kernel(const PqResolveArgs a)
{
    extern __shared__ unsigned long long pq_keys[]; // [2][cap2]
    __shared__ float s_pd;
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const uint32_t np = a.p_n[row], nq = a.q_n[row];
    const uint32_t bad = MK_FLAG_OVERFLOW | MK_FLAG_TIMEOUT;
    const uint32_t fl = (a.p_flags[row] | a.q_flags[row]);
    if ((fl & bad) || np > a.cap || nq > a.cap) {
        if (tid == 0) {
            a.accepted[row] = 0;
            a.token[row] = -1;
            if (a.flags) a.flags[row] = fl | MK_FLAG_OVERFLOW;
        }
        return;
    }
    uint32_t cap2 = 2;
    while (cap2 < a.cap)
        cap2 <<= 1;
    unsigned long long* kp = pq_keys;
    unsigned long long* kq = pq_keys + cap2;
    const int32_t d = a.draft_token[row];
    if (tid == 0)
        s_pd = 0.0f;
    __syncthreads();
    const float total_p = a.p_total[row], total_q = a.q_total[row];
    uint32_t n2p = 2, n2q = 2;
    while (n2p < np) n2p <<= 1;
    while (n2q < nq) n2q <<= 1;
    for (uint32_t i = tid; i < n2p; i += kPqThreads) {
        unsigned long long key = ~0ull;
        if (i < np) {
            const int32_t id = a.p_ids[(size_t)row * a.cap + i];
            const float q = a.p_q[(size_t)row * a.cap + i];
            key = ((unsigned long long)(uint32_t)id << 32) | __float_as_uint(q);
            if (id == d)
                s_pd = __fdiv_rn(q, total_p);
        }
        kp[i] = key;
    }
    for (uint32_t i = tid; i < n2q; i += kPqThreads) {
        unsigned long long key = ~0ull;
        if (i < nq) {
            const int32_t id = a.q_ids[(size_t)row * a.cap + i];
            key = ((unsigned long long)(uint32_t)id << 32) | __float_as_uint(a.q_q[(size_t)row * a.cap + i]);
        }
        kq[i] = key;
    }
    __syncthreads();
    const float pd = s_pd;
    const float qd = a.q_prob[row];
    const bool acc = __fmul_rn(a.u_accept[row], qd) < pd;
    if (acc) {
        if (tid == 0) {
            a.accepted[row] = 1;
            a.token[row] = d;
            if (a.flags) a.flags[row] = fl;
        }
        return;
    }
    if (a.n_vocab <= kPqBitmapVocab && a.cap <= 4096u && max(np, nq) > kPqRankMin) {
        pq_resolve_by_rank(a, row, np, nq, total_p, total_q, d, fl);
        return;
    }
    // sort both lists by id
    for (uint32_t k = 2; k <= max(n2p, n2q); k <<= 1) {
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            for (uint32_t i = tid; i < max(n2p, n2q); i += kPqThreads) {
                const uint32_t o = i ^ j;
                if (o > i) {
                    const bool up = (i & k) == 0;
                    if (k <= n2p && i < n2p) {
                        const unsigned long long x = kp[i], y = kp[o];
                        if ((x > y) == up) { kp[i] = y; kp[o] = x; }
                    }
                    if (k <= n2q && i < n2q) {
                        const unsigned long long x = kq[i], y = kq[o];
                        if ((x > y) == up) { kq[i] = y; kq[o] = x; }
                    }
                }
            }
            __syncthreads();
        }
    }
    // The residual max(0, p - q) is zero wherever p is: only the target's candidates matter, in ascending id. Every
    // thread looks its candidates' drafter probabilities up by binary search (the drafter's list is sorted by id
    // too) and leaves the residual beside the id; the float total and the walk, sequential by definition, are then
    // chains one warp runs on values handed round by shuffles.
    for (uint32_t i = tid; i < np; i += kPqThreads) {
        const unsigned long long kpi = kp[i];
        const uint32_t id = (uint32_t)(kpi >> 32);
        const float pn = __fdiv_rn(__uint_as_float((uint32_t)(kpi & 0xffffffffull)), total_p);
        uint32_t lo = 0, hi = nq;
        while (lo < hi) {
            const uint32_t mid = (lo + hi) >> 1;
            if ((uint32_t)(kq[mid] >> 32) < id)
                lo = mid + 1;
            else
                hi = mid;
        }
        float qn = 0.0f;
        if (lo < nq && (uint32_t)(kq[lo] >> 32) == id)
            qn = __fdiv_rn(__uint_as_float((uint32_t)(kq[lo] & 0xffffffffull)), total_q);
        kp[i] = ((unsigned long long)id << 32) | __float_as_uint(__fsub_rn(pn, qn));
    }
    __syncthreads();
    if (tid < 32) {
        const uint32_t lane = tid, full = 0xffffffffu;
        float total_r = 0.0f;
        uint32_t n_res = 0;
        for (uint32_t base = 0; base < np; base += 32u) {
            const float res = (base + lane < np) ? __uint_as_float((uint32_t)(kp[base + lane] & 0xffffffffull)) : 0.0f;
            const int cnt = (int)min(32u, np - base);
            for (int j = 0; j < cnt; ++j) {
                const float rj = __shfl_sync(full, res, j);
                if (rj > 0.0f) {
                    total_r = __fadd_rn(total_r, rj);
                    ++n_res;
                }
            }
        }
        float r = __fmul_rn(a.u_resample[row], total_r);
        int32_t tok = d, last = d;
        bool done = false;
        for (uint32_t base = 0; base < np && !done; base += 32u) {
            const unsigned long long e = (base + lane < np) ? kp[base + lane] : 0ull;
            const float res = __uint_as_float((uint32_t)(e & 0xffffffffull));
            const int32_t id = (int32_t)(uint32_t)(e >> 32);
            const int cnt = (int)min(32u, np - base);
            for (int j = 0; j < cnt && !done; ++j) {
                const float rj = __shfl_sync(full, res, j);
                const int32_t idj = __shfl_sync(full, id, j);
                if (rj > 0.0f) {
                    last = idj;
                    if (r < rj) {
                        tok = idj;
                        done = true;
                    } else {
                        r = __fsub_rn(r, rj);
                    }
                }
            }
        }
        if (!done)
            tok = last;
        if (lane == 0) {
            a.accepted[row] = 0;
            a.token[row] = n_res ? tok : d;
            if (a.flags) a.flags[row] = fl;
        }
    }
}

cudaError_t launch_pq_resolve(const PqResolveArgs& a, cudaStream_t stream)
{
    if (a.batch == 0)
        return cudaSuccess;
    uint32_t cap2 = 2;
    while (cap2 < a.cap)
        cap2 <<= 1;
    size_t smem = 2 * (size_t)cap2 * 8;
    if (a.n_vocab <= kPqBitmapVocab && a.cap <= 4096 && smem < kPqRankSmem)
        smem = kPqRankSmem;
    static bool configured[64] = {}; // the attribute is per device
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return e;
    if (smem > 48 * 1024 && !(dev >= 0 && dev < 64 && configured[dev])) {
        e = cudaFuncSetAttribute(pq_resolve_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess)
            return e;
        if (dev >= 0 && dev < 64)
            configured[dev] = true;
    }
    pq_resolve_kernel<<<a.batch, kPqThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

// ---- acceptance loop of a speculative round (src/gen/session.cpp:481-496, 505) -------------------------------------
__global__ void spec_resolve_kernel(uint32_t n_seq, uint32_t n_pos, const int32_t* accepted, const int32_t* token,
                                    int32_t* n_kept, int32_t* next_token)
{
    const uint32_t sq = blockIdx.x * blockDim.x + threadIdx.x;
    if (sq >= n_seq)
        return;
    uint32_t kept = 0;
    while (kept + 1 < n_pos && accepted[(size_t)sq * n_pos + kept])
        ++kept;
    n_kept[sq] = (int32_t)kept;
    next_token[sq] = token[(size_t)sq * n_pos + kept]; // the replacement, or the bonus position's token
}

cudaError_t launch_spec_resolve(uint32_t n_seq, uint32_t n_pos, const int32_t* accepted, const int32_t* token,
                                int32_t* n_kept, int32_t* next_token, cudaStream_t stream)
{
    if (n_seq == 0)
        return cudaSuccess;
    spec_resolve_kernel<<<(n_seq + 127) / 128, 128, 0, stream>>>(n_seq, n_pos, accepted, token, n_kept, next_token);
    return cudaGetLastError();
}

// ---- "is this token among the k largest raw logits" (ReasoningBudget::forced, src/server/openai.cpp:596-603) --------
// One CTA per row streams the row once with 128-bit loads and counts the logits strictly greater than the token's
// (NaN compares false, as in the reference's loop). HBM-bound: 4 bytes per column.
constexpr int kRankThreads = 512;
__global__ void __launch_bounds__(kRankThreads) rank_force_kernel(const float* logits, uint64_t ld, uint32_t n_vocab,
                                                                 const int32_t* token, uint32_t k, int32_t* forced,
                                                                 uint32_t* above)
{
    __shared__ uint32_t s_part[kRankThreads / 32];
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const int32_t t = token[row];
    if (t < 0 || (uint32_t)t >= n_vocab) { // no such token in this vocabulary: nothing is forced (openai.cpp:595)
        if (tid == 0) {
            if (forced) forced[row] = -1;
            if (above) above[row] = 0xffffffffu;
        }
        return;
    }
    const float* lrow = logits + (size_t)row * ld;
    const float v = __ldg(lrow + t);
    uint32_t cnt = 0;
    if (((reinterpret_cast<uintptr_t>(lrow) & 15u) == 0)) {
        const float4* p4 = reinterpret_cast<const float4*>(lrow);
        const uint32_t n4 = n_vocab / 4u;
        uint32_t i = tid;
        for (; i + 3u * kRankThreads < n4; i += 4u * kRankThreads) { // four loads in flight per thread
            const float4 x0 = __ldg(p4 + i), x1 = __ldg(p4 + i + kRankThreads), x2 = __ldg(p4 + i + 2 * kRankThreads),
                         x3 = __ldg(p4 + i + 3 * kRankThreads);
            cnt += (x0.x > v) + (x0.y > v) + (x0.z > v) + (x0.w > v) + (x1.x > v) + (x1.y > v) + (x1.z > v) + (x1.w > v) +
                   (x2.x > v) + (x2.y > v) + (x2.z > v) + (x2.w > v) + (x3.x > v) + (x3.y > v) + (x3.z > v) + (x3.w > v);
        }
        for (; i < n4; i += kRankThreads) {
            const float4 x = __ldg(p4 + i);
            cnt += (x.x > v) + (x.y > v) + (x.z > v) + (x.w > v);
        }
        for (uint32_t c = n4 * 4u + tid; c < n_vocab; c += kRankThreads)
            cnt += __ldg(lrow + c) > v;
    } else {
        for (uint32_t c = tid; c < n_vocab; c += kRankThreads)
            cnt += __ldg(lrow + c) > v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if ((tid & 31u) == 0)
        s_part[tid >> 5] = cnt;
    __syncthreads();
    if (tid == 0) {
        uint32_t total = 0;
        for (int w = 0; w < kRankThreads / 32; ++w)
            total += s_part[w];
        if (above) above[row] = total;
        if (forced) forced[row] = (total < k) ? t : -1;
    }
}

cudaError_t launch_rank_force(const float* logits, uint64_t ld, uint32_t batch, uint32_t n_vocab, const int32_t* token,
                              uint32_t k, int32_t* forced, uint32_t* above, cudaStream_t stream)
{
    if (batch == 0)
        return cudaSuccess;
    rank_force_kernel<<<batch, kRankThreads, 0, stream>>>(logits, ld, n_vocab, token, k, forced, above);
    return cudaGetLastError();
}

// ---- drafter pick (ds_markov + ds_draft_pick, src/kernels/dsv41.metal:664-742) ---------------------------------------
// score[b][v] = logits[b][v] + head[v] . embed[prev[b]]; draft[b] = argmax_v score (lowest id on ties);
// conf[b] = sigmoid([x[b], embed[prev[b]]] . w). The reference writes the scores to memory and picks in a second
// kernel; here the scores never leave the registers: each warp keeps a head row in registers (rank / 32 floats per
// lane), takes its dot product with every sequence's embedding row (shared memory) and folds it into a running best;
// CTAs combine through one 64-bit atomic maximum per sequence on (order key of the score, ~id); the last CTA to
// arrive writes the results: one launch per step. HBM-bound on the head
// matrix: 4 * rank bytes per vocabulary row, read once for all sequences of the launch.
constexpr int kPickThreads = 256, kPickMaxSeq = 8, kPickMaxRank = 256;

template <int kSeq> // sequences the launch can carry: 1 (the reference's case, fewer registers) or kPickMaxSeq
__global__ void __launch_bounds__(kPickThreads, kSeq == 1 ? 4 : 2) draft_score_kernel(const float* logits, uint64_t ld, const float* head,
                                                                  const float* embed, const int32_t* prev,
                                                                  uint32_t n_seq, uint32_t n_vocab, uint32_t rank,
                                                                  uint32_t n_embed, unsigned long long* best,
                                                                  const float* x, uint64_t x_ld, const float* w,
                                                                  uint32_t dim, int32_t* draft, float* conf)
{
    __shared__ __align__(16) float s_e[kSeq][kPickMaxRank];
    __shared__ unsigned long long s_best[kSeq];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    for (uint32_t i = tid; i < (uint32_t)kSeq * kPickMaxRank; i += kPickThreads) {
        const uint32_t b = i / kPickMaxRank, j = i - b * kPickMaxRank;
        const int32_t p = (b < n_seq) ? prev[b] : -1;
        s_e[b][j] = (j < rank && p >= 0 && (uint32_t)p < n_embed) ? __ldg(embed + (size_t)p * rank + j) : 0.0f;
    }
    if (tid < kSeq)
        s_best[tid] = 0ull;
    __syncthreads();
    unsigned long long mine[1] = {0ull}; // running best: of the one sequence, or of this lane's sequence (lane / 4)
    // Four head rows per warp and trip, each lane 2 x 4 consecutive floats of a row (128-bit loads; rank a multiple
    // of 4, the rest of a shorter rank reads as zero): 4 KB in flight per warp.
    constexpr uint32_t kRows = 4;
    const uint32_t warps = gridDim.x * (kPickThreads / 32);
    for (uint32_t v0 = (blockIdx.x * (kPickThreads / 32) + warp) * kRows; v0 < n_vocab; v0 += warps * kRows) {
        float4 h[kRows][2];
#pragma unroll
        for (uint32_t r = 0; r < kRows; ++r)
#pragma unroll
            for (uint32_t k = 0; k < 2; ++k) {
                const uint32_t i = 4u * lane + 128u * k;
                h[r][k] = (v0 + r < n_vocab && i < rank)
                              ? __ldg(reinterpret_cast<const float4*>(head + (size_t)(v0 + r) * rank + i))
                              : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        if constexpr (kSeq == 1) {
    #pragma unroll
            for (int b = 0; b < kSeq; ++b) {
                if ((uint32_t)b >= n_seq)
                    break;
                const float4 e0 = *reinterpret_cast<const float4*>(&s_e[b][4u * lane]);
                const float4 e1 = *reinterpret_cast<const float4*>(&s_e[b][4u * lane + 128u]);
    #pragma unroll
                for (uint32_t r = 0; r < kRows; ++r) {
                    float acc = h[r][0].x * e0.x;
                    acc = fmaf(h[r][0].y, e0.y, acc);
                    acc = fmaf(h[r][0].z, e0.z, acc);
                    acc = fmaf(h[r][0].w, e0.w, acc);
                    acc = fmaf(h[r][1].x, e1.x, acc);
                    acc = fmaf(h[r][1].y, e1.y, acc);
                    acc = fmaf(h[r][1].z, e1.z, acc);
                    acc = fmaf(h[r][1].w, e1.w, acc);
    #pragma unroll
                    for (int o = 16; o > 0; o >>= 1)
                        acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    const uint32_t v = v0 + r;
                    if (v < n_vocab) {
                        const float sc = __ldg(logits + (size_t)b * ld + v) + acc;
                        // larger score wins, then the lower id: the id enters complemented; NaN and -inf never win
                        // (`s > bv` from bv = -inf in the reference): key 0
                        const unsigned long long key = (sc > -__int_as_float(0x7f800000))
                                                           ? (((unsigned long long)order_key(sc) << 32) | (0xffffffffu - v))
                                                           : 0ull;
                        mine[b] = max(mine[b], key);
                    }
                }
            }
        } else {
            // 4 rows x 8 sequences = 32 dot products per trip: every lane forms its share of all 32, then a butterfly
            // that halves the number of values a lane holds at each of its five steps (31 shuffles instead of 160)
            // leaves lane l with the total of product l = sequence l / 4, row l % 4.
            static_assert(kSeq == 8 && kRows == 4, "the butterfly below is written for 32 products");
            float acc[32];
#pragma unroll
            for (int q = 0; q < kSeq; ++q) {
                const float4 e0 = *reinterpret_cast<const float4*>(&s_e[q][4u * lane]);
                const float4 e1 = *reinterpret_cast<const float4*>(&s_e[q][4u * lane + 128u]);
                // two lanes of the product per instruction (even and odd elements apart, added at the end): the kernel
                // is bound by the issue of its multiply-adds, not by memory
#pragma unroll
                for (uint32_t r = 0; r < kRows; ++r) {
                    float2 t = mul2(make_float2(h[r][0].x, h[r][0].y), make_float2(e0.x, e0.y));
                    t = fma2(make_float2(h[r][0].z, h[r][0].w), make_float2(e0.z, e0.w), t);
                    t = fma2(make_float2(h[r][1].x, h[r][1].y), make_float2(e1.x, e1.y), t);
                    t = fma2(make_float2(h[r][1].z, h[r][1].w), make_float2(e1.z, e1.w), t);
                    acc[q * 4 + (int)r] = t.x + t.y;
                }
            }
#pragma unroll
            for (int half = 16; half > 0; half >>= 1) {
                const bool upper = (lane & (uint32_t)half) != 0;
#pragma unroll
                for (int i = 0; i < half; ++i) {
                    const float send = upper ? acc[i] : acc[i + half];
                    const float keep = upper ? acc[i + half] : acc[i];
                    acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
                }
            }
            const uint32_t q = lane >> 2, v = v0 + (lane & 3u);
            if (q < n_seq && v < n_vocab) {
                const float sc = __ldg(logits + (size_t)q * ld + v) + acc[0];
                const unsigned long long key = (sc > -__int_as_float(0x7f800000))
                                                   ? (((unsigned long long)order_key(sc) << 32) | (0xffffffffu - v))
                                                   : 0ull;
                mine[0] = max(mine[0], key); // this lane's sequence is lane / 4
            }
        }
    }
    if constexpr (kSeq == 1) {
        if (lane == 0 && mine[0])
            atomicMax(&s_best[0], mine[0]);
    } else {
        unsigned long long m = mine[0]; // lanes 4q .. 4q+3 hold sequence q
        m = max(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = max(m, __shfl_xor_sync(0xffffffffu, m, 2));
        if ((lane & 3u) == 0 && (lane >> 2) < n_seq && m)
            atomicMax(&s_best[lane >> 2], m);
    }
    __syncthreads();
    if (tid < n_seq && s_best[tid])
        atomicMax(&best[tid], s_best[tid]);
    // The CTA that arrives last (a ticket counter behind the maxima) has every CTA's maximum in front of it: it
    // writes the drafts and the confidences (ds_draft_pick's second half) and leaves maxima and counter clear for the
    // next call.
    __shared__ uint32_t s_last;
    __shared__ float s_part[kPickThreads / 32];
    __threadfence();
    __syncthreads();
    if (tid == 0)
        s_last = atomicAdd(reinterpret_cast<unsigned int*>(best + kPickMaxSeq), 1u) == gridDim.x - 1u;
    __syncthreads();
    if (!s_last)
        return;
    __threadfence();
    for (uint32_t b = 0; b < n_seq; ++b) {
        float d = 0.0f;
        for (uint32_t i = tid; i < dim + rank; i += kPickThreads)
            d = fmaf(__ldg(w + i), i < dim ? __ldg(x + (size_t)b * x_ld + i) : s_e[b][i - dim], d);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            d += __shfl_xor_sync(0xffffffffu, d, o);
        if (lane == 0)
            s_part[warp] = d;
        __syncthreads();
        if (tid == 0) {
            float sum = 0.0f;
            for (int k = 0; k < kPickThreads / 32; ++k)
                sum += s_part[k];
            const unsigned long long key = *(volatile unsigned long long*)&best[b];
            best[b] = 0ull;
            draft[b] = key ? (int32_t)(0xffffffffu - (uint32_t)(key & 0xffffffffull)) : 0; // nothing comparable: id 0
            conf[b] = 1.0f / (1.0f + expf(-sum));
        }
        __syncthreads();
    }
    if (tid == 0)
        *reinterpret_cast<unsigned int*>(best + kPickMaxSeq) = 0u;
}

cudaError_t launch_draft_pick(const float* logits, uint64_t ld, const float* head, const float* embed, const float* x,
                              uint64_t x_ld, const float* w, const int32_t* prev, uint32_t n_seq, uint32_t n_vocab,
                              uint32_t rank, uint32_t dim, uint32_t n_embed, unsigned long long* best, int32_t* draft,
                              float* conf, cudaStream_t stream)
{
    if (n_seq == 0)
        return cudaSuccess;
    // `best` (the maxima, then the ticket counter) is zero on entry: the handle clears it once and the kernel's last
    // CTA clears what it has read
    const uint32_t rows_per_trip = (kPickThreads / 32) * 4;
    // persistent, grid-stride: as many CTAs as stay resident (four per SM for one sequence, two for several)
    const uint32_t grid = min((n_vocab + rows_per_trip - 1) / rows_per_trip, 148u * (n_seq == 1 ? 4u : 2u));
    if (n_seq == 1)
        draft_score_kernel<1><<<grid, kPickThreads, 0, stream>>>(logits, ld, head, embed, prev, n_seq, n_vocab, rank,
                                                                n_embed, best, x, x_ld, w, dim, draft, conf);
    else
        draft_score_kernel<kPickMaxSeq><<<grid, kPickThreads, 0, stream>>>(logits, ld, head, embed, prev, n_seq, n_vocab,
                                                                          rank, n_embed, best, x, x_ld, w, dim, draft, conf);
    return cudaGetLastError();
}

// ---- plain drafter pick (hy4_draft_pick, src/kernels/hy4f.metal:352-397) ------------------------------------------------
// draft = the largest logit (the lowest index on ties; 0 when nothing is above -inf), conf = sigmoid(conf_w . h + bias).
// One CTA per sequence, as the reference has one threadgroup: a latency kernel over one 0.5 MB row.
constexpr int kPlainPickThreads = 1024;
__global__ void __launch_bounds__(kPlainPickThreads) draft_pick_plain_kernel(const float* logits, uint64_t ld,
                                                                            uint32_t n_vocab, const float* h,
                                                                            uint64_t h_ld, const float* conf_w,
                                                                            uint32_t width, float conf_bias,
                                                                            int32_t* draft, float* conf, int32_t* next_prev)
{
    __shared__ unsigned long long s_key[kPlainPickThreads / 32];
    __shared__ float s_dot[kPlainPickThreads / 32];
    const uint32_t b = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const float* lrow = logits + (size_t)b * ld;
    const float ninf = -__int_as_float(0x7f800000);
    unsigned long long key = 0ull; // (order key of the value, ~index): the larger value, then the lower index
    auto take = [&](float v, uint32_t i) {
        if (v > ninf)
            key = max(key, ((unsigned long long)order_key(v) << 32) | (0xffffffffu - i));
    };
    if ((reinterpret_cast<uintptr_t>(lrow) & 15u) == 0) {
        const float4* p4 = reinterpret_cast<const float4*>(lrow);
        const uint32_t n4 = n_vocab / 4u;
        for (uint32_t i = tid; i < n4; i += kPlainPickThreads) {
            const float4 x = __ldg(p4 + i);
            take(x.x, 4u * i);
            take(x.y, 4u * i + 1u);
            take(x.z, 4u * i + 2u);
            take(x.w, 4u * i + 3u);
        }
        for (uint32_t c = n4 * 4u + tid; c < n_vocab; c += kPlainPickThreads)
            take(__ldg(lrow + c), c);
    } else {
        for (uint32_t c = tid; c < n_vocab; c += kPlainPickThreads)
            take(__ldg(lrow + c), c);
    }
    float d = 0.0f;
    for (uint32_t i = tid; i < width; i += kPlainPickThreads)
        d = fmaf(__ldg(conf_w + i), __ldg(h + (size_t)b * h_ld + i), d);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        key = max(key, __shfl_xor_sync(0xffffffffu, key, o));
        d += __shfl_xor_sync(0xffffffffu, d, o);
    }
    if (lane == 0) {
        s_key[warp] = key;
        s_dot[warp] = d;
    }
    __syncthreads();
    if (tid == 0) {
        unsigned long long k = 0ull;
        float sum = 0.0f;
        for (int i = 0; i < kPlainPickThreads / 32; ++i) {
            k = max(k, s_key[i]);
            sum += s_dot[i];
        }
        const int32_t id = k ? (int32_t)(0xffffffffu - (uint32_t)(k & 0xffffffffull)) : 0;
        draft[b] = id;
        if (next_prev)
            next_prev[b] = id;
        conf[b] = 1.0f / (1.0f + expf(-(sum + conf_bias)));
    }
}

cudaError_t launch_draft_pick_plain(const float* logits, uint64_t ld, uint32_t n_seq, uint32_t n_vocab, const float* h,
                                    uint64_t h_ld, const float* conf_w, uint32_t width, float conf_bias, int32_t* draft,
                                    float* conf, int32_t* next_prev, cudaStream_t stream)
{
    if (n_seq == 0)
        return cudaSuccess;
    draft_pick_plain_kernel<<<n_seq, kPlainPickThreads, 0, stream>>>(logits, ld, n_vocab, h, h_ld, conf_w, width,
                                                                    conf_bias, draft, conf, next_prev);
    return cudaGetLastError();
}

// ---- bookkeeping of one decode step (src/gen/session.cpp:416-444) ----------------------------------------------------
__global__ void decode_commit_kernel(uint32_t batch, const int32_t* sampled, const int32_t* forced, int32_t* history,
                                     uint64_t history_ld, uint32_t history_cap, int32_t* history_len,
                                     int32_t* next_input, int32_t* committed, uint32_t* flags)
{
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch)
        return;
    // a forced token bypasses the sampler but is accepted like any other (session.cpp:441-444)
    const int32_t t = (forced && forced[b] >= 0) ? forced[b] : sampled[b];
    if (committed)
        committed[b] = t;
    if (t < 0) // the row failed (overflow, timeout): nothing to commit
        return;
    if (next_input)
        next_input[b] = t;
    const int32_t len = history_len[b];
    if (len >= 0 && (uint32_t)len < history_cap) {
        history[(size_t)b * history_ld + (uint32_t)len] = t; // Sampler::accept (sampler.cpp:15-18)
        history_len[b] = len + 1;
    } else if (flags) {
        flags[b] |= MK_FLAG_HISTORY_FULL;
    }
}

cudaError_t launch_decode_commit(uint32_t batch, const int32_t* sampled, const int32_t* forced, int32_t* history,
                                 uint64_t history_ld, uint32_t history_cap, int32_t* history_len, int32_t* next_input,
                                 int32_t* committed, uint32_t* flags, cudaStream_t stream)
{
    if (batch == 0)
        return cudaSuccess;
    decode_commit_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(batch, sampled, forced, history, history_ld,
                                                                   history_cap, history_len, next_input, committed,
                                                                   flags);
    return cudaGetLastError();
}

// ---- bookkeeping of one speculative round (src/gen/session.cpp:451-506) ----------------------------------------------
// Per sequence: the drafts kept are accept()ed one by one as the reference emits them (:491), then the token that
// follows them — the replacement at the first rejection, or the bonus row's token — which the reference emits at the
// top of its next round (:456). The history grows by n_kept + 1 entries; next_input gets the token the engine runs
// next.
__global__ void spec_commit_kernel(uint32_t n_seq, uint32_t n_pos, const int32_t* drafts, const int32_t* n_kept,
                                   const int32_t* next_token, int32_t* history, uint64_t history_ld,
                                   uint32_t history_cap, int32_t* history_len, int32_t* next_input, uint32_t* flags)
{
    const uint32_t sq = blockIdx.x * blockDim.x + threadIdx.x;
    if (sq >= n_seq)
        return;
    const int32_t kept = n_kept[sq], nxt = next_token[sq];
    if (next_input)
        next_input[sq] = nxt;
    if (kept < 0 || nxt < 0) // a failed row (overflow, timeout): nothing is committed
        return;
    int32_t len = history_len[sq];
    for (int32_t i = 0; i <= kept; ++i) {
        const int32_t t = (i < kept) ? drafts[(size_t)sq * (n_pos - 1u) + (uint32_t)i] : nxt;
        if (len >= 0 && (uint32_t)len < history_cap) {
            history[(size_t)sq * history_ld + (uint32_t)len] = t; // Sampler::accept (sampler.cpp:15-18)
            ++len;
        } else if (flags) {
            flags[sq] |= MK_FLAG_HISTORY_FULL;
        }
    }
    history_len[sq] = len;
}

cudaError_t launch_spec_commit(uint32_t n_seq, uint32_t n_pos, const int32_t* drafts, const int32_t* n_kept,
                               const int32_t* next_token, int32_t* history, uint64_t history_ld, uint32_t history_cap,
                               int32_t* history_len, int32_t* next_input, uint32_t* flags, cudaStream_t stream)
{
    if (n_seq == 0)
        return cudaSuccess;
    spec_commit_kernel<<<(n_seq + 127) / 128, 128, 0, stream>>>(n_seq, n_pos, drafts, n_kept, next_token, history,
                                                                 history_ld, history_cap, history_len, next_input, flags);
    return cudaGetLastError();
}

} // namespace mk
