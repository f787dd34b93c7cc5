// Block-level exact selection and the final sampling arithmetic.
//
//  * CandidateBuffer   shared-memory list of (score, id) pairs a CTA collects
//                      while it streams a row.
//  * compact_topk      MSB-first radix select (8-bit digits over the 64-bit
//                      (score, ~id) key) that keeps exactly the k best entries;
//                      the reference does the same job per 1024-tile in
//                      shaders/fg_topk_select.comp:51-77 with 5/6-bit digits.
//  * sort_candidates   rank-by-counting sort of <= 64 survivors into sampling
//                      order (src/sampler.c:88-96 does it by insertion).
//  * finish_select     the select step of src/sampler.c:97-121 with the same
//                      fp64 operations in the same left-to-right order; only
//                      the exp() calls are spread over the lanes of a warp.
#pragma once

#include "fg_device_common.cuh"

namespace fgk {

template <int CAP>
struct CandidateBuffer {
    float score[CAP];
    uint32_t id[CAP];
    uint32_t hist[256];
    unsigned long long min_key;
    uint32_t count;      // slots handed out (may run past CAP; stores beyond CAP are dropped)
    uint32_t out_count;
    uint32_t eq_count;
    uint32_t sel_digit, sel_need, sel_bucket;
    float tau_score;     // current lower bound: k-th best (score, id) seen so far
    uint32_t tau_id;
};

// Sorted survivors and the select step's work arrays.
struct FinishBuffer {
    float score[kMaxK];
    uint32_t id[kMaxK];
    double raw[kMaxK];
    double tempered[kMaxK];
    uint32_t cutoff;
    uint32_t picked;
    uint32_t status;
};

// How the threads that share a candidate list meet: the whole CTA by default; a
// kernel whose CTA also holds warps with another job passes a named barrier instead.
struct WholeBlock {
    static __device__ __forceinline__ void sync() { __syncthreads(); }
};

// Keeps the k best of buf[0..n) (n <= CAP) at buf[0..k) in unspecified order,
// sets buf.tau_* to the k-th best and returns the new count.  All THREADS
// threads that meet at Bar (numbered 0 .. THREADS-1 by threadIdx.x) must call it
// with the same n and k.  n <= k is a no-op.
template <int THREADS, int CAP, class Bar = WholeBlock>
__device__ uint32_t compact_topk(CandidateBuffer<CAP> &buf, uint32_t n, uint32_t k) {
    static_assert(CAP % THREADS == 0, "buffer is a whole number of entries per thread");
    constexpr int PER = CAP / THREADS;
    if (n <= k) return n;
    const uint32_t tid = threadIdx.x;
    uint64_t key[PER];
    float score[PER];
    uint32_t id[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const uint32_t at = j * THREADS + tid;
        key[j] = 0;
        score[j] = 0.0f;
        id[j] = kPaddingId;
        if (at < n) {
            score[j] = buf.score[at];
            id[j] = buf.id[at];
            key[j] = select_key(score[j], id[j]);
        }
    }
    uint64_t prefix = 0;
    uint32_t need = k, bucket = 0;
    int shift = 56;
    for (int pass = 0; pass < 8; pass++) {
        if (tid < 256) buf.hist[tid] = 0;
        Bar::sync();
#pragma unroll
        for (int j = 0; j < PER; j++) {
            if (key[j] != 0 && (pass == 0 || (key[j] >> (shift + 8)) == prefix))
                atomicAdd(&buf.hist[(key[j] >> shift) & 255u], 1u);
        }
        Bar::sync();
        if (tid < 32) {
            // lane l owns digits 255-8l .. 248-8l, walked from the top
            uint32_t mine = 0;
#pragma unroll
            for (int b = 0; b < 8; b++) mine += buf.hist[255 - 8 * tid - b];
            uint32_t incl = mine;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t up = __shfl_up_sync(kFullMask, incl, d);
                if (tid >= (uint32_t)d) incl += up;
            }
            const unsigned reached = __ballot_sync(kFullMask, incl >= need);
            const int owner = __ffs(reached) - 1;  // need <= total, so some lane reaches it
            if ((int)tid == owner) {
                uint32_t above = incl - mine;
                for (int b = 0; b < 8; b++) {
                    const uint32_t digit = 255 - 8 * tid - b;
                    const uint32_t here = buf.hist[digit];
                    if (above + here >= need) {
                        buf.sel_digit = digit;
                        buf.sel_need = need - above;
                        buf.sel_bucket = here;
                        break;
                    }
                    above += here;
                }
            }
        }
        Bar::sync();
        prefix = (prefix << 8) | buf.sel_digit;
        need = buf.sel_need;
        bucket = buf.sel_bucket;
        if (bucket == need || shift == 0) break;
        shift -= 8;
    }
    if (tid == 0) {
        buf.out_count = 0;
        buf.eq_count = 0;
        buf.min_key = ~0ull;
    }
    Bar::sync();
#pragma unroll
    for (int j = 0; j < PER; j++) {
        if (key[j] == 0) continue;
        const uint64_t high = key[j] >> shift;
        bool take = high > prefix;
        if (!take && high == prefix) take = bucket == need || atomicAdd(&buf.eq_count, 1u) < need;
        if (take) {
            const uint32_t slot = atomicAdd(&buf.out_count, 1u);
            buf.score[slot] = score[j];
            buf.id[slot] = id[j];
            atomicMin(&buf.min_key, (unsigned long long)key[j]);
        }
    }
    Bar::sync();
    if (tid == 0) {
        buf.tau_score = key_to_float((uint32_t)(buf.min_key >> 32));
        buf.tau_id = ~(uint32_t)(buf.min_key & 0xffffffffull);
        buf.count = buf.out_count;
    }
    Bar::sync();
    return buf.out_count;
}

// buf[0..n), n <= 64, into fin.score/id in sampling order.  Entries that compare
// equal on (score, id) keep their buffer order.  All threads call; ends synced.
template <int CAP, class Bar = WholeBlock>
__device__ void sort_candidates(const CandidateBuffer<CAP> &buf, FinishBuffer &fin, uint32_t n) {
    const uint32_t tid = threadIdx.x;
    if (tid < n) {
        const float s = buf.score[tid];
        const uint32_t id = buf.id[tid];
        uint32_t rank = 0;
        for (uint32_t j = 0; j < n; j++) {
            const float t = buf.score[j];
            const uint32_t tj = buf.id[j];
            if (precedes(t, tj, s, id) || (t == s && tj == id && j < tid)) rank++;
        }
        fin.score[rank] = s;
        fin.id[rank] = id;
    }
    Bar::sync();
}

// The fused exchange of the vocabulary-sharded mode, device side (layout: fg_kernels.h).
struct PushTargets {
    unsigned char *window[16];
    uint32_t ranks, rank, half, pair_capacity, row_capacity;

    // where this rank's pair i of `row` lands in rank t's window
    __device__ __forceinline__ uint2 *pair(uint32_t t, uint32_t row, uint32_t k, uint32_t i) const {
        uint2 *pairs = reinterpret_cast<uint2 *>(window[t]);
        return pairs + ((size_t)half * ranks + rank) * pair_capacity + (size_t)row * k + i;
    }
    __device__ __forceinline__ uint32_t *arrived(uint32_t t, uint32_t row) const {
        uint32_t *counters = reinterpret_cast<uint32_t *>(
            window[t] + (size_t)2 * ranks * pair_capacity * sizeof(uint2));
        return counters + (size_t)half * row_capacity + row;
    }
};

struct SelectOutput {
    uint32_t *tokens;
    float *token_logits;
    uint32_t *row_status;
    unsigned long long *first_error;
    uint32_t *dbg_count;
    uint32_t *dbg_ids;
    float *dbg_scores;
    double *dbg_raw;
    double *dbg_tempered;
};

__device__ __forceinline__ void report_row(const SelectOutput &out, uint32_t row, uint32_t status,
                                           uint32_t token, float logit) {
    out.tokens[row] = token;
    out.token_logits[row] = logit;
    out.row_status[row] = status;
    if (status != kOk)
        atomicMin(out.first_error, ((unsigned long long)row << 8) | (unsigned long long)status);
}

// x[0] + x[1] + ... + x[n-1] added from the left, one rounding per addition, as the C loops
// of src/sampler.c:99-111 do; the loads of four terms go ahead of their additions.
__device__ __forceinline__ double ordered_sum(const double *x, uint32_t n) {
    double sum = 0.0;
    uint32_t i = 0;
    for (; i + 4 <= n; i += 4) {
        const double a = x[i], b = x[i + 1], c = x[i + 2], d = x[i + 3];
        sum += a;
        sum += b;
        sum += c;
        sum += d;
    }
    for (; i < n; i++) sum += x[i];
    return sum;
}

// The first i whose running sum x[0] + ... + x[i] (added from the left) satisfies
// `sum >= limit` (kStrictlyAbove: `limit < sum`); n when none does.
template <bool kStrictlyAbove>
__device__ __forceinline__ uint32_t ordered_reach(const double *x, uint32_t n, double limit) {
    double sum = 0.0;
    uint32_t i = 0;
    for (; i + 4 <= n; i += 4) {
        const double a = x[i], b = x[i + 1], c = x[i + 2], d = x[i + 3];
        const double s0 = sum + a, s1 = s0 + b, s2 = s1 + c, s3 = s2 + d;
        if (kStrictlyAbove ? limit < s0 : s0 >= limit) return i;
        if (kStrictlyAbove ? limit < s1 : s1 >= limit) return i + 1;
        if (kStrictlyAbove ? limit < s2 : s2 >= limit) return i + 2;
        if (kStrictlyAbove ? limit < s3 : s3 >= limit) return i + 3;
        sum = s3;
    }
    for (; i < n; i++) {
        sum += x[i];
        if (kStrictlyAbove ? limit < sum : sum >= limit) return i;
    }
    return n;
}

// Final step for one row; called by warp 0 of the CTA (all 32 lanes) with the
// candidates already in sampling order in fin.score/id[0..n), n = min(top_k,
// #finite).  Greedy rows never come here.
__device__ inline void finish_select(FinishBuffer &fin, uint32_t n, const SamplerConfig &cfg,
                              float uniform, uint32_t row, const SelectOutput &out) {
    const uint32_t lane = lane_id();
    if (n == 0) {  // src/sampler.c:97 "sampler received no finite candidates"
        if (lane == 0) {
            report_row(out, row, kErrFormat, kPaddingId, 0.0f);
            if (out.dbg_count) out.dbg_count[row] = 0;
        }
        return;
    }
    // Every lane has at most two candidates (n <= 64).  Their four exponentials -- the raw
    // and the tempered weight of each, the latter wanted only below the top-p cut, which is not
    // known yet -- do not wait for one another, so they are all started here.
    static_assert(kMaxK <= 64, "two candidates per lane");
    const double top_raw = (double)fin.score[0];
    const double temperature = (double)cfg.temperature;
    const double top_tempered = (double)fin.score[0] / temperature;
    const uint32_t i0 = lane, i1 = lane + 32;
    const double s0 = i0 < n ? (double)fin.score[i0] : top_raw;
    const double s1 = i1 < n ? (double)fin.score[i1] : top_raw;
    double raw0 = exp(s0 - top_raw), raw1 = exp(s1 - top_raw);
    const double tempered0 = exp(s0 / temperature - top_tempered);
    const double tempered1 = exp(s1 / temperature - top_tempered);
    if (i0 < n) fin.raw[i0] = raw0;
    if (i1 < n) fin.raw[i1] = raw1;
    __syncwarp();
    // the sums run left to right on one lane, as the C code's loops do; the divisions
    // are independent of one another and spread over the warp
    double raw_sum = 0.0;
    if (lane == 0) raw_sum = ordered_sum(fin.raw, n);
    raw_sum = __shfl_sync(kFullMask, raw_sum, 0);
    const bool raw_ok = raw_sum > 0.0 && !isinf(raw_sum) && !isnan(raw_sum);
    if (raw_ok) {
        raw0 = raw0 / raw_sum;
        raw1 = raw1 / raw_sum;
        if (i0 < n) fin.raw[i0] = raw0;
        if (i1 < n) fin.raw[i1] = raw1;
    }
    __syncwarp();
    if (lane == 0) {
        uint32_t cutoff = n;
        if (raw_ok) cutoff = min(n, ordered_reach<false>(fin.raw, n, (double)cfg.top_p) + 1u);
        fin.cutoff = cutoff;
        fin.status = raw_ok ? kOk : kErrFormat;  // "sampler raw softmax failed"
    }
    __syncwarp();
    if (fin.status != kOk) {
        if (lane == 0) {
            report_row(out, row, fin.status, kPaddingId, 0.0f);
            if (out.dbg_count) out.dbg_count[row] = 0;
        }
        return;
    }
    const uint32_t cutoff = fin.cutoff;
    if (i0 < n) fin.tempered[i0] = i0 < cutoff ? tempered0 : 0.0;
    if (i1 < n) fin.tempered[i1] = i1 < cutoff ? tempered1 : 0.0;
    __syncwarp();
    if (lane == 0) {
        const double weight_sum = ordered_sum(fin.tempered, cutoff);
        if (!(weight_sum > 0.0) || isinf(weight_sum) || isnan(weight_sum)) {
            fin.status = kErrFormat;  // "sampler temperature softmax failed"
        } else {
            float u = uniform;
            if (is_nonfinite(u) || u < 0.0f) u = 0.0f;
            if (u >= 1.0f) u = __uint_as_float(0x3f7fffffu);  // nextafterf(1, 0)
            const double draw = (double)u * weight_sum;
            fin.picked = min(cutoff - 1u, ordered_reach<true>(fin.tempered, cutoff, draw));
            if (out.dbg_tempered)
                for (uint32_t i = 0; i < cutoff; i++) fin.tempered[i] = fin.tempered[i] / weight_sum;
        }
    }
    __syncwarp();
    if (fin.status != kOk) {
        if (lane == 0) {
            report_row(out, row, fin.status, kPaddingId, 0.0f);
            if (out.dbg_count) out.dbg_count[row] = 0;
        }
        return;
    }
    if (lane == 0) report_row(out, row, kOk, fin.id[fin.picked], fin.score[fin.picked]);
    if (out.dbg_count) {
        if (lane == 0) out.dbg_count[row] = n;
        for (uint32_t i = lane; i < kMaxK; i += 32) {
            const size_t at = (size_t)row * kMaxK + i;
            const bool live = i < n;
            if (out.dbg_ids) out.dbg_ids[at] = live ? fin.id[i] : kPaddingId;
            if (out.dbg_scores) out.dbg_scores[at] = live ? fin.score[i] : 0.0f;
            if (out.dbg_raw) out.dbg_raw[at] = live ? fin.raw[i] : 0.0;
            if (out.dbg_tempered) out.dbg_tempered[at] = live ? fin.tempered[i] : 0.0;
        }
    }
}

}  // namespace fgk
