// Sampling without a top-k cut: top-p over the whole vocabulary, then temperature and
// inverse CDF — the reference's select step (src/sampler.c:97-121) with limit = every
// finite logit.  The reference caps candidates at 64; this is the documented
// generalisation for rows whose nucleus spans tens of thousands of tokens.
//
// The vocabulary is never sorted.  A persistent CTA per SM streams a row from HBM once
// (penalties applied on the way) into its own scratch row, which stays in L2, and then
// narrows down two positions of the (value descending, id ascending) order by MSB-first
// radix descent over the 32-bit monotone value key, 12 + 12 + 8 bits: first the element
// where the cumulative raw-softmax mass reaches top_p, then the element the draw lands
// on under the tempered weights.  Each level is one pass over the scratch row that
// builds a bucketed histogram of counts and masses in shared memory, followed by a
// block-wide prefix sum from the top bucket down.  Equal values are resolved on the
// id with the same descent (counts only).
//
// Masses are exp(s - max) in fp64, accumulated as 2^-40 fixed point in 64-bit
// integers: integer addition is associative, so the result does not depend on the
// order threads arrive in, and the 1e-12 grid is far below one element's weight.
// The reference adds doubles left to right; the two agree unless the top-p bound or
// the draw falls within ~1e-11 (relative) of an edge of the CDF.
#include "fg_block_select.cuh"
#include "fg_kernels.h"

namespace fgk {


constexpr int kNucleusThreads = 1024;
constexpr int kBuckets = 4096;
// per bucket: two masses (raw and tempered weights) and a count
constexpr size_t kNucleusHistogramBytes = kBuckets * (2 * sizeof(unsigned long long) + sizeof(uint32_t));

struct NucleusParams {
    const void *logits;
    uint32_t dtype;
    uint32_t rows, vocab;
    uint64_t row_stride;
    const SamplerConfig *configs;
    SamplerConfig config0;
    uint32_t config_count;
    const float *uniforms;
    float *scratch;            // gridDim.x rows of scratch_stride floats
    uint64_t scratch_stride;
    // history structures built by history_build_kernel, one per (row, split)
    const uint32_t *history_global;
    uint64_t history_stride_words;
    const void *history_meta;
    uint32_t splits, split_len, bitmap_words, count_capacity, dense_wide;
    SelectOutput out;
};

struct NucleusShared {
    unsigned long long *mass;         // kBuckets entries, dynamic shared memory: the masses a crossing search walks
    unsigned long long *other_mass;   // kBuckets entries: the tempered masses while `mass` holds the raw ones
    uint32_t *count;                  // kBuckets entries
    double table[64];                 // 2^(j/64)
    unsigned long long scan_mass[32];
    uint32_t scan_count[32];
    unsigned long long total_mass;
    float reduce_max[32];
    uint32_t reduce_count[32];
    // result of a scan
    uint32_t hit_bucket;
    unsigned long long hit_mass_before;
    uint32_t hit_count_before;
    uint32_t hit_found;
};

// exp(x) * 2^40 for x <= 0 as a 64-bit integer (round to nearest): argument reduction
// to n/64 * ln2 + r, |r| <= ln2/128, a 64-entry table of 2^(j/64) and a degree-5
// polynomial (truncation 4e-17).  Below e^-70 the weight is under the fixed-point grid.
__device__ __forceinline__ unsigned long long exp_fixed(double x, const double *table) {
    if (!(x > -70.0)) return 0ull;
    const double scaled = x * 92.33248261689366;                  // 64 / ln 2
    const double shifted = scaled + 6755399441055744.0;           // 1.5 * 2^52: rounds to nearest
    const int n = __double2loint(shifted);
    const double nd = shifted - 6755399441055744.0;
    double r = fma(nd, -1.0830424696249145e-02, x);               // ln2/64, high part
    r = fma(nd, -3.623510646634843e-19, r);                       // low part
    double p = fma(r, 8.3333333333333332e-03, 4.1666666666666664e-02);
    p = fma(p, r, 1.6666666666666666e-01);
    p = fma(p, r, 0.5);
    p = fma(p, r, 1.0);
    p = fma(p, r, 1.0);                                           // 1 + r + r^2/2 + ... + r^5/120
    const int j = n & 63, k = n >> 6;                             // floor division for negative n
    const double scale = __longlong_as_double((long long)(k + 40 + 1023) << 52);
    return __double2ull_rn(table[j] * p * scale);
}

// Block-wide: walk the buckets from the top; find the first bucket b where
// before + mass(>= b) reaches `target` (strict: exceeds it).  All threads call.
__device__ void find_crossing(NucleusShared &sh, uint32_t buckets, unsigned long long before,
                              unsigned long long target, bool strict) {
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t per = (buckets + kNucleusThreads - 1) / kNucleusThreads;
    // thread t owns buckets top-down: indices buckets-1 - (t*per + i)
    unsigned long long mine_mass = 0;
    uint32_t mine_count = 0;
    for (uint32_t i = 0; i < per; i++) {
        const uint32_t at = tid * per + i;
        if (at < buckets) {
            mine_mass += sh.mass[buckets - 1 - at];
            mine_count += sh.count[buckets - 1 - at];
        }
    }
    unsigned long long incl_mass = mine_mass;
    uint32_t incl_count = mine_count;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long up_mass = __shfl_up_sync(kFullMask, incl_mass, d);
        const uint32_t up_count = __shfl_up_sync(kFullMask, incl_count, d);
        if (lane >= (uint32_t)d) {
            incl_mass += up_mass;
            incl_count += up_count;
        }
    }
    if (lane == 31) {
        sh.scan_mass[warp] = incl_mass;
        sh.scan_count[warp] = incl_count;
    }
    if (tid == 0) sh.hit_found = 0;
    __syncthreads();
    unsigned long long prior_mass = before + incl_mass - mine_mass;
    uint32_t prior_count = incl_count - mine_count;
    for (uint32_t w = 0; w < warp; w++) {
        prior_mass += sh.scan_mass[w];
        prior_count += sh.scan_count[w];
    }
    const unsigned long long after = prior_mass + mine_mass;
    const bool was = strict ? prior_mass > target : prior_mass >= target;
    const bool now = strict ? after > target : after >= target;
    if (!was && now) {  // exactly one thread
        for (uint32_t i = 0; i < per; i++) {
            const uint32_t at = tid * per + i;
            if (at >= buckets) break;
            const uint32_t b = buckets - 1 - at;
            const unsigned long long next = prior_mass + sh.mass[b];
            if (strict ? next > target : next >= target) {
                sh.hit_bucket = b;
                sh.hit_mass_before = prior_mass;
                sh.hit_count_before = prior_count;
                sh.hit_found = 1;
                break;
            }
            prior_mass = next;
            prior_count += sh.count[b];
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void clear_histogram(NucleusShared &sh, uint32_t buckets) {
    for (uint32_t b = threadIdx.x; b < buckets; b += kNucleusThreads) {
        sh.mass[b] = 0;
        sh.count[b] = 0;
    }
    __syncthreads();
}

// Walks the scratch row: visit(value, index) for every element.  Eight values per thread
// are in flight (two 128-bit loads) before the first is used: with one scalar load per
// trip a pass over the row was a chain of L2 latencies.  Rows start 16-byte aligned.
template <class Visit>
__device__ __forceinline__ void walk_row(const float *values, uint32_t vocab, Visit visit) {
    const uint32_t tid = threadIdx.x;
    const float4 *wide = reinterpret_cast<const float4 *>(values);
    const uint32_t quads = vocab / 4u;
    uint32_t q = tid;
    for (; q + kNucleusThreads < quads; q += 2 * kNucleusThreads) {
        const float4 a = wide[q], b = wide[q + kNucleusThreads];
        const uint32_t ia = q * 4u, ib = (q + kNucleusThreads) * 4u;
        visit(a.x, ia);
        visit(a.y, ia + 1u);
        visit(a.z, ia + 2u);
        visit(a.w, ia + 3u);
        visit(b.x, ib);
        visit(b.y, ib + 1u);
        visit(b.z, ib + 2u);
        visit(b.w, ib + 3u);
    }
    if (q < quads) {
        const float4 a = wide[q];
        const uint32_t ia = q * 4u;
        visit(a.x, ia);
        visit(a.y, ia + 1u);
        visit(a.z, ia + 2u);
        visit(a.w, ia + 3u);
    }
    const uint32_t rest = quads * 4u + tid;
    if (rest < vocab) visit(values[rest], rest);
}

// Which elements of the scratch row take part in a descent.
struct Nucleus {
    uint32_t key;     // value key of the last element inside
    uint32_t id;      // ... and its id (ties on the key are ordered by id)
    bool everything;  // no cut yet: every finite value takes part
    __device__ __forceinline__ bool holds(uint32_t k, uint32_t i) const {
        return everything || k > key || (k == key && i <= id);
    }
};

// One radix descent over the scratch row.  Weights are exp(value * inv_t - top * inv_t);
// finds the first element of the (key descending, id ascending) order, restricted to
// `inside`, at which the cumulative weight reaches `target` (strict: exceeds it).
// When even the total does not, the last element inside is returned.  Outputs the
// element's key and id, the cumulative weight up to and including it and its rank.
// All threads of the CTA call it.
__device__ void descend(NucleusShared &sh, const float *values, uint32_t vocab, double inv_t,
                        double top, const Nucleus inside, unsigned long long target, bool strict,
                        uint32_t *out_key, uint32_t *out_id, unsigned long long *out_mass,
                        uint32_t *out_rank) {
    const uint32_t tid = threadIdx.x;
    const double top_scaled = top * inv_t;
    uint32_t prefix = 0;  // key bits fixed so far
    unsigned long long before = 0;
    uint32_t rank_before = 0;
    unsigned long long weight_of_key = 0;
    uint32_t same_key = 0;
    bool clipped = false;  // target beyond the total: steer to the last element inside
    const int shifts[3] = {20, 8, 0};
    const uint32_t widths[3] = {4096, 4096, 256};
    for (int level = 0; level < 3; level++) {
        const int shift = shifts[level];
        const uint32_t buckets = widths[level];
        clear_histogram(sh, buckets);
        for (uint32_t i = tid; i < vocab; i += kNucleusThreads) {
            const float v = values[i];
            if (is_nonfinite(v)) continue;
            const uint32_t key = float_key(v);
            if (level > 0 && (key >> (shift + (level == 1 ? 12 : 8))) != prefix) continue;
            if (!inside.holds(key, i)) continue;
            const unsigned long long w = exp_fixed((double)v * inv_t - top_scaled, sh.table);
            const uint32_t b = (key >> shift) & (buckets - 1);
            atomicAdd(&sh.mass[b], w);
            atomicAdd(&sh.count[b], 1u);
        }
        __syncthreads();
        if (!clipped) {
            find_crossing(sh, buckets, before, target, strict);
            // the total stays below the target (rounding of the draw, or top_p = 1): the
            // answer is the last element inside, i.e. the lowest non-empty bucket from here on
            if (!sh.hit_found) clipped = true;
            __syncthreads();
        }
        if (clipped) {
            // lowest non-empty bucket: scan by thread 0 (rare path)
            if (tid == 0) {
                unsigned long long m = before;
                uint32_t c = 0, last = 0;
                bool any = false;
                for (uint32_t at = 0; at < buckets; at++) {
                    const uint32_t b = buckets - 1 - at;
                    if (sh.count[b]) {
                        if (any) {
                            m += sh.mass[last];
                            c += sh.count[last];
                        }
                        last = b;
                        any = true;
                    }
                }
                sh.hit_bucket = last;
                sh.hit_mass_before = m;
                sh.hit_count_before = c;
                sh.hit_found = any ? 1u : 0u;
            }
            __syncthreads();
        }
        const uint32_t b = sh.hit_bucket;
        before = sh.hit_mass_before;
        rank_before += sh.hit_count_before;
        weight_of_key = sh.mass[b];
        same_key = sh.count[b];
        prefix = (prefix << (level == 2 ? 8 : 12)) | b;
        __syncthreads();
    }
    // `prefix` is now a full key; same_key elements share it, each weighing the same
    const uint32_t key = prefix;
    const unsigned long long each = same_key ? weight_of_key / same_key : 0;
    uint32_t need = same_key;  // how many of the equal-valued elements it takes, 1-based
    if (!clipped && each > 0) {
        // smallest j with before + j*each reaching the target
        const unsigned long long gap = target > before ? target - before : 0;
        unsigned long long j = strict ? gap / each + 1 : (gap + each - 1) / each;
        if (j < 1) j = 1;
        if (j < need) need = (uint32_t)j;
    }
    // the need-th smallest id among the elements with this key that are inside
    uint32_t id_prefix = 0, id_rank = need;
    if (same_key > 1) {
        for (int level = 0; level < 3; level++) {
            const int shift = shifts[level];
            const uint32_t buckets = widths[level];
            clear_histogram(sh, buckets);
            for (uint32_t i = tid; i < vocab; i += kNucleusThreads) {
                const float v = values[i];
                if (is_nonfinite(v) || float_key(v) != key || !inside.holds(key, i)) continue;
                if (level > 0 && (i >> (shift + (level == 1 ? 12 : 8))) != id_prefix) continue;
                // ascending ids: store reversed so the top-down walk visits small ids first
                atomicAdd(&sh.count[buckets - 1 - ((i >> shift) & (buckets - 1))], 1u);
                atomicAdd(&sh.mass[buckets - 1 - ((i >> shift) & (buckets - 1))], 1ull);
            }
            __syncthreads();
            find_crossing(sh, buckets, 0, id_rank, false);
            const uint32_t b = sh.hit_bucket;
            id_rank -= (uint32_t)sh.hit_mass_before;
            id_prefix = (id_prefix << (level == 2 ? 8 : 12)) | (buckets - 1 - b);
            __syncthreads();
        }
    } else {
        // the single element with this key: find its id
        if (tid == 0) sh.hit_bucket = kPaddingId;
        __syncthreads();
        for (uint32_t i = tid; i < vocab; i += kNucleusThreads) {
            const float v = values[i];
            if (!is_nonfinite(v) && float_key(v) == key && inside.holds(key, i)) sh.hit_bucket = i;
        }
        __syncthreads();
        id_prefix = sh.hit_bucket;
        __syncthreads();
    }
    *out_key = key;
    *out_id = id_prefix;
    *out_mass = before + (unsigned long long)need * each;
    *out_rank = rank_before + need;
}

// ---- the usual case: value buckets, then an exact look inside one bucket ----
//
// Buckets of equal width in the value itself, 1/256 wide and counted down from the
// row's maximum (bucket 0 holds the largest values; everything 16 below the maximum,
// where weights are below 2^-23, shares the last bucket).  Unlike the top bits of the
// float key this spreads real logit rows over hundreds of buckets, which keeps the
// shared-memory atomics apart.  One pass fills the histogram (this is where exp() is
// paid), a prefix sum finds the bucket in which the target is reached, a second pass
// gathers that bucket's members — a few hundred — and they are ordered exactly.

constexpr uint32_t kListCap = 2048;

struct NucleusList {
    float value[kListCap];
    uint32_t id[kListCap];
    float sorted_value[kListCap];
    uint32_t sorted_id[kListCap];
    unsigned long long weight[kListCap];  // of the sorted entries, then their running sum
    uint32_t count;
};

// (fp32 arithmetic: the bucket edges need not be exact, only the same in every pass and
// monotone in v, which one rounded subtraction and an exact scaling are; the fp64 pipe is
// what the histogram passes are short of)
__device__ __forceinline__ uint32_t value_bucket(float v, float top) {
    const float below = __fmul_rn(__fsub_rn(top, v), 256.0f);  // >= 0
    return below >= (float)(kBuckets - 1) ? (uint32_t)(kBuckets - 1) : (uint32_t)below;
}

// Like find_crossing but walking the buckets upwards from 0; also leaves the sum of
// all masses in sh.total_mass.  target_of(total) is evaluated once the total is known.
// All threads call.  sh.hit_found == 0 means the total never reaches the target.
template <typename TargetOf>
__device__ unsigned long long find_crossing_up(NucleusShared &sh, TargetOf target_of, bool strict) {
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    constexpr uint32_t per = kBuckets / kNucleusThreads;
    unsigned long long mine_mass = 0;
    uint32_t mine_count = 0;
#pragma unroll
    for (uint32_t i = 0; i < per; i++) {
        mine_mass += sh.mass[tid * per + i];
        mine_count += sh.count[tid * per + i];
    }
    unsigned long long incl_mass = mine_mass;
    uint32_t incl_count = mine_count;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long up_mass = __shfl_up_sync(kFullMask, incl_mass, d);
        const uint32_t up_count = __shfl_up_sync(kFullMask, incl_count, d);
        if (lane >= (uint32_t)d) {
            incl_mass += up_mass;
            incl_count += up_count;
        }
    }
    if (lane == 31) {
        sh.scan_mass[warp] = incl_mass;
        sh.scan_count[warp] = incl_count;
    }
    if (tid == 0) sh.hit_found = 0;
    __syncthreads();
    unsigned long long prior_mass = incl_mass - mine_mass, total = 0;
    uint32_t prior_count = incl_count - mine_count;
    for (uint32_t w = 0; w < kNucleusThreads / 32; w++) {
        if (w < warp) {
            prior_mass += sh.scan_mass[w];
            prior_count += sh.scan_count[w];
        }
        total += sh.scan_mass[w];
    }
    const unsigned long long target = target_of(total);
    const unsigned long long after = prior_mass + mine_mass;
    const bool was = strict ? prior_mass > target : prior_mass >= target;
    const bool now = strict ? after > target : after >= target;
    if (!was && now) {  // exactly one thread
#pragma unroll
        for (uint32_t i = 0; i < per; i++) {
            const uint32_t b = tid * per + i;
            const unsigned long long next = prior_mass + sh.mass[b];
            if (strict ? next > target : next >= target) {
                sh.hit_bucket = b;
                sh.hit_mass_before = prior_mass;
                sh.hit_count_before = prior_count;
                sh.hit_found = 1;
                break;
            }
            prior_mass = next;
            prior_count += sh.count[b];
        }
    }
    if (tid == 0) sh.total_mass = total;
    __syncthreads();
    return target;
}

struct Position {
    uint32_t key, id;            // the element found
    unsigned long long mass;     // cumulative weight up to and including it
    uint32_t rank;               // its 1-based position in the order
    unsigned long long total;    // weight of everything inside
    bool ok;                     // false: fall back to the generic descent
};

// One phase: among the elements `inside`, weights exp((v - top) * inv_t), find the
// first element of the (value descending, id ascending) order at which the running
// weight reaches target_of(total) (strict: exceeds it); if it never does, the last
// element inside.  All threads call.
// The members of one value bucket (restricted to `inside`), ordered exactly, and among them the
// first at which the running weight -- `before` plus the weights exp((v - top) * inv_t) of the
// members so far -- reaches `target` (strict: exceeds it); the last member when none does or
// when `clipped`.  ok = false: the bucket is empty or holds more than the list takes.  With
// `also_inv_t` != 0 the weights exp((v - top) * also_inv_t) of the members up to and including
// the one found are summed into *also_sum.  All threads call.
__device__ Position resolve_bucket(NucleusShared &sh, NucleusList &list, const float *values, uint32_t vocab,
                                   double inv_t, float top, const Nucleus inside, uint32_t bucket,
                                   uint32_t members, unsigned long long before, uint32_t rank_before,
                                   unsigned long long target, bool strict, bool clipped, double also_inv_t,
                                   unsigned long long *also_sum) {
    const uint32_t tid = threadIdx.x;
    Position found;
    found.ok = false;
    found.total = 0;
    if (members == 0 || members > kListCap) return found;  // crowded bucket (heavy ties): generic path
    if (tid == 0) list.count = 0;
    __syncthreads();
    walk_row(values, vocab, [&](float v, uint32_t i) {
        // (a NaN or an infinity has no bucket: the conversion below sends them to the last one or
        // to bucket 0, so they are looked at, and dropped, only there)
        if (value_bucket(v, top) != bucket) return;
        if (is_nonfinite(v) || !inside.holds(float_key(v), i)) return;
        const uint32_t slot = atomicAdd(&list.count, 1u);
        if (slot < kListCap) {
            list.value[slot] = v;
            list.id[slot] = i;
        }
    });
    __syncthreads();
    members = min(list.count, kListCap);  // (inside may hold fewer of the bucket than the histogram counted)
    if (members == 0) return found;
    // order them: rank by counting, (value descending, id ascending); -0.0 and +0.0 tie
    for (uint32_t a = tid; a < members; a += kNucleusThreads) {
        const float v = list.value[a];
        const uint32_t id = list.id[a];
        uint32_t rank = 0;
        for (uint32_t b = 0; b < members; b++) rank += precedes(list.value[b], list.id[b], v, id) ? 1u : 0u;
        list.sorted_value[rank] = v;
        list.sorted_id[rank] = id;
        list.weight[rank] = exp_fixed(((double)v - (double)top) * inv_t, sh.table);
    }
    __syncthreads();
    // running sum over at most 2048 entries: two per thread, then the usual scan
    {
        const uint32_t lane = tid & 31u, warp = tid >> 5;
        const uint32_t a0 = 2 * tid, a1 = 2 * tid + 1;
        const unsigned long long w0 = a0 < members ? list.weight[a0] : 0;
        const unsigned long long w1 = a1 < members ? list.weight[a1] : 0;
        unsigned long long incl = w0 + w1;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned long long up = __shfl_up_sync(kFullMask, incl, d);
            if (lane >= (uint32_t)d) incl += up;
        }
        if (lane == 31) sh.scan_mass[warp] = incl;
        __syncthreads();
        unsigned long long prior = incl - (w0 + w1);
        for (uint32_t w = 0; w < warp; w++) prior += sh.scan_mass[w];
        if (a0 < members) list.weight[a0] = before + prior + w0;
        if (a1 < members) list.weight[a1] = before + prior + w0 + w1;
        if (tid == 0) sh.hit_bucket = kPaddingId;
        __syncthreads();
    }
    // the first entry whose running sum reaches the target (exactly one thread sees the step)
    for (uint32_t a = tid; a < members; a += kNucleusThreads) {
        const unsigned long long here = list.weight[a];
        const unsigned long long prev = a ? list.weight[a - 1] : before;
        const bool was = strict ? prev > target : prev >= target;
        const bool now = strict ? here > target : here >= target;
        if (!clipped && !was && now) sh.hit_bucket = a;
    }
    __syncthreads();
    uint32_t at = sh.hit_bucket;
    if (clipped || at == kPaddingId) at = members - 1;
    found.key = float_key(list.sorted_value[at]);
    found.id = list.sorted_id[at];
    found.mass = list.weight[at];
    found.rank = rank_before + at + 1;
    found.ok = true;
    __syncthreads();
    if (also_sum != nullptr) {
        // the other weight of the members up to the one found (order does not matter: integers)
        unsigned long long part = 0;
        for (uint32_t a = tid; a <= at; a += kNucleusThreads)
            part += exp_fixed(((double)list.sorted_value[a] - (double)top) * also_inv_t, sh.table);
        const uint32_t lane = tid & 31u, warp = tid >> 5;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(kFullMask, part, d);
        if (lane == 0) sh.scan_mass[warp] = part;
        __syncthreads();
        unsigned long long sum = 0;
        for (int w = 0; w < kNucleusThreads / 32; w++) sum += sh.scan_mass[w];
        *also_sum = sum;
        __syncthreads();
    }
    return found;
}

// After a crossing search: the bucket it stopped in, or -- when the total never reaches the
// target (top_p = 1, a draw rounded up to the total) -- the last non-empty bucket.  Returns
// whether it was clipped; all threads call.
__device__ bool settle_crossing(NucleusShared &sh) {
    if (sh.hit_found) return false;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long m = 0;
        uint32_t c = 0, last = 0;
        bool any = false;
        for (uint32_t b = 0; b < kBuckets; b++) {
            if (sh.count[b]) {
                if (any) {
                    m += sh.mass[last];
                    c += sh.count[last];
                }
                last = b;
                any = true;
            }
        }
        sh.hit_bucket = last;
        sh.hit_mass_before = m;
        sh.hit_count_before = c;
    }
    __syncthreads();
    return true;
}

// One phase: among the elements `inside`, weights exp((v - top) * inv_t), find the
// first element of the (value descending, id ascending) order at which the running
// weight reaches target_of(total) (strict: exceeds it); if it never does, the last
// element inside.  All threads call.
template <typename TargetOf>
__device__ Position locate(NucleusShared &sh, NucleusList &list, const float *values, uint32_t vocab,
                           double inv_t, float top, const Nucleus inside, TargetOf target_of,
                           bool strict) {
    clear_histogram(sh, kBuckets);
    walk_row(values, vocab, [&](float v, uint32_t i) {
        if (is_nonfinite(v) || !inside.holds(float_key(v), i)) return;
        const unsigned long long w = exp_fixed(((double)v - (double)top) * inv_t, sh.table);
        const uint32_t b = value_bucket(v, top);
        atomicAdd(&sh.mass[b], w);
        atomicAdd(&sh.count[b], 1u);
    });
    __syncthreads();
    const unsigned long long target = find_crossing_up(sh, target_of, strict);
    const unsigned long long total = sh.total_mass;
    const bool clipped = settle_crossing(sh);
    const uint32_t bucket = sh.hit_bucket;
    const unsigned long long before = sh.hit_mass_before;
    const uint32_t rank_before = sh.hit_count_before;
    const uint32_t members = sh.count[bucket];
    __syncthreads();
    Position found = resolve_bucket(sh, list, values, vocab, inv_t, top, inside, bucket, members, before,
                                    rank_before, target, strict, clipped, 0.0, nullptr);
    found.total = total;
    return found;
}

// exp(x) for |x| <= 1/64 by its series to the sixth power (the next term is below 1e-16).
__device__ __forceinline__ double exp_small(double x) {
    double p = fma(x, 1.0 / 720.0, 1.0 / 120.0);
    p = fma(p, x, 1.0 / 24.0);
    p = fma(p, x, 1.0 / 6.0);
    p = fma(p, x, 0.5);
    p = fma(p, x, 1.0);
    return fma(p, x, 1.0);
}

// One pass over the row for both phases: per value bucket the count, the raw weights
// exp(v - top) and the tempered weights exp((v - top) * inv_t) of its members.  A member's
// weight is taken relative to the bucket's upper edge -- an argument of at most 1/256 (times
// inv_t), a short series instead of a full exp() -- as 2^-32 fixed point, and summed in two
// 16-bit halves with 32-bit shared-memory adds (a bucket of up to 65,535 members cannot
// overflow them; integer sums do not depend on the order of arrival).  The rounding of one
// member is 2^-33 of a member's weight; a whole row's worth stays below 1e-4 of one member's
// weight, three orders of magnitude under the smallest distance to an edge of the cumulative
// distribution that decides a row.  Afterwards every bucket's sums are scaled by the weight of
// its edge, exp(-b/256) (and its power inv_t), into the row's 2^-40 fixed point.  The last
// bucket (everything 16 below the maximum) and rows with inv_t > 4 take the full exp().
// Returns false when a bucket holds too many members for its sums (heavy ties).
__device__ bool fill_both(NucleusShared &sh, const float *values, uint32_t vocab, double inv_t, float top) {
    const uint32_t tid = threadIdx.x;
    // the two mass arrays, seen as four arrays of 32-bit sums
    uint32_t *raw_low = reinterpret_cast<uint32_t *>(sh.mass), *raw_high = raw_low + kBuckets;
    uint32_t *tempered_low = reinterpret_cast<uint32_t *>(sh.other_mass), *tempered_high = tempered_low + kBuckets;
    for (uint32_t b = tid; b < kBuckets; b += kNucleusThreads) {
        sh.mass[b] = 0;
        sh.other_mass[b] = 0;
        sh.count[b] = 0;
    }
    if (tid == 0) sh.hit_found = 0;
    __syncthreads();
    const bool series = inv_t <= 4.0;  // (1/256) * inv_t <= 1/64
    const double top_d = (double)top;
    constexpr double kOne = 4294967296.0;  // 2^32
    walk_row(values, vocab, [&](float v, uint32_t i) {
        if (is_nonfinite(v)) return;
        const uint32_t b = value_bucket(v, top);
        // v - (top - b/256): at most a bucket's width (and a rounding of the bucket's number) from 0
        const double x = ((double)v - top_d) + (double)b * (1.0 / 256.0);
        // (a weight of 1 and a rounding above it saturate at 2^32 - 1: half a unit, like any rounding)
        uint32_t r, t;
        if (series && b != (uint32_t)(kBuckets - 1)) {
            r = (uint32_t)min(__double2ull_rn(exp_small(x) * kOne), 0xffffffffull);
            t = (uint32_t)min(__double2ull_rn(exp_small(x * inv_t) * kOne), 0xffffffffull);
        } else {
            r = (uint32_t)min((exp_fixed(x, sh.table) + 128ull) >> 8, 0xffffffffull);
            t = (uint32_t)min((exp_fixed(x * inv_t, sh.table) + 128ull) >> 8, 0xffffffffull);
        }
        atomicAdd(&raw_low[b], r & 0xffffu);
        atomicAdd(&raw_high[b], r >> 16);
        atomicAdd(&tempered_low[b], t & 0xffffu);
        atomicAdd(&tempered_high[b], t >> 16);
        atomicAdd(&sh.count[b], 1u);
    });
    __syncthreads();
    // the halves back together (every thread reads the sums of its buckets before any of them is
    // overwritten: the 64-bit masses take the place of the 32-bit sums), scaled by the edge's
    // weight into the row's fixed point: 2^-32 -> 2^-40 is a factor 256
    constexpr int kOwn = kBuckets / kNucleusThreads;
    unsigned long long raw[kOwn], tempered[kOwn];
#pragma unroll
    for (int j = 0; j < kOwn; j++) {
        const uint32_t b = j * kNucleusThreads + tid;
        raw[j] = ((unsigned long long)raw_high[b] << 16) + raw_low[b];
        tempered[j] = ((unsigned long long)tempered_high[b] << 16) + tempered_low[b];
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kOwn; j++) {
        const uint32_t b = j * kNucleusThreads + tid;
        const uint32_t members = sh.count[b];
        if (members > 65535u) sh.hit_found = 1;  // (reused as "a bucket overflowed")
        const double edge = -(double)b * (1.0 / 256.0);
        sh.mass[b] = members ? __double2ull_rn((double)raw[j] * 256.0 * exp(edge)) : 0ull;
        sh.other_mass[b] = members ? __double2ull_rn((double)tempered[j] * 256.0 * exp(edge * inv_t)) : 0ull;
    }
    __syncthreads();
    const bool fits = sh.hit_found == 0;
    __syncthreads();
    return fits;
}

template <typename T>
__global__ void __launch_bounds__(kNucleusThreads, 1) nucleus_select_kernel(const NucleusParams p) {
    extern __shared__ __align__(16) unsigned char histogram_memory[];
    __shared__ NucleusShared sh;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    if (tid == 0) {
        sh.mass = reinterpret_cast<unsigned long long *>(histogram_memory);
        sh.other_mass = sh.mass + kBuckets;
        sh.count = reinterpret_cast<uint32_t *>(histogram_memory + 2 * kBuckets * sizeof(unsigned long long));
    }
    if (tid < 64) sh.table[tid] = exp2((double)tid / 64.0);
    float *values = p.scratch + (size_t)blockIdx.x * p.scratch_stride;
    NucleusList &list = *reinterpret_cast<NucleusList *>(histogram_memory + kNucleusHistogramBytes);
    __syncthreads();

    for (uint32_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const SamplerConfig cfg = p.config_count > 1 ? p.configs[row] : p.config0;
        if (cfg.temperature == 0.0f || cfg.top_k != 0) continue;  // the streaming kernel's rows

        // ---- pass 1: HBM -> penalised fp32 row in scratch, maximum on the way ----
        const T *columns = static_cast<const T *>(p.logits) + (size_t)row * p.row_stride;
        const Repetition repetition = make_repetition(cfg.repetition_penalty);
        const float flat_offset = penalty_offset(1u, cfg.presence_penalty, cfg.frequency_penalty);
        float best = __uint_as_float(0xff800000u);
        uint32_t finite = 0, bad_history = 0;
        for (uint32_t split = 0; split < p.splits; split++) {
            const uint32_t lo = split * p.split_len;
            const uint32_t n = min(p.split_len, p.vocab - lo);
            uint32_t flags = 0;
            HistoryView history = make_history_view(nullptr, 0, 0, false);
            if (p.history_meta != nullptr) {
                const size_t unit = (size_t)row * p.splits + split;
                const uint2 meta = reinterpret_cast<const uint2 *>(p.history_meta)[unit];
                flags = meta.x;
                if (meta.y) bad_history = meta.y;
                history = make_history_view(
                    const_cast<uint32_t *>(p.history_global) + unit * p.history_stride_words,
                    p.bitmap_words, p.count_capacity, p.dense_wide != 0);
            }
            // one column: penalise if seen, store, fold into the maximum
            auto take = [&](float v, uint32_t c, uint32_t word) {
                if ((word >> (c & 31u)) & 1u) {
                    float offset = flat_offset;
                    if (flags & 2u)
                        offset = penalty_offset(history.count(c >> 5, word, c & 31u),
                                                cfg.presence_penalty, cfg.frequency_penalty);
                    v = penalise_with_offset(v, offset, repetition);
                }
                if (!is_nonfinite(v)) {
                    best = fmaxf(best, v);
                    finite++;
                }
                return v;
            };
            const T *source = columns + lo;
            uint32_t done = 0;
            if ((reinterpret_cast<uintptr_t>(source) & 15u) == 0 && (lo & 3u) == 0) {
                // four columns per thread and trip (one vector load, one bitmap word, one
                // 128-bit store), two trips in flight
                const uint32_t quads = n / 4u;
                float4 *out = reinterpret_cast<float4 *>(values + lo);
                auto load4 = [&](uint32_t q) {
                    float4 v;
                    if (sizeof(T) == 2) {
                        const uint2 raw = reinterpret_cast<const uint2 *>(source)[q];
                        v = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                        __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
                    } else {
                        v = reinterpret_cast<const float4 *>(source)[q];
                    }
                    return v;
                };
                // What the history says about the four columns of a quad (they share a bitmap word).
                // The loads go out in two waves that wait for nothing but each other -- the word and
                // the running count of ids before it, then the four occurrence counts -- instead of
                // a chain of two loads per seen column.
                struct Seen {
                    uint32_t nibble;    // bit j: column 4q + j has been seen
                    uint32_t times[4];  // how often (with a frequency penalty)
                };
                auto look_up = [&](uint32_t q) {
                    Seen seen;
                    seen.nibble = 0;
                    seen.times[0] = seen.times[1] = seen.times[2] = seen.times[3] = 1u;
                    if (!(flags & 1u)) return seen;
                    const uint32_t c = q * 4u;
                    const uint32_t word = history.bitmap[c >> 5];
                    seen.nibble = (word >> (c & 31u)) & 15u;
                    if ((flags & 2u) && seen.nibble != 0) {
                        const uint32_t before = history.running[c >> 5] + __popc(word & ((1u << (c & 31u)) - 1u));
                        uint32_t at[4];
                        at[0] = before;
                        at[1] = at[0] + (seen.nibble & 1u);
                        at[2] = at[1] + ((seen.nibble >> 1) & 1u);
                        at[3] = at[2] + ((seen.nibble >> 2) & 1u);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint32_t slot = min(at[j], history.capacity - 1u);
                            seen.times[j] = history.wide ? static_cast<const uint32_t *>(history.dense)[slot]
                                                         : static_cast<const uint16_t *>(history.dense)[slot];
                        }
                    }
                    return seen;
                };
                auto settle = [&](float v, uint32_t j, const Seen &seen) {
                    if ((seen.nibble >> j) & 1u) {
                        float offset = flat_offset;
                        if (flags & 2u) offset = penalty_offset(seen.times[j], cfg.presence_penalty, cfg.frequency_penalty);
                        v = penalise_with_offset(v, offset, repetition);
                    }
                    if (!is_nonfinite(v)) {
                        best = fmaxf(best, v);
                        finite++;
                    }
                    return v;
                };
                auto take4 = [&](float4 v, uint32_t q, const Seen &seen) {
                    v.x = settle(v.x, 0u, seen);
                    v.y = settle(v.y, 1u, seen);
                    v.z = settle(v.z, 2u, seen);
                    v.w = settle(v.w, 3u, seen);
                    out[q] = v;
                };
                uint32_t q = tid;
                for (; q + kNucleusThreads < quads; q += 2 * kNucleusThreads) {
                    const float4 a = load4(q), b = load4(q + kNucleusThreads);
                    const Seen seen_a = look_up(q), seen_b = look_up(q + kNucleusThreads);
                    take4(a, q, seen_a);
                    take4(b, q + kNucleusThreads, seen_b);
                }
                if (q < quads) take4(load4(q), q, look_up(q));
                done = quads * 4u;
            }
            for (uint32_t c = done + tid; c < n; c += kNucleusThreads) {
                float v;
                if (sizeof(T) == 2) v = bf16_bits_to_float(reinterpret_cast<const uint16_t *>(source)[c]);
                else v = reinterpret_cast<const float *>(source)[c];
                const uint32_t word = (flags & 1u) ? history.bitmap[c >> 5] : 0u;
                values[lo + c] = take(v, c, word);
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            best = fmaxf(best, __shfl_xor_sync(kFullMask, best, d));
            finite += __shfl_xor_sync(kFullMask, finite, d);
        }
        if (lane == 0) {
            sh.reduce_max[warp] = best;
            sh.reduce_count[warp] = finite;
        }
        __syncthreads();  // also makes the scratch row visible to the whole CTA
        best = sh.reduce_max[0];
        finite = sh.reduce_count[0];
        for (int w = 1; w < kNucleusThreads / 32; w++) {
            best = fmaxf(best, sh.reduce_max[w]);
            finite += sh.reduce_count[w];
        }
        __syncthreads();
        if (bad_history || finite == 0) {
            // src/output.c:610-612 / src/sampler.c:97 "sampler received no finite candidates"
            if (tid == 0) {
                report_row(p.out, row, bad_history ? bad_history : kErrFormat, kPaddingId, 0.0f);
                if (p.out.dbg_count) p.out.dbg_count[row] = 0;
            }
            continue;
        }

        // ---- top-p on the un-tempered softmax: where does the mass reach top_p? ----
        Nucleus all;
        all.everything = true;
        all.key = 0;
        all.id = 0;
        const double top_p = (double)cfg.top_p;
        // cumulative / sum >= top_p  <=>  cumulative >= top_p * sum
        auto mass_target = [top_p](unsigned long long total) {
            const unsigned long long t = (unsigned long long)ceil(top_p * (double)total);
            return t > total ? total : t;
        };
        Nucleus nucleus;
        nucleus.everything = false;
        unsigned long long raw_sum, mass_at_cut;
        uint32_t size;
        const double inv_t = 1.0 / (double)cfg.temperature;
        float u = p.uniforms[row];
        if (is_nonfinite(u) || u < 0.0f) u = 0.0f;
        if (u >= 1.0f) u = __uint_as_float(0x3f7fffffu);
        const double draw_at = (double)u;
        // first element whose cumulative weight exceeds draw = u * sum
        auto draw_target = [draw_at](unsigned long long total) {
            return (unsigned long long)floor(draw_at * (double)total);
        };
        uint32_t picked_id = kPaddingId;
        unsigned long long weight_sum = 0;

        // ---- the usual way: one pass fills both histograms, each phase then looks into one bucket ----
        bool done = false;
        {
            const bool filled = fill_both(sh, values, p.vocab, inv_t, best);
            const unsigned long long cut_target = find_crossing_up(sh, mass_target, false);
            raw_sum = sh.total_mass;
            const bool cut_clipped = settle_crossing(sh);
            const uint32_t cut_bucket = sh.hit_bucket;
            const unsigned long long cut_before = sh.hit_mass_before;
            const uint32_t cut_rank_before = sh.hit_count_before;
            const uint32_t cut_members = sh.count[cut_bucket];
            __syncthreads();
            unsigned long long tempered_inside = 0;  // tempered weight of the bucket's members inside the nucleus
            const Position cut = resolve_bucket(sh, list, values, p.vocab, 1.0, best, all, cut_bucket, cut_members,
                                                cut_before, cut_rank_before, cut_target, false, cut_clipped, inv_t,
                                                &tempered_inside);
            if (filled && cut.ok) {
                nucleus.key = cut.key;
                nucleus.id = cut.id;
                mass_at_cut = cut.mass;
                size = cut.rank;
                // the tempered masses of the nucleus: whole buckets above the cut's, that bucket as
                // far as the nucleus reaches into it, nothing below
                if (tid == 0) {
                    unsigned long long *raw = sh.mass;
                    sh.mass = sh.other_mass;
                    sh.other_mass = raw;
                }
                __syncthreads();
                for (uint32_t b = tid; b < kBuckets; b += kNucleusThreads) {
                    if (b > cut_bucket) {
                        sh.mass[b] = 0;
                        sh.count[b] = 0;
                    } else if (b == cut_bucket) {
                        sh.mass[b] = tempered_inside;
                    }
                }
                __syncthreads();
                const unsigned long long pick_target = find_crossing_up(sh, draw_target, true);
                weight_sum = sh.total_mass;
                const bool pick_clipped = settle_crossing(sh);
                const uint32_t pick_bucket = sh.hit_bucket;
                const unsigned long long pick_before = sh.hit_mass_before;
                const uint32_t pick_members = sh.count[pick_bucket];
                __syncthreads();
                const Position pick = resolve_bucket(sh, list, values, p.vocab, inv_t, best, nucleus, pick_bucket,
                                                     pick_members, pick_before, 0u, pick_target, true, pick_clipped,
                                                     0.0, nullptr);
                if (pick.ok) {
                    picked_id = pick.id;
                    done = true;
                }
            }
        }
        if (!done) {
        // ---- a bucket too crowded to order in shared memory: phase by phase, with the exact descent ----
        const Position cut = locate(sh, list, values, p.vocab, 1.0, best, all, mass_target, false);
        if (cut.ok) {
            nucleus.key = cut.key;
            nucleus.id = cut.id;
            raw_sum = cut.total;
            mass_at_cut = cut.mass;
            size = cut.rank;
        } else {
            // a bucket too crowded to order in shared memory: the generic radix descent
            unsigned long long partial = 0;
            for (uint32_t i = tid; i < p.vocab; i += kNucleusThreads) {
                const float v = values[i];
                if (!is_nonfinite(v)) partial += exp_fixed((double)v - (double)best, sh.table);
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) partial += __shfl_xor_sync(kFullMask, partial, d);
            if (lane == 0) sh.scan_mass[warp] = partial;
            __syncthreads();
            raw_sum = 0;
            for (int w = 0; w < kNucleusThreads / 32; w++) raw_sum += sh.scan_mass[w];
            __syncthreads();
            descend(sh, values, p.vocab, 1.0, (double)best, all, mass_target(raw_sum), false, &nucleus.key,
                    &nucleus.id, &mass_at_cut, &size);
        }

        // ---- temperature weights of the nucleus, then the draw ----
        const Position pick = locate(sh, list, values, p.vocab, inv_t, best, nucleus, draw_target, true);
        if (pick.ok) {
            picked_id = pick.id;
            weight_sum = pick.total;
        } else {
            unsigned long long partial = 0;
            for (uint32_t i = tid; i < p.vocab; i += kNucleusThreads) {
                const float v = values[i];
                if (is_nonfinite(v)) continue;
                if (nucleus.holds(float_key(v), i))
                    partial += exp_fixed(((double)v - (double)best) * inv_t, sh.table);
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) partial += __shfl_xor_sync(kFullMask, partial, d);
            if (lane == 0) sh.scan_mass[warp] = partial;
            __syncthreads();
            weight_sum = 0;
            for (int w = 0; w < kNucleusThreads / 32; w++) weight_sum += sh.scan_mass[w];
            __syncthreads();
            uint32_t picked_key, picked_rank;
            unsigned long long picked_mass;
            descend(sh, values, p.vocab, inv_t, (double)best, nucleus, draw_target(weight_sum), true,
                    &picked_key, &picked_id, &picked_mass, &picked_rank);
        }
        }
        if (tid == 0) {
            if (weight_sum == 0 || raw_sum == 0 || picked_id >= p.vocab) {
                report_row(p.out, row, kErrFormat, kPaddingId, 0.0f);
            } else {
                report_row(p.out, row, kOk, picked_id, values[picked_id]);
            }
            if (p.out.dbg_count) p.out.dbg_count[row] = size;  // nucleus size; the list itself is not dumped
        }
        __syncthreads();
    }
}

}  // namespace fgk

using namespace fgk;


static constexpr size_t kNucleusDynamic = kNucleusHistogramBytes + sizeof(NucleusList);

extern "C" int fgk_nucleus_prepare(void) {
    cudaError_t e = cudaFuncSetAttribute(nucleus_select_kernel<float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kNucleusDynamic);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(nucleus_select_kernel<uint16_t>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kNucleusDynamic);
    return (int)e;
}

extern "C" int fgk_launch_nucleus_select(const fgk_nucleus_launch *l, void *stream) {
    NucleusParams p;
    p.logits = l->logits;
    p.dtype = l->dtype;
    p.rows = l->rows;
    p.vocab = l->vocab;
    p.row_stride = l->row_stride;
    p.configs = reinterpret_cast<const SamplerConfig *>(l->configs_device);
    p.config0.temperature = l->config0.temperature;
    p.config0.top_p = l->config0.top_p;
    p.config0.top_k = l->config0.top_k;
    p.config0.presence_penalty = l->config0.presence_penalty;
    p.config0.frequency_penalty = l->config0.frequency_penalty;
    p.config0.repetition_penalty = l->config0.repetition_penalty;
    p.config0.min_p = l->config0.min_p;
    p.config0.pad_ = 0;
    p.config0.seed = l->config0.seed;
    p.config_count = l->config_count;
    p.uniforms = l->uniforms;
    p.scratch = l->scratch;
    p.scratch_stride = l->scratch_stride;
    p.history_global = l->history_global;
    p.history_stride_words = l->history_stride_words;
    p.history_meta = l->history_meta;
    p.splits = l->splits;
    p.split_len = l->split_len;
    p.bitmap_words = l->bitmap_words;
    p.count_capacity = l->count_capacity;
    p.dense_wide = l->dense_wide;
    p.out.tokens = l->out.tokens;
    p.out.token_logits = l->out.token_logits;
    p.out.row_status = l->out.row_status;
    p.out.first_error = reinterpret_cast<unsigned long long *>(l->out.first_error);
    p.out.dbg_count = l->out.dbg_count;
    p.out.dbg_ids = l->out.dbg_ids;
    p.out.dbg_scores = l->out.dbg_scores;
    p.out.dbg_raw = l->out.dbg_raw;
    p.out.dbg_tempered = l->out.dbg_tempered;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (l->dtype == 1u)
        nucleus_select_kernel<uint16_t><<<l->ctas, kNucleusThreads, kNucleusDynamic, s>>>(p);
    else
        nucleus_select_kernel<float><<<l->ctas, kNucleusThreads, kNucleusDynamic, s>>>(p);
    return (int)cudaGetLastError();
}
