// Persistent sampling kernel for sm_100a: rows stream through a shared-memory ring
// that a warp of its own keeps full.
//
// One CTA = eight consumer warps + one copy warp, FGK_PERSIST_CTAS of them per SM,
// each working through rows  blockIdx.x, blockIdx.x + gridDim.x, ...
//
//   copy warp   one lane asks the copy engine (cp.async.bulk + mbarrier) for 16 KB
//               tiles, row after row, as fast as ring stages come free.  It never
//               waits for anything but a free stage, so bytes stay in flight while the
//               consumers build a history bitmap, cut a candidate list or finish a row
//               -- the next row's first tiles are already there when they come back.
//   consumers   per row: (1) bitmap of the ids in the row's token history, in shared
//               memory; (2) tile 0 gives a first admission bound; (3) every further
//               tile costs a 128-bit shared load, three maxima and one compare per
//               vector -- single elements are looked at only above the bound;
//               (4) the select step of src/sampler.c:80-122 on the k survivors.
//
// The kernel takes rows whose penalties can only lower a logit (presence >= 0,
// frequency >= 0, repetition >= 1, or no penalties / no history at all).  Then a raw
// value at or below the bound stays there, so the history matters only for the few
// values above it.  An id that was seen is charged  frequency * count + presence
// (src/sampler.c:52-58); the count is not tabulated per row (src/output.c:601-617
// keeps a vocabulary-wide table per session): when the penalty for count = 1 -- an
// upper bound of the penalised value -- still beats the bound, the id is put aside and
// its occurrences are counted in the token list when the list is next cut.  Everything
// else (penalties that can raise a logit, rows that are not 16-byte aligned, column
// splits) stays with stream_select_kernel.
#include <cstring>

#include "fg_block_select.cuh"
#include "fg_kernels.h"

namespace fgk {
namespace persist {

#ifndef FGK_PERSIST_STAGES
#define FGK_PERSIST_STAGES 4
#endif
#ifndef FGK_PERSIST_CTAS
#define FGK_PERSIST_CTAS 2
#endif

constexpr int kStages = FGK_PERSIST_STAGES;
constexpr int kConsumers = 256;
constexpr int kConsumerWarps = kConsumers / 32;
constexpr int kBlock = kConsumers + 64;  // + the copy warp and the closing warp
constexpr uint32_t kStageBytes = 16384;
constexpr int kVectors = 4;              // 128-bit vectors per consumer thread and tile
constexpr int kCandCap = 1024;
constexpr int kDeferCap = 256;           // ids put aside until their occurrences are counted
constexpr uint32_t kWaitPolls = 1u << 20;
constexpr uint32_t kNapNanoseconds = 2000;  // longest sleep inside one poll of an mbarrier

// The eight consumer warps meet at named barrier 1; the copy warp never does.
struct ConsumerBarrier {
    static __device__ __forceinline__ void sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
    static __device__ __forceinline__ bool sync_or(bool mine) {
        uint32_t any;
        asm volatile(
            "{\n\t.reg .pred in, out;\n\t"
            "setp.ne.u32 in, %1, 0;\n\t"
            "bar.red.or.pred out, 1, 256, in;\n\t"
            "selp.u32 %0, 1, 0, out;\n\t}"
            : "=r"(any)
            : "r"((uint32_t)mine)
            : "memory");
        return any != 0;
    }
};
using CB = ConsumerBarrier;

template <typename T>
struct Lanes;
template <>
struct Lanes<float> {
    static constexpr int kPer = 4;  // logits per 128-bit vector
    static __device__ __forceinline__ void unpack(const uint4 &raw, float *v) {
        v[0] = __uint_as_float(raw.x);
        v[1] = __uint_as_float(raw.y);
        v[2] = __uint_as_float(raw.z);
        v[3] = __uint_as_float(raw.w);
    }
};
template <>
struct Lanes<uint16_t> {  // bf16 bit patterns
    static constexpr int kPer = 8;
    static __device__ __forceinline__ void unpack(const uint4 &raw, float *v) {
        v[0] = __uint_as_float(raw.x << 16);
        v[1] = __uint_as_float(raw.x & 0xffff0000u);
        v[2] = __uint_as_float(raw.y << 16);
        v[3] = __uint_as_float(raw.y & 0xffff0000u);
        v[4] = __uint_as_float(raw.z << 16);
        v[5] = __uint_as_float(raw.z & 0xffff0000u);
        v[6] = __uint_as_float(raw.w << 16);
        v[7] = __uint_as_float(raw.w & 0xffff0000u);
    }
};

// What a CTA that shares a row leaves behind for the merge.
struct alignas(16) PartRecord {
    uint32_t count;         // finite candidates kept (<= k)
    uint32_t wild_id;       // smallest id holding a NaN/Inf (greedy rows), padding if none
    uint32_t wild_bits;     // its value
    uint32_t bad_history;   // 0, or the fg_status a broken history earns the row
};

struct Params {
    const void *logits;
    uint64_t row_stride;  // elements
    uint32_t rows, vocab;
    uint32_t vocab_offset, vocab_total;
    const uint32_t *history_tokens;
    const uint64_t *history_offsets;
    uint32_t history_max;
    uint32_t bitmap_words;          // 0: the batch has no history
    const SamplerConfig *configs;   // device copy when config_count > 1
    SamplerConfig config0;
    uint32_t config_count;
    uint32_t shard_k;               // != 0: write candidates instead of sampling
    const float *uniforms;
    float *shard_scores;
    uint32_t *shard_ids;
    // Work is dealt out in 16 KB tiles: CTA c takes tiles [c * tiles_per_cta, (c + 1) *
    // tiles_per_cta) of the batch's tile sequence (row after row), so a row may be shared
    // by several CTAs.  Each leaves its part's k best in `parts`; the last to finish
    // (ticket counter) merges them.
    // With enough rows for every CTA to have several, whole rows are dealt out instead
    // (tiles_per_cta == 0): CTA c takes rows c, c + ctas, c + 2 * ctas, ...  (the two CTAs
    // of an SM, c and c + SMs, then differ by at most one row between them).
    uint32_t tiles_per_cta;
    uint32_t max_parts;             // most CTAs that share one row
    float *part_scores;             // [rows][max_parts][kMaxK]
    uint32_t *part_ids;
    PartRecord *part_meta;          // [rows][max_parts]
    uint32_t *tickets;              // [rows], zero between launches
    SelectOutput out;
};

// One CTA's share of one row.
struct Unit {
    uint32_t row;
    uint32_t first, end;    // tiles [first, end) of the row
    uint32_t part, parts;   // which of how many shares of the row
};

// Walks the units of this CTA in order.
struct UnitWalk {
    uint64_t at, stop;      // position in the batch's tile sequence
    uint32_t row_tiles, per_cta;
    __device__ __forceinline__ UnitWalk(const Params &p, uint32_t row_tiles_)
        : row_tiles(row_tiles_), per_cta(p.tiles_per_cta) {
        const uint64_t all = (uint64_t)p.rows * row_tiles;
        if (per_cta == 0) {
            at = blockIdx.x;  // a row number in this mode
            stop = p.rows;
        } else {
            at = min((uint64_t)blockIdx.x * per_cta, all);
            stop = min(at + per_cta, all);
        }
    }
    __device__ __forceinline__ bool next(Unit &u) {
        if (at >= stop) return false;
        if (per_cta == 0) {
            u.row = (uint32_t)at;
            u.first = 0;
            u.end = row_tiles;
            u.part = 0;
            u.parts = 1;
            at += gridDim.x;
            return true;
        }
        u.row = (uint32_t)(at / row_tiles);
        u.first = (uint32_t)(at % row_tiles);
        u.end = (uint32_t)min((uint64_t)row_tiles, u.first + (stop - at));
        const uint64_t row_begin = (uint64_t)u.row * row_tiles;
        const uint32_t first_cta = (uint32_t)(row_begin / per_cta);
        const uint32_t last_cta = (uint32_t)((row_begin + row_tiles - 1) / per_cta);
        u.part = blockIdx.x - first_cta;
        u.parts = last_cta - first_cta + 1;
        at += u.end - u.first;
        return true;
    }
};

// What the consumers collect for one row.  There are two of these: while the closing
// warp turns one row's lists into its result the consumers fill the other.
struct Lists {
    CandidateBuffer<kCandCap> cand;
    float defer_raw[kDeferCap];      // raw logit of an id put aside
    uint32_t defer_id[kDeferCap];
    uint32_t defer_seen[kDeferCap];  // its occurrences in the history, once counted
    unsigned long long wild_key;     // greedy rows: min over NaN/Inf of (id << 32 | value bits)
    uint32_t defer_count;
    uint32_t bad_history;
};

struct Shared {
    Lists lists[2];
    FinishBuffer fin;                    // the closing warp's
    uint32_t closer_hist[256];
    uint32_t closer_count;
    alignas(8) uint64_t full[kStages];   // "the tile has landed"
    alignas(8) uint64_t empty[kStages];  // "the consumers are done with the stage"
    alignas(8) uint64_t ready[2];        // "the row's lists are complete"
    alignas(8) uint64_t vacant[2];       // "the closing warp is done with the lists"
    uint32_t through[2];             // warps that have finished the row's tiles, by row parity
    uint32_t ring_error;             // a bounded wait ran out
    uint32_t first_key;              // tile 0: the smallest of the warps' j-th largest keys
    uint32_t attention;              // a list is long or full: every warp comes to attend()
};

// What the consumers need to know about the row; lives in registers.
struct Row {
    const uint32_t *tokens;  // the row's history
    uint32_t history_len;
    uint32_t id_base;        // global id of column 0
    uint32_t k, cut_at;
    float flat_offset;       // charge for count = 1 (the exact charge when frequency is +-0)
    float presence, frequency;
    Repetition repetition;
    bool greedy, seen_any, with_counts;
};

__device__ __forceinline__ bool bounded_wait(uint64_t *barrier, uint32_t parity) {
    for (uint32_t polls = 0; polls < kWaitPolls; polls++)
        if (mbarrier_try_wait_sleeping(barrier, parity, kNapNanoseconds)) return true;
    return false;
}

// Shared words that warps watch while others change them.
__device__ __forceinline__ uint32_t peek(const uint32_t *word) {
    return *reinterpret_cast<const volatile uint32_t *>(word);
}
__device__ __forceinline__ void poke(uint32_t *word, uint32_t value) {
    *reinterpret_cast<volatile uint32_t *>(word) = value;
}

// One element whose raw value reaches the bound.  The bound is a (score, id) pair:
// the k-th best of some earlier state of the candidate list (or, before the first
// cut, tile 0's first bound with the padding id, which every id precedes).  What does
// not precede it can never be among the k best, in whatever order the warps run.
// Returns false when the list the element belongs on is full (the caller asks for a
// cut and offers the element again).
template <bool kGreedy>
__device__ __forceinline__ bool consider(Shared &sh, Lists &L, const Row &r, float x, uint32_t id, bool seen,
                                         float tau, uint32_t tau_id) {
    if (seen) {
        const float bound = penalise_with_offset(x, r.flat_offset, r.repetition);
        if (r.with_counts) {
            // the charge grows with the count, so `bound` is the most the id can keep
            const bool alive = bound >= tau;
            // greedy rows must also see NaN/Inf, raw or made by the penalty
            const bool wild = kGreedy && (__float_as_uint(x) & 0x7fffffffu) >= 0x6b000000u;
            if (!(alive || wild)) return true;
            const uint32_t slot = atomicAdd(&L.defer_count, 1u);
            if (slot >= (uint32_t)kDeferCap) return false;
            L.defer_raw[slot] = x;
            L.defer_id[slot] = id;
            if (slot >= (uint32_t)kDeferCap / 2) poke(&sh.attention, 1u);
            return true;
        }
        x = bound;
    }
    if (is_nonfinite(x)) {
        if (kGreedy) atomicMin(&L.wild_key, ((unsigned long long)id << 32) | __float_as_uint(x));
        return true;
    }
    if (!precedes(x, id, tau, tau_id)) return true;
    const uint32_t slot = atomicAdd(&L.cand.count, 1u);
    if (slot >= (uint32_t)kCandCap) return false;
    L.cand.score[slot] = x;
    L.cand.id[slot] = id;
    if (slot >= r.cut_at) poke(&sh.attention, 1u);
    return true;
}

// A cut that need not be exact: one histogram pass over the candidates' keys (256 bins
// between the smallest and the largest key in the list) finds the highest bin edge with
// at least k candidates at or above it; everything below goes, and the smallest score
// that stays is the new bound (with the padding id: a tie with it is still admitted).
// About a third of the barriers of the exact radix select.  Rows whose candidates
// crowd into one bin (constant rows) keep too many: the caller then cuts exactly.
// Every consumer calls it with the same `held` > k; returns what is left.
__device__ __forceinline__ uint32_t quick_cut(Lists &L, uint32_t held, uint32_t k) {
    constexpr int PER = kCandCap / kConsumers;
    CandidateBuffer<kCandCap> &buf = L.cand;
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    float score[PER];
    uint32_t id[PER], key[PER];
    uint32_t high = 0, low = 0xffffffffu;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const uint32_t at = j * kConsumers + tid;
        key[j] = 0;
        if (at < held) {
            score[j] = buf.score[at];
            id[j] = buf.id[at];
            key[j] = float_key(score[j]);  // finite, so never 0
            high = max(high, key[j]);
            low = min(low, key[j]);
        }
    }
    buf.hist[tid] = 0;
    if (tid == 0) {
        buf.sel_need = 0;             // largest key
        buf.sel_bucket = 0xffffffffu; // smallest key
        buf.out_count = 0;
        buf.eq_count = 0xffffffffu;   // smallest key that stays
    }
    CB::sync();
    high = __reduce_max_sync(kFullMask, high);
    low = __reduce_min_sync(kFullMask, low);
    if (lane == 0) {
        atomicMax(&buf.sel_need, high);
        atomicMin(&buf.sel_bucket, low);
    }
    CB::sync();
    const uint32_t base = buf.sel_bucket;
    const uint32_t range = buf.sel_need - base;
    const int shift = max(0, 24 - (int)__clz(range | 1u));  // (range >> shift) < 256
#pragma unroll
    for (int j = 0; j < PER; j++)
        if (key[j] != 0) atomicAdd(&buf.hist[(key[j] - base) >> shift], 1u);
    CB::sync();
    if (tid < 32) {
        // lane l owns bins 255-8l .. 248-8l, walked from the top
        uint32_t mine = 0;
#pragma unroll
        for (int b = 0; b < 8; b++) mine += buf.hist[255 - 8 * tid - b];
        uint32_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t up = __shfl_up_sync(kFullMask, incl, d);
            if (tid >= (uint32_t)d) incl += up;
        }
        const unsigned reached = __ballot_sync(kFullMask, incl >= k);
        const int owner = __ffs(reached) - 1;  // k < held, so some lane reaches it
        if ((int)tid == owner) {
            uint32_t above = incl - mine;
            for (int b = 0; b < 8; b++) {
                const uint32_t bin = 255 - 8 * tid - b;
                above += buf.hist[bin];
                if (above >= k) {
                    buf.sel_digit = bin;
                    break;
                }
            }
        }
    }
    CB::sync();
    const uint32_t edge = buf.sel_digit;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        if (key[j] != 0 && ((key[j] - base) >> shift) >= edge) {
            const uint32_t slot = atomicAdd(&buf.out_count, 1u);
            buf.score[slot] = score[j];
            buf.id[slot] = id[j];
            atomicMin(&buf.eq_count, key[j]);
        }
    }
    CB::sync();
    if (tid == 0) {
        buf.tau_score = key_to_float(buf.eq_count);
        buf.tau_id = kPaddingId;
        buf.count = buf.out_count;
    }
    CB::sync();
    return buf.out_count;
}

// The meeting of all consumer warps.  A warp comes here when it sees sh.attention
// up or when one of its lanes found a list full (it then raises the flag itself).
// Nobody appends to a list while the meeting is on.  Ids that were put aside get their occurrences counted in the row's token list
// and their exact penalised value, and join the candidates if they precede the bound;
// a long candidate list is cut back to its k best, which lifts the bound.
// Returns the bound's score (the pair is in L.cand.tau_*).
__device__ __noinline__ float attend(Shared &sh, Lists &L, const Row r) {
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    CB::sync();
    uint32_t aside = min(L.defer_count, (uint32_t)kDeferCap);
    uint32_t held = min(L.cand.count, (uint32_t)kCandCap);
    CB::sync();  // everyone has read the counts before anything rewrites them
    if (aside < (uint32_t)kDeferCap / 2) aside = 0;  // not worth a pass yet
    if (aside != 0) {
        if (held + aside > (uint32_t)kCandCap) {  // make room first
            compact_topk<kConsumers, kCandCap, CB>(L.cand, held, r.k);
            held = min(held, r.k);
        }
        if (tid < aside) L.defer_seen[tid] = 0;
        CB::sync();
        constexpr int kBatch = 8;
        for (uint32_t base = 0; base < r.history_len; base += kBatch * kConsumers) {
            uint32_t token[kBatch];
#pragma unroll
            for (int q = 0; q < kBatch; q++) {
                const uint32_t i = base + q * kConsumers + tid;
                token[q] = i < r.history_len ? r.tokens[i] : kPaddingId;  // the padding id is nobody's
            }
            for (uint32_t d = 0; d < aside; d++) {
                const uint32_t id = L.defer_id[d];
                uint32_t hits = 0;
#pragma unroll
                for (int q = 0; q < kBatch; q++) hits += token[q] == id ? 1u : 0u;
                hits = __reduce_add_sync(kFullMask, hits);
                if (lane == 0 && hits != 0) atomicAdd(&L.defer_seen[d], hits);
            }
        }
        CB::sync();
        const float tau = L.cand.tau_score;
        const uint32_t tau_id = L.cand.tau_id;
        if (tid < aside) {
            const uint32_t id = L.defer_id[tid];
            const float x = penalise_with_offset(
                L.defer_raw[tid], penalty_offset(L.defer_seen[tid], r.presence, r.frequency),
                r.repetition);
            if (is_nonfinite(x)) {
                if (r.greedy)
                    atomicMin(&L.wild_key, ((unsigned long long)id << 32) | __float_as_uint(x));
            } else if (precedes(x, id, tau, tau_id)) {
                const uint32_t slot = atomicAdd(&L.cand.count, 1u);  // room was made above
                L.cand.score[slot] = x;
                L.cand.id[slot] = id;
            }
        }
        CB::sync();
        if (tid == 0) L.defer_count = 0;
        held = min(L.cand.count, (uint32_t)kCandCap);
        CB::sync();
    }
    if (held >= r.cut_at) {
        held = quick_cut(L, held, r.k);
        // (a list the quick cut could not thin out is cut exactly, ties resolved by id)
        if (held >= (r.k + r.cut_at) / 2) compact_topk<kConsumers, kCandCap, CB>(L.cand, held, r.k);
    }
    if (tid == 0) sh.attention = 0;
    CB::sync();
    return L.cand.tau_score;
}

// Position in the ring; the copy warp and the consumers count tiles the same way.
struct RingCursor {
    uint32_t stage = 0, use = 0;  // `use` counts how often the ring has wrapped
    __device__ __forceinline__ void advance() {
        if (++stage == (uint32_t)kStages) {
            stage = 0;
            use++;
        }
    }
};

// One logit of a tile in the ring, by its position in the tile.
template <typename T>
__device__ __forceinline__ float tile_element(const unsigned char *stage, uint32_t position);
template <>
__device__ __forceinline__ float tile_element<float>(const unsigned char *stage, uint32_t position) {
    return reinterpret_cast<const float *>(stage)[position];
}
template <>
__device__ __forceinline__ float tile_element<uint16_t>(const unsigned char *stage, uint32_t position) {
    return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t *>(stage)[position] << 16);
}

// Offers this lane's pending elements of a tile (bit e = element e % kPer of its vector
// e / kPer) to the lists, re-reading them from the ring.  Stops at the first one that
// finds no room; returns what is left.
template <typename T, bool kGreedy>
__device__ __forceinline__ uint32_t offer(Shared &sh, Lists &L, const Row &r, const uint32_t *bitmap,
                                          const unsigned char *stage, uint32_t t, uint32_t pending,
                                          float tau, uint32_t tau_id) {
    constexpr int kPer = Lanes<T>::kPer;
    constexpr uint32_t kTile = kStageBytes / sizeof(T);
    while (pending != 0) {
        const uint32_t e = __ffs(pending) - 1;
        const uint32_t position = ((e / kPer) * kConsumers + threadIdx.x) * kPer + (e % kPer);
        const uint32_t column = t * kTile + position;
        const bool seen = r.seen_any && ((bitmap[column >> 5] >> (column & 31u)) & 1u);
        if (!consider<kGreedy>(sh, L, r, tile_element<T>(stage, position), r.id_base + column, seen, tau,
                               tau_id))
            break;
        pending &= pending - 1;
    }
    return pending;
}

// Offers until nothing is pending in the warp, meeting the other warps for a cut
// whenever a list is full.  All lanes of the warp call it together; returns the bound.
template <typename T, bool kGreedy>
__device__ __noinline__ float settle(Shared &sh, Lists &L, const Row r, const uint32_t *bitmap,
                                     const unsigned char *stage, uint32_t t, uint32_t pending,
                                     float tau) {
    for (;;) {
        pending = offer<T, kGreedy>(sh, L, r, bitmap, stage, t, pending, tau, L.cand.tau_id);
        if (!__any_sync(kFullMask, pending != 0)) return tau;
        poke(&sh.attention, 1u);
        tau = attend(sh, L, r);
    }
}

// The first tile of a unit, all warps together: every element is looked at.  The first bound is
// the smallest, over the warps, of each warp's j-th largest per-thread maximum of
// unseen finite values, j = ceil(k / warps): at least k distinct elements are that
// large.  (No bound when some warp has fewer than j such threads; everything finite
// is then a candidate until the first cut.)  Returns the bound.
template <typename T>
__device__ __noinline__ float first_tile(Shared &sh, Lists &L, const uint32_t *bitmap, const unsigned char *stage,
                                         uint32_t t, uint32_t valid_vectors, const Row r) {
    using V = Lanes<T>;
    constexpr int kPer = V::kPer;
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    const uint4 *vectors = reinterpret_cast<const uint4 *>(stage);
    float best = __uint_as_float(0xff800000u);
    bool have = false;
#pragma unroll
    for (int u = 0; u < kVectors; u++) {
        const uint32_t g = u * kConsumers + tid;
        if (g >= valid_vectors) continue;
        float v[kPer];
        V::unpack(vectors[g], v);
        const uint32_t column = t * (kStageBytes / (uint32_t)sizeof(T)) + g * kPer;
        const uint32_t bits =
            r.seen_any ? (bitmap[column >> 5] >> (column & 31u)) & ((1u << kPer) - 1u) : 0u;
#pragma unroll
        for (int j = 0; j < kPer; j++) {
            if (!((bits >> j) & 1u) && !is_nonfinite(v[j])) {
                best = fmaxf(best, v[j]);
                have = true;
            }
        }
    }
    uint32_t key = have ? float_key(best) : 0u;
    const uint32_t per_warp = (r.k + kConsumerWarps - 1) / kConsumerWarps;
    uint32_t kth = 0;
    for (uint32_t i = 0; i < per_warp; i++) {
        kth = __reduce_max_sync(kFullMask, key);
        if (kth == 0) break;
        const unsigned owners = __ballot_sync(kFullMask, key == kth);
        if ((int)lane == __ffs(owners) - 1) key = 0;
    }
    if (lane == 0) atomicMin(&sh.first_key, kth);
    CB::sync();
    const float tau = key_to_float(sh.first_key);
    if (tid == 0) {
        L.cand.tau_score = tau;
        L.cand.tau_id = kPaddingId;
    }
    CB::sync();
    // everything that reaches the bound raw is offered (greedy rows: and every NaN/Inf
    // or huge magnitude)
    uint32_t pending = 0;
#pragma unroll
    for (int u = 0; u < kVectors; u++) {
        const uint32_t g = u * kConsumers + tid;
        if (g >= valid_vectors) continue;
        float v[kPer];
        V::unpack(vectors[g], v);
#pragma unroll
        for (int j = 0; j < kPer; j++) {
            const bool wild = r.greedy && (__float_as_uint(v[j]) & 0x7fffffffu) >= 0x6b000000u;
            if (v[j] >= tau || wild) pending |= 1u << (u * kPer + j);
        }
    }
    return r.greedy ? settle<T, true>(sh, L, r, bitmap, stage, t, pending, tau)
                    : settle<T, false>(sh, L, r, bitmap, stage, t, pending, tau);
}

// What hot_tiles hands back: the tile it stopped at, why, and this lane's elements of
// that tile still to be offered.
constexpr uint32_t kStopDone = 0, kStopBefore = 1, kStopInside = 2;
struct Stop {
    uint32_t tile, why, pending;
};

// Largest of three; a NaN loses against a number, as with fmaxf.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
#ifdef FGK_NO_MAX3
    return fmaxf(fmaxf(a, b), c);
#else
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
#endif
}

// Largest of N values, three at a time (a short tree instead of a chain of N - 1).
template <int N>
__device__ __forceinline__ float largest(const float (&v)[N]) {
    float level[N];
#pragma unroll
    for (int i = 0; i < N; i++) level[i] = v[i];
    int n = N;
#pragma unroll
    for (int round = 0; round < 6; round++) {
        if (n <= 1) break;
        int m = 0;
#pragma unroll
        for (int i = 0; i < N; i += 3) {
            if (i >= n) break;
            if (i + 2 < n) level[m++] = fmax3(level[i], level[i + 1], level[i + 2]);
            else if (i + 1 < n) level[m++] = fmaxf(level[i], level[i + 1]);
            else level[m++] = level[i];
        }
        n = m;
    }
    return level[0];
}

// The hot loop of one warp over tiles first .. end-1 of a row; the warps run it
// independently of one another, at most a ring's depth apart.  It calls nothing:
// whatever is live across a call inside a loop is saved and restored on every trip.
// Per tile and thread: four 128-bit shared loads, a tree of maxima, one compare, one
// warp reduction that also carries the attention flag.  kRagged: the tiles may end
// early (`valid_vectors` of them hold data); only a row's last tile needs that.
//   kStopBefore  the attention flag is up and the warp has not touched `tile` yet
//   kStopInside  a lane found a list full; `pending` holds its elements of `tile`
//                still to be offered, and the warp still holds the stage
template <typename T, bool kGreedy, bool kRagged>
__device__ __noinline__ Stop hot_tiles(Shared &sh, Lists &L, const uint32_t *bitmap, const unsigned char *ring,
                                       uint32_t first, uint32_t end, uint32_t valid_vectors,
                                       const uint32_t row_sequence, const Row r, const float tau) {
    using V = Lanes<T>;
    constexpr int kPer = V::kPer;
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    const uint32_t tau_id = L.cand.tau_id;
    Stop stop;
    stop.pending = 0;
    for (uint32_t t = first; t < end; t++) {
        const uint32_t at = (row_sequence + t) % kStages, use = (row_sequence + t) / kStages;
        stop.tile = t;
        // ---- the tile is usually there, or lands within one nap ----
        if (!__all_sync(kFullMask, mbarrier_try_wait_sleeping(&sh.full[at], use & 1u, kNapNanoseconds))) {
            // otherwise wait for it watching the flag (a warp that holds this stage may be
            // waiting for this one at a meeting)
            for (uint32_t polls = 0;; polls++) {
                if (__any_sync(kFullMask, peek(&sh.attention) != 0)) {
                    stop.why = kStopBefore;
                    return stop;
                }
                const bool landed = peek(&sh.ring_error) != 0 ||
                                    mbarrier_try_wait_sleeping(&sh.full[at], use & 1u, kNapNanoseconds);
                if (__all_sync(kFullMask, landed)) break;
                if (polls >= kWaitPolls) poke(&sh.ring_error, 1u);  // values are then garbage; the row fails
            }
        }
        const unsigned char *stage = ring + (size_t)at * kStageBytes;
        const uint4 *vectors = reinterpret_cast<const uint4 *>(stage);
        uint4 raw[kVectors];
#pragma unroll
        for (int u = 0; u < kVectors; u++) {
            const uint32_t g = u * kConsumers + tid;
            // (the filler reads as a NaN in fp32 and as -inf in bf16: never reaches a bound)
            if (kRagged && g >= valid_vectors) raw[u] = make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);
            else raw[u] = vectors[g];
        }
        const uint32_t flagged = peek(&sh.attention);  // read early, used after the tile
        float v[kVectors * kPer];
#pragma unroll
        for (int u = 0; u < kVectors; u++) V::unpack(raw[u], &v[u * kPer]);
        bool hot = largest(v) >= tau;  // a NaN never wins a maximum
        if (kGreedy) {  // the argmax order must see NaN and both infinities, and magnitudes
                        // a repetition factor of at most 2^40 could push there
            uint32_t widest = 0;
#pragma unroll
            for (int e = 0; e < kVectors * kPer; e++) widest = max(widest, __float_as_uint(v[e]) & 0x7fffffffu);
            hot = hot || widest >= 0x6b000000u;
        }
        uint32_t pending = 0;
        if (hot) {
#pragma unroll
            for (int e = 0; e < kVectors * kPer; e++) {
                const bool live = !kRagged || (e / kPer) * kConsumers + tid < valid_vectors;
                const bool wild = kGreedy && (__float_as_uint(v[e]) & 0x7fffffffu) >= 0x6b000000u;
                if (live && (v[e] >= tau || wild)) pending |= 1u << e;
            }
            pending = offer<T, kGreedy>(sh, L, r, bitmap, stage, t, pending, tau, tau_id);
        }
        // one reduction tells the warp both things: somebody still has elements to offer (bit
        // 0), somebody saw the flag up (bit 1)
        const uint32_t news = __reduce_or_sync(kFullMask, (pending != 0 ? 1u : 0u) | (flagged != 0 ? 2u : 0u));
        if (news & 1u) {
            stop.why = kStopInside;
            stop.pending = pending;
            return stop;
        }
        if (lane == 0) mbarrier_arrive(&sh.empty[at]);  // the warp is done with the stage
        if (news & 2u) {
            stop.tile = t + 1;
            stop.why = kStopBefore;
            return stop;
        }
    }
    stop.tile = end;
    stop.why = kStopDone;
    return stop;
}

// Phase 1 of a row: bitmap of the history ids that fall into this kernel's columns.
// A token outside the vocabulary leaves its status in L.bad_history.
__device__ __noinline__ void build_bitmap(Lists &L, uint32_t *bitmap, const Params &p, const Row r) {
    const uint32_t tid = threadIdx.x;
    uint4 *wide = reinterpret_cast<uint4 *>(bitmap);
    const uint32_t quads = (p.bitmap_words + 3u) / 4u;  // the host rounds the allocation up
    for (uint32_t i = tid; i < quads; i += kConsumers) wide[i] = make_uint4(0, 0, 0, 0);
    CB::sync();
    constexpr int kBatch = 8;  // tokens per thread and trip, loaded before any is used
    for (uint32_t base = 0; base < r.history_len; base += kBatch * kConsumers) {
        uint32_t token[kBatch];
#pragma unroll
        for (int q = 0; q < kBatch; q++) {
            const uint32_t i = base + q * kConsumers + tid;
            token[q] = i < r.history_len ? r.tokens[i] : p.vocab_offset;
        }
#pragma unroll
        for (int q = 0; q < kBatch; q++) {
            if (base + q * kConsumers + tid >= r.history_len) continue;
            if (token[q] >= p.vocab_total) L.bad_history = kErrFormat;
            const uint32_t local = token[q] - p.vocab_offset;  // wraps for ids below the span
            if (local < p.vocab) {
                const uint32_t bit = 1u << (local & 31u);
                if ((bitmap[local >> 5] & bit) == 0) atomicOr(&bitmap[local >> 5], bit);
            }
        }
    }
    CB::sync();
}

// ------------------------------------------------------------------ closing warp
//
// When the consumers are through with a row they leave its lists behind and go on
// with the next row on the other pair of lists; this warp turns the lists into the
// row's result: it counts the occurrences of the ids still put aside, takes the exact
// k best of both lists (MSB-first radix select over the 64-bit (score, ~id) keys,
// 8-bit digits, the warp's own histogram), sorts them and runs the select step of
// src/sampler.c:80-122.

// Key of entry i of the row's lists (candidates first, then the ids that were put
// aside, whose defer_raw by now holds the exact penalised value); 0 = no entry.
__device__ __forceinline__ uint64_t list_key(const Lists &L, uint32_t held, uint32_t i) {
    if (i < held) return select_key(L.cand.score[i], L.cand.id[i]);
    const uint32_t d = i - held;
    return L.defer_id[d] == kPaddingId ? 0ull : select_key(L.defer_raw[d], L.defer_id[d]);
}

// The exact k best of a pair of lists, in sampling order, into sh.fin; returns how many.
__device__ __noinline__ uint32_t settle_lists(Shared &sh, Lists &L, const Row r) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t held = min(L.cand.count, (uint32_t)kCandCap);
    const uint32_t aside = min(L.defer_count, (uint32_t)kDeferCap);

    // ---- exact values of the ids put aside ----
    if (aside != 0) {
        for (uint32_t d = lane; d < aside; d += 32) L.defer_seen[d] = 0;
        __syncwarp();
        constexpr int kBatch = 8;
        for (uint32_t base = 0; base < r.history_len; base += kBatch * 32) {
            uint32_t token[kBatch];
#pragma unroll
            for (int q = 0; q < kBatch; q++) {
                const uint32_t i = base + q * 32 + lane;
                token[q] = i < r.history_len ? r.tokens[i] : kPaddingId;
            }
            for (uint32_t d = 0; d < aside; d++) {
                const uint32_t id = L.defer_id[d];
                uint32_t hits = 0;
#pragma unroll
                for (int q = 0; q < kBatch; q++) hits += token[q] == id ? 1u : 0u;
                hits = __reduce_add_sync(kFullMask, hits);
                if (lane == 0) L.defer_seen[d] += hits;
            }
        }
        __syncwarp();
        for (uint32_t d = lane; d < aside; d += 32) {
            const uint32_t id = L.defer_id[d];
            const float x = penalise_with_offset(
                L.defer_raw[d], penalty_offset(L.defer_seen[d], r.presence, r.frequency), r.repetition);
            if (is_nonfinite(x)) {
                if (r.greedy) atomicMin(&L.wild_key, ((unsigned long long)id << 32) | __float_as_uint(x));
                L.defer_id[d] = kPaddingId;
            } else {
                L.defer_raw[d] = x;
            }
        }
        __syncwarp();
    }

    // ---- the k best of held + aside entries ----
    const uint32_t entries = held + aside;
    uint32_t live = 0;
    for (uint32_t i = lane; i < entries; i += 32) live += list_key(L, held, i) != 0 ? 1u : 0u;
    live = __reduce_add_sync(kFullMask, live);
    const uint32_t keep = min(live, r.k);
    uint64_t prefix = 0;
    int shift = 64;  // keys whose bits above `shift` exceed `prefix` are in; equal ones fill up
    uint32_t need = keep;
    if (live > r.k) {
        shift = 56;
        for (int pass = 0; pass < 8; pass++) {
            for (uint32_t b = lane; b < 256; b += 32) sh.closer_hist[b] = 0;
            __syncwarp();
            for (uint32_t i = lane; i < entries; i += 32) {
                const uint64_t key = list_key(L, held, i);
                if (key != 0 && (pass == 0 || (key >> (shift + 8)) == prefix))
                    atomicAdd(&sh.closer_hist[(key >> shift) & 255u], 1u);
            }
            __syncwarp();
            // lane l owns digits 255-8l .. 248-8l, walked from the top
            uint32_t mine = 0;
#pragma unroll
            for (int b = 0; b < 8; b++) mine += sh.closer_hist[255 - 8 * lane - b];
            uint32_t incl = mine;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t up = __shfl_up_sync(kFullMask, incl, d);
                if (lane >= (uint32_t)d) incl += up;
            }
            const unsigned reached = __ballot_sync(kFullMask, incl >= need);
            const int owner = __ffs(reached) - 1;  // need <= live, so some lane reaches it
            uint32_t digit = 0, rest = 0, bucket = 0;
            if ((int)lane == owner) {
                uint32_t above = incl - mine;
                for (int b = 0; b < 8; b++) {
                    const uint32_t candidate = 255 - 8 * lane - b;
                    const uint32_t here = sh.closer_hist[candidate];
                    if (above + here >= need) {
                        digit = candidate;
                        rest = need - above;
                        bucket = here;
                        break;
                    }
                    above += here;
                }
            }
            digit = __shfl_sync(kFullMask, digit, owner);
            rest = __shfl_sync(kFullMask, rest, owner);
            bucket = __shfl_sync(kFullMask, bucket, owner);
            prefix = (prefix << 8) | digit;
            need = rest;
            __syncwarp();
            if (bucket == need || shift == 0) break;
            shift -= 8;
        }
    }
    // unsorted survivors go to the far end of the work arrays, the sort brings them forward
    float *loose_score = reinterpret_cast<float *>(sh.fin.raw);
    uint32_t *loose_id = reinterpret_cast<uint32_t *>(sh.fin.tempered);
    if (lane == 0) sh.closer_count = 0;
    __syncwarp();
    for (uint32_t i = lane; i < entries; i += 32) {
        const uint64_t key = list_key(L, held, i);
        if (key == 0) continue;
        // shift == 64: everything live is kept; otherwise compare the examined bits
        const bool take = shift == 64 || (key >> shift) >= prefix;
        if (take) {
            const uint32_t slot = atomicAdd(&sh.closer_count, 1u);
            if (slot < (uint32_t)kMaxK) {
                const bool from_cand = i < held;
                loose_score[slot] = from_cand ? L.cand.score[i] : L.defer_raw[i - held];
                loose_id[slot] = from_cand ? L.cand.id[i] : L.defer_id[i - held];
            }
        }
    }
    __syncwarp();
    const uint32_t kept = min(sh.closer_count, keep);
    float my_score[2];
    uint32_t my_id[2], my_rank[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint32_t e = lane + 32 * h;
        my_rank[h] = kPaddingId;
        if (e < kept) {
            my_score[h] = loose_score[e];
            my_id[h] = loose_id[e];
            uint32_t rank = 0;
            for (uint32_t j = 0; j < kept; j++) rank += precedes(loose_score[j], loose_id[j], my_score[h], my_id[h]) ? 1u : 0u;
            my_rank[h] = rank;
        }
    }
    __syncwarp();
#pragma unroll
    for (int h = 0; h < 2; h++) {
        if (my_rank[h] != kPaddingId) {
            sh.fin.score[my_rank[h]] = my_score[h];
            sh.fin.id[my_rank[h]] = my_id[h];
        }
    }
    __syncwarp();

    return kept;
}

// A unit's lists become its part of the row's result; the CTA that finishes a row's last
// part merges the parts and writes the result.
__device__ __noinline__ void close_unit(Shared &sh, Lists &L, const Params &p, const Unit u, const Row r,
                                        const SamplerConfig cfg, bool shard_mode) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t row = u.row;
    uint32_t kept = settle_lists(sh, L, r);
    uint32_t bad_history = L.bad_history;
    if (peek(&sh.ring_error)) bad_history = kErrLimit;  // a tile never landed
    uint32_t wild_id = (uint32_t)(L.wild_key >> 32);  // the padding id when nothing was seen
    uint32_t wild_bits = (uint32_t)L.wild_key;
    if (u.parts > 1) {
        const size_t mine = (size_t)row * p.max_parts + u.part;
        for (uint32_t i = lane; i < (uint32_t)kMaxK; i += 32) {
            p.part_scores[mine * kMaxK + i] = i < kept ? sh.fin.score[i] : 0.0f;
            p.part_ids[mine * kMaxK + i] = i < kept ? sh.fin.id[i] : kPaddingId;
        }
        if (lane == 0) {
            PartRecord record;
            record.count = kept;
            record.wild_id = wild_id;
            record.wild_bits = wild_bits;
            record.bad_history = bad_history;
            p.part_meta[mine] = record;
        }
        __threadfence();
        __syncwarp();
        uint32_t ticket = 0;
        if (lane == 0) ticket = atomicAdd(&p.tickets[row], 1u);
        ticket = __shfl_sync(kFullMask, ticket, 0);
        if (ticket != u.parts - 1) return;  // somebody else finishes the row
        __threadfence();
        if (lane == 0) p.tickets[row] = 0;  // ready for the next launch
        // every part's survivors into this slot's candidate list (parts * kMaxK <= kCandCap)
        uint32_t total = 0;
        bad_history = 0;
        wild_id = kPaddingId;
        wild_bits = 0;
        for (uint32_t j = 0; j < u.parts; j++) {
            const size_t from = (size_t)row * p.max_parts + j;
            const uint4 packed = __ldcg(reinterpret_cast<const uint4 *>(&p.part_meta[from]));
            const uint32_t count = min(packed.x, (uint32_t)kMaxK);
            for (uint32_t i = lane; i < count; i += 32) {
                L.cand.score[total + i] = __ldcg(&p.part_scores[from * kMaxK + i]);
                L.cand.id[total + i] = __ldcg(&p.part_ids[from * kMaxK + i]);
            }
            total += count;
            if (packed.w) bad_history = packed.w;
            if (packed.y < wild_id) {
                wild_id = packed.y;
                wild_bits = packed.z;
            }
        }
        if (lane == 0) {
            L.cand.count = total;
            L.defer_count = 0;
        }
        __syncwarp();
        kept = settle_lists(sh, L, r);
    }
    // ---- the row's result ----
    if (shard_mode) {
        for (uint32_t i = lane; i < r.k; i += 32) {
            const size_t at = (size_t)row * r.k + i;
            const bool ok = i < kept && !bad_history;
            p.shard_scores[at] = ok ? sh.fin.score[i] : __uint_as_float(0xff800000u);
            p.shard_ids[at] = ok ? sh.fin.id[i] : kPaddingId;
        }
        if (lane == 0) {
            p.out.row_status[row] = bad_history;
            if (bad_history) atomicMin(p.out.first_error, ((unsigned long long)row << 8) | bad_history);
        }
        return;
    }
    if (bad_history) {  // "history token ... is outside vocabulary", src/output.c:610-612
        if (lane == 0) {
            report_row(p.out, row, bad_history, kPaddingId, 0.0f);
            if (p.out.dbg_count) p.out.dbg_count[row] = 0;
        }
        return;
    }
    if (r.greedy) {
        if (lane == 0) {
            uint32_t status = kOk, token;
            float logit;
            if (wild_id != kPaddingId) {
                // a NaN/Inf beats every finite logit in the argmax order and is then
                // rejected: src/output.c:593 (no penalties) / 737-739 (penalised)
                status = penalties_active(cfg) ? kErrFormat : kErrMismatch;
                token = wild_id;
                logit = __uint_as_float(wild_bits);
            } else if (kept == 0) {
                status = kErrMismatch;
                token = kPaddingId;
                logit = 0.0f;
            } else {
                token = sh.fin.id[0];
                logit = sh.fin.score[0];
            }
            report_row(p.out, row, status, token, logit);
            if (p.out.dbg_count) {
                const bool ok = status == kOk;
                p.out.dbg_count[row] = ok ? 1u : 0u;
                if (p.out.dbg_ids) p.out.dbg_ids[(size_t)row * kMaxK] = ok ? token : kPaddingId;
                if (p.out.dbg_scores) p.out.dbg_scores[(size_t)row * kMaxK] = ok ? logit : 0.0f;
            }
        }
        return;
    }
    finish_select(sh.fin, kept, cfg, p.uniforms[row], row, p.out);
}

#ifdef FGK_PHASE_CLOCKS
__device__ unsigned long long fgk_persist_clocks[8];
#define FGK_PTICK(slot)                                                            \
    do {                                                                            \
        if (threadIdx.x == 0) {                                                     \
            const long long now = clock64();                                        \
            atomicAdd(&fgk_persist_clocks[slot], (unsigned long long)(now - tick)); \
            tick = now;                                                             \
        }                                                                           \
    } while (0)
#else
#define FGK_PTICK(slot) do { } while (0)
#endif

// The row as the consumers and the closing warp see it; *bad_history is the status a
// broken history earns the row (0 when it is fine).
__device__ __forceinline__ Row make_row(const Params &p, const SamplerConfig &cfg, uint32_t row,
                                        bool shard_mode, uint32_t *bad_history) {
    Row r;
    r.greedy = !shard_mode && cfg.temperature == 0.0f;
    r.k = shard_mode ? p.shard_k : (r.greedy ? 1u : cfg.top_k);
#ifndef FGK_PERSIST_CUT_AT
#define FGK_PERSIST_CUT_AT (4 * r.k + 64)
#endif
    r.cut_at = FGK_PERSIST_CUT_AT;
    r.id_base = p.vocab_offset;
    r.flat_offset = penalty_offset(1u, cfg.presence_penalty, cfg.frequency_penalty);
    r.presence = cfg.presence_penalty;
    r.frequency = cfg.frequency_penalty;
    r.repetition = make_repetition(cfg.repetition_penalty);
    r.tokens = nullptr;
    r.history_len = 0;
    *bad_history = 0;
    if (p.history_tokens != nullptr && p.history_offsets != nullptr && p.bitmap_words != 0 &&
        penalties_active(cfg)) {
        const uint64_t begin = p.history_offsets[row], end = p.history_offsets[row + 1];
        if (end < begin || end - begin > p.history_max) {
            *bad_history = kErrLimit;
        } else {
            r.tokens = p.history_tokens + begin;
            r.history_len = (uint32_t)(end - begin);
        }
    }
    r.seen_any = r.history_len != 0;
    r.with_counts = r.seen_any && cfg.frequency_penalty != 0.0f;
    // the host sends only rows whose penalties cannot raise a logit; a row that
    // slipped through is failed rather than sampled wrongly
    if (r.seen_any && !(cfg.presence_penalty >= 0.0f && cfg.frequency_penalty >= 0.0f &&
                        cfg.repetition_penalty >= 1.0f && r.repetition.tame))
        *bad_history = kErrLimit;
    return r;
}

// Does this kernel sample the row, or is it left to the kernel without a top-k cut?
__device__ __forceinline__ bool row_is_ours(const SamplerConfig &cfg, bool shard_mode) {
    return shard_mode || cfg.temperature == 0.0f || cfg.top_k != 0;
}

template <typename T>
__global__ void __launch_bounds__(kBlock, FGK_PERSIST_CTAS)
persistent_select_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(128) unsigned char dynamic[];
    __shared__ Shared sh;
    unsigned char *ring = dynamic;
    uint32_t *bitmap = reinterpret_cast<uint32_t *>(dynamic + (size_t)kStages * kStageBytes);

    const uint32_t tid = threadIdx.x;
    const bool shard_mode = p.shard_k != 0;
    const uint32_t row_bytes = p.vocab * (uint32_t)sizeof(T);
    const uint32_t tiles = (row_bytes + kStageBytes - 1) / kStageBytes;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kStages; s++) {
            mbarrier_init(&sh.full[s], 1);
            mbarrier_init(&sh.empty[s], kConsumerWarps);
        }
        for (int b = 0; b < 2; b++) {
            mbarrier_init(&sh.ready[b], 1);
            mbarrier_init(&sh.vacant[b], 1);
        }
        mbarrier_fence_init();
        sh.ring_error = 0;
    }
    __syncthreads();

    if (tid >= (uint32_t)kConsumers + 32u) {
        // ------------------------------------------------------------- closing warp
        uint32_t served = 0;
        UnitWalk walk(p, tiles);
        Unit u;
        while (walk.next(u)) {
            const SamplerConfig cfg = p.config_count > 1 ? p.configs[u.row] : p.config0;
            if (!row_is_ours(cfg, shard_mode)) continue;
            uint32_t bad_history;
            const Row r = make_row(p, cfg, u.row, shard_mode, &bad_history);
            const uint32_t b = served & 1u;
            // (a wait that runs out leaves garbage lists: the row is failed through ring_error)
            if (!peek(&sh.ring_error) && !bounded_wait(&sh.ready[b], (served >> 1) & 1u))
                poke(&sh.ring_error, 1u);
            __syncwarp();
            close_unit(sh, sh.lists[b], p, u, r, cfg, shard_mode);
            __syncwarp();
            if ((tid & 31u) == 0) mbarrier_arrive(&sh.vacant[b]);
            served++;
        }
        return;
    }
    if (tid >= (uint32_t)kConsumers) {
        // ---------------------------------------------------------------- copy warp
        if (tid != (uint32_t)kConsumers) return;
        const uint64_t policy = l2_policy_evict_first();
        RingCursor cursor;
        bool gave_up = false;
        UnitWalk walk(p, tiles);
        Unit u;
        while (!gave_up && walk.next(u)) {
            const SamplerConfig cfg = p.config_count > 1 ? p.configs[u.row] : p.config0;
            if (!row_is_ours(cfg, shard_mode)) continue;
            const unsigned char *source =
                static_cast<const unsigned char *>(p.logits) + (size_t)u.row * p.row_stride * sizeof(T);
            for (uint32_t t = u.first; t < u.end; t++) {
                if (cursor.use != 0 && !bounded_wait(&sh.empty[cursor.stage], (cursor.use - 1u) & 1u)) {
                    sh.ring_error = 1;  // the consumers see it and fail their rows
                    gave_up = true;
                    break;
                }
                const uint32_t bytes = min(kStageBytes, row_bytes - t * kStageBytes);
                mbarrier_expect(&sh.full[cursor.stage], bytes);
                bulk_copy_to_shared_hinted(ring + (size_t)cursor.stage * kStageBytes,
                                           source + (size_t)t * kStageBytes, bytes,
                                           &sh.full[cursor.stage], policy);
                cursor.advance();
            }
        }
        if (gave_up) {
            // copies already asked for still write into this CTA's shared memory: see them
            // land (bounded) before the CTA may go away
            for (int s = 0; s < kStages; s++) {
                const uint32_t issued = cursor.use + ((uint32_t)s < cursor.stage ? 1u : 0u);
                if (issued != 0) bounded_wait(&sh.full[s], (issued - 1u) & 1u);
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    const uint32_t lane = tid & 31u;
    uint32_t consumed = 0;      // tiles of earlier units
    uint32_t served = 0;        // units before this one
#ifdef FGK_PHASE_CLOCKS
    long long tick = clock64();
#endif
    UnitWalk walk(p, tiles);
    Unit u;
    while (walk.next(u)) {
        const uint32_t row = u.row;
        const SamplerConfig cfg = p.config_count > 1 ? p.configs[row] : p.config0;
        if (!row_is_ours(cfg, shard_mode)) continue;
        uint32_t bad_history;
        const Row r = make_row(p, cfg, row, shard_mode, &bad_history);
        // tile t of the row is ring tile row_sequence + t (unsigned arithmetic wraps as it should)
        const uint32_t row_sequence = consumed - u.first;
        const uint32_t b = served & 1u;
        Lists &L = sh.lists[b];
        // the closing warp must be done with these lists (it had them two rows ago)
        if (served >= 2u && !peek(&sh.ring_error) && !bounded_wait(&sh.vacant[b], ((served >> 1) - 1u) & 1u))
            poke(&sh.ring_error, 1u);
        if (tid == 0) {
            L.cand.count = 0;
            L.cand.tau_score = __uint_as_float(0xff800000u);
            L.cand.tau_id = kPaddingId;
            L.defer_count = 0;
            L.bad_history = bad_history;
            L.wild_key = ~0ull;
            sh.first_key = 0xffffffffu;
            sh.attention = 0;
            sh.through[b] = 0;
        }
        FGK_PTICK(5);
        if (r.seen_any) build_bitmap(L, bitmap, p, r);
        else CB::sync();
        FGK_PTICK(0);

        const uint32_t last_vectors = (row_bytes - (tiles - 1) * kStageBytes) / 16u;
        // ---- the unit's first tile, all warps together ----
        const uint32_t at0 = consumed % kStages;
        if (!peek(&sh.ring_error) && !bounded_wait(&sh.full[at0], (consumed / kStages) & 1u))
            poke(&sh.ring_error, 1u);
        float tau = first_tile<T>(sh, L, bitmap, ring + (size_t)at0 * kStageBytes, u.first,
                                  u.first + 1 == tiles ? last_vectors : kStageBytes / 16u, r);
        __syncwarp();
        if (lane == 0) mbarrier_arrive(&sh.empty[at0]);
        FGK_PTICK(1);

        // ---- the further tiles: each warp at its own pace ----
        // (a row's last tile may hold fewer than a stage's worth: it takes the variant of
        // the loop that checks, everything before it the one that does not)
        const uint32_t whole = kStageBytes / 16u;
        const uint32_t plain_end = (u.end == tiles && last_vectors != whole) ? u.end - 1 : u.end;
        for (uint32_t t = u.first + 1; t < u.end;) {
            const bool ragged = t >= plain_end;
            Stop stop;
            if (ragged)
                stop = r.greedy ? hot_tiles<T, true, true>(sh, L, bitmap, ring, t, u.end, last_vectors, row_sequence, r, tau)
                                : hot_tiles<T, false, true>(sh, L, bitmap, ring, t, u.end, last_vectors, row_sequence, r, tau);
            else
                stop = r.greedy ? hot_tiles<T, true, false>(sh, L, bitmap, ring, t, plain_end, whole, row_sequence, r, tau)
                                : hot_tiles<T, false, false>(sh, L, bitmap, ring, t, plain_end, whole, row_sequence, r, tau);
            t = stop.tile;
            if (stop.why == kStopDone) continue;  // on to the ragged tile, or out
            if (stop.why == kStopBefore) {
                FGK_PTICK(2);
                tau = attend(sh, L, r);
                FGK_PTICK(3);
#ifdef FGK_PHASE_CLOCKS
                if (tid == 0) atomicAdd(&fgk_persist_clocks[7], 1ull);
#endif
                continue;
            }
            const uint32_t at = (row_sequence + t) % kStages;
            const unsigned char *stage = ring + (size_t)at * kStageBytes;
            tau = r.greedy ? settle<T, true>(sh, L, r, bitmap, stage, t, stop.pending, tau)
                           : settle<T, false>(sh, L, r, bitmap, stage, t, stop.pending, tau);
            __syncwarp();
            if (lane == 0) mbarrier_arrive(&sh.empty[at]);
            t++;
        }
        FGK_PTICK(2);
        // ---- the end of the row ----
        // A call to attend() that is up must be answered by every warp, so a warp answers
        // what it sees before it counts itself through, and keeps answering until all
        // eight are through: from then on nobody can call.  The last one through hands
        // the lists to the closing warp.
        while (__any_sync(kFullMask, peek(&sh.attention) != 0)) attend(sh, L, r);
        __threadfence_block();
        __syncwarp();
        uint32_t through = 0;
        if (lane == 0) through = atomicAdd(&sh.through[b], 1u) + 1u;
        through = __shfl_sync(kFullMask, through, 0);
        if (through == (uint32_t)kConsumerWarps) {
            if (lane == 0) mbarrier_arrive(&sh.ready[b]);
        } else {
            for (;;) {
                if (__any_sync(kFullMask, peek(&sh.attention) != 0)) attend(sh, L, r);
                else if (__any_sync(kFullMask, peek(&sh.through[b]) == (uint32_t)kConsumerWarps)) break;
                else __nanosleep(100);  // leave the issue slots to the warps that still work
            }
        }
        FGK_PTICK(4);
        consumed += u.end - u.first;
        served++;
    }
}

}  // namespace persist
}  // namespace fgk

// ------------------------------------------------------------------ host side

#ifdef FGK_PHASE_CLOCKS
extern "C" int fgk_read_persist_clocks(unsigned long long *out, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out, fgk::persist::fgk_persist_clocks, sizeof(unsigned long long) * 8);
    if (e == cudaSuccess && reset) {
        unsigned long long zero[8] = {0};
        e = cudaMemcpyToSymbol(fgk::persist::fgk_persist_clocks, zero, sizeof(zero));
    }
    return (int)e;
}
#endif

using namespace fgk;

static persist::Params to_persist_params(const fgk_stream_launch *l) {
    persist::Params p;
    p.logits = l->logits;
    p.row_stride = l->row_stride;
    p.rows = l->rows;
    p.vocab = l->vocab;
    p.vocab_offset = l->vocab_offset;
    p.vocab_total = l->vocab_total;
    p.history_tokens = l->history_tokens;
    p.history_offsets = l->history_offsets;
    p.history_max = l->history_max;
    p.bitmap_words = l->bitmap_words;
    p.configs = static_cast<const SamplerConfig *>(l->configs_device);
    static_assert(sizeof(fg_sampler_config) == sizeof(SamplerConfig), "config layout");
    memcpy(&p.config0, &l->config0, sizeof(SamplerConfig));
    p.config_count = l->config_count;
    p.shard_k = l->shard_k;
    p.uniforms = l->uniforms;
    p.shard_scores = l->shard_scores;
    p.shard_ids = l->shard_ids;
    p.tiles_per_cta = l->split_len;  /* reused: tiles per CTA */
    p.max_parts = l->splits;         /* reused: most CTAs per row */
    p.part_scores = l->part_scores;
    p.part_ids = l->part_ids;
    p.part_meta = static_cast<persist::PartRecord *>(l->part_meta);
    p.tickets = l->tickets;
    p.out.tokens = l->out.tokens;
    p.out.token_logits = l->out.token_logits;
    p.out.row_status = l->out.row_status;
    p.out.first_error = reinterpret_cast<unsigned long long *>(l->out.first_error);
    p.out.dbg_count = l->out.dbg_count;
    p.out.dbg_ids = l->out.dbg_ids;
    p.out.dbg_scores = l->out.dbg_scores;
    p.out.dbg_raw = l->out.dbg_raw;
    p.out.dbg_tempered = l->out.dbg_tempered;
    return p;
}

extern "C" uint64_t fgk_persistent_dynamic_smem(uint32_t bitmap_words) {
    return (uint64_t)persist::kStages * persist::kStageBytes + (((uint64_t)bitmap_words + 3u) / 4u) * 16u;
}

// 16 KB tiles in a row of `vocab` logits.
extern "C" uint32_t fgk_persistent_row_tiles(uint32_t dtype, uint32_t vocab) {
    const uint64_t bytes = (uint64_t)vocab * (dtype == 1u ? 2u : 4u);
    return (uint32_t)((bytes + persist::kStageBytes - 1) / persist::kStageBytes);
}

// Most parts of one row the merge can take (parts * 64 survivors fit one candidate list).
extern "C" uint32_t fgk_persistent_max_parts(void) { return persist::kCandCap / kMaxK; }

extern "C" uint32_t fgk_persistent_ctas_per_sm(uint32_t dtype, uint64_t dynamic_smem) {
    int blocks = 0;
    const cudaError_t e =
        dtype == 0 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                         &blocks, persist::persistent_select_kernel<float>, persist::kBlock, (size_t)dynamic_smem)
                   : cudaOccupancyMaxActiveBlocksPerMultiprocessor(
                         &blocks, persist::persistent_select_kernel<uint16_t>, persist::kBlock, (size_t)dynamic_smem);
    return e == cudaSuccess && blocks > 0 ? (uint32_t)blocks : 0u;
}

extern "C" int fgk_persistent_prepare(void) {
    cudaError_t e = cudaFuncSetAttribute(persist::persistent_select_kernel<float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FGK_PERSIST_MAX_DYNAMIC_SMEM);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(persist::persistent_select_kernel<uint16_t>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, FGK_PERSIST_MAX_DYNAMIC_SMEM);
    return (int)e;
}

extern "C" int fgk_launch_persistent_select(const fgk_stream_launch *l, uint32_t ctas, void *stream) {
    const persist::Params p = to_persist_params(l);
    const size_t dynamic = (size_t)fgk_persistent_dynamic_smem(l->bitmap_words);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (l->dtype == 0)
        persist::persistent_select_kernel<float><<<ctas, persist::kBlock, dynamic, s>>>(p);
    else
        persist::persistent_select_kernel<uint16_t><<<ctas, persist::kBlock, dynamic, s>>>(p);
    return (int)cudaGetLastError();
}
