// Persistent sampling kernel for sm_100a: one CTA per SM, warps that never meet.
//
// A CTA works through its rows (or its shares of rows) one after the other.  Inside it
//
//   8 consumer warps    each owns a private pair of 8 KB stages in shared memory and asks
//                       the copy engine itself (cp.async.bulk + mbarrier) for every 8th
//                       2048-logit tile of the row: as soon as a stage has been looked at
//                       it is asked to fetch the warp's next tile -- of this row or the
//                       next -- so 64 KB are always on their way to the SM and no warp ever
//                       waits for another one's tile.  Per tile and lane: sixteen 128-bit
//                       shared loads, a maximum and one compare per vector; single elements
//                       are looked at only at or above the admission bound and go to the
//                       warp's own candidate list.
//   2 history warps     build the bitmaps of the next rows' token histories, up to three rows
//                       ahead, while the consumers stream the current row.  (A CTA's first
//                       bitmap is everybody's work: the consumers have nothing to read yet.)
//   2 closing warps     turn the lists of a finished row into its result (exact k best, the
//                       select step of src/sampler.c:80-122), taking rows in turn, while
//                       the consumers fill another of the three sets of lists.
//
// The warps of a row share one number, the admission bound: a 64-bit (score, ~id) key T
// such that at least k elements of the row are known to have a key >= T.  It starts from
// the warps' first tiles (each publishes the j-th largest of its lanes' maxima over ids
// the history has not seen, j = ceil(k / warps); the smallest of them bounds k elements).
// From then on every entry that goes on a list with its exact value is counted in a tally
// by score (256 bins between the first bound and the largest score of the first tiles); after
// every round of tiles one warp reads the tally and lifts the bound to the lower edge of the
// highest bin that, with the bins above it, holds k entries.  A row that wants a single
// candidate lifts the bound to every better candidate directly.  A stale bound is still a
// bound, so nobody waits for anybody after the first tile.
//
// The kernel takes rows whose penalties can only lower a logit (presence >= 0,
// frequency >= 0, repetition >= 1, or no penalties / no history at all).  Then a raw
// value below the bound stays below, so the history matters only for the few values
// at or above it.  An id that was seen is charged  frequency * count + presence
// (src/sampler.c:52-58); the count is not tabulated per row (src/output.c:601-617 keeps a
// vocabulary-wide table per session): the entry keeps its raw logit, is ordered by the
// charge for count = 1 -- an upper bound of its value -- and its occurrences are counted
// in the token list only if that upper bound reaches the bound the row ends with.
// Everything else (penalties that can raise a logit, rows that are not 16-byte aligned,
// column splits) stays with stream_select_kernel.
#include <cstring>

#include "fg_block_select.cuh"
#include "fg_kernels.h"

namespace fgk {
namespace persist {

constexpr int kWarps = 8;                       // consumer warps
constexpr int kHistoryWarps = 2;
constexpr int kClosers = 2;
constexpr int kStages = 2;                      // stages per consumer warp: one tile being looked at, one on its way
constexpr uint32_t kTileLogits = 2048;          // logits per tile: at most 64 per lane, a bit each in a mask
constexpr uint32_t kStageBytes = kTileLogits * 4;  // a stage holds a tile of the widest type
constexpr int kListCap = 128;                   // entries of one warp's candidate list (a multiple of 32, > 64)
constexpr int kListWords = kListCap / 32;
constexpr int kListSets = 3;                    // units whose lists exist at a time: one being filled, two being closed
constexpr int kTallyBins = 256;                 // bins of the per-unit score tally (eight per lane)
constexpr int kBlock = (kWarps + kHistoryWarps + kClosers) * 32;
constexpr uint32_t kDefaultPolls = 1u << 21;    // polls before a wait gives up: a second or two
constexpr uint32_t kNapNanoseconds = 400;       // sleep between two polls of a wait that may be long
constexpr uint32_t kHugeBits = 0x6b000000u;     // |x| >= 2^87: a repetition factor <= 2^40 may reach inf
constexpr uint32_t kSharedLimit = 227u * 1024u; // shared memory one CTA may ask for

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
// A tile is kTileLogits logits whatever their type: 8 KB of fp32, 4 KB of bf16.
template <typename T>
__host__ __device__ constexpr uint32_t tile_bytes() { return kTileLogits * (uint32_t)sizeof(T); }
template <typename T>
__host__ __device__ constexpr int tile_vectors() { return (int)(tile_bytes<T>() / 16u / 32u); }  // 128-bit vectors per lane

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
    uint32_t bitmap_buffers;        // 3 or 2: the next rows' bitmaps are built ahead; 1: no room for that
    const SamplerConfig *configs;   // device copy when config_count > 1
    SamplerConfig config0;
    uint32_t config_count;
    uint32_t shard_k;               // != 0: write candidates instead of sampling
    const float *uniforms;
    float *shard_scores;
    uint32_t *shard_ids;
    uint32_t shard_stride;          // elements between consecutive candidates (2: interleaved pairs)
    PushTargets push;               // ranks != 0: candidates go straight to every rank's window
    // Work is dealt out in 4 KB tiles: CTA c takes tiles [c * tiles_per_cta, (c + 1) *
    // tiles_per_cta) of the batch's tile sequence (row after row), so a row may be shared
    // by several CTAs.  Each leaves its part's k best in `parts`; the last to finish
    // (ticket counter) merges them.
    // With enough rows for every CTA to have several, whole rows are dealt out instead
    // (tiles_per_cta == 0): CTA c takes rows c, c + ctas, c + 2 * ctas, ...
    uint32_t tiles_per_cta;
    uint32_t max_parts;             // most CTAs that share one row
    float *part_scores;             // [rows][max_parts][kMaxK]
    uint32_t *part_ids;
    PartRecord *part_meta;          // [rows][max_parts]
    uint32_t *tickets;              // [rows], zero between launches
    // Session tables instead of token lists (the stateful executor): row r uses the counts and
    // the seen-bitmap of session row_slots[r], both indexed by token id; vocab_offset is 0.
    const uint32_t *slot_counts;    // [slots][vocab]
    const uint32_t *slot_bitmaps;   // [slots][slot_bitmap_words], a whole number of uint4 each
    const uint32_t *row_slots;      // [rows]
    uint32_t slot_bitmap_words;
    uint32_t wait_polls;            // polls before a wait gives up
    uint32_t withhold_cta, withhold_issue;  // test seam: that CTA's warp 0 never asks for that tile
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

// What the consumers collect for one unit: one private list per warp.  There are three of
// these: while the closing warps turn two into results the consumers fill the third.
// An entry is (score, id); when its bit in `deferred` is up the score is the RAW logit of
// an id the history has seen, whose occurrences have not been counted yet.  An entry whose
// id is the padding id is dead.
struct alignas(16) Lists {
    float score[kWarps][kListCap];
    uint32_t id[kWarps][kListCap];
    uint32_t deferred[kWarps][kListWords];
    uint32_t count[kWarps];                 // slots handed out (may run past kListCap)
    unsigned long long wild_key[kWarps];    // greedy rows: min over NaN/Inf of (id << 32 | value bits)
    unsigned long long bound;               // the admission bound T (only ever rises)
    uint32_t first_key;                     // smallest of the warps' first-tile keys
    uint32_t first_count;                   // warps that have published theirs
    uint32_t first_top;                     // largest score of the first tiles, as a key
    uint32_t bad_history;
    uint32_t tally[kTallyBins];             // exact entries by score, see Tally
};

struct Shared {
    FinishBuffer fin[kClosers];              // the closing warps'
    uint32_t hist[kClosers][256];
    uint32_t gathered[kClosers];
    alignas(8) uint64_t full[kWarps][kStages];  // "the tile has landed"
    alignas(8) uint64_t ready[kListSets];    // "every consumer warp is through with the unit"
    alignas(8) uint64_t vacant[kListSets];   // "the closing warp is done with the lists"
    alignas(8) uint64_t bitmap_ready[3];     // "the unit's history bitmap is complete"
    alignas(8) uint64_t bitmap_free[3];      // "every consumer warp is through with the bitmap buffer"
    uint32_t history_bad[3];                 // status a broken history earns the unit, by bitmap buffer
    uint32_t ring_error;                     // a bounded wait ran out
};

// What the warps need to know about the row; lives in registers.
struct Row {
    const uint32_t *tokens;  // the row's history
    const uint32_t *counts;        // or: its session's count table (then tokens is null)
    const uint32_t *table_bitmap;  //     and its session's seen-bitmap in global memory
    uint32_t history_len;
    uint32_t id_base;        // global id of column 0
    uint32_t k;
    float flat_offset;       // charge for count = 1 (the exact charge when frequency is +-0)
    float presence, frequency;
    Repetition repetition;
    bool greedy, seen_any, with_counts;
};

// Shared words that warps watch while others change them.
__device__ __forceinline__ uint32_t peek(const uint32_t *word) {
    return *reinterpret_cast<const volatile uint32_t *>(word);
}
__device__ __forceinline__ unsigned long long peek64(const unsigned long long *word) {
    return *reinterpret_cast<const volatile unsigned long long *>(word);
}
__device__ __forceinline__ void poke(uint32_t *word, uint32_t value) {
    *reinterpret_cast<volatile uint32_t *>(word) = value;
}

// Waits for a phase of an mbarrier, at most `polls` polls with a short sleep between them, and
// not at all once another wait of the CTA has run out.  A wait that runs out raises
// ring_error: the CTA's rows then end with FG_ERR_LIMIT and every later wait returns at
// once, so the kernel always comes back.
__device__ __forceinline__ bool bounded_wait(Shared &sh, uint64_t *barrier, uint32_t parity, uint32_t polls) {
    for (uint32_t i = 0; i < polls; i++) {
        if (mbarrier_try_wait(barrier, parity)) return true;
        if (peek(&sh.ring_error) != 0) return false;
        __nanosleep(kNapNanoseconds);  // (the warps that stream need the issue slots)
    }
    poke(&sh.ring_error, 1u);
    return false;
}

// The same for a tile that is on its way: the warp wants it the moment it lands.
__device__ __forceinline__ bool tile_wait(Shared &sh, uint64_t *barrier, uint32_t parity, uint32_t polls) {
    for (uint32_t i = 0; i < polls; i++) {
        if (mbarrier_try_wait(barrier, parity)) return true;
        if ((i & 15u) == 15u && peek(&sh.ring_error) != 0) return false;
    }
    poke(&sh.ring_error, 1u);
    return false;
}


__device__ __forceinline__ uint64_t warp_max_u64(uint64_t v) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const uint64_t other = __shfl_xor_sync(kFullMask, v, d);
        v = other > v ? other : v;
    }
    return v;
}
__device__ __forceinline__ uint64_t warp_min_u64(uint64_t v) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        const uint64_t other = __shfl_xor_sync(kFullMask, v, d);
        v = other < v ? other : v;
    }
    return v;
}

// Largest of three; a NaN loses against a number, as with fmaxf.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// max(m, v...) that turns NaN as soon as one operand is NaN.
template <int N>
__device__ __forceinline__ float propagating_max(float m, const float (&v)[N]) {
#pragma unroll
    for (int i = 0; i < N; i++) asm("max.NaN.f32 %0, %0, %1;" : "+f"(m) : "f"(v[i]));
    return m;
}

// Smallest of N values; a NaN loses against a number, as with fminf.
template <int N>
__device__ __forceinline__ float smallest(const float (&v)[N]) {
    float m = v[0];
#pragma unroll
    for (int i = 1; i < N; i++) m = fminf(m, v[i]);
    return m;
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

// One logit of a tile in shared memory, by its position in the tile.
template <typename T>
__device__ __forceinline__ float tile_element(const unsigned char *tile, uint32_t position);
template <>
__device__ __forceinline__ float tile_element<float>(const unsigned char *tile, uint32_t position) {
    return reinterpret_cast<const float *>(tile)[position];
}
template <>
__device__ __forceinline__ float tile_element<uint16_t>(const unsigned char *tile, uint32_t position) {
    return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t *>(tile)[position] << 16);
}

// Key of entry i of warp w's list: its exact (score, ~id) key, or -- for an entry whose
// occurrences are not counted yet -- the key of the most it can be worth.  0 = dead.
__device__ __forceinline__ uint64_t entry_key(const Lists &L, const Row &r, uint32_t w, uint32_t i, bool deferred) {
    const uint32_t id = L.id[w][i];
    if (id == kPaddingId) return 0ull;
    float s = L.score[w][i];
    if (deferred) {
        s = penalise_with_offset(s, r.flat_offset, r.repetition);
        if (is_nonfinite(s)) return ~0ull;  // (greedy rows keep these to report them)
    }
    return select_key(s, id);
}

// What becomes of one element whose raw value reaches the bound's score (or, in a greedy
// row, is NaN/Inf/huge): 0 it cannot be among the k best, 1 it goes on the list with its
// exact value (returned in *value), 2 it goes on the list with its raw logit because its
// occurrences are not counted yet.  Greedy rows note a NaN/Inf on the way.
template <bool kGreedy>
__device__ __forceinline__ uint32_t classify(Lists &L, const Row &r, uint32_t w, float x, uint32_t id, bool seen,
                                             uint64_t bound, float *value) {
    *value = x;
    if (seen) {
        const float most = penalise_with_offset(x, r.flat_offset, r.repetition);
        if (r.with_counts && r.counts != nullptr) {
            // the session's table holds the exact count: no waiting for a token scan
            const uint32_t seen_times = __ldg(&r.counts[id - r.id_base]);
            x = seen_times == 0 ? x
                : penalise_with_offset(x, penalty_offset(seen_times, r.presence, r.frequency), r.repetition);
            *value = x;
        } else if (r.with_counts) {
            // the charge grows with the count, so `most` is the most the id can keep
            const bool alive = !is_nonfinite(most) && select_key(most, id) >= bound;
            // greedy rows must also see NaN/Inf, raw or made by the penalty
            const bool wild = kGreedy && (__float_as_uint(x) & 0x7fffffffu) >= kHugeBits;
            return alive || wild ? 2u : 0u;
        } else {
            x = most;
            *value = most;
        }
    }
    if (is_nonfinite(x)) {
        if (kGreedy) atomicMin(&L.wild_key[w], ((unsigned long long)id << 32) | __float_as_uint(x));
        return 0u;
    }
    return select_key(x, id) >= bound ? 1u : 0u;
}

// The same out of line, for the few elements of a tile that need it.
struct Classified {
    uint32_t kind;
    float value;
};
template <bool kGreedy>
__device__ __noinline__ Classified classify_apart(Lists &L, const Row r, uint32_t w, float x, uint32_t id, bool seen,
                                                  uint64_t bound) {
    Classified c;
    c.kind = classify<kGreedy>(L, r, w, x, id, seen, bound, &c.value);
    return c;
}

// Counts the occurrences of the not-yet-counted entries of warp w's list whose upper bound
// reaches `bound`, and gives them their exact value (src/sampler.c:52-58).  An entry the
// penalty turns into NaN/Inf dies (greedy rows note it).  All lanes call; returns how many
// entries it settled.
__device__ __noinline__ uint32_t resolve_above(Lists &L, const Row r, uint32_t w, uint64_t bound) {
    const uint32_t lane = lane_id();
    const uint32_t n = min(L.count[w], (uint32_t)kListCap);
    uint32_t settled = 0;
    for (uint32_t word = 0; word < (uint32_t)kListWords; word++) {
        const uint32_t bits = L.deferred[w][word];
        if (bits == 0) continue;
        const uint32_t i = word * 32 + lane;
        const bool mine = ((bits >> lane) & 1u) != 0 && i < n;
        const uint32_t my_id = mine ? L.id[w][i] : kPaddingId;
        const float my_raw = mine ? L.score[w][i] : 0.0f;
        const bool need = mine && entry_key(L, r, w, i, true) >= bound;
        const uint32_t needs = __ballot_sync(kFullMask, need);
        if (needs == 0) continue;
        uint32_t my_hits = 0;
        constexpr int kBatch = 8;
        for (uint32_t base = 0; base < r.history_len; base += kBatch * 32) {
            uint32_t token[kBatch];
#pragma unroll
            for (int q = 0; q < kBatch; q++) {
                const uint32_t at = base + q * 32 + lane;
                token[q] = at < r.history_len ? r.tokens[at] : kPaddingId;  // the padding id is nobody's
            }
            for (uint32_t rest = needs; rest != 0; rest &= rest - 1) {
                const int owner = __ffs(rest) - 1;
                const uint32_t target = __shfl_sync(kFullMask, my_id, owner);
                uint32_t hits = 0;
#pragma unroll
                for (int q = 0; q < kBatch; q++) hits += token[q] == target ? 1u : 0u;
                hits = __reduce_add_sync(kFullMask, hits);
                if ((int)lane == owner) my_hits += hits;
            }
        }
        if (need) {
            const float exact = my_hits == 0 ? my_raw
                : penalise_with_offset(my_raw, penalty_offset(my_hits, r.presence, r.frequency), r.repetition);
            if (is_nonfinite(exact)) {
                if (r.greedy) atomicMin(&L.wild_key[w], ((unsigned long long)my_id << 32) | __float_as_uint(exact));
                L.id[w][i] = kPaddingId;
            } else {
                L.score[w][i] = exact;
            }
        }
        __syncwarp();
        if (lane == 0) L.deferred[w][word] = bits & ~needs;
        settled += __popc(needs);
        __syncwarp();
    }
    return settled;
}

// A consumer warp whose list is full keeps the exact k best of it (entries whose upper
// bound does not reach them go; the others are settled first) and lifts the row's bound
// to its own k-th best.  All lanes call; returns that key.
__device__ __noinline__ uint64_t local_cut(Lists &L, const Row r, uint32_t w) {
    const uint32_t lane = lane_id();
    uint64_t threshold = 0;
    for (;;) {
        const uint32_t n = min(L.count[w], (uint32_t)kListCap);
        uint64_t key[kListWords];
        uint32_t live = 0;
#pragma unroll
        for (int j = 0; j < kListWords; j++) {
            const uint32_t i = j * 32 + lane;
            const bool exact = i < n && ((L.deferred[w][j] >> lane) & 1u) == 0;
            key[j] = exact ? entry_key(L, r, w, i, false) : 0ull;
            live += key[j] != 0 ? 1u : 0u;
        }
        live = __reduce_add_sync(kFullMask, live);
        threshold = 0;
        if (live > r.k) {
            // the k-th largest key, bit by bit from the top
            for (int bit = 63; bit >= 0; bit--) {
                const uint64_t candidate = threshold | (1ull << bit);
                uint32_t reach = 0;
#pragma unroll
                for (int j = 0; j < kListWords; j++) reach += key[j] >= candidate ? 1u : 0u;
                if (__reduce_add_sync(kFullMask, reach) >= r.k) threshold = candidate;
            }
        }
        if (resolve_above(L, r, w, threshold) == 0) break;
    }
    // keep the exact entries at or above the threshold (what is still uncounted lies below it)
    const uint32_t n = min(L.count[w], (uint32_t)kListCap);
    float score[kListWords];
    uint32_t id[kListWords];
    bool keep[kListWords];
#pragma unroll
    for (int j = 0; j < kListWords; j++) {
        const uint32_t i = j * 32 + lane;
        const bool exact = i < n && ((L.deferred[w][j] >> lane) & 1u) == 0;
        score[j] = exact ? L.score[w][i] : 0.0f;
        id[j] = exact ? L.id[w][i] : kPaddingId;
        const uint64_t key = exact && id[j] != kPaddingId ? select_key(score[j], id[j]) : 0ull;
        keep[j] = key != 0 && key >= threshold;
    }
    __syncwarp();
    uint32_t base = 0;
#pragma unroll
    for (int j = 0; j < kListWords; j++) {
        const uint32_t mask = __ballot_sync(kFullMask, keep[j]);
        if (keep[j]) {
            const uint32_t at = base + __popc(mask & ((1u << lane) - 1u));
            L.score[w][at] = score[j];
            L.id[w][at] = id[j];
        }
        base += __popc(mask);
    }
    if (lane < (uint32_t)kListWords) L.deferred[w][lane] = 0;
    if (lane == 0) {
        L.count[w] = base;
        if (threshold != 0) atomicMax(&L.bound, (unsigned long long)threshold);
    }
    __syncwarp();
    return threshold;
}

// Where the exact entries of a unit lie, by score: bin b counts those whose score key is at
// least base + (b << shift), the last bin everything above.  Once the bins from the top down
// to b hold k entries, the lower edge of bin b bounds the row -- more tightly the further the
// row has been read.  base and top come from the warps' first tiles.
struct Tally {
    uint32_t base;   // score key of the first bound (bin 0 starts here)
    uint32_t shift;
    __device__ __forceinline__ void span(uint32_t low, uint32_t high) {
        base = low;
        const uint32_t range = high > low ? high - low : 0u;
        shift = range < (uint32_t)kTallyBins - 1u ? 0u : 25u - (uint32_t)__clz(range);  // (range >> shift) < 255
    }
    __device__ __forceinline__ uint32_t bin(uint32_t key) const {
        return min((key - base) >> shift, (uint32_t)kTallyBins - 1u);
    }
};

// The first bound of a unit.  Each warp that has a tile publishes the j-th largest of its
// lanes' maxima, j = ceil(k / warps with a tile); a lane whose maximum is not finite, or
// belongs to an id the history has seen (whose value the penalty will lower), publishes
// nothing.  At least j distinct elements of the tile are as large as that key and keep
// their value, so the smallest of the published keys bounds k elements.  (A warp with fewer
// than j such lanes publishes "no bound"; everything finite is then a candidate until some
// list is cut.)  The warp waits until all have published -- a tile's worth of skew at most,
// with the next tiles already on their way.  Returns the bound and the largest score of the
// first tiles, between which the tally is laid out.
struct FirstBound {
    uint32_t key;  // score key of the bound (0: none)
    uint32_t top;  // largest score of the first tiles, as a key
};
template <typename T>
__device__ __noinline__ FirstBound first_bound(Shared &sh, Lists &L, const Row r, const uint32_t *bitmap,
                                               const unsigned char *tile, uint32_t column0,
                                               uint32_t valid_vectors, uint32_t participants, uint32_t polls) {
    using V = Lanes<T>;
    constexpr int kPer = V::kPer;
    constexpr int kVectors = tile_vectors<T>();
    const uint32_t lane = lane_id();
    const uint4 *vectors = reinterpret_cast<const uint4 *>(tile);
    float best = __uint_as_float(0xff800000u);
    uint32_t where = 0;  // the vector that holds the lane's maximum
#pragma unroll
    for (int u = 0; u < kVectors; u++) {
        const uint32_t g = u * 32 + lane;
        if (g >= valid_vectors) continue;
        float v[kPer];
        V::unpack(vectors[g], v);
        const float m = largest(v);  // (a NaN never wins)
        if (m > best) {
            best = m;
            where = g;
        }
    }
    uint32_t key = 0;
    if (!is_nonfinite(best)) {
        // which element it is, and whether the history has seen its id
        float v[kPer];
        V::unpack(vectors[where], v);
        uint32_t j = 0;
#pragma unroll
        for (int e = kPer - 1; e >= 0; e--)
            if (v[e] == best) j = e;
        const uint32_t column = column0 + where * kPer + j;
        const bool seen = r.seen_any && ((bitmap[column >> 5] >> (column & 31u)) & 1u);
        if (!seen) key = float_key(best);
    }
    const uint32_t per_warp = (r.k + participants - 1) / participants;
    const uint32_t top = __reduce_max_sync(kFullMask, key);
    uint32_t kth = per_warp == 1u ? top : 0u;
    if (per_warp > 1u && per_warp <= 32u) {
        for (uint32_t i = 0; i < per_warp; i++) {
            kth = __reduce_max_sync(kFullMask, key);
            if (kth == 0) break;
            const unsigned owners = __ballot_sync(kFullMask, key == kth);
            if ((int)lane == __ffs(owners) - 1) key = 0;
        }
    }
    if (lane == 0) {
        atomicMin(&L.first_key, kth);
        atomicMax(&L.first_top, top);
        // a row that wants one candidate is bounded by the best any warp has seen
        if (r.k == 1u && top != 0) atomicMax(&L.bound, (unsigned long long)top << 32);
        __threadfence_block();
        atomicAdd(&L.first_count, 1u);
    }
    __syncwarp();
    for (uint32_t i = 0;; i++) {
        if (peek(&L.first_count) >= participants || peek(&sh.ring_error) != 0) break;
        if (i >= polls) {
            poke(&sh.ring_error, 1u);
            break;
        }
        __nanosleep(100);
    }
    __threadfence_block();
    FirstBound first;
    first.key = peek(&L.first_key);
    first.top = peek(&L.first_top);
    return first;
}

// The bound the tally allows: the lower edge of the highest bin such that it and the bins above
// it hold k entries.  All lanes call; lane 0 lifts the unit's bound.
__device__ __noinline__ void raise_bound(Lists &L, const Tally tally, uint32_t k) {
    const uint32_t lane = lane_id();
    // lane l owns bins 255-8l .. 248-8l, walked from the top
    uint32_t bins[8];
    uint32_t mine = 0;
#pragma unroll
    for (int b = 0; b < 8; b++) {
        bins[b] = peek(&L.tally[kTallyBins - 1 - 8 * lane - b]);
        mine += bins[b];
    }
    uint32_t incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(kFullMask, incl, d);
        if (lane >= (uint32_t)d) incl += up;
    }
    const unsigned reached = __ballot_sync(kFullMask, incl >= k);
    if (reached == 0) return;
    if ((int)lane == __ffs(reached) - 1) {
        uint32_t over = incl - mine;
        uint32_t bin = kTallyBins - 1 - 8 * lane;
#pragma unroll
        for (int b = 0; b < 8; b++) {
            over += bins[b];
            if (over >= k) break;
            bin--;
        }
        const uint64_t edge = (uint64_t)tally.base + ((uint64_t)bin << tally.shift);
        // (an edge below every finite score is no bound, and its key no number)
        if (edge >= 0x00800000ull && edge <= 0xff7fffffull) atomicMax(&L.bound, (unsigned long long)(edge << 32));
    }
}

// The elements of a tile that reach the bound go on the warp's list.  Only lanes that hold such
// an element look for it, in the vectors the scan marked (`hot`, a bit per vector of the lane),
// and note where (`take`, a bit per element of the lane); then all of them put one element each
// on the list at a time.  An id the history has seen, or a NaN/Inf of a greedy row, is classified
// first; every entry that goes on the list with its exact value lifts the bound (a row that wants
// one candidate) or is counted in the tally.  A list that is full is cut to its k best, which
// lifts the bound too, and the lanes go on where they stopped.  All lanes call; returns the bound
// the warp knows afterwards.
template <typename T, bool kGreedy>
__device__ __noinline__ uint64_t collect(Lists &L, const Row r, const uint32_t *bitmap, const unsigned char *tile,
                                         uint32_t column0, uint32_t valid_vectors, uint32_t w, uint32_t hot,
                                         uint64_t bound, const Tally tally) {
    using V = Lanes<T>;
    constexpr int kPer = V::kPer;
    const uint32_t lane = lane_id();
    const uint4 *vectors = reinterpret_cast<const uint4 *>(tile);
    float tau = key_to_float((uint32_t)(bound >> 32));
    uint64_t take = 0;  // bit u * kPer + j: element j of this lane's vector u
    for (; hot != 0; hot &= hot - 1) {
        const uint32_t u = __ffs(hot) - 1;
        const uint32_t g = u * 32 + lane;
        if (g >= valid_vectors) break;
        float v[kPer];
        V::unpack(vectors[g], v);
        uint32_t bits = 0;
#pragma unroll
        for (int j = 0; j < kPer; j++) {
            const bool wild = kGreedy && (__float_as_uint(v[j]) & 0x7fffffffu) >= kHugeBits;
            bits |= (v[j] >= tau || wild ? 1u : 0u) << j;
        }
        take |= (uint64_t)bits << (u * kPer);
    }
    for (;;) {
        bool stuck = false;
        while (take != 0 && !stuck) {
            const uint32_t e = __ffsll((long long)take) - 1;
            const uint32_t position = ((e / kPer) * 32 + lane) * kPer + (e % kPer);
            const float x = tile_element<T>(tile, position);
            const uint32_t column = column0 + position;
            const uint32_t id = r.id_base + column;
            const bool wild = kGreedy && (__float_as_uint(x) & 0x7fffffffu) >= kHugeBits;
            const bool seen = r.seen_any && ((bitmap[column >> 5] >> (column & 31u)) & 1u);
            float value = x;
            uint32_t kind;
            if (seen || wild) {
                const Classified c = classify_apart<kGreedy>(L, r, w, x, id, seen, bound);
                kind = c.kind;
                value = c.value;
            } else {
                // (an infinity is nobody's candidate; equal scores: the smaller id)
                kind = !is_nonfinite(x) && x >= tau && select_key(x, id) >= bound ? 1u : 0u;
            }
            if (kind != 0u) {
                const uint32_t slot = atomicAdd(&L.count[w], 1u);
                if (slot >= (uint32_t)kListCap) {
                    stuck = true;  // (the element stays in `take`)
                    continue;
                }
                L.score[w][slot] = kind == 2u ? x : value;
                L.id[w][slot] = id;
                if (kind == 2u) {
                    atomicOr(&L.deferred[w][slot >> 5], 1u << (slot & 31u));
                } else if (r.k == 1u) {
                    atomicMax(&L.bound, (unsigned long long)select_key(value, id));
                } else {
                    const uint32_t key = float_key(value);
                    if (key >= tally.base) atomicAdd(&L.tally[tally.bin(key)], 1u);
                }
            }
            take &= take - 1;
        }
        if (!__any_sync(kFullMask, stuck)) break;
        __syncwarp();
        bound = max(bound, local_cut(L, r, w));
        bound = max(bound, (uint64_t)peek64(&L.bound));
        tau = key_to_float((uint32_t)(bound >> 32));
    }
    return bound;
}

// The row as the warps see it; *bad_history is the status a broken history earns the
// row (0 when it is fine).
__device__ __forceinline__ Row make_row(const Params &p, const SamplerConfig &cfg, uint32_t row,
                                        bool shard_mode, uint32_t *bad_history) {
    Row r;
    // (a shard of a greedy row keeps k_shard candidates like any other, and on top of them
    // notes the NaN/Inf the argmax order would put first: the merge must see it)
    r.greedy = cfg.temperature == 0.0f;
    r.k = shard_mode ? p.shard_k : (r.greedy ? 1u : cfg.top_k);
    r.id_base = p.vocab_offset;
    r.flat_offset = penalty_offset(1u, cfg.presence_penalty, cfg.frequency_penalty);
    r.presence = cfg.presence_penalty;
    r.frequency = cfg.frequency_penalty;
    r.repetition = make_repetition(cfg.repetition_penalty);
    r.tokens = nullptr;
    r.counts = nullptr;
    r.table_bitmap = nullptr;
    r.history_len = 0;
    *bad_history = 0;
    if (p.slot_counts != nullptr && penalties_active(cfg)) {
        const uint32_t session = p.row_slots[row];
        r.counts = p.slot_counts + (size_t)session * p.vocab_total;
        r.table_bitmap = p.slot_bitmaps + (size_t)session * p.slot_bitmap_words;
    } else if (p.history_tokens != nullptr && p.history_offsets != nullptr && p.bitmap_words != 0 &&
        penalties_active(cfg)) {
        const uint64_t begin = p.history_offsets[row], end = p.history_offsets[row + 1];
        if (end < begin || end - begin > p.history_max) {
            *bad_history = kErrLimit;
        } else {
            r.tokens = p.history_tokens + begin;
            r.history_len = (uint32_t)(end - begin);
        }
    }
    r.seen_any = r.history_len != 0 || r.counts != nullptr;
    r.with_counts = r.seen_any && cfg.frequency_penalty != 0.0f;
    // the host sends only rows whose penalties cannot raise a logit; a row that
    // slipped through is failed rather than sampled wrongly
    if (r.seen_any && !(cfg.presence_penalty >= 0.0f && cfg.frequency_penalty >= 0.0f &&
                        cfg.repetition_penalty >= 1.0f && r.repetition.tame))
        *bad_history = kErrArgument;
    return r;
}

// Does this kernel sample the row, or is it left to the kernel without a top-k cut?
__device__ __forceinline__ bool row_is_ours(const SamplerConfig &cfg, bool shard_mode) {
    return shard_mode || cfg.temperature == 0.0f || cfg.top_k != 0;
}

__device__ __forceinline__ SamplerConfig row_config(const Params &p, uint32_t row) {
    return p.config_count > 1 ? p.configs[row] : p.config0;
}

// Walks the tiles one consumer warp asks the copy engine for -- every kWarps-th tile of
// each of the CTA's units, unit after unit -- kStages ahead of the tile the warp looks at.
struct Feeder {
    UnitWalk walk;
    Unit u;
    const unsigned char *row;  // first byte of the unit's row
    uint32_t t;
    uint32_t issued;
    bool live;
    __device__ __forceinline__ Feeder(const Params &p, uint32_t row_tiles) : walk(p, row_tiles), issued(0) {}
    template <typename T>
    __device__ __forceinline__ bool seek(const Params &p, uint32_t w, bool shard_mode) {
        while (walk.next(u)) {
            if (!row_is_ours(row_config(p, u.row), shard_mode)) continue;
            t = u.first + w;
            row = static_cast<const unsigned char *>(p.logits) + (size_t)u.row * p.row_stride * sizeof(T);
            if (t < u.end) return true;
        }
        return false;
    }
    // asks for the warp's next tile into `stage`; all lanes call, lane 0 talks to the engine
    template <typename T>
    __device__ __forceinline__ void issue(const Params &p, unsigned char *stage, uint64_t *full,
                                          uint32_t row_bytes, uint32_t w, bool shard_mode, uint64_t policy) {
        if (!live) return;
        if (lane_id() == 0) {
            const uint32_t bytes = min(tile_bytes<T>(), row_bytes - t * tile_bytes<T>());
            const bool withheld = w == 0 && blockIdx.x == p.withhold_cta && issued == p.withhold_issue;
            if (!withheld) {
                mbarrier_expect(full, bytes);
                bulk_copy_to_shared_hinted(stage, row + (size_t)t * tile_bytes<T>(), bytes, full, policy);
            }
        }
        issued++;
        t += kWarps;
        if (t >= u.end) live = seek<T>(p, w, shard_mode);
    }
};

// One consumer warp's share of one unit: its tiles against the bound, candidates onto its
// list.  Per tile and lane: the 128-bit vectors of the tile, a maximum of each against the
// bound's score.  Returns the number of tiles it has looked at.
template <typename T, bool kGreedy>
__device__ __forceinline__ uint32_t consume_unit(const Params &p, Shared &sh, Lists &L, const Row r, const Unit u,
                                              const uint32_t *bitmap, unsigned char *stages, Feeder &feeder,
                                              uint32_t consumed, uint32_t w, uint32_t tiles, uint32_t row_bytes,
                                              bool shard_mode, uint64_t policy, uint32_t polls
) {
    using V = Lanes<T>;
    constexpr int kPer = V::kPer;
    constexpr int kVectors = tile_vectors<T>();
    const uint32_t lane = lane_id();
    const uint32_t whole = tile_bytes<T>() / 16u;
    const uint32_t last_vectors = (row_bytes - (tiles - 1) * tile_bytes<T>()) / 16u;
    const uint32_t participants = min((uint32_t)kWarps, u.end - u.first);
    uint64_t bound = 0;
    Tally tally;
    tally.base = 0;
    tally.shift = 24;
    uint32_t done = 0;  // tiles of this unit so far
    uint32_t turn = w;  // after which of them it is this warp's turn to lift the bound
    for (uint32_t t = u.first + w; t < u.end; t += kWarps) {
        const uint32_t stage = consumed % kStages;
        tile_wait(sh, &sh.full[w][stage], (consumed / kStages) & 1u, polls);
        const unsigned char *tile = stages + (size_t)stage * kStageBytes;
        const uint32_t valid_vectors = t + 1 == tiles ? last_vectors : whole;
        const uint32_t column0 = t * kTileLogits;
        if (done == 0) {
            const FirstBound first =
                first_bound<T>(sh, L, r, bitmap, tile, column0, valid_vectors, participants, polls);
            bound = (uint64_t)first.key << 32;
            tally.span(first.key, first.top);
        }
        bound = max(bound, (uint64_t)peek64(&L.bound));
        const float tau = key_to_float((uint32_t)(bound >> 32));
        const uint4 *vectors = reinterpret_cast<const uint4 *>(tile);
        // which of the lane's vectors hold something at or above the bound's score (a NaN never
        // wins a maximum).  Greedy rows: the argmax order must also see NaN, both infinities
        // and magnitudes a repetition factor of at most 2^40 could push there -- a maximum that
        // keeps NaN and a minimum tell.  (Beyond the row's end: stale bytes, masked.)
        uint32_t hot = 0;
#pragma unroll
        for (int v8 = 0; v8 < kVectors; v8++) {
            float v[kPer];
            V::unpack(vectors[v8 * 32 + lane], v);
            bool look;
            if (kGreedy) {
                const float top = propagating_max(v[0], v);
                look = !(top < tau) || smallest(v) <= -__uint_as_float(kHugeBits);  // (NaN is not below anything)
            } else {
                look = largest(v) >= tau;
            }
            hot |= (look ? 1u : 0u) << v8;
        }
        if (valid_vectors != whole) {
#pragma unroll
            for (int v8 = 0; v8 < kVectors; v8++)
                if ((uint32_t)(v8 * 32) + lane >= valid_vectors) hot &= ~(1u << v8);
        }
        if (__any_sync(kFullMask, hot != 0))
            bound = collect<T, kGreedy>(L, r, bitmap, tile, column0, valid_vectors, w, hot, bound, tally);
        // The bound tightens as the row is read: the warps take turns, one after every round of
        // tiles, to see what the tally of all the warps' exact entries allows.  Nobody waits.
        if (r.k > 1u && done == turn) {
            raise_bound(L, tally, r.k);
            turn += participants;
        }
        done++;
        __syncwarp();
        consumed++;
        feeder.template issue<T>(p, stages + (size_t)stage * kStageBytes, &sh.full[w][stage], row_bytes, w,
                                 shard_mode, policy);
    }
    return consumed;
}

// ------------------------------------------------------------------ closing warp

// The key such that exactly k exact entries of the lists lie at or above it
// (0: there are at most k).  256-bin histogram passes over the range the k-th best can
// still lie in; each narrows the range to one bin.
__device__ __noinline__ uint64_t select_threshold(uint32_t *hist, const Lists &L, const Row r) {
    const uint32_t lane = lane_id();
    uint32_t exact = 0;
    uint64_t low = ~0ull, high = 0;
    for (uint32_t w = 0; w < (uint32_t)kWarps; w++) {
        const uint32_t n = min(L.count[w], (uint32_t)kListCap);
        for (uint32_t i = lane; i < n; i += 32) {
            if ((L.deferred[w][i >> 5] >> (i & 31u)) & 1u) continue;
            const uint64_t key = entry_key(L, r, w, i, false);
            if (key == 0) continue;
            exact++;
            low = key < low ? key : low;
            high = key > high ? key : high;
        }
    }
    exact = __reduce_add_sync(kFullMask, exact);
    if (exact <= r.k) return 0ull;
    low = warp_min_u64(low);
    high = warp_max_u64(high);
    uint32_t need = r.k;
    for (int pass = 0; pass < 9; pass++) {
        const uint64_t range = high - low;
        const int shift = range < 256ull ? 0 : 56 - __clzll((long long)range);  // (range >> shift) < 256
        for (uint32_t b = lane; b < 256; b += 32) hist[b] = 0;
        __syncwarp();
        for (uint32_t w = 0; w < (uint32_t)kWarps; w++) {
            const uint32_t n = min(L.count[w], (uint32_t)kListCap);
            for (uint32_t i = lane; i < n; i += 32) {
                if ((L.deferred[w][i >> 5] >> (i & 31u)) & 1u) continue;
                const uint64_t key = entry_key(L, r, w, i, false);
                if (key < low || key > high || key == 0) continue;
                atomicAdd(&hist[(uint32_t)((key - low) >> shift)], 1u);
            }
        }
        __syncwarp();
        // lane l owns bins 255-8l .. 248-8l, walked from the top
        uint32_t mine = 0;
#pragma unroll
        for (int b = 0; b < 8; b++) mine += hist[255 - 8 * lane - b];
        uint32_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t up = __shfl_up_sync(kFullMask, incl, d);
            if (lane >= (uint32_t)d) incl += up;
        }
        const unsigned reached = __ballot_sync(kFullMask, incl >= need);
        const int owner = __ffs(reached) - 1;  // need <= entries in range, so some lane reaches it
        uint32_t bin = 0, above = 0, inside = 0;
        if ((int)lane == owner) {
            uint32_t over = incl - mine;
            for (int b = 0; b < 8; b++) {
                const uint32_t candidate = 255 - 8 * lane - b;
                const uint32_t here = hist[candidate];
                if (over + here >= need) {
                    bin = candidate;
                    above = over;
                    inside = here;
                    break;
                }
                over += here;
            }
        }
        bin = __shfl_sync(kFullMask, bin, owner);
        above = __shfl_sync(kFullMask, above, owner);
        inside = __shfl_sync(kFullMask, inside, owner);
        __syncwarp();
        const uint64_t bin_low = low + ((uint64_t)bin << shift);
        if (above + inside == need || shift == 0) return bin_low;
        need -= above;
        const uint64_t bin_high = bin_low + ((1ull << shift) - 1ull);
        low = bin_low;
        high = bin_high < high ? bin_high : high;
    }
    return low;
}

// The exact k best of a set of lists, in sampling order, into `fin`; returns how many.  The
// long way: for lists that hold many more entries at or above the bound than a row wants.
__device__ __noinline__ uint32_t settle_wide(FinishBuffer &fin, uint32_t *hist, uint32_t *gathered, Lists &L,
                                            const Row r) {
    const uint32_t lane = lane_id();
    uint64_t threshold;
    for (;;) {
        threshold = select_threshold(hist, L, r);
        // entries not counted yet whose upper bound reaches the k best are settled, then the
        // selection is done again
        uint32_t any = 0;
        if (lane < (uint32_t)kWarps) {
#pragma unroll
            for (int j = 0; j < kListWords; j++) any |= L.deferred[lane][j];
        }
        uint32_t with = __ballot_sync(kFullMask, any != 0);
        uint32_t settled = 0;
        for (; with != 0; with &= with - 1) settled += resolve_above(L, r, __ffs(with) - 1, threshold);
        if (settled == 0) break;
    }
    // unsorted survivors go to the far end of the work arrays, the sort brings them forward
    float *loose_score = reinterpret_cast<float *>(fin.raw);
    uint32_t *loose_id = reinterpret_cast<uint32_t *>(fin.tempered);
    if (lane == 0) *gathered = 0;
    __syncwarp();
    for (uint32_t w = 0; w < (uint32_t)kWarps; w++) {
        const uint32_t n = min(L.count[w], (uint32_t)kListCap);
        for (uint32_t i = lane; i < n; i += 32) {
            if ((L.deferred[w][i >> 5] >> (i & 31u)) & 1u) continue;
            const uint64_t key = entry_key(L, r, w, i, false);
            if (key == 0 || key < threshold) continue;
            const uint32_t slot = atomicAdd(gathered, 1u);
            if (slot < (uint32_t)kMaxK) {
                loose_score[slot] = L.score[w][i];
                loose_id[slot] = L.id[w][i];
            }
        }
    }
    __syncwarp();
    const uint32_t kept = min(min(*gathered, (uint32_t)kMaxK), r.k);
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
            fin.score[my_rank[h]] = my_score[h];
            fin.id[my_rank[h]] = my_id[h];
        }
    }
    __syncwarp();
    return kept;
}

// The same, the short way.  Everything that can be among the k best lies at or above the
// unit's bound, and by the time a unit is closed that is little more than k entries: they are
// gathered densely (entries whose occurrences are not counted yet are settled first, if the
// most they can be worth reaches the bound), and every entry finds its place by counting the
// keys above its own.  Keys are distinct, so the places are a permutation.
constexpr uint32_t kDense = 128;  // keys the short way takes: the closer's 256-word table
__device__ __noinline__ uint32_t settle_lists(FinishBuffer &fin, uint32_t *hist, uint32_t *gathered, Lists &L,
                                             const Row r) {
    const uint32_t lane = lane_id();
    const uint64_t bound = peek64(&L.bound);
    {
        uint32_t any = 0;
        if (lane < (uint32_t)kWarps) {
#pragma unroll
            for (int j = 0; j < kListWords; j++) any |= L.deferred[lane][j];
        }
        for (uint32_t with = __ballot_sync(kFullMask, any != 0); with != 0; with &= with - 1)
            resolve_above(L, r, __ffs(with) - 1, bound);
    }
    uint64_t *dense = reinterpret_cast<uint64_t *>(hist);
    uint16_t *where = reinterpret_cast<uint16_t *>(fin.raw);  // list * kListCap + entry
    static_assert(kDense * sizeof(uint64_t) <= 256 * sizeof(uint32_t), "the dense keys fit the closer's table");
    static_assert(kWarps * kListCap <= 65536, "an entry's place fits 16 bits");
    uint32_t n = 0;
    for (uint32_t w = 0; w < (uint32_t)kWarps; w++) {
        const uint32_t count = min(L.count[w], (uint32_t)kListCap);
        for (uint32_t base = 0; base < count; base += 32) {
            const uint32_t i = base + lane;
            const bool exact = i < count && ((L.deferred[w][i >> 5] >> (i & 31u)) & 1u) == 0;
            const uint64_t key = exact ? entry_key(L, r, w, i, false) : 0ull;
            const bool take = key != 0 && key >= bound;
            const uint32_t takers = __ballot_sync(kFullMask, take);
            const uint32_t at = n + __popc(takers & ((1u << lane) - 1u));
            if (take && at < kDense) {
                dense[at] = key;
                where[at] = (uint16_t)(w * kListCap + i);
            }
            n += __popc(takers);
        }
    }
    __syncwarp();
    if (n > kDense) return settle_wide(fin, hist, gathered, L, r);
    constexpr int kOwned = kDense / 32;
    uint64_t mine[kOwned];
    uint32_t place[kOwned];
#pragma unroll
    for (int h = 0; h < kOwned; h++) {
        const uint32_t e = lane + 32 * h;
        mine[h] = e < n ? dense[e] : ~0ull;
        place[h] = 0;
    }
    const uint32_t owned = (n + 31u) / 32u;
#pragma unroll 4
    for (uint32_t j = 0; j < n; j++) {
        const uint64_t other = dense[j];
#pragma unroll
        for (int h = 0; h < kOwned; h++)
            if ((uint32_t)h < owned) place[h] += other > mine[h] ? 1u : 0u;
    }
    __syncwarp();
    const float *flat_score = &L.score[0][0];
    const uint32_t *flat_id = &L.id[0][0];
#pragma unroll
    for (int h = 0; h < kOwned; h++) {
        const uint32_t e = lane + 32 * h;
        if (e < n && place[h] < r.k) {
            const uint32_t from = where[e];
            fin.score[place[h]] = flat_score[from];
            fin.id[place[h]] = flat_id[from];
        }
    }
    __syncwarp();
    return min(n, r.k);
}

// A unit's lists become its part of the row's result; the CTA that finishes a row's last
// part merges the parts and writes the result.
__device__ __noinline__ void close_unit(Shared &sh, uint32_t closer, Lists &L, const Params &p, const Unit u, const Row r,
                                        const SamplerConfig cfg, bool shard_mode, uint32_t row_status) {
    const uint32_t lane = lane_id();
    const uint32_t row = u.row;
    FinishBuffer &fin = sh.fin[closer];
    uint32_t kept = settle_lists(fin, sh.hist[closer], &sh.gathered[closer], L, r);
    uint32_t bad_history = row_status ? row_status : L.bad_history;
    if (peek(&sh.ring_error)) {  // a tile never landed, or a warp never came
        bad_history = kErrLimit;
        if (lane == 0) atomicMin(p.out.first_error + 1, 1ull);  // the cause, for the host's message
    }
    unsigned long long wild = ~0ull;  // the padding id when nothing was seen
    if (lane < (uint32_t)kWarps) wild = L.wild_key[lane];
    wild = warp_min_u64(wild);
    uint32_t wild_id = (uint32_t)(wild >> 32);
    uint32_t wild_bits = (uint32_t)wild;
    if (u.parts > 1) {
        const size_t mine = (size_t)row * p.max_parts + u.part;
        for (uint32_t i = lane; i < (uint32_t)kMaxK; i += 32) {
            p.part_scores[mine * kMaxK + i] = i < kept ? fin.score[i] : 0.0f;
            p.part_ids[mine * kMaxK + i] = i < kept ? fin.id[i] : kPaddingId;
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
        // every part's survivors into this slot's lists, filled one after the other (the
        // host keeps parts * k within the lists' capacity)
        uint32_t total = 0;
        bad_history = 0;
        wild_id = kPaddingId;
        wild_bits = 0;
        float *flat_score = &L.score[0][0];
        uint32_t *flat_id = &L.id[0][0];
        for (uint32_t j = 0; j < u.parts; j++) {
            const size_t from = (size_t)row * p.max_parts + j;
            const uint4 packed = __ldcg(reinterpret_cast<const uint4 *>(&p.part_meta[from]));
            const uint32_t count = min(min(packed.x, (uint32_t)kMaxK), (uint32_t)(kWarps * kListCap) - total);
            for (uint32_t i = lane; i < count; i += 32) {
                flat_score[total + i] = __ldcg(&p.part_scores[from * kMaxK + i]);
                flat_id[total + i] = __ldcg(&p.part_ids[from * kMaxK + i]);
            }
            total += count;
            if (packed.w) bad_history = packed.w;
            if (packed.y < wild_id) {
                wild_id = packed.y;
                wild_bits = packed.z;
            }
        }
        if (lane < (uint32_t)kWarps) {
            const uint32_t before = lane * kListCap;
            L.count[lane] = total > before ? min(total - before, (uint32_t)kListCap) : 0u;
#pragma unroll
            for (int j = 0; j < kListWords; j++) L.deferred[lane][j] = 0;
        }
        __syncwarp();
        kept = settle_lists(fin, sh.hist[closer], &sh.gathered[closer], L, r);
    }
    // ---- the row's result ----
    if (shard_mode) {
        // a greedy row's NaN/Inf with the smallest id goes first, as the slice's argmax
        // cascade of src/output.c:320-344 would report it; the finite ones follow
        const uint32_t lead = r.greedy && wild_id != kPaddingId ? 1u : 0u;
        for (uint32_t i = lane; i < r.k; i += 32) {
            const size_t at = ((size_t)row * r.k + i) * p.shard_stride;
            const bool ok = i >= lead && i - lead < kept && !bad_history;
            float score = ok ? fin.score[i - lead] : __uint_as_float(0xff800000u);
            uint32_t id = ok ? fin.id[i - lead] : kPaddingId;
            if (lead && i == 0 && !bad_history) {
                score = __uint_as_float(wild_bits);
                id = wild_id;
            }
            if (p.push.ranks != 0) {
                // the fused exchange: the block lands in every rank's window, this one's too
                for (uint32_t t = 0; t < p.push.ranks; t++)
                    *p.push.pair(t, row, r.k, i) = make_uint2(__float_as_uint(score), id);
            } else {
                p.shard_scores[at] = score;
                p.shard_ids[at] = id;
            }
        }
        if (p.push.ranks != 0) {
            __threadfence_system();  // the pairs are visible on the peers before the arrivals are
            __syncwarp();
            if (lane < p.push.ranks) atomicAdd_system(p.push.arrived(lane, row), 1u);
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
                token = fin.id[0];
                logit = fin.score[0];
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
    finish_select(fin, kept, cfg, p.uniforms[row], row, p.out);
}

// One warp's share (`part` of `parts`) of a unit's history bitmap.  First the words of the
// unit's columns are cleared, or fetched from the session's bitmap; once all the warps that
// share the work have met (`meet`), the tokens are marked.  A token outside the vocabulary
// leaves its status in *bad.
template <class Meet>
__device__ __forceinline__ void build_bitmap(const Params &p, const Row &r, const Unit &u, uint32_t *bitmap,
                                             uint32_t part, uint32_t parts, uint32_t *bad_word, Meet meet) {
    const uint32_t lane = lane_id();
    const uint32_t column_begin = u.first * kTileLogits;
    const uint32_t column_end = min(p.vocab, u.end * kTileLogits);
    uint4 *wide = reinterpret_cast<uint4 *>(bitmap);
    const uint32_t quad_end = (column_end + 127u) / 128u;
    if (r.table_bitmap != nullptr) {  // the session keeps its bitmap: fetch the unit's part of it
        const uint4 *kept = reinterpret_cast<const uint4 *>(r.table_bitmap);
        for (uint32_t q = column_begin / 128u + part * 32 + lane; q < quad_end; q += 32 * parts)
            wide[q] = __ldg(&kept[q]);
    } else {
        for (uint32_t q = column_begin / 128u + part * 32 + lane; q < quad_end; q += 32 * parts)
            wide[q] = make_uint4(0, 0, 0, 0);
    }
    meet();
    constexpr int kBatch = 16;  // tokens per lane and trip, loaded before any is used
    uint32_t bad = 0;
    for (uint32_t base = part * kBatch * 32; base < r.history_len; base += parts * kBatch * 32) {
        uint32_t token[kBatch];
#pragma unroll
        for (int q = 0; q < kBatch; q++) {
            const uint32_t at = base + q * 32 + lane;
            token[q] = at < r.history_len ? r.tokens[at] : p.vocab_offset + column_end;
        }
#pragma unroll
        for (int q = 0; q < kBatch; q++) {
            if (base + q * 32 + lane >= r.history_len) continue;
            if (token[q] >= p.vocab_total) bad = kErrFormat;
            const uint32_t local = token[q] - p.vocab_offset;  // wraps for ids below the span
            if (local >= column_begin && local < column_end) {
                const uint32_t bit = 1u << (local & 31u);
                if ((bitmap[local >> 5] & bit) == 0) atomicOr(&bitmap[local >> 5], bit);
            }
        }
    }
    if (__any_sync(kFullMask, bad != 0) && lane == 0) atomicOr(bad_word, kErrFormat);
}
// Where the warps that share a bitmap's work meet: the history warps among themselves, or --
// for a CTA's first unit, when the consumer warps have nothing to read yet -- all of them.
struct HistoryWarpsMeet {
    __device__ __forceinline__ void operator()() const {
        asm volatile("bar.sync 2, %0;" ::"n"(kHistoryWarps * 32) : "memory");
    }
};
struct EverybodyMeets {
    __device__ __forceinline__ void operator()() const {
        asm volatile("bar.sync 3, %0;" ::"n"((kWarps + kHistoryWarps) * 32) : "memory");
    }
};

template <typename T>
__global__ void __launch_bounds__(kBlock, 1) persistent_select_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(128) unsigned char dynamic[];
    __shared__ Shared sh;
    unsigned char *ring = dynamic;
    Lists *lists = reinterpret_cast<Lists *>(dynamic + (size_t)kWarps * kStages * kStageBytes);
    uint32_t *bitmaps = reinterpret_cast<uint32_t *>(dynamic + (size_t)kWarps * kStages * kStageBytes + kListSets * sizeof(Lists));
    const uint32_t bitmap_stride = ((p.bitmap_words + 3u) / 4u) * 4u;  // words, a whole number of uint4

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const bool shard_mode = p.shard_k != 0;
    const uint32_t row_bytes = p.vocab * (uint32_t)sizeof(T);
    const uint32_t tiles = (p.vocab + kTileLogits - 1) / kTileLogits;
    const uint32_t polls = p.wait_polls ? p.wait_polls : kDefaultPolls;
    const uint32_t buffers = p.bitmap_buffers;

    if (tid == 0) {
        for (int w = 0; w < kWarps; w++)
            for (int s = 0; s < kStages; s++) mbarrier_init(&sh.full[w][s], 1);
        for (int b = 0; b < 3; b++) {
            mbarrier_init(&sh.bitmap_ready[b], kHistoryWarps);
            mbarrier_init(&sh.bitmap_free[b], kWarps);
            sh.history_bad[b] = 0;
        }
        for (int b = 0; b < kListSets; b++) {
            mbarrier_init(&sh.ready[b], kWarps);
            mbarrier_init(&sh.vacant[b], 1);
            lists[b].bound = 0;
            lists[b].first_key = 0xffffffffu;
            lists[b].first_count = 0;
            lists[b].first_top = 0;
            lists[b].bad_history = 0;
            for (int i = 0; i < kTallyBins; i++) lists[b].tally[i] = 0;
        }
        mbarrier_fence_init();
        sh.ring_error = 0;
    }
    __syncthreads();

    if (warp >= (uint32_t)(kWarps + kHistoryWarps)) {
        // ------------------------------------------------------------ closing warps
        // Closer c takes the units that use list set c: every other unit.
        const uint32_t closer = warp - (kWarps + kHistoryWarps);
        uint32_t served = 0;
        UnitWalk walk(p, tiles);
        Unit u;
        while (walk.next(u)) {
            const SamplerConfig cfg = row_config(p, u.row);
            if (!row_is_ours(cfg, shard_mode)) continue;
            if ((served & 1u) != closer) {
                served++;
                continue;
            }
            const uint32_t b = served % kListSets;
            uint32_t row_status;
            const Row r = make_row(p, cfg, u.row, shard_mode, &row_status);
            Lists &L = lists[b];
            // (a wait that runs out leaves garbage lists: the row is failed through ring_error)
            bounded_wait(sh, &sh.ready[b], (served / kListSets) & 1u, polls);
            __syncwarp();
            close_unit(sh, closer, L, p, u, r, cfg, shard_mode, row_status);
            __syncwarp();
            // the lists' shared words, clean for the unit after next (a warp that is ahead of
            // the others must not meet what they published for another row)
            for (uint32_t i = lane; i < (uint32_t)kTallyBins; i += 32) L.tally[i] = 0;
            __syncwarp();
            if (lane == 0) {
                L.bound = 0;
                L.first_key = 0xffffffffu;
                L.first_count = 0;
                L.first_top = 0;
                L.bad_history = 0;
                mbarrier_arrive(&sh.vacant[b]);
            }
            __syncwarp();
            served++;
        }
        return;
    }
    if (warp >= (uint32_t)kWarps) {
        // ------------------------------------------------------------ history warps
        // The bitmap of the history ids that fall into the unit's columns, built ahead of the
        // consumers by as many units as there are spare buffers (two, one) or as soon as they
        // are through with the previous unit (none).  A token outside the vocabulary leaves
        // its status behind.
        const uint32_t helper = warp - kWarps;
        uint32_t served = 0;
        UnitWalk walk(p, tiles);
        Unit u;
        while (walk.next(u)) {
            const SamplerConfig cfg = row_config(p, u.row);
            if (!row_is_ours(cfg, shard_mode)) continue;
            uint32_t row_status;
            const Row r = make_row(p, cfg, u.row, shard_mode, &row_status);
            const uint32_t slot = served % buffers;
            // the consumers must be through with the unit that used the buffer last (each buffer
            // has a barrier of its own: one phase per use, however far the consumers have got)
            if (served >= buffers) bounded_wait(sh, &sh.bitmap_free[slot], (served / buffers - 1u) & 1u, polls);
            if (helper == 0 && lane == 0 && served != 0) sh.history_bad[slot] = 0;
            if (r.seen_any) {
                uint32_t *bitmap = bitmaps + (size_t)slot * bitmap_stride;
                if (served == 0) {
                    // the CTA's first unit: the consumer warps lend a hand (see below)
                    build_bitmap(p, r, u, bitmap, kWarps + helper, kWarps + kHistoryWarps, &sh.history_bad[slot],
                                 EverybodyMeets());
                    EverybodyMeets()();  // everybody's marks are in
                } else {
                    build_bitmap(p, r, u, bitmap, helper, kHistoryWarps, &sh.history_bad[slot], HistoryWarpsMeet());
                }
            }
            __threadfence_block();
            __syncwarp();
            if (lane == 0) mbarrier_arrive(&sh.bitmap_ready[slot]);
            served++;
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    const uint32_t w = warp;
    const uint64_t policy = l2_policy_evict_first();
    unsigned char *stages = ring + (size_t)w * kStages * kStageBytes;
    Feeder feeder(p, tiles);
    feeder.live = feeder.template seek<T>(p, w, shard_mode);
#pragma unroll
    for (int s = 0; s < kStages; s++)
        feeder.template issue<T>(p, stages + (size_t)s * kStageBytes, &sh.full[w][s], row_bytes, w, shard_mode, policy);
    {
        // The CTA's first unit: nothing has landed yet, so the consumer warps help the history
        // warps with its bitmap (every warp comes to the same decision from the same inputs).
        UnitWalk ahead(p, tiles);
        Unit u0;
        bool found = false;
        while (!found && ahead.next(u0)) found = row_is_ours(row_config(p, u0.row), shard_mode);
        if (found) {
            uint32_t ignored;
            const Row r0 = make_row(p, row_config(p, u0.row), u0.row, shard_mode, &ignored);
            if (r0.seen_any) {
                build_bitmap(p, r0, u0, bitmaps, w, kWarps + kHistoryWarps, &sh.history_bad[0], EverybodyMeets());
                EverybodyMeets()();
            }
        }
    }
    uint32_t consumed = 0;  // tiles of this warp so far
    uint32_t served = 0;    // units before this one
    UnitWalk walk(p, tiles);
    Unit u;
    while (walk.next(u)) {
        const SamplerConfig cfg = row_config(p, u.row);
        if (!row_is_ours(cfg, shard_mode)) continue;
        uint32_t row_status;
        const Row r = make_row(p, cfg, u.row, shard_mode, &row_status);
        const uint32_t b = served % kListSets;
        Lists &L = lists[b];
        const uint32_t slot = served % buffers;
        const uint32_t *bitmap = bitmaps + (size_t)slot * bitmap_stride;
        // the closing warp must be done with these lists (it got them three units ago)
        if (served >= (uint32_t)kListSets) bounded_wait(sh, &sh.vacant[b], (served / kListSets - 1u) & 1u, polls);
        if (lane < (uint32_t)kListWords) L.deferred[w][lane] = 0;
        if (lane == 0) {
            L.count[w] = 0;
            L.wild_key[w] = ~0ull;
        }
        bounded_wait(sh, &sh.bitmap_ready[slot], (served / buffers) & 1u, polls);
        if (w == 0 && lane == 0) L.bad_history = sh.history_bad[slot];
        __syncwarp();
        consumed = r.greedy ? consume_unit<T, true>(p, sh, L, r, u, bitmap, stages, feeder, consumed, w, tiles,
                                                    row_bytes, shard_mode, policy, polls)
                            : consume_unit<T, false>(p, sh, L, r, u, bitmap, stages, feeder, consumed, w, tiles,
                                                     row_bytes, shard_mode, policy, polls);
        __threadfence_block();
        __syncwarp();
        if (lane == 0) {
            mbarrier_arrive(&sh.ready[b]);
            mbarrier_arrive(&sh.bitmap_free[slot]);
        }
        served++;
    }
    // copies asked for but never looked at (only after a wait ran out) still write into this
    // CTA's shared memory: see them land, bounded, before the CTA may go away
    while (consumed < feeder.issued) {
        const uint32_t stage = consumed % kStages;
        for (uint32_t i = 0; i < polls; i++) {
            if (mbarrier_try_wait(&sh.full[w][stage], (consumed / kStages) & 1u)) break;
            __nanosleep(kNapNanoseconds);
        }
        consumed++;
    }
}

}  // namespace persist
}  // namespace fgk

// ------------------------------------------------------------------ host side


using namespace fgk;

static persist::Params to_persist_params(const fgk_stream_launch *l) {
    persist::Params p;
    memset(&p, 0, sizeof(p));
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
    p.shard_stride = l->shard_stride ? l->shard_stride : 1u;
    for (int t = 0; t < 16; t++) p.push.window[t] = static_cast<unsigned char *>(l->push.window[t]);
    p.push.ranks = l->push.ranks;
    p.push.rank = l->push.rank;
    p.push.half = l->push.half;
    p.push.pair_capacity = l->push.pair_capacity;
    p.push.row_capacity = l->push.row_capacity;
    p.tiles_per_cta = l->split_len;  /* reused: tiles per CTA */
    p.max_parts = l->splits;         /* reused: most CTAs per row */
    p.part_scores = l->part_scores;
    p.part_ids = l->part_ids;
    p.part_meta = static_cast<persist::PartRecord *>(l->part_meta);
    p.tickets = l->tickets;
    p.slot_counts = l->slot_counts;
    p.slot_bitmaps = l->slot_bitmaps;
    p.row_slots = l->row_slots;
    p.slot_bitmap_words = l->slot_bitmap_words;
    p.wait_polls = l->wait_polls;
    p.withhold_cta = l->withhold_armed ? l->withhold_cta : 0xffffffffu;
    p.withhold_issue = l->withhold_issue;
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

// Dynamic shared memory for a history bitmap of `bitmap_words` words: the stages, the
// sets of lists and as many bitmap buffers as fit, three at most.  0: not even one.
extern "C" uint64_t fgk_persistent_dynamic_smem(uint32_t bitmap_words, uint32_t *bitmap_buffers) {
    const uint64_t fixed = (uint64_t)persist::kWarps * persist::kStages * persist::kStageBytes +
                           persist::kListSets * sizeof(persist::Lists);
    const uint64_t bitmap = (((uint64_t)bitmap_words + 3u) / 4u) * 16u;
    const uint64_t room = persist::kSharedLimit - sizeof(persist::Shared) - 256u;
    uint32_t buffers = 3;
    while (buffers > 1u && fixed + buffers * bitmap > room) buffers--;
    if (fixed + buffers * bitmap > room) return 0;
    if (bitmap_buffers) *bitmap_buffers = buffers;
    return fixed + buffers * bitmap;
}

// Tiles (of 2048 logits, whatever their type) in a row of `vocab` logits.
extern "C" uint32_t fgk_persistent_row_tiles(uint32_t dtype, uint32_t vocab) {
    (void)dtype;
    return (vocab + persist::kTileLogits - 1) / persist::kTileLogits;
}

// Tiles one CTA looks at side by side (a share of a row shorter than this leaves warps idle).
extern "C" uint32_t fgk_persistent_tiles_abreast(void) { return persist::kWarps; }

// Most parts of one row the merge can take when every part hands over up to k survivors.
extern "C" uint32_t fgk_persistent_max_parts(uint32_t k) {
    if (k == 0 || k > (uint32_t)kMaxK) k = kMaxK;
    return (uint32_t)(persist::kWarps * persist::kListCap) / k;
}

extern "C" int fgk_persistent_prepare(void) {
    cudaError_t e = cudaFuncSetAttribute(persist::persistent_select_kernel<float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(persist::kSharedLimit - sizeof(persist::Shared) - 256u));
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(persist::persistent_select_kernel<uint16_t>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(persist::kSharedLimit - sizeof(persist::Shared) - 256u));
    return (int)e;
}

extern "C" int fgk_launch_persistent_select(const fgk_stream_launch *l, uint32_t ctas, void *stream) {
    persist::Params p = to_persist_params(l);
    uint32_t buffers = 1;
    const size_t dynamic = (size_t)fgk_persistent_dynamic_smem(l->bitmap_words, &buffers);
    if (dynamic == 0) return (int)cudaErrorInvalidValue;
    p.bitmap_buffers = buffers;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (l->dtype == 0)
        persist::persistent_select_kernel<float><<<ctas, persist::kBlock, dynamic, s>>>(p);
    else
        persist::persistent_select_kernel<uint16_t><<<ctas, persist::kBlock, dynamic, s>>>(p);
    return (int)cudaGetLastError();
}
