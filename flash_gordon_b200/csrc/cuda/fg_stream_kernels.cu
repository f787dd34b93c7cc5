// Fused sampling kernels for sm_100a: one pass over the logits in HBM.
//
// Grid: (splits, rows).  CTA (s, r) owns columns [s*split_len, (s+1)*split_len)
// of row r and
//   1. builds, in shared memory, the part of the row's token history that falls
//      into its columns: a bitmap of seen ids, a running popcount per bitmap word
//      and a dense count per seen id (src/output.c:601-617 builds a vocab-wide
//      count table per session instead);
//   2. streams its columns with 128-bit loads (next tile prefetched into
//      registers), applies the penalties of src/sampler.c:46-60 to seen ids in
//      registers, and keeps every value that can still be among the k best in a
//      shared-memory candidate list; the list is cut back to k with a radix
//      select whenever it fills, which also raises the admission threshold;
//   3. hands its k best to the row's last-arriving CTA (ticket counter), which
//      merges the splits and runs the select step of src/sampler.c:80-122.
// Logits are read once; nothing vocabulary-sized is written.
#include <type_traits>

#include "fg_block_select.cuh"
#include "fg_kernels.h"

namespace fgk {

constexpr int kThreads = 256;
constexpr int kElemsPerThread = 16;
constexpr int kTile = kThreads * kElemsPerThread;  // 4096 logits per CTA iteration
constexpr int kCandCap = 1024;
constexpr uint32_t kMaxSplits = 16;  // the merge of 16 x 64 survivors fits one candidate buffer

struct alignas(16) PartMeta {
    uint32_t count;         // finite candidates this split kept (<= k)
    uint32_t wild_id;       // smallest id holding a NaN/Inf (greedy rows), padding if none
    uint32_t wild_bits;     // its value
    uint32_t bad_history;   // 0, or the fg_status a broken history earns the row
};

struct StreamParams {
    const void *logits;
    uint64_t row_stride;
    uint32_t rows, vocab;
    uint32_t vocab_offset, vocab_total;
    uint32_t splits, split_len;
    const uint32_t *history_tokens;
    const uint64_t *history_offsets;
    const SamplerConfig *configs;  // device copy when config_count > 1
    SamplerConfig config0;
    uint32_t config_count;
    uint32_t shard_k;               // != 0: write candidates instead of sampling
    const float *uniforms;
    float *shard_scores;
    uint32_t *shard_ids;
    uint32_t shard_stride;          // elements between consecutive candidates (2: interleaved pairs)
    PushTargets push;               // ranks != 0: candidates go straight to every rank's window
    float *part_scores;             // [rows][splits][64]
    uint32_t *part_ids;
    PartMeta *part_meta;            // [rows][splits]
    uint32_t *tickets;              // [rows], zero between launches
    uint32_t history_max;           // caller's bound on any row's history length
    uint32_t bitmap_words;          // shared-memory layout (0: no history structure)
    uint32_t count_capacity;        // entries of the dense count array (0: counts unused)
    uint32_t dense_wide;            // dense counts are u32 (histories longer than 65,535)
    // history structures built by history_build_kernel, one slot per (row, split)
    uint32_t *history_global;
    uint64_t history_stride_words;
    void *history_meta;
    SelectOutput out;
};

struct StreamShared {
    CandidateBuffer<kCandCap> cand;
    FinishBuffer fin;
    uint32_t scan[kThreads / 32];
    uint32_t distinct;
    uint32_t bad_history;
    unsigned long long wild_key;  // greedy rows: min over NaN/Inf of (id << 32 | value bits)
    uint32_t wild_id;
    uint32_t wild_bits;
    uint32_t is_last;
    uint32_t overflow;            // a value found no slot in the candidate list
};

template <typename T>
struct Loader;

template <>
struct Loader<float> {
    static constexpr int kVectors = 4;        // 4 x (4 fp32) per thread per tile
    static constexpr int kPerVector = 4;
    // ragged edge / unaligned row: element-wise, columns past the end read as -inf
    static __device__ __forceinline__ uint4 load_guarded(const float *p, uint32_t first, uint32_t n) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) w[j] = first + j < n ? __float_as_uint(p[first + j]) : 0xff800000u;
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ void unpack(const uint4 &raw, float *v) {
        v[0] = __uint_as_float(raw.x);
        v[1] = __uint_as_float(raw.y);
        v[2] = __uint_as_float(raw.z);
        v[3] = __uint_as_float(raw.w);
    }
};

template <>
struct Loader<uint16_t> {                     // bf16 bit patterns
    static constexpr int kVectors = 2;        // 2 x (8 bf16) per thread per tile
    static constexpr int kPerVector = 8;
    static __device__ __forceinline__ uint4 load_guarded(const uint16_t *p, uint32_t first,
                                                         uint32_t n) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint32_t low = first + 2 * q < n ? p[first + 2 * q] : 0xff80u;
            const uint32_t high = first + 2 * q + 1 < n ? p[first + 2 * q + 1] : 0xff80u;
            w[q] = low | (high << 16);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
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

// Column (relative to the split) of element j of vector u of this thread.
template <typename T>
__device__ __forceinline__ uint32_t column_of(uint32_t tile_base, int u, int j) {
    return tile_base + (u * kThreads + threadIdx.x) * Loader<T>::kPerVector + j;
}

// Tile -> raw registers.  Full, 16-byte aligned vectors use one 128-bit load;
// ragged edges and unaligned rows fall back to guarded scalar loads.  Lanes past
// the end read as -inf and are masked out by the caller.
template <typename T>
__device__ __forceinline__ void load_tile(const T *columns, uint32_t tile_base, uint32_t n,
                                          bool aligned, uint4 (&raw)[Loader<T>::kVectors]) {
    using L = Loader<T>;
#pragma unroll
    for (int u = 0; u < L::kVectors; u++) {
        const uint32_t first = column_of<T>(tile_base, u, 0);
        if (aligned && first + L::kPerVector <= n) {
            raw[u] = load_stream_128(columns + first);
        } else {
            raw[u] = L::load_guarded(columns, first, n);
        }
    }
}

// k-th largest of one key per thread (0 = no key), by bitwise search from the
// top bit; 0 when fewer than k threads hold a key.  All threads call.
__device__ __forceinline__ uint32_t block_kth_key(uint32_t my_key, uint32_t k) {
    uint32_t found = 0;
#pragma unroll 1
    for (int bit = 31; bit >= 0; bit--) {
        const uint32_t trial = found | (1u << bit);
        if ((uint32_t)__syncthreads_count(my_key >= trial) >= k) found = trial;
    }
    return found;
}

// Sixteen logits of one thread, passed by value into the rarely taken paths so the
// hot loop keeps them in registers.
struct Values16 {
    float v[kElemsPerThread];
};

// Per-element look at one thread's values: which ones are finite and can still make
// the top k (bit e of the result), and, for greedy rows, the smallest id holding a
// NaN/Inf (merged into sh.wild_key as id << 32 | value bits).  `inclusive` admits
// ties with the bound: they can only matter inside the tile that produced the bound,
// because later columns carry larger ids and lose the tie.
template <typename T>
__device__ __forceinline__ uint32_t classify(const Values16 &x, uint32_t tile_base, uint32_t n,
                                             float tau, bool inclusive, bool greedy,
                                             uint32_t id_base, unsigned long long *wild_key) {
    using L = Loader<T>;
    uint32_t pending = 0;
#pragma unroll
    for (int e = 0; e < kElemsPerThread; e++) {
        const uint32_t column = column_of<T>(tile_base, e / L::kPerVector, e % L::kPerVector);
        if (column >= n) continue;
        const bool wild = is_nonfinite(x.v[e]);
        if (wild) {
            if (greedy)
                atomicMin(wild_key, ((unsigned long long)(id_base + column) << 32) |
                                        __float_as_uint(x.v[e]));
            continue;
        }
        if (inclusive ? x.v[e] >= tau : x.v[e] > tau) pending |= 1u << e;
    }
    return pending;
}

// Appends the pending values of a warp to the candidate list (one shared-memory
// atomic per element position and warp).  Stored bits are cleared from `pending`;
// returns true when the list is past half full or a value found no slot.
template <typename T>
__device__ __forceinline__ bool append_pending(CandidateBuffer<kCandCap> &cand, const Values16 &x,
                                               uint32_t &pending, uint32_t tile_base,
                                               uint32_t id_base) {
    using L = Loader<T>;
    const uint32_t lane = lane_id();
    bool trouble = false;
#pragma unroll
    for (int e = 0; e < kElemsPerThread; e++) {
        const bool mine = (pending >> e) & 1u;
        const unsigned votes = __ballot_sync(kFullMask, mine);
        if (votes == 0) continue;
        const int leader = __ffs(votes) - 1;
        uint32_t base = 0;
        if ((int)lane == leader) {
            base = atomicAdd(&cand.count, (uint32_t)__popc(votes));
            // ask for a cut well before the list is full: it also lifts the bound
            if (base + __popc(votes) > kCandCap / 2) trouble = true;
        }
        base = __shfl_sync(kFullMask, base, leader);
        if (mine) {
            const uint32_t slot = base + __popc(votes & ((1u << lane) - 1u));
            if (slot < kCandCap) {
                cand.score[slot] = x.v[e];
                cand.id[slot] =
                    id_base + column_of<T>(tile_base, e / L::kPerVector, e % L::kPerVector);
                pending &= ~(1u << e);
            } else {
                trouble = true;
            }
        }
    }
    return trouble;
}

// Warp-level slow path of a tile: some lane holds a value above the bound (or, on a
// greedy row, a NaN/Inf), or the tile is one that looks at every element anyway.  Returns this thread's leftovers and whether the
// block must cut the list.
template <typename T>
__device__ __noinline__ uint32_t tile_slow_path(CandidateBuffer<kCandCap> &cand, Values16 x,
                                                uint32_t tile_base, uint32_t n, float tau,
                                                bool inclusive, bool greedy, uint32_t id_base,
                                                unsigned long long *wild_key, bool *trouble) {
    uint32_t pending = classify<T>(x, tile_base, n, tau, inclusive, greedy, id_base, wild_key);
    *trouble = false;
    if (__any_sync(kFullMask, pending != 0))
        *trouble = append_pending<T>(cand, x, pending, tile_base, id_base);
    return pending;
}

// Block-level: the list is (nearly) full.  Cut it back to the k best, which lifts
// the bound, drop leftovers that no longer qualify, and store the rest; repeat until
// nothing is left over.  Every thread of the CTA calls this together.  Returns the
// new bound.
template <typename T>
__device__ __noinline__ float resolve_overflow(CandidateBuffer<kCandCap> &cand, Values16 x,
                                               uint32_t pending, uint32_t tile_base, uint32_t k,
                                               uint32_t id_base) {
    using L = Loader<T>;
    float tau;
    for (;;) {
        const uint32_t held = min(cand.count, (uint32_t)kCandCap);
        __syncthreads();  // everyone has read count before the cut rewrites it
        compact_topk<kThreads, kCandCap>(cand, held, k);
        tau = cand.tau_score;
        const uint32_t tau_id = cand.tau_id;
        bool left = false;
#pragma unroll
        for (int e = 0; e < kElemsPerThread; e++) {
            if ((pending >> e) & 1u) {
                const uint32_t id =
                    id_base + column_of<T>(tile_base, e / L::kPerVector, e % L::kPerVector);
                if (precedes(x.v[e], id, tau, tau_id)) left = true;
                else pending &= ~(1u << e);
            }
        }
        if (!__syncthreads_or(left)) break;
        bool trouble = false;
        if (__any_sync(kFullMask, pending != 0))
            trouble = append_pending<T>(cand, x, pending, tile_base, id_base);
        if (!__syncthreads_or(trouble)) break;
    }
    return tau;
}

__device__ __forceinline__ HistoryView history_view(const StreamParams &p, uint32_t *memory) {
    return make_history_view(memory, p.bitmap_words, p.count_capacity, p.dense_wide != 0);
}

// Flags build_history hands back.
constexpr uint32_t kSeenAny = 1u;      // the row has penalties and history inside this split
constexpr uint32_t kWithCounts = 2u;   // ... and a frequency penalty, so counts are kept

// Phase 1, once per CTA: the part of the row's token history that falls into
// columns [lo, lo + n) becomes a bitmap of seen columns, an exclusive running
// popcount per bitmap word and, per seen column, the offset
// frequency * count + presence it will be charged (src/output.c:601-617 keeps a
// vocabulary-wide count table per session instead).  Kept out of line so its
// registers do not weigh on the streaming loop.
__device__ __noinline__ uint32_t build_history(const StreamParams &p, StreamShared &sh,
                                               uint32_t *dyn_smem, uint32_t row, uint32_t lo,
                                               uint32_t n, const SamplerConfig cfg) {
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const HistoryView view = history_view(p, dyn_smem);
    uint32_t *bitmap = view.bitmap;
    uint16_t *running = view.running;
    const uint32_t words = (n + 31u) >> 5;
    uint32_t history_len = 0;
    const uint32_t *history = nullptr;
    if (p.history_tokens != nullptr && p.history_offsets != nullptr) {
        const uint64_t begin = p.history_offsets[row], end = p.history_offsets[row + 1];
        history = p.history_tokens + begin;
        history_len = (uint32_t)(end - begin);
        // the shared-memory count array was sized from the caller's bound
        if (end < begin || end - begin > p.history_max) {
            history_len = 0;
            if (tid == 0) sh.bad_history = kErrLimit;
        }
    }
    const bool seen_any = penalties_active(cfg) && p.bitmap_words != 0 && history_len != 0;
    const bool with_counts = seen_any && cfg.frequency_penalty != 0.0f && p.count_capacity != 0;
    if (!seen_any) return 0;

    for (uint32_t w = tid; w < words; w += kThreads) bitmap[w] = 0;
    __syncthreads();
    const uint32_t first_global = p.vocab_offset + lo;
    // four tokens per thread and trip, loaded before any is used: the loop is a chain of
    // global-load latencies otherwise
    for (uint32_t base = 0; base < history_len; base += 4 * kThreads) {
        uint32_t token[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint32_t i = base + q * kThreads + tid;
            token[q] = i < history_len ? history[i] : 0u;
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
            if (base + q * kThreads + tid >= history_len) continue;
            if (token[q] >= p.vocab_total) sh.bad_history = kErrFormat;
            const uint32_t local = token[q] - first_global;  // wraps for ids below the split
            if (local < n) {
                const uint32_t bit = 1u << (local & 31u);
                if ((bitmap[local >> 5] & bit) == 0) atomicOr(&bitmap[local >> 5], bit);
            }
        }
    }
    __syncthreads();
    if (!with_counts) return kSeenAny;

    // exclusive running popcount per word: each thread owns a contiguous run of words
    const uint32_t per = (words + kThreads - 1) / kThreads;
    const uint32_t w0 = min(tid * per, words), w1 = min(w0 + per, words);
    uint32_t mine = 0;
    for (uint32_t w = w0; w < w1; w++) mine += __popc(bitmap[w]);
    uint32_t incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(kFullMask, incl, d);
        if (lane >= (uint32_t)d) incl += up;
    }
    if (lane == 31) sh.scan[warp] = incl;
    __syncthreads();
    uint32_t before = incl - mine;
    for (uint32_t q = 0; q < warp; q++) before += sh.scan[q];
    if (tid == kThreads - 1) sh.distinct = before + mine;
    for (uint32_t w = w0; w < w1; w++) {
        running[w] = (uint16_t)before;  // the host keeps count_capacity below 65,536
        before += __popc(bitmap[w]);
    }
    __syncthreads();
    // the host sizes count_capacity >= min(history_max, split_len) >= distinct
    const uint32_t distinct = min(sh.distinct, p.count_capacity);
    uint32_t *dense_words = static_cast<uint32_t *>(view.dense);
    const uint32_t dense_word_count = view.wide ? distinct : (distinct + 1) / 2;
    for (uint32_t i = tid; i < dense_word_count; i += kThreads) dense_words[i] = 0;
    __syncthreads();
    for (uint32_t base = 0; base < history_len; base += 4 * kThreads) {
        uint32_t token[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint32_t i = base + q * kThreads + tid;
            token[q] = i < history_len ? history[i] : 0u;
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint32_t local = token[q] - first_global;
            if (base + q * kThreads + tid < history_len && local < n) {
                const uint32_t at = view.slot(local >> 5, bitmap[local >> 5], local & 31u);
                // 16-bit counts share a word: add into the right half (a half cannot carry,
                // a history that could overflow it uses 32-bit counts)
                if (view.wide) atomicAdd(&dense_words[at], 1u);
                else atomicAdd(&dense_words[at >> 1], 1u << (16u * (at & 1u)));
            }
        }
    }
    __syncthreads();
    return kSeenAny | kWithCounts;
}

// What the tile routines need to know about the row; a few registers.
struct RowState {
    uint32_t n;          // columns in this split
    uint32_t id_base;    // global id of column 0
    uint32_t k;
    uint32_t flags;      // kSeenAny | kWithCounts
    bool greedy;
    bool aligned;
    float flat_offset;   // offset when counts are not kept (frequency is +-0)
    float presence, frequency;
    Repetition repetition;
};

// Cuts the candidate list back to its k best (which lifts the admission bound) and
// returns the new bound.  Every thread of the CTA calls it.
__device__ __noinline__ float cut_list(StreamShared &sh, uint32_t k) {
    __syncthreads();
    const uint32_t held = min(sh.cand.count, (uint32_t)kCandCap);
    __syncthreads();  // everyone has read count before the cut rewrites it
    compact_topk<kThreads, kCandCap>(sh.cand, held, k);
    return sh.cand.tau_score;
}

// Tile -> sixteen penalised values per thread, element by element (any alignment,
// any raggedness).  Columns past the end come back as -inf.
template <typename T>
__device__ __forceinline__ void load_penalised(const StreamParams &p, const uint32_t *dyn_smem,
                                               const T *columns, uint32_t tile_base,
                                               const RowState &row, Values16 &x) {
    using L = Loader<T>;
    uint4 raw[L::kVectors];
    load_tile<T>(columns, tile_base, row.n, row.aligned, raw);
#pragma unroll
    for (int u = 0; u < L::kVectors; u++) L::unpack(raw[u], &x.v[u * L::kPerVector]);
    if ((row.flags & kSeenAny) == 0) return;
    const HistoryView view = history_view(p, const_cast<uint32_t *>(dyn_smem));
#pragma unroll
    for (int e = 0; e < kElemsPerThread; e++) {
        const uint32_t column = column_of<T>(tile_base, e / L::kPerVector, e % L::kPerVector);
        if (column >= row.n) continue;
        const uint32_t word = view.bitmap[column >> 5];
        if (((word >> (column & 31u)) & 1u) == 0) continue;
        float offset = row.flat_offset;
        if (row.flags & kWithCounts)
            offset = penalty_offset(view.count(column >> 5, word, column & 31u),
                                    row.presence, row.frequency);
        x.v[e] = penalise_with_offset(x.v[e], offset, row.repetition);
    }
}

// A tile of the fast loop pushed more values than the list could take (sorted or
// constant rows do that).  Take back what the tile stored, then feed the tile again
// from memory an eighth at a time with a cut before each eighth, so the list can
// never overflow: k + kThreads * 2 <= kCandCap.  Ties with the bound are resolved on
// the id, as the bound may now come from this very tile.  Every thread of the CTA
// calls it.  Returns the new bound.
template <typename T>
__device__ __noinline__ float redo_tile(const StreamParams &p, StreamShared &sh,
                                        const uint32_t *dyn_smem, const T *columns, uint32_t t,
                                        const RowState row) {
    using L = Loader<T>;
    static_assert(kMaxK + kThreads * 2 <= kCandCap, "an eighth of a tile fits behind the k survivors");
    constexpr int PER = kCandCap / kThreads;
    const uint32_t tid = threadIdx.x;
    const uint32_t tile_base = t * kTile;
    const uint32_t first_id = row.id_base + tile_base;

    __syncthreads();
    const uint32_t held = min(sh.cand.count, (uint32_t)kCandCap);
    float score[PER];
    uint32_t id[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const uint32_t at = j * kThreads + tid;
        id[j] = kPaddingId;
        score[j] = 0.0f;
        if (at < held) {
            score[j] = sh.cand.score[at];
            id[j] = sh.cand.id[at];
        }
    }
    __syncthreads();
    if (tid == 0) {
        sh.cand.count = 0;
        sh.overflow = 0;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < PER; j++) {
        if (id[j] != kPaddingId && id[j] - first_id >= (uint32_t)kTile) {  // not from this tile
            const uint32_t slot = atomicAdd(&sh.cand.count, 1u);
            sh.cand.score[slot] = score[j];
            sh.cand.id[slot] = id[j];
        }
    }
    Values16 x;
    load_penalised<T>(p, dyn_smem, columns, tile_base, row, x);
#pragma unroll
    for (int eighth = 0; eighth < 8; eighth++) {
        const float tau = cut_list(sh, row.k);
        const uint32_t tau_id = sh.cand.tau_id;
#pragma unroll
        for (int e = eighth * 2; e < eighth * 2 + 2; e++) {
            const uint32_t column = column_of<T>(tile_base, e / L::kPerVector, e % L::kPerVector);
            if (column >= row.n) continue;
            if (is_nonfinite(x.v[e])) {
                if (row.greedy)
                    atomicMin(&sh.wild_key, ((unsigned long long)(row.id_base + column) << 32) |
                                                __float_as_uint(x.v[e]));
                continue;
            }
            if (precedes(x.v[e], row.id_base + column, tau, tau_id)) {
                const uint32_t slot = atomicAdd(&sh.cand.count, 1u);
                sh.cand.score[slot] = x.v[e];
                sh.cand.id[slot] = row.id_base + column;
            }
        }
    }
    return cut_list(sh, row.k);
}

// One tile looked at element by element: tile 0 (it sets the admission bound), the
// ragged last tile, and every tile of a row that is not 16-byte aligned.  Loads its
// own data; out of line, so its sixteen values may live on the stack.  Every thread
// of the CTA calls it.  Returns the new bound.
template <typename T>
__device__ __noinline__ float careful_tile(const StreamParams &p, StreamShared &sh,
                                           uint32_t *dyn_smem, const T *columns, uint32_t t,
                                           const RowState row, float tau) {
    using L = Loader<T>;
    const uint32_t tile_base = t * kTile;
    Values16 x;
    load_penalised<T>(p, dyn_smem, columns, tile_base, row, x);
    if (t == 0) {
        // A valid lower bound for the k-th best: the k-th largest of the per-thread
        // maxima (k distinct elements are at least that large).
        float best = __uint_as_float(0xff800000u);
        uint32_t have = 0;
#pragma unroll
        for (int e = 0; e < kElemsPerThread; e++) {
            const bool exists =
                column_of<T>(tile_base, e / L::kPerVector, e % L::kPerVector) < row.n;
            if (exists && !is_nonfinite(x.v[e])) {
                best = fmaxf(best, x.v[e]);
                have = 1;
            }
        }
        tau = key_to_float(block_kth_key(have ? float_key(best) : 0u, row.k));
    }
    uint32_t pending = classify<T>(x, tile_base, row.n, tau, t == 0, row.greedy, row.id_base,
                                   &sh.wild_key);
    bool trouble = false;
    if (__any_sync(kFullMask, pending != 0))
        trouble = append_pending<T>(sh.cand, x, pending, tile_base, row.id_base);
    if (__syncthreads_or(trouble))
        tau = resolve_overflow<T>(sh.cand, x, pending, tile_base, row.k, row.id_base);
    return tau;
}

// Phases 3 and 4, once per CTA: cut the list to this split's k best; with several
// splits per row hand them to the row's last-arriving CTA, which merges all splits;
// then write the row's result (shard candidates, greedy winner, or the select step
// of src/sampler.c:80-122).  Every thread of the CTA calls it.
__device__ __noinline__ void finish_split(const StreamParams &p, StreamShared &sh, uint32_t row,
                                          uint32_t split, uint32_t k, bool greedy,
                                          bool shard_mode, const SamplerConfig cfg) {
    const uint32_t tid = threadIdx.x;
    __syncthreads();
    uint32_t held = min(sh.cand.count, (uint32_t)kCandCap);
    __syncthreads();
    held = compact_topk<kThreads, kCandCap>(sh.cand, held, k);
    __syncthreads();

    uint32_t bad_history = sh.bad_history;
    uint32_t wild_id = (uint32_t)(sh.wild_key >> 32);  // the padding id when nothing was seen
    uint32_t wild_bits = (uint32_t)sh.wild_key;

    if (p.splits > 1) {
        const size_t slot = (size_t)row * p.splits + split;
        if (tid < kMaxK) {
            p.part_scores[slot * kMaxK + tid] = tid < held ? sh.cand.score[tid] : 0.0f;
            p.part_ids[slot * kMaxK + tid] = tid < held ? sh.cand.id[tid] : kPaddingId;
        }
        if (tid == 0) {
            PartMeta meta;
            meta.count = held;
            meta.wild_id = wild_id;
            meta.wild_bits = wild_bits;
            meta.bad_history = bad_history;
            p.part_meta[slot] = meta;
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) sh.is_last = atomicAdd(&p.tickets[row], 1u) == p.splits - 1 ? 1u : 0u;
        __syncthreads();
        if (!sh.is_last) return;
        __threadfence();
        if (tid == 0) {
            p.tickets[row] = 0;  // ready for the next launch
            sh.cand.count = 0;
        }
        // gather every split's survivors into the candidate buffer
        uint32_t total = 0;
        bad_history = 0;
        wild_id = kPaddingId;
        wild_bits = 0;
        for (uint32_t s = 0; s < p.splits; s++) {
            const size_t from = (size_t)row * p.splits + s;
            const uint4 packed = __ldcg(reinterpret_cast<const uint4 *>(&p.part_meta[from]));
            const uint32_t count = packed.x;
            if (tid < count) {
                sh.cand.score[total + tid] = __ldcg(&p.part_scores[from * kMaxK + tid]);
                sh.cand.id[total + tid] = __ldcg(&p.part_ids[from * kMaxK + tid]);
            }
            total += count;
            if (packed.w) bad_history = packed.w;
            if (packed.y < wild_id) {
                wild_id = packed.y;
                wild_bits = packed.z;
            }
        }
        __syncthreads();
        if (tid == 0) sh.cand.count = total;
        __syncthreads();
        held = compact_topk<kThreads, kCandCap>(sh.cand, total, k);
    }

    if (shard_mode) {
        sort_candidates(sh.cand, sh.fin, held);
        // a greedy row's NaN/Inf with the smallest id goes first, as the slice's argmax
        // cascade of src/output.c:320-344 would report it; the finite ones follow
        const uint32_t lead = greedy && wild_id != kPaddingId ? 1u : 0u;
        if (tid < k) {
            const size_t at = ((size_t)row * k + tid) * p.shard_stride;
            const bool live = tid >= lead && tid - lead < held && !bad_history;
            float score = live ? sh.fin.score[tid - lead] : __uint_as_float(0xff800000u);
            uint32_t id = live ? sh.fin.id[tid - lead] : kPaddingId;
            if (lead && tid == 0 && !bad_history) {
                score = __uint_as_float(wild_bits);
                id = wild_id;
            }
            if (p.push.ranks != 0) {
                // the fused exchange: the block lands in every rank's window, this one's too
                for (uint32_t t = 0; t < p.push.ranks; t++)
                    *p.push.pair(t, row, k, tid) = make_uint2(__float_as_uint(score), id);
            } else {
                p.shard_scores[at] = score;
                p.shard_ids[at] = id;
            }
        }
        if (p.push.ranks != 0) {
            __threadfence_system();  // the pairs are visible on the peers before the arrivals are
            __syncthreads();
            if (tid < p.push.ranks) atomicAdd_system(p.push.arrived(tid, row), 1u);
        }
        if (tid == 0) {
            p.out.row_status[row] = bad_history;
            if (bad_history)
                atomicMin(p.out.first_error, ((unsigned long long)row << 8) | bad_history);
        }
        return;
    }
    if (bad_history) {  // "history token ... is outside vocabulary", src/output.c:610-612
        if (tid == 0) {
            report_row(p.out, row, bad_history, kPaddingId, 0.0f);
            if (p.out.dbg_count) p.out.dbg_count[row] = 0;
        }
        return;
    }
    if (greedy) {
        if (tid == 0) {
            uint32_t status = kOk, token;
            float logit;
            if (wild_id != kPaddingId) {
                // a NaN/Inf beats every finite logit in the argmax order and is then
                // rejected: src/output.c:593 (no penalties) / 737-739 (penalised)
                status = penalties_active(cfg) ? kErrFormat : kErrMismatch;
                token = wild_id;
                logit = __uint_as_float(wild_bits);
            } else if (held == 0) {
                status = kErrMismatch;
                token = kPaddingId;
                logit = 0.0f;
            } else {
                token = sh.cand.id[0];
                logit = sh.cand.score[0];
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
    sort_candidates(sh.cand, sh.fin, held);
    if (tid < 32) finish_select(sh.fin, held, cfg, p.uniforms[row], row, p.out);
}

// The hot loop: tiles 1 .. full_tiles-1 of a 16-byte aligned row.  128-bit loads at
// constant offsets from one running pointer (the next tile is in flight while this one
// is examined), one bitmap word and one compare per vector; single elements are only
// looked at by lanes that hold a value above the admission bound.  A function of its
// own, and one that calls nothing: whatever is live across a call inside a loop gets
// saved and restored on every trip.  So when the candidate list needs attention (a cut,
// or a tile that overflowed it) the loop stops and says so; the caller deals with it
// and comes back.  Returns the last tile it examined, with kNeedsAttention set if it
// stopped early.
//
// kLowering: every penalty of the row can only lower a logit (presence >= 0,
// frequency >= 0, repetition >= 1, all three roundings are monotone).  A raw value at
// or below the bound then stays there once penalised, so the history is consulted
// only for the few values that beat the bound raw.  Otherwise seen ids are penalised
// before anything is compared.
constexpr uint32_t kNeedsAttention = 0x80000000u;

template <typename T, bool kLowering>
__device__ __noinline__ uint32_t fast_tiles(const StreamParams &p, StreamShared &sh,
                                            const uint32_t *dyn_smem, const T *columns,
                                            uint32_t first_tile, uint32_t full_tiles,
                                            const RowState state, const float tau) {
    using L = Loader<T>;
    const uint32_t tid = threadIdx.x;
    const bool greedy = state.greedy;
    const uint32_t n = state.n;
    (void)n;
    constexpr uint32_t kTileVectors = kTile / L::kPerVector;  // 128-bit vectors per tile
    // this thread's vector u sits in bitmap word (tile_base / 32) + u * kWordsPerStep
    // + word_lane, at bit bit_lane
    constexpr uint32_t kWordsPerStep = kThreads * L::kPerVector / 32;
    const uint32_t word_lane = tid * L::kPerVector / 32;
    const uint32_t bit_lane = (tid * L::kPerVector) & 31u;
    const bool seen_any = state.flags & kSeenAny, with_counts = state.flags & kWithCounts;
    const HistoryView view = history_view(p, const_cast<uint32_t *>(dyn_smem));
    const uint32_t *bitmap = view.bitmap + word_lane;
    // cut the list once it holds a few multiples of k: the bound stays close to the
    // true k-th best and fewer values reach the list at all
    const uint32_t cut_at = 4 * state.k + 64;
    const uint4 *source =
        reinterpret_cast<const uint4 *>(columns) + tid + (size_t)first_tile * kTileVectors;
    uint4 raw[L::kVectors];
#pragma unroll
    for (int u = 0; u < L::kVectors; u++) raw[u] = load_stream_128(source + u * kThreads);
    for (uint32_t t = first_tile; t < full_tiles; t++) {
        source += kTileVectors;
        const bool more = t + 1 < full_tiles;
        const uint32_t tile_word = t * (kTile / 32);
        bool want_cut = false;
        // one 128-bit vector at a time: its register slot is refilled with the next
        // tile's data as soon as it has been unpacked
#pragma unroll
        for (int u = 0; u < L::kVectors; u++) {
            float v[L::kPerVector];
            L::unpack(raw[u], v);
            if (more) raw[u] = load_stream_128(source + u * kThreads);
            if (!kLowering && seen_any) {
                const uint32_t word = bitmap[tile_word + u * kWordsPerStep];
                const uint32_t bits = (word >> bit_lane) & ((1u << L::kPerVector) - 1u);
                if (bits != 0) {
#pragma unroll
                    for (int j = 0; j < L::kPerVector; j++) {
                        if (bits & (1u << j)) {
                            float offset = state.flat_offset;
                            if (with_counts)
                                offset = penalty_offset(
                                    view.count(tile_word + u * kWordsPerStep + word_lane, word,
                                               bit_lane + j),
                                    state.presence, state.frequency);
                            v[j] = penalise_with_offset(v[j], offset, state.repetition);
                        }
                    }
                }
            }
            float top = v[0];  // NaN never compares above the bound
#pragma unroll
            for (int j = 1; j < L::kPerVector; j++) top = fmaxf(top, v[j]);
            bool hot = top > tau;
            if (greedy) {  // the argmax order must see NaN and both infinities
                uint32_t widest = 0;
#pragma unroll
                for (int j = 0; j < L::kPerVector; j++)
                    widest = max(widest, __float_as_uint(v[j]) & 0x7fffffffu);
                // also magnitudes a penalty could push to infinity (|v| >= 2^87 with a
                // repetition factor of at most 2^40)
                hot = hot || widest >= (kLowering ? 0x6b000000u : 0x7f800000u);
            }
            if (hot) {
                // Few lanes get here once the bound has settled.  Later columns carry
                // larger ids than whatever produced the bound, so a tie with it loses.
                const uint32_t first_id = state.id_base + column_of<T>(t * kTile, u, 0);
                if (kLowering && seen_any) {
                    const uint32_t word = bitmap[tile_word + u * kWordsPerStep];
                    const uint32_t bits = (word >> bit_lane) & ((1u << L::kPerVector) - 1u);
#pragma unroll
                    for (int j = 0; j < L::kPerVector; j++) {
                        if (bits & (1u << j)) {
                            float offset = state.flat_offset;
                            if (with_counts)
                                offset = penalty_offset(
                                    view.count(tile_word + u * kWordsPerStep + word_lane, word,
                                               bit_lane + j),
                                    state.presence, state.frequency);
                            v[j] = penalise_with_offset(v[j], offset, state.repetition);
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < L::kPerVector; j++) {
                    if (is_nonfinite(v[j])) {
                        if (greedy)
                            atomicMin(&sh.wild_key, ((unsigned long long)(first_id + j) << 32) |
                                                        __float_as_uint(v[j]));
                    } else if (v[j] > tau) {
                        const uint32_t slot = atomicAdd(&sh.cand.count, 1u);
                        if (slot < (uint32_t)kCandCap) {
                            sh.cand.score[slot] = v[j];
                            sh.cand.id[slot] = first_id + j;
                        } else {
                            sh.overflow = 1;
                        }
                        want_cut = want_cut || slot >= cut_at;
                    }
                }
            }
        }
        // one barrier per tile: does the list need attention?
        if (__syncthreads_or(want_cut)) return t | kNeedsAttention;
    }
    return full_tiles - 1;
}


template <typename T>
__global__ void __launch_bounds__(kThreads, 4)
stream_select_kernel(const __grid_constant__ StreamParams p) {
    using L = Loader<T>;
    extern __shared__ __align__(16) uint32_t dyn_smem[];
    __shared__ StreamShared sh;

    const uint32_t tid = threadIdx.x;
    const uint32_t split = blockIdx.x, row = blockIdx.y;
    const SamplerConfig cfg = p.config_count > 1 ? p.configs[row] : p.config0;
    const bool shard_mode = p.shard_k != 0;
    // (a shard of a greedy row keeps k_shard candidates like any other, and on top of them
    // notes the NaN/Inf the argmax order would put first: the merge must see it)
    const bool greedy = cfg.temperature == 0.0f;
    if (!shard_mode && !greedy && cfg.top_k == 0) return;  // rows without a top-k cut use the nucleus kernel

    const uint32_t lo = split * p.split_len;
    const T *columns = static_cast<const T *>(p.logits) + (size_t)row * p.row_stride + lo;
    RowState state;
    state.n = min(p.split_len, p.vocab - lo);
    state.id_base = p.vocab_offset + lo;
    state.k = shard_mode ? p.shard_k : (greedy ? 1u : cfg.top_k);
    state.greedy = greedy;
    state.aligned = (reinterpret_cast<uintptr_t>(columns) & 15u) == 0;
    // without a count array frequency is +-0 and the product does not depend on the count
    state.flat_offset = penalty_offset(1u, cfg.presence_penalty, cfg.frequency_penalty);
    state.presence = cfg.presence_penalty;
    state.frequency = cfg.frequency_penalty;
    state.repetition = make_repetition(cfg.repetition_penalty);

    if (tid == 0) {
        sh.cand.count = 0;
        sh.cand.tau_score = __uint_as_float(0xff800000u);
        sh.cand.tau_id = kPaddingId;
        sh.bad_history = 0;
        sh.wild_key = ~0ull;
        sh.distinct = 0;
        sh.overflow = 0;
    }
    __syncthreads();

    // ---- 1. history slice -> bitmap / running popcount / offsets ----
    state.flags = build_history(p, sh, dyn_smem, row, lo, state.n, cfg);

    // ---- 2. stream the columns ----
    // Tiles 1 .. full-1 of a 16-byte aligned row take the fast loop below: 128-bit
    // loads at constant offsets from one running pointer (next tile in flight while
    // this one is examined), one bitmap word per vector, one compare per vector.
    // Everything else goes through careful_tile.
    const uint32_t n = state.n;
    const uint32_t tiles = (n + kTile - 1) / kTile;
    const uint32_t full_tiles = state.aligned ? n / kTile : 0;
    float tau = careful_tile<T>(p, sh, dyn_smem, columns, 0, state, __uint_as_float(0xff800000u));

    // can the row's penalties only lower a logit?  (rows without history count as such)
    const bool lowering = !(state.flags & kSeenAny) ||
                          (cfg.presence_penalty >= 0.0f && cfg.frequency_penalty >= 0.0f &&
                           cfg.repetition_penalty >= 1.0f && state.repetition.tame);
    for (uint32_t t = 1; t < full_tiles;) {
        const uint32_t stopped =
            lowering ? fast_tiles<T, true>(p, sh, dyn_smem, columns, t, full_tiles, state, tau)
                     : fast_tiles<T, false>(p, sh, dyn_smem, columns, t, full_tiles, state, tau);
        t = (stopped & ~kNeedsAttention) + 1;
        if (stopped & kNeedsAttention) {
            // a tile pushed more than the list holds: feed it again in pieces;
            // otherwise the list is merely long: cut it, which lifts the bound
            if (sh.overflow) tau = redo_tile<T>(p, sh, dyn_smem, columns, t - 1, state);
            else tau = cut_list(sh, state.k);
        }
    }
    // the ragged end of an aligned row, or every further tile of an unaligned one
    for (uint32_t t = full_tiles > 1 ? full_tiles : 1; t < tiles; t++)
        tau = careful_tile<T>(p, sh, dyn_smem, columns, t, state, tau);

    // ---- 3./4. this split's k best, the row's result ----
    finish_split(p, sh, row, split, state.k, greedy, shard_mode, cfg);
}


// ================================================================== history pass
//
// The history structures of a whole batch, built by a pass of their own into global
// memory: the kernel without a top-k cut reads them from there.

// Per (row, split): what build_history returned and the status a broken history earns.
struct alignas(8) HistoryMeta {
    uint32_t flags;
    uint32_t bad_history;
};

// build_history in shared memory, then the structure is copied verbatim to the unit's
// slot in global memory.
__global__ void __launch_bounds__(kThreads) history_build_kernel(const __grid_constant__ StreamParams p) {
    extern __shared__ __align__(16) uint32_t dyn_smem[];
    __shared__ StreamShared sh;
    const uint32_t tid = threadIdx.x;
    const uint32_t split = blockIdx.x, row = blockIdx.y;
    const SamplerConfig cfg = p.config_count > 1 ? p.configs[row] : p.config0;
    const uint32_t lo = split * p.split_len;
    const uint32_t n = min(p.split_len, p.vocab - lo);
    if (tid == 0) {
        sh.bad_history = 0;
        sh.distinct = 0;
    }
    __syncthreads();
    const uint32_t flags = build_history(p, sh, dyn_smem, row, lo, n, cfg);
    __syncthreads();
    const size_t unit = (size_t)row * p.splits + split;
    if (flags) {
        uint32_t *out = p.history_global + unit * p.history_stride_words;
        const uint32_t words = (uint32_t)p.history_stride_words;
        for (uint32_t i = tid; i < words; i += kThreads) out[i] = dyn_smem[i];
    }
    if (tid == 0) {
        HistoryMeta meta;
        meta.flags = flags;
        meta.bad_history = sh.bad_history;
        reinterpret_cast<HistoryMeta *>(p.history_meta)[unit] = meta;
    }
}

// ---------------------------------------------------------------- merge kernel
//
// One CTA per row over `shards` blocks of k_shard candidates each (the layout an
// all-gather leaves: [shard][row][k_shard]); also serves fg_sampler_select
// (one row, one shard, count candidates).  Range check and fold follow
// worker_output_split_combine, src/runtime.c:2437-2466.

struct MergeParams {
    const float *scores;
    const uint32_t *ids;
    uint32_t rows, shards, k_shard;
    uint32_t stride;                // elements between consecutive candidates (2: interleaved (value, id) pairs)
    uint64_t shard_pitch;           // candidates between consecutive shards' blocks
    uint32_t *arrived;              // fused exchange: per-row arrival counters of this rank's window
    uint32_t arrival_target, wait_polls;
    uint32_t check_spans;           // sharded merge: range-check ids, a NaN/Inf finalist is an error
    uint32_t span_first[16], span_width[16];
    const SamplerConfig *configs;
    SamplerConfig config0;
    uint32_t config_count;
    const float *uniforms;
    SelectOutput out;
};

__global__ void __launch_bounds__(kThreads) merge_select_kernel(const MergeParams p) {
    __shared__ StreamShared sh;
    const uint32_t tid = threadIdx.x, row = blockIdx.x;
    const SamplerConfig cfg = p.config_count > 1 ? p.configs[row] : p.config0;
    const bool greedy = cfg.temperature == 0.0f;
    const uint32_t k = greedy ? 1u : cfg.top_k;
    if (tid == 0) {
        sh.cand.count = 0;
        sh.bad_history = 0;
        sh.wild_id = kPaddingId;
        sh.wild_bits = 0;
        sh.is_last = 1;
        if (p.arrived != nullptr) {
            // The fused exchange: every rank's shard kernel stores its block of this row into
            // this rank's window and then counts itself in.  Wait for all of them -- bounded:
            // a rank that never comes fails the row instead of hanging the GPU.
            const uint32_t polls = p.wait_polls ? p.wait_polls : (1u << 21);
            uint32_t seen = 0;
            for (uint32_t i = 0; i < polls; i++) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.arrived + row) : "memory");
                if (seen >= p.arrival_target) break;
                __nanosleep(1000);
            }
            if (seen < p.arrival_target) sh.is_last = 0;
            // all are in: the counter starts from zero again for the call after next, which is
            // the earliest any rank can store into this half of the window again
            else p.arrived[row] = 0;
        }
    }
    __syncthreads();
    if (!sh.is_last) {  // not every rank's candidates came: FG_ERR_LIMIT, as a partial that misses its deadline
        if (tid == 0) {
            report_row(p.out, row, kErrLimit, kPaddingId, 0.0f);
            atomicMin(p.out.first_error + 1, 1ull);
            if (p.out.dbg_count) p.out.dbg_count[row] = 0;
        }
        return;
    }
    const uint32_t total = p.shards * p.k_shard;  // <= kCandCap, checked by the host
    for (uint32_t i = tid; i < total; i += kThreads) {
        const uint32_t shard = i / p.k_shard, within = i % p.k_shard;
        const size_t at = ((size_t)shard * p.shard_pitch + (size_t)row * p.k_shard + within) * p.stride;
        const float score = p.scores[at];
        const uint32_t id = p.ids[at];
        if (id == kPaddingId && p.check_spans) continue;  // padding of a short shard
        if (p.check_spans && (id < p.span_first[shard] || id - p.span_first[shard] >= p.span_width[shard]))
            sh.bad_history = 1;  // id outside its shard's span
        if (is_nonfinite(score)) {
            if (greedy && p.check_spans) atomicMin(&sh.wild_id, id);
            continue;  // the select step drops non-finite candidates, src/sampler.c:89
        }
        const uint32_t slot = atomicAdd(&sh.cand.count, 1u);
        sh.cand.score[slot] = score;
        sh.cand.id[slot] = id;
    }
    __syncthreads();
    if (greedy && sh.wild_id != kPaddingId) {
        for (uint32_t i = tid; i < total; i += kThreads) {
            const uint32_t shard = i / p.k_shard, within = i % p.k_shard;
            const size_t at = ((size_t)shard * p.shard_pitch + (size_t)row * p.k_shard + within) * p.stride;
            if (p.ids[at] == sh.wild_id && is_nonfinite(p.scores[at]))
                sh.wild_bits = __float_as_uint(p.scores[at]);
        }
    }
    __syncthreads();
    if (sh.bad_history) {
        if (tid == 0) {
            report_row(p.out, row, kErrMismatch, kPaddingId, 0.0f);
            if (p.out.dbg_count) p.out.dbg_count[row] = 0;
        }
        return;
    }
    uint32_t held = sh.cand.count;
    __syncthreads();
    held = compact_topk<kThreads, kCandCap>(sh.cand, held, k);
    if (greedy) {
        if (tid == 0) {
            uint32_t status = kOk, token = kPaddingId;
            float logit = 0.0f;
            if (sh.wild_id != kPaddingId) {
                status = kErrMismatch;  // "invalid combined output finalist", runtime.c:2461-2463
                token = sh.wild_id;
                logit = __uint_as_float(sh.wild_bits);
            } else if (held == 0) {
                status = p.check_spans ? kErrMismatch : kErrFormat;
            } else {
                token = sh.cand.id[0];
                logit = sh.cand.score[0];
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
    sort_candidates(sh.cand, sh.fin, held);
    if (tid < 32) finish_select(sh.fin, held, cfg, p.uniforms ? p.uniforms[row] : 0.0f, row, p.out);
}

}  // namespace fgk

// ------------------------------------------------------------------ launchers

using namespace fgk;

static SelectOutput make_output(const fgk_select_output *o) {
    SelectOutput out;
    out.tokens = o->tokens;
    out.token_logits = o->token_logits;
    out.row_status = o->row_status;
    out.first_error = reinterpret_cast<unsigned long long *>(o->first_error);
    out.dbg_count = o->dbg_count;
    out.dbg_ids = o->dbg_ids;
    out.dbg_scores = o->dbg_scores;
    out.dbg_raw = o->dbg_raw;
    out.dbg_tempered = o->dbg_tempered;
    return out;
}

static SamplerConfig to_device_config(const fg_sampler_config *c) {
    SamplerConfig d;
    d.temperature = c->temperature;
    d.top_p = c->top_p;
    d.top_k = c->top_k;
    d.presence_penalty = c->presence_penalty;
    d.frequency_penalty = c->frequency_penalty;
    d.repetition_penalty = c->repetition_penalty;
    d.min_p = c->min_p;
    d.pad_ = 0;
    d.seed = c->seed;
    return d;
}

extern "C" uint32_t fgk_stream_max_splits(void) { return kMaxSplits; }
extern "C" uint32_t fgk_stream_tile(void) { return kTile; }
extern "C" uint64_t fgk_stream_part_meta_bytes(void) { return sizeof(PartMeta); }

// bitmap words, then (only when counts are kept) 16-bit running popcounts and the
// dense counts, 16 or 32 bits each
extern "C" uint64_t fgk_stream_dynamic_smem(uint32_t bitmap_words, uint32_t count_capacity,
                                            uint32_t dense_wide) {
    uint64_t words = bitmap_words;
    if (count_capacity)
        words += (bitmap_words + 1) / 2 + (dense_wide ? count_capacity : (count_capacity + 1) / 2);
    return words * sizeof(uint32_t);
}

extern "C" int fgk_stream_prepare(void) {
    // opt in to the large dynamic shared-memory carve-out once per process
    cudaError_t e = cudaFuncSetAttribute(stream_select_kernel<float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FGK_STREAM_MAX_DYNAMIC_SMEM);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(stream_select_kernel<uint16_t>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 FGK_STREAM_MAX_DYNAMIC_SMEM);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(history_build_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 FGK_STREAM_MAX_DYNAMIC_SMEM);
    return (int)e;
}

static StreamParams to_stream_params(const fgk_stream_launch *l) {
    StreamParams p;
    p.logits = l->logits;
    p.row_stride = l->row_stride;
    p.rows = l->rows;
    p.vocab = l->vocab;
    p.vocab_offset = l->vocab_offset;
    p.vocab_total = l->vocab_total;
    p.splits = l->splits;
    p.split_len = l->split_len;
    p.history_tokens = l->history_tokens;
    p.history_offsets = l->history_offsets;
    p.configs = reinterpret_cast<const SamplerConfig *>(l->configs_device);
    p.config0 = to_device_config(&l->config0);
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
    p.part_scores = l->part_scores;
    p.part_ids = l->part_ids;
    p.part_meta = reinterpret_cast<PartMeta *>(l->part_meta);
    p.tickets = l->tickets;
    p.history_max = l->history_max;
    p.bitmap_words = l->bitmap_words;
    p.count_capacity = l->count_capacity;
    p.dense_wide = l->dense_wide;
    p.history_global = l->history_global;
    p.history_stride_words = l->history_stride_words;
    p.history_meta = l->history_meta;
    p.out = make_output(&l->out);
    return p;
}

extern "C" int fgk_launch_stream_select(const fgk_stream_launch *l, void *stream) {
    const StreamParams p = to_stream_params(l);
    const dim3 grid(l->splits, l->rows);
    const size_t dynamic = fgk_stream_dynamic_smem(l->bitmap_words, l->count_capacity, l->dense_wide);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (l->dtype == 1u)
        stream_select_kernel<uint16_t><<<grid, kThreads, dynamic, s>>>(p);
    else
        stream_select_kernel<float><<<grid, kThreads, dynamic, s>>>(p);
    return (int)cudaGetLastError();
}

extern "C" int fgk_launch_history_build(const fgk_stream_launch *l, void *stream) {
    const StreamParams p = to_stream_params(l);
    const size_t dynamic = fgk_stream_dynamic_smem(l->bitmap_words, l->count_capacity, l->dense_wide);
    history_build_kernel<<<dim3(l->splits, l->rows), kThreads, dynamic, static_cast<cudaStream_t>(stream)>>>(p);
    return (int)cudaGetLastError();
}

extern "C" int fgk_launch_merge_select(const fgk_merge_launch *l, void *stream) {
    MergeParams p;
    p.scores = l->scores;
    p.ids = l->ids;
    p.rows = l->rows;
    p.shards = l->shards;
    p.k_shard = l->k_shard;
    p.stride = l->stride ? l->stride : 1u;
    p.shard_pitch = l->shard_pitch ? l->shard_pitch : (uint64_t)l->rows * l->k_shard;
    p.arrived = l->arrived;
    p.arrival_target = l->arrival_target;
    p.wait_polls = l->wait_polls;
    p.check_spans = l->check_spans;
    for (int i = 0; i < 16; i++) {
        p.span_first[i] = l->span_first[i];
        p.span_width[i] = l->span_width[i];
    }
    p.configs = reinterpret_cast<const SamplerConfig *>(l->configs_device);
    p.config0 = to_device_config(&l->config0);
    p.config_count = l->config_count;
    p.uniforms = l->uniforms;
    p.out = make_output(&l->out);
    merge_select_kernel<<<l->rows, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return (int)cudaGetLastError();
}

// ------------------------------------------------- scratch that nobody allocates
//
// For callers that cannot allocate device memory at all, the hand-off area of the
// split path lives in the library image itself: every GPU that loads the library
// carries these 4 MiB until the process exits.  In host code the array's name is
// only a stand-in for the symbol; the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.

static __device__ __align__(256) unsigned char fgk_static_scratch[FGK_STATIC_SCRATCH_BYTES];

extern "C" int fgk_static_scratch_address(int device, void **address) {
    static void *known[64];
    if (device < 0 || device >= 64) return (int)cudaErrorInvalidDevice;
    if (!known[device]) {
        int current = -1;
        cudaError_t e = cudaGetDevice(&current);
        if (e != cudaSuccess) return (int)e;
        if (current != device) return (int)cudaErrorInvalidDevice;  // the caller makes it current first
        void *found = nullptr;
        e = cudaGetSymbolAddress(&found, fgk_static_scratch);
        if (e != cudaSuccess) return (int)e;
        // the kernel's shared-memory opt-in belongs to the same once-per-device set-up
        const int prepared = fgk_stream_prepare();
        if (prepared != 0) return prepared;
        known[device] = found;
    }
    *address = known[device];
    return 0;
}
