// Device operators with the dispatch shape of the reference's three sampler
// shaders (one launch = one dispatch of the reference's cascade):
//   apply_penalties  shaders/fg_apply_penalties.comp   (src/vk.c:1808-1824)
//   argmax_reduce    shaders/fg_argmax_reduce.comp     (src/vk.c:2260)
//   topk_select      shaders/fg_topk_select*.comp      (src/vk.c:2237-2256)
// plus the history count table of src/output.c:601-628.
// The fused batched path (fg_stream_kernels.cu) does not go through these; they
// exist so code written against the reference's operator level keeps working.
#include "fg_block_select.cuh"
#include "fg_kernels.h"

namespace fgk {

constexpr int kOpThreads = 256;

// ---- penalties: 4 logits and 4 counts per thread per step, 128-bit accesses ----
__global__ void __launch_bounds__(kOpThreads)
apply_penalties_kernel(float *logits, const uint32_t *counts, uint32_t values, float presence,
                       float frequency, float repetition, bool vector_ok) {
    const uint32_t stride = gridDim.x * blockDim.x;
    const uint32_t thread = blockIdx.x * blockDim.x + threadIdx.x;
    if (vector_ok) {
        const uint32_t quads = values >> 2;
        for (uint32_t q = thread; q < quads; q += stride) {
            const uint4 seen = load_stream_128(counts + 4 * (size_t)q);
            if ((seen.x | seen.y | seen.z | seen.w) == 0) continue;  // nothing to rewrite
            float4 v = *reinterpret_cast<const float4 *>(logits + 4 * (size_t)q);
            if (seen.x) v.x = penalise(v.x, seen.x, presence, frequency, repetition);
            if (seen.y) v.y = penalise(v.y, seen.y, presence, frequency, repetition);
            if (seen.z) v.z = penalise(v.z, seen.z, presence, frequency, repetition);
            if (seen.w) v.w = penalise(v.w, seen.w, presence, frequency, repetition);
            *reinterpret_cast<float4 *>(logits + 4 * (size_t)q) = v;
        }
        for (uint32_t i = (quads << 2) + thread; i < values; i += stride) {
            const uint32_t seen = counts[i];
            if (seen) logits[i] = penalise(logits[i], seen, presence, frequency, repetition);
        }
    } else {
        for (uint32_t i = thread; i < values; i += stride) {
            const uint32_t seen = counts[i];
            if (seen) logits[i] = penalise(logits[i], seen, presence, frequency, repetition);
        }
    }
}

// ---- argmax: one winner per 4096-element tile ----
__global__ void __launch_bounds__(kOpThreads)
argmax_reduce_kernel(float *out_scores, uint32_t *out_ids, const float *scores,
                     const uint32_t *ids, uint32_t count) {
    __shared__ float warp_score[kOpThreads / 32];
    __shared__ uint32_t warp_id[kOpThreads / 32];
    const uint32_t base = blockIdx.x * 4096u;
    float best = __uint_as_float(0xff800000u);
    uint32_t best_id = kPaddingId;
#pragma unroll 4
    for (uint32_t item = threadIdx.x; item < 4096u; item += kOpThreads) {
        const uint32_t source = base + item;
        if (source < count) {
            const float score = scores[source];
            const uint32_t id = ids ? ids[source] : source;
            if (argmax_before(score, id, best, best_id)) {
                best = score;
                best_id = id;
            }
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const float other = __shfl_down_sync(kFullMask, best, d);
        const uint32_t other_id = __shfl_down_sync(kFullMask, best_id, d);
        if (argmax_before(other, other_id, best, best_id)) {
            best = other;
            best_id = other_id;
        }
    }
    if ((threadIdx.x & 31u) == 0) {
        warp_score[threadIdx.x >> 5] = best;
        warp_id[threadIdx.x >> 5] = best_id;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kOpThreads / 32; w++) {
            if (argmax_before(warp_score[w], warp_id[w], best, best_id)) {
                best = warp_score[w];
                best_id = warp_id[w];
            }
        }
        out_scores[blockIdx.x] = best;
        out_ids[blockIdx.x] = best_id;
    }
}

// ---- top-k: the k best finite entries of every 1024-element tile ----
__global__ void __launch_bounds__(kOpThreads)
topk_select_kernel(float *out_scores, uint32_t *out_ids, const float *scores,
                   const uint32_t *ids, uint32_t count, uint32_t k) {
    __shared__ CandidateBuffer<1024> cand;
    __shared__ FinishBuffer fin;
    const uint32_t tid = threadIdx.x;
    const uint32_t base = blockIdx.x * 1024u;
    if (tid == 0) cand.count = 0;
    __syncthreads();
    // compacting finite entries with a warp ballot keeps slot order irrelevant:
    // the select below is exact whatever order they arrive in
    for (uint32_t item = tid; item < 1024u; item += kOpThreads) {
        const uint32_t source = base + item;
        bool keep = false;
        float score = 0.0f;
        uint32_t id = kPaddingId;
        if (source < count) {
            score = scores[source];
            id = ids ? ids[source] : source;
            keep = !is_nonfinite(score) && id != kPaddingId;
        }
        const unsigned votes = __ballot_sync(kFullMask, keep);
        if (votes) {
            const int leader = __ffs(votes) - 1;
            uint32_t slot = 0;
            if ((int)(tid & 31u) == leader) slot = atomicAdd(&cand.count, (uint32_t)__popc(votes));
            slot = __shfl_sync(kFullMask, slot, leader) + __popc(votes & ((1u << (tid & 31u)) - 1u));
            if (keep) {
                cand.score[slot] = score;
                cand.id[slot] = id;
            }
        }
    }
    __syncthreads();
    uint32_t held = cand.count;
    __syncthreads();
    held = compact_topk<kOpThreads, 1024>(cand, held, k);
    sort_candidates(cand, fin, held);
    if (tid < k) {
        const size_t at = (size_t)blockIdx.x * k + tid;
        out_scores[at] = tid < held ? fin.score[tid] : __uint_as_float(0xff800000u);
        out_ids[at] = tid < held ? fin.id[tid] : kPaddingId;
    }
}

// ---- history: saturating occurrence counts ----
__global__ void __launch_bounds__(kOpThreads)
history_add_kernel(uint32_t *counts, uint32_t vocab, const uint32_t *history, uint32_t count,
                   uint32_t *bad) {
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const uint32_t token = history[i];
        if (token >= vocab) {
            atomicMin(bad, i);  // first offending position, src/output.c:610-612
            continue;
        }
        uint32_t seen = counts[token];
        while (seen != 0xffffffffu) {  // saturate, src/output.c:613
            const uint32_t was = atomicCAS(&counts[token], seen, seen + 1u);
            if (was == seen) break;
            seen = was;
        }
    }
}

// ---- sorted top-512 of every 4096-element tile ----
// shaders/fg_topk_reduce_v2.comp:10, 27-85: the best 512 (score, id) pairs of the tile in the
// order `before`: a padding id (0xffffffff) last; a NaN/Inf before every finite score, smaller
// id first among them; then larger score, then smaller id.  The shader sorts 64-slot runs
// and merges them pairwise; here the tile's 4096 64-bit keys are sorted by one bitonic
// network in shared memory -- the key is the order: class and score in the high word, the
// inverted id in the low word -- and each key drags along its position in the tile, from
// which the untouched score bits (NaN payloads, the sign of zero) are fetched at the end.
constexpr int kReduceTile = 4096, kReduceKeep = 512, kReduceThreads = 1024;

__device__ __forceinline__ uint64_t reduce_key(float score, uint32_t id) {
    if (id == kPaddingId) return 0ull;
    const uint32_t high = is_nonfinite(score) ? 0xffffffffu : float_key(score);  // finite keys stop at 0xff7fffff
    return ((uint64_t)high << 32) | (uint64_t)(~id);
}

__global__ void __launch_bounds__(kReduceThreads)
topk_reduce_kernel(float *out_scores, uint32_t *out_ids, const float *scores, const uint32_t *ids,
                   uint32_t count, uint32_t produced) {
    __shared__ uint64_t key[kReduceTile];
    __shared__ uint16_t from[kReduceTile];
    const uint32_t tid = threadIdx.x, base = blockIdx.x * kReduceTile;
    const uint32_t here = min((uint32_t)kReduceTile, count - base);
    for (uint32_t i = tid; i < (uint32_t)kReduceTile; i += kReduceThreads) {
        key[i] = i < here ? reduce_key(scores[base + i], ids ? ids[base + i] : base + i) : 0ull;
        from[i] = (uint16_t)i;
    }
    __syncthreads();
    for (uint32_t size = 2; size <= (uint32_t)kReduceTile; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            for (uint32_t pair = tid; pair < (uint32_t)kReduceTile / 2; pair += kReduceThreads) {
                // the pair's lower index: `pair` with a zero bit slipped in at `stride`
                const uint32_t low = ((pair & ~(stride - 1)) << 1) | (pair & (stride - 1));
                const uint32_t high = low | stride;
                const bool descending = (low & size) == 0;
                const uint64_t a = key[low], b = key[high];
                if ((a < b) == descending) {
                    key[low] = b;
                    key[high] = a;
                    const uint16_t moved = from[low];
                    from[low] = from[high];
                    from[high] = moved;
                }
            }
            __syncthreads();
        }
    }
    const uint32_t valid = min((uint32_t)kReduceKeep, here);
    for (uint32_t i = tid; i < (uint32_t)kReduceKeep; i += kReduceThreads) {
        const uint32_t at = blockIdx.x * kReduceKeep + i;
        if (at >= produced) continue;  // (a lone short tile hands back `count` entries, src/vk.c:2235)
        const uint32_t source = base + from[i];
        out_scores[at] = i < valid ? scores[source] : __uint_as_float(0xff800000u);
        out_ids[at] = i < valid ? (ids ? ids[source] : source) : kPaddingId;
    }
}

// ---- router: the k best of each token's expert logits and their gate weights ----
// src/q38_math.c:48-64 (fg_q38_router_topk): softmax over all experts in fp64, the k largest
// logits (ties: smaller id), their probabilities rounded to fp32 and renormalised by their
// fp64 sum.  A NaN or +Inf logit makes the token's probabilities meaningless: the ids come
// back as 0xffffffff and the weights as 0 (shaders/fg_router_top10.glsl:38-51), and the call
// reports it.  One warp per token.
__global__ void __launch_bounds__(128)
router_topk_kernel(uint32_t *out_ids, float *out_weights, const float *logits, uint32_t tokens,
                   uint32_t experts, uint32_t k, uint32_t *bad) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= tokens) return;
    const float *row = logits + (size_t)token * experts;
    float top = __uint_as_float(0xff800000u);
    bool broken = false;
    for (uint32_t i = lane; i < experts; i += 32) {
        const float v = row[i];
        broken = broken || v != v || v == __uint_as_float(0x7f800000u);
        top = fmaxf(top, v);
    }
    broken = __any_sync(kFullMask, broken);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) top = fmaxf(top, __shfl_xor_sync(kFullMask, top, d));
    double total = 0.0;
    for (uint32_t i = lane; i < experts; i += 32) total += exp((double)row[i] - (double)top);
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) total += __shfl_xor_sync(kFullMask, total, d);
    if (broken || !(total > 0.0)) {
        for (uint32_t slot = lane; slot < k; slot += 32) {
            out_ids[(size_t)token * k + slot] = kPaddingId;
            out_weights[(size_t)token * k + slot] = 0.0f;
        }
        if (lane == 0) atomicMin(bad, token);
        return;
    }
    // k rounds of "the best that is not taken yet"; a lane remembers what it gave away
    uint64_t floor_key = ~0ull;  // keys at or above this have been taken
    double picked_sum = 0.0;
    float my_weight = 0.0f;
    uint32_t my_id = kPaddingId;
    for (uint32_t slot = 0; slot < k; slot++) {
        uint64_t best = 0;
        for (uint32_t i = lane; i < experts; i += 32) {
            const uint64_t candidate = ((uint64_t)float_key(row[i]) << 32) | (uint64_t)(~i);
            if (candidate < floor_key && candidate > best) best = candidate;
        }
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) {
            const uint64_t other = __shfl_xor_sync(kFullMask, best, d);
            best = other > best ? other : best;
        }
        floor_key = best;
        const uint32_t id = ~(uint32_t)best;
        const float weight = (float)(exp((double)row[id] - (double)top) / total);
        picked_sum += (double)weight;
        if (lane == slot % 32u) {  // (k <= 32: one slot per lane)
            my_id = id;
            my_weight = weight;
        }
    }
    if (lane < k) {
        out_ids[(size_t)token * k + lane] = my_id;
        out_weights[(size_t)token * k + lane] = (float)((double)my_weight / picked_sum);
    }
}

// ---- the executor's session tables ----
// After a step: src/output.c:742, 752 -- a token picked with penalties active joins its
// session's history; the count saturates as in src/output.c:619-628.
__global__ void __launch_bounds__(kOpThreads)
session_increment_kernel(uint32_t *slot_counts, uint32_t *slot_bitmaps, uint32_t vocab,
                         uint32_t slot_bitmap_words, const uint32_t *row_slots, const uint32_t *tokens,
                         const uint32_t *row_status, const unsigned char *active, uint32_t rows) {
    const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows || !active[row] || row_status[row] != 0u) return;
    const uint32_t token = tokens[row];
    if (token >= vocab) return;
    uint32_t *counts = slot_counts + (size_t)row_slots[row] * vocab;
    uint32_t seen = counts[token];
    while (seen != 0xffffffffu) {  // two rows of a batch may share a session
        const uint32_t was = atomicCAS(&counts[token], seen, seen + 1u);
        if (was == seen) break;
        seen = was;
    }
    atomicOr(&slot_bitmaps[(size_t)row_slots[row] * slot_bitmap_words + (token >> 5)], 1u << (token & 31u));
}

__global__ void __launch_bounds__(kOpThreads)
session_bitmap_kernel(uint32_t *bitmap, const uint32_t *counts, uint32_t vocab, uint32_t bitmap_words) {
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t word = blockIdx.x * blockDim.x + threadIdx.x; word < bitmap_words; word += stride) {
        uint32_t bits = 0;
        for (uint32_t b = 0; b < 32u; b++) {
            const uint32_t token = word * 32u + b;
            if (token < vocab && counts[token] != 0u) bits |= 1u << b;
        }
        bitmap[word] = bits;
    }
}

}  // namespace fgk

using namespace fgk;

static uint32_t blocks_for(uint32_t items_per_block_step, uint32_t items) {
    uint32_t blocks = (items + items_per_block_step - 1) / items_per_block_step;
    if (blocks == 0) blocks = 1;
    if (blocks > 148u * 8u) blocks = 148u * 8u;  // a few CTAs per SM, grid-stride beyond
    return blocks;
}

extern "C" int fgk_launch_apply_penalties(float *logits, const uint32_t *counts, uint32_t values,
                                          float presence, float frequency, float repetition,
                                          void *stream) {
    const bool vector_ok = ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(counts)) & 15u) == 0;
    apply_penalties_kernel<<<blocks_for(kOpThreads * 4, values), kOpThreads, 0,
                             static_cast<cudaStream_t>(stream)>>>(logits, counts, values, presence,
                                                                   frequency, repetition, vector_ok);
    return (int)cudaGetLastError();
}

extern "C" int fgk_launch_apply_penalties_seen(float *scores, const uint32_t *seen, uint32_t values,
                                               float presence, float frequency, float repetition,
                                               void *stream) {
    return fgk_launch_apply_penalties(scores, seen, values, presence, frequency, repetition, stream);
}

extern "C" int fgk_launch_argmax_reduce(float *out_scores, uint32_t *out_ids, const float *scores,
                                        const uint32_t *ids, uint32_t count, void *stream) {
    const uint32_t groups = (count + 4095u) / 4096u;
    argmax_reduce_kernel<<<groups, kOpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        out_scores, out_ids, scores, ids, count);
    return (int)cudaGetLastError();
}

extern "C" int fgk_launch_topk_select(float *out_scores, uint32_t *out_ids, const float *scores,
                                      const uint32_t *ids, uint32_t count, uint32_t k,
                                      void *stream) {
    const uint32_t groups = (count + 1023u) / 1024u;
    topk_select_kernel<<<groups, kOpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        out_scores, out_ids, scores, ids, count, k);
    return (int)cudaGetLastError();
}

extern "C" int fgk_launch_history_add(uint32_t *counts, uint32_t vocab, const uint32_t *history,
                                      uint32_t count, uint32_t *bad, void *stream) {
    if (count == 0) return 0;
    history_add_kernel<<<blocks_for(kOpThreads, count), kOpThreads, 0,
                         static_cast<cudaStream_t>(stream)>>>(counts, vocab, history, count, bad);
    return (int)cudaGetLastError();
}

extern "C" int fgk_launch_session_increment(uint32_t *slot_counts, uint32_t *slot_bitmaps, uint32_t vocab,
                                            uint32_t slot_bitmap_words, const uint32_t *row_slots,
                                            const uint32_t *tokens, const uint32_t *row_status,
                                            const unsigned char *active, uint32_t rows, void *stream) {
    if (rows == 0) return 0;
    session_increment_kernel<<<(rows + kOpThreads - 1) / kOpThreads, kOpThreads, 0,
                               static_cast<cudaStream_t>(stream)>>>(slot_counts, slot_bitmaps, vocab,
                                                                    slot_bitmap_words, row_slots, tokens,
                                                                    row_status, active, rows);
    return (int)cudaGetLastError();
}

extern "C" int fgk_launch_session_bitmap(uint32_t *bitmap, const uint32_t *counts, uint32_t vocab,
                                         uint32_t bitmap_words, void *stream) {
    session_bitmap_kernel<<<blocks_for(kOpThreads, bitmap_words), kOpThreads, 0,
                            static_cast<cudaStream_t>(stream)>>>(bitmap, counts, vocab, bitmap_words);
    return (int)cudaGetLastError();
}

extern "C" int fgk_launch_topk_reduce(float *out_scores, uint32_t *out_ids, const float *scores,
                                      const uint32_t *ids, uint32_t count, uint32_t produced, void *stream) {
    const uint32_t groups = (count + kReduceTile - 1) / kReduceTile;
    topk_reduce_kernel<<<groups, kReduceThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        out_scores, out_ids, scores, ids, count, produced);
    return (int)cudaGetLastError();
}

extern "C" int fgk_launch_router_topk(uint32_t *out_ids, float *out_weights, const float *logits,
                                      uint32_t tokens, uint32_t experts, uint32_t k, uint32_t *bad,
                                      void *stream) {
    router_topk_kernel<<<(tokens + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        out_ids, out_weights, logits, tokens, experts, k, bad);
    return (int)cudaGetLastError();
}
