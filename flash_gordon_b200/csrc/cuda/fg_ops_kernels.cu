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
