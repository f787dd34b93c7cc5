/* Shared between the host translation units; not installed. */
#ifndef FG_B200_HOST_INTERNAL_H
#define FG_B200_HOST_INTERNAL_H

#include "fg_cuda_sampler.h"
#include "../cuda/fg_kernels.h"

struct fg_cuda_context {
    int device;
    void *own_stream;
    void *stream;
    uint32_t sm_count;
    bool batch_active;
    uint64_t launches;
    uint32_t forced_splits;
    uint32_t path;          /* FG_CUDA_PATH_* */
    /* test seam of the ring kernel (fg_cuda_internal_ring_controls) */
    uint32_t ring_deal, ring_wait_polls, ring_withhold_armed, ring_withhold_cta, ring_withhold_issue;

    /* Set by the stateful executor around a call: the batch's penalties come from session
     * tables (counts [slots][vocab], seen-bitmaps [slots][words], one session index per row)
     * instead of token lists.  Only the ring kernel reads them. */
    const uint32_t *session_counts;
    const uint32_t *session_bitmaps;
    const uint32_t *session_rows;
    uint32_t session_bitmap_words;

    /* Set by the multi-GPU layer around a shard step whose candidates go straight to the
     * ranks' windows (the fused exchange) instead of to a local buffer. */
    const fgk_push *push;

    /* device scratch, grown on demand and then reused (no allocation on a warm call) */
    void *parts;            /* candidate hand-off between the splits of a row */
    size_t parts_bytes;
    uint32_t *tickets;      /* one arrival counter per row, zero between launches */
    size_t tickets_bytes;
    void *history;          /* ring path: history structures, one per (row, split) */
    size_t history_bytes;
    void *nucleus;          /* one fp32 scratch row per persistent CTA of the nucleus kernel */
    size_t nucleus_bytes;
    void *configs;          /* per-row configs when they differ */
    size_t configs_bytes;
    uint64_t *first_error;  /* one device word */
    void *staging;          /* host-entry inputs and outputs */
    size_t staging_bytes;
    void *pinned;           /* pinned host bounce buffer */
    size_t pinned_bytes;
    uint64_t last_scratch_bytes;
};

struct fg_cuda_tensor {
    fg_cuda_context *context;
    unsigned char *base;
    uint64_t bytes;
    bool owns;
};

/* cudaError_t (as int) -> fg_status with a message naming `what`. */
fg_status fg_cuda_fail(fg_error *err, int cuda_error, const char *what);
/* Makes the context's device current; FG_ERR_UNAVAILABLE on failure. */
fg_status fg_cuda_enter(fg_cuda_context *context, fg_error *err);
/* Grow-only device buffer. */
fg_status fg_cuda_reserve(void **buffer, size_t *have, size_t want, bool zero,
                          fg_cuda_context *context, fg_error *err);
fg_status fg_cuda_reserve_pinned(fg_cuda_context *context, size_t want, fg_error *err);
/* Process-wide context used by the host-pointer fg_sampler_* entry points. */
fg_status fg_cuda_default_context(fg_cuda_context **out, fg_error *err);
void fg_cuda_default_lock(void);
void fg_cuda_default_unlock(void);
fg_status fg_cuda_internal_ring_controls(fg_cuda_context *context, uint32_t deal, uint32_t wait_polls,
                                         uint32_t armed, uint32_t cta, uint32_t issue);
/* The two steps of the vocabulary-sharded mode with an explicit candidate layout (stride 1:
 * separate score and id arrays; 2: interleaved (value, id) pairs); both only enqueue.  The
 * multi-GPU layer calls them with its exchange buffers. */
fg_status fg_cuda_shard_topk_layout(fg_cuda_context *context, const fg_cuda_sample_args *args,
                                    uint32_t vocab_offset, uint32_t vocab_total, uint32_t k_shard,
                                    float *candidate_scores, uint32_t *candidate_ids, uint32_t stride,
                                    fg_error *err);
/* the merge step of the fused exchange: where the shards' blocks lie in this rank's window,
 * and the arrival counters it waits on (bounded) before it reads a row */
typedef struct fg_cuda_arrivals {
    uint64_t shard_pitch;     /* candidates between consecutive shards' blocks */
    uint32_t *arrived;        /* one counter per row; set back to zero by the merge */
    uint32_t target;          /* a row is complete at this count */
    uint32_t wait_polls;      /* 0: about two seconds */
} fg_cuda_arrivals;
fg_status fg_cuda_merge_select_layout(fg_cuda_context *context, const fg_cuda_sample_args *args,
                                      const float *candidate_scores, const uint32_t *candidate_ids,
                                      uint32_t stride, uint32_t shards, uint32_t k_shard,
                                      const uint32_t *shard_first, const uint32_t *shard_width,
                                      bool keep_errors, const fg_cuda_arrivals *arrivals, fg_error *err);
/* Waits for the context's stream and turns the device's error word into a status. */
fg_status fg_cuda_collect(fg_cuda_context *context, fg_error *err);
/* fg_sampler_config_validate with the optional "top_k == 0" extension. */
bool fg_cuda_config_ok(const fg_sampler_config *config, bool allow_no_topk);

#endif
