/*
 * Context, tensors and the device-operator / batched entry points of
 * fg_cuda_sampler.h.  This layer is C17: it validates arguments with the
 * reference's rules (src/vk.c:1808-1824, 2237-2256, 2260; src/output.c:601-628,
 * 702-755), plans the launch and calls the CUDA translation units through
 * fg_kernels.h.  It performs no sampling arithmetic itself.
 */
#include "fg_host_internal.h"

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ helpers */

fg_status fg_cuda_fail(fg_error *err, int cuda_error, const char *what) {
    /* cudaErrorMemoryAllocation = 2; no device / no driver = 100 / 35 / 3 */
    fg_status status = FG_ERR_IO;
    if (cuda_error == 2) status = FG_ERR_OOM;
    else if (cuda_error == 100 || cuda_error == 35 || cuda_error == 3 || cuda_error == 101 ||
             cuda_error == 999)
        status = FG_ERR_UNAVAILABLE;
    fg_error_set(err, status, "%s failed: %s (cuda error %d)", what, fgk_error_string(cuda_error),
                 cuda_error);
    return status;
}

fg_status fg_cuda_enter(fg_cuda_context *context, fg_error *err) {
    const int e = fgk_set_device(context->device);
    return e ? fg_cuda_fail(err, e, "selecting the CUDA device") : FG_OK;
}

fg_status fg_cuda_reserve(void **buffer, size_t *have, size_t want, bool zero,
                          fg_cuda_context *context, fg_error *err) {
    if (*have >= want && *buffer) return FG_OK;
    /* growing discards the old contents; wait for work that may still read them */
    int e = fgk_stream_synchronize(context->stream);
    if (e) return fg_cuda_fail(err, e, "draining the stream");
    if (*buffer) fgk_free(*buffer);
    *buffer = NULL;
    *have = 0;
    size_t rounded = (size_t)fg_align_up_u64(want + want / 4u, 256u);
    e = fgk_malloc(buffer, rounded);
    if (e) return fg_cuda_fail(err, e, "allocating device scratch");
    if (zero) {
        e = fgk_memset_async(*buffer, 0, rounded, context->stream);
        if (e) return fg_cuda_fail(err, e, "clearing device scratch");
    }
    *have = rounded;
    return FG_OK;
}

fg_status fg_cuda_reserve_pinned(fg_cuda_context *context, size_t want, fg_error *err) {
    if (context->pinned_bytes >= want && context->pinned) return FG_OK;
    int e = fgk_stream_synchronize(context->stream);
    if (e) return fg_cuda_fail(err, e, "draining the stream");
    if (context->pinned) fgk_host_free(context->pinned);
    context->pinned = NULL;
    context->pinned_bytes = 0;
    size_t rounded = (size_t)fg_align_up_u64(want + want / 4u, 4096u);
    e = fgk_host_alloc(&context->pinned, rounded);
    if (e) return fg_cuda_fail(err, e, "allocating pinned host memory");
    context->pinned_bytes = rounded;
    return FG_OK;
}

/* ------------------------------------------------------------------ context */

fg_status fg_cuda_context_create(int device, fg_cuda_context **out, fg_error *err) {
    if (!out || device < 0) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid CUDA context arguments");
        return FG_ERR_ARGUMENT;
    }
    *out = NULL;
    int count = 0;
    int e = fgk_device_count(&count);
    if (e || count <= 0) {
        fg_error_set(err, FG_ERR_UNAVAILABLE, "no usable CUDA device: %s",
                     e ? fgk_error_string(e) : "device count is zero");
        return FG_ERR_UNAVAILABLE;
    }
    if (device >= count) {
        fg_error_set(err, FG_ERR_ARGUMENT, "CUDA device %d does not exist (%d present)", device, count);
        return FG_ERR_ARGUMENT;
    }
    fg_cuda_context *c = calloc(1, sizeof(*c));
    if (!c) {
        fg_error_set(err, FG_ERR_OOM, "out of host memory");
        return FG_ERR_OOM;
    }
    c->device = device;
    int sms = 0;
    e = fgk_set_device(device);
    if (!e) e = fgk_device_sm_count(device, &sms);
    if (!e) e = fgk_stream_create(&c->own_stream);
    if (!e) e = fgk_stream_prepare();
    if (!e) e = fgk_persistent_prepare();
    if (!e) e = fgk_nucleus_prepare();
    if (!e) e = fgk_malloc((void **)&c->first_error, 256u);
    if (e) {
        fg_status status = fg_cuda_fail(err, e, "opening the CUDA context");
        fg_cuda_context_destroy(c);
        return status;
    }
    c->stream = c->own_stream;
    c->sm_count = (uint32_t)sms;
    *out = c;
    return FG_OK;
}

void fg_cuda_context_destroy(fg_cuda_context *c) {
    if (!c) return;
    if (fgk_set_device(c->device) == 0) {
        if (c->stream) fgk_stream_synchronize(c->stream);
        if (c->parts) fgk_free(c->parts);
        if (c->tickets) fgk_free(c->tickets);
        if (c->configs) fgk_free(c->configs);
        if (c->history) fgk_free(c->history);
        if (c->nucleus) fgk_free(c->nucleus);
        if (c->first_error) fgk_free(c->first_error);
        if (c->staging) fgk_free(c->staging);
        if (c->pinned) fgk_host_free(c->pinned);
        if (c->own_stream) fgk_stream_destroy(c->own_stream);
    }
    free(c);
}

fg_status fg_cuda_context_set_stream(fg_cuda_context *c, void *cuda_stream, fg_error *err) {
    if (!c) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid CUDA context");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    int e = fgk_stream_synchronize(c->stream); /* scratch is shared between the two streams */
    if (e) return fg_cuda_fail(err, e, "draining the stream");
    c->stream = cuda_stream;
    return FG_OK;
}

fg_status fg_cuda_context_reset_stream(fg_cuda_context *c, fg_error *err) {
    return fg_cuda_context_set_stream(c, c ? c->own_stream : NULL, err);
}

void *fg_cuda_context_stream(const fg_cuda_context *c) { return c ? c->stream : NULL; }
int fg_cuda_context_device(const fg_cuda_context *c) { return c ? c->device : -1; }
uint32_t fg_cuda_context_sm_count(const fg_cuda_context *c) { return c ? c->sm_count : 0u; }
uint64_t fg_cuda_context_launches(const fg_cuda_context *c) { return c ? c->launches : 0u; }
uint64_t fg_cuda_context_scratch_bytes(const fg_cuda_context *c) { return c ? c->last_scratch_bytes : 0u; }

fg_status fg_cuda_context_set_splits(fg_cuda_context *c, uint32_t splits, fg_error *err) {
    if (!c || splits > fgk_stream_max_splits()) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid split count");
        return FG_ERR_ARGUMENT;
    }
    c->forced_splits = splits;
    return FG_OK;
}

fg_status fg_cuda_context_set_path(fg_cuda_context *c, uint32_t path, fg_error *err) {
    if (!c || path > FG_CUDA_PATH_RING_IF_POSSIBLE) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid streaming path");
        return FG_ERR_ARGUMENT;
    }
    c->path = path;
    return FG_OK;
}

/* Test seam (declared in fg_host_internal.h only): how the ring kernel deals out work
 * (0 as the planner likes, 1 whole rows, 2 tiles), how many polls its device-side waits
 * take before they give up (0 = default), and one tile that is never fetched so that a wait
 * does run out (armed != 0: warp 0 of CTA `cta` skips its `issue`-th request). */
fg_status fg_cuda_internal_ring_controls(fg_cuda_context *c, uint32_t deal, uint32_t wait_polls,
                                         uint32_t armed, uint32_t cta, uint32_t issue) {
    if (!c || deal > 2u) return FG_ERR_ARGUMENT;
    c->ring_deal = deal;
    c->ring_wait_polls = wait_polls;
    c->ring_withhold_armed = armed;
    c->ring_withhold_cta = cta;
    c->ring_withhold_issue = issue;
    return FG_OK;
}

fg_status fg_cuda_begin(fg_cuda_context *c, fg_error *err) {
    if (!c || c->batch_active) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid CUDA batch begin");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status == FG_OK) c->batch_active = true;
    return status;
}

fg_status fg_cuda_end(fg_cuda_context *c, fg_error *err) {
    if (!c || !c->batch_active) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid CUDA batch end");
        return FG_ERR_ARGUMENT;
    }
    c->batch_active = false;
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    const int e = fgk_stream_synchronize(c->stream);
    return e ? fg_cuda_fail(err, e, "waiting for the CUDA batch") : FG_OK;
}

bool fg_cuda_batch_active(const fg_cuda_context *c) { return c && c->batch_active; }

/* ------------------------------------------------------------------ tensors */

fg_status fg_cuda_tensor_create(fg_cuda_context *c, uint64_t bytes, fg_cuda_tensor **out,
                                fg_error *err) {
    if (!c || !bytes || !out) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid CUDA tensor arguments");
        return FG_ERR_ARGUMENT;
    }
    *out = NULL;
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    fg_cuda_tensor *t = calloc(1, sizeof(*t));
    if (!t) {
        fg_error_set(err, FG_ERR_OOM, "out of host memory");
        return FG_ERR_OOM;
    }
    /* round the allocation so 128-bit accesses near the end stay inside it */
    int e = fgk_malloc((void **)&t->base, (size_t)fg_align_up_u64(bytes, 256u));
    if (!e) e = fgk_memset_async(t->base, 0, (size_t)fg_align_up_u64(bytes, 256u), c->stream);
    if (e) {
        status = fg_cuda_fail(err, e, "allocating a CUDA tensor");
        if (t->base) fgk_free(t->base);
        free(t);
        return status;
    }
    t->context = c;
    t->bytes = bytes;
    t->owns = true;
    *out = t;
    return FG_OK;
}

fg_status fg_cuda_tensor_view(fg_cuda_tensor *base, uint64_t offset, uint64_t bytes,
                              fg_cuda_tensor **out, fg_error *err) {
    if (!base || !out || !bytes || offset > base->bytes || bytes > base->bytes - offset) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid CUDA tensor view");
        return FG_ERR_ARGUMENT;
    }
    fg_cuda_tensor *t = calloc(1, sizeof(*t));
    if (!t) {
        fg_error_set(err, FG_ERR_OOM, "out of host memory");
        return FG_ERR_OOM;
    }
    t->context = base->context;
    t->base = base->base + offset;
    t->bytes = bytes;
    t->owns = false;
    *out = t;
    return FG_OK;
}

fg_status fg_cuda_tensor_wrap(fg_cuda_context *c, void *device_pointer, uint64_t bytes,
                              fg_cuda_tensor **out, fg_error *err) {
    if (!c || !device_pointer || !bytes || !out) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid CUDA tensor wrap");
        return FG_ERR_ARGUMENT;
    }
    fg_cuda_tensor *t = calloc(1, sizeof(*t));
    if (!t) {
        fg_error_set(err, FG_ERR_OOM, "out of host memory");
        return FG_ERR_OOM;
    }
    t->context = c;
    t->base = device_pointer;
    t->bytes = bytes;
    t->owns = false;
    *out = t;
    return FG_OK;
}

void fg_cuda_tensor_destroy(fg_cuda_tensor *t) {
    if (!t) return;
    if (t->owns && t->base && fgk_set_device(t->context->device) == 0) {
        fgk_stream_synchronize(t->context->stream);
        fgk_free(t->base);
    }
    free(t);
}

uint64_t fg_cuda_tensor_bytes(const fg_cuda_tensor *t) { return t ? t->bytes : 0u; }
void *fg_cuda_tensor_device_pointer(const fg_cuda_tensor *t) { return t ? t->base : NULL; }

static bool tensor_range(const fg_cuda_tensor *t, uint64_t offset, uint64_t bytes) {
    return t && offset <= t->bytes && bytes <= t->bytes - offset;
}

fg_status fg_cuda_tensor_write(fg_cuda_tensor *t, uint64_t offset, const void *data, uint64_t bytes,
                               fg_error *err) {
    if (!tensor_range(t, offset, bytes) || (bytes && !data)) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid CUDA tensor write");
        return FG_ERR_ARGUMENT;
    }
    if (!bytes) return FG_OK;
    fg_status status = fg_cuda_enter(t->context, err);
    if (status != FG_OK) return status;
    int e = fgk_copy_to_device_async(t->base + offset, data, (size_t)bytes, t->context->stream);
    /* the caller may reuse `data` at once */
    if (!e) e = fgk_stream_synchronize(t->context->stream);
    return e ? fg_cuda_fail(err, e, "writing a CUDA tensor") : FG_OK;
}

fg_status fg_cuda_tensor_read(const fg_cuda_tensor *t, uint64_t offset, void *data, uint64_t bytes,
                              fg_error *err) {
    if (!tensor_range(t, offset, bytes) || (bytes && !data)) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid CUDA tensor read");
        return FG_ERR_ARGUMENT;
    }
    if (!bytes) return FG_OK;
    fg_status status = fg_cuda_enter(t->context, err);
    if (status != FG_OK) return status;
    int e = fgk_copy_to_host_async(data, t->base + offset, (size_t)bytes, t->context->stream);
    if (!e) e = fgk_stream_synchronize(t->context->stream);
    return e ? fg_cuda_fail(err, e, "reading a CUDA tensor") : FG_OK;
}

/* --------------------------------------------------------- device operators */

static bool on_context(const fg_cuda_context *c, const fg_cuda_tensor *t) {
    return t && t->context == c;
}

fg_status fg_cuda_apply_penalties(fg_cuda_context *c, fg_cuda_tensor *logits,
                                  const fg_cuda_tensor *counts, uint32_t values,
                                  float presence_penalty, float frequency_penalty,
                                  float repetition_penalty, fg_error *err) {
    /* src/vk.c:1812-1819 */
    if (!c || !values || !on_context(c, logits) || !on_context(c, counts) ||
        !tensor_range(logits, 0, (uint64_t)values * 4u) ||
        !tensor_range(counts, 0, (uint64_t)values * 4u) || !isfinite(presence_penalty) ||
        !isfinite(frequency_penalty) || !isfinite(repetition_penalty) ||
        repetition_penalty <= 0.0f) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid vocabulary penalty dispatch");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    const int e = fgk_launch_apply_penalties((float *)logits->base, (const uint32_t *)counts->base,
                                             values, presence_penalty, frequency_penalty,
                                             repetition_penalty, c->stream);
    c->launches++;
    return e ? fg_cuda_fail(err, e, "penalty kernel") : FG_OK;
}

fg_status fg_cuda_argmax_reduce(fg_cuda_context *c, fg_cuda_tensor *out_scores,
                                fg_cuda_tensor *out_ids, const fg_cuda_tensor *in_scores,
                                const fg_cuda_tensor *in_ids, uint32_t count,
                                uint32_t *output_count, fg_error *err) {
    const uint32_t groups = (uint32_t)(((uint64_t)count + 4095u) / 4096u);
    /* src/vk.c:2260 */
    if (!c || !count || !output_count || !tensor_range(in_scores, 0, (uint64_t)count * 4u) ||
        (in_ids && !tensor_range(in_ids, 0, (uint64_t)count * 4u)) ||
        !tensor_range(out_scores, 0, (uint64_t)groups * 4u) ||
        !tensor_range(out_ids, 0, (uint64_t)groups * 4u)) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid argmax reduction dispatch");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    const int e = fgk_launch_argmax_reduce((float *)out_scores->base, (uint32_t *)out_ids->base,
                                           (const float *)in_scores->base,
                                           in_ids ? (const uint32_t *)in_ids->base : NULL, count,
                                           c->stream);
    c->launches++;
    if (e) return fg_cuda_fail(err, e, "argmax kernel");
    *output_count = groups;
    return FG_OK;
}

fg_status fg_cuda_topk_select(fg_cuda_context *c, fg_cuda_tensor *out_scores,
                              fg_cuda_tensor *out_ids, const fg_cuda_tensor *in_scores,
                              const fg_cuda_tensor *in_ids, uint32_t count, uint32_t k,
                              uint32_t *output_count, fg_error *err) {
    const uint64_t groups = ((uint64_t)count + 1023u) / 1024u;
    const uint64_t produced = groups * k;
    /* src/vk.c:2240-2249 */
    if (!c || !count || k < 1u || k > 64u || !output_count || produced > UINT32_MAX ||
        !tensor_range(in_scores, 0, (uint64_t)count * 4u) ||
        (in_ids && !tensor_range(in_ids, 0, (uint64_t)count * 4u)) ||
        !tensor_range(out_scores, 0, produced * 4u) || !tensor_range(out_ids, 0, produced * 4u)) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid generation top-k selection dispatch");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    const int e = fgk_launch_topk_select((float *)out_scores->base, (uint32_t *)out_ids->base,
                                         (const float *)in_scores->base,
                                         in_ids ? (const uint32_t *)in_ids->base : NULL, count, k,
                                         c->stream);
    c->launches++;
    if (e) return fg_cuda_fail(err, e, "top-k kernel");
    *output_count = (uint32_t)produced;
    return FG_OK;
}

fg_status fg_cuda_topk_reduce(fg_cuda_context *c, fg_cuda_tensor *out_scores, fg_cuda_tensor *out_ids,
                              const fg_cuda_tensor *in_scores, const fg_cuda_tensor *in_ids, uint32_t count,
                              uint32_t *output_count, fg_error *err) {
    /* src/vk.c:2235 */
    const uint64_t groups = ((uint64_t)count + 4095u) / 4096u;
    uint64_t produced = groups * 512u;
    if (groups == 1u && count < 512u) produced = count;
    if (!c || !count || !output_count || !tensor_range(in_scores, 0, (uint64_t)count * 4u) ||
        (in_ids && !tensor_range(in_ids, 0, (uint64_t)count * 4u)) ||
        !tensor_range(out_scores, 0, produced * 4u) || !tensor_range(out_ids, 0, produced * 4u)) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid top-k reduction dispatch");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    const int e = fgk_launch_topk_reduce((float *)out_scores->base, (uint32_t *)out_ids->base,
                                         (const float *)in_scores->base,
                                         in_ids ? (const uint32_t *)in_ids->base : NULL, count,
                                         (uint32_t)produced, c->stream);
    c->launches++;
    if (e) return fg_cuda_fail(err, e, "top-k reduction kernel");
    *output_count = (uint32_t)produced;
    return FG_OK;
}

fg_status fg_cuda_router_topk(fg_cuda_context *c, fg_cuda_tensor *selected, fg_cuda_tensor *gates,
                              const fg_cuda_tensor *logits, uint32_t experts, uint32_t tokens, uint32_t k,
                              fg_error *err) {
    /* src/vk.c:2257 (fixed at 512 experts and k = 10 there); src/q38_math.c:49 */
    const uint64_t pairs = (uint64_t)tokens * k;
    if (!c || !experts || !tokens || !k || k > experts || k > 32u ||
        !tensor_range(logits, 0, (uint64_t)tokens * experts * 4u) || !tensor_range(selected, 0, pairs * 4u) ||
        !tensor_range(gates, 0, pairs * 4u)) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid GPU router top-k dispatch");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    uint32_t *bad = (uint32_t *)c->first_error + 8; /* a word of the context's 256-byte block */
    int e = fgk_memset_async(bad, 0xff, 4u, c->stream);
    if (!e) e = fgk_launch_router_topk((uint32_t *)selected->base, (float *)gates->base,
                                       (const float *)logits->base, tokens, experts, k, bad, c->stream);
    c->launches++;
    uint32_t first_bad = UINT32_MAX;
    if (!e) e = fgk_copy_to_host_async(&first_bad, bad, 4u, c->stream);
    if (!e) e = fgk_stream_synchronize(c->stream);
    if (e) return fg_cuda_fail(err, e, "router kernel");
    if (first_bad != UINT32_MAX) {  /* src/q38_math.c:61 */
        fg_error_set(err, FG_ERR_FORMAT, "router probabilities are not finite (token %u)", first_bad);
        return FG_ERR_FORMAT;
    }
    return FG_OK;
}

fg_status fg_cuda_history_reset(fg_cuda_context *c, fg_cuda_tensor *counts, uint32_t vocab,
                                const uint32_t *history, uint32_t count, fg_error *err) {
    /* src/output.c:604-606 */
    if (!c || !vocab || !on_context(c, counts) || !tensor_range(counts, 0, (uint64_t)vocab * 4u) ||
        count > FG_NATIVE_CONTEXT || (count && !history)) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid output history");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    const size_t bytes = (size_t)count * 4u;
    status = fg_cuda_reserve(&c->staging, &c->staging_bytes, bytes + 64u, false, c, err);
    if (status != FG_OK) return status;
    uint32_t *bad = (uint32_t *)c->staging;
    uint32_t *tokens = (uint32_t *)((unsigned char *)c->staging + 64u);
    const uint32_t none = UINT32_MAX;
    int e = fgk_memset_async(counts->base, 0, (size_t)vocab * 4u, c->stream);
    if (!e) e = fgk_copy_to_device_async(bad, &none, 4u, c->stream);
    if (!e && count) e = fgk_copy_to_device_async(tokens, history, bytes, c->stream);
    if (!e && count) {
        e = fgk_launch_history_add((uint32_t *)counts->base, vocab, tokens, count, bad, c->stream);
        c->launches++;
    }
    uint32_t first_bad = UINT32_MAX;
    if (!e) e = fgk_copy_to_host_async(&first_bad, bad, 4u, c->stream);
    if (!e) e = fgk_stream_synchronize(c->stream);
    if (e) return fg_cuda_fail(err, e, "history kernel");
    if (first_bad != UINT32_MAX) {
        fg_error_set(err, FG_ERR_FORMAT, "history token %u is outside vocabulary", first_bad);
        return FG_ERR_FORMAT;
    }
    return FG_OK;
}

fg_status fg_cuda_history_increment(fg_cuda_context *c, fg_cuda_tensor *counts, uint32_t vocab,
                                    uint32_t token, fg_error *err) {
    /* src/output.c:621-622 */
    if (!c || !on_context(c, counts) || !tensor_range(counts, 0, (uint64_t)vocab * 4u) ||
        token >= vocab) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid output history token");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    status = fg_cuda_reserve(&c->staging, &c->staging_bytes, 128u, false, c, err);
    if (status != FG_OK) return status;
    uint32_t *bad = (uint32_t *)c->staging;
    uint32_t *slot = (uint32_t *)((unsigned char *)c->staging + 64u);
    int e = fgk_copy_to_device_async(slot, &token, 4u, c->stream);
    if (!e) {
        e = fgk_launch_history_add((uint32_t *)counts->base, vocab, slot, 1u, bad, c->stream);
        c->launches++;
    }
    return e ? fg_cuda_fail(err, e, "history kernel") : FG_OK;
}

/* ------------------------------------------------------------ fused batched */

typedef struct stream_plan {
    uint32_t splits, split_len, bitmap_words, count_capacity, dense_wide;
    size_t dynamic_smem;
} stream_plan;

/* Picks how many CTAs share a row.  Every CTA of a row rebuilds the row's history
 * structure and pays the fixed cost of a split, so one CTA per row is best as
 * soon as there are enough rows to occupy every CTA slot of the GPU; with fewer
 * rows a row is cut into as many column ranges as it takes to fill the slots.
 * Results do not depend on the choice. */
static bool plan_stream(const fg_cuda_context *c, uint32_t rows, uint32_t vocab,
                        uint32_t history_max, bool penalties, bool counts, stream_plan *plan) {
    const uint32_t max_splits = fgk_stream_max_splits();
    const uint32_t tile = fgk_stream_tile();
    const uint32_t slots = c->sm_count * 4u;
    uint32_t want = c->forced_splits;
    if (!want) {
        want = rows >= slots ? 1u : (slots + rows - 1u) / rows;
        /* a split shorter than two tiles is all fixed cost */
        const uint32_t most = vocab / (2u * tile) ? vocab / (2u * tile) : 1u;
        if (want > most) want = most;
        if (want > max_splits) want = max_splits;
    }
    for (; want <= max_splits; want++) {
        uint32_t len = (vocab + want - 1u) / want;
        len = (len + 127u) & ~127u;
        stream_plan p;
        p.splits = (vocab + len - 1u) / len;
        p.split_len = len;
        p.bitmap_words = penalties ? (len + 31u) / 32u : 0u;
        p.count_capacity = (penalties && counts) ? (history_max < len ? history_max : len) : 0u;
        if (p.count_capacity == 0u && penalties && counts) p.count_capacity = 1u;
        p.dense_wide = history_max > 65535u ? 1u : 0u;
        p.dynamic_smem = (size_t)fgk_stream_dynamic_smem(p.bitmap_words, p.count_capacity, p.dense_wide);
        /* running popcounts are 16 bits wide; more splits shrink both limits */
        if (p.count_capacity > 65535u || p.dynamic_smem > FGK_STREAM_MAX_DYNAMIC_SMEM) continue;
        *plan = p;
        return true;
    }
    return false;
}

typedef struct batch_traits {
    bool penalties, counts, sampled, nucleus, topk_rows;
    bool raising; /* some row's penalties can raise a logit (or its repetition factor is extreme) */
} batch_traits;

static fg_status check_batch(const fg_cuda_context *c, const fg_cuda_sample_args *a, bool shard,
                             batch_traits *traits, fg_error *err) {
    if (!c || !a || !a->logits || !a->rows || !a->vocab || a->row_stride < a->vocab ||
        (a->dtype != FG_CUDA_F32 && a->dtype != FG_CUDA_BF16) || !a->configs ||
        (a->config_count != 1u && a->config_count != a->rows) || !a->row_status ||
        (!shard && (!a->tokens || !a->token_logits)) ||
        ((a->history_tokens == NULL) != (a->history_offsets == NULL)) ||
        a->history_max > FG_NATIVE_CONTEXT) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid batched sampling arguments");
        return FG_ERR_ARGUMENT;
    }
    memset(traits, 0, sizeof(*traits));
    const bool allow = (a->flags & FG_CUDA_SAMPLE_ALLOW_NO_TOPK) != 0u && !shard;
    for (uint32_t i = 0; i < a->config_count; i++) {
        const fg_sampler_config *cfg = &a->configs[i];
        if (!fg_cuda_config_ok(cfg, allow)) {
            fg_error_set(err, FG_ERR_ARGUMENT, "invalid sampler controls");
            return FG_ERR_ARGUMENT;
        }
        if (fg_sampler_penalties_active(cfg)) {
            traits->penalties = true;
            if (!(cfg->presence_penalty >= 0.0f && cfg->frequency_penalty >= 0.0f &&
                  cfg->repetition_penalty >= 1.0f && cfg->repetition_penalty <= 0x1p40f))
                traits->raising = true;
        }
        if (cfg->frequency_penalty != 0.0f) traits->counts = true;
        if (cfg->temperature != 0.0f) {
            traits->sampled = true;
            if (cfg->top_k == 0u) traits->nucleus = true;
            else traits->topk_rows = true;
        } else {
            traits->topk_rows = true;
        }
    }
    if (shard) traits->topk_rows = true;
    if (traits->sampled && !shard && !a->uniforms) {
        fg_error_set(err, FG_ERR_ARGUMENT, "sampled rows need one uniform draw each");
        return FG_ERR_ARGUMENT;
    }
    if ((!a->history_tokens || a->history_max == 0u) && !c->session_counts)
        traits->penalties = traits->counts = false;
    return FG_OK;
}

static void fill_output(fgk_select_output *out, const fg_cuda_context *c,
                        const fg_cuda_sample_args *a) {
    memset(out, 0, sizeof(*out));
    out->tokens = a->tokens;
    out->token_logits = a->token_logits;
    out->row_status = a->row_status;
    out->first_error = c->first_error;
    if (a->debug) {
        out->dbg_count = a->debug->candidate_count;
        out->dbg_ids = a->debug->candidate_ids;
        out->dbg_scores = a->debug->candidate_scores;
        out->dbg_raw = a->debug->raw_probability;
        out->dbg_tempered = a->debug->tempered_probability;
    }
}

/* Uploads per-row configs when they differ; *device is NULL for a shared config. */
static fg_status upload_configs(fg_cuda_context *c, const fg_cuda_sample_args *a,
                                const void **device, fg_error *err) {
    *device = NULL;
    if (a->config_count == 1u) return FG_OK;
    const size_t bytes = (size_t)a->config_count * sizeof(fg_sampler_config);
    fg_status status = fg_cuda_reserve(&c->configs, &c->configs_bytes, bytes, false, c, err);
    if (status != FG_OK) return status;
    const int e = fgk_copy_to_device_async(c->configs, a->configs, bytes, c->stream);
    if (e) return fg_cuda_fail(err, e, "uploading sampler configs");
    *device = c->configs;
    return FG_OK;
}

/* Waits for the stream and turns the device's first-error word into a status.  The word
 * after it says why a row ended with FG_ERR_LIMIT when it was not the history's length. */
static fg_status collect_status(fg_cuda_context *c, fg_error *err) {
    uint64_t words[2] = {UINT64_MAX, UINT64_MAX};
    int e = fgk_copy_to_host_async(words, c->first_error, 16u, c->stream);
    if (!e) e = fgk_stream_synchronize(c->stream);
    if (e) return fg_cuda_fail(err, e, "sampling kernels");
    if (words[0] == UINT64_MAX) return FG_OK;
    const fg_status status = (fg_status)(words[0] & 0xffu);
    const uint64_t row = words[0] >> 8;
    const char *why = "row failed";
    if (status == FG_ERR_FORMAT) why = "no finite candidate, invalid penalized finalist, softmax failure or history token outside vocabulary";
    else if (status == FG_ERR_MISMATCH) why = "invalid output finalist";
    else if (status == FG_ERR_LIMIT && words[1] == 1u) why = "a device-side wait ran out (a tile never landed or a warp never came)";
    else if (status == FG_ERR_LIMIT) why = "history longer than history_max";
    else if (status == FG_ERR_ARGUMENT) why = "a penalty that can raise a logit reached the kernel for lowering penalties";
    fg_error_set(err, status, "row %llu: %s", (unsigned long long)row, why);
    return status;
}

static fg_status run_stream(fg_cuda_context *c, const fg_cuda_sample_args *a,
                            const batch_traits *traits, uint32_t vocab_offset,
                            uint32_t vocab_total, uint32_t shard_k, float *shard_scores,
                            uint32_t *shard_ids, uint32_t shard_stride, fg_error *err) {
    stream_plan plan;
    if (!plan_stream(c, a->rows, a->vocab, a->history_max, traits->penalties, traits->counts, &plan)) {
        fg_error_set(err, FG_ERR_LIMIT, "history structure does not fit shared memory");
        return FG_ERR_LIMIT;
    }
    fg_status status = FG_OK;
    const size_t slots = (size_t)a->rows * plan.splits;
    const size_t meta_bytes = (size_t)fgk_stream_part_meta_bytes();
    const size_t part_bytes = plan.splits > 1u ? slots * (64u * 8u + meta_bytes) : 0u;
    status = fg_cuda_reserve((void **)&c->tickets, &c->tickets_bytes, (size_t)a->rows * 4u, true, c, err);
    const void *configs_device = NULL;
    if (status == FG_OK) status = upload_configs(c, a, &configs_device, err);
    if (status != FG_OK) return status;
    c->last_scratch_bytes = part_bytes + (size_t)a->rows * 4u +
                            (a->config_count > 1u ? (size_t)a->rows * sizeof(fg_sampler_config) : 0u);

    fgk_stream_launch l;
    memset(&l, 0, sizeof(l));
    l.logits = a->logits;
    l.dtype = a->dtype;
    l.rows = a->rows;
    l.vocab = a->vocab;
    l.row_stride = a->row_stride;
    l.vocab_offset = vocab_offset;
    l.vocab_total = vocab_total;
    l.splits = plan.splits;
    l.split_len = plan.split_len;
    l.history_tokens = traits->penalties ? a->history_tokens : NULL;
    l.history_offsets = traits->penalties ? a->history_offsets : NULL;
    l.history_max = a->history_max;
    l.configs_device = configs_device;
    l.config0 = a->configs[0];
    l.config_count = a->config_count;
    l.shard_k = shard_k;
    l.uniforms = a->uniforms;
    l.shard_scores = shard_scores;
    l.shard_ids = shard_ids;
    l.shard_stride = shard_stride;
    if (c->push) l.push = *c->push;
    l.tickets = c->tickets;
    l.bitmap_words = plan.bitmap_words;
    l.count_capacity = plan.count_capacity;
    l.dense_wide = plan.dense_wide;
    fill_output(&l.out, c, a);
    /* Whole rows the copy engine can fetch (16-byte aligned starts and lengths) whose
     * penalties cannot raise a logit may go through the persistent ring kernel; the
     * rest, and anything the caller pinned to it, through the register-prefetch kernel. */
    const size_t element = a->dtype == FG_CUDA_BF16 ? 2u : 4u;
    const uint32_t whole_bitmap = traits->penalties ? (a->vocab + 31u) / 32u : 0u;
    const bool ring_ok = ((uintptr_t)a->logits % 16u) == 0u && (a->row_stride * element) % 16u == 0u &&
                         ((size_t)a->vocab * element) % 16u == 0u && c->forced_splits <= 1u &&
                         !(traits->penalties && traits->raising) &&
                         fgk_persistent_dynamic_smem(whole_bitmap, NULL) != 0u;
    if (c->session_counts && !(ring_ok && c->path != FG_CUDA_PATH_REGISTERS && vocab_offset == 0u)) {
        /* (the executor then falls back to token lists) */
        fg_error_set(err, FG_ERR_UNAVAILABLE, "session tables are read by the ring kernel only");
        return FG_ERR_UNAVAILABLE;
    }
    if (c->path == FG_CUDA_PATH_RING && !ring_ok) {
        fg_error_set(err, FG_ERR_ARGUMENT,
                     "the ring path needs whole 16-byte aligned rows and penalties that only lower logits");
        return FG_ERR_ARGUMENT;
    }
    /* AUTO: the persistent kernel whenever it can take the batch. */
    const uint32_t most = c->sm_count; /* one CTA per SM */
    const bool take_ring = c->path != FG_CUDA_PATH_REGISTERS;
    if (ring_ok && take_ring) {
        /* When work goes out in tiles, every CTA gets the same number, so a row may be shared
         * by several CTAs.  A share is at least as long as the CTA's warps look at side by
         * side, and so long that no row has more parts than the merge takes. */
        uint32_t k_most = shard_k;
        for (uint32_t i = 0; !shard_k && i < a->config_count; i++) {
            const uint32_t k = a->configs[i].temperature == 0.0f ? 1u : a->configs[i].top_k;
            if (k > k_most) k_most = k;
        }
        const uint32_t row_tiles = fgk_persistent_row_tiles(a->dtype, a->vocab);
        const uint64_t all_tiles = (uint64_t)a->rows * row_tiles;
        const uint32_t parts_limit = fgk_persistent_max_parts(k_most);
        uint64_t per_cta = (all_tiles + most - 1u) / most;
        const uint64_t shortest = (row_tiles + parts_limit - 2u) / (parts_limit - 1u);
        if (per_cta < shortest) per_cta = shortest;
        if (per_cta < fgk_persistent_tiles_abreast()) per_cta = fgk_persistent_tiles_abreast();
        uint32_t ctas = (uint32_t)((all_tiles + per_cta - 1u) / per_cta);
        uint32_t max_parts = (uint32_t)((row_tiles + per_cta - 1u) / per_cta) + 1u;
        if (max_parts > parts_limit) max_parts = parts_limit;
        /* Whole rows are dealt out unless there are very few, very long rows: a shared row costs
         * its fixed work once per part and a merge through global memory, which only pays when a
         * single CTA would be alone with a row of a million logits.  (Measured on B200, vocabulary
         * 151,936: one row 39 against 69 us, 128 rows 51 against 67 us, 256 rows 47 against 63 us.) */
        const bool few_long_rows = a->rows * 4u < most && row_tiles > 512u;
        const bool whole_rows = c->ring_deal == 1u || (c->ring_deal == 0u && !few_long_rows);
        if (whole_rows) {
            per_cta = 0u;
            ctas = a->rows < most ? a->rows : most;
            max_parts = 1u;
        }
        const size_t part_slots = max_parts > 1u ? (size_t)a->rows * max_parts : 0u; /* whole rows leave no parts */
        l.part_scores = NULL;
        l.part_ids = NULL;
        l.part_meta = NULL;
        if (part_slots != 0u) {
            status = fg_cuda_reserve(&c->parts, &c->parts_bytes, part_slots * (64u * 8u + 16u), false, c, err);
            if (status != FG_OK) return status;
            unsigned char *base = c->parts;
            l.part_scores = (float *)base;
            l.part_ids = (uint32_t *)(base + part_slots * 64u * 4u);
            l.part_meta = base + part_slots * 64u * 8u;
        }
        l.splits = max_parts;
        l.split_len = (uint32_t)per_cta;
        l.bitmap_words = whole_bitmap;
        l.slot_counts = c->session_counts;
        l.slot_bitmaps = c->session_bitmaps;
        l.row_slots = c->session_rows;
        l.slot_bitmap_words = c->session_bitmap_words;
        l.wait_polls = c->ring_wait_polls;
        l.withhold_armed = c->ring_withhold_armed;
        l.withhold_cta = c->ring_withhold_cta;
        l.withhold_issue = c->ring_withhold_issue;
        c->last_scratch_bytes = part_slots * (64u * 8u + 16u) + (size_t)a->rows * 4u +
                                (a->config_count > 1u ? (size_t)a->rows * sizeof(fg_sampler_config) : 0u);
        const int e = fgk_launch_persistent_select(&l, ctas, c->stream);
        c->launches++;
        return e ? fg_cuda_fail(err, e, "persistent ring kernel") : FG_OK;
    }
    /* the streaming kernel's hand-off between the splits of a row, reserved only when it runs */
    if (part_bytes) {
        status = fg_cuda_reserve(&c->parts, &c->parts_bytes, part_bytes, false, c, err);
        if (status != FG_OK) return status;
        unsigned char *base = c->parts;
        l.part_scores = (float *)base;
        l.part_ids = (uint32_t *)(base + slots * 64u * 4u);
        l.part_meta = base + slots * 64u * 8u;
    }
    const int e = fgk_launch_stream_select(&l, c->stream);
    c->launches++;
    return e ? fg_cuda_fail(err, e, "streaming select kernel") : FG_OK;
}

/* Rows without a top-k cut: history pass (when there are penalties), then the
 * persistent nucleus kernel, one scratch row per CTA. */
static fg_status run_nucleus(fg_cuda_context *c, const fg_cuda_sample_args *a,
                             const batch_traits *traits, fg_error *err) {
    fg_cuda_context planner = *c;
    planner.forced_splits = 1u; /* as few column ranges as the history structure's limits allow */
    stream_plan plan;
    if (!plan_stream(&planner, a->rows, a->vocab, a->history_max, traits->penalties, traits->counts, &plan)) {
        fg_error_set(err, FG_ERR_LIMIT, "history structure does not fit shared memory");
        return FG_ERR_LIMIT;
    }
    const uint32_t ctas = a->rows < c->sm_count ? a->rows : c->sm_count;
    const size_t stride = (size_t)fg_align_up_u64(a->vocab, 64u);
    fg_status status = fg_cuda_reserve(&c->nucleus, &c->nucleus_bytes, (size_t)ctas * stride * 4u, false, c, err);
    const void *configs_device = NULL;
    if (status == FG_OK) status = upload_configs(c, a, &configs_device, err);
    if (status != FG_OK) return status;
    const size_t slots = (size_t)a->rows * plan.splits;

    fgk_nucleus_launch n;
    memset(&n, 0, sizeof(n));
    n.logits = a->logits;
    n.dtype = a->dtype;
    n.rows = a->rows;
    n.vocab = a->vocab;
    n.row_stride = a->row_stride;
    n.configs_device = configs_device;
    n.config0 = a->configs[0];
    n.config_count = a->config_count;
    n.uniforms = a->uniforms;
    n.scratch = c->nucleus;
    n.scratch_stride = stride;
    n.ctas = ctas;
    n.splits = plan.splits;
    n.split_len = plan.split_len;
    n.bitmap_words = plan.bitmap_words;
    n.count_capacity = plan.count_capacity;
    n.dense_wide = plan.dense_wide;
    fill_output(&n.out, c, a);
    c->last_scratch_bytes = (size_t)ctas * stride * 4u;
    if (traits->penalties) {
        const size_t stride_words = plan.dynamic_smem / 4u;
        const size_t meta_at = (size_t)fg_align_up_u64(slots * stride_words * 4u, 256u);
        status = fg_cuda_reserve(&c->history, &c->history_bytes, meta_at + slots * 8u, false, c, err);
        if (status != FG_OK) return status;
        fgk_stream_launch h;
        memset(&h, 0, sizeof(h));
        h.rows = a->rows;
        h.vocab = a->vocab;
        h.vocab_total = a->vocab;
        h.splits = plan.splits;
        h.split_len = plan.split_len;
        h.history_tokens = a->history_tokens;
        h.history_offsets = a->history_offsets;
        h.history_max = a->history_max;
        h.configs_device = configs_device;
        h.config0 = a->configs[0];
        h.config_count = a->config_count;
        h.bitmap_words = plan.bitmap_words;
        h.count_capacity = plan.count_capacity;
        h.dense_wide = plan.dense_wide;
        h.history_global = c->history;
        h.history_stride_words = stride_words;
        h.history_meta = (unsigned char *)c->history + meta_at;
        const int e = fgk_launch_history_build(&h, c->stream);
        c->launches++;
        if (e) return fg_cuda_fail(err, e, "history kernel");
        n.history_global = c->history;
        n.history_stride_words = stride_words;
        n.history_meta = h.history_meta;
        c->last_scratch_bytes += meta_at + slots * 8u;
    }
    const int e = fgk_launch_nucleus_select(&n, c->stream);
    c->launches++;
    return e ? fg_cuda_fail(err, e, "nucleus kernel") : FG_OK;
}

static fg_status arm_first_error(fg_cuda_context *c, fg_error *err) {
    const int e = fgk_memset_async(c->first_error, 0xff, 16u, c->stream); /* the error word and its cause */
    return e ? fg_cuda_fail(err, e, "arming the error word") : FG_OK;
}

fg_status fg_cuda_sample_batch(fg_cuda_context *c, const fg_cuda_sample_args *a, fg_error *err) {
    batch_traits traits;
    fg_status status = check_batch(c, a, false, &traits, err);
    if (status != FG_OK) return status;
    status = fg_cuda_enter(c, err);
    if (status == FG_OK) status = arm_first_error(c, err);
    if (status == FG_OK && traits.topk_rows)
        status = run_stream(c, a, &traits, 0u, a->vocab, 0u, NULL, NULL, 1u, err);
    if (status == FG_OK && traits.nucleus) status = run_nucleus(c, a, &traits, err);
    if (status != FG_OK || (a->flags & FG_CUDA_SAMPLE_ASYNC)) return status;
    return collect_status(c, err);
}

/* The shard step with an explicit candidate layout (stride 1: two arrays, 2: interleaved
 * (value, id) pairs).  Enqueues only. */
fg_status fg_cuda_shard_topk_layout(fg_cuda_context *c, const fg_cuda_sample_args *a, uint32_t vocab_offset,
                                    uint32_t vocab_total, uint32_t k_shard, float *candidate_scores,
                                    uint32_t *candidate_ids, uint32_t stride, fg_error *err) {
    batch_traits traits;
    fg_status status = check_batch(c, a, true, &traits, err);
    if (status != FG_OK) return status;
    if (k_shard < 1u || k_shard > 64u || ((!candidate_scores || !candidate_ids) && !c->push) ||
        (uint64_t)vocab_offset + a->vocab > vocab_total) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid vocabulary shard arguments");
        return FG_ERR_ARGUMENT;
    }
    status = fg_cuda_enter(c, err);
    if (status == FG_OK) status = arm_first_error(c, err);
    if (status == FG_OK)
        status = run_stream(c, a, &traits, vocab_offset, vocab_total, k_shard, candidate_scores,
                            candidate_ids, stride, err);
    return status;
}

fg_status fg_cuda_shard_topk(fg_cuda_context *c, const fg_cuda_sample_args *a, uint32_t vocab_offset,
                             uint32_t vocab_total, uint32_t k_shard, float *candidate_scores,
                             uint32_t *candidate_ids, fg_error *err) {
    const fg_status status = fg_cuda_shard_topk_layout(c, a, vocab_offset, vocab_total, k_shard,
                                                       candidate_scores, candidate_ids, 1u, err);
    if (status != FG_OK || (a->flags & FG_CUDA_SAMPLE_ASYNC)) return status;
    return collect_status(c, err);
}

/* The merge step over [shard][row][k_shard] candidates with an explicit layout.  Enqueues
 * only; does not re-arm the error word when `keep_errors` (the shard step of the same call
 * may already have noted a row). */
fg_status fg_cuda_merge_select_layout(fg_cuda_context *c, const fg_cuda_sample_args *a,
                                      const float *candidate_scores, const uint32_t *candidate_ids,
                                      uint32_t stride, uint32_t shards, uint32_t k_shard,
                                      const uint32_t *shard_first, const uint32_t *shard_width,
                                      bool keep_errors, const fg_cuda_arrivals *arrivals, fg_error *err) {
    if (!c || !a || !a->rows || !a->configs || (a->config_count != 1u && a->config_count != a->rows) ||
        !a->tokens || !a->token_logits || !a->row_status || !candidate_scores || !candidate_ids ||
        !shards || shards > 16u || k_shard < 1u || k_shard > 64u || !shard_first || !shard_width) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid shard merge arguments");
        return FG_ERR_ARGUMENT;
    }
    bool sampled = false;
    for (uint32_t i = 0; i < a->config_count; i++) {
        if (!fg_cuda_config_ok(&a->configs[i], false)) {
            fg_error_set(err, FG_ERR_ARGUMENT, "invalid sampler controls");
            return FG_ERR_ARGUMENT;
        }
        if (a->configs[i].temperature != 0.0f) {
            sampled = true;
            /* the union of shard top-k lists holds the global top-k only up to k_shard */
            if (a->configs[i].top_k > k_shard) {
                fg_error_set(err, FG_ERR_ARGUMENT, "top_k %u exceeds the %u candidates each shard sent",
                             a->configs[i].top_k, k_shard);
                return FG_ERR_ARGUMENT;
            }
        }
    }
    if (sampled && !a->uniforms) {
        fg_error_set(err, FG_ERR_ARGUMENT, "sampled rows need one uniform draw each");
        return FG_ERR_ARGUMENT;
    }
    fg_status status = fg_cuda_enter(c, err);
    if (status == FG_OK && !keep_errors) status = arm_first_error(c, err);
    const void *configs_device = NULL;
    if (status == FG_OK) status = upload_configs(c, a, &configs_device, err);
    if (status != FG_OK) return status;
    fgk_merge_launch l;
    memset(&l, 0, sizeof(l));
    l.scores = candidate_scores;
    l.ids = candidate_ids;
    l.rows = a->rows;
    l.shards = shards;
    l.k_shard = k_shard;
    l.stride = stride;
    if (arrivals) {
        l.shard_pitch = arrivals->shard_pitch;
        l.arrived = arrivals->arrived;
        l.arrival_target = arrivals->target;
        l.wait_polls = arrivals->wait_polls;
    }
    l.check_spans = 1u;
    for (uint32_t s = 0; s < shards; s++) {
        l.span_first[s] = shard_first[s];
        l.span_width[s] = shard_width[s];
    }
    l.configs_device = configs_device;
    l.config0 = a->configs[0];
    l.config_count = a->config_count;
    l.uniforms = a->uniforms;
    fill_output(&l.out, c, a);
    const int e = fgk_launch_merge_select(&l, c->stream);
    c->launches++;
    return e ? fg_cuda_fail(err, e, "merge kernel") : FG_OK;
}

fg_status fg_cuda_merge_select(fg_cuda_context *c, const fg_cuda_sample_args *a,
                               const float *candidate_scores, const uint32_t *candidate_ids,
                               uint32_t shards, uint32_t k_shard, const uint32_t *shard_first,
                               const uint32_t *shard_width, fg_error *err) {
    const fg_status status = fg_cuda_merge_select_layout(c, a, candidate_scores, candidate_ids, 1u, shards,
                                                         k_shard, shard_first, shard_width, false, NULL, err);
    if (status != FG_OK || (a->flags & FG_CUDA_SAMPLE_ASYNC)) return status;
    return collect_status(c, err);
}

fg_status fg_cuda_collect(fg_cuda_context *c, fg_error *err) { return collect_status(c, err); }

/* Host-buffer form: stage in, sample, stage out. */
fg_status fg_cuda_sample_batch_host(fg_cuda_context *c, const fg_cuda_sample_args *h, fg_error *err) {
    batch_traits traits;
    fg_status status = check_batch(c, h, false, &traits, err);
    if (status != FG_OK) return status;
    if (h->debug) {
        fg_error_set(err, FG_ERR_ARGUMENT, "the host entry point takes no debug dump");
        return FG_ERR_ARGUMENT;
    }
    status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    const size_t element = h->dtype == FG_CUDA_BF16 ? 2u : 4u;
    const size_t logits_bytes = ((size_t)(h->rows - 1u) * h->row_stride + h->vocab) * element;
    uint64_t history_total = 0;
    if (h->history_offsets) history_total = h->history_offsets[h->rows];
    const size_t offsets_bytes = h->history_offsets ? ((size_t)h->rows + 1u) * 8u : 0u;
    const size_t tokens_bytes = (size_t)history_total * 4u;
    const size_t rows4 = (size_t)h->rows * 4u;
    size_t at = 0;
#define CARVE(name, bytes) const size_t name = at; at = (size_t)fg_align_up_u64(at + (bytes), 256u)
    CARVE(at_logits, logits_bytes);
    CARVE(at_offsets, offsets_bytes);
    CARVE(at_history, tokens_bytes);
    CARVE(at_uniforms, rows4);
    CARVE(at_tokens, rows4);
    CARVE(at_token_logits, rows4);
    CARVE(at_status, rows4);
#undef CARVE
    status = fg_cuda_reserve(&c->staging, &c->staging_bytes, at, false, c, err);
    if (status != FG_OK) return status;
    unsigned char *d = c->staging;
    int e = fgk_copy_to_device_async(d + at_logits, h->logits, logits_bytes, c->stream);
    if (!e && offsets_bytes) e = fgk_copy_to_device_async(d + at_offsets, h->history_offsets, offsets_bytes, c->stream);
    if (!e && tokens_bytes) e = fgk_copy_to_device_async(d + at_history, h->history_tokens, tokens_bytes, c->stream);
    if (!e && h->uniforms) e = fgk_copy_to_device_async(d + at_uniforms, h->uniforms, rows4, c->stream);
    if (e) return fg_cuda_fail(err, e, "copying sampling inputs to the device");
    fg_cuda_sample_args a = *h;
    a.logits = d + at_logits;
    a.history_offsets = offsets_bytes ? (const uint64_t *)(d + at_offsets) : NULL;
    a.history_tokens = offsets_bytes ? (const uint32_t *)(d + at_history) : NULL;
    a.uniforms = h->uniforms ? (const float *)(d + at_uniforms) : NULL;
    a.tokens = (uint32_t *)(d + at_tokens);
    a.token_logits = (float *)(d + at_token_logits);
    a.row_status = (uint32_t *)(d + at_status);
    a.flags = h->flags | FG_CUDA_SAMPLE_ASYNC;
    status = fg_cuda_sample_batch(c, &a, err);
    if (status != FG_OK) return status;
    e = fgk_copy_to_host_async(h->tokens, a.tokens, rows4, c->stream);
    if (!e) e = fgk_copy_to_host_async(h->token_logits, a.token_logits, rows4, c->stream);
    if (!e) e = fgk_copy_to_host_async(h->row_status, a.row_status, rows4, c->stream);
    if (e) return fg_cuda_fail(err, e, "copying sampling results to the host");
    return collect_status(c, err);
}

/* ------------------------------------------------- the entry that allocates nothing */

fg_status fg_cuda_sample_batch_static(int device, void *cuda_stream, const fg_cuda_sample_args *a,
                                      fg_error *err) {
    int sms = 0;
    int e = device < 0 ? 101 : fgk_set_device(device);
    if (!e) e = fgk_device_sm_count(device, &sms);
    if (e) return fg_cuda_fail(err, e, "selecting the CUDA device");
    /* a context on the stack: only its SM count is read by the checks and the planner */
    fg_cuda_context view;
    memset(&view, 0, sizeof(view));
    view.device = device;
    view.stream = cuda_stream;
    view.sm_count = (uint32_t)sms;
    batch_traits traits;
    fg_status status = check_batch(&view, a, false, &traits, err);
    if (status != FG_OK) return status;
    if (traits.nucleus) {
        fg_error_set(err, FG_ERR_UNAVAILABLE,
                     "sampling without a top-k cut needs a scratch row per SM; it is offered by fg_cuda_sample_batch only");
        return FG_ERR_UNAVAILABLE;
    }
    void *scratch = NULL;
    /* first call per device: cudaGetSymbolAddress and the kernel's shared-memory opt-in */
    e = fgk_static_scratch_address(device, &scratch);
    if (e) return fg_cuda_fail(err, e, "preparing the built-in scratch");

    stream_plan plan;
    if (!plan_stream(&view, a->rows, a->vocab, a->history_max, traits.penalties, traits.counts, &plan)) {
        fg_error_set(err, FG_ERR_LIMIT, "history structure does not fit shared memory");
        return FG_ERR_LIMIT;
    }
    /* layout: error word | tickets | per-row configs | split hand-off; fewer splits if it does not fit */
    const size_t meta_bytes = (size_t)fgk_stream_part_meta_bytes();
    const size_t at_tickets = 256u;
    const size_t at_configs = at_tickets + (size_t)fg_align_up_u64((uint64_t)a->rows * 4u, 256u);
    const size_t at_parts = at_configs + (a->config_count > 1u
        ? (size_t)fg_align_up_u64((uint64_t)a->rows * sizeof(fg_sampler_config), 256u) : 0u);
    size_t part_bytes = 0;
    for (;;) {
        const size_t slots = (size_t)a->rows * plan.splits;
        part_bytes = plan.splits > 1u ? slots * (64u * 8u + meta_bytes) : 0u;
        if (at_parts + part_bytes <= FGK_STATIC_SCRATCH_BYTES) break;
        if (plan.splits == 1u) {
            fg_error_set(err, FG_ERR_LIMIT,
                         "%u rows need %zu bytes of scratch; the built-in scratch holds %u",
                         a->rows, at_parts + part_bytes, (unsigned)FGK_STATIC_SCRATCH_BYTES);
            return FG_ERR_LIMIT;
        }
        /* the planner treats a forced count as a starting point and may hand back a larger
         * one (shared memory, 16-bit counts): only a strictly smaller plan is progress */
        const uint32_t before = plan.splits;
        view.forced_splits = plan.splits - 1u;
        if (!plan_stream(&view, a->rows, a->vocab, a->history_max, traits.penalties, traits.counts, &plan) ||
            plan.splits >= before) {
            fg_error_set(err, FG_ERR_LIMIT, "no split count fits both shared memory and the built-in scratch");
            return FG_ERR_LIMIT;
        }
    }
    unsigned char *base = scratch;
    /* the array keeps whatever the previous call left: the error word and the arrival
     * counters must start clean */
    e = fgk_memset_async(base, 0xff, 8u, cuda_stream);
    if (!e) e = fgk_memset_async(base + at_tickets, 0, (size_t)a->rows * 4u, cuda_stream);
    if (!e && a->config_count > 1u)
        e = fgk_copy_to_device_async(base + at_configs, a->configs,
                                     (size_t)a->rows * sizeof(fg_sampler_config), cuda_stream);
    if (e) return fg_cuda_fail(err, e, "clearing the built-in scratch");

    fgk_stream_launch l;
    memset(&l, 0, sizeof(l));
    l.logits = a->logits;
    l.dtype = a->dtype;
    l.rows = a->rows;
    l.vocab = a->vocab;
    l.row_stride = a->row_stride;
    l.vocab_offset = 0u;
    l.vocab_total = a->vocab;
    l.splits = plan.splits;
    l.split_len = plan.split_len;
    l.history_tokens = traits.penalties ? a->history_tokens : NULL;
    l.history_offsets = traits.penalties ? a->history_offsets : NULL;
    l.history_max = a->history_max;
    l.configs_device = a->config_count > 1u ? base + at_configs : NULL;
    l.config0 = a->configs[0];
    l.config_count = a->config_count;
    l.uniforms = a->uniforms;
    if (part_bytes) {
        const size_t slots = (size_t)a->rows * plan.splits;
        l.part_scores = (float *)(base + at_parts);
        l.part_ids = (uint32_t *)(base + at_parts + slots * 64u * 4u);
        l.part_meta = base + at_parts + slots * 64u * 8u;
    }
    l.tickets = (uint32_t *)(base + at_tickets);
    l.bitmap_words = plan.bitmap_words;
    l.count_capacity = plan.count_capacity;
    l.dense_wide = plan.dense_wide;
    view.first_error = (uint64_t *)base;
    fill_output(&l.out, &view, a);
    e = fgk_launch_stream_select(&l, cuda_stream);
    return e ? fg_cuda_fail(err, e, "streaming select kernel") : FG_OK;
}
