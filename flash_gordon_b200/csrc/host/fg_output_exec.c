/*
 * The stateful output executor of fg_cuda_sampler.h: session slots whose token history
 * lives on the GPU between decode steps, in the shape of the reference's fg_output executor
 * (include/fg_output.h:42-66; session slot src/output.c:40-52, history table :601-628,
 * one-token orchestration :702-755).
 *
 * Per session the reference keeps one table of occurrence counts, vocabulary long
 * (src/output.c:525).  So does this executor, on the device, plus a bitmap of the ids that
 * occur at all; the ring kernel fetches the bitmap (19 KB for 151,936 ids) instead of
 * rebuilding it from the token list on every step, and reads exact counts from the table.
 * After a step the tokens picked with penalties active are added to their sessions by a
 * small kernel on the same stream (src/output.c:742, 752).
 *
 * The token lists themselves are kept on the host as well: they are what
 * fg_output_history_reset is given, and what the register-prefetch kernel needs for the
 * batches the ring kernel does not take (penalties that can raise a logit, unaligned rows).
 */
#include "fg_host_internal.h"

#include <stdlib.h>
#include <string.h>

struct fg_cuda_output_executor {
    fg_cuda_context *context;
    uint32_t vocab, slots, capacity, bitmap_words, session;
    uint32_t *counts;      /* device [slots][vocab] */
    uint32_t *bitmaps;     /* device [slots][bitmap_words] */
    uint32_t *log;         /* host [slots][capacity] */
    uint32_t *length;      /* host [slots] */
    /* per-call staging, grown on demand */
    void *device_rows;     /* row -> session (u32), active flags (u8), then outputs for the one-row calls */
    size_t device_rows_bytes;
    void *device_history;  /* the fallback's CSR */
    size_t device_history_bytes;
    uint32_t *host_rows;   /* pinned: sessions | tokens | token logits | statuses */
    size_t host_rows_bytes;
    uint32_t *bad;         /* device word for history_reset */
};

static fg_status argument(fg_error *err, const char *why) {
    fg_error_set(err, FG_ERR_ARGUMENT, "%s", why);
    return FG_ERR_ARGUMENT;
}

fg_status fg_cuda_output_executor_create(fg_cuda_context *context, uint32_t vocab, uint32_t session_slots,
                                         uint32_t history_capacity, fg_cuda_output_executor **out,
                                         fg_error *err) {
    if (!context || !out || !vocab || !session_slots || session_slots > 65536u || !history_capacity ||
        history_capacity > FG_NATIVE_CONTEXT)
        return argument(err, "invalid output executor arguments");
    *out = NULL;
    fg_status status = fg_cuda_enter(context, err);
    if (status != FG_OK) return status;
    fg_cuda_output_executor *x = calloc(1, sizeof(*x));
    if (!x) {
        fg_error_set(err, FG_ERR_OOM, "out of host memory");
        return FG_ERR_OOM;
    }
    x->context = context;
    x->vocab = vocab;
    x->slots = session_slots;
    x->capacity = history_capacity;
    x->bitmap_words = ((vocab + 127u) / 128u) * 4u;  /* a whole number of 16-byte quads */
    x->log = malloc((size_t)session_slots * history_capacity * sizeof(uint32_t));
    x->length = calloc(session_slots, sizeof(uint32_t));
    int e = 0;
    if (!x->log || !x->length) {
        fg_error_set(err, FG_ERR_OOM, "out of host memory");
        status = FG_ERR_OOM;
    }
    const size_t counts_bytes = (size_t)session_slots * vocab * 4u;
    const size_t bitmaps_bytes = (size_t)session_slots * x->bitmap_words * 4u;
    if (status == FG_OK) e = fgk_malloc((void **)&x->counts, counts_bytes);
    if (status == FG_OK && !e) e = fgk_malloc((void **)&x->bitmaps, bitmaps_bytes);
    if (status == FG_OK && !e) e = fgk_malloc((void **)&x->bad, 256u);
    if (status == FG_OK && !e) e = fgk_memset_async(x->counts, 0, counts_bytes, context->stream);
    if (status == FG_OK && !e) e = fgk_memset_async(x->bitmaps, 0, bitmaps_bytes, context->stream);
    if (status == FG_OK && e) status = fg_cuda_fail(err, e, "allocating the session tables");
    if (status != FG_OK) {
        fg_cuda_output_executor_destroy(x);
        return status;
    }
    *out = x;
    return FG_OK;
}

void fg_cuda_output_executor_destroy(fg_cuda_output_executor *x) {
    if (!x) return;
    if (fgk_set_device(x->context->device) == 0) {
        if (x->context->stream) fgk_stream_synchronize(x->context->stream);
        if (x->counts) fgk_free(x->counts);
        if (x->bitmaps) fgk_free(x->bitmaps);
        if (x->bad) fgk_free(x->bad);
        if (x->device_rows) fgk_free(x->device_rows);
        if (x->device_history) fgk_free(x->device_history);
        if (x->host_rows) fgk_host_free(x->host_rows);
    }
    free(x->log);
    free(x->length);
    free(x);
}

void fg_cuda_output_set_session(fg_cuda_output_executor *x, uint32_t session_slot) {
    /* (the reference ignores a slot outside its table the same way, src/output.c:40-47) */
    if (x && session_slot < x->slots) x->session = session_slot;
}

uint32_t fg_cuda_output_session(const fg_cuda_output_executor *x) { return x ? x->session : 0u; }
uint32_t fg_cuda_output_history_length(const fg_cuda_output_executor *x, uint32_t session_slot) {
    return x && session_slot < x->slots ? x->length[session_slot] : 0u;
}

fg_status fg_cuda_output_history_reset(fg_cuda_output_executor *x, const uint32_t *history, uint32_t count,
                                       fg_error *err) {
    if (!x || (count && !history) || count > x->capacity)
        return argument(err, "invalid output history");
    for (uint32_t i = 0; i < count; i++) {
        if (history[i] >= x->vocab) {  /* src/output.c:610-612 */
            fg_error_set(err, FG_ERR_FORMAT, "history token %u at %u is outside vocabulary", history[i], i);
            return FG_ERR_FORMAT;
        }
    }
    fg_cuda_context *c = x->context;
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    uint32_t *counts = x->counts + (size_t)x->session * x->vocab;
    uint32_t *bitmap = x->bitmaps + (size_t)x->session * x->bitmap_words;
    int e = fgk_memset_async(counts, 0, (size_t)x->vocab * 4u, c->stream);
    if (!e && count) {
        status = fg_cuda_reserve(&x->device_history, &x->device_history_bytes, (size_t)count * 4u, false, c, err);
        if (status != FG_OK) return status;
        e = fgk_copy_to_device_async(x->device_history, history, (size_t)count * 4u, c->stream);
        if (!e) e = fgk_memset_async(x->bad, 0xff, 4u, c->stream);
        if (!e) e = fgk_launch_history_add(counts, x->vocab, x->device_history, count, x->bad, c->stream);
        c->launches++;
    }
    if (!e) e = fgk_launch_session_bitmap(bitmap, counts, x->vocab, x->bitmap_words, c->stream);
    c->launches++;
    /* `history` is the caller's: the copy must have left it before the call returns */
    if (!e) e = fgk_stream_synchronize(c->stream);
    if (e) return fg_cuda_fail(err, e, "resetting the session history");
    memcpy(x->log + (size_t)x->session * x->capacity, history, (size_t)count * 4u);
    x->length[x->session] = count;
    return FG_OK;
}

/* Grows the per-call staging for `rows` rows. */
static fg_status stage_rows(fg_cuda_output_executor *x, uint32_t rows, fg_error *err) {
    fg_cuda_context *c = x->context;
    const size_t device_bytes = (size_t)rows * (4u + 4u + 4u + 4u + 4u); /* sessions, active, tokens, logits, status */
    fg_status status = fg_cuda_reserve(&x->device_rows, &x->device_rows_bytes, device_bytes, false, c, err);
    if (status != FG_OK) return status;
    const size_t host_bytes = (size_t)rows * 5u * 4u;
    if (x->host_rows_bytes < host_bytes) {
        int e = fgk_stream_synchronize(c->stream);
        if (!e && x->host_rows) e = fgk_host_free(x->host_rows);
        x->host_rows = NULL;
        x->host_rows_bytes = 0;
        if (!e) e = fgk_host_alloc((void **)&x->host_rows, host_bytes + host_bytes / 4u);
        if (e) return fg_cuda_fail(err, e, "allocating pinned staging");
        x->host_rows_bytes = host_bytes + host_bytes / 4u;
    }
    return FG_OK;
}

/* One decode step for `args->rows` rows, row r belonging to session slots[r]: sample with the
 * sessions' histories, then add every token picked with penalties active to its session. */
fg_status fg_cuda_output_sample_sessions(fg_cuda_output_executor *x, const fg_cuda_sample_args *args,
                                         const uint32_t *slots, fg_error *err) {
    if (!x || !args || !slots || !args->rows || !args->configs ||
        (args->config_count != 1u && args->config_count != args->rows) || args->history_tokens ||
        args->history_offsets || args->vocab != x->vocab || !args->tokens || !args->row_status ||
        (args->flags & FG_CUDA_SAMPLE_ASYNC))
        return argument(err, "invalid executor sampling arguments");
    const uint32_t rows = args->rows;
    bool any_active = false;
    uint32_t longest = 0;
    for (uint32_t r = 0; r < rows; r++) {
        if (slots[r] >= x->slots) return argument(err, "session slot outside the executor's table");
        if (x->length[slots[r]] > longest) longest = x->length[slots[r]];
        if (fg_sampler_penalties_active(&args->configs[args->config_count == 1u ? 0u : r])) any_active = true;
    }
    fg_cuda_context *c = x->context;
    fg_status status = fg_cuda_enter(c, err);
    if (status == FG_OK) status = stage_rows(x, rows, err);
    if (status != FG_OK) return status;
    uint32_t *host_sessions = x->host_rows;
    unsigned char *host_active = (unsigned char *)(x->host_rows + rows);
    uint32_t *device_sessions = x->device_rows;
    unsigned char *device_active = (unsigned char *)(device_sessions + rows);
    for (uint32_t r = 0; r < rows; r++) {
        host_sessions[r] = slots[r];
        host_active[r] = fg_sampler_penalties_active(&args->configs[args->config_count == 1u ? 0u : r]) ? 1u : 0u;
    }
    int e = fgk_copy_to_device_async(device_sessions, host_sessions, (size_t)rows * 4u, c->stream);
    if (!e) e = fgk_copy_to_device_async(device_active, host_active, rows, c->stream);
    if (e) return fg_cuda_fail(err, e, "staging the session indices");

    fg_cuda_sample_args call = *args;
    call.flags |= FG_CUDA_SAMPLE_ASYNC;
    call.history_max = longest ? longest : 1u;
    fg_error quiet = {0};
    /* rows without a top-k cut are another kernel's, which reads token lists */
    const bool tables = any_active && !(args->flags & FG_CUDA_SAMPLE_ALLOW_NO_TOPK);
    if (tables) {
        c->session_counts = x->counts;
        c->session_bitmaps = x->bitmaps;
        c->session_rows = device_sessions;
        c->session_bitmap_words = x->bitmap_words;
    }
    status = tables || !any_active ? fg_cuda_sample_batch(c, &call, &quiet) : FG_ERR_UNAVAILABLE;
    c->session_counts = c->session_bitmaps = c->session_rows = NULL;
    c->session_bitmap_words = 0;
    if (status == FG_ERR_UNAVAILABLE && any_active) {
        /* the ring kernel cannot take this batch: token lists through the other kernel */
        uint64_t total = 0;
        for (uint32_t r = 0; r < rows; r++) total += x->length[slots[r]];
        const size_t offsets_at = (size_t)fg_align_up_u64(total * 4u, 256u);
        status = fg_cuda_reserve(&x->device_history, &x->device_history_bytes,
                                 offsets_at + ((size_t)rows + 1u) * 8u, false, c, err);
        if (status != FG_OK) return status;
        uint32_t *packed = malloc(offsets_at + ((size_t)rows + 1u) * 8u);
        if (!packed) {
            fg_error_set(err, FG_ERR_OOM, "out of host memory");
            return FG_ERR_OOM;
        }
        uint64_t *offsets = (uint64_t *)((unsigned char *)packed + offsets_at);
        uint64_t at = 0;
        for (uint32_t r = 0; r < rows; r++) {
            offsets[r] = at;
            memcpy(packed + at, x->log + (size_t)slots[r] * x->capacity, (size_t)x->length[slots[r]] * 4u);
            at += x->length[slots[r]];
        }
        offsets[rows] = at;
        e = fgk_copy_to_device_async(x->device_history, packed, offsets_at + ((size_t)rows + 1u) * 8u, c->stream);
        if (!e) e = fgk_stream_synchronize(c->stream); /* `packed` is freed below */
        free(packed);
        if (e) return fg_cuda_fail(err, e, "staging the token lists");
        call.history_tokens = x->device_history;
        call.history_offsets = (const uint64_t *)((unsigned char *)x->device_history + offsets_at);
        status = fg_cuda_sample_batch(c, &call, err);
    } else if (status != FG_OK && err) {
        *err = quiet;
    }
    if (status != FG_OK) return status;
    if (any_active) {
        e = fgk_launch_session_increment(x->counts, x->bitmaps, x->vocab, x->bitmap_words, device_sessions,
                                         args->tokens, args->row_status, device_active, rows, c->stream);
        c->launches++;
        if (e) return fg_cuda_fail(err, e, "session increment kernel");
    }
    /* tokens and statuses back, for the host's copy of the histories */
    uint32_t *host_tokens = x->host_rows + 2u * rows, *host_status = x->host_rows + 3u * rows;
    e = fgk_copy_to_host_async(host_tokens, args->tokens, (size_t)rows * 4u, c->stream);
    if (!e) e = fgk_copy_to_host_async(host_status, args->row_status, (size_t)rows * 4u, c->stream);
    if (e) return fg_cuda_fail(err, e, "reading the step's tokens");
    status = fg_cuda_collect(c, err); /* waits for the stream */
    for (uint32_t r = 0; r < rows; r++) {
        if (!host_active[r] || host_status[r] != (uint32_t)FG_OK) continue;
        uint32_t *length = &x->length[slots[r]];
        if (*length < x->capacity) x->log[(size_t)slots[r] * x->capacity + (*length)++] = host_tokens[r];
    }
    return status;
}

fg_status fg_cuda_output_history_increment(fg_cuda_output_executor *x, uint32_t token, fg_error *err) {
    if (!x) return argument(err, "invalid output executor");
    if (token >= x->vocab) {  /* src/output.c:622-624 */
        fg_error_set(err, FG_ERR_FORMAT, "history token %u is outside vocabulary", token);
        return FG_ERR_FORMAT;
    }
    fg_cuda_context *c = x->context;
    fg_status status = fg_cuda_enter(c, err);
    if (status == FG_OK) status = stage_rows(x, 1u, err);
    if (status != FG_OK) return status;
    /* one "row": this session, this token, status OK, active */
    uint32_t *host = x->host_rows;
    host[0] = x->session;
    host[1] = 1u;          /* active byte (little end first) */
    host[2] = token;
    host[3] = 0u;          /* FG_OK */
    uint32_t *device = x->device_rows;
    int e = fgk_copy_to_device_async(device, host, 16u, c->stream);
    if (!e) e = fgk_launch_session_increment(x->counts, x->bitmaps, x->vocab, x->bitmap_words, device, device + 2,
                                             device + 3, (const unsigned char *)(device + 1), 1u, c->stream);
    c->launches++;
    if (!e) e = fgk_stream_synchronize(c->stream);
    if (e) return fg_cuda_fail(err, e, "session increment kernel");
    uint32_t *length = &x->length[x->session];
    if (*length < x->capacity) x->log[(size_t)x->session * x->capacity + (*length)++] = token;
    return FG_OK;
}

fg_status fg_cuda_output_sample(fg_cuda_output_executor *x, const fg_cuda_tensor *logits,
                                const fg_sampler_config *config, float uniform, uint32_t *token, float *logit,
                                fg_error *err) {
    if (!x || !logits || !config || !token || !logit || logits->bytes < (uint64_t)x->vocab * 4u)
        return argument(err, "invalid output sampling arguments");
    fg_cuda_context *c = x->context;
    fg_status status = fg_cuda_enter(c, err);
    if (status == FG_OK) status = stage_rows(x, 8u, err);
    if (status != FG_OK) return status;
    /* device: [5 rows' worth of staging for the batched call][uniform, token, logit, status] */
    float *device_uniform = (float *)((uint32_t *)x->device_rows + 20);
    uint32_t *device_token = (uint32_t *)device_uniform + 1;
    float *device_logit = (float *)device_uniform + 2;
    uint32_t *device_status = (uint32_t *)device_uniform + 3;
    float *host_uniform = (float *)(x->host_rows + 20);
    *host_uniform = uniform;
    int e = fgk_copy_to_device_async(device_uniform, host_uniform, 4u, c->stream);
    if (e) return fg_cuda_fail(err, e, "staging the uniform draw");
    fg_cuda_sample_args args;
    memset(&args, 0, sizeof(args));
    args.logits = logits->base;
    args.dtype = FG_CUDA_F32;
    args.rows = 1u;
    args.vocab = x->vocab;
    args.row_stride = x->vocab;
    args.config_count = 1u;
    args.configs = config;
    args.uniforms = device_uniform;
    args.tokens = device_token;
    args.token_logits = device_logit;
    args.row_status = device_status;
    const uint32_t slot = x->session;
    status = fg_cuda_output_sample_sessions(x, &args, &slot, err);
    /* (the batched step has synchronised; its host copy of the token is the answer) */
    float back[2];
    e = fgk_copy_to_host_async(back, device_token, 8u, c->stream);
    if (!e) e = fgk_stream_synchronize(c->stream);
    if (e) return fg_cuda_fail(err, e, "reading the sampled token");
    memcpy(token, &back[0], 4);
    *logit = back[1];
    return status;
}

fg_status fg_cuda_output_greedy(fg_cuda_output_executor *x, const fg_cuda_tensor *logits, uint32_t *token,
                                float *logit, fg_error *err) {
    /* src/output.c:560-599: the argmax of the raw logits, no penalties, no history update */
    fg_sampler_config greedy;
    fg_sampler_config_greedy(&greedy);
    return fg_cuda_output_sample(x, logits, &greedy, 0.0f, token, logit, err);
}
