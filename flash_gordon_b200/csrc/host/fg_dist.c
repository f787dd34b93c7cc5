/*
 * The multi-GPU layer of fg_cuda_sampler.h: one process per GPU, one communicator per
 * process.  It holds the ncclComm_t and the exchange buffers; the kernels are the ones the
 * single-GPU entries launch.
 *
 * Vocabulary shards follow the reference's split output head: every slice reduces its own
 * columns (src/output.c:320-344), sends a small partial, and the partials are range-checked
 * against the slice spans and folded (src/runtime.c:2437-2466; spans as
 * src/protocol.c:93-105).  The reference sends one 12-byte (token_index, value, id) partial
 * per slice over TCP and only for greedy decoding; here a slice sends k_shard (value, id)
 * pairs per row in one all-gather over NVLink, so top-k / top-p sampling works too.
 */
#include "fg_host_internal.h"

#include <stdlib.h>
#include <string.h>

struct fg_dist {
    fg_cuda_context *context;
    void *comm;            /* ncclComm_t; NULL once aborted */
    uint32_t ranks, rank, timeout_ms;
    void *send;            /* this rank's [rows][k] (value, id) pairs */
    size_t send_bytes;
    void *gathered;        /* [rank][rows][k] pairs after the exchange */
    size_t gathered_bytes;
    /* the fused exchange: this rank's window and every rank's, as mapped into this process */
    void *window;
    size_t window_bytes;
    void *peer_window[16];
    uint32_t pair_capacity, row_capacity;
    uint32_t calls;        /* fused calls so far: the half alternates */
    void *handles;         /* device staging for the handle exchange */
};

static fg_status nccl_status(fg_dist *d, int code, const char *what, fg_error *err) {
    if (code == 0) return FG_OK;
    if (code == FGK_NCCL_MISSING) {
        fg_error_set(err, FG_ERR_UNAVAILABLE, "%s: libnccl.so.2 could not be loaded", what);
        return FG_ERR_UNAVAILABLE;
    }
    if (code == FGK_NCCL_TIMEOUT) {
        /* a rank never came: end whatever still waits for it on the GPU, fail closed */
        if (d && d->comm) {
            fgk_nccl_abort(d->comm);
            d->comm = NULL;
        }
        fg_error_set(err, FG_ERR_LIMIT, "%s: not every rank joined within %u ms; communicator aborted",
                     what, d ? d->timeout_ms : 0u);
        return FG_ERR_LIMIT;
    }
    if (code == FGK_NCCL_FAILED) {
        fg_error_set(err, FG_ERR_IO, "%s: NCCL reported an error", what);
        return FG_ERR_IO;
    }
    return fg_cuda_fail(err, code, what);
}

static void close_windows(fg_dist *d) {
    for (uint32_t r = 0; r < d->ranks; r++) {
        if (d->peer_window[r] && r != d->rank) fgk_ipc_close(d->peer_window[r]);
        d->peer_window[r] = NULL;
    }
    if (d->window) fgk_free(d->window);
    d->window = NULL;
    d->window_bytes = 0;
}

fg_status fg_dist_unique_id(void *id, fg_error *err) {
    if (!id) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid unique id buffer");
        return FG_ERR_ARGUMENT;
    }
    return nccl_status(NULL, fgk_nccl_unique_id(id), "creating the communicator id", err);
}

fg_status fg_dist_create(fg_cuda_context *context, uint32_t ranks, uint32_t rank, const void *id,
                         uint32_t timeout_ms, fg_dist **out, fg_error *err) {
    if (!context || !out || !id || ranks == 0u || ranks > 16u || rank >= ranks) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid communicator arguments");
        return FG_ERR_ARGUMENT;
    }
    *out = NULL;
    fg_status status = fg_cuda_enter(context, err);
    if (status != FG_OK) return status;
    fg_dist *d = calloc(1, sizeof(*d));
    if (!d) {
        fg_error_set(err, FG_ERR_OOM, "out of host memory");
        return FG_ERR_OOM;
    }
    d->context = context;
    d->ranks = ranks;
    d->rank = rank;
    d->timeout_ms = timeout_ms ? timeout_ms : FG_DIST_DEFAULT_TIMEOUT_MS;
    status = nccl_status(d, fgk_nccl_create(&d->comm, ranks, rank, id, d->timeout_ms),
                         "creating the communicator", err);
    if (status != FG_OK) {
        free(d);
        return status;
    }
    *out = d;
    return FG_OK;
}

void fg_dist_destroy(fg_dist *d) {
    if (!d) return;
    if (fgk_set_device(d->context->device) == 0) {
        if (d->context->stream) fgk_stream_synchronize(d->context->stream);
        if (d->comm) fgk_nccl_destroy(d->comm);
        if (d->send) fgk_free(d->send);
        if (d->gathered) fgk_free(d->gathered);
        close_windows(d);
        if (d->handles) fgk_free(d->handles);
    }
    free(d);
}

uint32_t fg_dist_ranks(const fg_dist *d) { return d ? d->ranks : 0u; }
uint32_t fg_dist_rank(const fg_dist *d) { return d ? d->rank : 0u; }

void fg_dist_shard_span(uint32_t vocab_total, uint32_t shards, uint32_t shard, uint32_t *first,
                        uint32_t *width) {
    /* equal widths, the last shard takes the remainder (src/protocol.c:99-103) */
    const uint32_t each = shards ? vocab_total / shards : 0u;
    const uint32_t begin = shard * each;
    if (first) *first = begin;
    if (width) *width = shard + 1u == shards ? vocab_total - begin : each;
}

/* Waits for the stream against the communicator's deadline, then reads the error word. */
static fg_status finish(fg_dist *d, const char *what, fg_error *err) {
    const int waited = fgk_stream_wait_deadline(d->context->stream, d->timeout_ms);
    if (waited) return nccl_status(d, waited, what, err);
    return fg_cuda_collect(d->context, err);
}

fg_status fg_dist_sample_vocab_sharded(fg_dist *d, const fg_cuda_sample_args *a, uint32_t vocab_total,
                                       uint32_t k_shard, fg_error *err) {
    if (!d || !a || k_shard < 1u || k_shard > 64u || !a->rows) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid sharded sampling arguments");
        return FG_ERR_ARGUMENT;
    }
    if (!d->comm) {
        fg_error_set(err, FG_ERR_UNAVAILABLE, "the communicator was aborted after a rank failed to join");
        return FG_ERR_UNAVAILABLE;
    }
    uint32_t first[16], width[16];
    for (uint32_t s = 0; s < d->ranks; s++) fg_dist_shard_span(vocab_total, d->ranks, s, &first[s], &width[s]);
    if (a->vocab != width[d->rank]) {
        fg_error_set(err, FG_ERR_ARGUMENT, "rank %u holds %u columns, its span of %u has %u", d->rank,
                     a->vocab, vocab_total, width[d->rank]);
        return FG_ERR_ARGUMENT;
    }
    fg_cuda_context *c = d->context;
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    const size_t mine = (size_t)a->rows * k_shard * 8u;
    status = fg_cuda_reserve(&d->send, &d->send_bytes, mine, false, c, err);
    if (status == FG_OK)
        status = fg_cuda_reserve(&d->gathered, &d->gathered_bytes, mine * d->ranks, false, c, err);
    if (status != FG_OK) return status;

    /* 1. this rank's columns -> k_shard (value, id) pairs per row, written as pairs */
    status = fg_cuda_shard_topk_layout(c, a, first[d->rank], vocab_total, k_shard, (float *)d->send,
                                       (uint32_t *)d->send + 1, 2u, err);
    if (status != FG_OK) return status;
    /* 2. the one exchange */
    status = nccl_status(d, fgk_nccl_all_gather(d->comm, d->send, d->gathered, mine, c->stream, d->timeout_ms),
                         "all-gather of the shard candidates", err);
    c->launches++;
    if (status != FG_OK) return status;
    /* 3. span check, merge under (value desc, global id asc), select -- on every rank */
    status = fg_cuda_merge_select_layout(c, a, (const float *)d->gathered, (const uint32_t *)d->gathered + 1,
                                         2u, d->ranks, k_shard, first, width, true, NULL, err);
    if (status != FG_OK || (a->flags & FG_CUDA_SAMPLE_ASYNC)) return status;
    return finish(d, "vocabulary-sharded sampling", err);
}

/* Makes sure every rank has a window that takes `rows` rows of k pairs from every rank, and
 * that this process can store into all of them.  Collective: every rank calls it with the
 * same sizes (they sample the same rows), so all grow together. */
static fg_status ensure_windows(fg_dist *d, uint32_t rows, uint32_t k, fg_error *err) {
    const uint64_t pairs = (uint64_t)rows * k;
    if (d->window && pairs <= d->pair_capacity && rows <= d->row_capacity) return FG_OK;
    fg_cuda_context *c = d->context;
    int e = fgk_stream_synchronize(c->stream);
    if (e) return fg_cuda_fail(err, e, "draining the stream");
    close_windows(d);
    d->pair_capacity = (uint32_t)(pairs + pairs / 4u);
    d->row_capacity = rows + rows / 4u;
    const size_t bytes = (size_t)2u * d->ranks * d->pair_capacity * 8u + (size_t)2u * d->row_capacity * 4u;
    e = fgk_malloc(&d->window, bytes);
    if (!e) e = fgk_memset_async(d->window, 0, bytes, c->stream);
    if (!e && !d->handles) e = fgk_malloc(&d->handles, (size_t)(d->ranks + 1u) * FGK_IPC_HANDLE_BYTES);
    if (e) return fg_cuda_fail(err, e, "allocating the exchange window");
    d->window_bytes = bytes;
    d->calls = 0;
    d->peer_window[d->rank] = d->window;
    if (d->ranks > 1u) {
        /* every rank's handle to every rank: one small all-gather through device memory */
        unsigned char mine[FGK_IPC_HANDLE_BYTES], all[16 * FGK_IPC_HANDLE_BYTES];
        e = fgk_ipc_handle(d->window, mine);
        unsigned char *send = (unsigned char *)d->handles + (size_t)d->ranks * FGK_IPC_HANDLE_BYTES;
        if (!e) e = fgk_copy_to_device_async(send, mine, FGK_IPC_HANDLE_BYTES, c->stream);
        if (e) return fg_cuda_fail(err, e, "exporting the exchange window");
        fg_status status = nccl_status(d, fgk_nccl_all_gather(d->comm, send, d->handles, FGK_IPC_HANDLE_BYTES,
                                                              c->stream, d->timeout_ms),
                                       "exchanging the window handles", err);
        if (status != FG_OK) return status;
        e = fgk_copy_to_host_async(all, d->handles, (size_t)d->ranks * FGK_IPC_HANDLE_BYTES, c->stream);
        if (e) return fg_cuda_fail(err, e, "reading the window handles");
        const int waited = fgk_stream_wait_deadline(c->stream, d->timeout_ms);
        if (waited) return nccl_status(d, waited, "exchanging the window handles", err);
        for (uint32_t r = 0; r < d->ranks; r++) {
            if (r == d->rank) continue;
            e = fgk_ipc_open(all + (size_t)r * FGK_IPC_HANDLE_BYTES, &d->peer_window[r]);
            if (e) return fg_cuda_fail(err, e, "mapping a peer's exchange window");
        }
    } else {
        e = fgk_stream_synchronize(c->stream);
        if (e) return fg_cuda_fail(err, e, "clearing the exchange window");
    }
    return FG_OK;
}

fg_status fg_dist_sample_vocab_sharded_fused(fg_dist *d, const fg_cuda_sample_args *a, uint32_t vocab_total,
                                             uint32_t k_shard, fg_error *err) {
    if (!d || !a || k_shard < 1u || k_shard > 64u || !a->rows) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid sharded sampling arguments");
        return FG_ERR_ARGUMENT;
    }
    if (!d->comm) {
        fg_error_set(err, FG_ERR_UNAVAILABLE, "the communicator was aborted after a rank failed to join");
        return FG_ERR_UNAVAILABLE;
    }
    uint32_t first[16], width[16];
    for (uint32_t s = 0; s < d->ranks; s++) fg_dist_shard_span(vocab_total, d->ranks, s, &first[s], &width[s]);
    if (a->vocab != width[d->rank]) {
        fg_error_set(err, FG_ERR_ARGUMENT, "rank %u holds %u columns, its span of %u has %u", d->rank,
                     a->vocab, vocab_total, width[d->rank]);
        return FG_ERR_ARGUMENT;
    }
    fg_cuda_context *c = d->context;
    fg_status status = fg_cuda_enter(c, err);
    if (status == FG_OK) status = ensure_windows(d, a->rows, k_shard, err);
    if (status != FG_OK) return status;
    /* Alternate calls use alternate halves of the windows: a rank can be one call ahead of
     * another (it cannot start the call after, whose merge needs this one's blocks from
     * everybody), so what it stores never lands on what a slower rank still reads. */
    const uint32_t half = d->calls & 1u;
    fgk_push push;
    memset(&push, 0, sizeof(push));
    for (uint32_t r = 0; r < d->ranks; r++) push.window[r] = d->peer_window[r];
    push.ranks = d->ranks;
    push.rank = d->rank;
    push.half = half;
    push.pair_capacity = d->pair_capacity;
    push.row_capacity = d->row_capacity;
    /* 1. this rank's columns -> k_shard pairs per row, stored into every rank's window */
    c->push = &push;
    status = fg_cuda_shard_topk_layout(c, a, first[d->rank], vocab_total, k_shard, NULL, NULL, 2u, err);
    c->push = NULL;
    if (status != FG_OK) return status;
    d->calls++;
    /* 2. merge what has landed here: a row is read once all ranks have counted themselves in
     * (the merge sets the row's counter back to zero) */
    unsigned char *mine = d->window;
    const unsigned char *pairs = mine + (size_t)half * d->ranks * d->pair_capacity * 8u;
    uint32_t *counters = (uint32_t *)(mine + (size_t)2u * d->ranks * d->pair_capacity * 8u) +
                         (size_t)half * d->row_capacity;
    fg_cuda_arrivals arrivals = {d->pair_capacity, counters, d->ranks, 0u};
    status = fg_cuda_merge_select_layout(c, a, (const float *)pairs, (const uint32_t *)pairs + 1, 2u, d->ranks,
                                         k_shard, first, width, true, &arrivals, err);
    if (status != FG_OK || (a->flags & FG_CUDA_SAMPLE_ASYNC)) return status;
    status = finish(d, "vocabulary-sharded sampling (fused exchange)", err);
    if (status == FG_ERR_LIMIT && d->comm) {  /* a rank never stored its blocks: the counters are out of step for good */
        fgk_nccl_abort(d->comm);
        d->comm = NULL;
    }
    return status;
}

fg_status fg_dist_gather_rows(fg_dist *d, const uint32_t *tokens, const float *token_logits,
                              const uint32_t *row_status, uint32_t rows, uint32_t *all_tokens,
                              float *all_token_logits, uint32_t *all_row_status, fg_error *err) {
    if (!d || !tokens || !token_logits || !row_status || !rows || !all_tokens || !all_token_logits ||
        !all_row_status) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid row gather arguments");
        return FG_ERR_ARGUMENT;
    }
    if (!d->comm) {
        fg_error_set(err, FG_ERR_UNAVAILABLE, "the communicator was aborted after a rank failed to join");
        return FG_ERR_UNAVAILABLE;
    }
    fg_cuda_context *c = d->context;
    fg_status status = fg_cuda_enter(c, err);
    if (status != FG_OK) return status;
    /* three all-gathers of rows * 4 bytes each: the arrays stay the caller's, nothing is packed */
    const size_t bytes = (size_t)rows * 4u;
    int e = fgk_nccl_all_gather(d->comm, tokens, all_tokens, bytes, c->stream, d->timeout_ms);
    if (!e) e = fgk_nccl_all_gather(d->comm, token_logits, all_token_logits, bytes, c->stream, d->timeout_ms);
    if (!e) e = fgk_nccl_all_gather(d->comm, row_status, all_row_status, bytes, c->stream, d->timeout_ms);
    if (e) return nccl_status(d, e, "all-gather of the row results", err);
    const int waited = fgk_stream_wait_deadline(c->stream, d->timeout_ms);
    return waited ? nccl_status(d, waited, "all-gather of the row results", err) : FG_OK;
}
