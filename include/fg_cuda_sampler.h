/*
 * CUDA (sm_100a) sampling operators behind a C ABI.
 *
 * Three groups of entry points:
 *
 *   1. Context and tensors.  A context binds one GPU and one stream and owns
 *      the scratch the kernels need; a tensor is a byte range of device memory
 *      (owned, a view of another tensor, or wrapped caller memory).  They stand
 *      in for the reference's fg_vk_context / fg_vk_tensor
 *      (include/fg_vk.h:6-8, 89-90, 147-148, 206-224).
 *
 *   2. Device operators with the argument meaning and error behaviour of the
 *      reference's Vulkan wrappers (src/vk.c:1808-1824, 2237-2256, 2260) plus
 *      the history table of the output executor (src/output.c:601-628).
 *
 *   3. Fused batched sampling: one call turns `rows` rows of vocabulary logits
 *      into `rows` token ids (penalties, greedy argmax or top-k / top-p /
 *      temperature selection), reading each logit from HBM once.  The
 *      reference does this one row per call in fg_output_sample
 *      (src/output.c:702-755); the per-row result is the same.
 *
 * Conventions: every function returns fg_status; `err` may be NULL; the
 * library never frees or retains caller memory; a context is used by one
 * thread at a time.  Work is enqueued on the context's stream; calls that hand
 * data back to the host (tensor_read, fg_cuda_end, the *_host entry and the
 * synchronous form of fg_cuda_sample_batch) wait for it.
 */
#ifndef FG_B200_CUDA_SAMPLER_H
#define FG_B200_CUDA_SAMPLER_H

#include "fg.h"
#include "fg_sampler.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fg_cuda_context fg_cuda_context;
typedef struct fg_cuda_tensor fg_cuda_tensor;

/* ------------------------------------------------------------------ context */

/* Opens `device`, creates the context's stream and scratch.  Stands in for
 * fg_vk_open (include/fg_vk.h:89).  FG_ERR_UNAVAILABLE when no CUDA device or
 * driver is usable. */
fg_status fg_cuda_context_create(int device, fg_cuda_context **out, fg_error *err);
/* Stands in for fg_vk_close (include/fg_vk.h:90).  NULL is ignored. */
void fg_cuda_context_destroy(fg_cuda_context *context);
/* Run on a stream the caller owns (a cudaStream_t passed as void*; NULL is the
 * CUDA default stream).  No reference counterpart: Vulkan queues are owned by
 * the reference's context. */
fg_status fg_cuda_context_set_stream(fg_cuda_context *context, void *cuda_stream, fg_error *err);
/* Back to the stream the context created for itself. */
fg_status fg_cuda_context_reset_stream(fg_cuda_context *context, fg_error *err);
/* The cudaStream_t work is enqueued on. */
void *fg_cuda_context_stream(const fg_cuda_context *context);
int fg_cuda_context_device(const fg_cuda_context *context);
/* Number of streaming multiprocessors of the bound GPU (grid sizing, reports). */
uint32_t fg_cuda_context_sm_count(const fg_cuda_context *context);
/* Kernels launched by this context since creation (bench bookkeeping). */
uint64_t fg_cuda_context_launches(const fg_cuda_context *context);
/* Tuning knob, no reference counterpart: how many CTAs share one row in the
 * fused path (0 = chosen per call from rows, vocabulary and SM count; at most
 * 16).  Results never depend on it. */
fg_status fg_cuda_context_set_splits(fg_cuda_context *context, uint32_t splits, fg_error *err);
/* Tuning knob, no reference counterpart: which of the two fused kernels a batch
 * with a top-k cut takes — the persistent kernel that streams rows through a
 * shared-memory ring fed by bulk copies (rows whose start, stride and length are
 * multiples of 16 bytes, penalties that cannot raise a logit), or the
 * register-prefetch kernel (anything).  AUTO is the library's choice: the ring
 * kernel whenever it can take the batch.  RING fails with FG_ERR_ARGUMENT on a
 * batch it cannot take, RING_IF_POSSIBLE falls back instead (as AUTO does).
 * Results never depend on it. */
#define FG_CUDA_PATH_AUTO             0u
#define FG_CUDA_PATH_REGISTERS        1u
#define FG_CUDA_PATH_RING             2u
#define FG_CUDA_PATH_RING_IF_POSSIBLE 3u
fg_status fg_cuda_context_set_path(fg_cuda_context *context, uint32_t path, fg_error *err);
/* fg_vk_begin / fg_vk_end (include/fg_vk.h:147-148): the reference records
 * dispatches into one submission and waits on its fence at `end`.  Here begin
 * only marks the batch; end waits for the stream and surfaces device errors. */
fg_status fg_cuda_begin(fg_cuda_context *context, fg_error *err);
fg_status fg_cuda_end(fg_cuda_context *context, fg_error *err);
bool fg_cuda_batch_active(const fg_cuda_context *context);

/* ------------------------------------------------------------------ tensors */

/* fg_vk_tensor_create (include/fg_vk.h:206): `bytes` of zero-filled device memory. */
fg_status fg_cuda_tensor_create(fg_cuda_context *context, uint64_t bytes,
                                fg_cuda_tensor **out, fg_error *err);
/* fg_vk_tensor_view (include/fg_vk.h:208): a window into `base`; never owns memory. */
fg_status fg_cuda_tensor_view(fg_cuda_tensor *base, uint64_t offset, uint64_t bytes,
                              fg_cuda_tensor **out, fg_error *err);
/* Wrap device memory the caller allocated (e.g. the output of an lm_head GEMM).
 * No reference counterpart: its tensors are always context allocations. */
fg_status fg_cuda_tensor_wrap(fg_cuda_context *context, void *device_pointer, uint64_t bytes,
                              fg_cuda_tensor **out, fg_error *err);
/* fg_vk_tensor_destroy (include/fg_vk.h:212). */
void fg_cuda_tensor_destroy(fg_cuda_tensor *tensor);
/* fg_vk_tensor_bytes (include/fg_vk.h:213). */
uint64_t fg_cuda_tensor_bytes(const fg_cuda_tensor *tensor);
/* Device address; plays the part of fg_vk_tensor_map (include/fg_vk.h:217) for
 * code that hands the memory to other CUDA work.  Not host-dereferenceable. */
void *fg_cuda_tensor_device_pointer(const fg_cuda_tensor *tensor);
/* fg_vk_tensor_write / fg_vk_tensor_read (include/fg_vk.h:221-224): host <-> device
 * copies ordered with the context's stream; read waits for completion. */
fg_status fg_cuda_tensor_write(fg_cuda_tensor *tensor, uint64_t offset, const void *data,
                               uint64_t bytes, fg_error *err);
fg_status fg_cuda_tensor_read(const fg_cuda_tensor *tensor, uint64_t offset, void *data,
                              uint64_t bytes, fg_error *err);

/* --------------------------------------------------------- device operators */

/* fg_vk_apply_penalties (src/vk.c:1808-1824) + shaders/fg_apply_penalties.comp.
 * In place over logits[0..values): ids whose count is zero are untouched; the
 * others get  v = (v > 0 ? v / repetition : v * repetition)  when repetition
 * != 1, then  v - (frequency * (float)count + presence),  each step rounded to
 * fp32 with no fused multiply-add (the association of src/sampler.c:46-60). */
fg_status fg_cuda_apply_penalties(fg_cuda_context *context, fg_cuda_tensor *logits,
                                  const fg_cuda_tensor *counts, uint32_t values,
                                  float presence_penalty, float frequency_penalty,
                                  float repetition_penalty, fg_error *err);

/* fg_vk_argmax_reduce (src/vk.c:2260) + shaders/fg_argmax_reduce.comp.  One
 * (score, id) winner per 4096-element tile under the reference's total order
 * (padding id 0xffffffff loses; a non-finite score beats a finite one; then
 * larger score; then smaller id).  *output_count = ceil(count / 4096).
 * in_ids == NULL means ids are 0..count-1 (the reference materialises that
 * table, src/output.c:526-528; here it is never read from memory). */
fg_status fg_cuda_argmax_reduce(fg_cuda_context *context, fg_cuda_tensor *out_scores,
                                fg_cuda_tensor *out_ids, const fg_cuda_tensor *in_scores,
                                const fg_cuda_tensor *in_ids, uint32_t count,
                                uint32_t *output_count, fg_error *err);

/* fg_vk_topk_select (src/vk.c:2237-2256) + shaders/fg_topk_select*.comp.  The k
 * best finite (score, id) pairs of every 1024-element tile, ordered inside the
 * tile by (score descending, id ascending); missing entries are padded with
 * (-inf, 0xffffffff).  1 <= k <= 64.  *output_count = ceil(count / 1024) * k.
 * in_ids == NULL means ids are 0..count-1. */
fg_status fg_cuda_topk_select(fg_cuda_context *context, fg_cuda_tensor *out_scores,
                              fg_cuda_tensor *out_ids, const fg_cuda_tensor *in_scores,
                              const fg_cuda_tensor *in_ids, uint32_t count, uint32_t k,
                              uint32_t *output_count, fg_error *err);

/* fg_vk_topk_reduce (src/vk.c:2235) + shaders/fg_topk_reduce_v2.comp: the 512 best
 * (score, id) pairs of every 4096-element tile, SORTED by the order of that shader: a padding
 * id last, a NaN/Inf before every finite score (smaller id first among them), then larger
 * score, then smaller id.  The reference's long-context block selection cascades it
 * (src/qsa.c:833-855).  *output_count = ceil(count / 4096) * 512, or `count` when a lone tile
 * holds fewer than 512; short tiles are padded with (-inf, 0xffffffff).  in_ids == NULL means
 * ids are 0..count-1. */
fg_status fg_cuda_topk_reduce(fg_cuda_context *context, fg_cuda_tensor *out_scores,
                              fg_cuda_tensor *out_ids, const fg_cuda_tensor *in_scores,
                              const fg_cuda_tensor *in_ids, uint32_t count, uint32_t *output_count,
                              fg_error *err);

/* fg_vk_router_top10 (src/vk.c:2257) generalised to any k <= 32, with the arithmetic of the
 * reference's CPU statement fg_q38_router_topk (src/q38_math.c:48-64): per token the k
 * largest of `experts` logits (ties: smaller id) into selected[tokens][k], and into
 * gates[tokens][k] their softmax probabilities over ALL experts (fp64), rounded to fp32 and
 * renormalised by their sum.  A token with a NaN or +Inf logit gets ids 0xffffffff and
 * weights 0 (as the shader leaves them) and the call returns FG_ERR_FORMAT naming it. */
fg_status fg_cuda_router_topk(fg_cuda_context *context, fg_cuda_tensor *selected, fg_cuda_tensor *gates,
                              const fg_cuda_tensor *logits, uint32_t experts, uint32_t tokens, uint32_t k,
                              fg_error *err);

/* fg_output_history_reset (src/output.c:601-617) for a device-resident table:
 * counts[0..vocab) = occurrences of each id in history[0..count) (host
 * pointer), saturating at UINT32_MAX.  count <= FG_NATIVE_CONTEXT; an id
 * >= vocab yields FG_ERR_FORMAT. */
fg_status fg_cuda_history_reset(fg_cuda_context *context, fg_cuda_tensor *counts,
                                uint32_t vocab, const uint32_t *history, uint32_t count,
                                fg_error *err);
/* fg_output_history_increment (src/output.c:619-628). */
fg_status fg_cuda_history_increment(fg_cuda_context *context, fg_cuda_tensor *counts,
                                    uint32_t vocab, uint32_t token, fg_error *err);

/* ------------------------------------------------------------ fused batched */

typedef enum fg_cuda_dtype {
    FG_CUDA_F32  = 0,
    FG_CUDA_BF16 = 1   /* widened exactly to fp32 before any arithmetic */
} fg_cuda_dtype;

/* Bits of fg_cuda_sample_args.flags. */
#define FG_CUDA_SAMPLE_ASYNC     1u  /* enqueue only; caller reads row_status itself       */
#define FG_CUDA_SAMPLE_ALLOW_NO_TOPK 2u /* top_k == 0 means "no top-k cut" (top-p over all) */

/* Optional per-row dump of the final candidate list (device pointers, each
 * rows * 64 entries except count: rows).  Entries are in sampling order
 * (score descending, id ascending).  probabilities are the doubles the select
 * step used, rounded to fp64 storage: raw = exp(s_i - s_0) / sum over the
 * top-k set, tempered = w_i / temp_sum over the top-p survivors (0 beyond). */
typedef struct fg_cuda_sample_debug {
    uint32_t *candidate_count;
    uint32_t *candidate_ids;
    float    *candidate_scores;
    double   *raw_probability;
    double   *tempered_probability;
} fg_cuda_sample_debug;

/* One batched sampling call.  Device pointers unless marked HOST. */
typedef struct fg_cuda_sample_args {
    const void     *logits;          /* rows x row_stride elements of `dtype`               */
    uint32_t        dtype;           /* fg_cuda_dtype                                         */
    uint32_t        rows;
    uint32_t        vocab;           /* logits per row that are read                          */
    uint32_t        flags;
    uint64_t        row_stride;      /* elements between row starts, >= vocab                 */
    const uint32_t *history_tokens;  /* CSR payload; NULL when no row has history             */
    const uint64_t *history_offsets; /* rows + 1 entries; row r owns [off[r], off[r+1])       */
    uint32_t        history_max;     /* HOST-known upper bound of any row's history length    */
    uint32_t        config_count;    /* 1 (shared by all rows) or rows                        */
    const fg_sampler_config *configs;/* HOST pointer                                          */
    const float    *uniforms;        /* rows; one U[0,1) draw per row (unused by greedy rows) */
    uint32_t       *tokens;          /* out, rows                                             */
    float          *token_logits;    /* out, rows: penalised raw logit of the pick            */
    uint32_t       *row_status;      /* out, rows: fg_status per row                          */
    const fg_cuda_sample_debug *debug; /* HOST pointer to the struct; may be NULL             */
} fg_cuda_sample_args;

/* Per row: A. history -> counts (src/output.c:601-617); B. penalties
 * (src/sampler.c:46-60); C. temperature == 0: argmax under the reference's
 * total order, a non-finite winner is an error (FG_ERR_FORMAT with penalties
 * active, FG_ERR_MISMATCH without; src/output.c:593, 737-739); temperature > 0:
 * the top_k best finite logits (score descending, id ascending), then top-p on
 * the untempered softmax of that set, then temperature softmax and inverse CDF
 * with the row's uniform (src/sampler.c:80-122).
 * Configs are validated like fg_sampler_config_validate; with
 * FG_CUDA_SAMPLE_ALLOW_NO_TOPK, top_k == 0 is also accepted.
 * Returns the status of the lowest failing row (FG_OK when all rows are OK);
 * with FG_CUDA_SAMPLE_ASYNC returns after enqueueing. */
fg_status fg_cuda_sample_batch(fg_cuda_context *context, const fg_cuda_sample_args *args,
                               fg_error *err);

/* Same call with every buffer in HOST memory: copies inputs to the device,
 * samples, copies tokens / token_logits / row_status back.  This is what a
 * reference-shaped caller (logits produced elsewhere, token needed on the
 * host) binds; `debug` must be NULL. */
fg_status fg_cuda_sample_batch_host(fg_cuda_context *context, const fg_cuda_sample_args *host_args,
                                    fg_error *err);

/* Vocabulary-sharded sampling, step 1 (per GPU).  The logits are columns
 * [vocab_offset, vocab_offset + args->vocab) of a vocab_total-wide head;
 * history ids are global and only those inside the shard are applied.  Writes
 * the shard's k_shard best finite (score, global id) pairs per row, padded
 * with (-inf, 0xffffffff), into candidate_scores / candidate_ids
 * (rows x k_shard, device).  The reference's analogue is the split head's
 * per-slice argmax partial (src/output.c:320-344, ids pre-offset by
 * first_row); here the partial carries k_shard entries instead of one.
 * tokens / token_logits / uniforms of `args` are ignored. */
fg_status fg_cuda_shard_topk(fg_cuda_context *context, const fg_cuda_sample_args *args,
                             uint32_t vocab_offset, uint32_t vocab_total, uint32_t k_shard,
                             float *candidate_scores, uint32_t *candidate_ids, fg_error *err);

/* Step 2, after the exchange: every row has `shards` blocks of k_shard
 * candidates, laid out [shard][row][k_shard] (the order an all-gather leaves
 * them in).  Each candidate id must lie inside its shard's span
 * [shard_first[s], shard_first[s] + shard_width[s]) (HOST arrays), else the
 * row fails with FG_ERR_MISMATCH — the check of worker_output_split_combine
 * (src/runtime.c:2437-2466).  Then the merged set is sampled exactly as in
 * fg_cuda_sample_batch (greedy rows: fold under the argmax total order).
 * Uses configs / uniforms / tokens / token_logits / row_status / debug /
 * rows / flags of `args`. */
fg_status fg_cuda_merge_select(fg_cuda_context *context, const fg_cuda_sample_args *args,
                               const float *candidate_scores, const uint32_t *candidate_ids,
                               uint32_t shards, uint32_t k_shard,
                               const uint32_t *shard_first, const uint32_t *shard_width,
                               fg_error *err);

/* ------------------------------------------------------- stateful executor */

/* Session slots whose token history stays on the GPU between decode steps: the shape of
 * the reference's output executor (include/fg_output.h:42-66), which keeps one occurrence
 * table per session (src/output.c:525, 601-628) and adds every token it picks with
 * penalties active (src/output.c:742, 752).  Logits come from the caller (the lm_head that
 * produces them is not part of this library); everything after them is here.
 *   vocab             logits per row (fp32 for the one-row calls)
 *   session_slots     sessions the executor can hold (the reference has 2)
 *   history_capacity  most tokens one session's history may hold (<= FG_NATIVE_CONTEXT) */
typedef struct fg_cuda_output_executor fg_cuda_output_executor;
/* fg_output_executor_create / _destroy (include/fg_output.h:42-43). */
fg_status fg_cuda_output_executor_create(fg_cuda_context *context, uint32_t vocab, uint32_t session_slots,
                                         uint32_t history_capacity, fg_cuda_output_executor **out,
                                         fg_error *err);
void fg_cuda_output_executor_destroy(fg_cuda_output_executor *executor);
/* fg_output_set_session / fg_output_session (include/fg_output.h:49-50): the session the
 * one-row calls below serve.  A slot outside the table is ignored. */
void fg_cuda_output_set_session(fg_cuda_output_executor *executor, uint32_t session_slot);
uint32_t fg_cuda_output_session(const fg_cuda_output_executor *executor);
uint32_t fg_cuda_output_history_length(const fg_cuda_output_executor *executor, uint32_t session_slot);
/* fg_output_history_reset (include/fg_output.h:44-46; src/output.c:601-617): the current
 * session's history becomes history[0..count) (HOST).  A token >= vocab: FG_ERR_FORMAT. */
fg_status fg_cuda_output_history_reset(fg_cuda_output_executor *executor, const uint32_t *history,
                                       uint32_t count, fg_error *err);
/* fg_output_history_increment (include/fg_output.h:51-52; src/output.c:619-628). */
fg_status fg_cuda_output_history_increment(fg_cuda_output_executor *executor, uint32_t token, fg_error *err);
/* fg_output_greedy (include/fg_output.h:55-56; src/output.c:560-599) on a row of fp32 logits:
 * argmax of the raw logits; a NaN/Inf finalist is FG_ERR_MISMATCH. */
fg_status fg_cuda_output_greedy(fg_cuda_output_executor *executor, const fg_cuda_tensor *logits,
                                uint32_t *token, float *logit, fg_error *err);
/* fg_output_sample (include/fg_output.h:64-66; src/output.c:702-755) on a row of fp32 logits
 * with the current session's history; when the config's penalties are active the picked
 * token joins that history. */
fg_status fg_cuda_output_sample(fg_cuda_output_executor *executor, const fg_cuda_tensor *logits,
                                const fg_sampler_config *config, float uniform, uint32_t *token,
                                float *logit, fg_error *err);
/* The same for a whole decode step (no reference counterpart: it decodes one row per call):
 * args as for fg_cuda_sample_batch with history_tokens / history_offsets NULL and without
 * FG_CUDA_SAMPLE_ASYNC; row r belongs to session slots[r] (HOST array).  Rows whose
 * penalties are active and that end FG_OK add their token to their session. */
fg_status fg_cuda_output_sample_sessions(fg_cuda_output_executor *executor, const fg_cuda_sample_args *args,
                                         const uint32_t *slots, fg_error *err);

/* ---------------------------------------------------------------- multi-GPU */

/* One process per GPU; a fg_dist joins `ranks` of them through one NCCL communicator
 * bound to the context's GPU and stream.  It stands in for the reference's fabric on the
 * output path (include/fg_fabric.h; the split head's partials, src/runtime.c:2534-2561):
 * TCP sockets there, NCCL over NVLink here.  libnccl.so.2 is opened on first use (the
 * FG_NCCL_LIBRARY variable names another file); FG_ERR_UNAVAILABLE when it is missing.
 *
 * Row partition needs none of this on the data path: rows are independent, each
 * rank samples its own block with fg_cuda_sample_batch.  fg_dist_gather_rows is for
 * callers that want every rank's results on every rank.
 *
 * Every call that waits for other ranks has a deadline (`timeout_ms`, 0 = 30 s).  When
 * it passes, the communicator is aborted -- which also ends a collective that still
 * waits on the GPU -- the call returns FG_ERR_LIMIT, and later calls on this fg_dist
 * return FG_ERR_UNAVAILABLE.  The reference turns a partial that misses its 4 s
 * deadline into FG_ERR_LIMIT the same way (src/runtime.c:2379-2435). */
typedef struct fg_dist fg_dist;
#define FG_DIST_UNIQUE_ID_BYTES 128u
#define FG_DIST_DEFAULT_TIMEOUT_MS 30000u

/* Rank 0 fills `id` (FG_DIST_UNIQUE_ID_BYTES bytes, HOST) and carries it to the other
 * ranks by whatever means the processes already share (the reference's ranks know
 * each other from the manifest); every rank then passes the same bytes to
 * fg_dist_create. */
fg_status fg_dist_unique_id(void *id, fg_error *err);
fg_status fg_dist_create(fg_cuda_context *context, uint32_t ranks, uint32_t rank, const void *id,
                         uint32_t timeout_ms, fg_dist **out, fg_error *err);
/* NULL is ignored.  Destroy before the context. */
void fg_dist_destroy(fg_dist *dist);
uint32_t fg_dist_ranks(const fg_dist *dist);
uint32_t fg_dist_rank(const fg_dist *dist);

/* Column span of `shard` when vocab_total columns are split over `shards` GPUs: equal
 * widths, the last one takes the remainder -- the rule of the reference's 4-way split
 * (src/protocol.c:93-105). */
void fg_dist_shard_span(uint32_t vocab_total, uint32_t shards, uint32_t shard, uint32_t *first,
                        uint32_t *width);

/* Vocabulary-sharded sampling, all three steps, called by every rank with its own
 * columns of the same rows (`args->logits`: rows x its span's width, `args->vocab` that
 * width; history ids are global; configs, uniforms and outputs as in
 * fg_cuda_sample_batch, identical on every rank):
 *   1. fg_cuda_shard_topk on this rank's columns, written as (fp32 value, uint32 global
 *      id) pairs straight into the send buffer;
 *   2. one ncclAllGather of rows * k_shard * 8 bytes per rank;
 *   3. fg_cuda_merge_select over the gathered [rank][row][k_shard] pairs, on every rank
 *      (every rank ends with the same tokens).
 * Nothing is copied between the steps.  sampled rows need top_k <= k_shard. */
fg_status fg_dist_sample_vocab_sharded(fg_dist *dist, const fg_cuda_sample_args *args,
                                       uint32_t vocab_total, uint32_t k_shard, fg_error *err);

/* The same call with the exchange fused into the two kernels: the shard kernel stores every
 * row's block of pairs straight into every rank's window over NVLink (plain stores on peer
 * pointers, then one system-scope add on the row's arrival counter there), and the merge
 * kernel waits -- bounded -- until all ranks have counted themselves in for a row before it
 * reads its own window.  Two launches per call and no collective kernel; results are
 * identical.  The windows are mapped with CUDA IPC on first use (all ranks on one machine),
 * and the first call and any call with more rows than before is collective.  A rank that
 * never stores its blocks fails the rows with FG_ERR_LIMIT after about two seconds and the
 * communicator is closed, as above. */
fg_status fg_dist_sample_vocab_sharded_fused(fg_dist *dist, const fg_cuda_sample_args *args,
                                             uint32_t vocab_total, uint32_t k_shard, fg_error *err);

/* Row partition, optional: all ranks' results on every rank.  Every rank passes `rows`
 * results (device arrays; the same count on every rank) and gets ranks * rows back in
 * rank order.  Waits for completion. */
fg_status fg_dist_gather_rows(fg_dist *dist, const uint32_t *tokens, const float *token_logits,
                              const uint32_t *row_status, uint32_t rows, uint32_t *all_tokens,
                              float *all_token_logits, uint32_t *all_row_status, fg_error *err);

/* No counterpart in the reference.  fg_cuda_sample_batch for callers that must not
 * allocate GPU memory: a serving process whose own arena already owns the whole
 * device (so cudaMalloc fails, or may not be called by policy), or a decode loop
 * that cannot afford the device-wide stall an allocation can cause.  It needs no
 * fg_cuda_context and calls neither cudaMalloc/cudaFree nor any allocating
 * library routine: the kernel's scratch (arrival counters, per-row configs, the
 * hand-off between the CTAs that share a row) lives in a 4 MiB array compiled
 * into the library, which every GPU that loads the library holds until exit.
 *   - `device` and `cuda_stream` (a cudaStream_t, NULL = default stream) say where
 *     to run; inputs and outputs are the caller's device buffers as in
 *     fg_cuda_sample_batch (args->debug allowed, top_k == 0 rows not supported).
 *   - Always asynchronous: it returns once the work is enqueued; per-row results
 *     are in args->row_status after the caller synchronises the stream.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device made current); make that first
 *     call before starting any stream capture.  With per-row configs
 *     (config_count > 1) every call copies the caller's host array to the
 *     device, so a captured graph would replay that copy from the same host
 *     address: pass one config when capturing.
 *   - Limit: 256 + 4*rows (+ 40*rows with per-row configs) + 528*rows*splits
 *     bytes must fit 4 MiB; the split count is lowered to make it fit and
 *     FG_ERR_LIMIT names the sizes when even one CTA per row does not
 *     (about 95,000 rows).
 *   - All calls share the one array.  It keeps the previous call's contents (what
 *     must start at zero is cleared on the stream by each call), and two calls
 *     whose kernels overlap on the GPU — different streams, or different host
 *     threads — race on it: issue them one after another on one stream. */
fg_status fg_cuda_sample_batch_static(int device, void *cuda_stream,
                                      const fg_cuda_sample_args *args, fg_error *err);

/* Bytes of context scratch the last fg_cuda_sample_batch / shard_topk used
 * (reports and tests). */
uint64_t fg_cuda_context_scratch_bytes(const fg_cuda_context *context);

#ifdef __cplusplus
}
#endif

#endif /* FG_B200_CUDA_SAMPLER_H */
