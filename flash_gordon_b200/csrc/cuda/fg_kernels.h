/*
 * Internal seam between the C17 host layer (csrc/host) and the CUDA
 * translation units (csrc/cuda).  Plain C types only.  Every fgk_* function
 * returns a cudaError_t value as int (0 = success) unless stated otherwise;
 * the host layer turns it into fg_status and a message.  Not installed, not
 * part of the public ABI.
 */
#ifndef FG_B200_KERNELS_H
#define FG_B200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#include "fg_sampler.h"

#ifdef __cplusplus
extern "C" {
#endif

/* dynamic shared memory a streaming CTA may ask for (static part comes on top) */
#define FGK_STREAM_MAX_DYNAMIC_SMEM (200 * 1024)

/* ---- runtime plumbing (fg_runtime.cu) ---- */
int fgk_device_count(int *count);
int fgk_set_device(int device);
int fgk_device_sm_count(int device, int *sm_count);
int fgk_stream_create(void **stream);
int fgk_stream_destroy(void *stream);
int fgk_stream_synchronize(void *stream);
int fgk_malloc(void **pointer, size_t bytes);
int fgk_free(void *pointer);
int fgk_host_alloc(void **pointer, size_t bytes); /* pinned */
int fgk_host_free(void *pointer);
int fgk_memset_async(void *pointer, int value, size_t bytes, void *stream);
int fgk_copy_to_device_async(void *device, const void *host, size_t bytes, void *stream);
int fgk_copy_to_host_async(void *host, const void *device, size_t bytes, void *stream);
const char *fgk_error_string(int cuda_error);

/* ---- outputs shared by the sampling launches ---- */
typedef struct fgk_select_output {
    uint32_t *tokens;
    float *token_logits;
    uint32_t *row_status;
    uint64_t *first_error; /* device word: min over failing rows of (row << 8 | status) */
    uint32_t *dbg_count;
    uint32_t *dbg_ids;
    float *dbg_scores;
    double *dbg_raw;
    double *dbg_tempered;
} fgk_select_output;

/* ---- the fused exchange of the vocabulary-sharded mode ----
 * Instead of leaving its candidates in local memory for an all-gather, a shard kernel stores
 * its block of every row -- shard_k (value, id) pairs -- straight into the window of every
 * rank (its own included) over NVLink, then adds one to that row's arrival counter there.
 * A window is laid out  pairs[2][ranks][pair_capacity]  then  arrived[2][row_capacity]
 * (two halves, used by alternate calls); the merge kernel of a rank reads only its own
 * window, after the row's counter says that every rank's block has landed.  Plain stores
 * and system-scope atomics on peer pointers: no multicast, no TMA. */
typedef struct fgk_push {
    void *window[16];        /* every rank's window as mapped into this process; NULL when off */
    uint32_t ranks, rank;
    uint32_t half;           /* which half of the windows this call uses */
    uint32_t pair_capacity;  /* pairs per (half, rank) */
    uint32_t row_capacity;
} fgk_push;

/* ---- streaming select (fg_stream_kernels.cu) ---- */
typedef struct fgk_stream_launch {
    const void *logits;
    uint32_t dtype; /* 0 fp32, 1 bf16 */
    uint32_t rows, vocab;
    uint64_t row_stride;
    uint32_t vocab_offset, vocab_total;
    uint32_t splits, split_len;
    const uint32_t *history_tokens;
    const uint64_t *history_offsets;
    uint32_t history_max;
    const void *configs_device; /* rows x 40 bytes when config_count > 1 */
    fg_sampler_config config0;
    uint32_t config_count;
    uint32_t shard_k;
    const float *uniforms;
    float *shard_scores;
    uint32_t *shard_ids;
    uint32_t shard_stride; /* elements between consecutive candidates: 0 or 1 separate arrays, 2 (value, id) pairs */
    fgk_push push;         /* ranks != 0: the shard's candidates go to the ranks' windows instead */
    float *part_scores;
    uint32_t *part_ids;
    void *part_meta;
    uint32_t *tickets;
    uint32_t bitmap_words;
    uint32_t count_capacity;
    uint32_t dense_wide;
    /* history pass only: global home of the per-(row, split) history structures */
    uint32_t *history_global;
    uint64_t history_stride_words;
    void *history_meta; /* 8 bytes per (row, split); NULL when the batch has no history */
    /* persistent kernel only: session tables in place of token lists (the stateful executor):
     * counts [slots][vocab] and seen-bitmaps [slots][slot_bitmap_words], row r uses session
     * row_slots[r]; all three NULL otherwise */
    const uint32_t *slot_counts;
    const uint32_t *slot_bitmaps;
    const uint32_t *row_slots;
    uint32_t slot_bitmap_words;
    /* persistent kernel only: polls before a device-side wait gives up (0 = the default, about
     * two seconds), and the test seam that makes one wait run out: warp 0 of CTA withhold_cta
     * never asks the copy engine for its withhold_issue-th tile */
    uint32_t wait_polls;
    uint32_t withhold_armed, withhold_cta, withhold_issue;
    fgk_select_output out;
} fgk_stream_launch;

uint32_t fgk_stream_max_splits(void);
uint32_t fgk_stream_tile(void);
uint64_t fgk_stream_part_meta_bytes(void);
uint64_t fgk_stream_dynamic_smem(uint32_t bitmap_words, uint32_t count_capacity, uint32_t dense_wide);
int fgk_stream_prepare(void);
int fgk_launch_stream_select(const fgk_stream_launch *launch, void *stream);

/* ---- persistent ring kernel (fg_persistent_kernel.cu) ----
 * Takes a fgk_stream_launch with rows and row stride multiples of 16 bytes and only rows
 * whose penalties cannot raise a logit.  Work is dealt out in 4 KB tiles: `split_len`
 * holds the tiles per CTA (0: whole rows, dealt round-robin), `splits` the most CTAs that
 * can share one row; part_* and tickets as for the streaming kernel.  Of the history
 * fields it uses bitmap_words alone (the bitmaps live in dynamic shared memory). */
/* dynamic shared memory for that bitmap size and how many bitmap buffers fit (2 or 1);
 * 0 when the kernel cannot take the vocabulary */
uint64_t fgk_persistent_dynamic_smem(uint32_t bitmap_words, uint32_t *bitmap_buffers);
uint32_t fgk_persistent_row_tiles(uint32_t dtype, uint32_t vocab);
uint32_t fgk_persistent_tiles_abreast(void);
/* most parts of one row the merge takes when each hands over up to k survivors */
uint32_t fgk_persistent_max_parts(uint32_t k);
int fgk_persistent_prepare(void);
int fgk_launch_persistent_select(const fgk_stream_launch *launch, uint32_t ctas, void *stream);

typedef struct fgk_merge_launch {
    const float *scores;
    const uint32_t *ids;
    uint32_t rows, shards, k_shard;
    uint32_t stride; /* elements between consecutive candidates: 0 or 1 separate arrays, 2 (value, id) pairs */
    uint64_t shard_pitch; /* candidates between consecutive shards' blocks (0: rows * k_shard) */
    /* fused exchange: row r may be read once arrived[r] >= arrival_target (NULL: at once), and
     * the kernel then sets the counter back to zero; the wait gives up after wait_polls polls
     * (0: about two seconds) and fails the row */
    uint32_t *arrived;
    uint32_t arrival_target;
    uint32_t wait_polls;
    uint32_t check_spans;
    uint32_t span_first[16], span_width[16];
    const void *configs_device;
    fg_sampler_config config0;
    uint32_t config_count;
    const float *uniforms;
    fgk_select_output out;
} fgk_merge_launch;

int fgk_launch_merge_select(const fgk_merge_launch *launch, void *stream);

/* scratch compiled into the library image (no allocation); address valid on `device`,
 * which must be current on the first call for that device */
#define FGK_STATIC_SCRATCH_BYTES (4u << 20)
int fgk_static_scratch_address(int device, void **address);

/* ---- sampling without a top-k cut (fg_nucleus_kernel.cu) ---- */
typedef struct fgk_nucleus_launch {
    const void *logits;
    uint32_t dtype;
    uint32_t rows, vocab;
    uint64_t row_stride;
    const void *configs_device;
    fg_sampler_config config0;
    uint32_t config_count;
    const float *uniforms;
    float *scratch;          /* ctas rows of scratch_stride floats */
    uint64_t scratch_stride;
    uint32_t ctas;           /* persistent CTAs, one scratch row each */
    const uint32_t *history_global;
    uint64_t history_stride_words;
    const void *history_meta;
    uint32_t splits, split_len, bitmap_words, count_capacity, dense_wide;
    fgk_select_output out;
} fgk_nucleus_launch;

int fgk_nucleus_prepare(void);
int fgk_launch_nucleus_select(const fgk_nucleus_launch *launch, void *stream);
/* the history pass (fills history_global / history_meta) */
int fgk_launch_history_build(const fgk_stream_launch *launch, void *stream);

/* ---- NCCL behind plain C (fg_nccl.cu); libnccl.so.2 is opened on first use ---- */
#define FGK_NCCL_ID_BYTES 128
#define FGK_NCCL_MISSING (-1) /* the library or one of its symbols could not be loaded */
#define FGK_NCCL_TIMEOUT (-2) /* a deadline passed while waiting for other ranks */
#define FGK_NCCL_FAILED  (-3) /* NCCL reported an error */
int fgk_nccl_load(void);
int fgk_nccl_version(void); /* 0 when NCCL cannot be loaded */
int fgk_nccl_unique_id(void *id128);
int fgk_nccl_create(void **comm, uint32_t ranks, uint32_t rank, const void *id128, uint32_t timeout_ms);
int fgk_nccl_all_gather(void *comm, const void *send, void *receive, size_t bytes_per_rank, void *stream,
                        uint32_t timeout_ms);
void fgk_nccl_abort(void *comm);
void fgk_nccl_destroy(void *comm);
/* cudaStreamSynchronize with a deadline: 0, a cudaError_t, or FGK_NCCL_TIMEOUT */
int fgk_stream_wait_deadline(void *stream, uint32_t timeout_ms);
/* device memory of another process on this machine (CUDA IPC): 64-byte handles */
#define FGK_IPC_HANDLE_BYTES 64
int fgk_ipc_handle(void *device_pointer, void *handle64);
int fgk_ipc_open(const void *handle64, void **device_pointer);
int fgk_ipc_close(void *device_pointer);

/* ---- device operators (fg_ops_kernels.cu) ---- */
int fgk_launch_apply_penalties(float *logits, const uint32_t *counts, uint32_t values,
                               float presence, float frequency, float repetition, void *stream);
/* scores[i] penalised with seen[i] (already gathered), for fg_sampler_apply_penalties */
int fgk_launch_apply_penalties_seen(float *scores, const uint32_t *seen, uint32_t values,
                                    float presence, float frequency, float repetition,
                                    void *stream);
int fgk_launch_argmax_reduce(float *out_scores, uint32_t *out_ids, const float *scores,
                             const uint32_t *ids, uint32_t count, void *stream);
int fgk_launch_topk_select(float *out_scores, uint32_t *out_ids, const float *scores,
                           const uint32_t *ids, uint32_t count, uint32_t k, void *stream);
/* the best 512 of every 4096-element tile, sorted; writes the first `produced` outputs */
int fgk_launch_topk_reduce(float *out_scores, uint32_t *out_ids, const float *scores, const uint32_t *ids,
                           uint32_t count, uint32_t produced, void *stream);
/* per token the k best of `experts` logits and their gate weights; *bad (device word, armed
 * with 0xffffffff) gets the lowest token whose logits hold a NaN or +Inf */
int fgk_launch_router_topk(uint32_t *out_ids, float *out_weights, const float *logits, uint32_t tokens,
                           uint32_t experts, uint32_t k, uint32_t *bad, void *stream);
/* The executor's tables after a step: for every row that ended FG_OK and whose penalties are
 * active, the sampled token's count goes up by one (saturating) and its seen-bit is set in
 * the row's session (src/output.c:619-628, 742, 752).  `active` holds one byte per row. */
int fgk_launch_session_increment(uint32_t *slot_counts, uint32_t *slot_bitmaps, uint32_t vocab,
                                 uint32_t slot_bitmap_words, const uint32_t *row_slots,
                                 const uint32_t *tokens, const uint32_t *row_status,
                                 const unsigned char *active, uint32_t rows, void *stream);
/* one session's bitmap rebuilt from its count table */
int fgk_launch_session_bitmap(uint32_t *bitmap, const uint32_t *counts, uint32_t vocab,
                              uint32_t bitmap_words, void *stream);
/* counts += occurrences of history[0..count); *bad (device word) set when an id >= vocab */
int fgk_launch_history_add(uint32_t *counts, uint32_t vocab, const uint32_t *history,
                           uint32_t count, uint32_t *bad, void *stream);

#ifdef __cplusplus
}
#endif

#endif
