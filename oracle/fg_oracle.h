/*
 * TEST INFRASTRUCTURE — interface of the CPU oracle for the token-sampling
 * path.  Nothing in the product library includes or links this.
 *
 * Two shared objects are built from the same pipeline source:
 *   oracle/libfgoracle.so     pipeline + this repository's restatement of the
 *                             reference's host sampler ("port")
 *   oracle/_ref/libfgref.so   pipeline + the reference's own objects, compiled
 *                             where they lie in the reference tree ("reference")
 * fgo_kind() tells which one a handle is.
 */
#ifndef FG_ORACLE_H
#define FG_ORACLE_H

#include "fg_sampler.h"

#ifdef __cplusplus
extern "C" {
#endif

#define FGO_PADDING_ID 0xffffffffu
#define FGO_DTYPE_F32 0u
#define FGO_DTYPE_BF16 1u

/* "port" or "reference". */
const char *fgo_kind(void);

/* src/output.c:484-498 (defined by the port or by the reference object). */
bool fg_output_better(float left, uint32_t left_id, float right, uint32_t right_id);
void fg_output_combine(float left, uint32_t left_id, float right, uint32_t right_id,
                       float *value, uint32_t *id);

/* src/output.c:601-617. */
fg_status fgo_history_counts(uint32_t *counts, uint32_t vocab, const uint32_t *history,
                             uint32_t count, fg_error *err);
/* shaders/fg_apply_penalties.comp:12-19 with the shader's own association
 * (value - frequency*count) - presence.  Informative only: parity is defined
 * by fg_sampler_apply_penalties. */
void fgo_apply_penalties_shader(float *logits, const uint32_t *counts, uint32_t values,
                                float presence, float frequency, float repetition);
/* shaders/fg_argmax_reduce.comp:26-57; ids == NULL means 0..count-1.  Returns groups. */
uint32_t fgo_argmax_reduce(float *out_scores, uint32_t *out_ids, const float *scores,
                           const uint32_t *ids, uint32_t count);
/* shaders/fg_topk_select_fallback.comp:22-43; ids == NULL means 0..count-1.
 * Returns ceil(count/1024)*k. */
/* shaders/fg_topk_reduce_v2.comp + src/vk.c:2235: sorted top-512 of every 4096-element tile */
uint32_t fgo_topk_reduce(float *out_scores, uint32_t *out_ids, const float *scores,
                         const uint32_t *ids, uint32_t count);
/* src/q38_math.c:48-64 restated */
fg_status fgo_router_topk(const float *logits, uint32_t count, uint32_t k, uint32_t *ids, float *weights);
uint32_t fgo_topk_select(float *out_scores, uint32_t *out_ids, const float *scores,
                         const uint32_t *ids, uint32_t count, uint32_t k);

/* Candidate list handed to the select step, in sampling order, with the
 * probabilities it used (zero beyond the respective cut). */
typedef struct fgo_candidates {
    uint32_t count;
    uint32_t ids[64];
    float scores[64];
    double raw_probability[64];
    double tempered_probability[64];
    /* rows without a top-k cut only: how many candidates the nucleus kept, and the smallest
     * distance (in units of the total mass) of top_p and of the draw from an edge of the
     * cumulative distribution -- a result can depend on the summation order only when this
     * is within rounding of zero */
    uint32_t nucleus;
    double edge_margin;
} fgo_candidates;

/* The reference's select generalised to any candidate count and to
 * top_k == 0 ("no top-k cut"); identical to fg_sampler_select on its domain
 * (count <= 64, 1 <= top_k <= 64).  `margin`, when given, receives the
 * smallest relative distance between the draw and a CDF edge. */
fg_status fgo_select_general(const fg_sampler_config *config, bool allow_no_topk,
                             const float *scores, const uint32_t *ids, uint32_t count,
                             float uniform, uint32_t *token, float *logit,
                             uint32_t *nucleus, double *margin, fg_error *err);

/* One row through the whole path of src/output.c:702-755 (logits already
 * computed): history -> counts, penalties, then greedy cascade or top-k
 * cascade + select.  `logits` has `vocab` fp32 values and is overwritten with
 * the penalised values.  scratch must hold 6*vocab + 512 uint32 words. */
fg_status fgo_sample_row(float *logits, uint32_t vocab, const uint32_t *history,
                         uint32_t history_count, const fg_sampler_config *config,
                         bool allow_no_topk, float uniform, uint32_t *token, float *logit,
                         fgo_candidates *candidates, uint32_t *scratch, fg_error *err);

/* Rows in parallel over `threads` host threads.  Returns the status of the
 * lowest failing row. */
fg_status fgo_sample_batch(const void *logits, uint32_t dtype, uint32_t rows, uint32_t vocab,
                           uint64_t row_stride, const uint32_t *history_tokens,
                           const uint64_t *history_offsets, const fg_sampler_config *configs,
                           uint32_t config_count, bool allow_no_topk, const float *uniforms,
                           uint32_t *tokens, float *token_logits, uint32_t *row_status,
                           fgo_candidates *candidates, uint32_t threads);

/* Vocabulary-sharded path: per-shard penalties + top-k_shard with global ids,
 * then range check (src/runtime.c:2437-2466), merge and select. */
fg_status fgo_shard_topk(const void *logits, uint32_t dtype, uint32_t rows, uint32_t shard_vocab,
                         uint64_t row_stride, uint32_t vocab_offset, uint32_t vocab_total,
                         const uint32_t *history_tokens, const uint64_t *history_offsets,
                         const fg_sampler_config *configs, uint32_t config_count,
                         uint32_t k_shard, float *candidate_scores, uint32_t *candidate_ids,
                         uint32_t *row_status);
fg_status fgo_merge_select(const float *candidate_scores, const uint32_t *candidate_ids,
                           uint32_t shards, uint32_t rows, uint32_t k_shard,
                           const uint32_t *shard_first, const uint32_t *shard_width,
                           const fg_sampler_config *configs, uint32_t config_count,
                           const float *uniforms, uint32_t *tokens, float *token_logits,
                           uint32_t *row_status, fgo_candidates *candidates);

#ifdef __cplusplus
}
#endif

#endif
