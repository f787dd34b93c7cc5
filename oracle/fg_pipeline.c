/*
 * TEST INFRASTRUCTURE — CPU oracle for the token-sampling path.
 *
 * Checker for the CUDA kernels and the timed CPU baseline; never part of the
 * product library.  It restates in C the arithmetic of the three Vulkan
 * shaders that have no CPU twin in the reference and strings them together the
 * way the reference's output executor does.  The host sampler functions it
 * calls (fg_sampler_apply_penalties, fg_sampler_select, fg_output_better) come
 * from whichever objects this file is linked with: this repository's port
 * (libfgoracle.so) or the reference's own sources (oracle/_ref/libfgref.so).
 *
 * Beyond the reference's domain (batches, bf16 rows, top_k == 0, candidate
 * sets larger than 64, vocabulary shards) the functions here are this
 * repository's documented generalisation; reference tests do not pin them.
 */
#include "fg_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#ifndef FGO_KIND
#define FGO_KIND "port"
#endif

const char *fgo_kind(void) { return FGO_KIND; }

/* ------------------------------------------------ history (output.c:601-617) */

fg_status fgo_history_counts(uint32_t *counts, uint32_t vocab, const uint32_t *history,
                             uint32_t count, fg_error *err) {
    if (counts == NULL || count > FG_NATIVE_CONTEXT || (count != 0u && history == NULL)) {
        fg_error_set(err, FG_ERR_ARGUMENT, "invalid output history");
        return FG_ERR_ARGUMENT;
    }
    memset(counts, 0, (size_t)vocab * sizeof *counts);
    for (uint32_t i = 0; i < count; i++) {
        const uint32_t token = history[i];
        if (token >= vocab) {
            fg_error_set(err, FG_ERR_FORMAT, "history token %u is outside vocabulary", i);
            return FG_ERR_FORMAT;
        }
        if (counts[token] != UINT32_MAX) counts[token]++;
    }
    return FG_OK;
}

/* ------------------------- fg_apply_penalties.comp:12-19, shader association */

void fgo_apply_penalties_shader(float *logits, const uint32_t *counts, uint32_t values,
                                float presence, float frequency, float repetition) {
    for (uint32_t id = 0; id < values; id++) {
        if (counts[id] == 0u) continue;
        volatile float value = logits[id];
        if (repetition != 1.0f) value = value > 0.0f ? value / repetition : value * repetition;
        volatile float scaled = frequency * (float)counts[id];
        volatile float partial = value - scaled;
        logits[id] = partial - presence;
    }
}

/* ------------------------------------------ fg_argmax_reduce.comp:26-57 */

uint32_t fgo_argmax_reduce(float *out_scores, uint32_t *out_ids, const float *scores,
                           const uint32_t *ids, uint32_t count) {
    const uint32_t tile = 4096u;
    const uint32_t groups = (count + tile - 1u) / tile;
    for (uint32_t g = 0; g < groups; g++) {
        const uint32_t begin = g * tile;
        const uint32_t end = count - begin < tile ? count : begin + tile;
        /* The shader starts every lane at (-inf, padding) and folds with
         * before(); before() is a strict total order, so lane striding and the
         * tree do not change the winner and a linear fold restates it. */
        float best = -INFINITY;
        uint32_t best_id = FGO_PADDING_ID;
        for (uint32_t i = begin; i < end; i++) {
            const uint32_t id = ids ? ids[i] : i;
            if (fg_output_better(scores[i], id, best, best_id)) {
                best = scores[i];
                best_id = id;
            }
        }
        out_scores[g] = best;
        out_ids[g] = best_id;
    }
    return groups;
}

/* ------------------------------- fg_topk_select_fallback.comp:14-43 */

/* The shader's before(): padding loses, a non-finite left operand never wins,
 * otherwise larger score, then smaller id. */
static bool topk_before(float a, uint32_t a_id, float b, uint32_t b_id) {
    const bool a_pad = a_id == FGO_PADDING_ID, b_pad = b_id == FGO_PADDING_ID;
    if (a_pad || b_pad) return !a_pad && b_pad;
    if (!isfinite(a)) return false;
    if (!isfinite(b)) return true;
    return a > b || (a == b && a_id < b_id);
}

uint32_t fgo_topk_select(float *out_scores, uint32_t *out_ids, const float *scores,
                         const uint32_t *ids, uint32_t count, uint32_t k) {
    const uint32_t tile = 1024u;
    const uint32_t groups = (count + tile - 1u) / tile;
    for (uint32_t g = 0; g < groups; g++) {
        const uint32_t begin = g * tile;
        const uint32_t end = count - begin < tile ? count : begin + tile;
        float *top = out_scores + (size_t)g * k;
        uint32_t *top_id = out_ids + (size_t)g * k;
        /* The shader runs k rounds of "best not yet taken".  Keeping the k best
         * seen so far in rank order yields the same k entries in the same
         * order, because topk_before is a strict total order on valid entries. */
        for (uint32_t r = 0; r < k; r++) {
            top[r] = -INFINITY;
            top_id[r] = FGO_PADDING_ID;
        }
        for (uint32_t i = begin; i < end; i++) {
            const float value = scores[i];
            if (!isfinite(value)) continue; /* stored as (-inf, padding) by the shader */
            const uint32_t id = ids ? ids[i] : i;
            if (id == FGO_PADDING_ID) continue;
            if (!topk_before(value, id, top[k - 1u], top_id[k - 1u])) continue;
            uint32_t slot = k - 1u;
            while (slot > 0u && topk_before(value, id, top[slot - 1u], top_id[slot - 1u])) {
                top[slot] = top[slot - 1u];
                top_id[slot] = top_id[slot - 1u];
                slot--;
            }
            top[slot] = value;
            top_id[slot] = id;
        }
    }
    return groups * k;
}

/* shaders/fg_topk_reduce_v2.comp:10: the order of the sorted top-512 kernel.  Unlike the
 * generation selector above, a NaN/Inf comes BEFORE every finite score here. */
static bool reduce_before(float a, uint32_t a_id, float b, uint32_t b_id) {
    const bool a_pad = a_id == FGO_PADDING_ID, b_pad = b_id == FGO_PADDING_ID;
    if (a_pad || b_pad) return !a_pad && b_pad;
    const bool a_wild = !isfinite(a), b_wild = !isfinite(b);
    if (a_wild || b_wild) return a_wild != b_wild ? a_wild : a_id < b_id;
    return a > b || (a == b && a_id < b_id);
}

/* shaders/fg_topk_reduce_v2.comp:27-85 + src/vk.c:2235: the best 512 of every 4096-element
 * tile, sorted; a short tile is padded with (-inf, padding id); a lone tile with fewer
 * than 512 entries hands back just those.  (The shader sorts 64-slot runs and merges them;
 * an insertion into a sorted prefix gives the same sequence, the order being total.) */
uint32_t fgo_topk_reduce(float *out_scores, uint32_t *out_ids, const float *scores,
                         const uint32_t *ids, uint32_t count) {
    const uint32_t tile = 4096u, keep = 512u;
    const uint32_t groups = (count + tile - 1u) / tile;
    uint32_t produced = groups * keep;
    if (groups == 1u && count < keep) produced = count;
    for (uint32_t g = 0; g < groups; g++) {
        const uint32_t begin = g * tile;
        const uint32_t here = count - begin < tile ? count - begin : tile;
        float top[512];
        uint32_t top_id[512];
        uint32_t held = 0;
        for (uint32_t i = 0; i < here; i++) {
            const float value = scores[begin + i];
            const uint32_t id = ids ? ids[begin + i] : begin + i;
            if (held == keep && !reduce_before(value, id, top[keep - 1u], top_id[keep - 1u])) continue;
            uint32_t slot = held < keep ? held++ : keep - 1u;
            while (slot > 0u && reduce_before(value, id, top[slot - 1u], top_id[slot - 1u])) {
                top[slot] = top[slot - 1u];
                top_id[slot] = top_id[slot - 1u];
                slot--;
            }
            top[slot] = value;
            top_id[slot] = id;
        }
        for (uint32_t i = 0; i < keep; i++) {
            const size_t at = (size_t)g * keep + i;
            if (at >= produced) break;
            out_scores[at] = i < held ? top[i] : -INFINITY;
            out_ids[at] = i < held ? top_id[i] : FGO_PADDING_ID;
        }
    }
    return produced;
}

/* src/q38_math.c:48-64 (fg_q38_router_topk), restated: softmax over all experts in fp64,
 * the k largest logits (ties: smaller id), their probabilities rounded to fp32 and
 * renormalised by their fp64 sum. */
fg_status fgo_router_topk(const float *logits, uint32_t count, uint32_t k, uint32_t *ids, float *weights) {
    if (!logits || !ids || !weights || count == 0u || k == 0u || k > count) return FG_ERR_ARGUMENT;
    float top = -INFINITY;
    for (uint32_t i = 0; i < count; i++)
        if (logits[i] > top) top = logits[i];
    double total = 0.0;
    for (uint32_t i = 0; i < count; i++) total += exp((double)logits[i] - top);
    double picked = 0.0;
    for (uint32_t slot = 0; slot < k; slot++) {
        uint32_t best = UINT32_MAX;
        float best_value = -INFINITY;
        for (uint32_t i = 0; i < count; i++) {
            bool taken = false;
            for (uint32_t j = 0; j < slot && !taken; j++) taken = ids[j] == i;
            if (!taken && (logits[i] > best_value || (logits[i] == best_value && i < best))) {
                best = i;
                best_value = logits[i];
            }
        }
        ids[slot] = best;
        weights[slot] = (float)(exp((double)best_value - top) / total);
        picked += weights[slot];
    }
    if (!(picked > 0.0)) return FG_ERR_FORMAT;
    for (uint32_t slot = 0; slot < k; slot++) weights[slot] = (float)(weights[slot] / picked);
    return FG_OK;
}

/* ------------------------------------------------- generalised select (A.5) */

typedef struct ranked {
    float score;
    uint32_t id;
    uint32_t position;
} ranked;

static int ranked_compare(const void *pa, const void *pb) {
    const ranked *a = pa, *b = pb;
    if (a->score != b->score) return a->score > b->score ? -1 : 1;
    if (a->id != b->id) return a->id < b->id ? -1 : 1;
    /* equal score and id: the reference's insertion sort keeps arrival order */
    return a->position < b->position ? -1 : (a->position > b->position ? 1 : 0);
}

static double relative_gap(double a, double b, double scale) {
    const double gap = fabs(a - b);
    return scale > 0.0 ? gap / scale : gap;
}

fg_status fgo_select_general(const fg_sampler_config *config, bool allow_no_topk,
                             const float *scores, const uint32_t *ids, uint32_t count,
                             float uniform, uint32_t *token, float *logit,
                             uint32_t *nucleus, double *margin, fg_error *err) {
    fg_sampler_config checked;
    bool config_ok = config != NULL;
    if (config_ok) {
        checked = *config;
        if (allow_no_topk && checked.top_k == 0u) checked.top_k = 1u;
        config_ok = fg_sampler_config_validate(&checked, err) == FG_OK;
    }
    if (!config_ok || scores == NULL || ids == NULL || count == 0u || token == NULL ||
        logit == NULL) {
        if (err != NULL && err->message[0] == '\0')
            fg_error_set(err, FG_ERR_ARGUMENT, "invalid sampler candidates");
        return err != NULL && err->code != FG_OK ? err->code : FG_ERR_ARGUMENT;
    }
    ranked *order = malloc((size_t)count * sizeof *order);
    if (order == NULL) {
        fg_error_set(err, FG_ERR_OOM, "oracle select out of memory");
        return FG_ERR_OOM;
    }
    uint32_t kept = 0;
    for (uint32_t i = 0; i < count; i++) {
        if (!isfinite(scores[i])) continue;
        order[kept].score = scores[i];
        order[kept].id = ids[i];
        order[kept].position = i;
        kept++;
    }
    fg_status status = FG_OK;
    double least = INFINITY;
    if (kept == 0u) {
        fg_error_set(err, FG_ERR_FORMAT, "sampler received no finite candidates");
        status = FG_ERR_FORMAT;
        goto done;
    }
    qsort(order, kept, sizeof *order, ranked_compare);
    if (config->temperature == 0.0f) {
        *token = order[0].id;
        *logit = order[0].score;
        if (nucleus) *nucleus = 1u;
        goto done;
    }
    {
        const uint32_t limit =
            (config->top_k != 0u && config->top_k < kept) ? config->top_k : kept;
        const double top_raw = order[0].score;
        double raw_sum = 0.0;
        for (uint32_t r = 0; r < limit; r++) raw_sum += exp((double)order[r].score - top_raw);
        if (!(raw_sum > 0.0) || !isfinite(raw_sum)) {
            fg_error_set(err, FG_ERR_FORMAT, "sampler raw softmax failed");
            status = FG_ERR_FORMAT;
            goto done;
        }
        uint32_t survivors = limit;
        double mass = 0.0, before_cross = 0.0;
        for (uint32_t r = 0; r < limit; r++) {
            before_cross = mass;
            mass += exp((double)order[r].score - top_raw) / raw_sum;
            if (mass >= config->top_p) {
                survivors = r + 1u;
                break;
            }
        }
        if (survivors < limit || mass >= config->top_p) {
            least = fmin(least, relative_gap(mass, config->top_p, 1.0));
            least = fmin(least, relative_gap(before_cross, config->top_p, 1.0));
        }
        const double temperature = (double)config->temperature;
        const double top_tempered = (double)order[0].score / temperature;
        double weight_sum = 0.0;
        for (uint32_t r = 0; r < survivors; r++)
            weight_sum += exp((double)order[r].score / temperature - top_tempered);
        if (!(weight_sum > 0.0) || !isfinite(weight_sum)) {
            fg_error_set(err, FG_ERR_FORMAT, "sampler temperature softmax failed");
            status = FG_ERR_FORMAT;
            goto done;
        }
        if (!isfinite(uniform) || uniform < 0.0f) uniform = 0.0f;
        if (uniform >= 1.0f) uniform = nextafterf(1.0f, 0.0f);
        const double draw = (double)uniform * weight_sum;
        uint32_t pick = survivors - 1u;
        double walked = 0.0, previous = 0.0;
        for (uint32_t r = 0; r < survivors; r++) {
            previous = walked;
            walked += exp((double)order[r].score / temperature - top_tempered);
            if (draw < walked) {
                pick = r;
                break;
            }
        }
        least = fmin(least, relative_gap(walked, draw, weight_sum));
        if (pick > 0u) least = fmin(least, relative_gap(previous, draw, weight_sum));
        *token = order[pick].id;
        *logit = order[pick].score;
        if (nucleus) *nucleus = survivors;
    }
done:
    if (margin) *margin = least;
    free(order);
    return status;
}

/* Fill the candidate report for a list that is already the top-k set. */
static void report_candidates(fgo_candidates *out, const fg_sampler_config *config,
                              const float *scores, const uint32_t *ids, uint32_t count) {
    memset(out, 0, sizeof *out);
    ranked order[64];
    uint32_t kept = 0;
    for (uint32_t i = 0; i < count && i < 64u; i++) {
        if (!isfinite(scores[i])) continue;
        order[kept].score = scores[i];
        order[kept].id = ids[i];
        order[kept].position = i;
        kept++;
    }
    qsort(order, kept, sizeof order[0], ranked_compare);
    uint32_t limit = kept;
    if (config->temperature != 0.0f && config->top_k != 0u && config->top_k < limit)
        limit = config->top_k;
    if (config->temperature == 0.0f && limit > 1u) limit = 1u;
    out->count = limit;
    for (uint32_t r = 0; r < limit; r++) {
        out->ids[r] = order[r].id;
        out->scores[r] = order[r].score;
    }
    if (limit == 0u || config->temperature == 0.0f) return;
    const double top_raw = order[0].score;
    double raw_sum = 0.0;
    for (uint32_t r = 0; r < limit; r++) raw_sum += exp((double)order[r].score - top_raw);
    uint32_t survivors = limit;
    double mass = 0.0;
    for (uint32_t r = 0; r < limit; r++) {
        const double p = exp((double)order[r].score - top_raw) / raw_sum;
        out->raw_probability[r] = p;
        mass += p;
        if (survivors == limit && mass >= config->top_p) survivors = r + 1u;
    }
    const double temperature = (double)config->temperature;
    const double top_tempered = (double)order[0].score / temperature;
    double weight_sum = 0.0;
    for (uint32_t r = 0; r < survivors; r++)
        weight_sum += exp((double)order[r].score / temperature - top_tempered);
    for (uint32_t r = 0; r < survivors; r++)
        out->tempered_probability[r] =
            exp((double)order[r].score / temperature - top_tempered) / weight_sum;
}

/* ------------------------------------- one row (output.c:560-567, 702-755) */

fg_status fgo_sample_row(float *logits, uint32_t vocab, const uint32_t *history,
                         uint32_t history_count, const fg_sampler_config *config,
                         bool allow_no_topk, float uniform, uint32_t *token, float *logit,
                         fgo_candidates *candidates, uint32_t *scratch, fg_error *err) {
    fg_sampler_config checked = *config;
    if (allow_no_topk && checked.top_k == 0u) checked.top_k = 1u;
    fg_status status = fg_sampler_config_validate(&checked, err);
    if (status != FG_OK) return status;
    if (candidates) memset(candidates, 0, sizeof *candidates);

    /* scratch: counts[V] iota[V] ids[2][V+128] scores[2][V+128] */
    const size_t lane = (size_t)vocab + 128u;
    uint32_t *counts = scratch;
    uint32_t *iota = scratch + vocab;
    uint32_t *ping_ids[2] = {scratch + 2u * (size_t)vocab, scratch + 2u * (size_t)vocab + lane};
    float *ping_scores[2] = {(float *)(scratch + 2u * (size_t)vocab + 2u * lane),
                             (float *)(scratch + 2u * (size_t)vocab + 3u * lane)};

    const bool penalties = fg_sampler_penalties_active(config);
    for (uint32_t i = 0; i < vocab; i++) iota[i] = i;
    if (penalties) {
        status = fgo_history_counts(counts, vocab, history, history_count, err);
        if (status != FG_OK) return status;
        /* output.c:719-724 (GPU) restated through its CPU twin, sampler.c:46-60 */
        fg_sampler_apply_penalties(logits, iota, counts, vocab, config);
    }

    if (config->temperature == 0.0f) {
        /* output.c:565 / 727-733: cascade until one finalist is left. */
        const float *cur_scores = logits;
        const uint32_t *cur_ids = iota;
        uint32_t current = vocab;
        float **dst_scores = ping_scores;
        uint32_t **dst_ids = ping_ids;
        uint32_t slot = 0;
        float one_score;
        uint32_t one_id;
        if (current == 1u) {
            one_score = cur_scores[0];
            one_id = cur_ids[0];
        } else {
            while (current > 1u) {
                current = fgo_argmax_reduce(dst_scores[slot], dst_ids[slot], cur_scores, cur_ids,
                                            current);
                cur_scores = dst_scores[slot];
                cur_ids = dst_ids[slot];
                slot ^= 1u;
            }
            one_score = cur_scores[0];
            one_id = cur_ids[0];
        }
        if (one_id >= vocab || !isfinite(one_score)) {
            *token = one_id;
            *logit = one_score;
            if (penalties) {
                fg_error_set(err, FG_ERR_FORMAT, "invalid penalized output finalist");
                return FG_ERR_FORMAT; /* output.c:737-739 */
            }
            fg_error_set(err, FG_ERR_MISMATCH, "invalid output finalist at token %u", one_id);
            return FG_ERR_MISMATCH; /* output.c:593 */
        }
        *token = one_id;
        *logit = one_score;
        if (candidates) {
            candidates->count = 1u;
            candidates->ids[0] = one_id;
            candidates->scores[0] = one_score;
        }
        return FG_OK;
    }

    if (config->top_k == 0u) {
        /* Generalisation: no top-k cut, every finite logit is a candidate. */
        uint32_t nucleus = 0;
        double margin = INFINITY;
        const fg_status status = fgo_select_general(config, true, logits, iota, vocab, uniform, token,
                                                    logit, &nucleus, &margin, err);
        if (candidates) {  /* (no candidate dump beyond 64; the nucleus size and the edge margin) */
            candidates->nucleus = nucleus;
            candidates->edge_margin = margin;
        }
        return status;
    }

    /* output.c:681-700: tile top-k cascade until at most k entries remain. */
    const uint32_t k = config->top_k;
    const float *cur_scores = logits;
    const uint32_t *cur_ids = iota;
    uint32_t produced = vocab;
    float **dst_scores = ping_scores;
    uint32_t **dst_ids = ping_ids;
    /* a pass writes at most ceil(V/1024)*64 <= V/16 + 64 entries */
    uint32_t slot = 0;
    do {
        produced = fgo_topk_select(dst_scores[slot], dst_ids[slot], cur_scores, cur_ids, produced, k);
        cur_scores = dst_scores[slot];
        cur_ids = dst_ids[slot];
        slot ^= 1u;
    } while (produced > k);
    if (candidates) report_candidates(candidates, config, cur_scores, cur_ids, k);
    /* output.c:751 */
    return fg_sampler_select(config, cur_scores, cur_ids, k, uniform, token, logit, err);
}

/* ------------------------------------------------------------ batched rows */

static void widen_row(float *dst, const void *logits, uint32_t dtype, uint64_t element_offset,
                      uint32_t vocab) {
    if (dtype == FGO_DTYPE_BF16) {
        const uint16_t *src = (const uint16_t *)logits + element_offset;
        for (uint32_t i = 0; i < vocab; i++) {
            const uint32_t bits = (uint32_t)src[i] << 16;
            memcpy(&dst[i], &bits, sizeof bits);
        }
    } else {
        memcpy(dst, (const float *)logits + element_offset, (size_t)vocab * sizeof(float));
    }
}

typedef struct batch_job {
    const void *logits;
    uint32_t dtype, rows, vocab;
    uint64_t row_stride;
    const uint32_t *history_tokens;
    const uint64_t *history_offsets;
    const fg_sampler_config *configs;
    uint32_t config_count;
    bool allow_no_topk;
    const float *uniforms;
    uint32_t *tokens;
    float *token_logits;
    uint32_t *row_status;
    fgo_candidates *candidates;
    uint32_t threads, index;
} batch_job;

static void *batch_worker(void *arg) {
    const batch_job *job = arg;
    float *row = malloc((size_t)job->vocab * sizeof *row);
    uint32_t *scratch = malloc((6u * (size_t)job->vocab + 512u) * sizeof *scratch);
    if (row == NULL || scratch == NULL) {
        for (uint32_t r = job->index; r < job->rows; r += job->threads)
            job->row_status[r] = FG_ERR_OOM;
        free(row);
        free(scratch);
        return NULL;
    }
    for (uint32_t r = job->index; r < job->rows; r += job->threads) {
        widen_row(row, job->logits, job->dtype, (uint64_t)r * job->row_stride, job->vocab);
        const fg_sampler_config *config = &job->configs[job->config_count == 1u ? 0u : r];
        const uint32_t *history = NULL;
        uint32_t history_count = 0;
        if (job->history_tokens != NULL && job->history_offsets != NULL) {
            history = job->history_tokens + job->history_offsets[r];
            history_count = (uint32_t)(job->history_offsets[r + 1u] - job->history_offsets[r]);
        }
        uint32_t token = FGO_PADDING_ID;
        float logit = 0.0f;
        fg_error err = {0};
        const fg_status status = fgo_sample_row(
            row, job->vocab, history, history_count, config, job->allow_no_topk,
            job->uniforms ? job->uniforms[r] : 0.0f, &token, &logit,
            job->candidates ? &job->candidates[r] : NULL, scratch, &err);
        job->row_status[r] = (uint32_t)status;
        job->tokens[r] = token;
        job->token_logits[r] = logit;
    }
    free(row);
    free(scratch);
    return NULL;
}

fg_status fgo_sample_batch(const void *logits, uint32_t dtype, uint32_t rows, uint32_t vocab,
                           uint64_t row_stride, const uint32_t *history_tokens,
                           const uint64_t *history_offsets, const fg_sampler_config *configs,
                           uint32_t config_count, bool allow_no_topk, const float *uniforms,
                           uint32_t *tokens, float *token_logits, uint32_t *row_status,
                           fgo_candidates *candidates, uint32_t threads) {
    if (logits == NULL || rows == 0u || vocab == 0u || configs == NULL || tokens == NULL ||
        token_logits == NULL || row_status == NULL ||
        (config_count != 1u && config_count != rows))
        return FG_ERR_ARGUMENT;
    if (threads == 0u) threads = 1u;
    if (threads > rows) threads = rows;
    if (threads > 256u) threads = 256u;
    batch_job jobs[256];
    pthread_t handles[256];
    for (uint32_t t = 0; t < threads; t++) {
        jobs[t] = (batch_job){logits, dtype, rows, vocab, row_stride, history_tokens,
                              history_offsets, configs, config_count, allow_no_topk, uniforms,
                              tokens, token_logits, row_status, candidates, threads, t};
    }
    if (threads == 1u) {
        batch_worker(&jobs[0]);
    } else {
        uint32_t started = 0;
        for (; started < threads; started++)
            if (pthread_create(&handles[started], NULL, batch_worker, &jobs[started]) != 0) break;
        for (uint32_t t = started; t < threads; t++) batch_worker(&jobs[t]);
        for (uint32_t t = 0; t < started; t++) pthread_join(handles[t], NULL);
    }
    for (uint32_t r = 0; r < rows; r++)
        if (row_status[r] != FG_OK) return (fg_status)row_status[r];
    return FG_OK;
}

/* ------------------------------------------------------ vocabulary shards */

fg_status fgo_shard_topk(const void *logits, uint32_t dtype, uint32_t rows, uint32_t shard_vocab,
                         uint64_t row_stride, uint32_t vocab_offset, uint32_t vocab_total,
                         const uint32_t *history_tokens, const uint64_t *history_offsets,
                         const fg_sampler_config *configs, uint32_t config_count,
                         uint32_t k_shard, float *candidate_scores, uint32_t *candidate_ids,
                         uint32_t *row_status) {
    if (logits == NULL || rows == 0u || shard_vocab == 0u || k_shard == 0u || k_shard > 64u ||
        (uint64_t)vocab_offset + shard_vocab > vocab_total || configs == NULL ||
        candidate_scores == NULL || candidate_ids == NULL || row_status == NULL)
        return FG_ERR_ARGUMENT;
    float *row = malloc((size_t)shard_vocab * sizeof *row);
    uint32_t *global_ids = malloc((size_t)shard_vocab * sizeof *global_ids);
    uint32_t *counts = malloc((size_t)vocab_total * sizeof *counts);
    float *ping_scores = malloc(((size_t)shard_vocab + 256u) * sizeof *ping_scores);
    uint32_t *ping_ids = malloc(((size_t)shard_vocab + 256u) * sizeof *ping_ids);
    fg_status first = FG_OK;
    if (!row || !global_ids || !counts || !ping_scores || !ping_ids) {
        first = FG_ERR_OOM;
        goto out;
    }
    /* the slice's ids are pre-offset by its first row, output.c:226-227 */
    for (uint32_t i = 0; i < shard_vocab; i++) global_ids[i] = vocab_offset + i;
    for (uint32_t r = 0; r < rows; r++) {
        const fg_sampler_config *config = &configs[config_count == 1u ? 0u : r];
        widen_row(row, logits, dtype, (uint64_t)r * row_stride, shard_vocab);
        fg_status status = FG_OK;
        if (fg_sampler_penalties_active(config)) {
            const uint32_t *history = NULL;
            uint32_t history_count = 0;
            if (history_tokens && history_offsets) {
                history = history_tokens + history_offsets[r];
                history_count = (uint32_t)(history_offsets[r + 1u] - history_offsets[r]);
            }
            fg_error err = {0};
            status = fgo_history_counts(counts, vocab_total, history, history_count, &err);
            if (status == FG_OK)
                fg_sampler_apply_penalties(row, global_ids, counts, shard_vocab, config);
        }
        float *dst = candidate_scores + (size_t)r * k_shard;
        uint32_t *dst_ids = candidate_ids + (size_t)r * k_shard;
        if (status == FG_OK) {
            const float *cur_scores = row;
            const uint32_t *cur_ids = global_ids;
            uint32_t produced = shard_vocab, slot = 0;
            float *half_scores[2] = {ping_scores, ping_scores + shard_vocab / 2u + 128u};
            uint32_t *half_ids[2] = {ping_ids, ping_ids + shard_vocab / 2u + 128u};
            do {
                produced = fgo_topk_select(half_scores[slot], half_ids[slot], cur_scores, cur_ids,
                                           produced, k_shard);
                cur_scores = half_scores[slot];
                cur_ids = half_ids[slot];
                slot ^= 1u;
            } while (produced > k_shard);
            memcpy(dst, cur_scores, (size_t)k_shard * sizeof *dst);
            memcpy(dst_ids, cur_ids, (size_t)k_shard * sizeof *dst_ids);
            if (config->temperature == 0.0f) {
                /* A greedy slice reports its argmax-order winner (src/output.c:320-344),
                 * and that order puts a NaN/Inf before every finite value, smallest id
                 * first (src/output.c:484-492): it leads the slice's candidates so that the
                 * fold of src/runtime.c:2458-2463 meets it and rejects the row. */
                for (uint32_t i = 0; i < shard_vocab; i++) {
                    if (isfinite(row[i])) continue;
                    memmove(dst + 1, dst, (size_t)(k_shard - 1u) * sizeof *dst);
                    memmove(dst_ids + 1, dst_ids, (size_t)(k_shard - 1u) * sizeof *dst_ids);
                    dst[0] = row[i];
                    dst_ids[0] = global_ids[i];
                    break;
                }
            }
        } else {
            for (uint32_t i = 0; i < k_shard; i++) {
                dst[i] = -INFINITY;
                dst_ids[i] = FGO_PADDING_ID;
            }
        }
        row_status[r] = (uint32_t)status;
        if (status != FG_OK && first == FG_OK) first = status;
    }
out:
    free(row);
    free(global_ids);
    free(counts);
    free(ping_scores);
    free(ping_ids);
    return first;
}

fg_status fgo_merge_select(const float *candidate_scores, const uint32_t *candidate_ids,
                           uint32_t shards, uint32_t rows, uint32_t k_shard,
                           const uint32_t *shard_first, const uint32_t *shard_width,
                           const fg_sampler_config *configs, uint32_t config_count,
                           const float *uniforms, uint32_t *tokens, float *token_logits,
                           uint32_t *row_status, fgo_candidates *candidates) {
    if (!candidate_scores || !candidate_ids || shards == 0u || shards > 16u || rows == 0u ||
        k_shard == 0u || k_shard > 64u || !shard_first || !shard_width || !configs || !tokens ||
        !token_logits || !row_status)
        return FG_ERR_ARGUMENT;
    fg_status first = FG_OK;
    float merged[16 * 64], picked[64], spare[64];
    uint32_t merged_ids[16 * 64], picked_ids[64], spare_ids[64];
    for (uint32_t r = 0; r < rows; r++) {
        const fg_sampler_config *config = &configs[config_count == 1u ? 0u : r];
        fg_status status = FG_OK;
        uint32_t total = 0;
        for (uint32_t s = 0; s < shards && status == FG_OK; s++) {
            const size_t base = ((size_t)s * rows + r) * k_shard;
            for (uint32_t i = 0; i < k_shard; i++) {
                const uint32_t id = candidate_ids[base + i];
                if (id != FGO_PADDING_ID &&
                    (id < shard_first[s] || id - shard_first[s] >= shard_width[s])) {
                    status = FG_ERR_MISMATCH; /* runtime.c:2451-2456 */
                    break;
                }
                merged[total] = candidate_scores[base + i];
                merged_ids[total] = id;
                total++;
            }
        }
        uint32_t token = FGO_PADDING_ID;
        float logit = 0.0f;
        if (status == FG_OK && config->temperature == 0.0f) {
            /* runtime.c:2458-2459: fold the partials with the argmax order. */
            float best = merged[0];
            uint32_t best_id = merged_ids[0];
            for (uint32_t i = 1; i < total; i++)
                fg_output_combine(merged[i], merged_ids[i], best, best_id, &best, &best_id);
            token = best_id;
            logit = best;
            if (best_id == FGO_PADDING_ID || !isfinite(best)) status = FG_ERR_MISMATCH;
            if (candidates) {
                memset(&candidates[r], 0, sizeof candidates[r]);
                if (status == FG_OK) {
                    candidates[r].count = 1u;
                    candidates[r].ids[0] = best_id;
                    candidates[r].scores[0] = best;
                }
            }
        } else if (status == FG_OK) {
            /* the union is one more round of the tile cascade (output.c:689-696) */
            const float *cur = merged;
            const uint32_t *cur_ids = merged_ids;
            uint32_t produced = total, flip = 0;
            const uint32_t k = config->top_k;
            float *dst[2] = {picked, spare};
            uint32_t *dst_ids[2] = {picked_ids, spare_ids};
            do {
                produced = fgo_topk_select(dst[flip], dst_ids[flip], cur, cur_ids, produced, k);
                cur = dst[flip];
                cur_ids = dst_ids[flip];
                flip ^= 1u;
            } while (produced > k);
            fg_error err = {0};
            if (candidates) report_candidates(&candidates[r], config, cur, cur_ids, k);
            status = fg_sampler_select(config, cur, cur_ids, k, uniforms ? uniforms[r] : 0.0f,
                                       &token, &logit, &err);
        }
        tokens[r] = token;
        token_logits[r] = logit;
        row_status[r] = (uint32_t)status;
        if (status != FG_OK && first == FG_OK) first = status;
    }
    return first;
}
