/*
 * The fg_sampler.h entry points (host pointers), argument meaning and error
 * behaviour of the reference's src/sampler.c.
 *
 * Request set-up (defaults, validation, the xorshift64* stream) is host code,
 * as it is on the reference's coordinator.  The two functions that do
 * per-candidate arithmetic — apply_penalties and select — stage their inputs
 * to the GPU and run the same kernels as the batched path; there is no CPU
 * arithmetic path behind them.
 */
#include "fg_host_internal.h"

#include <math.h>
#include <pthread.h>
#include <string.h>

#define FG_GOLDEN_SEED UINT64_C(0x9e3779b97f4a7c15) /* src/sampler.c:6 */

static _Thread_local fg_status last_status = FG_OK;

fg_status fg_sampler_last_status(void) { return last_status; }

/* src/sampler.c:8-22: the two presets differ in three fields only. */
static void preset(fg_sampler_config *config, float temperature, float top_p, uint32_t top_k) {
    if (!config) return;
    memset(config, 0, sizeof(*config));
    config->temperature = temperature;
    config->top_p = top_p;
    config->top_k = top_k;
    config->repetition_penalty = 1.0f;
    config->seed = FG_GOLDEN_SEED;
}

void fg_sampler_config_greedy(fg_sampler_config *config) { preset(config, 0.0f, 1.0f, 1u); }

void fg_sampler_config_defaults(fg_sampler_config *config) { preset(config, 1.0f, 0.95f, 20u); }

bool fg_cuda_config_ok(const fg_sampler_config *c, bool allow_no_topk) {
    if (!c) return false;
    if (!isfinite(c->temperature) || c->temperature < 0.0f) return false;
    if (!isfinite(c->top_p) || c->top_p <= 0.0f || c->top_p > 1.0f) return false;
    if (c->top_k > 64u) return false;
    if (c->top_k == 0u && !allow_no_topk) return false;
    if (!isfinite(c->presence_penalty) || fabsf(c->presence_penalty) > 2.0f) return false;
    if (!isfinite(c->frequency_penalty) || fabsf(c->frequency_penalty) > 2.0f) return false;
    if (!isfinite(c->repetition_penalty) || c->repetition_penalty <= 0.0f) return false;
    if (!isfinite(c->min_p) || c->min_p != 0.0f) return false;
    return true;
}

/* src/sampler.c:24-38 */
fg_status fg_sampler_config_validate(const fg_sampler_config *config, fg_error *err) {
    if (fg_cuda_config_ok(config, false)) return FG_OK;
    fg_error_set(err, FG_ERR_ARGUMENT, "invalid sampler controls");
    return FG_ERR_ARGUMENT;
}

/* src/sampler.c:40-44 */
bool fg_sampler_penalties_active(const fg_sampler_config *config) {
    if (!config) return false;
    return config->presence_penalty != 0.0f || config->frequency_penalty != 0.0f ||
           config->repetition_penalty != 1.0f;
}

/* src/sampler.c:62-65 */
void fg_sampler_state_init(fg_sampler_state *state, uint64_t seed) {
    if (state) state->state = seed ? seed : FG_GOLDEN_SEED;
}

/* src/sampler.c:67-73: xorshift64* step, top 24 bits scaled to [0, 1). */
float fg_sampler_uniform(fg_sampler_state *state) {
    uint64_t s = state->state;
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    state->state = s;
    const uint64_t mixed = s * UINT64_C(0x2545F4914F6CDD1D);
    return (float)((double)(mixed >> 40) * 0x1p-24);
}

/* ------------------------------------------------------- process-wide context */

static pthread_mutex_t default_mutex = PTHREAD_MUTEX_INITIALIZER;
static fg_cuda_context *default_context;

void fg_cuda_default_lock(void) { pthread_mutex_lock(&default_mutex); }
void fg_cuda_default_unlock(void) { pthread_mutex_unlock(&default_mutex); }

fg_status fg_cuda_default_context(fg_cuda_context **out, fg_error *err) {
    if (!default_context) {
        fg_status status = fg_cuda_context_create(0, &default_context, err);
        if (status != FG_OK) {
            default_context = NULL;
            return status;
        }
    }
    *out = default_context;
    return fg_cuda_enter(default_context, err);
}

/* ------------------------------------------------ src/sampler.c:46-60 on the GPU */

void fg_sampler_apply_penalties(float *scores, const uint32_t *ids, const uint32_t *counts,
                                uint32_t count, const fg_sampler_config *config) {
    if (!scores || !ids || !counts || !config) return;
    last_status = FG_OK;
    if (!count) return;
    fg_error err = {0};
    fg_cuda_default_lock();
    fg_cuda_context *ctx = NULL;
    fg_status status = fg_cuda_default_context(&ctx, &err);
    const size_t bytes = (size_t)count * 4u;
    /* device: [scores | seen]; pinned: [scores | seen] */
    if (status == FG_OK) status = fg_cuda_reserve(&ctx->staging, &ctx->staging_bytes, 2u * bytes + 32u, false, ctx, &err);
    if (status == FG_OK) status = fg_cuda_reserve_pinned(ctx, 2u * bytes, &err);
    if (status == FG_OK) {
        float *pinned_scores = ctx->pinned;
        uint32_t *pinned_seen = (uint32_t *)((unsigned char *)ctx->pinned + bytes);
        /* staging only: the id indirection of the C signature is resolved while the
         * operands are packed for the copy */
        memcpy(pinned_scores, scores, bytes);
        for (uint32_t i = 0; i < count; i++) pinned_seen[i] = counts[ids[i]];
        float *device_scores = ctx->staging;
        uint32_t *device_seen = (uint32_t *)((unsigned char *)ctx->staging + fg_align_up_u64(bytes, 16u));
        int e = fgk_copy_to_device_async(device_scores, pinned_scores, bytes, ctx->stream);
        if (!e) e = fgk_copy_to_device_async(device_seen, pinned_seen, bytes, ctx->stream);
        if (!e) {
            e = fgk_launch_apply_penalties_seen(device_scores, device_seen, count,
                                                config->presence_penalty, config->frequency_penalty,
                                                config->repetition_penalty, ctx->stream);
            ctx->launches++;
        }
        if (!e) e = fgk_copy_to_host_async(pinned_scores, device_scores, bytes, ctx->stream);
        if (!e) e = fgk_stream_synchronize(ctx->stream);
        if (e) status = fg_cuda_fail(&err, e, "penalty kernel");
        else memcpy(scores, pinned_scores, bytes);
    }
    fg_cuda_default_unlock();
    last_status = status;
}

/* ----------------------------------------------- src/sampler.c:80-122 on the GPU */

fg_status fg_sampler_select(const fg_sampler_config *config, const float *scores,
                            const uint32_t *ids, uint32_t count, float uniform,
                            uint32_t *token, float *logit, fg_error *err) {
    /* argument handling of src/sampler.c:83-87, including its two quirks: an
     * earlier message is kept and an earlier non-zero code is returned */
    if (fg_sampler_config_validate(config, err) != FG_OK || !scores || !ids || !count ||
        count > 64u || !token || !logit) {
        if (err && !err->message[0]) fg_error_set(err, FG_ERR_ARGUMENT, "invalid sampler candidates");
        last_status = err && err->code ? err->code : FG_ERR_ARGUMENT;
        return last_status;
    }
    bool any_finite = false;
    for (uint32_t i = 0; i < count; i++) any_finite = any_finite || isfinite(scores[i]);

    fg_cuda_default_lock();
    fg_cuda_context *ctx = NULL;
    fg_status status = fg_cuda_default_context(&ctx, err);
    /* device staging: scores[64] ids[64] uniform token logit status first_error */
    enum { SCORES = 0, IDS = 256, UNIFORM = 512, TOKEN = 528, LOGIT = 532, STATUS = 536, TOTAL = 544 };
    if (status == FG_OK) status = fg_cuda_reserve(&ctx->staging, &ctx->staging_bytes, TOTAL, false, ctx, err);
    if (status == FG_OK) status = fg_cuda_reserve_pinned(ctx, TOTAL, err);
    if (status == FG_OK) {
        unsigned char *pinned = ctx->pinned, *device = ctx->staging;
        memcpy(pinned + SCORES, scores, (size_t)count * 4u);
        memcpy(pinned + IDS, ids, (size_t)count * 4u);
        memcpy(pinned + UNIFORM, &uniform, 4u);
        const uint64_t none = UINT64_MAX;
        fgk_merge_launch launch;
        memset(&launch, 0, sizeof(launch));
        launch.scores = (const float *)(device + SCORES);
        launch.ids = (const uint32_t *)(device + IDS);
        launch.rows = 1u;
        launch.shards = 1u;
        launch.k_shard = count;
        launch.check_spans = 0u;
        launch.config0 = *config;
        launch.config_count = 1u;
        launch.uniforms = (const float *)(device + UNIFORM);
        launch.out.tokens = (uint32_t *)(device + TOKEN);
        launch.out.token_logits = (float *)(device + LOGIT);
        launch.out.row_status = (uint32_t *)(device + STATUS);
        launch.out.first_error = ctx->first_error;
        int e = fgk_copy_to_device_async(device, pinned, UNIFORM + 4u, ctx->stream);
        if (!e) e = fgk_copy_to_device_async(ctx->first_error, &none, 8u, ctx->stream);
        if (!e) {
            e = fgk_launch_merge_select(&launch, ctx->stream);
            ctx->launches++;
        }
        if (!e) e = fgk_copy_to_host_async(pinned + TOKEN, device + TOKEN, 12u, ctx->stream);
        if (!e) e = fgk_stream_synchronize(ctx->stream);
        if (e) {
            status = fg_cuda_fail(err, e, "select kernel");
        } else {
            uint32_t row_status;
            memcpy(&row_status, pinned + STATUS, 4u);
            status = (fg_status)row_status;
            if (status == FG_OK) {
                memcpy(token, pinned + TOKEN, 4u);
                memcpy(logit, pinned + LOGIT, 4u);
            } else if (!any_finite) {
                fg_error_set(err, status, "sampler received no finite candidates");
            } else {
                /* src/sampler.c:102 cannot be what failed: the un-tempered sum holds
                 * exp(0) for the best finite candidate and at most 63 terms in (0, 1],
                 * so it is finite and positive; what is left is src/sampler.c:111 */
                fg_error_set(err, status, "sampler temperature softmax failed");
            }
        }
    }
    fg_cuda_default_unlock();
    last_status = status;
    return status;
}
