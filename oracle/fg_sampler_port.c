/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference's host sampler.
 *
 * This file is the checker for the CUDA path, never the product: only tests,
 * the smoke check and the CPU-baseline legs of the benchmark link it.  It
 * restates, in fresh code, the algorithm of the reference's src/sampler.c and
 * src/util.c; every function cites the lines it follows.  Floating-point
 * operations keep the reference's order and width (fp32 penalties without
 * fused multiply-add, fp64 softmax sums accumulated left to right) because
 * parity is judged bit for bit.
 *
 * Pinned against: the reference's own tests/test_sampler.c (compiled unchanged
 * against this file by oracle/Makefile, target `check`) and, when the reference
 * tree is present, the reference objects themselves (oracle/_ref) on random
 * inputs (tests/test_oracle_vs_reference.py) and the committed vectors in
 * tests/golden/.
 */
#include "fg_sampler.h"

#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

/* ---- src/util.c:6-8 ---- */

void fg_error_set(fg_error *err, fg_status code, const char *fmt, ...) {
    if (err == NULL) return;
    va_list args;
    va_start(args, fmt);
    err->code = code;
    vsnprintf(err->message, sizeof err->message, fmt, args);
    va_end(args);
}

uint64_t fg_align_up_u64(uint64_t value, uint64_t alignment) {
    if (alignment == 0) return value;
    return (value + alignment - 1u) & ~(alignment - 1u);
}

bool fg_is_aligned_u64(uint64_t value, uint64_t alignment) {
    return alignment != 0 && (value & (alignment - 1u)) == 0;
}

/* ---- src/sampler.c:6-22 ---- */

#define PORT_DEFAULT_SEED UINT64_C(0x9e3779b97f4a7c15)

static void fill_config(fg_sampler_config *c, float temperature, float top_p, uint32_t top_k) {
    c->temperature = temperature;
    c->top_p = top_p;
    c->top_k = top_k;
    c->presence_penalty = 0.0f;
    c->frequency_penalty = 0.0f;
    c->repetition_penalty = 1.0f;
    c->min_p = 0.0f;
    c->seed = PORT_DEFAULT_SEED;
}

void fg_sampler_config_greedy(fg_sampler_config *config) {
    if (config) fill_config(config, 0.0f, 1.0f, 1u);
}

void fg_sampler_config_defaults(fg_sampler_config *config) {
    if (config) fill_config(config, 1.0f, 0.95f, 20u);
}

/* ---- src/sampler.c:24-38 ---- */

static bool in_closed_range(float v, float lo, float hi) {
    return isfinite(v) && !(v < lo) && !(v > hi);
}

fg_status fg_sampler_config_validate(const fg_sampler_config *config, fg_error *err) {
    bool ok = config != NULL;
    ok = ok && isfinite(config->temperature) && !(config->temperature < 0.0f);
    ok = ok && isfinite(config->top_p) && config->top_p > 0.0f && !(config->top_p > 1.0f);
    ok = ok && config->top_k >= 1u && config->top_k <= 64u;
    ok = ok && in_closed_range(config->presence_penalty, -2.0f, 2.0f);
    ok = ok && in_closed_range(config->frequency_penalty, -2.0f, 2.0f);
    ok = ok && isfinite(config->repetition_penalty) && config->repetition_penalty > 0.0f;
    ok = ok && isfinite(config->min_p) && config->min_p == 0.0f;
    if (ok) return FG_OK;
    fg_error_set(err, FG_ERR_ARGUMENT, "invalid sampler controls");
    return FG_ERR_ARGUMENT;
}

/* ---- src/sampler.c:40-44 ---- */

bool fg_sampler_penalties_active(const fg_sampler_config *config) {
    if (config == NULL) return false;
    return config->presence_penalty != 0.0f || config->frequency_penalty != 0.0f ||
           config->repetition_penalty != 1.0f;
}

/* ---- src/sampler.c:46-60 ----
 * volatile temporaries pin every intermediate to fp32 and forbid contraction
 * whatever flags the file is built with. */

void fg_sampler_apply_penalties(float *scores, const uint32_t *ids, const uint32_t *counts,
                                uint32_t count, const fg_sampler_config *config) {
    if (scores == NULL || ids == NULL || counts == NULL || config == NULL) return;
    const float repetition = config->repetition_penalty;
    const float frequency = config->frequency_penalty;
    const float presence = config->presence_penalty;
    for (uint32_t i = 0; i < count; i++) {
        const uint32_t seen = counts[ids[i]];
        if (seen == 0u) continue;
        volatile float value = scores[i];
        if (repetition != 1.0f) {
            if (value > 0.0f) value = value / repetition;
            else value = value * repetition;
        }
        volatile float scaled = frequency * (float)seen;
        volatile float offset = scaled + presence;
        scores[i] = value - offset;
    }
}

/* ---- src/sampler.c:62-73: xorshift64*, 24-bit uniform ---- */

void fg_sampler_state_init(fg_sampler_state *state, uint64_t seed) {
    if (state) state->state = seed != 0 ? seed : PORT_DEFAULT_SEED;
}

float fg_sampler_uniform(fg_sampler_state *state) {
    uint64_t x = state->state;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    state->state = x;
    const uint64_t scrambled = x * UINT64_C(2685821657736338717);
    const uint64_t top24 = scrambled >> 40;
    return (float)((double)top24 * (1.0 / 16777216.0));
}

/* ---- src/sampler.c:75-122 ---- */

static bool ranks_before(float a, uint32_t a_id, float b, uint32_t b_id) {
    if (a != b) return a > b;
    return a_id < b_id;
}

fg_status fg_sampler_select(const fg_sampler_config *config, const float *scores,
                            const uint32_t *ids, uint32_t count, float uniform,
                            uint32_t *token, float *logit, fg_error *err) {
    const bool config_ok = fg_sampler_config_validate(config, err) == FG_OK;
    if (!config_ok || scores == NULL || ids == NULL || count == 0u || count > 64u ||
        token == NULL || logit == NULL) {
        /* sampler.c:83-87: keep an earlier message, return an earlier code. */
        if (err != NULL && err->message[0] == '\0')
            fg_error_set(err, FG_ERR_ARGUMENT, "invalid sampler candidates");
        if (err != NULL && err->code != FG_OK) return err->code;
        return FG_ERR_ARGUMENT;
    }

    /* sampler.c:88-96: insertion sort of the finite candidates. */
    uint32_t sorted[64];
    uint32_t kept = 0;
    for (uint32_t i = 0; i < count; i++) {
        if (!isfinite(scores[i])) continue;
        uint32_t slot = kept;
        while (slot > 0u) {
            const uint32_t prev = sorted[slot - 1u];
            if (!ranks_before(scores[i], ids[i], scores[prev], ids[prev])) break;
            sorted[slot] = prev;
            slot--;
        }
        sorted[slot] = i;
        kept++;
    }
    if (kept == 0u) {
        fg_error_set(err, FG_ERR_FORMAT, "sampler received no finite candidates");
        return FG_ERR_FORMAT;
    }
    const uint32_t best = sorted[0];
    if (config->temperature == 0.0f) {
        *token = ids[best];
        *logit = scores[best];
        return FG_OK;
    }

    /* sampler.c:99-102: untempered softmax denominator over the top_k set. */
    const uint32_t limit = kept < config->top_k ? kept : config->top_k;
    const double top_raw = scores[best];
    double raw_sum = 0.0;
    for (uint32_t r = 0; r < limit; r++) raw_sum += exp((double)scores[sorted[r]] - top_raw);
    if (!(raw_sum > 0.0) || !isfinite(raw_sum)) {
        fg_error_set(err, FG_ERR_FORMAT, "sampler raw softmax failed");
        return FG_ERR_FORMAT;
    }

    /* sampler.c:103-107: top-p keeps the candidate that crosses the mass. */
    uint32_t survivors = limit;
    double mass = 0.0;
    for (uint32_t r = 0; r < limit; r++) {
        mass += exp((double)scores[sorted[r]] - top_raw) / raw_sum;
        if (mass >= config->top_p) {
            survivors = r + 1u;
            break;
        }
    }

    /* sampler.c:108-111: temperature weights of the survivors. */
    const double temperature = (double)config->temperature;
    const double top_tempered = (double)scores[best] / temperature;
    double weight_sum = 0.0;
    for (uint32_t r = 0; r < survivors; r++)
        weight_sum += exp((double)scores[sorted[r]] / temperature - top_tempered);
    if (!(weight_sum > 0.0) || !isfinite(weight_sum)) {
        fg_error_set(err, FG_ERR_FORMAT, "sampler temperature softmax failed");
        return FG_ERR_FORMAT;
    }

    /* sampler.c:112-119: clamp the draw, walk the CDF. */
    if (!isfinite(uniform) || uniform < 0.0f) uniform = 0.0f;
    if (uniform >= 1.0f) uniform = nextafterf(1.0f, 0.0f);
    const double draw = (double)uniform * weight_sum;
    uint32_t pick = survivors - 1u;
    double walked = 0.0;
    for (uint32_t r = 0; r < survivors; r++) {
        walked += exp((double)scores[sorted[r]] / temperature - top_tempered);
        if (draw < walked) {
            pick = r;
            break;
        }
    }
    *token = ids[sorted[pick]];
    *logit = scores[sorted[pick]];
    return FG_OK;
}
