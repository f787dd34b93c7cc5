/*
 * fg_sampler_config_from_json (include/fg_request.h).  Host C17.
 *
 * A single forward scan over the request body: the top-level object's members are walked
 * once, the eight sampler members are picked up as they come by, everything else is skipped
 * by a small recogniser of JSON values (strings with escapes, nested arrays and objects to a
 * bounded depth).  Ranges, defaults and texts follow src/api.c:1606-1631 of the reference.
 */
#include "fg_request.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

typedef struct scan {
    const char *at, *end;
} scan;

enum { MAX_DEPTH = 64 };

static void skip_space(scan *s) {
    while (s->at < s->end && (*s->at == ' ' || *s->at == '\t' || *s->at == '\n' || *s->at == '\r')) s->at++;
}

static bool take(scan *s, char c) {
    skip_space(s);
    if (s->at < s->end && *s->at == c) {
        s->at++;
        return true;
    }
    return false;
}

/* a string; *begin / *length give its raw bytes between the quotes */
static bool take_string(scan *s, const char **begin, size_t *length) {
    if (!take(s, '"')) return false;
    const char *start = s->at;
    while (s->at < s->end && *s->at != '"') {
        if ((unsigned char)*s->at < 0x20) return false;
        if (*s->at == '\\') {
            s->at++;
            if (s->at >= s->end) return false;
            if (*s->at == 'u') {
                if (s->end - s->at < 5) return false;
                s->at += 4;
            } else if (!strchr("\"\\/bfnrt", *s->at)) {
                return false;
            }
        }
        s->at++;
    }
    if (s->at >= s->end) return false;
    if (begin) *begin = start;
    if (length) *length = (size_t)(s->at - start);
    s->at++;
    return true;
}

/* a number, by the JSON grammar; its value through strtod on a bounded copy */
static bool take_number(scan *s, double *value) {
    skip_space(s);
    const char *start = s->at;
    if (s->at < s->end && *s->at == '-') s->at++;
    if (s->at >= s->end) return false;
    if (*s->at == '0') {
        s->at++;
    } else if (*s->at >= '1' && *s->at <= '9') {
        while (s->at < s->end && *s->at >= '0' && *s->at <= '9') s->at++;
    } else {
        return false;
    }
    if (s->at < s->end && *s->at == '.') {
        s->at++;
        if (s->at >= s->end || *s->at < '0' || *s->at > '9') return false;
        while (s->at < s->end && *s->at >= '0' && *s->at <= '9') s->at++;
    }
    if (s->at < s->end && (*s->at == 'e' || *s->at == 'E')) {
        s->at++;
        if (s->at < s->end && (*s->at == '+' || *s->at == '-')) s->at++;
        if (s->at >= s->end || *s->at < '0' || *s->at > '9') return false;
        while (s->at < s->end && *s->at >= '0' && *s->at <= '9') s->at++;
    }
    char copy[64];
    const size_t length = (size_t)(s->at - start);
    if (length >= sizeof(copy)) {  /* absurdly long literal: still a number, read what fits exactly */
        char *heap = malloc(length + 1);
        if (!heap) return false;
        memcpy(heap, start, length);
        heap[length] = 0;
        *value = strtod(heap, NULL);
        free(heap);
        return true;
    }
    memcpy(copy, start, length);
    copy[length] = 0;
    *value = strtod(copy, NULL);
    return true;
}

static bool take_word(scan *s, const char *word) {
    skip_space(s);
    const size_t length = strlen(word);
    if ((size_t)(s->end - s->at) < length || memcmp(s->at, word, length) != 0) return false;
    s->at += length;
    return true;
}

static bool skip_value(scan *s, int depth) {
    if (depth > MAX_DEPTH) return false;
    skip_space(s);
    if (s->at >= s->end) return false;
    const char c = *s->at;
    if (c == '"') return take_string(s, NULL, NULL);
    if (c == '{' || c == '[') {
        const char close = c == '{' ? '}' : ']';
        s->at++;
        if (take(s, close)) return true;
        do {
            if (c == '{' && (!take_string(s, NULL, NULL) || !take(s, ':'))) return false;
            if (!skip_value(s, depth + 1)) return false;
        } while (take(s, ','));
        return take(s, close);
    }
    if (c == 't') return take_word(s, "true");
    if (c == 'f') return take_word(s, "false");
    if (c == 'n') return take_word(s, "null");
    double ignored;
    return take_number(s, &ignored);
}

typedef enum { F_TEMPERATURE, F_TOP_P, F_TOP_K, F_SEED, F_PRESENCE, F_FREQUENCY, F_REPETITION, F_MIN_P, F_COUNT } field;

static const char *const field_names[F_COUNT] = {"temperature", "top_p", "top_k", "seed", "presence_penalty",
                                                 "frequency_penalty", "repetition_penalty", "min_p"};

static fg_status refuse(fg_error *err, const char *why) {
    fg_error_set(err, FG_ERR_ARGUMENT, "%s", why);
    return FG_ERR_ARGUMENT;
}

/* One sampler member; `is_number` false when its value was of another type. */
static fg_status apply(field which, bool is_number, double v, fg_sampler_config *config, fg_error *err) {
    switch (which) {
    case F_TEMPERATURE:
        if (!is_number || !isfinite(v) || v < 0.0 || v > FLT_MAX)
            return refuse(err, "temperature must be a finite non-negative number");
        config->temperature = (float)v;
        return FG_OK;
    case F_TOP_P:
        if (!is_number || !isfinite(v) || v <= 0.0 || v > 1.0)
            return refuse(err, "top_p must be greater than 0 and at most 1");
        config->top_p = (float)v;
        return FG_OK;
    case F_TOP_K:
        if (!is_number || !(v >= 1.0 && v <= 64.0) || v != (double)(uint32_t)v)
            return refuse(err, "top_k must be an integer from 1 through 64");
        config->top_k = (uint32_t)v;
        return FG_OK;
    case F_SEED:
        if (!is_number || !isfinite(v) || v < 0.0 || v > 9007199254740991.0 || v != floor(v))
            return refuse(err, "seed must be a non-negative integer");
        config->seed = (uint64_t)v;
        return FG_OK;
    case F_PRESENCE:
        if (!is_number || !isfinite(v)) return refuse(err, "presence_penalty must be finite");
        config->presence_penalty = (float)v;
        return FG_OK;
    case F_FREQUENCY:
        if (!is_number || !isfinite(v)) return refuse(err, "frequency_penalty must be finite");
        config->frequency_penalty = (float)v;
        return FG_OK;
    case F_REPETITION:
        if (!is_number || !isfinite(v)) return refuse(err, "repetition_penalty must be finite");
        config->repetition_penalty = (float)v;
        return FG_OK;
    case F_MIN_P:
        if (!is_number || !isfinite(v) || v != 0.0) return refuse(err, "min_p currently supports only 0");
        config->min_p = 0.0f;
        return FG_OK;
    default:
        return FG_OK;
    }
}

fg_status fg_sampler_config_from_json(const char *json, size_t bytes, fg_sampler_config *config,
                                      fg_error *err) {
    if (!json || !config) return refuse(err, "invalid request arguments");
    fg_sampler_config_defaults(config);
    scan s = {json, json + bytes};
    bool seen[F_COUNT] = {false};
    /* the reference reads its members in a fixed order, so the first failing field in THAT
     * order is the one reported: values are collected first, applied afterwards */
    bool present[F_COUNT] = {false}, numeric[F_COUNT] = {false};
    double number[F_COUNT] = {0};
    bool object = take(&s, '{');
    if (object && !take(&s, '}')) {
        do {
            const char *name;
            size_t length;
            if (!take_string(&s, &name, &length) || !take(&s, ':')) {
                object = false;
                break;
            }
            int which = -1;
            for (int f = 0; f < F_COUNT; f++)
                if (strlen(field_names[f]) == length && memcmp(field_names[f], name, length) == 0) which = f;
            if (which >= 0 && !seen[which]) {
                seen[which] = true;
                present[which] = true;
                skip_space(&s);
                const char *before = s.at;
                double v = 0.0;
                if (s.at < s.end && (*s.at == '-' || (*s.at >= '0' && *s.at <= '9')) && take_number(&s, &v)) {
                    numeric[which] = true;
                    number[which] = v;
                } else {
                    s.at = before;
                    if (!skip_value(&s, 0)) {
                        object = false;
                        break;
                    }
                }
            } else if (!skip_value(&s, 0)) {
                object = false;
                break;
            }
        } while (take(&s, ','));
        if (object) object = take(&s, '}');
    }
    skip_space(&s);
    if (!object || s.at != s.end) {
        fg_error_set(err, FG_ERR_FORMAT, "request body is not a JSON object");
        return FG_ERR_FORMAT;
    }
    for (int f = 0; f < F_COUNT; f++) {
        if (!present[f]) continue;
        const fg_status status = apply((field)f, numeric[f], number[f], config, err);
        if (status != FG_OK) return status;
    }
    return fg_sampler_config_validate(config, err);
}
