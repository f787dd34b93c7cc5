/*
 * Codecs of include/fg_output_wire.h.  Host C17, no GPU involved.
 *
 * Each fixed-size message is described once, as a table of fields (offset on the wire,
 * offset in the struct, kind); one encoder and one decoder walk the tables.  Checks are the
 * reference's and fail closed: wrong size, set reserved bytes, routes outside the rank
 * layout, sampler blocks that do not validate, draws outside [0, 1), tokens outside the
 * vocabulary and non-finite values are all refused (src/protocol.c:1156-1166, 1275-1289,
 * 1328-1367).
 */
#include "fg_output_wire.h"

#include <math.h>
#include <stddef.h>
#include <stdio.h>
#include <string.h>

typedef enum { WIRE_U8, WIRE_U32, WIRE_F32 } wire_kind;

typedef struct wire_field {
    uint16_t at;      /* byte offset in the message */
    uint16_t member;  /* byte offset in the struct */
    wire_kind kind;
} wire_field;

static void store_be32(uint8_t *to, uint32_t value) {
    for (int i = 3; i >= 0; i--) {
        to[i] = (uint8_t)(value & 0xffu);
        value >>= 8;
    }
}

static uint32_t load_be32(const uint8_t *from) {
    uint32_t value = 0;
    for (int i = 0; i < 4; i++) value = (value << 8) | from[i];
    return value;
}

static void pack(uint8_t *message, const void *record, const wire_field *fields, size_t count) {
    const uint8_t *base = record;
    for (size_t i = 0; i < count; i++) {
        const wire_field *f = &fields[i];
        if (f->kind == WIRE_U8) {
            message[f->at] = base[f->member];
        } else {  /* a float travels as its bit pattern */
            uint32_t word;
            memcpy(&word, base + f->member, 4);
            store_be32(message + f->at, word);
        }
    }
}

static void unpack(void *record, const uint8_t *message, const wire_field *fields, size_t count) {
    uint8_t *base = record;
    for (size_t i = 0; i < count; i++) {
        const wire_field *f = &fields[i];
        if (f->kind == WIRE_U8) {
            base[f->member] = message[f->at];
        } else {
            const uint32_t word = load_be32(message + f->at);
            memcpy(base + f->member, &word, 4);
        }
    }
}

#define FIELD(at, type, member, kind) {(uint16_t)(at), (uint16_t)offsetof(type, member), kind}
#define COUNT(table) (sizeof(table) / sizeof((table)[0]))

/* byte 0 source, 1 destination, 2 flags, 3 session slot, 4 token index, 8 temperature,
 * 12 top_p, 16 top_k, 20 uniform, 24 presence, 28 frequency, 32 repetition, 36 min_p */
static const wire_field config_fields[] = {
    FIELD(0, fg_output_config, source_rank, WIRE_U8),
    FIELD(1, fg_output_config, destination_rank, WIRE_U8),
    FIELD(2, fg_output_config, flags, WIRE_U8),
    FIELD(3, fg_output_config, session_slot, WIRE_U8),
    FIELD(4, fg_output_config, token_index, WIRE_U32),
    FIELD(8, fg_output_config, sampler.temperature, WIRE_F32),
    FIELD(12, fg_output_config, sampler.top_p, WIRE_F32),
    FIELD(16, fg_output_config, sampler.top_k, WIRE_U32),
    FIELD(20, fg_output_config, uniform, WIRE_F32),
    FIELD(24, fg_output_config, sampler.presence_penalty, WIRE_F32),
    FIELD(28, fg_output_config, sampler.frequency_penalty, WIRE_F32),
    FIELD(32, fg_output_config, sampler.repetition_penalty, WIRE_F32),
    FIELD(36, fg_output_config, sampler.min_p, WIRE_F32),
};

/* byte 0 source, 1 destination, 2-3 reserved, 4 token index, 8 token, 12 logit */
static const wire_field result_fields[] = {
    FIELD(0, fg_output_result, source_rank, WIRE_U8),
    FIELD(1, fg_output_result, destination_rank, WIRE_U8),
    FIELD(4, fg_output_result, token_index, WIRE_U32),
    FIELD(8, fg_output_result, token, WIRE_U32),
    FIELD(12, fg_output_result, logit, WIRE_F32),
};

static const wire_field partial_fields[] = {
    FIELD(0, fg_output_partial, token_index, WIRE_U32),
    FIELD(4, fg_output_partial, value, WIRE_F32),
    FIELD(8, fg_output_partial, id, WIRE_U32),
};

fg_wire_limits fg_wire_limits_reference(void) {
    const fg_wire_limits limits = {8u, 4u, 2u, 248320u};
    return limits;
}

static fg_status refuse(fg_error *err, fg_status status, const char *why) {
    fg_error_set(err, status, "%s", why);
    return status;
}

/* ------------------------------------------------------------------ config */

static bool sampler_is_unset(const fg_sampler_config *s) {
    return s->temperature == 0.0f && s->top_p == 0.0f && s->top_k == 0u && s->presence_penalty == 0.0f &&
           s->frequency_penalty == 0.0f && s->repetition_penalty == 0.0f && s->min_p == 0.0f;
}

static fg_status check_config(const fg_wire_limits *limits, const fg_output_config *config, fg_error *err) {
    if (!limits || !config || config->source_rank >= limits->rank_count ||
        config->destination_rank != limits->output_rank || config->session_slot >= limits->session_slots)
        return refuse(err, FG_ERR_FORMAT, "invalid output config route");
    if (!sampler_is_unset(&config->sampler) && fg_sampler_config_validate(&config->sampler, err) != FG_OK)
        return FG_ERR_FORMAT;
    if (!isfinite(config->uniform) || config->uniform < 0.0f || config->uniform >= 1.0f)
        return refuse(err, FG_ERR_FORMAT, "invalid output config sampler draw");
    return FG_OK;
}

fg_status fg_output_config_encode_with(const fg_wire_limits *limits, uint8_t output[FG_OUTPUT_CONFIG_BYTES],
                                       const fg_output_config *config, fg_error *err) {
    if (!output) return refuse(err, FG_ERR_ARGUMENT, "output config buffer is null");
    const fg_status status = check_config(limits, config, err);
    if (status != FG_OK) return status;
    pack(output, config, config_fields, COUNT(config_fields));
    return FG_OK;
}

fg_status fg_output_config_decode_with(const fg_wire_limits *limits, fg_output_config *config,
                                       const uint8_t *payload, uint32_t bytes, fg_error *err) {
    if (!config || !payload) return refuse(err, FG_ERR_ARGUMENT, "invalid output config input");
    const uint8_t known = FG_OUTPUT_CONFIG_FLAG_SPLIT | FG_OUTPUT_CONFIG_FLAG_SPLIT_4;
    const bool four_without_split = bytes == FG_OUTPUT_CONFIG_BYTES &&
                                    (payload[2] & FG_OUTPUT_CONFIG_FLAG_SPLIT_4) &&
                                    !(payload[2] & FG_OUTPUT_CONFIG_FLAG_SPLIT);
    if (bytes != FG_OUTPUT_CONFIG_BYTES || (payload[2] & ~known) || four_without_split)
        return refuse(err, FG_ERR_FORMAT, "invalid output config size or reserved bytes");
    memset(config, 0, sizeof(*config));
    unpack(config, payload, config_fields, COUNT(config_fields));
    return check_config(limits, config, err);
}

/* ------------------------------------------------------------------ result */

static fg_status check_result(const fg_wire_limits *limits, const fg_output_result *result, fg_error *err) {
    if (!limits || !result || result->source_rank != limits->output_rank ||
        result->destination_rank >= limits->rank_count || result->token >= limits->vocab ||
        !isfinite(result->logit))
        return refuse(err, FG_ERR_FORMAT, "invalid output result");
    return FG_OK;
}

fg_status fg_output_result_encode_with(const fg_wire_limits *limits, uint8_t output[FG_OUTPUT_RESULT_BYTES],
                                       const fg_output_result *result, fg_error *err) {
    if (!output) return refuse(err, FG_ERR_ARGUMENT, "output result buffer is null");
    const fg_status status = check_result(limits, result, err);
    if (status != FG_OK) return status;
    memset(output, 0, FG_OUTPUT_RESULT_BYTES);
    pack(output, result, result_fields, COUNT(result_fields));
    return FG_OK;
}

fg_status fg_output_result_decode_with(const fg_wire_limits *limits, fg_output_result *result,
                                       const uint8_t *payload, uint32_t bytes, fg_error *err) {
    if (!result || !payload) return refuse(err, FG_ERR_ARGUMENT, "invalid output result input");
    if (bytes != FG_OUTPUT_RESULT_BYTES || payload[2] || payload[3])
        return refuse(err, FG_ERR_FORMAT, "invalid output result size or reserved bytes");
    memset(result, 0, sizeof(*result));
    unpack(result, payload, result_fields, COUNT(result_fields));
    return check_result(limits, result, err);
}

/* ----------------------------------------------------------------- partial */

static fg_status check_partial(const fg_wire_limits *limits, const fg_output_partial *partial, fg_error *err) {
    if (!limits || !partial || partial->id >= limits->vocab || !isfinite(partial->value))
        return refuse(err, FG_ERR_FORMAT, "invalid output partial");
    return FG_OK;
}

fg_status fg_output_partial_encode_with(const fg_wire_limits *limits, uint8_t output[FG_OUTPUT_PARTIAL_BYTES],
                                        const fg_output_partial *partial, fg_error *err) {
    if (!output) return refuse(err, FG_ERR_ARGUMENT, "output partial buffer is null");
    const fg_status status = check_partial(limits, partial, err);
    if (status != FG_OK) return status;
    pack(output, partial, partial_fields, COUNT(partial_fields));
    return FG_OK;
}

fg_status fg_output_partial_decode_with(const fg_wire_limits *limits, fg_output_partial *partial,
                                        const uint8_t *payload, uint32_t bytes, fg_error *err) {
    if (!partial || !payload) return refuse(err, FG_ERR_ARGUMENT, "invalid output partial input");
    if (bytes != FG_OUTPUT_PARTIAL_BYTES) return refuse(err, FG_ERR_FORMAT, "invalid output partial size");
    memset(partial, 0, sizeof(*partial));
    unpack(partial, payload, partial_fields, COUNT(partial_fields));
    return check_partial(limits, partial, err);
}

/* ----------------------------------------------------------------- history */

/* count (u32), session slot (u8), three reserved bytes, then count tokens */
fg_status fg_output_history_encode_with(const fg_wire_limits *limits, uint8_t *output, uint32_t capacity,
                                        uint32_t *bytes, const fg_output_history *history, fg_error *err) {
    if (!limits || !output || !bytes || !history || history->count > FG_NATIVE_CONTEXT ||
        (history->count && !history->tokens) || history->session_slot >= limits->session_slots)
        return refuse(err, FG_ERR_ARGUMENT, "invalid output history");
    const uint64_t needed = FG_OUTPUT_HISTORY_HEADER_BYTES + (uint64_t)history->count * 4u;
    if (needed > capacity || needed > FG_WIRE_MAX_FRAME_BYTES)
        return refuse(err, FG_ERR_LIMIT, "output history buffer is too small");
    store_be32(output, history->count);
    output[4] = history->session_slot;
    output[5] = output[6] = output[7] = 0u;
    uint8_t *cursor = output + FG_OUTPUT_HISTORY_HEADER_BYTES;
    for (uint32_t i = 0; i < history->count; i++, cursor += 4) {
        if (history->tokens[i] >= limits->vocab)
            return refuse(err, FG_ERR_FORMAT, "output history token is outside vocabulary");
        store_be32(cursor, history->tokens[i]);
    }
    *bytes = (uint32_t)needed;
    return FG_OK;
}

fg_status fg_output_history_decode_with(const fg_wire_limits *limits, fg_output_history *history,
                                        uint32_t *storage, uint32_t capacity, const uint8_t *payload,
                                        uint32_t bytes, fg_error *err) {
    if (!limits || !history || !payload || bytes < FG_OUTPUT_HISTORY_HEADER_BYTES)
        return refuse(err, FG_ERR_ARGUMENT, "invalid output history input");
    const uint32_t count = load_be32(payload);
    const uint8_t slot = payload[4];
    const bool reserved = payload[5] || payload[6] || payload[7];
    const uint64_t needed = FG_OUTPUT_HISTORY_HEADER_BYTES + (uint64_t)count * 4u;
    if (reserved || slot >= limits->session_slots || count > FG_NATIVE_CONTEXT || count > capacity ||
        needed != bytes || (count && !storage))
        return refuse(err, FG_ERR_FORMAT, "invalid output history size or reserved bytes");
    const uint8_t *cursor = payload + FG_OUTPUT_HISTORY_HEADER_BYTES;
    for (uint32_t i = 0; i < count; i++, cursor += 4) {
        const uint32_t token = load_be32(cursor);
        if (token >= limits->vocab)
            return refuse(err, FG_ERR_FORMAT, "output history token is outside vocabulary");
        storage[i] = token;
    }
    history->tokens = storage;
    history->count = count;
    history->session_slot = slot;
    return FG_OK;
}

/* ------------------------------------------- the reference's own signatures */

#define WITH_REFERENCE_LIMITS const fg_wire_limits limits = fg_wire_limits_reference()

fg_status fg_output_config_encode(uint8_t output[FG_OUTPUT_CONFIG_BYTES], const fg_output_config *config,
                                  fg_error *err) {
    WITH_REFERENCE_LIMITS;
    return fg_output_config_encode_with(&limits, output, config, err);
}
fg_status fg_output_config_decode(fg_output_config *config, const uint8_t *payload, uint32_t bytes,
                                  fg_error *err) {
    WITH_REFERENCE_LIMITS;
    return fg_output_config_decode_with(&limits, config, payload, bytes, err);
}
fg_status fg_output_result_encode(uint8_t output[FG_OUTPUT_RESULT_BYTES], const fg_output_result *result,
                                  fg_error *err) {
    WITH_REFERENCE_LIMITS;
    return fg_output_result_encode_with(&limits, output, result, err);
}
fg_status fg_output_result_decode(fg_output_result *result, const uint8_t *payload, uint32_t bytes,
                                  fg_error *err) {
    WITH_REFERENCE_LIMITS;
    return fg_output_result_decode_with(&limits, result, payload, bytes, err);
}
fg_status fg_output_partial_encode(uint8_t output[FG_OUTPUT_PARTIAL_BYTES], const fg_output_partial *partial,
                                   fg_error *err) {
    WITH_REFERENCE_LIMITS;
    return fg_output_partial_encode_with(&limits, output, partial, err);
}
fg_status fg_output_partial_decode(fg_output_partial *partial, const uint8_t *payload, uint32_t bytes,
                                   fg_error *err) {
    WITH_REFERENCE_LIMITS;
    return fg_output_partial_decode_with(&limits, partial, payload, bytes, err);
}
fg_status fg_output_history_encode(uint8_t *output, uint32_t capacity, uint32_t *bytes,
                                   const fg_output_history *history, fg_error *err) {
    WITH_REFERENCE_LIMITS;
    return fg_output_history_encode_with(&limits, output, capacity, bytes, history, err);
}
fg_status fg_output_history_decode(fg_output_history *history, uint32_t *storage, uint32_t capacity,
                                   const uint8_t *payload, uint32_t bytes, fg_error *err) {
    WITH_REFERENCE_LIMITS;
    return fg_output_history_decode_with(&limits, history, storage, capacity, payload, bytes, err);
}

/* ------------------------------------------------------------- split layout */

/* Slice 0 always stays on the output owner (rank 4); the others go to ranks 0, 1, 2 in
 * that order.  Two ways: rows [0, 140,048) and the rest.  Four ways: equal quarters, the
 * last one takes the remainder. */
static const uint32_t split_ranks[FG_OUTPUT_SPLIT_WAYS_MAX] = {4u, 0u, 1u, 2u};

bool fg_output_split_way_for_rank(uint32_t ways, uint32_t rank, uint32_t *way) {
    if (ways != FG_OUTPUT_SPLIT_WAYS_MIN && ways != FG_OUTPUT_SPLIT_WAYS_MAX) return false;
    for (uint32_t slot = 0; slot < ways; slot++) {
        if (split_ranks[slot] != rank) continue;
        if (way) *way = slot;
        return true;
    }
    return false;
}

uint32_t fg_output_split_rank(uint32_t ways, uint32_t way) {
    if ((ways == FG_OUTPUT_SPLIT_WAYS_MIN || ways == FG_OUTPUT_SPLIT_WAYS_MAX) && way < ways)
        return split_ranks[way];
    return UINT32_MAX;  /* no such slice (src/protocol.c:39-44) */
}

void fg_output_split_span(uint32_t ways, uint32_t way, uint32_t *first_row, uint32_t *rows) {
    const uint32_t vocab = fg_wire_limits_reference().vocab;
    uint32_t first = 0u, count = 0u;
    if (ways == FG_OUTPUT_SPLIT_WAYS_MIN && way < 2u) {
        first = way ? FG_OUTPUT_SPLIT_FIRST_ROWS : 0u;
        count = way ? vocab - FG_OUTPUT_SPLIT_FIRST_ROWS : FG_OUTPUT_SPLIT_FIRST_ROWS;
    } else if (ways == FG_OUTPUT_SPLIT_WAYS_MAX && way < FG_OUTPUT_SPLIT_WAYS_MAX) {
        const uint32_t quarter = vocab / FG_OUTPUT_SPLIT_WAYS_MAX;
        first = way * quarter;
        count = way + 1u == FG_OUTPUT_SPLIT_WAYS_MAX ? vocab - first : quarter;
    }
    if (first_row) *first_row = first;
    if (rows) *rows = count;
}

/* ---------------------------------------------------------------- logit dump */

static const char dump_magic[8] = {'F', 'G', 'L', 'O', 'G', '0', '1', '\n'};

fg_status fg_logit_dump_read(const char *path, float *logits, uint32_t capacity, uint32_t *vocab,
                             bool check_finite, fg_error *err) {
    if (!path || !vocab) return refuse(err, FG_ERR_ARGUMENT, "invalid logit dump arguments");
    FILE *file = fopen(path, "rb");
    if (!file) {
        fg_error_set(err, FG_ERR_IO, "cannot open logit dump: %s", path);
        return FG_ERR_IO;
    }
    uint8_t head[12];
    fg_status status = FG_OK;
    if (fread(head, 1u, sizeof(head), file) != sizeof(head) || memcmp(head, dump_magic, 8) != 0) {
        fg_error_set(err, FG_ERR_FORMAT, "bad logit dump header: %s", path);
        status = FG_ERR_FORMAT;
    }
    uint32_t count = 0;
    if (status == FG_OK) {
        count = (uint32_t)head[8] | ((uint32_t)head[9] << 8) | ((uint32_t)head[10] << 16) | ((uint32_t)head[11] << 24);
        *vocab = count;
        if (fseek(file, 0, SEEK_END) != 0 || ftell(file) != (long)(12u + (uint64_t)count * 4u)) {
            fg_error_set(err, FG_ERR_FORMAT, "logit dump %s does not hold %u logits", path, count);
            status = FG_ERR_FORMAT;
        }
    }
    if (status == FG_OK && logits) {
        if (count > capacity) {
            fg_error_set(err, FG_ERR_LIMIT, "logit dump holds %u logits, room for %u", count, capacity);
            status = FG_ERR_LIMIT;
        } else if (fseek(file, 12, SEEK_SET) != 0) {
            fg_error_set(err, FG_ERR_IO, "cannot read logit dump: %s", path);
            status = FG_ERR_IO;
        } else {
            for (uint32_t i = 0; i < count && status == FG_OK; i++) {
                uint8_t raw[4];
                if (fread(raw, 1u, 4u, file) != 4u) {
                    fg_error_set(err, FG_ERR_IO, "cannot read logit dump: %s", path);
                    status = FG_ERR_IO;
                    break;
                }
                const uint32_t word = (uint32_t)raw[0] | ((uint32_t)raw[1] << 8) | ((uint32_t)raw[2] << 16) |
                                      ((uint32_t)raw[3] << 24);
                memcpy(&logits[i], &word, 4);
                if (check_finite && !isfinite(logits[i])) {
                    fg_error_set(err, FG_ERR_FORMAT, "non-finite logit %u in %s", i, path);
                    status = FG_ERR_FORMAT;
                }
            }
        }
    }
    fclose(file);
    return status;
}

fg_status fg_logit_dump_write(const char *path, const float *logits, uint32_t vocab, fg_error *err) {
    if (!path || !logits || !vocab) return refuse(err, FG_ERR_ARGUMENT, "invalid logit dump arguments");
    FILE *file = fopen(path, "wb");
    bool written = file && fwrite(dump_magic, 1u, 8u, file) == 8u;
    const uint8_t size[4] = {(uint8_t)vocab, (uint8_t)(vocab >> 8), (uint8_t)(vocab >> 16), (uint8_t)(vocab >> 24)};
    written = written && fwrite(size, 1u, 4u, file) == 4u;
    for (uint32_t i = 0; written && i < vocab; i++) {
        uint32_t word;
        memcpy(&word, &logits[i], 4);
        const uint8_t raw[4] = {(uint8_t)word, (uint8_t)(word >> 8), (uint8_t)(word >> 16), (uint8_t)(word >> 24)};
        written = fwrite(raw, 1u, 4u, file) == 4u;
    }
    if (file && fclose(file) != 0) written = false;
    if (!written) {
        fg_error_set(err, FG_ERR_IO, "cannot write logit dump: %s", path);
        return FG_ERR_IO;
    }
    return FG_OK;
}
