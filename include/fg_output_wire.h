/*
 * Wire and file formats on either side of the sampling path, so that a reference
 * coordinator can talk to this sampler and recorded logits can be replayed through it.
 *
 * Same structs, function names, byte layouts and fail-closed checks as the reference's
 * codecs for the output messages (include/fg_protocol.h:449-498, 566-571, 744-759;
 * src/protocol.c:1156-1166 config, 1275-1281 result, 1283-1289 partial, 1328-1367 history;
 * split spans src/protocol.c:23-37, 93-105) and its full-vocabulary logit dump
 * (src/output.c:568-591, read back by tools/q4_quality.py:45-58).  All integers and floats
 * are big-endian on the wire; the dump file is little-endian.
 *
 * The reference fixes the deployment's numbers at compile time (8 ranks, the output owner
 * is rank 4, 2 session slots, a 248,320-token vocabulary).  The functions with the
 * reference's names use exactly those; the *_with variants take a fg_wire_limits so that a
 * deployment with another vocabulary or rank layout can use the same codecs.
 */
#ifndef FG_B200_OUTPUT_WIRE_H
#define FG_B200_OUTPUT_WIRE_H

#include "fg.h"
#include "fg_sampler.h"

#ifdef __cplusplus
extern "C" {
#endif

#define FG_OUTPUT_CONFIG_BYTES 40u          /* include/fg_protocol.h:39,46 */
#define FG_OUTPUT_RESULT_BYTES 16u          /* include/fg_protocol.h:41 */
#define FG_OUTPUT_PARTIAL_BYTES 12u         /* include/fg_protocol.h:483 */
#define FG_OUTPUT_HISTORY_HEADER_BYTES 8u   /* include/fg_protocol.h:47 */
#define FG_OUTPUT_HISTORY_MAX_BYTES (FG_OUTPUT_HISTORY_HEADER_BYTES + FG_NATIVE_CONTEXT * 4u)
#define FG_OUTPUT_CONFIG_FLAG_SPLIT 1u      /* include/fg_protocol.h:480-481 */
#define FG_OUTPUT_CONFIG_FLAG_SPLIT_4 2u
#define FG_OUTPUT_SPLIT_FIRST_ROWS 140048u  /* include/fg_protocol.h:484-486 */
#define FG_OUTPUT_SPLIT_WAYS_MIN 2u
#define FG_OUTPUT_SPLIT_WAYS_MAX 4u
#define FG_WIRE_MAX_FRAME_BYTES (64u * 1024u * 1024u) /* include/fg_protocol.h:10 */

/* What the reference's codecs check messages against. */
typedef struct fg_wire_limits {
    uint32_t rank_count;     /* 8   (include/fg.h:13) */
    uint32_t output_rank;    /* 4   (include/fg_output.h:15-18) */
    uint32_t session_slots;  /* 2   (include/fg_protocol.h:32) */
    uint32_t vocab;          /* 248,320 (include/fg_q38_schema.h:6) */
} fg_wire_limits;
/* The reference deployment's numbers. */
fg_wire_limits fg_wire_limits_reference(void);

/* FG_MSG_OUTPUT_CONFIG: the sampler controls and the uniform draw of one token, sent by the
 * coordinator to the output owner (include/fg_protocol.h:469-478). */
typedef struct fg_output_config {
    uint8_t source_rank;
    uint8_t destination_rank;
    uint8_t flags;
    uint8_t session_slot;
    uint32_t token_index;
    fg_sampler_config sampler;
    float uniform;
} fg_output_config;

/* FG_MSG_OUTPUT_RESULT: the sampled token on its way back (include/fg_protocol.h:461-467). */
typedef struct fg_output_result {
    uint8_t source_rank;
    uint8_t destination_rank;
    uint32_t token_index;
    uint32_t token;
    float logit;
} fg_output_result;

/* FG_MSG_OUTPUT_PARTIAL: one slice's argmax finalist (include/fg_protocol.h:494-498). */
typedef struct fg_output_partial {
    uint32_t token_index;
    float value;
    uint32_t id;
} fg_output_partial;

/* FG_MSG_OUTPUT_HISTORY: a session's token history for the penalties
 * (include/fg_protocol.h:566-571). */
typedef struct fg_output_history {
    const uint32_t *tokens;
    uint32_t count;
    uint8_t session_slot;
} fg_output_history;

/* An all-zero sampler block means "unset" and is let through; any other must pass
 * fg_sampler_config_validate; the draw must be finite in [0, 1) (src/protocol.c:1160). */
fg_status fg_output_config_encode(uint8_t output[FG_OUTPUT_CONFIG_BYTES], const fg_output_config *config,
                                  fg_error *err);
fg_status fg_output_config_decode(fg_output_config *config, const uint8_t *payload, uint32_t bytes,
                                  fg_error *err);
fg_status fg_output_result_encode(uint8_t output[FG_OUTPUT_RESULT_BYTES], const fg_output_result *result,
                                  fg_error *err);
fg_status fg_output_result_decode(fg_output_result *result, const uint8_t *payload, uint32_t bytes,
                                  fg_error *err);
fg_status fg_output_partial_encode(uint8_t output[FG_OUTPUT_PARTIAL_BYTES], const fg_output_partial *partial,
                                   fg_error *err);
fg_status fg_output_partial_decode(fg_output_partial *partial, const uint8_t *payload, uint32_t bytes,
                                   fg_error *err);
fg_status fg_output_history_encode(uint8_t *output, uint32_t capacity, uint32_t *bytes,
                                   const fg_output_history *history, fg_error *err);
/* `storage` (capacity tokens) receives the tokens; history->tokens points into it. */
fg_status fg_output_history_decode(fg_output_history *history, uint32_t *storage, uint32_t capacity,
                                   const uint8_t *payload, uint32_t bytes, fg_error *err);

/* The same codecs against other limits. */
fg_status fg_output_config_encode_with(const fg_wire_limits *limits, uint8_t output[FG_OUTPUT_CONFIG_BYTES],
                                       const fg_output_config *config, fg_error *err);
fg_status fg_output_config_decode_with(const fg_wire_limits *limits, fg_output_config *config,
                                       const uint8_t *payload, uint32_t bytes, fg_error *err);
fg_status fg_output_result_encode_with(const fg_wire_limits *limits, uint8_t output[FG_OUTPUT_RESULT_BYTES],
                                       const fg_output_result *result, fg_error *err);
fg_status fg_output_result_decode_with(const fg_wire_limits *limits, fg_output_result *result,
                                       const uint8_t *payload, uint32_t bytes, fg_error *err);
fg_status fg_output_partial_encode_with(const fg_wire_limits *limits, uint8_t output[FG_OUTPUT_PARTIAL_BYTES],
                                        const fg_output_partial *partial, fg_error *err);
fg_status fg_output_partial_decode_with(const fg_wire_limits *limits, fg_output_partial *partial,
                                        const uint8_t *payload, uint32_t bytes, fg_error *err);
fg_status fg_output_history_encode_with(const fg_wire_limits *limits, uint8_t *output, uint32_t capacity,
                                        uint32_t *bytes, const fg_output_history *history, fg_error *err);
fg_status fg_output_history_decode_with(const fg_wire_limits *limits, fg_output_history *history,
                                        uint32_t *storage, uint32_t capacity, const uint8_t *payload,
                                        uint32_t bytes, fg_error *err);

/* The split output head's layout (src/protocol.c:23-37, 93-105): which slice a rank runs,
 * which rank runs a slice, and a slice's vocabulary rows. */
bool fg_output_split_way_for_rank(uint32_t ways, uint32_t rank, uint32_t *way);
uint32_t fg_output_split_rank(uint32_t ways, uint32_t way);
void fg_output_split_span(uint32_t ways, uint32_t way, uint32_t *first_row, uint32_t *rows);

/* The full-vocabulary logit dump the reference's output executor writes when
 * FG_EVAL_LOGITS[_DIR] is set (src/output.c:568-591): "FGLOG01\n", a little-endian uint32
 * vocabulary size, then that many little-endian fp32 logits.
 * fg_logit_dump_read: reads `path`; *vocab gets the size; when `logits` is not NULL it must
 * have room for `capacity` values and receives them.  FG_ERR_IO when the file cannot be
 * read, FG_ERR_FORMAT for a bad header, size or (when check_finite) a NaN/Inf,
 * FG_ERR_LIMIT when capacity is too small. */
fg_status fg_logit_dump_read(const char *path, float *logits, uint32_t capacity, uint32_t *vocab,
                             bool check_finite, fg_error *err);
fg_status fg_logit_dump_write(const char *path, const float *logits, uint32_t vocab, fg_error *err);

#ifdef __cplusplus
}
#endif

#endif /* FG_B200_OUTPUT_WIRE_H */
