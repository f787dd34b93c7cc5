/*
 * Token sampler: the drop-in surface.  Same eight functions, same two structs
 * and the same argument meaning as the reference's include/fg_sampler.h:6-32
 * (implementation there: src/sampler.c).  All pointers are HOST pointers.
 *
 * What runs where in this library:
 *   - config_greedy / config_defaults / config_validate / penalties_active and
 *     the xorshift64* stream (state_init / uniform) are plain host C: they are
 *     request set-up, drawn once per token on the coordinator.
 *   - apply_penalties and select stage their (small) inputs to the GPU, run
 *     the CUDA kernels and copy the result back.  There is no CPU arithmetic
 *     path: without a usable CUDA device apply_penalties leaves the scores
 *     untouched and reports through fg_sampler_last_status(), and select
 *     returns FG_ERR_UNAVAILABLE.
 * Batched, device-resident sampling lives in fg_cuda_sampler.h.
 */
#ifndef FG_B200_SAMPLER_H
#define FG_B200_SAMPLER_H

#include "fg.h"

#ifdef __cplusplus
extern "C" {
#endif

/* 40 bytes, natural alignment: seven 4-byte fields, 4 bytes of padding, then
 * the 8-byte seed (reference include/fg_sampler.h:6-15).  The same 40 bytes
 * travel on the reference's wire (include/fg_protocol.h:39,46). */
typedef struct fg_sampler_config {
    float    temperature;        /* 0 selects greedy argmax                    */
    float    top_p;              /* (0, 1]                                      */
    uint32_t top_k;              /* 1..64                                       */
    float    presence_penalty;   /* [-2, 2], subtracted once from seen ids      */
    float    frequency_penalty;  /* [-2, 2], times the occurrence count         */
    float    repetition_penalty; /* > 0, divides positive / multiplies others   */
    float    min_p;              /* must be exactly 0                           */
    uint64_t seed;               /* seed of the per-request uniform stream      */
} fg_sampler_config;

/* Caller-owned xorshift64* state (reference include/fg_sampler.h:17-19). */
typedef struct fg_sampler_state {
    uint64_t state;
} fg_sampler_state;

/* Replaces src/sampler.c:8-14. */
void fg_sampler_config_greedy(fg_sampler_config *config);
/* Replaces src/sampler.c:16-22. */
void fg_sampler_config_defaults(fg_sampler_config *config);
/* Replaces src/sampler.c:24-38. */
fg_status fg_sampler_config_validate(const fg_sampler_config *config, fg_error *err);
/* Replaces src/sampler.c:62-65. */
void fg_sampler_state_init(fg_sampler_state *state, uint64_t seed);
/* Replaces src/sampler.c:67-73. */
float fg_sampler_uniform(fg_sampler_state *state);
/* Replaces src/sampler.c:80-122; sort, softmaxes and inverse CDF run on the GPU. */
fg_status fg_sampler_select(const fg_sampler_config *config,
                            const float *scores, const uint32_t *ids, uint32_t count,
                            float uniform, uint32_t *token, float *logit, fg_error *err);
/* Replaces src/sampler.c:40-44. */
bool fg_sampler_penalties_active(const fg_sampler_config *config);
/* Replaces src/sampler.c:46-60; the per-score arithmetic runs on the GPU. */
void fg_sampler_apply_penalties(float *scores, const uint32_t *ids,
                                const uint32_t *counts, uint32_t count,
                                const fg_sampler_config *config);

/* No counterpart in the reference: fg_sampler_apply_penalties returns void, so
 * a device failure inside it is reported here (status of the most recent
 * host-pointer call made by this thread; FG_OK after a successful one). */
fg_status fg_sampler_last_status(void);

#ifdef __cplusplus
}
#endif

#endif /* FG_B200_SAMPLER_H */
