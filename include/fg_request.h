/*
 * The request-level validation surface of the sampling path: the sampler fields of a chat
 * completion request (a JSON object) become a fg_sampler_config, with the reference's
 * ranges, defaults and error texts.
 *
 * Restates parse_sampler_controls of the reference's HTTP front end (src/api.c:1606-1631;
 * documented in README.md:149-159; its tests are tests/test_api.c:1000-1064).  That function
 * is private to the reference's api.c and takes its own JSON tree; here the entry point
 * takes the request body's bytes, so that a front end written in anything can call it.
 */
#ifndef FG_B200_REQUEST_H
#define FG_B200_REQUEST_H

#include <stddef.h>

#include "fg.h"
#include "fg_sampler.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Reads the top-level members "temperature", "top_p", "top_k", "seed", "presence_penalty",
 * "frequency_penalty", "repetition_penalty" and "min_p" of the JSON object in
 * json[0..bytes) into *config; members that are absent keep the defaults (temperature 1.0,
 * top_p 0.95, top_k 20, no penalties); every other member is skipped, whatever its value.
 * When a member occurs twice the first one counts, as in the reference's object lookup.
 *
 * FG_ERR_ARGUMENT with the reference's message when a field has the wrong type or range:
 *   temperature   finite number >= 0           "temperature must be a finite non-negative number"
 *   top_p         0 < number <= 1              "top_p must be greater than 0 and at most 1"
 *   top_k         integer 1 .. 64              "top_k must be an integer from 1 through 64"
 *   seed          integer 0 .. 2^53 - 1        "seed must be a non-negative integer"
 *   *_penalty     finite number                "... must be finite"
 *   min_p         exactly 0                    "min_p currently supports only 0"
 * and then whatever fg_sampler_config_validate says about the whole (penalties outside
 * [-2, 2], repetition <= 0: "invalid sampler controls").  FG_ERR_FORMAT when the bytes are
 * not a JSON object. */
fg_status fg_sampler_config_from_json(const char *json, size_t bytes, fg_sampler_config *config,
                                      fg_error *err);

#ifdef __cplusplus
}
#endif

#endif /* FG_B200_REQUEST_H */
