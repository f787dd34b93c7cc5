/*
 * TEST INFRASTRUCTURE: drives the host-only C of the library (wire codecs, logit dump,
 * request parser) with seeded random and mutated inputs under AddressSanitizer and
 * UndefinedBehaviorSanitizer.  Built and run by tests/test_cpu_sanitizers.py; a finding makes
 * the process abort.  The decoders must fail closed on anything, never read past `bytes`.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "fg_output_wire.h"
#include "fg_request.h"

static uint64_t state = 0x9e3779b97f4a7c15ull;
static uint32_t next(void) {
    state ^= state >> 12;
    state ^= state << 25;
    state ^= state >> 27;
    return (uint32_t)((state * 2685821657736338717ull) >> 32);
}

int main(void) {
    fg_error err;
    unsigned accepted = 0, refused = 0;
    /* fixed-size messages: exact-size heap buffers so that one byte too far is caught */
    for (int round = 0; round < 20000; round++) {
        const uint32_t sizes[] = {0, 1, 11, 12, 13, 15, 16, 17, 39, 40, 41, 64};
        const uint32_t bytes = sizes[next() % (sizeof(sizes) / sizeof(sizes[0]))];
        uint8_t *payload = malloc(bytes ? bytes : 1);
        for (uint32_t i = 0; i < bytes; i++) payload[i] = (uint8_t)(next() % 7 ? next() : next() % 6);
        fg_output_config config;
        fg_output_result result;
        fg_output_partial partial;
        memset(&err, 0, sizeof(err));
        if (fg_output_config_decode(&config, payload, bytes, &err) == FG_OK) {
            uint8_t again[FG_OUTPUT_CONFIG_BYTES];
            if (fg_output_config_encode(again, &config, &err) != FG_OK || memcmp(again, payload, sizeof(again)) != 0) {
                fprintf(stderr, "config round trip differs\n");
                return 1;
            }
            accepted++;
        } else {
            refused++;
        }
        if (fg_output_result_decode(&result, payload, bytes, &err) == FG_OK) {
            uint8_t again[FG_OUTPUT_RESULT_BYTES];
            if (fg_output_result_encode(again, &result, &err) != FG_OK || memcmp(again, payload, sizeof(again)) != 0) {
                fprintf(stderr, "result round trip differs\n");
                return 1;
            }
            accepted++;
        }
        if (fg_output_partial_decode(&partial, payload, bytes, &err) == FG_OK) accepted++;
        free(payload);
    }
    /* histories: header says anything, storage is exactly as long as claimed */
    for (int round = 0; round < 5000; round++) {
        const uint32_t count = next() % 40;
        const uint32_t bytes = next() % 3 ? 8 + count * 4 : next() % 200;
        uint8_t *payload = malloc(bytes ? bytes : 1);
        for (uint32_t i = 0; i < bytes; i++) payload[i] = (uint8_t)next();
        if (bytes >= 8 && next() % 2) {
            payload[0] = payload[1] = payload[2] = 0;
            payload[3] = (uint8_t)count;
            payload[4] = (uint8_t)(next() % 3);
            payload[5] = payload[6] = payload[7] = (uint8_t)(next() % 5 == 0);
            for (uint32_t i = 8; i + 3 < bytes; i += 4) payload[i] = payload[i + 1] = 0;
        }
        const uint32_t capacity = next() % 48;
        uint32_t *storage = malloc(capacity ? capacity * 4 : 1);
        fg_output_history history;
        memset(&err, 0, sizeof(err));
        if (fg_output_history_decode(&history, storage, capacity, payload, bytes, &err) == FG_OK) {
            uint8_t *again = malloc(bytes);
            uint32_t used = 0;
            if (fg_output_history_encode(again, bytes, &used, &history, &err) != FG_OK || used != bytes ||
                memcmp(again, payload, bytes) != 0) {
                fprintf(stderr, "history round trip differs\n");
                return 1;
            }
            free(again);
            accepted++;
        } else {
            refused++;
        }
        free(storage);
        free(payload);
    }
    /* request bodies: a valid body with random single-byte damage and random truncation */
    const char *body = "{\"model\":\"m\",\"temperature\":0.7,\"top_p\":0.8,\"top_k\":20,\"seed\":7,\"min_p\":0,"
                       "\"presence_penalty\":1.5,\"frequency_penalty\":-0.25,\"repetition_penalty\":1.05,"
                       "\"messages\":[{\"role\":\"user\",\"content\":\"a \\\"quoted\\\" \\u00e9 {[}] text\"}],"
                       "\"nested\":{\"top_k\":[1,2,{\"x\":null}],\"t\":true,\"f\":false,\"e\":1e-3}}";
    const size_t length = strlen(body);
    for (int round = 0; round < 40000; round++) {
        size_t bytes = next() % 4 ? length : next() % (length + 1);
        char *copy = malloc(bytes ? bytes : 1);
        memcpy(copy, body, bytes);
        for (uint32_t damage = next() % 4; damage && bytes; damage--) copy[next() % bytes] = (char)(next() % 96 + 32);
        fg_sampler_config config;
        memset(&err, 0, sizeof(err));
        const fg_status status = fg_sampler_config_from_json(copy, bytes, &config, &err);
        if (status == FG_OK) {
            if (fg_sampler_config_validate(&config, &err) != FG_OK) {
                fprintf(stderr, "accepted a config that does not validate\n");
                return 1;
            }
            accepted++;
        } else {
            refused++;
        }
        free(copy);
    }
    /* logit dumps: write, damage, read */
    char path[] = "/tmp/fg_fuzz_dump_XXXXXX";
    const int handle = mkstemp(path);
    if (handle >= 0) {
        float values[257];
        for (int i = 0; i < 257; i++) values[i] = (float)i * 0.5f - 60.0f;
        if (fg_logit_dump_write(path, values, 257, &err) != FG_OK) return 1;
        float back[257];
        uint32_t vocab = 0;
        if (fg_logit_dump_read(path, back, 257, &vocab, true, &err) != FG_OK || vocab != 257 ||
            memcmp(back, values, sizeof(values)) != 0)
            return 1;
        for (int round = 0; round < 200; round++) {
            FILE *file = fopen(path, "r+b");
            if (!file) break;
            fseek(file, (long)(next() % (12 + 257 * 4)), SEEK_SET);
            fputc((int)(next() & 0xff), file);
            fclose(file);
            float small[100];
            if (next() % 2) (void)fg_logit_dump_read(path, back, 257, &vocab, true, &err);
            else (void)fg_logit_dump_read(path, small, 100, &vocab, true, &err);
        }
        remove(path);
    }
    printf("accepted %u, refused %u\n", accepted, refused);
    return accepted > 0 && refused > 0 ? 0 : 1;
}
