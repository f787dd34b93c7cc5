/*
 * Core status and error types shared by every entry point of the sampler
 * library.  ABI-compatible with the reference's include/fg.h:45-62: the
 * numeric values of fg_status and the layout of fg_error (status word followed
 * by a 512-byte message) are what existing callers were compiled against.
 * Only the parts the token-sampling path needs are declared here.
 */
#ifndef FG_B200_CORE_H
#define FG_B200_CORE_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Longest token history a penalty table accepts (reference include/fg.h:25,
 * enforced at src/output.c:604). */
#define FG_NATIVE_CONTEXT 262144u

/* Status codes; the gap at 1 is part of the ABI (reference include/fg.h:45-55). */
typedef enum fg_status {
    FG_OK              = 0,
    FG_ERR_ARGUMENT    = 2,
    FG_ERR_IO          = 3,
    FG_ERR_FORMAT      = 4,
    FG_ERR_MISMATCH    = 5,
    FG_ERR_OOM         = 6,
    FG_ERR_UNAVAILABLE = 7,
    FG_ERR_LIMIT       = 8,
    FG_ERR_INTERRUPTED = 9
} fg_status;

/* Optional out-parameter of every fallible call; may be NULL
 * (reference include/fg.h:57-60, src/util.c:6). */
typedef struct fg_error {
    fg_status code;
    char message[512];
} fg_error;

/* printf-style setter; a NULL err is ignored.  Replaces src/util.c:6. */
void fg_error_set(fg_error *err, fg_status code, const char *fmt, ...);
/* Replace src/util.c:7-8; kept so objects built against the reference header link. */
uint64_t fg_align_up_u64(uint64_t value, uint64_t alignment);
bool fg_is_aligned_u64(uint64_t value, uint64_t alignment);

#ifdef __cplusplus
}
#endif

#endif /* FG_B200_CORE_H */
