/*
 * Error record and alignment helpers of the core header.
 * Behaviour of the reference's src/util.c:6-8: a NULL error record is ignored,
 * the message is truncated to the 512-byte field, alignment 0 is a no-op.
 */
#include "fg.h"

#include <stdarg.h>
#include <stdio.h>

void fg_error_set(fg_error *err, fg_status code, const char *fmt, ...) {
    if (!err) return;
    err->code = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err->message, sizeof(err->message), fmt, ap);
    va_end(ap);
}

uint64_t fg_align_up_u64(uint64_t value, uint64_t alignment) {
    return alignment ? (value + (alignment - 1u)) & ~(alignment - 1u) : value;
}

bool fg_is_aligned_u64(uint64_t value, uint64_t alignment) {
    return alignment != 0u && (value & (alignment - 1u)) == 0u;
}
