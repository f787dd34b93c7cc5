/*
 * TEST INFRASTRUCTURE — CPU restatement of the argmax total order of the
 * reference's output executor (src/output.c:484-498), which is also the
 * `before()` of shaders/fg_argmax_reduce.comp:14-24.  Checker only; never
 * linked into the product library.  The reference build of the oracle
 * (oracle/_ref) links the reference's own object instead of this file.
 */
#include <math.h>
#include <stdbool.h>
#include <stdint.h>

#define PORT_PADDING_ID 0xffffffffu

/* src/output.c:484-492.  Padding loses to anything real; a NaN or infinity
 * beats every finite score; two non-finite scores are ordered by id alone;
 * finite scores by value, then by the smaller id. */
bool fg_output_better(float left, uint32_t left_id, float right, uint32_t right_id) {
    const bool left_pad = left_id == PORT_PADDING_ID;
    const bool right_pad = right_id == PORT_PADDING_ID;
    if (left_pad) return false;
    if (right_pad) return true;
    const bool left_wild = !isfinite(left);
    const bool right_wild = !isfinite(right);
    if (left_wild && right_wild) return left_id < right_id;
    if (left_wild) return true;
    if (right_wild) return false;
    if (left > right) return true;
    return left == right && left_id < right_id;
}

/* src/output.c:494-498. */
void fg_output_combine(float left, uint32_t left_id, float right, uint32_t right_id,
                       float *value, uint32_t *id) {
    const bool take_left = fg_output_better(left, left_id, right, right_id);
    if (value) *value = take_left ? left : right;
    if (id) *id = take_left ? left_id : right_id;
}
