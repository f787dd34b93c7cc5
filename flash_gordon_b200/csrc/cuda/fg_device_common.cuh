// Device-side building blocks shared by the sampling kernels (sm_100a).
//
// Everything here is exact integer / IEEE arithmetic: the orders, the penalty
// formula and the key mapping must agree bit for bit with the reference's C
// sampler (src/sampler.c) and argmax order (src/output.c:484-492).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fgk {

constexpr uint32_t kPaddingId = 0xffffffffu;
constexpr unsigned kFullMask = 0xffffffffu;
constexpr int kMaxK = 64;

__device__ __forceinline__ bool is_nonfinite(float v) {
    return (__float_as_uint(v) & 0x7f800000u) == 0x7f800000u;
}

// src/sampler.c:75-78 — the sampling order: larger score first, then smaller id.
__device__ __forceinline__ bool precedes(float a, uint32_t a_id, float b, uint32_t b_id) {
    return a > b || (a == b && a_id < b_id);
}

// src/output.c:484-492 / shaders/fg_argmax_reduce.comp:14-24 — the argmax order.
__device__ __forceinline__ bool argmax_before(float a, uint32_t a_id, float b, uint32_t b_id) {
    const bool a_pad = a_id == kPaddingId, b_pad = b_id == kPaddingId;
    if (a_pad || b_pad) return !a_pad && b_pad;
    const bool a_wild = is_nonfinite(a), b_wild = is_nonfinite(b);
    if (a_wild || b_wild) return a_wild != b_wild ? a_wild : a_id < b_id;
    return a > b || (a == b && a_id < b_id);
}

// src/sampler.c:52-58 for one seen id.  Round-to-nearest intrinsics keep nvcc
// from contracting frequency*count + presence into a fused multiply-add.
__device__ __forceinline__ float penalise(float v, uint32_t seen, float presence, float frequency,
                                          float repetition) {
    if (repetition != 1.0f) v = v > 0.0f ? __fdiv_rn(v, repetition) : __fmul_rn(v, repetition);
    const float offset = __fadd_rn(__fmul_rn(frequency, __uint2float_rn(seen)), presence);
    return __fsub_rn(v, offset);
}

// v / repetition without the special-function unit.  With r = RN(1/repetition),
// q = RN(v*r), e = v - q*repetition (exact in one FMA) and RN(q + e*r) is the
// correctly rounded quotient (Markstein); checked equal to IEEE division on
// 1.7e10 random and adversarial operand pairs on B200.  Operands whose exponent is
// far from 1 could overflow or go subnormal inside the sequence and take the
// IEEE-division instruction instead.
struct Repetition {
    float value;
    float reciprocal;
    bool active;   // value != 1
    bool tame;     // 2^-40 <= value <= 2^40
};

__device__ __forceinline__ Repetition make_repetition(float value) {
    Repetition r;
    r.value = value;
    r.reciprocal = __frcp_rn(value);
    r.active = value != 1.0f;
    r.tame = value >= 0x1p-40f && value <= 0x1p40f;
    return r;
}

// src/sampler.c:52-58 with the offset  frequency*count + presence  precomputed.
__device__ __forceinline__ float penalise_with_offset(float v, float offset, const Repetition &rep) {
    if (rep.active) {
        if (v > 0.0f) {
            if (rep.tame && v >= 0x1p-40f && v <= 0x1p40f) {
                const float q = __fmul_rn(v, rep.reciprocal);
                const float e = __fmaf_rn(-q, rep.value, v);
                v = __fmaf_rn(e, rep.reciprocal, q);
            } else {
                v = __fdiv_rn(v, rep.value);
            }
        } else {
            v = __fmul_rn(v, rep.value);
        }
    }
    return __fsub_rn(v, offset);
}

// frequency * (float)count + presence, as src/sampler.c:57-58 rounds it.
__device__ __forceinline__ float penalty_offset(uint32_t seen, float presence, float frequency) {
    return __fadd_rn(__fmul_rn(frequency, __uint2float_rn(seen)), presence);
}

// Monotone map finite fp32 -> uint32 (larger float, larger key); -0.0 and +0.0
// share a key because every comparator of the reference's C code treats them as
// equal and falls through to the id.  Key 0 is below every finite value.
__device__ __forceinline__ uint32_t float_key(float v) {
    uint32_t bits = __float_as_uint(v);
    if (bits == 0x80000000u) bits = 0u;
    return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

// Inverse of float_key for thresholds; key 0 means "below everything".
__device__ __forceinline__ float key_to_float(uint32_t key) {
    if (key == 0u) return __uint_as_float(0xff800000u);  // -inf
    const uint32_t bits = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
    return __uint_as_float(bits);
}

// 64-bit selection key: value key in the high word, inverted id in the low word,
// so "larger key" is exactly `precedes`.
__device__ __forceinline__ uint64_t select_key(float v, uint32_t id) {
    return (static_cast<uint64_t>(float_key(v)) << 32) | static_cast<uint64_t>(~id);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }

// 128-bit streaming load: read-only path, no L1 allocation (every logit is
// touched once).
__device__ __forceinline__ uint4 load_stream_128(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// ---- asynchronous bulk copies (the non-tensor form of TMA) and their mbarriers ----
// One thread asks the copy engine for `bytes` (a multiple of 16, both addresses
// 16-byte aligned) from global into this CTA's shared memory; completion is counted
// on an mbarrier the consumers poll.  No multicast anywhere.

__device__ __forceinline__ uint32_t shared_address(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbarrier_init(uint64_t *barrier, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(barrier)), "r"(arrivals));
}

__device__ __forceinline__ void mbarrier_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// the producer's arrival, announcing how many bytes the copy will deliver
__device__ __forceinline__ void mbarrier_expect(uint64_t *barrier, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(barrier)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbarrier_try_wait(uint64_t *barrier, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(shared_address(barrier)), "r"(parity)
        : "memory");
    return done != 0;
}

// The same, but the thread may sleep for up to `nanoseconds` while the phase is not
// complete: a warp that waits this way leaves the issue slots to the warps that work.
__device__ __forceinline__ bool mbarrier_try_wait_sleeping(uint64_t *barrier, uint32_t parity,
                                                           uint32_t nanoseconds) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(shared_address(barrier)), "r"(parity), "r"(nanoseconds)
        : "memory");
    return done != 0;
}

// Bounded wait: gives up after about a second's worth of polls and reports false, so
// a copy that never lands becomes an error status instead of a hung GPU.
__device__ __forceinline__ bool mbarrier_wait(uint64_t *barrier, uint32_t parity) {
    for (uint32_t polls = 0; polls < (1u << 22); polls++)
        if (mbarrier_try_wait(barrier, parity)) return true;
    return false;
}

__device__ __forceinline__ void bulk_copy_to_shared(void *shared_destination, const void *global_source,
                                                    uint32_t bytes, uint64_t *barrier) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            shared_address(shared_destination)),
        "l"(global_source), "r"(bytes), "r"(shared_address(barrier))
        : "memory");
}

// a consumer's arrival: "this stage may be overwritten"
__device__ __forceinline__ void mbarrier_arrive(uint64_t *barrier) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(shared_address(barrier)) : "memory");
}

// L2 policy for bytes that are read exactly once: first in line for eviction, so
// that they do not push out what is read again (token histories, scratch rows).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

__device__ __forceinline__ void bulk_copy_to_shared_hinted(void *shared_destination,
                                                           const void *global_source, uint32_t bytes,
                                                           uint64_t *barrier, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, "
        "[%3], %4;" ::"r"(shared_address(shared_destination)),
        "l"(global_source), "r"(bytes), "r"(shared_address(barrier)), "l"(policy)
        : "memory");
}

// The POD the kernels read; layout of fg_sampler_config (include/fg_sampler.h).
struct SamplerConfig {
    float temperature;
    float top_p;
    uint32_t top_k;
    float presence_penalty;
    float frequency_penalty;
    float repetition_penalty;
    float min_p;
    uint32_t pad_;
    uint64_t seed;
};
static_assert(sizeof(SamplerConfig) == 40, "fg_sampler_config is 40 bytes");

__device__ __forceinline__ bool penalties_active(const SamplerConfig &c) {
    return c.presence_penalty != 0.0f || c.frequency_penalty != 0.0f ||
           c.repetition_penalty != 1.0f;
}

// Picture of the part of a row's history that falls into one column range, in shared
// or global memory:
//   bitmap   bit c set = column c occurs in the history            u32[bitmap_words]
//   running  number of seen columns before each bitmap word        u16[bitmap_words]
//   dense    occurrences of each seen column, in column order      u16 or u32[capacity]
// (u32 counts only when a history may be longer than 65,535 tokens.)
struct HistoryView {
    uint32_t *bitmap;
    uint16_t *running;
    void *dense;
    uint32_t capacity;
    bool wide;

    __device__ __forceinline__ uint32_t slot(uint32_t word_index, uint32_t word, uint32_t bit) const {
        return min(running[word_index] + __popc(word & ((1u << bit) - 1u)), capacity - 1);
    }
    __device__ __forceinline__ uint32_t count(uint32_t word_index, uint32_t word, uint32_t bit) const {
        const uint32_t at = slot(word_index, word, bit);
        return wide ? static_cast<const uint32_t *>(dense)[at]
                    : static_cast<const uint16_t *>(dense)[at];
    }
};

__device__ __forceinline__ HistoryView make_history_view(uint32_t *memory, uint32_t bitmap_words,
                                                         uint32_t capacity, bool wide) {
    HistoryView h;
    h.bitmap = memory;
    h.running = reinterpret_cast<uint16_t *>(memory + bitmap_words);
    h.dense = memory + bitmap_words + (bitmap_words + 1) / 2;
    h.capacity = capacity;
    h.wide = wide;
    return h;
}

// fg_status values used on the device (include/fg.h).
constexpr uint32_t kOk = 0u, kErrArgument = 2u, kErrFormat = 4u, kErrMismatch = 5u, kErrLimit = 8u;

}  // namespace fgk
