/* 16-bit storage types of the public API (counterpart of the reference's include/baremetal/types.h:12-37):
 * raw-bit typedefs plus host-side conversions. bf16 conversion rounds to nearest, ties to even. */
#ifndef BAREMETAL_TYPES_H
#define BAREMETAL_TYPES_H

#include <stddef.h>
#include <stdint.h>
#include <string.h>

typedef uint16_t bm_bf16_t;
typedef uint16_t bm_fp16_t;

static inline float bm_bf16_to_f32(bm_bf16_t h) {
    const uint32_t bits = (uint32_t)h << 16;
    float out;
    memcpy(&out, &bits, sizeof out);
    return out;
}

static inline bm_bf16_t bm_f32_to_bf16(float f) {
    uint32_t bits;
    memcpy(&bits, &f, sizeof bits);
    bits += 0x7FFFu + ((bits >> 16) & 1u); /* round half to even on the dropped 16 bits */
    return (bm_bf16_t)(bits >> 16);
}

static inline void bm_f32_to_bf16_array(const float* src, bm_bf16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = bm_f32_to_bf16(src[i]);
}

static inline void bm_bf16_to_f32_array(const bm_bf16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = bm_bf16_to_f32(src[i]);
}

#endif
