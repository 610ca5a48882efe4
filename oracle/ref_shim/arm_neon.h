// TEST INFRASTRUCTURE: x86 stand-ins for the AArch64 NEON intrinsics that the reference's CPU expert engine
// (runtime/tier/cpuband.cpp) uses, so that its unmodified arithmetic can be compiled and run on an x86-64 host as the
// parity oracle and the timed CPU baseline. Integer operations are exact; vfmaq_n_f32 is a fused multiply-add like the
// AArch64 instruction; vaddvq_f32 adds pairwise, (v0 + v1) + (v2 + v3), the order of the AArch64 FADDP sequence.
// Needs -mavx2 -mfma.
#pragma once
#include <cstdint>
#include <immintrin.h>

typedef __m128 float32x4_t;
struct int32x4_t { __m128i v; };
struct uint8x16_t { __m128i v; };
struct int8x16_t { __m128i v; };
struct int8x16x2_t { int8x16_t val[2]; };

static inline float32x4_t vdupq_n_f32(float a) { return _mm_set1_ps(a); }
static inline int32x4_t vdupq_n_s32(int32_t a) { return {_mm_set1_epi32(a)}; }
static inline uint8x16_t vdupq_n_u8(uint8_t a) { return {_mm_set1_epi8((char) a)}; }
static inline int8x16_t vdupq_n_s8(int8_t a) { return {_mm_set1_epi8(a)}; }
static inline uint8x16_t vld1q_u8(const uint8_t* p) { return {_mm_loadu_si128((const __m128i*) p)}; }
static inline int8x16_t vld1q_s8(const int8_t* p) { return {_mm_loadu_si128((const __m128i*) p)}; }
static inline uint8x16_t vandq_u8(uint8x16_t a, uint8x16_t b) { return {_mm_and_si128(a.v, b.v)}; }
static inline uint8x16_t vshrq_n_u8(uint8x16_t a, int n) { return {_mm_and_si128(_mm_srli_epi16(a.v, n), _mm_set1_epi8((char) (0xff >> n)))}; }
static inline int8x16_t vreinterpretq_s8_u8(uint8x16_t a) { return {a.v}; }
static inline int8x16_t vsubq_s8(int8x16_t a, int8x16_t b) { return {_mm_sub_epi8(a.v, b.v)}; }
static inline int8x16x2_t vzipq_s8(int8x16_t a, int8x16_t b) { return {{{_mm_unpacklo_epi8(a.v, b.v)}, {_mm_unpackhi_epi8(a.v, b.v)}}}; }
// lane i += sum of the four int8 products 4i .. 4i+3
static inline int32x4_t vdotq_s32(int32x4_t acc, int8x16_t a, int8x16_t b)
{
    const __m256i m = _mm256_madd_epi16(_mm256_cvtepi8_epi16(a.v), _mm256_cvtepi8_epi16(b.v));
    const __m128i d = _mm_hadd_epi32(_mm256_castsi256_si128(m), _mm256_extracti128_si256(m, 1));
    return {_mm_add_epi32(acc.v, d)};
}
static inline float32x4_t vcvtq_f32_s32(int32x4_t a) { return _mm_cvtepi32_ps(a.v); }
static inline float32x4_t vfmaq_n_f32(float32x4_t acc, float32x4_t a, float s) { return _mm_fmadd_ps(a, _mm_set1_ps(s), acc); }
static inline float vaddvq_f32(float32x4_t a)
{
    float v[4]; _mm_storeu_ps(v, a);
    return (v[0] + v[1]) + (v[2] + v[3]);
}
