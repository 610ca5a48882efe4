// TEST INFRASTRUCTURE: x86 stand-ins for the AArch64 NEON intrinsics that the reference's CPU expert engine
// (runtime/tier/cpuband.cpp) uses, so that its unmodified arithmetic can be compiled and run on an x86-64 host as the
// parity oracle and the timed CPU baseline. Integer operations are exact; vfmaq_n_f32 is a fused multiply-add like the
// AArch64 instruction; vaddvq_f32 adds pairwise, (v0 + v1) + (v2 + v3), the order of the AArch64 FADDP sequence.
// Three builds of the two intrinsics in the engine's inner loop (cpuband.cpp:80-104), all bit-identical in their results:
//   default           vdotq_s32 as widening 16-bit multiply-adds (AVX2), vfmaq_n_f32 as an FMA            needs -mavx2 -mfma
//   HMOE_SHIM_VNNI    vdotq_s32 as one AVX-512-VNNI dot-product instruction (the x86 counterpart of SDOT)  + -mavx512vl -mavx512vnni
//   HMOE_SHIM_SCALAR  both as plain scalar loops (a strawman: what the engine costs without SIMD)
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
#if defined(HMOE_SHIM_SCALAR)
    alignas(16) int8_t x[16], y[16]; alignas(16) int32_t c[4];
    _mm_store_si128((__m128i*) x, a.v); _mm_store_si128((__m128i*) y, b.v); _mm_store_si128((__m128i*) c, acc.v);
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 4; ++j) c[i] += (int32_t) x[4 * i + j] * (int32_t) y[4 * i + j];
    return {_mm_load_si128((const __m128i*) c)};
#elif defined(HMOE_SHIM_VNNI)
    // vpdpbusd multiplies unsigned by signed bytes: |a| x (b with a's sign). Exact for every a and every b != -128; the engine's
    // b operands are activation codes in [-127, 127] (cpuband.cpp:106-111) and its a operands int4 values in [-8, 7].
    return {_mm_dpbusd_epi32(acc.v, _mm_abs_epi8(a.v), _mm_sign_epi8(b.v, a.v))};
#else
    const __m256i m = _mm256_madd_epi16(_mm256_cvtepi8_epi16(a.v), _mm256_cvtepi8_epi16(b.v));
    const __m128i d = _mm_hadd_epi32(_mm256_castsi256_si128(m), _mm256_extracti128_si256(m, 1));
    return {_mm_add_epi32(acc.v, d)};
#endif
}
static inline float32x4_t vcvtq_f32_s32(int32x4_t a) { return _mm_cvtepi32_ps(a.v); }
static inline float32x4_t vfmaq_n_f32(float32x4_t acc, float32x4_t a, float s)
{
#if defined(HMOE_SHIM_SCALAR)
    alignas(16) float x[4], c[4];
    _mm_store_ps(x, a); _mm_store_ps(c, acc);
    for (int i = 0; i < 4; ++i) c[i] = __builtin_fmaf(x[i], s, c[i]);
    return _mm_load_ps(c);
#else
    return _mm_fmadd_ps(a, _mm_set1_ps(s), acc);
#endif
}
static inline float vaddvq_f32(float32x4_t a)
{
    float v[4]; _mm_storeu_ps(v, a);
    return (v[0] + v[1]) + (v[2] + v[3]);
}
