// TEST INFRASTRUCTURE ONLY — part of the CPU oracle; the CUDA product never includes this file.
//
// IEEE binary16 / bfloat16 <-> binary32 conversions, round-to-nearest-even, restating what the
// `half` crate 2.7.1 (`f16::from_f32`, `bf16::from_f32`, `to_f32`) does for the reference's
// NativeData coercions (src/hlir.rs:362-393, 1435-1453).  Written from the IEEE-754 definitions.
#pragma once
#include <cstdint>
#include <cstring>

namespace orc {

static inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// bfloat16: top 16 bits of binary32, RNE on the discarded 16 bits; NaN stays NaN (quiet bit set).
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t round = 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)((u + round) >> 16);
}
static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

// binary16: 1 sign, 5 exponent (bias 15), 10 mantissa bits.
static inline uint16_t f32_to_f16(float f) {
    uint32_t u = f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((a >> 13) & 0x3ffu));   // NaN
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);                          // >= 65536 -> inf (incl. inf)
    if (a >= 0x38800000u) {                                                            // normal half range
        uint32_t m = a - 0x38000000u;             // rebias exponent 127 -> 15
        uint32_t r = m + 0xfffu + ((m >> 13) & 1u);
        return (uint16_t)(sign | (r >> 13));     // a carry out of the mantissa bumps the exponent; 65520+ -> inf
    }
    if (a < 0x33000000u) return (uint16_t)sign;   // < 2^-25 rounds to zero
    // subnormal half: value = mant * 2^-24
    uint32_t e = a >> 23;                         // biased f32 exponent, 102..112
    uint32_t mant = (a & 0x7fffffu) | 0x800000u;  // 24-bit significand
    uint32_t shift = 126u - e;                    // 14..24: result = mant >> shift with RNE
    uint32_t q = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1u);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}
static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0x1fu) return bits_f32(sign | 0x7f800000u | (m << 13));
    if (e != 0) return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
    if (m == 0) return bits_f32(sign);
    // subnormal: m * 2^-24, exact in f32
    float v = (float)m * 5.9604644775390625e-08f;
    return sign ? -v : v;
}

}  // namespace orc
