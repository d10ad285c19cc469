// TEST INFRASTRUCTURE ONLY — part of the CPU oracle; the CUDA product never includes this file.
//
// Counter-based synthetic-tensor generator.  There are no checkpoints in this environment (the
// reference downloads them, examples/llama/src/hf.rs:26-50), so both the oracle and the CUDA
// library regenerate every tensor element from (seed, tensor id, element index).  This is the
// oracle's own statement of that generator; tests check it bit-for-bit against what the CUDA
// library produces.
//
//   key(seed, tid)     = mix(seed + G * (tid + 1))
//   r(key, idx, lane)  = mix(key + G * (2*idx + lane)),  lane in {0,1}
//   int8 quant         = ((r(…,0) >> 32) * 255 >> 32) - 127                 uniform on [-127, 127]
//   standard normal    = sqrt(-2 ln u1) * cos(2 pi u2) in binary64,
//                        u1 = ((r(…,0) >> 11) + 1) * 2^-53, u2 = (r(…,1) >> 11) * 2^-53
//   Q8_0 block scale   = f16( (float)( |0.02 * z| / 127 ) )
//   token id           = (r(…,0) >> 32) * vocab >> 32
// mix is the SplitMix64 output function (Steele, Lea, Flood 2014), G = 0x9E3779B97F4A7C15.
#pragma once
#include <cmath>
#include <cstdint>
#include "halfs.hpp"

namespace orc {

static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static const uint64_t kGolden = 0x9E3779B97F4A7C15ull;
static inline uint64_t rng_key(uint64_t seed, uint64_t tid) { return mix64(seed + kGolden * (tid + 1)); }
static inline uint64_t rng_draw(uint64_t key, uint64_t idx, uint64_t lane) {
    return mix64(key + kGolden * (2 * idx + lane));
}
static inline int rng_int8(uint64_t key, uint64_t idx) {
    uint64_t r = rng_draw(key, idx, 0) >> 32;
    return (int)((r * 255ull) >> 32) - 127;
}
static inline double rng_normal(uint64_t key, uint64_t idx) {
    double u1 = (double)((rng_draw(key, idx, 0) >> 11) + 1) * 0x1.0p-53;
    double u2 = (double)(rng_draw(key, idx, 1) >> 11) * 0x1.0p-53;
    return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586476925 * u2);
}
static inline uint16_t rng_q8_scale(uint64_t key, uint64_t block) {
    return f32_to_f16((float)(std::fabs(0.02 * rng_normal(key, block)) / 127.0));
}
static inline float rng_weight_f32(uint64_t key, uint64_t idx) { return (float)(0.02 * rng_normal(key, idx)); }
static inline uint32_t rng_token(uint64_t key, uint64_t idx, uint32_t vocab) {
    return (uint32_t)(((rng_draw(key, idx, 0) >> 32) * (uint64_t)vocab) >> 32);
}

}  // namespace orc
