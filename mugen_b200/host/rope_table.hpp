// Host evaluation of the rotary cos/sin values the append kernel consumes.
//
// The reference computes, per appended token and per pair i of the 64 rope dims,
//   freq  = yarn_rope_freq(i, 64, factor, original_ctx, theta)   src/core/model/transformer.cpp:41-70
//   angle = float(pos) * freq ;  cos(angle), sin(angle)           :3965-3969
// with the C library's float functions.  Device cosf/sinf/powf/logf are not bit-identical to
// glibc's, so the table is built here, on the host, with the same calls in the same order, and
// uploaded; the kernel only looks values up.  Compile without FMA contraction.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>

namespace mugen::mla {

inline float yarn_rope_freq(uint32_t pair, uint32_t rope_dim, float factor, uint32_t original_ctx,
                            float theta)
{
    const float plain = 1.0f / std::pow(theta, 2.0f * static_cast<float>(pair) /
                                                   static_cast<float>(rope_dim));
    if (factor <= 1.0f) return plain;
    const float rot_fast = 32.0f, rot_slow = 1.0f;
    const float two_pi = 2.0f * static_cast<float>(M_PI);
    const float ln_theta = std::log(theta);
    const float ctx = static_cast<float>(original_ctx);
    const float dim = static_cast<float>(rope_dim);
    float first = std::floor(dim * std::log(ctx / (rot_fast * two_pi)) / (2.0f * ln_theta));
    float last  = std::ceil (dim * std::log(ctx / (rot_slow * two_pi)) / (2.0f * ln_theta));
    first = std::max(first, 0.0f);
    last  = std::min(last, static_cast<float>(rope_dim / 2 - 1));
    const float x = static_cast<float>(pair);
    if (x < first) return plain;
    if (x > last) return plain / factor;
    float mix = (x - first) / std::max(0.001f, last - first);
    mix = std::max(0.0f, std::min(1.0f, mix));
    return plain * (1.0f - mix) + (plain / factor) * mix;
}

// Fills rows [pos_begin, pos_end) of a [pos][64] table: 32 cosines then 32 sines per position.
inline void fill_rope_rows(float* table, uint32_t pos_begin, uint32_t pos_end, float factor,
                           uint32_t original_ctx, float theta)
{
    float freq[32];
    for (uint32_t i = 0; i < 32; i++) freq[i] = yarn_rope_freq(i, 64, factor, original_ctx, theta);
    for (uint32_t p = pos_begin; p < pos_end; p++) {
        float* row = table + static_cast<size_t>(p - pos_begin) * 64;
        for (uint32_t i = 0; i < 32; i++) {
            const float angle = static_cast<float>(p) * freq[i];
            row[i] = std::cos(angle);
            row[32 + i] = std::sin(angle);
        }
    }
}

}  // namespace mugen::mla
