// TEST INFRASTRUCTURE ONLY — a CPU restatement of the reference's MLA decode
// arithmetic, used as the checker by tests/, by __graft_entry__.smoke() and as the
// timed CPU baseline of bench.py.  Nothing in the product path may link, import
// or call this file.
//
// Parity status: PINNED for attention, yarn_rope_freq and the KVCache counter —
// the functions below are compared bit for bit with the reference's own code
// compiled from its sources (oracle/ref_harness.cpp -> oracle/_ref/libmugen_ref.so)
// and with the committed fixtures under tests/golden/ that were produced by that
// build.  The append arithmetic is inline code inside the reference's forward()
// (src/core/model/transformer.cpp:3930-3979) and cannot be called on its own; its
// restatement here follows that block statement by statement and is pinned only
// through the pieces it shares with callable reference code (yarn_rope_freq).
//
// Build flags matter: -ffp-contract=off (no FMA contraction; the reference is
// built in ISO mode) and F16C for the _Float16 conversions (round to nearest even).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr uint32_t kRank = 512;      // kv_lora_rank
constexpr uint32_t kRope = 64;       // qk_rope_head_dim
constexpr uint32_t kNope = 128;      // qk_nope_head_dim
constexpr uint32_t kVDim = 128;      // v_head_dim
constexpr uint32_t kRow  = kRank + kRope;
constexpr uint32_t kQDim = kNope + kRope;

// storage dtypes
constexpr uint32_t DT_F16 = 0, DT_BF16 = 1;
// weight encodings (GGML type ids as in src/model/ggml_types.h:12-40, plus BF16 = 30)
constexpr uint32_t W_F16 = 1, W_Q4_0 = 2, W_Q8_0 = 8, W_BF16 = 30;

inline float bf16_to_f32(uint16_t b) {
    uint32_t u = uint32_t(b) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_bf16(float f) {           // round to nearest even, NaN kept quiet
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return uint16_t(u >> 16);
}
inline float ld(const void* p, size_t i, uint32_t dt) {
    if (dt == DT_F16) return static_cast<float>(static_cast<const _Float16*>(p)[i]);
    return bf16_to_f32(static_cast<const uint16_t*>(p)[i]);
}
inline void st(void* p, size_t i, float v, uint32_t dt) {
    if (dt == DT_F16) static_cast<_Float16*>(p)[i] = static_cast<_Float16>(v);
    else static_cast<uint16_t*>(p)[i] = f32_to_bf16(v);
}

// src/core/model/transformer.cpp:41-70
float yarn_freq(uint32_t pair, uint32_t rope_dim, float factor, uint32_t orig_ctx, float theta)
{
    const float base = 1.0f / std::pow(theta, 2.0f * float(pair) / float(rope_dim));
    if (factor <= 1.0f) return base;
    const float fast = 32.0f, slow = 1.0f;
    const float ln_theta = std::log(theta);
    const float ctx = float(orig_ctx);
    const float dim = float(rope_dim);
    float lo = std::floor(dim * std::log(ctx / (fast * 2.0f * float(M_PI))) / (2.0f * ln_theta));
    float hi = std::ceil (dim * std::log(ctx / (slow * 2.0f * float(M_PI))) / (2.0f * ln_theta));
    lo = std::max(lo, 0.0f);
    hi = std::min(hi, float(rope_dim / 2 - 1));
    const float x = float(pair);
    if (x < lo) return base;
    if (x > hi) return base / factor;
    float t = (x - lo) / std::max(0.001f, hi - lo);
    t = std::max(0.0f, std::min(1.0f, t));
    return base * (1.0f - t) + (base / factor) * t;
}

// NeoX-paired rotation of one 64-wide vector at position pos
// (src/core/model/transformer.cpp:3905-3916 for q, :3964-3975 for k_rope).
void rope64(const void* in, void* out, size_t off, uint32_t pos, float factor,
            uint32_t orig_ctx, float theta, uint32_t dt)
{
    const uint32_t half = kRope / 2;
    float a[kRope];
    for (uint32_t i = 0; i < kRope; i++) a[i] = ld(in, off + i, dt);
    for (uint32_t i = 0; i < half; i++) {
        const float f = yarn_freq(i, kRope, factor, orig_ctx, theta);
        const float ang = float(pos) * f;
        const float c = std::cos(ang), s = std::sin(ang);
        const float x0 = a[i], x1 = a[i + half];
        st(out, off + i,        x0 * c - x1 * s, dt);
        st(out, off + i + half, x1 * c + x0 * s, dt);
    }
}

// src/core/model/transformer.cpp:2489-2534, plus a BF16 row type for bf16 caches.
void weight_row(const void* w, uint32_t type, uint32_t row, float* out)
{
    if (type == W_F16) {
        const auto* r = static_cast<const _Float16*>(w) + size_t(row) * kRank;
        for (uint32_t i = 0; i < kRank; i++) out[i] = static_cast<float>(r[i]);
    } else if (type == W_BF16) {
        const auto* r = static_cast<const uint16_t*>(w) + size_t(row) * kRank;
        for (uint32_t i = 0; i < kRank; i++) out[i] = bf16_to_f32(r[i]);
    } else if (type == W_Q8_0) {
        const uint32_t nb = kRank / 32;
        const auto* base = static_cast<const uint8_t*>(w) + size_t(row) * nb * 34;
        for (uint32_t b = 0; b < nb; b++) {
            const uint8_t* blk = base + size_t(b) * 34;
            _Float16 d;
            std::memcpy(&d, blk, 2);
            const float s = static_cast<float>(d);
            const auto* q = reinterpret_cast<const int8_t*>(blk + 2);
            for (uint32_t j = 0; j < 32; j++) out[b * 32 + j] = s * float(q[j]);
        }
    } else if (type == W_Q4_0) {
        const uint32_t nb = kRank / 32;
        const auto* base = static_cast<const uint8_t*>(w) + size_t(row) * nb * 18;
        for (uint32_t b = 0; b < nb; b++) {
            const uint8_t* blk = base + size_t(b) * 18;
            _Float16 d;
            std::memcpy(&d, blk, 2);
            const float s = static_cast<float>(d);
            for (uint32_t j = 0; j < 16; j++) {
                out[b * 32 + j]      = float(int(blk[2 + j] & 0x0F) - 8) * s;
                out[b * 32 + j + 16] = float(int(blk[2 + j] >> 4) - 8) * s;
            }
        }
    } else {
        std::memset(out, 0, kRank * sizeof(float));   // reference: warn + zero row
    }
}

// src/core/model/transformer.cpp:2539-2623 for one sequence.  With `partial`
// non-null the routine stops before the division by the softmax sum and before
// W_UV and emits, per head, (max, sum, unnormalised acc[512]) over rows
// [row_begin, row_end) — the quantity a KV-range shard contributes.
void attention_one(const void* q, const void* cache, uint32_t row_begin, uint32_t row_end,
                   const void* w_uk, const void* w_uv, uint32_t w_type, uint32_t n_heads,
                   void* out, uint32_t dt, float* partial)
{
    const float scale = 1.0f / std::sqrt(float(kQDim));
    const uint32_t n = row_end - row_begin;
    std::vector<float> wrow(kRank), qabs(kRank), acc(kRank), sc(n ? n : 1);
    for (uint32_t h = 0; h < n_heads; h++) {
        const size_t qoff = size_t(h) * kQDim;
        std::fill(qabs.begin(), qabs.end(), 0.0f);
        for (uint32_t i = 0; i < kNope; i++) {
            const float qi = ld(q, qoff + i, dt);
            if (qi == 0.0f) continue;
            weight_row(w_uk, w_type, h * kNope + i, wrow.data());
            for (uint32_t d = 0; d < kRank; d++) qabs[d] += qi * wrow[d];
        }
        for (uint32_t t = 0; t < n; t++) {
            const size_t roff = size_t(row_begin + t) * kRow;
            float s = 0.0f;
            for (uint32_t d = 0; d < kRank; d++) s += qabs[d] * ld(cache, roff + d, dt);
            for (uint32_t d = 0; d < kRope; d++)
                s += ld(q, qoff + kNope + d, dt) * ld(cache, roff + kRank + d, dt);
            sc[t] = s * scale;
        }
        float mx = -INFINITY;
        for (uint32_t t = 0; t < n; t++) mx = std::max(mx, sc[t]);
        float sum = 0.0f;
        for (uint32_t t = 0; t < n; t++) {
            sc[t] = std::exp(sc[t] - mx);
            sum += sc[t];
        }
        if (!partial)
            for (uint32_t t = 0; t < n; t++) sc[t] /= sum;
        std::fill(acc.begin(), acc.end(), 0.0f);
        for (uint32_t t = 0; t < n; t++) {
            const size_t roff = size_t(row_begin + t) * kRow;
            const float p = sc[t];
            for (uint32_t d = 0; d < kRank; d++) acc[d] += p * ld(cache, roff + d, dt);
        }
        if (partial) {
            float* ph = partial + size_t(h) * (kRank + 2);
            ph[0] = mx;
            ph[1] = sum;
            std::memcpy(ph + 2, acc.data(), kRank * sizeof(float));
            continue;
        }
        for (uint32_t j = 0; j < kVDim; j++) {
            weight_row(w_uv, w_type, h * kVDim + j, wrow.data());
            float v = 0.0f;
            for (uint32_t d = 0; d < kRank; d++) v += acc[d] * wrow[d];
            st(out, size_t(h) * kVDim + j, v, dt);
        }
    }
}

}  // namespace

extern "C" {

float oracle_yarn_rope_freq(uint32_t pair, uint32_t rope_dim, float factor,
                            uint32_t orig_ctx, float theta)
{
    return yarn_freq(pair, rope_dim, factor, orig_ctx, theta);
}

// cos/sin of float(pos)*freq_i for the 32 pairs, as the reference evaluates them.
void oracle_rope_cos_sin(uint32_t pos, float factor, uint32_t orig_ctx, float theta,
                         float* cos_out, float* sin_out)
{
    for (uint32_t i = 0; i < kRope / 2; i++) {
        const float ang = float(pos) * yarn_freq(i, kRope, factor, orig_ctx, theta);
        cos_out[i] = std::cos(ang);
        sin_out[i] = std::sin(ang);
    }
}

// Append arithmetic, steps G of the decode driver (transformer.cpp:3930-3979; batched twin
// :1263-1313): n rows kv_a[n][576] -> latent rows out[n][576], row r at positions[r].
void oracle_append_rows(const void* kv_a, uint32_t n, const uint32_t* positions,
                        const void* norm_w, float eps, float factor, uint32_t orig_ctx,
                        float theta, uint32_t dt, void* out)
{
    for (uint32_t r = 0; r < n; r++) {
        const size_t off = size_t(r) * kRow;
        float ss = 0.0f;
        for (uint32_t i = 0; i < kRank; i++) {
            const float v = ld(kv_a, off + i, dt);
            ss += v * v;
        }
        ss = 1.0f / std::sqrt(ss / float(kRank) + eps);
        for (uint32_t i = 0; i < kRank; i++) {
            const float v = ld(kv_a, off + i, dt) * ss;
            st(out, off + i, v * ld(norm_w, i, dt), dt);
        }
        rope64(kv_a, out, off + kRank, positions[r], factor, orig_ctx, theta, dt);
    }
}

// Step E of the decode driver (transformer.cpp:3882-3921): rotate the last 64 dims of each
// head of q[n_heads][192] in place.
void oracle_q_rope(void* q, uint32_t n_heads, uint32_t pos, float factor, uint32_t orig_ctx,
                   float theta, uint32_t dt)
{
    for (uint32_t h = 0; h < n_heads; h++)
        rope64(q, q, size_t(h) * kQDim + kNope, pos, factor, orig_ctx, theta, dt);
}

void oracle_mla_attention(const void* q, const void* cache, uint32_t seq_len,
                          const void* w_uk, const void* w_uv, uint32_t w_type,
                          uint32_t n_heads, void* out, uint32_t dt)
{
    attention_one(q, cache, 0, seq_len, w_uk, w_uv, w_type, n_heads, out, dt, nullptr);
}

// Per-head (max, sum, acc[512]) over cache rows [row_begin, row_end): partial[n_heads][514].
void oracle_mla_partial(const void* q, const void* cache, uint32_t row_begin, uint32_t row_end,
                        const void* w_uk, uint32_t w_type, uint32_t n_heads, uint32_t dt,
                        float* partial)
{
    attention_one(q, cache, row_begin, row_end, w_uk, nullptr, w_type, n_heads, nullptr, dt,
                  partial);
}

// n_seq independent sequences over n_threads host threads.
void oracle_mla_attention_batch(const void* q, const void* const* cache_ptrs,
                                const uint32_t* seq_lens, uint32_t n_seq,
                                const void* w_uk, const void* w_uv, uint32_t w_type,
                                uint32_t n_heads, void* out, uint32_t dt, uint32_t n_threads)
{
    if (n_threads == 0) n_threads = 1;
    auto work = [&](uint32_t tid) {
        for (uint32_t s = tid; s < n_seq; s += n_threads) {
            const auto* qs = static_cast<const uint16_t*>(q) + size_t(s) * n_heads * kQDim;
            auto* os = static_cast<uint16_t*>(out) + size_t(s) * n_heads * kVDim;
            attention_one(qs, cache_ptrs[s], 0, seq_lens[s], w_uk, w_uv, w_type, n_heads, os,
                          dt, nullptr);
        }
    };
    std::vector<std::thread> pool;
    for (uint32_t t = 1; t < n_threads; t++) pool.emplace_back(work, t);
    work(0);
    for (auto& th : pool) th.join();
}

// Sequence-length counter semantics of the reference KVCache as the MLA model uses it
// (src/core/memory/kv_cache.cpp:281-285, 313-321, 343-357 with zero materialised rows).
struct oracle_counter { uint32_t phantom; };
void oracle_counter_advance(oracle_counter* c, uint32_t n) { c->phantom += n; }
void oracle_counter_truncate(oracle_counter* c, uint32_t n) { c->phantom = n; }
void oracle_counter_clear(oracle_counter* c) { c->phantom = 0; }
uint32_t oracle_counter_seq_len(const oracle_counter* c) { return c->phantom; }

}  // extern "C"
