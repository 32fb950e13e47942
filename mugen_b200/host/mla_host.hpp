// C++23 host-side mirror of the reference's attention-op / KV-cache interface, over the C ABI of
// include/mugen_mla.h.  Header-only; link against libmugen_mla.so.  No CUDA headers needed: a
// stream travels as void*.
//
//   mugen::mla::LatentKVCache   mugen::KVCache's contract (src/core/memory/kv_cache.h:20-47):
//                               create() -> std::expected<unique_ptr, string>, append() -> bool,
//                               seq_len / advance_seq_len / truncate / clear / config — with a
//                               sequence id added, because the reference holds one implicit sequence.
//   mugen::mla::MlaAttention    cpu_mla_attention's call shape
//                               (src/core/model/transformer.cpp:2539-2541): (q, layer, seq_len, out),
//                               batched over sequences, plus the decode-step scheduler.
// Error convention as in the reference model API (transformer.h:84-111): std::expected<T, std::string>.
#pragma once

#include <cstdint>
#include <expected>
#include <memory>
#include <span>
#include <string>
#include <vector>

#include "../../include/mugen_mla.h"

namespace mugen::mla {

using Status = std::expected<void, std::string>;

struct LatentKVCacheConfig {
    uint32_t n_layers = 0;
    uint32_t n_heads = 0;
    uint32_t max_seq_len = 8192;     // KVCacheConfig::max_seq_len's default (kv_cache.h:15)
    uint32_t n_pages = 0;
    uint32_t max_seqs = 1;
    uint32_t max_rows = 0;
    uint32_t max_position = 0;
    bool bf16 = false;               // false: IEEE half, the reference's element type
    float rope_theta = 10000.0f;
    float rms_norm_eps = 1e-5f;      // the reference's default (transformer.cpp:2920)
    float rope_scaling_factor = 0.0f;
    uint32_t rope_original_ctx = 0;
    int device = 0;
    uint32_t kernel = MLA_KERNEL_AUTO;
};

class MlaAttention;

class LatentKVCache {
public:
    static auto create(LatentKVCacheConfig cfg) -> std::expected<std::unique_ptr<LatentKVCache>, std::string>
    {
        mla_config c{};
        c.n_layers = cfg.n_layers;
        c.n_heads = cfg.n_heads;
        c.kv_lora_rank = 512;
        c.qk_nope_head_dim = 128;
        c.qk_rope_head_dim = 64;
        c.v_head_dim = 128;
        c.rope_theta = cfg.rope_theta;
        c.rms_norm_eps = cfg.rms_norm_eps;
        c.rope_scaling_factor = cfg.rope_scaling_factor;
        c.rope_original_ctx = cfg.rope_original_ctx;
        c.max_seq_len = cfg.max_seq_len;
        c.page_tokens = 64;
        c.n_pages = cfg.n_pages;
        c.max_seqs = cfg.max_seqs;
        c.max_rows = cfg.max_rows;
        c.dtype = cfg.bf16 ? MLA_DTYPE_BF16 : MLA_DTYPE_F16;
        c.device = cfg.device;
        c.kernel = cfg.kernel;
        c.max_position = cfg.max_position;
        mla_ctx* h = nullptr;
        if (mla_create(&c, &h) != MLA_OK) return std::unexpected(std::string(mla_last_error(nullptr)));
        return std::unique_ptr<LatentKVCache>(new LatentKVCache(h, cfg));
    }

    ~LatentKVCache() { mla_destroy(h_); }
    LatentKVCache(const LatentKVCache&) = delete;
    LatentKVCache& operator=(const LatentKVCache&) = delete;

    auto new_sequence() -> std::expected<uint32_t, std::string>
    {
        uint32_t id = 0;
        if (mla_seq_create(h_, &id) != MLA_OK) return std::unexpected(err());
        return id;
    }
    auto free_sequence(uint32_t seq) -> Status { return wrap(mla_seq_free(h_, seq)); }

    // KVCache::append's convention: false on a bad layer or on overflow (kv_cache.cpp:161-169).
    // kv_a: DEVICE [n][576] rows straight from the W_kv_a projection.
    auto append(uint32_t layer, std::span<const uint32_t> seq_ids, std::span<const uint32_t> positions,
                const void* kv_a, void* stream = nullptr) -> bool
    {
        if (seq_ids.size() != positions.size()) return false;
        return mla_append_rows(h_, layer, uint32_t(seq_ids.size()), seq_ids.data(), positions.data(), kv_a,
                               stream) == MLA_OK;
    }

    auto seq_len(uint32_t seq) const -> uint32_t
    {
        uint32_t n = 0;
        mla_seq_len(h_, seq, &n);
        return n;
    }
    auto advance_seq_len(uint32_t seq, uint32_t n = 1) -> Status { return wrap(mla_advance(h_, seq, n)); }
    auto truncate(uint32_t seq, uint32_t new_len) -> Status { return wrap(mla_truncate(h_, seq, new_len)); }
    // rollback of a speculative verify step for many sequences (uspp_scheduler.cpp:222-237)
    auto rollback(const std::vector<uint32_t>& seqs, const std::vector<uint32_t>& keep_lens) -> Status {
        if (seqs.size() != keep_lens.size()) return std::unexpected("rollback: one keep length per sequence");
        return wrap(mla_rollback(h_, uint32_t(seqs.size()), seqs.data(), keep_lens.data()));
    }
    auto clear(uint32_t seq) -> Status { return wrap(mla_clear(h_, seq)); }
    auto set_base_position(uint32_t seq, uint32_t base) -> Status { return wrap(mla_seq_set_base(h_, seq, base)); }
    auto config() const -> const LatentKVCacheConfig& { return cfg_; }
    auto free_pages() const -> uint32_t
    {
        uint32_t n = 0;
        mla_free_pages(h_, &n);
        return n;
    }
    auto last_error() const -> std::string { return err(); }
    auto handle() const -> mla_ctx* { return h_; }

private:
    friend class MlaAttention;
    LatentKVCache(mla_ctx* h, LatentKVCacheConfig cfg) : h_(h), cfg_(cfg) {}
    auto err() const -> std::string { return mla_last_error(h_); }
    auto wrap(int rc) const -> Status
    {
        if (rc == MLA_OK) return {};
        return std::unexpected(err());
    }
    mla_ctx* h_;
    LatentKVCacheConfig cfg_;
};

class MlaAttention {
public:
    explicit MlaAttention(LatentKVCache& cache) : c_(cache) {}

    // W_UK / W_UV as (n_heads*128) x 512 row-major host buffers in a GGML type the reference's
    // dequant_weight_row accepts (F16, Q8_0, Q4_0) or BF16; norm: [512] in the cache dtype.
    auto set_layer_weights(uint32_t layer, const void* w_uk, const void* w_uv, uint32_t ggml_type,
                           const void* kv_norm) -> Status
    {
        return c_.wrap(mla_set_layer_weights(c_.h_, layer, w_uk, w_uv, ggml_type, kv_norm));
    }

    // cpu_mla_attention(q, lw, layer, seq_len, out) for a batch: row r attends the first
    // seq_lens[r] rows of sequence seq_ids[r].  q / out: DEVICE buffers.
    auto attend(uint32_t layer, std::span<const uint32_t> seq_ids, std::span<const uint32_t> seq_lens,
                const void* q, void* out, void* stream = nullptr) -> Status
    {
        if (seq_ids.size() != seq_lens.size()) return std::unexpected(std::string("seq_ids and seq_lens differ in length"));
        return c_.wrap(mla_attend_rows(c_.h_, layer, uint32_t(seq_ids.size()), seq_ids.data(), seq_lens.data(), q,
                                       out, stream));
    }

    // Step E of the reference's decode driver (transformer.cpp:3882-3921) inside the absorb kernel: q is then
    // passed as the W_q projection left it.  Off by default (cpu_mla_attention takes rotated queries).
    auto set_q_rope_in_kernel(bool on) -> Status { return c_.wrap(mla_set_q_rope(c_.h_, on ? 1 : 0)); }

    // Decode-step scheduler: begin -> per layer (append, attend) -> end.
    auto step_begin(std::span<const uint32_t> seq_ids, std::span<const uint32_t> n_new = {}, void* stream = nullptr)
        -> Status
    {
        return c_.wrap(mla_step_begin(c_.h_, uint32_t(seq_ids.size()), seq_ids.data(),
                                      n_new.empty() ? nullptr : n_new.data(), stream));
    }
    auto step_append(uint32_t layer, const void* kv_a, void* stream = nullptr) -> Status
    {
        return c_.wrap(mla_step_append(c_.h_, layer, kv_a, stream));
    }
    auto step_attend(uint32_t layer, const void* q, void* out, void* stream = nullptr) -> Status
    {
        return c_.wrap(mla_step_attend(c_.h_, layer, q, out, stream));
    }
    auto step_layer_host(uint32_t layer, const void* kv_a, const void* q, void* out, void* stream = nullptr) -> Status
    {
        return c_.wrap(mla_step_layer_host(c_.h_, layer, kv_a, q, out, stream));
    }
    auto step_end() -> Status { return c_.wrap(mla_step_end(c_.h_)); }

    // Fails if any kernel raised the device status word since the last call.
    auto check_device(void* stream = nullptr) -> Status
    {
        uint32_t st = 0;
        return c_.wrap(mla_status(c_.h_, stream, &st));
    }

private:
    LatentKVCache& c_;
};

}  // namespace mugen::mla
