// TEST INFRASTRUCTURE ONLY — never linked into, imported by or called from the product path.
//
// Builds the reference's own CPU MLA code into a shared object so that the CPU
// restatement in mla_oracle.cpp (and, through it, the CUDA kernels) can be
// checked against the real thing.  The reference sources are compiled where
// they lie (REF_ROOT, passed by the Makefile as include paths); nothing is
// copied.  Functions reached:
//   * mugen::TransformerModel::Impl::cpu_mla_attention   src/core/model/transformer.cpp:2539-2623
//   * mugen::yarn_rope_freq (file-static)                 src/core/model/transformer.cpp:41-70
//   * mugen::KVCache (sequence-length bookkeeping)        src/core/memory/kv_cache.cpp
// cpu_mla_attention is a member of a private nested struct, hence the build flag
// -fno-access-control and the #include of the .cpp itself.  The Metal device
// abstraction it is written against is replaced by the host stand-ins below
// (on Apple unified memory a "buffer" is plain host memory, so buffer_contents
// is the identity).
#include "core/model/transformer.cpp"

#include <cstdlib>
#include <thread>

namespace mugen {

struct MetalCompute::Impl {};
MetalCompute::MetalCompute() = default;
MetalCompute::~MetalCompute() = default;

auto MetalCompute::buffer_contents(void* buffer) const -> void* { return buffer; }
auto MetalCompute::read_buffer(void* buffer, void* dst, size_t bytes) const -> bool {
    std::memcpy(dst, buffer, bytes);
    return true;
}
auto MetalCompute::create_buffer(size_t bytes, bool) -> void* { return std::calloc(1, bytes); }
auto MetalCompute::create_buffer_from_data(const void* data, size_t bytes) -> void* {
    void* p = std::malloc(bytes);
    std::memcpy(p, data, bytes);
    return p;
}
auto MetalCompute::create_buffer_nocopy(void* data, size_t) -> void* { return data; }
auto MetalCompute::compile_library(const std::string&, const std::string&)
    -> std::expected<void*, std::string> { return std::unexpected("no Metal on this host"); }
auto MetalCompute::get_function(void*, const std::string&)
    -> std::expected<void*, std::string> { return std::unexpected("no Metal on this host"); }
auto MetalCompute::create_pipeline(void*)
    -> std::expected<void*, std::string> { return std::unexpected("no Metal on this host"); }
auto MetalCompute::dispatch_sync(const DispatchParams&)
    -> std::expected<double, std::string> { return std::unexpected("no Metal on this host"); }
auto MetalCompute::dispatch_chain_sync(const std::vector<std::vector<DispatchParams>>&)
    -> std::expected<double, std::string> { return std::unexpected("no Metal on this host"); }

auto BufferManager::find_expert(const ExpertKey&) const -> const void* { return nullptr; }
auto MmapLoader::is_page_aligned(const void*) -> bool { return false; }
auto GGUFParser::tensor_by_name(std::string_view) const -> const TensorInfo* { return nullptr; }

}  // namespace mugen

namespace {

struct RefCall {
    mugen::MetalCompute gpu;
    mugen::TransformerModel::Impl impl;
    mugen::LayerWeights lw;
};

void fill(RefCall& rc, uint32_t n_heads, uint32_t max_seq, const void* cache,
          const void* w_uk, const void* w_uv, uint32_t w_type)
{
    auto& c = rc.impl.cfg;
    c = mugen::ModelConfig{};
    c.n_heads = n_heads;
    c.n_layers = 1;
    c.kv_lora_rank = 512;
    c.qk_nope_head_dim = 128;
    c.qk_rope_head_dim = 64;
    c.v_head_dim = 128;
    rc.impl.gpu = &rc.gpu;
    rc.impl.buf_kv_compressed = {const_cast<void*>(cache)};
    rc.impl.scratch_scores_.assign(max_seq, 0.0f);
    rc.lw.attn_k_b_buf = const_cast<void*>(w_uk);
    rc.lw.attn_v_b_buf = const_cast<void*>(w_uv);
    rc.lw.attn_k_b_type = static_cast<mugen::GGMLType>(w_type);
    rc.lw.attn_v_b_type = static_cast<mugen::GGMLType>(w_type);
}

}  // namespace

extern "C" {

// GGMLType values the reference's dequant_weight_row understands.
uint32_t ref_ggml_f16()  { return static_cast<uint32_t>(mugen::GGMLType::F16); }
uint32_t ref_ggml_q8_0() { return static_cast<uint32_t>(mugen::GGMLType::Q8_0); }
uint32_t ref_ggml_q4_0() { return static_cast<uint32_t>(mugen::GGMLType::Q4_0); }

float ref_yarn_rope_freq(uint32_t dim_idx, uint32_t rope_dim, float factor,
                         uint32_t original_ctx, float theta)
{
    return mugen::yarn_rope_freq(dim_idx, rope_dim, factor, original_ctx, theta);
}

// One call of the reference attention for one sequence.
//   q      [n_heads][192] f16, cache [seq_len][576] f16 (contiguous rows),
//   w_uk / w_uv  (n_heads*128) x 512 in the given GGML type, out [n_heads][128] f16.
void ref_mla_attention(const void* q, const void* cache, uint32_t seq_len,
                       const void* w_uk, const void* w_uv, uint32_t w_type,
                       uint32_t n_heads, void* out)
{
    RefCall rc;
    fill(rc, n_heads, seq_len, cache, w_uk, w_uv, w_type);
    rc.impl.cpu_mla_attention(static_cast<const mugen::f16*>(q), rc.lw, 0, seq_len,
                              static_cast<mugen::f16*>(out));
}

// The same call over n_seq independent sequences on n_threads host threads (one
// Impl, hence one score scratch, per thread).  cache_ptrs[i] / seq_lens[i] per
// sequence; q is [n_seq][n_heads][192], out is [n_seq][n_heads][128].
void ref_mla_attention_batch(const void* q, const void* const* cache_ptrs,
                             const uint32_t* seq_lens, uint32_t n_seq,
                             const void* w_uk, const void* w_uv, uint32_t w_type,
                             uint32_t n_heads, void* out, uint32_t n_threads)
{
    if (n_threads == 0) n_threads = 1;
    auto worker = [&](uint32_t tid) {
        for (uint32_t s = tid; s < n_seq; s += n_threads) {
            RefCall rc;
            fill(rc, n_heads, seq_lens[s], cache_ptrs[s], w_uk, w_uv, w_type);
            const auto* qs = static_cast<const mugen::f16*>(q) + size_t(s) * n_heads * 192;
            auto* os = static_cast<mugen::f16*>(out) + size_t(s) * n_heads * 128;
            rc.impl.cpu_mla_attention(qs, rc.lw, 0, seq_lens[s], os);
        }
    };
    std::vector<std::thread> pool;
    for (uint32_t t = 1; t < n_threads; t++) pool.emplace_back(worker, t);
    worker(0);
    for (auto& th : pool) th.join();
}

// The reference KVCache in the degenerate shape the MLA model builds it with
// (src/core/model/transformer.cpp:3367-3379): a sequence-length counter.
void* ref_kvcache_create(uint32_t n_layers, uint32_t max_seq_len)
{
    mugen::KVCacheConfig kc{};
    kc.n_layers = n_layers;
    kc.n_kv_heads = 1;
    kc.head_dim = 1;
    kc.max_seq_len = max_seq_len;
    kc.quantize_4bit = true;
    kc.fp16_preserve_last = 256;
    auto r = mugen::KVCache::create(kc);
    if (!r) return nullptr;
    return r->release();
}
void ref_kvcache_destroy(void* p) { delete static_cast<mugen::KVCache*>(p); }
uint32_t ref_kvcache_seq_len(void* p) { return static_cast<mugen::KVCache*>(p)->seq_len(); }
void ref_kvcache_advance(void* p, uint32_t n) { static_cast<mugen::KVCache*>(p)->advance_seq_len(n); }
void ref_kvcache_truncate(void* p, uint32_t n) { static_cast<mugen::KVCache*>(p)->truncate(n); }
void ref_kvcache_clear(void* p) { static_cast<mugen::KVCache*>(p)->clear(); }

}  // extern "C"
