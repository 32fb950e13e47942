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
//   * mugen::TransformerModel::from_gguf_impl + forward() src/core/model/transformer.cpp:2899-3430, 3564-4455
//     on a tiny synthetic deepseek2 GGUF file: the MLA metadata keys, the attn_kv_b split, and above all the
//     inline append (RMSNorm + NeoX/YaRN RoPE + scatter, :3930-3987) and q RoPE (:3882-3921) of the decode driver,
//     which are not callable functions
// cpu_mla_attention is a member of a private nested struct, hence the build flag
// -fno-access-control and the #include of the .cpp itself.  The Metal device
// abstraction it is written against is replaced by the host stand-ins below
// (on Apple unified memory a "buffer" is plain host memory, so buffer_contents
// is the identity).
#include "core/model/transformer.cpp"

#include <cmath>
#include <cstdlib>
#include <fstream>
#include <functional>
#include <thread>

// ---- host stand-ins for the Metal device abstraction -------------------------------------------------
// A "buffer" is plain host memory (on Apple unified memory buffer_contents is the identity as well).  A
// "pipeline" is a pointer to the kernel's name, and dispatch_sync interprets DispatchParams for the few
// kernels the MLA decode branch of forward() launches (src/core/model/transformer.cpp:3839-4200):
// rms_norm, matvec_f16, scatter_kv, elementwise_add, silu_mul, embedding_lookup.  Their arithmetic is a
// plain C++ restatement of the MSL sources (src/metal/kernel_sources.h:55-98, 260-315, 357-390, 1555-1570,
// 3003-3014) — the shaders themselves cannot run on this host.  Where MSL leaves the order of a reduction to
// the hardware (simd_sum) the restatement adds lanes in index order.  These stand-ins only FEED the code under
// test (the inline append, steps G+H, and the q RoPE, step E, which are host C++ in the reference and run
// unmodified); taps record what that code read and wrote.
namespace {

const char* const kKernelNames[] = {
    "rms_norm", "matvec_f16", "matvec_q4_0", "matvec_q4_k", "matvec_q8_0", "softmax", "rope", "silu",
    "elementwise_mul", "elementwise_add", "embedding_lookup", "moe_gate", "moe_gate_grouped", "moe_reduce",
    "attention_decode", "matmul_f16", "matmul_q4_0", "matmul_f16_naive", "matmul_q4_0_naive", "batch_rope",
    "bias_broadcast", "prefill_attention", "flash_prefill_attention", "flash_attention_decode", "scatter_kv",
    "silu_mul", "argmax_f16"};

// observers installed by ref_model_forward (single-threaded use)
std::function<void(void* buffer, size_t bytes)> g_on_read;
std::function<void(const mugen::MetalCompute::DispatchParams&, const char* kernel, bool after)> g_on_dispatch;

template <typename T> T constant_of(const mugen::MetalCompute::DispatchParams& dp, size_t i) {
    T v;
    std::memcpy(&v, dp.constants[i].first, sizeof(T));
    return v;
}

using mugen::f16;

void host_rms_norm(const mugen::MetalCompute::DispatchParams& dp)
{
    const auto* in = static_cast<const f16*>(dp.buffers[0]);
    const auto* w = static_cast<const f16*>(dp.buffers[1]);
    auto* out = static_cast<f16*>(dp.buffers[2]);
    const uint32_t n = constant_of<uint32_t>(dp, 0);
    const float eps = constant_of<float>(dp, 1);
    const size_t tg = dp.group_size[0];
    const size_t rows = std::max<size_t>(1, dp.grid_size[0] / tg);
    for (size_t r = 0; r < rows; r++) {
        // thread t adds elements t, t+tg, ...; 32-lane groups are summed, then the group sums
        std::vector<float> part(tg, 0.0f);
        for (size_t t = 0; t < tg; t++)
            for (size_t i = t; i < n; i += tg) {
                const float v = static_cast<float>(in[r * n + i]);
                part[t] += v * v;
            }
        float total = 0.0f;
        for (size_t g = 0; g < tg; g += 32) {
            float gs = 0.0f;
            for (size_t l = g; l < std::min(tg, g + 32); l++) gs += part[l];
            total += gs;
        }
        const float inv = 1.0f / std::sqrt(total / static_cast<float>(n) + eps);
        for (size_t i = 0; i < n; i++)
            out[r * n + i] = static_cast<f16>(static_cast<float>(in[r * n + i]) * inv * static_cast<float>(w[i]));
    }
}

void host_matvec_f16(const mugen::MetalCompute::DispatchParams& dp)
{
    const auto* mat = static_cast<const f16*>(dp.buffers[0]);
    const auto* vec = static_cast<const f16*>(dp.buffers[1]);
    auto* out = static_cast<f16*>(dp.buffers[2]);
    const uint32_t m = constant_of<uint32_t>(dp, 0), k = constant_of<uint32_t>(dp, 1);
    for (uint32_t r = 0; r < m; r++) {
        float lane[32] = {0.0f};
        for (uint32_t c = 0; c < k; c++) lane[c % 32] += static_cast<float>(mat[size_t(r) * k + c]) * static_cast<float>(vec[c]);
        float acc = 0.0f;
        for (float v : lane) acc += v;
        out[r] = static_cast<f16>(acc);
    }
}

auto host_dispatch(const mugen::MetalCompute::DispatchParams& dp) -> std::expected<double, std::string>
{
    const char* name = static_cast<const char*>(dp.pipeline);
    if (!name) return std::unexpected("dispatch without a pipeline");
    const std::string k(name);
    if (g_on_dispatch) g_on_dispatch(dp, name, false);
    if (k == "rms_norm") host_rms_norm(dp);
    else if (k == "matvec_f16") host_matvec_f16(dp);
    else if (k == "scatter_kv") {
        const auto* src = static_cast<const f16*>(dp.buffers[0]);
        auto* dst = static_cast<f16*>(dp.buffers[1]);
        const uint32_t off = constant_of<uint32_t>(dp, 0), cnt = constant_of<uint32_t>(dp, 1);
        for (uint32_t i = 0; i < cnt; i++) dst[size_t(off) + i] = src[i];
    } else if (k == "elementwise_add" || k == "elementwise_mul") {
        const auto* a = static_cast<const f16*>(dp.buffers[0]);
        const auto* b = static_cast<const f16*>(dp.buffers[1]);
        auto* o = static_cast<f16*>(dp.buffers[2]);
        const uint32_t n = constant_of<uint32_t>(dp, 0);
        for (uint32_t i = 0; i < n; i++) o[i] = k == "elementwise_add" ? a[i] + b[i] : a[i] * b[i];
    } else if (k == "silu_mul") {
        const auto* g = static_cast<const f16*>(dp.buffers[0]);
        const auto* u = static_cast<const f16*>(dp.buffers[1]);
        auto* o = static_cast<f16*>(dp.buffers[2]);
        const uint32_t n = constant_of<uint32_t>(dp, 0);
        for (uint32_t i = 0; i < n; i++) {
            const float x = static_cast<float>(g[i]);
            o[i] = static_cast<f16>((x / (1.0f + std::exp(-x))) * static_cast<float>(u[i]));
        }
    } else if (k == "embedding_lookup") {
        const auto* table = static_cast<const f16*>(dp.buffers[0]);
        const auto* ids = static_cast<const uint32_t*>(dp.buffers[1]);
        auto* o = static_cast<f16*>(dp.buffers[2]);
        const uint32_t dim = constant_of<uint32_t>(dp, 0), n = constant_of<uint32_t>(dp, 1);
        for (uint32_t t = 0; t < n; t++)
            for (uint32_t i = 0; i < dim; i++) o[size_t(t) * dim + i] = table[size_t(ids[t]) * dim + i];
    } else {
        return std::unexpected("kernel '" + k + "' has no host restatement in this harness");
    }
    if (g_on_dispatch) g_on_dispatch(dp, name, true);
    return 0.0;
}

}  // namespace

namespace mugen {

struct MetalCompute::Impl {};
MetalCompute::MetalCompute() = default;
MetalCompute::~MetalCompute() = default;

auto MetalCompute::buffer_contents(void* buffer) const -> void* { return buffer; }
auto MetalCompute::read_buffer(void* buffer, void* dst, size_t bytes) const -> bool {
    if (g_on_read) g_on_read(buffer, bytes);
    std::memcpy(dst, buffer, bytes);
    return true;
}
auto MetalCompute::create_buffer(size_t bytes, bool) -> void* { return std::calloc(1, bytes ? bytes : 1); }
auto MetalCompute::create_buffer_from_data(const void* data, size_t bytes) -> void* {
    void* p = std::malloc(bytes ? bytes : 1);
    std::memcpy(p, data, bytes);
    return p;
}
auto MetalCompute::create_buffer_nocopy(void* data, size_t) -> void* { return data; }
auto MetalCompute::compile_library(const std::string&, const std::string&)
    -> std::expected<void*, std::string> { return const_cast<char*>("host kernel table"); }
auto MetalCompute::get_function(void*, const std::string& name)
    -> std::expected<void*, std::string> {
    for (const char* k : kKernelNames)
        if (name == k) return const_cast<char*>(k);
    return std::unexpected("unknown kernel " + name);
}
auto MetalCompute::create_pipeline(void* function)
    -> std::expected<void*, std::string> { return function; }
auto MetalCompute::dispatch_sync(const DispatchParams& dp)
    -> std::expected<double, std::string> { return host_dispatch(dp); }
auto MetalCompute::dispatch_chain_sync(const std::vector<std::vector<DispatchParams>>& groups)
    -> std::expected<double, std::string> {
    for (const auto& g : groups)
        for (const auto& dp : g)
            if (auto r = host_dispatch(dp); !r) return r;
    return 0.0;
}

auto BufferManager::find_expert(const ExpertKey&) const -> const void* { return nullptr; }
auto MmapLoader::is_page_aligned(const void*) -> bool { return false; }

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

// ---- the reference model on a GGUF file --------------------------------------------------------------
struct RefModel {
    mugen::MetalCompute gpu;
    std::vector<char> file;                                // the GGUF bytes (stands in for the mmap)
    std::unique_ptr<mugen::TransformerModel> model;
    std::string error;
};

static std::string g_model_error;
const char* ref_model_last_error() { return g_model_error.c_str(); }

// Parses the file with the reference's GGUFParser and builds the model with from_gguf_impl.
void* ref_model_load(const char* path)
{
    auto parsed = mugen::GGUFParser::parse(path);
    if (!parsed) { g_model_error = "parse: " + parsed.error(); return nullptr; }
    auto rm = std::make_unique<RefModel>();
    std::ifstream f(path, std::ios::binary);
    rm->file.assign(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
    auto m = mugen::TransformerModel::from_gguf_impl(&rm->gpu, *parsed, {rm->file.data()});
    if (!m) { g_model_error = "from_gguf: " + m.error(); return nullptr; }
    rm->model = std::move(*m);
    return rm.release();
}
void ref_model_free(void* h) { delete static_cast<RefModel*>(h); }

// cfg[0..11] = n_layers, n_heads, embed_dim, kv_lora_rank, q_lora_rank, qk_nope, qk_rope, v_head_dim,
// rope_original_ctx, max_seq_len, vocab, ffn_dim; fcfg[0..2] = rope_theta, rope_scaling_factor, rms_norm_eps
void ref_model_config(void* h, uint32_t* cfg, float* fcfg)
{
    auto& d = *static_cast<RefModel*>(h)->model->impl_;
    const auto& c = d.cfg;
    const uint32_t v[12] = {c.n_layers, c.n_heads, c.embed_dim, c.kv_lora_rank, c.q_lora_rank, c.qk_nope_head_dim,
                            c.qk_rope_head_dim, c.v_head_dim, c.rope_original_ctx, d.kv_cache->config().max_seq_len,
                            c.vocab_size, c.ffn_dim};
    std::memcpy(cfg, v, sizeof(v));
    fcfg[0] = c.rope_theta; fcfg[1] = c.rope_scaling_factor; fcfg[2] = c.rms_norm_eps;
}

// Copies a layer's weight as the loaded model holds it.  which: 0 = W_UK (attn_k_b, after any split of attn_kv_b),
// 1 = W_UV, 2 = kv_a norm, 3 = attn_kv_a_mqa, 4 = attn_q_a, 5 = attn_q_a_norm, 6 = attn_q_b, 7 = attn_q (no LoRA),
// 8 = attn_output, 9 = attn_norm.  Returns the GGML type (norms: F16) or 0xFFFFFFFF when absent.
uint32_t ref_model_weight(void* h, uint32_t layer, uint32_t which, void* out, size_t bytes)
{
    auto& d = *static_cast<RefModel*>(h)->model->impl_;
    auto& lw = d.layers[layer];
    void* src = nullptr;
    uint32_t type = static_cast<uint32_t>(mugen::GGMLType::F16);
    switch (which) {
        case 0: src = lw.attn_k_b_buf; type = static_cast<uint32_t>(lw.attn_k_b_type); break;
        case 1: src = lw.attn_v_b_buf; type = static_cast<uint32_t>(lw.attn_v_b_type); break;
        case 2: src = lw.attn_kv_a_norm_buf; break;
        case 3: src = lw.attn_kv_a_mqa_buf; type = static_cast<uint32_t>(lw.attn_kv_a_mqa_type); break;
        case 4: src = lw.attn_q_a_buf; type = static_cast<uint32_t>(lw.attn_q_a_type); break;
        case 5: src = lw.attn_q_a_norm_buf; break;
        case 6: src = lw.attn_q_b_buf; type = static_cast<uint32_t>(lw.attn_q_b_type); break;
        case 7: src = lw.wq_buf; type = static_cast<uint32_t>(lw.wq_type); break;
        case 8: src = lw.wo_buf; type = static_cast<uint32_t>(lw.wo_type); break;
        case 9: src = lw.attn_norm_buf; break;
        default: break;
    }
    if (!src) return 0xFFFFFFFFu;
    std::memcpy(out, src, bytes);
    return type;
}

// One decode call of the reference's forward() for `token` at `pos`, with taps.  Per layer the taps record
//   hidden_in   [embed]      input of the attention RMSNorm (step A)
//   q_pre       [H][192]     q as the projection left it, read by step E
//   q_post      [H][192]     q after the reference's RoPE loop, read by step I
//   kv_a_pre    [576]        kv_a as the W_kv_a projection left it, read by step G
//   attn_out    [H][128]     output of cpu_mla_attention, input of Wo (step J)
//   hidden_mid  [embed]      hidden state after Wo + residual (input of the FFN RMSNorm, step L)
// Each output array is [n_layers][...] f16; any may be NULL.  Returns 0, or 1 with ref_model_last_error().
int ref_model_forward(void* h, uint32_t token, uint32_t pos, void* hidden_in, void* q_pre, void* q_post,
                      void* kv_a_pre, void* attn_out, void* hidden_mid)
{
    auto* rm = static_cast<RefModel*>(h);
    auto& d = *rm->model->impl_;
    const auto& c = d.cfg;
    const size_t E = c.embed_dim, QD = size_t(c.n_heads) * (c.qk_nope_head_dim + c.qk_rope_head_dim),
                 KD = c.kv_lora_rank + c.qk_rope_head_dim, OD = size_t(c.n_heads) * c.v_head_dim;
    int layer = -1;
    int q_reads = 0;
    auto put = [&](void* dst, size_t per_layer, const void* src) {
        if (dst && layer >= 0) std::memcpy(static_cast<mugen::f16*>(dst) + size_t(layer) * per_layer, src, per_layer * 2);
    };
    g_on_dispatch = [&](const mugen::MetalCompute::DispatchParams& dp, const char* kernel, bool after) {
        const std::string k(kernel);
        if (!after && k == "rms_norm") {
            for (uint32_t L = 0; L < c.n_layers; L++) {
                if (dp.buffers[1] == d.layers[L].attn_norm_buf) { layer = int(L); q_reads = 0; put(hidden_in, E, dp.buffers[0]); }
                else if (dp.buffers[1] == d.layers[L].ffn_norm_buf) put(hidden_mid, E, dp.buffers[0]);
            }
        }
        if (!after && k.rfind("matvec", 0) == 0 && dp.buffers[1] == d.buf_mla_attn_out) put(attn_out, OD, dp.buffers[1]);
    };
    g_on_read = [&](void* buffer, size_t) {
        if (buffer == d.buf_mla_kv_a) put(kv_a_pre, KD, buffer);
        else if (buffer == d.buf_mla_q) { put(q_reads == 0 ? q_pre : q_post, QD, buffer); q_reads++; }
    };
    auto r = rm->model->forward({token}, pos);
    g_on_dispatch = nullptr;
    g_on_read = nullptr;
    if (!r) { g_model_error = "forward: " + r.error(); return 1; }
    return 0;
}

// Latent cache rows [row_begin, row_begin + n) of a layer as the reference wrote them (f16 [n][576]).
void ref_model_cache_rows(void* h, uint32_t layer, uint32_t row_begin, uint32_t n, void* out)
{
    auto& d = *static_cast<RefModel*>(h)->model->impl_;
    const size_t KD = d.cfg.kv_lora_rank + d.cfg.qk_rope_head_dim;
    std::memcpy(out, static_cast<const mugen::f16*>(d.buf_kv_compressed[layer]) + size_t(row_begin) * KD, size_t(n) * KD * 2);
}
uint32_t ref_model_seq_len(void* h) { return static_cast<RefModel*>(h)->model->impl_->kv_cache->seq_len(); }
void ref_model_truncate(void* h, uint32_t n) { static_cast<RefModel*>(h)->model->impl_->kv_cache->truncate(n); }

}  // extern "C"
