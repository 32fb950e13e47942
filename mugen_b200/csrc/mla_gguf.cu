// GGUF ingestion for the MLA path (C ABI, host code only): the attention shape of a deepseek2 model file into an
// mla_config, and its per-layer W_UK / W_UV / kv_a-norm tensors into a context.  The file reader is
// host/gguf_reader.hpp; this file maps its results onto the library's own entry points.
#include "../../include/mugen_mla.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <memory>
#include <string>
#include <vector>

#include "../host/gguf_reader.hpp"

using mugen::mla::GgufFile;

struct mla_gguf {
    GgufFile file;
};

namespace {

thread_local std::string g_gguf_error;

int gfail(int code, std::string msg)
{
    g_gguf_error = std::move(msg);
    return code;
}

// W_UK / W_UV of a layer as mla_set_layer_weights takes them; F32 tensors become half first, which is what the
// reference's loader does with an F32 weight (src/core/model/transformer.cpp:3131-3134).
int layer_weights(mla_gguf* g, uint32_t layer, std::vector<uint8_t>& w_uk, std::vector<uint8_t>& w_uv, uint32_t& w_type)
{
    uint32_t type = 0;
    if (!g->file.layer_kv_b(layer, w_uk, w_uv, type)) return gfail(MLA_ERR_INVALID, g->file.error());
    auto to_half = [](std::vector<uint8_t>& w) {
        const size_t n = w.size() / 4;
        std::vector<uint8_t> h(n * 2);
        for (size_t i = 0; i < n; i++) {
            float f;
            std::memcpy(&f, w.data() + 4 * i, 4);
            const uint16_t b = __half_as_ushort(__float2half_rn(f));
            std::memcpy(h.data() + 2 * i, &b, 2);
        }
        w.swap(h);
    };
    switch (type) {
        case mugen::mla::GGML_F32: to_half(w_uk); to_half(w_uv); w_type = MLA_W_F16; break;
        case mugen::mla::GGML_F16: w_type = MLA_W_F16; break;
        case mugen::mla::GGML_BF16: w_type = MLA_W_BF16; break;
        case mugen::mla::GGML_Q8_0: w_type = MLA_W_Q8_0; break;
        case mugen::mla::GGML_Q4_0: w_type = MLA_W_Q4_0; break;
        default: return gfail(MLA_ERR_UNSUPPORTED, "tensor type " + std::to_string(type) + " is not one of F32, F16, BF16, Q8_0, Q4_0");
    }
    return MLA_OK;
}

}  // namespace

extern "C" {

const char* mla_gguf_last_error(void) { return g_gguf_error.c_str(); }

int mla_gguf_open(const char* path, mla_gguf** out)
{
    if (!path || !out) return gfail(MLA_ERR_INVALID, "null argument");
    *out = nullptr;
    auto g = std::make_unique<mla_gguf>();
    if (!g->file.open(path)) return gfail(MLA_ERR_INVALID, g->file.error());
    *out = g.release();
    return MLA_OK;
}

void mla_gguf_close(mla_gguf* g) { delete g; }

int mla_gguf_get_info(const mla_gguf* g, mla_gguf_info* info)
{
    if (!g || !info) return gfail(MLA_ERR_INVALID, "null argument");
    const auto& c = g->file.info();
    *info = mla_gguf_info{c.n_layers, c.n_heads, c.embed, c.context_length, c.kv_lora_rank, c.q_lora_rank, c.qk_nope, c.qk_rope,
                          c.v_head_dim, c.rope_original_ctx, c.rope_theta, c.rope_scaling_factor, c.rms_norm_eps};
    return MLA_OK;
}

int mla_gguf_fill_config(const mla_gguf* g, mla_config* cfg)
{
    if (!g || !cfg) return gfail(MLA_ERR_INVALID, "null argument");
    const auto& c = g->file.info();
    cfg->n_layers = c.n_layers;
    cfg->n_heads = c.n_heads;
    cfg->kv_lora_rank = c.kv_lora_rank;
    cfg->qk_nope_head_dim = c.qk_nope;
    cfg->qk_rope_head_dim = c.qk_rope;
    cfg->v_head_dim = c.v_head_dim;
    cfg->rope_theta = c.rope_theta;
    cfg->rms_norm_eps = c.rms_norm_eps;
    cfg->rope_scaling_factor = c.rope_scaling_factor;
    cfg->rope_original_ctx = c.rope_original_ctx;
    if (cfg->max_seq_len == 0) cfg->max_seq_len = c.context_length ? c.context_length : 8192;   // the reference's default
    return MLA_OK;
}

int mla_gguf_layer_weights(mla_gguf* g, uint32_t layer, void* w_uk, void* w_uv, size_t capacity_each, uint32_t* w_type,
                           size_t* bytes_each, uint16_t* kv_norm_f16)
{
    if (!g || !w_type || !bytes_each) return gfail(MLA_ERR_INVALID, "null argument");
    if (layer >= g->file.info().n_layers) return gfail(MLA_ERR_INVALID, "layer out of range");
    std::vector<uint8_t> k, v;
    if (int e = layer_weights(g, layer, k, v, *w_type)) return e;
    if (k.size() != v.size()) return gfail(MLA_ERR_UNSUPPORTED, "W_UK and W_UV differ in size (qk_nope_head_dim != v_head_dim)");
    *bytes_each = k.size();
    if (w_uk && w_uv) {
        if (capacity_each < k.size()) return gfail(MLA_ERR_CAPACITY, "weight buffers too small: need " + std::to_string(k.size()) + " bytes each");
        std::memcpy(w_uk, k.data(), k.size());
        std::memcpy(w_uv, v.data(), v.size());
    }
    if (kv_norm_f16) {
        std::vector<float> nw;
        if (!g->file.layer_kv_a_norm(layer, nw)) return gfail(MLA_ERR_INVALID, g->file.error());
        for (size_t i = 0; i < nw.size(); i++) kv_norm_f16[i] = __half_as_ushort(__float2half_rn(nw[i]));
    }
    return MLA_OK;
}

int mla_gguf_register(mla_ctx* ctx, mla_gguf* g, uint32_t ctx_dtype)
{
    if (!ctx || !g) return gfail(MLA_ERR_INVALID, "null argument");
    const auto& c = g->file.info();
    for (uint32_t layer = 0; layer < c.n_layers; layer++) {
        std::vector<uint8_t> k, v;
        uint32_t w_type = 0;
        if (int e = layer_weights(g, layer, k, v, w_type)) return e;
        std::vector<float> nw;
        if (!g->file.layer_kv_a_norm(layer, nw)) return gfail(MLA_ERR_INVALID, g->file.error());
        std::vector<uint16_t> norm(nw.size());
        for (size_t i = 0; i < nw.size(); i++)
            norm[i] = ctx_dtype == MLA_DTYPE_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(nw[i]))
                                                  : __half_as_ushort(__float2half_rn(nw[i]));
        if (int e = mla_set_layer_weights(ctx, layer, k.data(), v.data(), w_type, norm.data()))
            return gfail(e, std::string("layer ") + std::to_string(layer) + ": " + mla_last_error(ctx));
    }
    return MLA_OK;
}

}  // extern "C"
