// Reader of the parts of a GGUF model file that the MLA path needs: the attention shape and RoPE
// metadata of a `deepseek2` model and, per layer, the W_UK / W_UV / kv_a-norm tensors.  Pure C++ (no
// CUDA) so it is unit-tested without a device.
//
// What it takes over from the reference: the MLA metadata keys of TransformerModel::from_gguf_impl
// (src/core/model/transformer.cpp:2951-3011), the attn_k_b / attn_v_b loading and the split of a merged
// attn_kv_b tensor whose rows per head are [qk_nope rows | v_head_dim rows] (:3178-3221), and the
// conversion of F32 norm weights to half at load (:2850-2869).  File layout per the GGUF specification
// (the reference's own reader is src/model/gguf_parser.cpp:158-330): magic, version, counts, key/value
// pairs, tensor infos with dimensions innermost first, data section aligned to general.alignment (32).
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace mugen::mla {

enum : uint32_t { GGML_F32 = 0, GGML_F16 = 1, GGML_Q4_0 = 2, GGML_Q8_0 = 8, GGML_BF16 = 30 };

struct GgufTensor {
    std::vector<uint64_t> dims;      // innermost first
    uint32_t type = 0;
    uint64_t offset = 0;             // from the start of the data section
};

struct GgufMlaInfo {
    std::string arch;
    uint32_t n_layers = 0, n_heads = 0, embed = 0, context_length = 0;
    uint32_t kv_lora_rank = 0, q_lora_rank = 0, qk_rope = 0, qk_nope = 0, v_head_dim = 0;
    float rope_theta = 10000.0f, rope_scaling_factor = 0.0f, rms_norm_eps = 1e-5f;
    uint32_t rope_original_ctx = 0;
};

class GgufFile {
public:
    ~GgufFile() { close(); }
    GgufFile() = default;
    GgufFile(const GgufFile&) = delete;
    GgufFile& operator=(const GgufFile&) = delete;

    const std::string& error() const { return err_; }
    const GgufMlaInfo& info() const { return info_; }
    const GgufTensor* tensor(const std::string& name) const {
        auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }

    bool open(const char* path) {
        close();
        fd_ = ::open(path, O_RDONLY);
        if (fd_ < 0) return fail(std::string("cannot open ") + path);
        struct stat st {};
        if (fstat(fd_, &st) != 0 || st.st_size < 24) return fail("file too small to be a GGUF file");
        size_ = size_t(st.st_size);
        void* p = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (p == MAP_FAILED) { base_ = nullptr; return fail("mmap failed"); }
        base_ = static_cast<const uint8_t*>(p);
        pos_ = 0;
        uint32_t magic = 0, version = 0;
        uint64_t n_tensors = 0, n_kv = 0;
        if (!rd(magic) || magic != 0x46554747u) return fail("not a GGUF file (bad magic)");
        if (!rd(version) || version < 2 || version > 3) return fail("unsupported GGUF version " + std::to_string(version));
        if (!rd(n_tensors) || !rd(n_kv) || n_tensors > (1u << 24) || n_kv > (1u << 20)) return fail("implausible GGUF counts");
        uint64_t alignment = 32;
        for (uint64_t i = 0; i < n_kv; i++) {
            std::string key;
            uint32_t vt = 0;
            if (!rd_str(key) || !rd(vt)) return fail("truncated key/value section");
            if (!rd_value(key, vt)) return fail("bad value for key " + key);
        }
        if (auto it = ints_.find("general.alignment"); it != ints_.end() && it->second > 0) alignment = uint64_t(it->second);
        for (uint64_t i = 0; i < n_tensors; i++) {
            std::string name;
            uint32_t nd = 0;
            GgufTensor t;
            if (!rd_str(name) || !rd(nd) || nd > 8) return fail("truncated tensor info");
            t.dims.resize(nd);
            for (auto& d : t.dims)
                if (!rd(d)) return fail("truncated tensor info");
            if (!rd(t.type) || !rd(t.offset)) return fail("truncated tensor info");
            tensors_[name] = std::move(t);
        }
        data_ = (pos_ + alignment - 1) / alignment * alignment;
        return fill_info();
    }

    void close() {
        if (base_) munmap(const_cast<uint8_t*>(base_), size_);
        if (fd_ >= 0) ::close(fd_);
        base_ = nullptr;
        fd_ = -1;
        tensors_.clear();
        ints_.clear();
        floats_.clear();
        strings_.clear();
    }

    // bytes of `rows` rows of 512 values in a GGML type this path can decode; 0 = unsupported
    static size_t row_bytes_512(uint32_t type) {
        switch (type) {
            case GGML_F16: case GGML_BF16: return 512 * 2;
            case GGML_F32: return 512 * 4;
            case GGML_Q8_0: return 512 / 32 * 34;
            case GGML_Q4_0: return 512 / 32 * 18;
            default: return 0;
        }
    }

    // W_UK ((H*128) x 512) and W_UV ((H*128) x 512) of a layer in their GGML encoding, and which encoding.
    // Separate attn_k_b / attn_v_b tensors are taken as they are; a merged attn_kv_b is split per head into its
    // first qk_nope rows (W_UK) and its following v_head_dim rows (W_UV).
    bool layer_kv_b(uint32_t layer, std::vector<uint8_t>& w_uk, std::vector<uint8_t>& w_uv, uint32_t& type) {
        const std::string blk = "blk." + std::to_string(layer) + ".";
        const uint32_t H = info_.n_heads, nope = info_.qk_nope, vd = info_.v_head_dim;
        const GgufTensor* kb = tensor(blk + "attn_k_b.weight");
        const GgufTensor* vb = tensor(blk + "attn_v_b.weight");
        if (kb && vb) {
            if (kb->type != vb->type) return fail("attn_k_b and attn_v_b of layer " + std::to_string(layer) + " differ in type");
            type = kb->type;
            const size_t bpr = row_bytes_512(type);
            if (!bpr) return fail("unsupported tensor type " + std::to_string(type) + " for attn_k_b");
            if (!expect_dims(*kb, 512, uint64_t(H) * nope, blk + "attn_k_b.weight") ||
                !expect_dims(*vb, 512, uint64_t(H) * vd, blk + "attn_v_b.weight"))
                return false;
            return copy_out(*kb, size_t(H) * nope * bpr, w_uk) && copy_out(*vb, size_t(H) * vd * bpr, w_uv);
        }
        const GgufTensor* kvb = tensor(blk + "attn_kv_b.weight");
        if (!kvb) return fail("layer " + std::to_string(layer) + " has neither attn_k_b + attn_v_b nor attn_kv_b");
        type = kvb->type;
        const size_t bpr = row_bytes_512(type);
        if (!bpr) return fail("unsupported tensor type " + std::to_string(type) + " for attn_kv_b");
        if (!expect_dims(*kvb, 512, uint64_t(H) * (nope + vd), blk + "attn_kv_b.weight")) return false;
        const uint8_t* raw = at(*kvb, size_t(H) * (nope + vd) * bpr);
        if (!raw) return false;
        w_uk.resize(size_t(H) * nope * bpr);
        w_uv.resize(size_t(H) * vd * bpr);
        for (uint32_t h = 0; h < H; h++) {
            std::memcpy(w_uk.data() + size_t(h) * nope * bpr, raw + size_t(h) * (nope + vd) * bpr, size_t(nope) * bpr);
            std::memcpy(w_uv.data() + size_t(h) * vd * bpr, raw + (size_t(h) * (nope + vd) + nope) * bpr, size_t(vd) * bpr);
        }
        return true;
    }

    // attn_kv_a_norm of a layer as floats (stored F32 or F16 in the file)
    bool layer_kv_a_norm(uint32_t layer, std::vector<float>& w) {
        const std::string name = "blk." + std::to_string(layer) + ".attn_kv_a_norm.weight";
        const GgufTensor* t = tensor(name);
        if (!t) return fail("missing tensor " + name);
        if (t->dims.size() != 1 || t->dims[0] != info_.kv_lora_rank) return fail(name + " has the wrong shape");
        w.resize(info_.kv_lora_rank);
        if (t->type == GGML_F32) {
            const uint8_t* p = at(*t, w.size() * 4);
            if (!p) return false;
            std::memcpy(w.data(), p, w.size() * 4);
        } else if (t->type == GGML_F16) {
            const uint8_t* p = at(*t, w.size() * 2);
            if (!p) return false;
            for (size_t i = 0; i < w.size(); i++) {
                uint16_t hbits;
                std::memcpy(&hbits, p + 2 * i, 2);
                w[i] = half_to_float(hbits);
            }
        } else {
            return fail(name + " must be F32 or F16");
        }
        return true;
    }

    static float half_to_float(uint16_t h) {
        const uint32_t s = uint32_t(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u;
        uint32_t u;
        if (e == 0) {
            if (m == 0) u = s;
            else {
                int sh = 0;
                uint32_t mm = m;
                while (!(mm & 1024u)) { mm <<= 1; sh++; }
                u = s | ((113u - sh) << 23) | ((mm & 1023u) << 13);
            }
        } else if (e == 31) u = s | 0x7F800000u | (m << 13);
        else u = s | ((e + 112u) << 23) | (m << 13);
        float f;
        std::memcpy(&f, &u, 4);
        return f;
    }

private:
    bool fail(std::string m) { err_ = std::move(m); return false; }
    template <typename V> bool rd(V& v) {
        if (pos_ + sizeof(V) > size_) return false;
        std::memcpy(&v, base_ + pos_, sizeof(V));
        pos_ += sizeof(V);
        return true;
    }
    bool rd_str(std::string& s) {
        uint64_t n = 0;
        if (!rd(n) || n > size_ - pos_) return false;
        s.assign(reinterpret_cast<const char*>(base_ + pos_), size_t(n));
        pos_ += size_t(n);
        return true;
    }
    // reads (and keeps, for scalars and strings) one value of GGUF value type vt
    bool rd_value(const std::string& key, uint32_t vt, bool keep = true) {
        switch (vt) {
            case 0: { uint8_t v; if (!rd(v)) return false; if (keep) ints_[key] = v; return true; }
            case 1: { int8_t v; if (!rd(v)) return false; if (keep) ints_[key] = v; return true; }
            case 2: { uint16_t v; if (!rd(v)) return false; if (keep) ints_[key] = v; return true; }
            case 3: { int16_t v; if (!rd(v)) return false; if (keep) ints_[key] = v; return true; }
            case 4: { uint32_t v; if (!rd(v)) return false; if (keep) ints_[key] = v; return true; }
            case 5: { int32_t v; if (!rd(v)) return false; if (keep) ints_[key] = v; return true; }
            case 6: { float v; if (!rd(v)) return false; if (keep) floats_[key] = v; return true; }
            case 7: { uint8_t v; if (!rd(v)) return false; if (keep) ints_[key] = v ? 1 : 0; return true; }
            case 8: { std::string v; if (!rd_str(v)) return false; if (keep) strings_[key] = v; return true; }
            case 9: {
                uint32_t et = 0;
                uint64_t n = 0;
                if (!rd(et) || !rd(n) || et == 9) return false;
                for (uint64_t i = 0; i < n; i++)
                    if (!rd_value(key, et, false)) return false;
                return true;
            }
            case 10: { uint64_t v; if (!rd(v)) return false; if (keep) ints_[key] = int64_t(v); return true; }
            case 11: { int64_t v; if (!rd(v)) return false; if (keep) ints_[key] = v; return true; }
            case 12: { double v; if (!rd(v)) return false; if (keep) floats_[key] = v; return true; }
            default: return false;
        }
    }
    bool get_u32(const std::string& key, uint32_t& out) const {
        auto it = ints_.find(key);
        if (it == ints_.end()) return false;
        out = uint32_t(it->second);
        return true;
    }
    bool fill_info() {
        GgufMlaInfo& c = info_;
        c = GgufMlaInfo{};
        if (auto it = strings_.find("general.architecture"); it != strings_.end()) c.arch = it->second;
        if (c.arch.empty()) return fail("general.architecture is missing");
        const std::string a = c.arch + ".";
        get_u32(a + "block_count", c.n_layers);
        get_u32(a + "attention.head_count", c.n_heads);
        get_u32(a + "embedding_length", c.embed);
        get_u32(a + "context_length", c.context_length);
        get_u32(a + "attention.kv_lora_rank", c.kv_lora_rank);
        get_u32(a + "attention.q_lora_rank", c.q_lora_rank);
        if (c.kv_lora_rank > 0) get_u32(a + "rope.dimension_count", c.qk_rope);
        uint32_t key_length = 0;
        if (get_u32(a + "attention.key_length", key_length) && c.qk_rope > 0 && key_length > c.qk_rope)
            c.qk_nope = key_length - c.qk_rope;
        if (c.kv_lora_rank > 0) get_u32(a + "attention.value_length", c.v_head_dim);
        if (get_u32(a + "attention.key_length_mla", key_length) && c.qk_rope > 0) c.qk_nope = key_length - c.qk_rope;
        get_u32(a + "attention.value_length_mla", c.v_head_dim);
        if (auto it = floats_.find(a + "rope.freq_base"); it != floats_.end()) c.rope_theta = float(it->second);
        if (auto it = floats_.find(a + "rope.scaling.factor"); it != floats_.end()) c.rope_scaling_factor = float(it->second);
        get_u32(a + "rope.scaling.original_context_length", c.rope_original_ctx);
        if (auto it = floats_.find(a + "attention.layer_norm_rms_epsilon"); it != floats_.end()) c.rms_norm_eps = float(it->second);
        if (c.n_layers == 0 || c.n_heads == 0) return fail("block_count / attention.head_count missing");
        if (c.kv_lora_rank == 0) return fail("not an MLA model: " + a + "attention.kv_lora_rank is absent");
        return true;
    }
    bool expect_dims(const GgufTensor& t, uint64_t inner, uint64_t outer, const std::string& name) {
        if (t.dims.size() != 2 || t.dims[0] != inner || t.dims[1] != outer)
            return fail(name + " has the wrong shape");
        return true;
    }
    const uint8_t* at(const GgufTensor& t, size_t bytes) {
        if (data_ + t.offset + bytes > size_) { fail("tensor data extends past the end of the file"); return nullptr; }
        return base_ + data_ + t.offset;
    }
    bool copy_out(const GgufTensor& t, size_t bytes, std::vector<uint8_t>& out) {
        const uint8_t* p = at(t, bytes);
        if (!p) return false;
        out.assign(p, p + bytes);
        return true;
    }

    int fd_ = -1;
    const uint8_t* base_ = nullptr;
    size_t size_ = 0, pos_ = 0, data_ = 0;
    std::map<std::string, GgufTensor> tensors_;
    std::map<std::string, int64_t> ints_;
    std::map<std::string, double> floats_;
    std::map<std::string, std::string> strings_;
    GgufMlaInfo info_;
    std::string err_;
};

}  // namespace mugen::mla
