// C ABI of the B200 MLA decode path (see include/mugen_mla.h): context, paged latent cache,
// per-step scheduling metadata, kernel dispatch.  Host logic only; kernels live beside it.
#include "../../include/mugen_mla.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../host/page_table.hpp"
#include "../host/rope_table.hpp"
#include "mla_launch.h"

using mugen::mla::PageTable;
using mugen::mla::Segment;

namespace {

thread_local std::string g_create_error;

constexpr int kMetaRing = 4;

struct LayerW {
    void* w_uk = nullptr;   // stored transposed per head: [h][512][128]
    void* w_uk_rows = nullptr;   // as registered, (H*128) x 512: the prefill path expands keys with it
    void* w_uv = nullptr;
    void* norm = nullptr;
    bool set = false;
    // W_UV as ([H*128 outputs][512 dims]) with a box of 64 dims x 128 outputs, for the tcgen05 merge kernel
    alignas(64) CUtensorMap w_uv_map;
    // W_UK^T as ([H*512 d][128 i]) with a box of 64 i x 256 d, for the tcgen05 absorb kernel
    alignas(64) CUtensorMap w_uk_map;
    bool has_map = false;
};

// projection weights of one layer's attention block (mla_set_block_weights), all in the storage type on the device
struct BlockW {
    uint32_t embed = 0, q_lora = 0;
    void *attn_norm = nullptr, *q_a = nullptr, *q_a_norm = nullptr, *q_b = nullptr, *q = nullptr, *kv_a = nullptr, *wo = nullptr;
    bool set = false;
};

struct MetaBuf {
    void* host = nullptr;       // pinned
    cudaEvent_t done = nullptr;
    bool in_flight = false;
};

}  // namespace

struct mla_ctx {
    mla_config cfg{};
    int sm_count = 0;
    uint32_t kernel = MLA_KERNEL_MMA;
    std::unique_ptr<PageTable> pt;
    std::string err;
    uint64_t launches = 0;

    char* pool = nullptr;           // [layers][n_pages*64][576] elements
    uint64_t pool_slots = 0;        // token slots per layer
    std::vector<LayerW> layers;
    std::vector<BlockW> blocks;
    // workspaces of the block projections, grown on demand: normalised hidden state, q_a, float K-slice partials,
    // and the block's q / kv_a / attention output when the library owns them (mla_step_block)
    void *blk_hidden2 = nullptr, *blk_qa = nullptr, *blk_q = nullptr, *blk_kv = nullptr, *blk_out = nullptr;
    float* blk_partial = nullptr;
    size_t blk_hidden2_cap = 0, blk_qa_cap = 0, blk_q_cap = 0, blk_kv_cap = 0, blk_out_cap = 0, blk_partial_cap = 0;
    float* cos_sin = nullptr;       // device [max positions][64]
    uint32_t cs_rows = 0;           // positions filled so far
    uint32_t cs_cap = 0;

    void* q_abs = nullptr;          // [max_rows][H][576]
    float* recs = nullptr;          // [max_segs][H][514]
    uint32_t max_segs = 0;
    uint32_t workers = 1;
    uint32_t* status_dev = nullptr;
    // tensor maps of the tcgen05 attention kernels (make_tensor_maps; indices mla::kMap*)
    alignas(64) CUtensorMap tmaps[mla::kMapCount];

    // metadata upload ring
    MetaBuf ring[kMetaRing];
    int ring_next = 0;
    size_t meta_cap = 0;
    char* meta_dev = nullptr;
    mla::StepMeta meta{};
    // A step that holds prefill chunks (sequences taking >= kPrefillMin new tokens) has a second plan: its query rows
    // are the step's OTHER rows, the chunks go through the expanded-form prefill kernels (run_layer).  The explicit
    // per-layer calls (mla_step_append / _attend / _attend_partial) keep using the first plan, in which every new token
    // is a decode-style query row.
    mla::StepMeta meta_b{};
    bool has_plan_b = false;
    struct Chunk { uint32_t seq_id, q_row0, n_new, start, base_pos; };
    std::vector<Chunk> chunks;
    uint32_t step_rows = 0;          // rows of the step in the caller's q / kv_a / out tensors
    // prefill workspaces, grown on demand: gathered latent rows, expanded keys and values, rotated chunk queries
    void *pf_latent = nullptr, *pf_kx = nullptr, *pf_vx = nullptr, *pf_q = nullptr;
    size_t pf_latent_cap = 0, pf_kx_cap = 0, pf_vx_cap = 0, pf_q_cap = 0;

    // pages of the last planned step per persistent worker (mla_step_balance)
    uint32_t plan_workers = 0, plan_min_pages = 0, plan_max_pages = 0;
    uint32_t step_new_rows = 0;     // rows the open step appends (a KV-range shard that does not own the tail has none)

    // step state
    bool in_step = false;
    std::vector<uint32_t> step_seqs, step_nnew, step_tbl_off;

    // optional per-launch timing of the attention kernel
    bool q_rope_in_kernel = false;  // queries arrive before their RoPE (mla_set_q_rope)
    bool profiling = false;
    uint32_t prof_stride = 1, prof_seq = 0;     // every prof_stride-th attention launch is timed
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof_events;
    size_t prof_used = 0;

    // host-buffer entry point staging
    void *h_in = nullptr, *h_out = nullptr, *d_kv = nullptr, *d_q = nullptr, *d_out = nullptr;
    // page-locked callers: copies run on two streams of their own so that layer L+1's inputs and layer L-1's
    // outputs move while layer L computes; one event triple per layer orders copy-in -> compute -> copy-out
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    struct HostEv { cudaEvent_t in = nullptr, compute = nullptr, out = nullptr; bool used = false, pending = false; };
    std::vector<HostEv> host_ev;
};

namespace {

int fail(mla_ctx* c, int code, std::string msg)
{
    if (c) c->err = std::move(msg);
    else g_create_error = std::move(msg);
    return code;
}

#define CU_TRY(c, expr)                                                                           \
    do {                                                                                          \
        cudaError_t e__ = (expr);                                                                 \
        if (e__ != cudaSuccess)                                                                   \
            return fail((c), MLA_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__)); \
    } while (0)

// Every entry point that launches or copies makes the context's device current first: a host thread that
// drives several contexts (one per GPU) would otherwise launch on whichever device it used last.
#define USE_DEVICE(c) CU_TRY((c), cudaSetDevice((c)->cfg.device))

int pt_code(mla_ctx* c, int e)
{
    if (e == mugen::mla::PT_OK) return MLA_OK;
    c->err = c->pt->error();
    return e;   // PT_* values equal the MLA_ERR_* values they stand for
}

size_t align16(size_t x) { return (x + 15) & ~size_t(15); }

inline float half_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }
inline uint16_t f32_to_half_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }
inline uint16_t f32_to_bf16_bits(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }

// Decodes (n_rows x 512) weights of GGML type `w_type` into the context storage dtype.
int decode_weights(mla_ctx* c, const void* w, uint32_t w_type, size_t n_rows, std::vector<uint16_t>& out)
{
    const size_t n = n_rows * mla::kRank;
    out.resize(n);
    const bool to_half = c->cfg.dtype == MLA_DTYPE_F16;
    auto put = [&](size_t i, float v) { out[i] = to_half ? f32_to_half_bits(v) : f32_to_bf16_bits(v); };
    if (w_type == MLA_W_F16) {
        const auto* s = static_cast<const uint16_t*>(w);
        if (to_half) std::memcpy(out.data(), s, n * 2);
        else for (size_t i = 0; i < n; i++) put(i, half_bits_to_f32(s[i]));
    } else if (w_type == MLA_W_BF16) {
        const auto* s = static_cast<const uint16_t*>(w);
        if (!to_half) std::memcpy(out.data(), s, n * 2);
        else for (size_t i = 0; i < n; i++) {
            const uint32_t u = uint32_t(s[i]) << 16;
            float f;
            std::memcpy(&f, &u, 4);
            put(i, f);
        }
    } else if (w_type == MLA_W_Q8_0) {
        const auto* s = static_cast<const uint8_t*>(w);
        const size_t nb = n / 32;
        for (size_t b = 0; b < nb; b++) {
            const uint8_t* blk = s + b * 34;
            uint16_t d;
            std::memcpy(&d, blk, 2);
            const float sc = half_bits_to_f32(d);
            for (int j = 0; j < 32; j++) put(b * 32 + j, sc * float(int8_t(blk[2 + j])));
        }
    } else if (w_type == MLA_W_Q4_0) {
        const auto* s = static_cast<const uint8_t*>(w);
        const size_t nb = n / 32;
        for (size_t b = 0; b < nb; b++) {
            const uint8_t* blk = s + b * 18;
            uint16_t d;
            std::memcpy(&d, blk, 2);
            const float sc = half_bits_to_f32(d);
            for (int j = 0; j < 16; j++) {
                put(b * 32 + j, float(int(blk[2 + j] & 0x0F) - 8) * sc);
                put(b * 32 + j + 16, float(int(blk[2 + j] >> 4) - 8) * sc);
            }
        }
    } else {
        return fail(c, MLA_ERR_UNSUPPORTED, "weight type " + std::to_string(w_type) +
                                                " is not one of F16, BF16, Q8_0, Q4_0");
    }
    return MLA_OK;
}

int ensure_rope_rows(mla_ctx* c, uint32_t upto, cudaStream_t st)
{
    if (upto <= c->cs_rows) return MLA_OK;
    if (upto > c->cs_cap)
        return fail(c, MLA_ERR_CAPACITY, "position " + std::to_string(upto - 1) +
                                             " beyond the rotary table capacity " + std::to_string(c->cs_cap));
    // grow in chunks so that a decode loop does not upload one row per step
    uint32_t target = std::min<uint32_t>(c->cs_cap, std::max<uint32_t>(upto, c->cs_rows + 4096));
    std::vector<float> rows(size_t(target - c->cs_rows) * mla::kRope);
    mugen::mla::fill_rope_rows(rows.data(), c->cs_rows, target, c->cfg.rope_scaling_factor,
                               c->cfg.rope_original_ctx, c->cfg.rope_theta);
    CU_TRY(c, cudaMemcpyAsync(c->cos_sin + size_t(c->cs_rows) * mla::kRope, rows.data(),
                              rows.size() * sizeof(float), cudaMemcpyHostToDevice, st));
    CU_TRY(c, cudaStreamSynchronize(st));   // `rows` is pageable and about to go away
    c->cs_rows = target;
    return MLA_OK;
}

struct RowSpec {
    uint32_t seq_index;   // index into the step's sequence list
    uint32_t attend_len;  // rows attended (0 allowed)
    uint32_t pos;         // global position of the appended token (append only)
    uint64_t slot;        // destination slot (append only)
};

// Packs the step metadata, uploads it through the pinned ring and points c->meta (plan_b: c->meta_b) at it.
// att_row: for each query row its row in the caller's tensors (plan_b only).
int upload_meta(mla_ctx* c, const std::vector<uint32_t>& seq_ids, const std::vector<RowSpec>& rows,
                bool with_segments, cudaStream_t st, bool plan_b = false, const std::vector<uint32_t>* att_row = nullptr)
{
    const uint32_t R = uint32_t(rows.size()), S = uint32_t(seq_ids.size());
    std::vector<uint32_t> lens(R);
    for (uint32_t r = 0; r < R; r++) lens[r] = rows[r].attend_len;
    std::vector<Segment> segs;
    std::vector<uint32_t> row_seg_begin, cta_seg_begin;
    if (with_segments) {
        if (c->kernel == MLA_KERNEL_TCGEN05_PAIR128)
            // a worker pays about five tiles' time per segment it starts (queries, pipeline fill, state drain: ~10 us)
            mugen::mla::plan_min_makespan(lens, mla::kPage, c->workers, segs, row_seg_begin, cta_seg_begin, 2u, 5u);
        else
            mugen::mla::plan_balanced(lens, mla::kPage, c->workers, segs, row_seg_begin, cta_seg_begin, 1u);
        if (segs.size() > c->max_segs)
            return fail(c, MLA_ERR_CAPACITY, "step needs " + std::to_string(segs.size()) +
                                                 " KV segments, workspace holds " + std::to_string(c->max_segs));
    } else {
        row_seg_begin.assign(R + 1, 0);
        cta_seg_begin.assign(1, 0);
    }
    const uint32_t G = uint32_t(segs.size()), W = uint32_t(cta_seg_begin.size()) - 1;
    if (with_segments) {
        c->plan_workers = W;
        c->plan_min_pages = ~0u;
        c->plan_max_pages = 0;
        for (uint32_t w = 0; w < W; w++) {
            uint32_t pages = 0;
            for (uint32_t g = cta_seg_begin[w]; g < cta_seg_begin[w + 1]; g++) pages += segs[g].page_end - segs[g].page_begin;
            c->plan_min_pages = std::min(c->plan_min_pages, pages);
            c->plan_max_pages = std::max(c->plan_max_pages, pages);
        }
        if (W == 0) c->plan_min_pages = 0;
    }
    size_t tbl_total = 0;
    std::vector<uint32_t> tbl_off(S);
    for (uint32_t i = 0; i < S; i++) {
        tbl_off[i] = uint32_t(tbl_total);
        tbl_total += c->pt->seq(seq_ids[i])->pages.size();
    }
    // layout
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align16(off + bytes); return o; };
    const size_t o_slot = take(size_t(R) * 8), o_seq = take(size_t(R) * 4), o_len = take(size_t(R) * 4),
                 o_pos = take(size_t(R) * 4), o_tblo = take(size_t(S) * 4), o_tbl = take(tbl_total * 4 + 4),
                 o_sr = take(size_t(G) * 4), o_sb = take(size_t(G) * 4), o_se = take(size_t(G) * 4),
                 o_rsb = take(size_t(R + 1) * 4), o_csb = take(size_t(W + 1) * 4), o_att = take(att_row ? size_t(R) * 4 : 0);
    if (off > c->meta_cap)
        return fail(c, MLA_ERR_CAPACITY, "step metadata (" + std::to_string(off) + " B) exceeds the buffer (" +
                                             std::to_string(c->meta_cap) + " B)");
    MetaBuf& mb = c->ring[c->ring_next];
    c->ring_next = (c->ring_next + 1) % kMetaRing;
    if (mb.in_flight) {
        CU_TRY(c, cudaEventSynchronize(mb.done));
        mb.in_flight = false;
    }
    char* h = static_cast<char*>(mb.host);
    auto* p_slot = reinterpret_cast<uint64_t*>(h + o_slot);
    auto* p_seq = reinterpret_cast<uint32_t*>(h + o_seq);
    auto* p_len = reinterpret_cast<uint32_t*>(h + o_len);
    auto* p_pos = reinterpret_cast<uint32_t*>(h + o_pos);
    for (uint32_t r = 0; r < R; r++) {
        p_slot[r] = rows[r].slot;
        p_seq[r] = rows[r].seq_index;
        p_len[r] = rows[r].attend_len;
        p_pos[r] = rows[r].pos;
    }
    std::memcpy(h + o_tblo, tbl_off.data(), size_t(S) * 4);
    auto* p_tbl = reinterpret_cast<uint32_t*>(h + o_tbl);
    for (uint32_t i = 0; i < S; i++) {
        const auto& pg = c->pt->seq(seq_ids[i])->pages;
        std::memcpy(p_tbl + tbl_off[i], pg.data(), pg.size() * 4);
    }
    auto* p_sr = reinterpret_cast<uint32_t*>(h + o_sr);
    auto* p_sb = reinterpret_cast<uint32_t*>(h + o_sb);
    auto* p_se = reinterpret_cast<uint32_t*>(h + o_se);
    for (uint32_t g = 0; g < G; g++) {
        p_sr[g] = segs[g].row;
        p_sb[g] = segs[g].page_begin;
        p_se[g] = segs[g].page_end;
    }
    std::memcpy(h + o_rsb, row_seg_begin.data(), size_t(R + 1) * 4);
    std::memcpy(h + o_csb, cta_seg_begin.data(), size_t(W + 1) * 4);
    if (att_row) std::memcpy(h + o_att, att_row->data(), size_t(R) * 4);
    char* d = c->meta_dev + (plan_b ? c->meta_cap : 0);
    if (off) CU_TRY(c, cudaMemcpyAsync(d, h, off, cudaMemcpyHostToDevice, st));
    CU_TRY(c, cudaEventRecord(mb.done, st));
    mb.in_flight = true;

    mla::StepMeta& m = plan_b ? c->meta_b : c->meta;
    m.row_slot = reinterpret_cast<const uint64_t*>(d + o_slot);
    m.row_seq = reinterpret_cast<const uint32_t*>(d + o_seq);
    m.row_len = reinterpret_cast<const uint32_t*>(d + o_len);
    m.row_pos = reinterpret_cast<const uint32_t*>(d + o_pos);
    m.seq_tbl_off = reinterpret_cast<const uint32_t*>(d + o_tblo);
    m.tables = reinterpret_cast<const uint32_t*>(d + o_tbl);
    m.seg_row = reinterpret_cast<const uint32_t*>(d + o_sr);
    m.seg_page_begin = reinterpret_cast<const uint32_t*>(d + o_sb);
    m.seg_page_end = reinterpret_cast<const uint32_t*>(d + o_se);
    m.row_seg_begin = reinterpret_cast<const uint32_t*>(d + o_rsb);
    m.cta_seg_begin = reinterpret_cast<const uint32_t*>(d + o_csb);
    m.rows = R;
    m.segs = G;
    m.ctas = W;
    // by default the rows to append are the query rows themselves
    m.app_rows = R;
    m.app_pos = m.row_pos;
    m.app_slot = m.row_slot;
    m.att_row = att_row ? reinterpret_cast<const uint32_t*>(d + o_att) : nullptr;
    return MLA_OK;
}

char* layer_pool(mla_ctx* c, uint32_t layer)
{
    return c->pool + size_t(layer) * c->pool_slots * mla::kRow * 2;
}

int check_layer(mla_ctx* c, uint32_t layer, bool need_weights)
{
    if (layer >= c->cfg.n_layers) return fail(c, MLA_ERR_INVALID, "layer " + std::to_string(layer) + " out of range");
    if (need_weights && !c->layers[layer].set)
        return fail(c, MLA_ERR_STATE, "weights of layer " + std::to_string(layer) + " were never registered");
    return MLA_OK;
}

int run_append(mla_ctx* c, uint32_t layer, const void* kv_a, cudaStream_t st)
{
    mla::launch_append(int(c->cfg.dtype), kv_a, layer_pool(c, layer), c->pool_slots, c->layers[layer].norm,
                       c->cos_sin, c->cs_rows, c->cfg.rms_norm_eps, c->meta, c->status_dev, st);
    c->launches += c->meta.app_rows ? 1 : 0;
    CU_TRY(c, cudaGetLastError());
    return MLA_OK;
}

int run_merge(mla_ctx* c, uint32_t layer, const float* recs, const uint32_t* row_seg_begin, uint32_t n_parts, void* out,
              float* exported, uint32_t rows, cudaStream_t st, const uint32_t* att_row = nullptr);

// absorb -> split-KV attention -> merge (+ W_UV, or export of the merged partial state)
// With fused_kv_a the absorb launch also appends the step's new rows (the caller then skips run_append).
int run_attend(mla_ctx* c, uint32_t layer, const void* q, void* out, float* exported, cudaStream_t st,
               const void* fused_kv_a = nullptr, bool kv_a_settled = false, bool plan_b = false)
{
    const mla::StepMeta& m = plan_b ? c->meta_b : c->meta;
    if (m.rows == 0) return MLA_OK;
    const uint32_t H = c->cfg.n_heads;
    const LayerW& lw = c->layers[layer];
    if (lw.has_map) {
        const int ae = mla::launch_absorb_tc5(int(c->cfg.dtype), q, &lw.w_uk_map, c->q_abs, m.rows, H, fused_kv_a,
                                              layer_pool(c, layer), c->pool_slots, lw.norm, c->cos_sin, c->cs_rows,
                                              c->cfg.rms_norm_eps, m, c->q_rope_in_kernel, !kv_a_settled, c->status_dev, st);
        if (ae != 0) return fail(c, MLA_ERR_CUDA, std::string("absorb launch: ") + cudaGetErrorString(cudaError_t(ae)));
    } else {
        if (fused_kv_a) return fail(c, MLA_ERR_STATE, "fused append needs the layer's tensor maps");
        if (c->q_rope_in_kernel) return fail(c, MLA_ERR_UNSUPPORTED, "in-kernel q RoPE needs the layer's tensor maps");
        if (m.att_row) return fail(c, MLA_ERR_UNSUPPORTED, "a step with prefill chunks needs the layer's tensor maps");
        mla::launch_absorb(int(c->cfg.dtype), q, lw.w_uk, c->q_abs, m.rows, H, st);
    }
    int e;
    const bool timed = c->profiling && c->prof_used < c->prof_events.size() && (c->prof_seq++ % c->prof_stride) == 0;
    if (timed) CU_TRY(c, cudaEventRecord(c->prof_events[c->prof_used].first, st));
    // the W_UK the stream will want next: the following layer's (the first layer's after the last: the next step)
    const LayerW& nlw = c->layers[(layer + 1) % c->cfg.n_layers];
    const void* next_w = nlw.set ? nlw.w_uk : nullptr;
    if (c->kernel == MLA_KERNEL_TCGEN05_PAIR128)
        // short work lists (few sequences on this GPU) are bound by load latency, not bandwidth: prefetch one tile ahead
        e = mla::launch_decode_tc5_pair128(int(c->cfg.dtype), c->tmaps, layer_pool(c, layer), layer, c->cfg.n_pages, m, c->recs, H,
                                           c->plan_max_pages <= 64 ? 1u : 0u, next_w, next_w ? uint32_t(size_t(H) * mla::kNope * mla::kRank * 2) : 0u,
                                           c->status_dev, st);
    else if (c->kernel == MLA_KERNEL_TCGEN05)
        e = mla::launch_decode_tc5(int(c->cfg.dtype), c->tmaps, layer, c->cfg.n_pages, m, c->recs, H, c->status_dev, st);
    else if (c->kernel == MLA_KERNEL_TCGEN05_T16)
        e = mla::launch_decode_tc5_t16(int(c->cfg.dtype), c->tmaps, layer, c->cfg.n_pages, m, c->recs, H, c->status_dev, st);
    else
        e = mla::launch_decode_mma(int(c->cfg.dtype), c->q_abs, layer_pool(c, layer), c->cfg.n_pages, m,
                                   c->recs, H, c->status_dev, st);
    if (e != 0) return fail(c, MLA_ERR_CUDA, std::string("attention launch: ") + cudaGetErrorString(cudaError_t(e)));
    if (timed) CU_TRY(c, cudaEventRecord(c->prof_events[c->prof_used++].second, st));
    if (int rc = run_merge(c, layer, c->recs, m.row_seg_begin, 0, out, exported, m.rows, st, m.att_row)) return rc;
    c->launches += 3;
    CU_TRY(c, cudaGetLastError());
    return MLA_OK;
}

// Sequences that take at least this many new tokens in a step go through the prefill kernels.
constexpr uint32_t kPrefillMin = 64;

int grow_buf(mla_ctx* c, void** p, size_t* cap, size_t bytes)
{
    if (bytes <= *cap) return MLA_OK;
    CU_TRY(c, cudaDeviceSynchronize());          // an earlier launch may still use the smaller buffer
    if (*p) cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    CU_TRY(c, cudaMalloc(p, bytes + bytes / 4));
    *cap = bytes + bytes / 4;
    return MLA_OK;
}

// The chunks of the open step, one after the other: gather the sequence's latent rows (the chunk's own rows were
// appended by the launch before), expand them into per-head keys and values with W_UK / W_UV, run causal flash
// attention of the chunk's queries over them.  Reference semantics: src/core/model/transformer.cpp:1263-1337.
int run_chunks(mla_ctx* c, uint32_t layer, const void* q, void* out, cudaStream_t st)
{
    const uint32_t H = c->cfg.n_heads;
    const LayerW& lw = c->layers[layer];
    const int dt = int(c->cfg.dtype);
    for (const auto& ch : c->chunks) {
        const uint32_t total = ch.start + ch.n_new;
        if (int e = grow_buf(c, &c->pf_latent, &c->pf_latent_cap, size_t(total) * mla::kRow * 2)) return e;
        if (int e = grow_buf(c, &c->pf_kx, &c->pf_kx_cap, size_t(total) * H * mla::kNope * 2)) return e;
        if (int e = grow_buf(c, &c->pf_vx, &c->pf_vx_cap, size_t(total) * H * mla::kVDim * 2)) return e;
        // the sequence's block table inside the first plan's upload
        uint32_t si = 0;
        for (; si < c->step_seqs.size(); si++) if (c->step_seqs[si] == ch.seq_id) break;
        const uint32_t* table = c->meta.tables + c->step_tbl_off[si];
        int rc = mla::launch_gather_rows(layer_pool(c, layer), c->pool_slots, table, total, c->pf_latent, c->status_dev, st);
        if (rc) return fail(c, MLA_ERR_CUDA, std::string("gather launch: ") + cudaGetErrorString(cudaError_t(rc)));
        rc = mla::launch_gemm_tc5(dt, c->pf_latent, mla::kRow, lw.w_uk_rows, mla::kRank, total, H * mla::kNope, mla::kRank, c->pf_kx,
                                  nullptr, 1, c->status_dev, st);
        if (rc == 0)
            rc = mla::launch_gemm_tc5(dt, c->pf_latent, mla::kRow, lw.w_uv, mla::kRank, total, H * mla::kVDim, mla::kRank, c->pf_vx,
                                      nullptr, 1, c->status_dev, st);
        if (rc) return fail(c, rc == -1 ? MLA_ERR_INVALID : MLA_ERR_CUDA, "key / value expansion launch failed");
        const void* qp = q;
        uint32_t q_rows_total = c->step_rows, q_row0 = ch.q_row0;
        if (c->q_rope_in_kernel) {           // the chunk's queries arrive before their RoPE: rotate a copy
            if (int e = grow_buf(c, &c->pf_q, &c->pf_q_cap, size_t(ch.n_new) * H * mla::kQDim * 2)) return e;
            rc = mla::launch_rotate_q_rows(dt, static_cast<const char*>(q) + size_t(ch.q_row0) * H * mla::kQDim * 2, c->pf_q, ch.n_new, H,
                                           ch.base_pos + ch.start, c->cos_sin, c->cs_rows, c->status_dev, st);
            if (rc) return fail(c, MLA_ERR_CUDA, std::string("query rotation launch: ") + cudaGetErrorString(cudaError_t(rc)));
            c->launches++;
            qp = c->pf_q;
            q_rows_total = ch.n_new;
            q_row0 = 0;
        }
        // out rows are addressed from the chunk's first row in either case
        rc = mla::launch_prefill_tc5(dt, qp, q_rows_total, q_row0, ch.n_new, ch.start, c->pf_kx, c->pf_vx, c->pf_latent,
                                     static_cast<char*>(out) + (size_t(ch.q_row0) - q_row0) * H * mla::kVDim * 2, H, c->status_dev, st);
        if (rc) return fail(c, rc == -1 ? MLA_ERR_INVALID : MLA_ERR_CUDA, "prefill attention launch failed");
        c->launches += 4;
    }
    CU_TRY(c, cudaGetLastError());
    return MLA_OK;
}

// one layer of a step: append + attention, with the append riding in the absorb launch where it can.
// kv_a_settled: kv_a was complete before the kernel launched just ahead of this layer's started (see launch_absorb_tc5).
int run_layer(mla_ctx* c, uint32_t layer, const void* kv_a, const void* q, void* out, cudaStream_t st, bool kv_a_settled = false)
{
    if (c->has_plan_b) {
        // decode-style rows through the second plan (their append covers ALL new rows of the step), then the chunks
        if (c->meta_b.rows && c->layers[layer].has_map) {
            if (int e = run_attend(c, layer, q, out, nullptr, st, kv_a, kv_a_settled, true)) return e;
        } else {
            if (int e = run_append(c, layer, kv_a, st)) return e;
        }
        return run_chunks(c, layer, q, out, st);
    }
    if (c->layers[layer].has_map) return run_attend(c, layer, q, out, nullptr, st, kv_a, kv_a_settled);
    if (int e = run_append(c, layer, kv_a, st)) return e;
    return run_attend(c, layer, q, out, nullptr, st);
}

using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point: no link-time libcuda.
TensorMapEncodeFn tensor_map_encoder()
{
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    return reinterpret_cast<TensorMapEncodeFn>(fn);
}

int make_weight_map(mla_ctx* c, uint32_t layer)
{
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return fail(c, MLA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const CUtensorMapDataType dt = c->cfg.dtype == MLA_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const cuuint64_t dims[2] = {cuuint64_t(mla::kRank), cuuint64_t(c->cfg.n_heads) * mla::kVDim};
    const cuuint64_t strides[1] = {cuuint64_t(mla::kRank) * 2};
    const cuuint32_t box[2] = {64, cuuint32_t(mla::kVDim)};
    const cuuint32_t estr[2] = {1, 1};
    LayerW& lw = c->layers[layer];
    const CUresult r = enc(&lw.w_uv_map, dt, 2, lw.w_uv, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(c, MLA_ERR_CUDA, "cuTensorMapEncodeTiled(W_UV) failed with code " + std::to_string(int(r)));
    const cuuint64_t kdims[2] = {cuuint64_t(mla::kNope), cuuint64_t(c->cfg.n_heads) * mla::kRank};
    const cuuint64_t kstrides[1] = {cuuint64_t(mla::kNope) * 2};
    const cuuint32_t kbox[2] = {64, 256};
    const CUresult r2 = enc(&lw.w_uk_map, dt, 2, lw.w_uk, kdims, kstrides, kbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r2 != CUDA_SUCCESS)
        return fail(c, MLA_ERR_CUDA, "cuTensorMapEncodeTiled(W_UK) failed with code " + std::to_string(int(r2)));
    lw.has_map = true;
    return MLA_OK;
}

// merge of the partial states + W_UV: tensor-core kernel, or the scalar one when the merged state is exported
int run_merge(mla_ctx* c, uint32_t layer, const float* recs, const uint32_t* row_seg_begin, uint32_t n_parts, void* out,
              float* exported, uint32_t rows, cudaStream_t st, const uint32_t* att_row)
{
    const LayerW& lw = c->layers[layer];
    if (!exported && lw.has_map) {
        const int e = mla::launch_merge_tc5(int(c->cfg.dtype), recs, row_seg_begin, n_parts, &lw.w_uv_map, out, rows,
                                            c->cfg.n_heads, att_row, c->status_dev, st);
        if (e != 0) return fail(c, MLA_ERR_CUDA, std::string("merge launch: ") + cudaGetErrorString(cudaError_t(e)));
        return MLA_OK;
    }
    mla::launch_merge(int(c->cfg.dtype), recs, row_seg_begin, n_parts, lw.w_uv, out, exported, rows, c->cfg.n_heads, st, att_row);
    return MLA_OK;
}

int make_tensor_maps(mla_ctx* c)
{
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return fail(c, MLA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const CUtensorMapDataType dt = c->cfg.dtype == MLA_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    auto encode = [&](int slot, const char* what, cuuint32_t rank, void* basep, const cuuint64_t* dims,
                      const cuuint64_t* strides, const cuuint32_t* box) -> int {
        const CUresult r = enc(&c->tmaps[slot], dt, rank, basep, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(c, MLA_ERR_CUDA, std::string("cuTensorMapEncodeTiled(") + what + ") failed with code " + std::to_string(int(r)));
        return MLA_OK;
    };
    {   // cache pool: 576 values innermost, then the token slots of a layer, then layers;
        // box = 64 values (128 B, one swizzle row) x 64 tokens (one page)
        const cuuint64_t dims[3] = {cuuint64_t(mla::kRow), c->pool_slots, c->cfg.n_layers};
        const cuuint64_t strides[2] = {cuuint64_t(mla::kRow) * 2, c->pool_slots * mla::kRow * 2};
        const cuuint32_t box[3] = {64, 64, 1};
        if (int e = encode(mla::kMapPoolSub, "cache pool", 3, c->pool, dims, strides, box)) return e;
    }
    // Whole-row views: the 576 values of a row are exposed as (64 values, 9 chunks) with the chunk
    // dimension OUTSIDE the row dimension, so one box {64 values, R rows, C chunks} lands in shared
    // memory as C consecutive swizzled sub-tiles [R rows][128 B] — a whole operand in ONE TMA
    // instruction instead of nine (a TMA issue costs its thread ~100 cycles).
    {
        const cuuint64_t dims[4] = {64, c->pool_slots, 9, c->cfg.n_layers};
        const cuuint64_t strides[3] = {cuuint64_t(mla::kRow) * 2, 128, c->pool_slots * mla::kRow * 2};
        const cuuint32_t box_v[4] = {64, 64, 2, 1}, box_page[4] = {64, 64, 9, 1};
        if (int e = encode(mla::kMapPoolV, "cache pool, two chunks of a page", 4, c->pool, dims, strides, box_v)) return e;
        if (int e = encode(mla::kMapPoolPage, "cache pool, whole page", 4, c->pool, dims, strides, box_page)) return e;
        // 64 spare rows behind the queries: boxes of 64 head rows may start at the last row's heads
        const cuuint64_t qdims[3] = {64, cuuint64_t(c->cfg.max_rows) * c->cfg.n_heads + 64, 9};
        const cuuint64_t qstrides[2] = {cuuint64_t(mla::kRow) * 2, 128};
        const cuuint32_t qbox[3] = {64, 64, 9};
        if (int e = encode(mla::kMapQueries, "absorbed queries", 3, c->q_abs, qdims, qstrides, qbox)) return e;
        const cuuint32_t qbox16[3] = {64, 16, 9};
        if (int e = encode(mla::kMapQueries16, "absorbed queries, 16 heads", 3, c->q_abs, qdims, qstrides, qbox16)) return e;
    }
    return MLA_OK;
}

}  // namespace

extern "C" {

int mla_create(const mla_config* cfg, mla_ctx** out)
{
    if (!cfg || !out) return fail(nullptr, MLA_ERR_INVALID, "null argument");
    *out = nullptr;
    // same wording as KVCache::create's validation (src/core/memory/kv_cache.cpp:146-159)
    if (cfg->n_layers == 0) return fail(nullptr, MLA_ERR_INVALID, "n_layers must be > 0");
    if (cfg->n_heads == 0) return fail(nullptr, MLA_ERR_INVALID, "n_heads must be > 0");
    if (cfg->max_seq_len == 0) return fail(nullptr, MLA_ERR_INVALID, "max_seq_len must be > 0");
    if (cfg->kv_lora_rank != 512 || cfg->qk_nope_head_dim != 128 || cfg->qk_rope_head_dim != 64 ||
        cfg->v_head_dim != 128)
        return fail(nullptr, MLA_ERR_UNSUPPORTED,
                    "only kv_lora_rank 512, qk_nope_head_dim 128, qk_rope_head_dim 64, v_head_dim 128 are built");
    if (cfg->page_tokens != 64) return fail(nullptr, MLA_ERR_UNSUPPORTED, "page_tokens must be 64");
    if (cfg->n_pages == 0 || cfg->max_seqs == 0) return fail(nullptr, MLA_ERR_INVALID, "n_pages and max_seqs must be > 0");
    if (cfg->dtype > MLA_DTYPE_BF16) return fail(nullptr, MLA_ERR_INVALID, "dtype must be MLA_DTYPE_F16 or MLA_DTYPE_BF16");
    if (cfg->kernel > MLA_KERNEL_TCGEN05_T16) return fail(nullptr, MLA_ERR_INVALID, "unknown kernel selector");

    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0)
        return fail(nullptr, MLA_ERR_CUDA, std::string("no CUDA device: ") + cudaGetErrorString(e) +
                                               " (this library has no CPU path)");
    if (cfg->device < 0 || cfg->device >= ndev) return fail(nullptr, MLA_ERR_INVALID, "device ordinal out of range");

    auto c = std::make_unique<mla_ctx>();
    c->cfg = *cfg;
    if (c->cfg.max_rows == 0) c->cfg.max_rows = c->cfg.max_seqs;
    mla_ctx* cp = c.get();
    auto bail = [&](int code) { g_create_error = cp->err; mla_destroy(c.release()); return code; };
#define CR_TRY(expr)                                                                            \
    do {                                                                                        \
        cudaError_t e__ = (expr);                                                               \
        if (e__ != cudaSuccess) {                                                               \
            cp->err = std::string(#expr) + ": " + cudaGetErrorString(e__);                     \
            return bail(MLA_ERR_CUDA);                                                          \
        }                                                                                       \
    } while (0)
    CR_TRY(cudaSetDevice(cfg->device));
    cudaDeviceProp prop{};
    CR_TRY(cudaGetDeviceProperties(&prop, cfg->device));
    c->sm_count = prop.multiProcessorCount;
    if (prop.major != 10)
        { cp->err = "this library is built for sm_100a only; device is sm_" + std::to_string(prop.major * 10 + prop.minor);
          return bail(MLA_ERR_UNSUPPORTED); }
    // 128-head groups go to the SM-pair kernel; up to 16 heads take the transposed tcgen05 form (tokens as rows, the
    // heads as 16 columns); everything between fills (part of) the 64-row tiles of the single-block kernel, which
    // streams the cache once per 64 heads (measured at 32 heads, 64 sequences x 8192 tokens: 128 us against 186 us for
    // two passes of the 16-column form and 300 us for mma.sync)
    c->kernel = cfg->kernel != MLA_KERNEL_AUTO ? cfg->kernel
              : (cfg->n_heads % 128 == 0 && c->sm_count % 2 == 0) ? uint32_t(MLA_KERNEL_TCGEN05_PAIR128)
              : cfg->n_heads > 16 ? uint32_t(MLA_KERNEL_TCGEN05) : uint32_t(MLA_KERNEL_TCGEN05_T16);
    const uint32_t H = cfg->n_heads;
    if (c->kernel == MLA_KERNEL_TCGEN05_PAIR128) c->workers = std::max<uint32_t>(1, (c->sm_count / 2) / ((H + 127) / 128));
    else if (c->kernel == MLA_KERNEL_TCGEN05) c->workers = std::max<uint32_t>(1, c->sm_count / ((H + 63) / 64));
    else if (c->kernel == MLA_KERNEL_TCGEN05_T16) c->workers = std::max<uint32_t>(1, c->sm_count / ((H + 15) / 16));
    else c->workers = std::max<uint32_t>(1, c->sm_count * 2 / ((H + 15) / 16));

    c->pt = std::make_unique<PageTable>(cfg->page_tokens, cfg->n_pages, cfg->max_seqs, cfg->max_seq_len);
    c->layers.resize(cfg->n_layers);
    c->blocks.resize(cfg->n_layers);
    c->pool_slots = uint64_t(cfg->n_pages) * cfg->page_tokens;
    const size_t pool_bytes = size_t(cfg->n_layers) * c->pool_slots * mla::kRow * 2;
    CR_TRY(cudaMalloc(&c->pool, pool_bytes));
    // zero-fill: rows past a sequence's end inside its last page are multiplied by P = 0 and
    // must therefore hold finite values
    CR_TRY(cudaMemset(c->pool, 0, pool_bytes));
    for (auto& lw : c->layers) {
        CR_TRY(cudaMalloc(&lw.w_uk, size_t(H) * mla::kNope * mla::kRank * 2));
        CR_TRY(cudaMalloc(&lw.w_uk_rows, size_t(H) * mla::kNope * mla::kRank * 2));
        CR_TRY(cudaMalloc(&lw.w_uv, size_t(H) * mla::kVDim * mla::kRank * 2));
        CR_TRY(cudaMalloc(&lw.norm, mla::kRank * 2));
    }
    // rotary table: one row per position a sequence can reach
    c->cs_cap = std::max(cfg->max_seq_len, cfg->max_position);
    CR_TRY(cudaMalloc(&c->cos_sin, size_t(c->cs_cap) * mla::kRope * sizeof(float)));
    const uint32_t R = c->cfg.max_rows;
    // 64 spare rows: the tcgen05 kernel fetches queries in boxes of 64 head rows
    CR_TRY(cudaMalloc(&c->q_abs, (size_t(R) * H + 64) * mla::kRow * 2));
    CR_TRY(cudaMemset(c->q_abs, 0, (size_t(R) * H + 64) * mla::kRow * 2));
    c->max_segs = c->workers + R;
    CR_TRY(cudaMalloc(&c->recs, size_t(c->max_segs) * H * mla::kPart * sizeof(float)));
    CR_TRY(cudaMalloc(&c->status_dev, sizeof(uint32_t)));
    CR_TRY(cudaMemset(c->status_dev, 0, sizeof(uint32_t)));
    const size_t max_pages_per_seq = (size_t(cfg->max_seq_len) + cfg->page_tokens - 1) / cfg->page_tokens;
    const size_t tbl_entries = std::min<size_t>(size_t(cfg->max_seqs) * max_pages_per_seq, cfg->n_pages) + 4;
    c->meta_cap = align16(size_t(R) * 8) + 3 * align16(size_t(R) * 4) + align16(size_t(cfg->max_seqs) * 4) +
                  align16(tbl_entries * 4 + 4) + 3 * align16(size_t(c->max_segs) * 4) +
                  align16(size_t(R + 1) * 4) + align16(size_t(c->workers + 1) * 4) + align16(size_t(R) * 4) + 256;
    CR_TRY(cudaMalloc(&c->meta_dev, 2 * c->meta_cap));                // the two plans of a step live side by side
    for (auto& mb : c->ring) {
        CR_TRY(cudaMallocHost(&mb.host, c->meta_cap));
        CR_TRY(cudaEventCreateWithFlags(&mb.done, cudaEventDisableTiming));
    }
    if (int ce = mla::decode_mma_configure()) {
        cp->err = std::string("mma attention kernel configuration: ") + cudaGetErrorString(cudaError_t(ce));
        return bail(MLA_ERR_CUDA);
    }
    if (int ce = mla::merge_mma_configure()) {
        cp->err = std::string("mma merge kernel configuration: ") + cudaGetErrorString(cudaError_t(ce));
        return bail(MLA_ERR_CUDA);
    }
    if (int ce = mla::prefill_tc5_configure()) {
        cp->err = std::string("tcgen05 prefill kernel configuration: ") + cudaGetErrorString(cudaError_t(ce));
        return bail(MLA_ERR_CUDA);
    }
    if (int ce = mla::gemm_tc5_configure()) {
        cp->err = std::string("tcgen05 projection kernel configuration: ") + cudaGetErrorString(cudaError_t(ce));
        return bail(MLA_ERR_CUDA);
    }
    if (int ce = mla::absorb_tc5_configure()) {
        cp->err = std::string("tcgen05 absorb kernel configuration: ") + cudaGetErrorString(cudaError_t(ce));
        return bail(MLA_ERR_CUDA);
    }
    if (int ce = mla::merge_tc5_configure()) {
        cp->err = std::string("tcgen05 merge kernel configuration: ") + cudaGetErrorString(cudaError_t(ce));
        return bail(MLA_ERR_CUDA);
    }
    if (c->kernel == MLA_KERNEL_TCGEN05_PAIR128) {
        if (int rc = make_tensor_maps(cp)) return bail(rc);
        if (int ce = mla::decode_tc5_pair128_configure()) {
            cp->err = std::string("tcgen05 pair128 kernel configuration: ") + cudaGetErrorString(cudaError_t(ce));
            return bail(MLA_ERR_CUDA);
        }
    }
    if (c->kernel == MLA_KERNEL_TCGEN05) {
        if (int rc = make_tensor_maps(cp)) return bail(rc);
        if (int ce = mla::decode_tc5_configure()) {
            cp->err = std::string("tcgen05 kernel configuration: ") + cudaGetErrorString(cudaError_t(ce));
            return bail(MLA_ERR_CUDA);
        }
    }
    if (c->kernel == MLA_KERNEL_TCGEN05_T16) {
        if (int rc = make_tensor_maps(cp)) return bail(rc);
        if (int ce = mla::decode_tc5_t16_configure()) {
            cp->err = std::string("tcgen05 16-head kernel configuration: ") + cudaGetErrorString(cudaError_t(ce));
            return bail(MLA_ERR_CUDA);
        }
    }
#undef CR_TRY
    *out = c.release();
    return MLA_OK;
}

void mla_destroy(mla_ctx* c)
{
    if (!c) return;
    cudaSetDevice(c->cfg.device);
    cudaDeviceSynchronize();
    cudaFree(c->pool);
    for (auto& lw : c->layers) { cudaFree(lw.w_uk); cudaFree(lw.w_uk_rows); cudaFree(lw.w_uv); cudaFree(lw.norm); }
    cudaFree(c->pf_latent); cudaFree(c->pf_kx); cudaFree(c->pf_vx); cudaFree(c->pf_q);
    cudaFree(c->cos_sin);
    cudaFree(c->q_abs);
    cudaFree(c->recs);
    cudaFree(c->status_dev);
    cudaFree(c->meta_dev);
    for (auto& mb : c->ring) {
        if (mb.host) cudaFreeHost(mb.host);
        if (mb.done) cudaEventDestroy(mb.done);
    }
    for (auto& pe : c->prof_events) { cudaEventDestroy(pe.first); cudaEventDestroy(pe.second); }
    if (c->h_in) cudaFreeHost(c->h_in);
    if (c->h_out) cudaFreeHost(c->h_out);
    cudaFree(c->d_kv); cudaFree(c->d_q); cudaFree(c->d_out);
    for (auto& b : c->blocks) { cudaFree(b.attn_norm); cudaFree(b.q_a); cudaFree(b.q_a_norm); cudaFree(b.q_b); cudaFree(b.q); cudaFree(b.kv_a); cudaFree(b.wo); }
    cudaFree(c->blk_hidden2); cudaFree(c->blk_qa); cudaFree(c->blk_q); cudaFree(c->blk_kv); cudaFree(c->blk_out); cudaFree(c->blk_partial);
    for (auto& ev : c->host_ev) { cudaEventDestroy(ev.in); cudaEventDestroy(ev.compute); cudaEventDestroy(ev.out); }
    if (c->copy_in) cudaStreamDestroy(c->copy_in);
    if (c->copy_out) cudaStreamDestroy(c->copy_out);
    delete c;
}

const char* mla_last_error(const mla_ctx* c) { return c ? c->err.c_str() : g_create_error.c_str(); }

int mla_status(mla_ctx* c, void* stream, uint32_t* device_status)
{
    if (!c || !device_status) return MLA_ERR_INVALID;
    USE_DEVICE(c);
    auto st = static_cast<cudaStream_t>(stream);
    uint32_t v = 0;
    CU_TRY(c, cudaMemcpyAsync(&v, c->status_dev, 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(c, cudaStreamSynchronize(st));
    if (v) CU_TRY(c, cudaMemsetAsync(c->status_dev, 0, 4, st));
    *device_status = v;
    if (v) return fail(c, MLA_ERR_DEVICE, "device status word = " + std::to_string(v));
    return MLA_OK;
}

int mla_set_layer_weights(mla_ctx* c, uint32_t layer, const void* w_uk, const void* w_uv, uint32_t w_type,
                          const void* kv_norm)
{
    if (!c || !w_uk || !w_uv || !kv_norm) return fail(c, MLA_ERR_INVALID, "null argument");
    if (int e = check_layer(c, layer, false)) return e;
    CU_TRY(c, cudaSetDevice(c->cfg.device));
    std::vector<uint16_t> buf;
    const size_t H = c->cfg.n_heads;
    if (int e = decode_weights(c, w_uk, w_type, H * mla::kNope, buf)) return e;
    {   // the absorb kernel reads W_UK transposed per head: [h][d][i] (contraction index contiguous)
        std::vector<uint16_t> tr(buf.size());
        for (size_t h = 0; h < H; h++)
            for (size_t i = 0; i < size_t(mla::kNope); i++)
                for (size_t d = 0; d < size_t(mla::kRank); d++)
                    tr[(h * mla::kRank + d) * mla::kNope + i] = buf[(h * mla::kNope + i) * mla::kRank + d];
        CU_TRY(c, cudaMemcpy(c->layers[layer].w_uk, tr.data(), tr.size() * 2, cudaMemcpyHostToDevice));
        CU_TRY(c, cudaMemcpy(c->layers[layer].w_uk_rows, buf.data(), buf.size() * 2, cudaMemcpyHostToDevice));
    }
    if (int e = decode_weights(c, w_uv, w_type, H * mla::kVDim, buf)) return e;
    CU_TRY(c, cudaMemcpy(c->layers[layer].w_uv, buf.data(), buf.size() * 2, cudaMemcpyHostToDevice));
    CU_TRY(c, cudaMemcpy(c->layers[layer].norm, kv_norm, mla::kRank * 2, cudaMemcpyHostToDevice));
    if (int e = make_weight_map(c, layer)) return e;
    c->layers[layer].set = true;
    return MLA_OK;
}

int mla_seq_create(mla_ctx* c, uint32_t* id)
{
    if (!c || !id) return MLA_ERR_INVALID;
    return pt_code(c, c->pt->seq_create(id));
}
// While a step is open its uploaded block tables name the sequences' pages: giving pages back (or moving a
// counter the step is about to move) in between would let another sequence take pages the kernels still read.
static int refuse_in_step(mla_ctx* c, const char* what)
{
    return fail(c, MLA_ERR_STATE, std::string(what) + " is not allowed while a step is open");
}
int mla_seq_free(mla_ctx* c, uint32_t id)
{
    if (!c) return MLA_ERR_INVALID;
    if (c->in_step) return refuse_in_step(c, "seq_free");
    return pt_code(c, c->pt->seq_free(id));
}
int mla_seq_len(const mla_ctx* c, uint32_t id, uint32_t* len)
{
    if (!c || !len) return MLA_ERR_INVALID;
    return c->pt->seq_len(id, len);
}
int mla_advance(mla_ctx* c, uint32_t id, uint32_t n)
{
    if (!c) return MLA_ERR_INVALID;
    if (c->in_step) return refuse_in_step(c, "advance");
    return pt_code(c, c->pt->advance(id, n));
}
int mla_truncate(mla_ctx* c, uint32_t id, uint32_t n)
{
    if (!c) return MLA_ERR_INVALID;
    if (c->in_step) return refuse_in_step(c, "truncate");
    return pt_code(c, c->pt->truncate(id, n));
}
int mla_rollback(mla_ctx* c, uint32_t n_seq, const uint32_t* seq_ids, const uint32_t* keep_lens)
{
    if (!c || (n_seq && (!seq_ids || !keep_lens))) return fail(c, MLA_ERR_INVALID, "null argument");
    if (c->in_step) return refuse_in_step(c, "rollback");
    for (uint32_t i = 0; i < n_seq; i++)
        if (!c->pt->seq(seq_ids[i])) return fail(c, MLA_ERR_INVALID, "unknown sequence id " + std::to_string(seq_ids[i]));
    for (uint32_t i = 0; i < n_seq; i++)
        if (c->pt->seq(seq_ids[i])->len > keep_lens[i])
            if (int e = pt_code(c, c->pt->truncate(seq_ids[i], keep_lens[i]))) return e;
    return MLA_OK;
}
int mla_clear(mla_ctx* c, uint32_t id)
{
    if (!c) return MLA_ERR_INVALID;
    if (c->in_step) return refuse_in_step(c, "clear");
    return pt_code(c, c->pt->clear(id));
}
int mla_seq_set_base(mla_ctx* c, uint32_t id, uint32_t base) { return c ? pt_code(c, c->pt->set_base(id, base)) : MLA_ERR_INVALID; }
int mla_free_pages(const mla_ctx* c, uint32_t* n)
{
    if (!c || !n) return MLA_ERR_INVALID;
    *n = c->pt->free_pages();
    return MLA_OK;
}
int mla_shuffle_free_pages(mla_ctx* c, uint64_t seed)
{
    if (!c) return MLA_ERR_INVALID;
    c->pt->shuffle_free(seed);
    return MLA_OK;
}
int mla_seq_pages(const mla_ctx* c, uint32_t id, uint32_t* pages, uint32_t cap, uint32_t* n_pages)
{
    if (!c || !n_pages) return MLA_ERR_INVALID;
    const auto* s = c->pt->seq(id);
    if (!s) return MLA_ERR_INVALID;
    *n_pages = uint32_t(s->pages.size());
    if (pages) std::memcpy(pages, s->pages.data(), std::min<size_t>(cap, s->pages.size()) * 4);
    return MLA_OK;
}

int mla_append_rows(mla_ctx* c, uint32_t layer, uint32_t n, const uint32_t* seq_ids, const uint32_t* positions,
                    const void* kv_a, void* stream)
{
    if (!c || (n && (!seq_ids || !positions || !kv_a))) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (int e = check_layer(c, layer, true)) return e;
    if (c->in_step) return fail(c, MLA_ERR_STATE, "explicit-position calls are not allowed while a step is open");
    if (n > c->cfg.max_rows) return fail(c, MLA_ERR_CAPACITY, "more rows than max_rows");
    auto st = static_cast<cudaStream_t>(stream);
    std::vector<uint32_t> seqs;
    std::vector<RowSpec> rows(n);
    uint32_t max_pos = 0;
    for (uint32_t r = 0; r < n; r++) {
        const auto* s = c->pt->seq(seq_ids[r]);
        if (!s) return fail(c, MLA_ERR_INVALID, "unknown sequence id " + std::to_string(seq_ids[r]));
        if (positions[r] < s->base_pos) return fail(c, MLA_ERR_INVALID, "position below the sequence's base position");
        const uint32_t local = positions[r] - s->base_pos;
        if (int e = pt_code(c, c->pt->reserve(seq_ids[r], local + 1))) return e;
        rows[r] = {0, 0, positions[r], c->pt->slot(seq_ids[r], local)};
        max_pos = std::max(max_pos, positions[r]);
    }
    if (n) if (int e = ensure_rope_rows(c, max_pos + 1, st)) return e;
    if (int e = upload_meta(c, seqs, rows, false, st)) return e;
    return run_append(c, layer, kv_a, st);
}

int mla_attend_rows(mla_ctx* c, uint32_t layer, uint32_t n, const uint32_t* seq_ids, const uint32_t* attend_lens,
                    const void* q, void* out, void* stream)
{
    if (!c || (n && (!seq_ids || !attend_lens || !q || !out))) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (int e = check_layer(c, layer, true)) return e;
    if (c->in_step) return fail(c, MLA_ERR_STATE, "explicit-position calls are not allowed while a step is open");
    if (n > c->cfg.max_rows) return fail(c, MLA_ERR_CAPACITY, "more rows than max_rows");
    auto st = static_cast<cudaStream_t>(stream);
    std::vector<uint32_t> seqs;
    std::vector<RowSpec> rows(n);
    uint32_t max_pos = 0;
    for (uint32_t r = 0; r < n; r++) {
        const auto* s = c->pt->seq(seq_ids[r]);
        if (!s) return fail(c, MLA_ERR_INVALID, "unknown sequence id " + std::to_string(seq_ids[r]));
        if (uint64_t(attend_lens[r]) > uint64_t(s->pages.size()) * mla::kPage)
            return fail(c, MLA_ERR_INVALID, "attend length " + std::to_string(attend_lens[r]) +
                                                " reaches rows that were never appended");
        uint32_t idx = 0;
        for (; idx < seqs.size(); idx++) if (seqs[idx] == seq_ids[r]) break;
        if (idx == seqs.size()) seqs.push_back(seq_ids[r]);
        // the query stands at the last attended position (matters only when the library rotates q)
        const uint32_t qpos = s->base_pos + (attend_lens[r] ? attend_lens[r] - 1 : 0);
        rows[r] = {idx, attend_lens[r], qpos, 0};
        max_pos = std::max(max_pos, qpos);
    }
    if (n && c->q_rope_in_kernel) if (int e = ensure_rope_rows(c, max_pos + 1, st)) return e;
    if (int e = upload_meta(c, seqs, rows, true, st)) return e;
    return run_attend(c, layer, q, out, nullptr, st);
}

int mla_step_begin(mla_ctx* c, uint32_t n_seq, const uint32_t* seq_ids, const uint32_t* n_new, void* stream)
{
    if (!c || (n_seq && !seq_ids)) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (c->in_step) return fail(c, MLA_ERR_STATE, "step_begin while a step is open");
    auto st = static_cast<cudaStream_t>(stream);
    std::vector<uint32_t> seqs(seq_ids, seq_ids + n_seq);
    std::vector<uint32_t> nn(n_seq, 1);
    if (n_new) nn.assign(n_new, n_new + n_seq);
    uint64_t total = 0;
    for (uint32_t i = 0; i < n_seq; i++) {
        if (!c->pt->seq(seqs[i])) return fail(c, MLA_ERR_INVALID, "unknown sequence id " + std::to_string(seqs[i]));
        for (uint32_t j = 0; j < i; j++)
            if (seqs[j] == seqs[i]) return fail(c, MLA_ERR_INVALID, "sequence listed twice in one step");
        total += std::max<uint32_t>(nn[i], 1);
    }
    if (total > c->cfg.max_rows) return fail(c, MLA_ERR_CAPACITY, "step has " + std::to_string(total) + " rows, max_rows is " + std::to_string(c->cfg.max_rows));
    // reserve first (all-or-nothing per sequence; on failure earlier reservations stay, harmless)
    uint32_t max_pos = 0;
    for (uint32_t i = 0; i < n_seq; i++) {
        const auto* s = c->pt->seq(seqs[i]);
        if (int e = pt_code(c, c->pt->reserve(seqs[i], s->len + nn[i]))) return e;
        if (nn[i]) max_pos = std::max(max_pos, s->base_pos + s->len + nn[i] - 1);
    }
    if (total) if (int e = ensure_rope_rows(c, max_pos + 1, st)) return e;
    std::vector<RowSpec> rows;
    rows.reserve(total);
    for (uint32_t i = 0; i < n_seq; i++) {
        const auto* s = c->pt->seq(seqs[i]);
        if (nn[i] == 0) {                                              // query-only row
            if (c->q_rope_in_kernel)
                return fail(c, MLA_ERR_UNSUPPORTED, "a query-only row has no position of its own: rotate q on the caller's side "
                                                    "(mla_set_q_rope(ctx, 0)) for KV-range shards that do not own the tail");
            rows.push_back({i, s->len, 0, ~uint64_t(0)});
        }
        for (uint32_t t = 0; t < nn[i]; t++) {
            const uint32_t local = s->len + t;
            rows.push_back({i, local + 1, s->base_pos + local, c->pt->slot(seqs[i], local)});
        }
    }
    if (int e = upload_meta(c, seqs, rows, true, st)) return e;
    c->step_new_rows = 0;
    for (uint32_t i = 0; i < n_seq; i++) c->step_new_rows += nn[i];
    // table offsets of the step's sequences inside the upload (the prefill path gathers rows through them)
    c->step_tbl_off.resize(n_seq);
    {
        uint32_t o = 0;
        for (uint32_t i = 0; i < n_seq; i++) { c->step_tbl_off[i] = o; o += uint32_t(c->pt->seq(seqs[i])->pages.size()); }
    }
    c->step_rows = uint32_t(rows.size());
    c->chunks.clear();
    c->has_plan_b = false;
    bool any_chunk = false;
    for (uint32_t i = 0; i < n_seq; i++) any_chunk = any_chunk || nn[i] >= kPrefillMin;
    if (any_chunk && c->kernel != MLA_KERNEL_MMA) {
        std::vector<RowSpec> rows_b;
        std::vector<uint32_t> att_row;
        uint32_t r = 0;
        for (uint32_t i = 0; i < n_seq; i++) {
            const auto* sq = c->pt->seq(seqs[i]);
            const uint32_t cnt = std::max<uint32_t>(nn[i], 1);
            if (nn[i] >= kPrefillMin) {
                c->chunks.push_back({seqs[i], r, nn[i], sq->len, sq->base_pos});
            } else {
                for (uint32_t t = 0; t < cnt; t++) { rows_b.push_back(rows[r + t]); att_row.push_back(r + t); }
            }
            r += cnt;
        }
        const uint32_t plan_workers = c->plan_workers, plan_min = c->plan_min_pages, plan_max = c->plan_max_pages;
        if (int e = upload_meta(c, seqs, rows_b, true, st, true, &att_row)) return e;
        (void)plan_workers; (void)plan_min; (void)plan_max;
        // the append of the second plan still writes every new row of the step, in the caller's order
        c->meta_b.app_rows = c->meta.rows;
        c->meta_b.app_pos = c->meta.row_pos;
        c->meta_b.app_slot = c->meta.row_slot;
        c->has_plan_b = true;
    }
    c->step_seqs = std::move(seqs);
    c->step_nnew = std::move(nn);
    c->in_step = true;
    return MLA_OK;
}

int mla_step_append(mla_ctx* c, uint32_t layer, const void* kv_a, void* stream)
{
    if (!c || !kv_a) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (!c->in_step) return fail(c, MLA_ERR_STATE, "step_append outside step_begin/step_end");
    if (int e = check_layer(c, layer, true)) return e;
    return run_append(c, layer, kv_a, static_cast<cudaStream_t>(stream));
}

int mla_step_attend(mla_ctx* c, uint32_t layer, const void* q, void* out, void* stream)
{
    if (!c || !q || !out) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (!c->in_step) return fail(c, MLA_ERR_STATE, "step_attend outside step_begin/step_end");
    if (int e = check_layer(c, layer, true)) return e;
    return run_attend(c, layer, q, out, nullptr, static_cast<cudaStream_t>(stream));
}

int mla_step_layers(mla_ctx* c, uint32_t layer_begin, uint32_t n_layers, const void* kv_a, const void* q, void* out,
                    void* stream)
{
    if (!c || !kv_a || !q || !out) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (!c->in_step) return fail(c, MLA_ERR_STATE, "step_layers outside step_begin/step_end");
    if (uint64_t(layer_begin) + n_layers > c->cfg.n_layers) return fail(c, MLA_ERR_INVALID, "layer range out of bounds");
    auto st = static_cast<cudaStream_t>(stream);
    const size_t rows = c->meta.rows, H = c->cfg.n_heads;
    const size_t kv_b = rows * mla::kRow * 2, q_b = rows * H * mla::kQDim * 2, o_b = rows * H * mla::kVDim * 2;
    for (uint32_t i = 0; i < n_layers; i++) {
        const uint32_t layer = layer_begin + i;
        if (int e = check_layer(c, layer, true)) return e;
        // the caller's kv_a for ALL layers existed before this call: from the second layer on, the kernel ahead of the
        // layer's first launch is this library's own and kv_a was complete before it started
        if (int e = run_layer(c, layer, static_cast<const char*>(kv_a) + i * kv_b, static_cast<const char*>(q) + i * q_b,
                              static_cast<char*>(out) + i * o_b, st, i > 0))
            return e;
    }
    return MLA_OK;
}

int mla_step_attend_partial(mla_ctx* c, uint32_t layer, const void* q, float* partial, void* stream)
{
    if (!c || !q || !partial) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (!c->in_step) return fail(c, MLA_ERR_STATE, "step_attend_partial outside step_begin/step_end");
    if (int e = check_layer(c, layer, true)) return e;
    return run_attend(c, layer, q, nullptr, partial, static_cast<cudaStream_t>(stream));
}

int mla_step_layer_partial(mla_ctx* c, uint32_t layer, const void* kv_a, const void* q, float* partial, void* stream)
{
    if (!c || !q || !partial) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (!c->in_step) return fail(c, MLA_ERR_STATE, "step_layer_partial outside step_begin/step_end");
    if (int e = check_layer(c, layer, true)) return e;
    if (c->has_plan_b) return fail(c, MLA_ERR_UNSUPPORTED, "a step with prefill chunks has no partial form");
    if (c->step_new_rows && !kv_a) return fail(c, MLA_ERR_INVALID, "the step appends rows on this GPU: kv_a is needed");
    auto st = static_cast<cudaStream_t>(stream);
    if (!c->step_new_rows) kv_a = nullptr;           // query-only rows: nothing to append, kv_a is never read
    if (kv_a && !c->layers[layer].has_map) {
        if (int e = run_append(c, layer, kv_a, st)) return e;
        kv_a = nullptr;
    }
    return run_attend(c, layer, q, nullptr, partial, st, kv_a);
}

int mla_merge_partials(mla_ctx* c, uint32_t layer, uint32_t n_parts, uint32_t rows, const float* partials,
                       void* out, void* stream)
{
    if (!c || !partials || !out || n_parts == 0) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (int e = check_layer(c, layer, true)) return e;
    if (int rc = run_merge(c, layer, partials, nullptr, n_parts, out, nullptr, rows, static_cast<cudaStream_t>(stream)))
        return rc;
    c->launches += rows ? 1 : 0;
    CU_TRY(c, cudaGetLastError());
    return MLA_OK;
}

static bool is_pinned(const void* p)
{
    cudaPointerAttributes at{};
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeHost;
}

int mla_step_layer_host(mla_ctx* c, uint32_t layer, const void* kv_a_host, const void* q_host, void* out_host,
                        void* stream)
{
    if (!c || !kv_a_host || !q_host || !out_host) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (!c->in_step) return fail(c, MLA_ERR_STATE, "step_layer_host outside step_begin/step_end");
    if (int e = check_layer(c, layer, true)) return e;
    auto st = static_cast<cudaStream_t>(stream);
    const size_t R = c->cfg.max_rows, H = c->cfg.n_heads, rows = c->meta.rows, L = c->cfg.n_layers;
    const size_t kv_cap = R * mla::kRow * 2, q_cap = R * H * mla::kQDim * 2, o_cap = R * H * mla::kVDim * 2;
    const size_t kv_b = rows * mla::kRow * 2, q_b = rows * H * mla::kQDim * 2, o_b = rows * H * mla::kVDim * 2;
    if (!c->d_kv) {
        // one device slot per layer: the layers of a step then queue up without waiting for
        // each other's copies
        CU_TRY(c, cudaMalloc(&c->d_kv, L * kv_cap));
        CU_TRY(c, cudaMalloc(&c->d_q, L * q_cap));
        CU_TRY(c, cudaMalloc(&c->d_out, L * o_cap));
    }
    char* d_kv = static_cast<char*>(c->d_kv) + layer * kv_cap;
    char* d_q = static_cast<char*>(c->d_q) + layer * q_cap;
    char* d_out = static_cast<char*>(c->d_out) + layer * o_cap;
    const bool direct = is_pinned(kv_a_host) && is_pinned(q_host) && is_pinned(out_host);
    if (direct) {
        // page-locked caller buffers: fully asynchronous; out_host is complete when mla_step_end returns
        if (!c->copy_in) {
            CU_TRY(c, cudaStreamCreateWithFlags(&c->copy_in, cudaStreamNonBlocking));
            CU_TRY(c, cudaStreamCreateWithFlags(&c->copy_out, cudaStreamNonBlocking));
            c->host_ev.resize(L);
            for (auto& ev : c->host_ev) {
                CU_TRY(c, cudaEventCreateWithFlags(&ev.in, cudaEventDisableTiming));
                CU_TRY(c, cudaEventCreateWithFlags(&ev.compute, cudaEventDisableTiming));
                CU_TRY(c, cudaEventCreateWithFlags(&ev.out, cudaEventDisableTiming));
            }
        }
        auto& ev = c->host_ev[layer];
        // this layer's device slots were last read / written by its previous use
        if (ev.used) CU_TRY(c, cudaStreamWaitEvent(c->copy_in, ev.compute, 0));
        CU_TRY(c, cudaMemcpyAsync(d_kv, kv_a_host, kv_b, cudaMemcpyHostToDevice, c->copy_in));
        CU_TRY(c, cudaMemcpyAsync(d_q, q_host, q_b, cudaMemcpyHostToDevice, c->copy_in));
        CU_TRY(c, cudaEventRecord(ev.in, c->copy_in));
        CU_TRY(c, cudaStreamWaitEvent(st, ev.in, 0));
        if (ev.used) CU_TRY(c, cudaStreamWaitEvent(st, ev.out, 0));
        if (int e = run_layer(c, layer, d_kv, d_q, d_out, st)) return e;
        CU_TRY(c, cudaEventRecord(ev.compute, st));
        CU_TRY(c, cudaStreamWaitEvent(c->copy_out, ev.compute, 0));
        CU_TRY(c, cudaMemcpyAsync(out_host, d_out, o_b, cudaMemcpyDeviceToHost, c->copy_out));
        CU_TRY(c, cudaEventRecord(ev.out, c->copy_out));
        ev.used = ev.pending = true;
        return MLA_OK;
    }
    if (!c->h_in) {
        CU_TRY(c, cudaMallocHost(&c->h_in, kv_cap + q_cap));
        CU_TRY(c, cudaMallocHost(&c->h_out, o_cap));
    }
    // pageable caller buffers: staged through page-locked memory, synchronous
    CU_TRY(c, cudaStreamSynchronize(st));
    std::memcpy(c->h_in, kv_a_host, kv_b);
    std::memcpy(static_cast<char*>(c->h_in) + kv_cap, q_host, q_b);
    CU_TRY(c, cudaMemcpyAsync(d_kv, c->h_in, kv_b, cudaMemcpyHostToDevice, st));
    CU_TRY(c, cudaMemcpyAsync(d_q, static_cast<char*>(c->h_in) + kv_cap, q_b, cudaMemcpyHostToDevice, st));
    if (int e = run_layer(c, layer, d_kv, d_q, d_out, st)) return e;
    CU_TRY(c, cudaMemcpyAsync(c->h_out, d_out, o_b, cudaMemcpyDeviceToHost, st));
    CU_TRY(c, cudaStreamSynchronize(st));
    std::memcpy(out_host, c->h_out, o_b);
    return MLA_OK;
}

int mla_step_end(mla_ctx* c)
{
    if (!c) return MLA_ERR_INVALID;
    if (!c->in_step) return fail(c, MLA_ERR_STATE, "step_end without step_begin");
    // The step closes and the counters move whatever happens below (the rows were written by kernels already
    // queued); the first error is reported after that.
    c->in_step = false;
    int rc = MLA_OK;
    cudaSetDevice(c->cfg.device);
    for (auto& ev : c->host_ev)              // outputs of mla_step_layer_host must have landed in the caller's buffers
        if (ev.pending) {
            const cudaError_t e = cudaEventSynchronize(ev.out);
            if (e != cudaSuccess && rc == MLA_OK)
                rc = fail(c, MLA_ERR_CUDA, std::string("cudaEventSynchronize(output copy): ") + cudaGetErrorString(e));
            ev.pending = false;
        }
    for (size_t i = 0; i < c->step_seqs.size(); i++)
        if (int e = pt_code(c, c->pt->advance(c->step_seqs[i], c->step_nnew[i])))
            if (rc == MLA_OK) rc = e;
    return rc;
}

int mla_step_info(const mla_ctx* c, uint32_t* rows, uint32_t* segments)
{
    if (!c) return MLA_ERR_INVALID;
    if (rows) *rows = c->meta.rows;
    if (segments) *segments = c->meta.segs;
    return MLA_OK;
}

int mla_step_balance(const mla_ctx* c, uint32_t* workers, uint32_t* min_pages, uint32_t* max_pages)
{
    if (!c) return MLA_ERR_INVALID;
    if (workers) *workers = c->plan_workers;
    if (min_pages) *min_pages = c->plan_min_pages;
    if (max_pages) *max_pages = c->plan_max_pages;
    return MLA_OK;
}

int mla_launch_count(const mla_ctx* c, uint64_t* n)
{
    if (!c || !n) return MLA_ERR_INVALID;
    *n = c->launches;
    return MLA_OK;
}

int mla_set_q_rope(mla_ctx* c, int in_kernel)
{
    if (!c) return MLA_ERR_INVALID;
    if (c->in_step) return fail(c, MLA_ERR_STATE, "mla_set_q_rope inside step_begin/step_end");
    c->q_rope_in_kernel = in_kernel != 0;
    return MLA_OK;
}

int mla_selftest_wait_timeout(mla_ctx* c, uint64_t limit_cycles, void* stream, uint32_t* waited_cycles)
{
    if (!c) return MLA_ERR_INVALID;
    USE_DEVICE(c);
    if (limit_cycles == 0 || limit_cycles > 2000000000ull)
        return fail(c, MLA_ERR_INVALID, "limit_cycles must be in 1 .. 2e9 (about a second)");
    auto st = static_cast<cudaStream_t>(stream);
    uint32_t* report = nullptr;
    CU_TRY(c, cudaMalloc(&report, 8));
    mla::launch_wait_timeout_selftest(static_cast<long long>(limit_cycles), c->status_dev, report, st);
    c->launches++;
    uint32_t host[2] = {1, 0};
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(host, report, 8, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(report);
    if (e != cudaSuccess) return fail(c, MLA_ERR_CUDA, std::string("wait-timeout self-test: ") + cudaGetErrorString(e));
    if (waited_cycles) *waited_cycles = host[1];
    if (host[0] != 0) return fail(c, MLA_ERR_DEVICE, "the self-test's wait did not give up");
    return MLA_OK;
}

int mla_profile_enable(mla_ctx* c, int on)
{
    if (!c) return MLA_ERR_INVALID;
    USE_DEVICE(c);
    if (on && c->prof_events.empty()) {
        c->prof_events.resize(8192);
        for (auto& pe : c->prof_events) {
            CU_TRY(c, cudaEventCreate(&pe.first));
            CU_TRY(c, cudaEventCreate(&pe.second));
        }
    }
    c->profiling = on != 0;
    c->prof_stride = on > 1 ? uint32_t(on) : 1;
    c->prof_seq = 0;
    return MLA_OK;
}

int mla_profile_read(mla_ctx* c, uint32_t* launches, float* total_ms)
{
    if (!c || !launches || !total_ms) return MLA_ERR_INVALID;
    USE_DEVICE(c);
    float sum = 0.0f;
    for (size_t i = 0; i < c->prof_used; i++) {
        CU_TRY(c, cudaEventSynchronize(c->prof_events[i].second));
        float ms = 0.0f;
        CU_TRY(c, cudaEventElapsedTime(&ms, c->prof_events[i].first, c->prof_events[i].second));
        sum += ms;
    }
    *launches = uint32_t(c->prof_used);
    *total_ms = sum;
    c->prof_used = 0;
    return MLA_OK;
}

const char* mla_kernel_name(const mla_ctx* c)
{
    if (!c) return "";
    return c->kernel == MLA_KERNEL_TCGEN05_PAIR128 ? "tcgen05-pair128" : c->kernel == MLA_KERNEL_TCGEN05 ? "tcgen05"
         : c->kernel == MLA_KERNEL_TCGEN05_T16 ? "tcgen05-t16" : "mma";
}

int mla_read_rows(mla_ctx* c, uint32_t layer, uint32_t id, uint32_t row_begin, uint32_t n, void* host_out, void* stream)
{
    if (!c || !host_out) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (int e = check_layer(c, layer, false)) return e;
    const auto* s = c->pt->seq(id);
    if (!s) return fail(c, MLA_ERR_INVALID, "unknown sequence id");
    if (uint64_t(row_begin) + n > uint64_t(s->pages.size()) * mla::kPage)
        return fail(c, MLA_ERR_INVALID, "rows were never appended");
    auto st = static_cast<cudaStream_t>(stream);
    const size_t rb = mla::kRow * 2;
    for (uint32_t r = 0; r < n;) {   // one copy per page run
        const uint32_t row = row_begin + r;
        const uint32_t in_page = std::min<uint32_t>(n - r, mla::kPage - row % mla::kPage);
        CU_TRY(c, cudaMemcpyAsync(static_cast<char*>(host_out) + size_t(r) * rb,
                                  layer_pool(c, layer) + c->pt->slot(id, row) * rb, size_t(in_page) * rb,
                                  cudaMemcpyDeviceToHost, st));
        r += in_page;
    }
    CU_TRY(c, cudaStreamSynchronize(st));
    return MLA_OK;
}

int mla_write_rows(mla_ctx* c, uint32_t layer, uint32_t id, uint32_t row_begin, uint32_t n, const void* dev_rows,
                   void* stream)
{
    if (!c || (n && !dev_rows)) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (int e = check_layer(c, layer, false)) return e;
    if (!c->pt->seq(id)) return fail(c, MLA_ERR_INVALID, "unknown sequence id");
    if (c->in_step) return fail(c, MLA_ERR_STATE, "write_rows is not allowed while a step is open");
    if (int e = pt_code(c, c->pt->reserve(id, row_begin + n))) return e;
    auto st = static_cast<cudaStream_t>(stream);
    std::vector<uint32_t> seqs{id};
    std::vector<RowSpec> none;
    if (int e = upload_meta(c, seqs, none, false, st)) return e;
    mla::launch_write_rows(dev_rows, layer_pool(c, layer), c->pool_slots, c->meta.tables, row_begin, n,
                           c->status_dev, st);
    c->launches += n ? 1 : 0;
    CU_TRY(c, cudaGetLastError());
    return MLA_OK;
}

}  // extern "C"

// ---- attention block: the projections around the op -----------------------------------------------------------
namespace {

int grow(mla_ctx* c, void** p, size_t* cap, size_t bytes)
{
    if (bytes <= *cap) return MLA_OK;
    CU_TRY(c, cudaDeviceSynchronize());          // an earlier launch may still use the smaller buffer
    if (*p) cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    CU_TRY(c, cudaMalloc(p, bytes));
    *cap = bytes;
    return MLA_OK;
}

// out[rows][N] = act[rows][K] . W[N][K]^T, rounded to the storage type, then `mode` (0 store, 1 RMSNorm(w), 2 += res)
int project(mla_ctx* c, const void* act, const void* W, uint32_t rows, uint32_t N, uint32_t K, int mode, const void* w,
            const void* res, void* out, cudaStream_t st)
{
    uint32_t splits = mla::gemm_tc5_splits(rows, N, K, uint32_t(c->sm_count));
    const bool direct = splits == 1 && mode == 0;
    if (!direct)
        if (int e = grow(c, reinterpret_cast<void**>(&c->blk_partial), &c->blk_partial_cap, size_t(splits) * rows * N * sizeof(float))) return e;
    int rc = mla::launch_gemm_tc5(int(c->cfg.dtype), act, K, W, K, rows, N, K, direct ? out : nullptr,
                                  direct ? nullptr : c->blk_partial, splits, c->status_dev, st);
    if (rc == -1) return fail(c, MLA_ERR_INVALID, "projection operands must be 16-byte aligned with row lengths that are multiples of 8");
    if (rc != 0) return fail(c, MLA_ERR_CUDA, std::string("projection launch: ") + cudaGetErrorString(cudaError_t(rc)));
    c->launches++;
    if (!direct) {
        rc = mla::launch_gemm_finalize(int(c->cfg.dtype), c->blk_partial, splits, rows, N, mode, w, c->cfg.rms_norm_eps, res, out, st);
        if (rc != 0) return fail(c, MLA_ERR_CUDA, std::string("projection finalize launch: ") + cudaGetErrorString(cudaError_t(rc)));
        c->launches++;
    }
    return MLA_OK;
}

int block_of(mla_ctx* c, uint32_t layer, const BlockW** out)
{
    if (layer >= c->cfg.n_layers) return fail(c, MLA_ERR_INVALID, "layer " + std::to_string(layer) + " out of range");
    if (!c->blocks[layer].set) return fail(c, MLA_ERR_STATE, "block weights of layer " + std::to_string(layer) + " were never registered");
    *out = &c->blocks[layer];
    return MLA_OK;
}

int project_in(mla_ctx* c, const BlockW& b, uint32_t rows, const void* hidden, void* q, void* kv_a, cudaStream_t st)
{
    const uint32_t E = b.embed, H = c->cfg.n_heads, QD = H * uint32_t(mla::kQDim);
    if (int e = grow(c, &c->blk_hidden2, &c->blk_hidden2_cap, size_t(rows) * E * 2)) return e;
    if (int rc = mla::launch_rmsnorm_rows(int(c->cfg.dtype), hidden, b.attn_norm, c->blk_hidden2, rows, E, c->cfg.rms_norm_eps, st))
        return fail(c, MLA_ERR_CUDA, std::string("rmsnorm launch: ") + cudaGetErrorString(cudaError_t(rc)));
    c->launches++;
    if (b.q_lora) {
        if (int e = grow(c, &c->blk_qa, &c->blk_qa_cap, size_t(rows) * b.q_lora * 2)) return e;
        if (int e = project(c, c->blk_hidden2, b.q_a, rows, b.q_lora, E, 1, b.q_a_norm, nullptr, c->blk_qa, st)) return e;
        if (int e = project(c, c->blk_qa, b.q_b, rows, QD, b.q_lora, 0, nullptr, nullptr, q, st)) return e;
    } else {
        if (int e = project(c, c->blk_hidden2, b.q, rows, QD, E, 0, nullptr, nullptr, q, st)) return e;
    }
    return project(c, c->blk_hidden2, b.kv_a, rows, uint32_t(mla::kRow), E, 0, nullptr, nullptr, kv_a, st);
}

}  // namespace

extern "C" {

int mla_set_block_weights(mla_ctx* c, uint32_t layer, const mla_block_weights* w)
{
    if (!c || !w) return fail(c, MLA_ERR_INVALID, "null argument");
    if (layer >= c->cfg.n_layers) return fail(c, MLA_ERR_INVALID, "layer " + std::to_string(layer) + " out of range");
    USE_DEVICE(c);
    const uint32_t E = w->embedding_length, R = w->q_lora_rank, H = c->cfg.n_heads;
    if (E == 0 || E % 8 || R % 8) return fail(c, MLA_ERR_INVALID, "embedding_length and q_lora_rank must be multiples of 8");
    if (!w->attn_norm || !w->kv_a_mqa || !w->wo || (R ? (!w->q_a || !w->q_a_norm || !w->q_b) : !w->q))
        return fail(c, MLA_ERR_INVALID, "missing projection weight for this q_lora_rank");
    BlockW& b = c->blocks[layer];
    auto put = [&](void** dst, const void* src, size_t n) -> int {
        if (*dst) { cudaFree(*dst); *dst = nullptr; }
        if (!src) return MLA_OK;
        CU_TRY(c, cudaMalloc(dst, n * 2));
        CU_TRY(c, cudaMemcpy(*dst, src, n * 2, cudaMemcpyHostToDevice));
        return MLA_OK;
    };
    b.set = false;
    if (int e = put(&b.attn_norm, w->attn_norm, E)) return e;
    if (int e = put(&b.q_a, R ? w->q_a : nullptr, size_t(R) * E)) return e;
    if (int e = put(&b.q_a_norm, R ? w->q_a_norm : nullptr, R)) return e;
    if (int e = put(&b.q_b, R ? w->q_b : nullptr, size_t(H) * mla::kQDim * R)) return e;
    if (int e = put(&b.q, R ? nullptr : w->q, size_t(H) * mla::kQDim * E)) return e;
    if (int e = put(&b.kv_a, w->kv_a_mqa, size_t(mla::kRow) * E)) return e;
    if (int e = put(&b.wo, w->wo, size_t(E) * H * mla::kVDim)) return e;
    b.embed = E;
    b.q_lora = R;
    b.set = true;
    return MLA_OK;
}

int mla_block_project_in(mla_ctx* c, uint32_t layer, uint32_t rows, const void* hidden, void* q, void* kv_a, void* stream)
{
    if (!c || (rows && (!hidden || !q || !kv_a))) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    const BlockW* b = nullptr;
    if (int e = block_of(c, layer, &b)) return e;
    if (rows == 0) return MLA_OK;
    return project_in(c, *b, rows, hidden, q, kv_a, static_cast<cudaStream_t>(stream));
}

int mla_block_project_out(mla_ctx* c, uint32_t layer, uint32_t rows, const void* attn_out, void* hidden, void* stream)
{
    if (!c || (rows && (!attn_out || !hidden))) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    const BlockW* b = nullptr;
    if (int e = block_of(c, layer, &b)) return e;
    if (rows == 0) return MLA_OK;
    // hidden = hidden + W_o . attn_out: the residual is read and the sum written by the finalize kernel
    return project(c, attn_out, b->wo, rows, b->embed, c->cfg.n_heads * uint32_t(mla::kVDim), 2, nullptr, hidden, hidden,
                   static_cast<cudaStream_t>(stream));
}

int mla_step_block(mla_ctx* c, uint32_t layer, void* hidden, void* stream)
{
    if (!c || !hidden) return fail(c, MLA_ERR_INVALID, "null argument");
    USE_DEVICE(c);
    if (!c->in_step) return fail(c, MLA_ERR_STATE, "step_block outside step_begin/step_end");
    if (!c->q_rope_in_kernel)
        return fail(c, MLA_ERR_STATE, "the block's q projection is not rotated: enable mla_set_q_rope(ctx, 1) first");
    if (int e = check_layer(c, layer, true)) return e;
    const BlockW* b = nullptr;
    if (int e = block_of(c, layer, &b)) return e;
    auto st = static_cast<cudaStream_t>(stream);
    const uint32_t rows = c->meta.rows, H = c->cfg.n_heads;
    if (rows == 0) return MLA_OK;
    if (int e = grow(c, &c->blk_q, &c->blk_q_cap, size_t(rows) * H * mla::kQDim * 2)) return e;
    if (int e = grow(c, &c->blk_kv, &c->blk_kv_cap, size_t(rows) * mla::kRow * 2)) return e;
    if (int e = grow(c, &c->blk_out, &c->blk_out_cap, size_t(rows) * H * mla::kVDim * 2)) return e;
    if (int e = project_in(c, *b, rows, hidden, c->blk_q, c->blk_kv, st)) return e;
    if (int e = run_layer(c, layer, c->blk_kv, c->blk_q, c->blk_out, st)) return e;
    return project(c, c->blk_out, b->wo, rows, b->embed, H * uint32_t(mla::kVDim), 2, nullptr, hidden, hidden, st);
}

}  // extern "C"
