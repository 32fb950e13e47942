// Split-KV absorbed MLA attention on the 5th-generation tensor cores of sm_100a:
// tcgen05.mma with accumulators in tensor memory (TMEM), cache tiles staged by TMA.
//
// One persistent block per SM slot x one group of 64 heads.  A block walks its list of KV
// segments (runs of whole pages of one query row); per 64-token page tile:
//
//   TMA      page tile [64 tok][576] -> shared memory as 9 swizzled sub-tiles [64 tok][64 dims]
//   QK       S[64 heads x 64 tok]   = Q'[64 x 576] . K^T          36 x tcgen05.mma  M=64  N=64 K=16
//                                     A = Q' (K-major), B = cache sub-tiles (K-major)
//   softmax  four threads per head read its row of S from TMEM (tcgen05.ld), log2-domain online
//            softmax with lazy rescaling (the running reference maximum moves only when a tile
//            exceeds it by more than 2^8), writes P (bf16/f16) to shared memory
//   PV       O^T[512 dims x 64 heads] += V^T[512 x 64 tok] . P^T   16 x tcgen05.mma M=128 N=64 K=16
//                                     A = the SAME cache sub-tiles read MN-major (no second copy,
//                                     no transpose), B = P (K-major)
//
// The transposed PV keeps all 128 TMEM lanes busy at M=128 and leaves O^T in 256 columns
// (4 chunks of 128 latent dims x 64 head columns); the other 256 hold four partial score tiles of
// 64 columns, one per QK issuer (the softmax copies them to registers at once and hands the
// columns back, so the next tile's QK overlaps the exponentials).
// Warp roles: warp 0 = TMA producer, warps 1-6 = MMA issuers (four for QK, two for PV; warp 1 also
// owns the TMEM allocation), warps 7-10 = softmax, correction and epilogue (warp w touches TMEM
// lanes 32*(w%4) .. +31).
// Output per (segment, head): m (reference maximum, log2 domain), l, acc[512] — 514 floats.
//
// Every mbarrier wait is bounded: after ~2 s a waiter raises ST_WAIT_TIMEOUT in the status word,
// sets the block's abort flag and every role leaves its loops; TMEM is freed on all paths.
#include "mla_launch.h"
#include "mla_tc5.cuh"

namespace mla {

namespace {

using namespace tc5;

constexpr int TILE = 64;                          // tokens per tile = one page
constexpr int HG = 64;                            // heads per block
constexpr int NSUB = kRow / 64;                   // 9 sub-tiles of 64 dims
constexpr int SUB_BYTES = TILE * 128;             // 8 KB
constexpr int KV_STAGE_BYTES = NSUB * SUB_BYTES;  // 73,728
constexpr int KV_STAGES = 2;
// No L2 prefetch ahead of the loads: measured at 64 heads x 64 sequences x 8192 tokens, prefetching 4 pages ahead with
// the tensor map takes the kernel from 124 us (0.75 of the measured HBM peak) to 155 us (0.60).
constexpr int Q_BYTES = NSUB * HG * 128;          // 73,728
constexpr int P_BYTES = HG * 128;                 // 8,192
constexpr int OFF_Q = 0;
constexpr int OFF_KV = OFF_Q + Q_BYTES;
constexpr int OFF_P = OFF_KV + KV_STAGES * KV_STAGE_BYTES;
constexpr int OFF_MISC = OFF_P + P_BYTES;         // barriers, alpha, tmem base, abort flag
constexpr int MISC_BYTES = 640;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;   // +1024: manual 1 KB alignment

constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_O = 0;                     // 4 x 64 columns
constexpr uint32_t COL_S = 256;                   // 4 partial score tiles x 64 columns

constexpr int N_QK = 4, N_PV = 2;                 // MMA-issuing warps for QK and for PV
constexpr int NUM_THREADS = 32 * (1 + N_QK + N_PV + 4);   // producer + issuers + 4 softmax warps
constexpr int SOFTMAX_THREADS = 128;
constexpr float RESCALE_THRESHOLD = 8.0f;         // log2 units

// barrier slots inside the misc area (8 bytes each)
enum { B_QFULL = 0, B_QEMPTY, B_KVFULL0, B_KVFULL1, B_KVEMPTY0, B_KVEMPTY1, B_SFULL0, B_SFULL1,
       B_SEMPTY0, B_SEMPTY1, B_PFULL, B_PEMPTY, B_OFULL, B_COUNT };


struct SegInfo {
    uint32_t row, page_begin, n_tiles, n_tok;
};

__device__ __forceinline__ SegInfo load_seg(const StepMeta& m, uint32_t seg) {
    SegInfo s;
    s.row = m.seg_row[seg];
    s.page_begin = m.seg_page_begin[seg];
    const uint32_t pe = m.seg_page_end[seg];
    const uint32_t len = m.row_len[s.row];
    const uint32_t tb = s.page_begin * kPage, te = min(len, pe * kPage);
    s.n_tok = te > tb ? te - tb : 0;
    s.n_tiles = (s.n_tok + TILE - 1) / TILE;
    return s;
}

template <typename T>
__global__ void __launch_bounds__(NUM_THREADS, 1)
decode_tc5_kernel(const __grid_constant__ CUtensorMap map_kv, const __grid_constant__ CUtensorMap map_q,
                  uint32_t layer, uint32_t n_pages, StepMeta m, float* __restrict__ recs, uint32_t H,
                  float scale_log2, uint32_t* __restrict__ status)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = smem_raw + (base - raw);
    const uint32_t sQ = base + OFF_Q, sKV = base + OFF_KV, sP = base + OFF_P;
    const uint32_t sBar = base + OFF_MISC;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC + 112);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 116);
    float* alpha_s = reinterpret_cast<float*>(sm + OFF_MISC + 128);          // [2][64], by tile parity
    auto bar = [&](int i) { return sBar + 8u * uint32_t(i); };

    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t cta = blockIdx.x, h0 = blockIdx.y * HG;
    const uint32_t seg_begin = m.cta_seg_begin[cta], seg_end = m.cta_seg_begin[cta + 1];

    grid_launch_dependents();
    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar(B_QFULL), 1);
        mbar_init(bar(B_QEMPTY), N_QK);
        mbar_init(bar(B_KVFULL0), 1);
        mbar_init(bar(B_KVFULL1), 1);
        mbar_init(bar(B_KVEMPTY0), N_PV);
        mbar_init(bar(B_KVEMPTY1), N_PV);
        mbar_init(bar(B_SFULL0), N_QK);
        mbar_init(bar(B_SFULL1), N_QK);
        mbar_init(bar(B_SEMPTY0), SOFTMAX_THREADS);
        mbar_init(bar(B_SEMPTY1), SOFTMAX_THREADS);
        mbar_init(bar(B_PFULL), SOFTMAX_THREADS);
        mbar_init(bar(B_PEMPTY), N_PV);
        mbar_init(bar(B_OFULL), N_PV);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    // queries, new cache rows and the state records belong to earlier kernels of the stream (the step's metadata does not:
    // it was uploaded before the first of them started)
    grid_dependency_wait();

    if (warp == 0) {
        // ===================== TMA producer =====================
        if (lane == 0) {
            uint32_t t = 0, nseg = 0;
            bool ok = true;
            for (uint32_t seg = seg_begin; seg < seg_end && ok; seg++) {
                const SegInfo s = load_seg(m, seg);
                if (s.n_tiles == 0) continue;
                // Q' of this row's head group: 9 boxes of [64 heads][64 dims]
                ok = mbar_wait(bar(B_QEMPTY), (nseg & 1) ^ 1, abort_flag, status);
                if (!ok) break;
                mbar_expect_tx(bar(B_QFULL), Q_BYTES);
                tma_load_3d(sQ, &map_q, bar(B_QFULL), 0, int(s.row * H + h0), 0);          // all 9 sub-tiles in one box
                const uint32_t* tbl = m.tables + m.seq_tbl_off[m.row_seq[s.row]];
                for (uint32_t j = 0; j < s.n_tiles; j++, t++) {
                    const uint32_t st = t % KV_STAGES;
                    ok = mbar_wait(bar(B_KVEMPTY0 + st), ((t / KV_STAGES) & 1) ^ 1, abort_flag, status);
                    if (!ok) break;
                    uint32_t page = tbl[s.page_begin + j];
                    if (page >= n_pages) {
                        atomicOr(status, ST_BAD_PAGE);
                        page = 0;
                    }
                    mbar_expect_tx(bar(B_KVFULL0 + st), KV_STAGE_BYTES);
                    const uint32_t dst = sKV + st * KV_STAGE_BYTES;
                    tma_load_4d(dst, &map_kv, bar(B_KVFULL0 + st), 0, int(page * kPage), 0, int(layer));   // whole page
                }
                nseg++;
            }
        }
    } else if (warp <= N_QK + N_PV) {
        // ===================== MMA issuers =====================
        // A tcgen05.mma costs its issuing warp about a hundred cycles before the next one can go,
        // far more than the tensor core needs for these small shapes (N = 64, K = 16), so one
        // issuer leaves the pipe mostly idle.  Six warps issue concurrently, each into its own
        // accumulators: warps 1-4 split the 36 k-steps of QK into four partial score tiles
        // (sub-tiles 0-2, 3-4, 5-6, 7-8; the softmax adds them), warps 5-6 take two of the four
        // 128-dim chunks of O^T each.  The warp runs the loop uniformly (operands stay in uniform
        // registers) and one elected lane issues.
        constexpr uint32_t IDESC_QK = instr_desc(Fmt<T>::v, 64, TILE, 0, 0);
        constexpr uint32_t IDESC_PV = instr_desc(Fmt<T>::v, 128, HG, 1, 0);
        constexpr uint32_t HI = desc_hi(1024);          // every operand: 8-row groups 1024 B apart
        static_assert(KV_STAGES == 2, "descriptor bases below assume two cache stages");
        const bool is_qk = warp <= N_QK;
        const uint32_t part = is_qk ? warp - 1 : warp - 1 - N_QK;
        const int c_lo = part == 0 ? 0 : 1 + 2 * int(part), c_hi = 3 + 2 * int(part);   // QK sub-tile range
        const uint32_t qk_a = desc_lo(sQ, 16);          // Q' (K-major)
        const uint32_t kv_k0 = desc_lo(sKV, 16), kv_k1 = desc_lo(sKV + KV_STAGE_BYTES, 16);                 // tile as K
        const uint32_t kv_v0 = desc_lo(sKV, SUB_BYTES), kv_v1 = desc_lo(sKV + KV_STAGE_BYTES, SUB_BYTES);   // tile as V^T
        const uint32_t pv_b = desc_lo(sP, 16);          // P (K-major)
        uint32_t t = 0, nseg = 0;
        bool ok = true;
        for (uint32_t seg = seg_begin; seg < seg_end && ok; seg++) {
            const SegInfo s = load_seg(m, seg);
            if (s.n_tiles == 0) continue;
            if (is_qk) ok = mbar_wait(bar(B_QFULL), nseg & 1, abort_flag, status);
            for (uint32_t j = 0; j < s.n_tiles && ok; j++, t++) {
                const uint32_t st = t % KV_STAGES;
                if (is_qk) {
                    ok = mbar_wait(bar(B_KVFULL0 + st), (t / KV_STAGES) & 1, abort_flag, status) &&
                         mbar_wait(bar(B_SEMPTY0), (t & 1) ^ 1, abort_flag, status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t b0 = st ? kv_k1 : kv_k0;
                    const uint32_t d = tmem + COL_S + part * TILE;
                    if (elect_one()) {
#pragma unroll
                        for (int c = 0; c < NSUB; c++) {
                            if (c >= c_lo && c < c_hi) {
#pragma unroll
                                for (int k = 0; k < 4; k++)
                                    tc_mma(d, qk_a + ((c * (HG * 128) + k * 32) >> 4), HI, b0 + ((c * SUB_BYTES + k * 32) >> 4),
                                           HI, IDESC_QK, (c == c_lo && k == 0) ? 0u : 1u);
                            }
                        }
                        tc_commit(bar(B_SFULL0));
                        if (j + 1 == s.n_tiles) tc_commit(bar(B_QEMPTY));
                    }
                    __syncwarp();
                } else {
                    ok = mbar_wait(bar(B_PFULL), t & 1, abort_flag, status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a0 = st ? kv_v1 : kv_v0;
                    const uint32_t fresh = j == 0 ? 0u : 1u;
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < TILE / 16; k++)
#pragma unroll
                            for (int cc = 0; cc < 2; cc++) {      // 128 latent dims per chunk = 2 sub-tiles
                                const uint32_t c = part * 2 + cc;
                                tc_mma(tmem + COL_O + c * HG, a0 + ((2 * c * SUB_BYTES + k * 2048) >> 4), HI,
                                       pv_b + ((k * 32) >> 4), HI, IDESC_PV, k == 0 ? fresh : 1u);
                            }
                        tc_commit(bar(B_KVEMPTY0 + st));
                        tc_commit(bar(B_PEMPTY));
                        if (j + 1 == s.n_tiles) tc_commit(bar(B_OFULL));
                    }
                    __syncwarp();
                }
            }
            nseg++;
        }
    } else {
        // ===================== softmax / correction / epilogue =====================
        // S (M=64 layout) keeps the warp's 16 head rows in TMEM lanes 0-15 of its sub-partition.
        // A 16x256b load spreads them over all 32 threads: thread i holds, for each block k of 8
        // tokens, tokens 8k+2(i%4), +1 of head rows i/4 and i/4+8 — so a row is shared by the 4
        // threads of a quad and row reductions are two shuffles.
        // The 128 threads meet at a named barrier every tile.  A failed (timed-out / aborted)
        // wait never makes a thread leave early on its own: the failure is carried to the next
        // barrier, OR-reduced there, and all 128 threads leave together.
        const uint32_t q4 = warp % 4;                         // TMEM sub-partition of this warp
        const uint32_t lane_base = (q4 * 32u) << 16;
        const uint32_t qd = lane & 3;
        const uint32_t r_a = q4 * 16 + lane / 4, r_b = r_a + 8;   // head rows (within the group)
        float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
        uint32_t t = 0, nseg = 0;
        bool fail = false;
        auto wait_w = [&](uint32_t b, uint32_t parity) {      // warp-uniform bounded wait
            if (!fail) fail = !mbar_wait(b, parity, abort_flag, status);
            fail = __any_sync(0xffffffffu, fail);
        };
        auto group_or = [&](bool pred) -> bool {              // barrier over the 128 threads + OR
            uint32_t r;
            asm volatile(
                "{\n.reg .pred pi, po;\n"
                "setp.ne.b32 pi, %1, 0;\n"
                "barrier.cta.red.or.pred po, 1, 128, pi;\n"
                "selp.u32 %0, 1, 0, po;\n}\n"
                : "=r"(r) : "r"(uint32_t(pred)) : "memory");
            return r != 0;
        };
        auto quad_max = [](float v) {
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
            return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
        };
        auto quad_sum = [](float v) {
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            return v + __shfl_xor_sync(0xffffffffu, v, 2);
        };
        bool stop = false;
        for (uint32_t seg = seg_begin; seg < seg_end && !stop; seg++) {
            const SegInfo s = load_seg(m, seg);
            if (s.n_tiles == 0) {
                // nothing to attend: the state of an empty range
                const uint32_t st = tid - (NUM_THREADS - SOFTMAX_THREADS);
                for (uint32_t h = 0; h < HG; h++) {
                    if (h0 + h >= H) break;
                    float* rc = recs + (size_t(seg) * H + h0 + h) * kPart;
                    for (uint32_t d = st; d < kRank; d += SOFTMAX_THREADS) rc[2 + d] = 0.0f;
                    if (st == 0) { rc[0] = -INFINITY; rc[1] = 0.0f; }
                }
                continue;
            }
            m_a = m_b = -INFINITY;
            l_a = l_b = 0.0f;
            for (uint32_t j = 0; j < s.n_tiles; j++, t++) {
                const uint32_t sb = t & 1;
                float* alpha_t = alpha_s + sb * HG;
                wait_w(bar(B_SFULL0), t & 1);
                uint32_t sv[32];
                if (!fail) {
                    tc_fence_after();
                    uint32_t sw[32];
                    tc_ld16x256_x8(tmem + lane_base + COL_S, sv);
                    tc_ld16x256_x8(tmem + lane_base + COL_S + TILE, sw);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) sv[i] = __float_as_uint(__uint_as_float(sv[i]) + __uint_as_float(sw[i]));
                    tc_ld16x256_x8(tmem + lane_base + COL_S + 2 * TILE, sw);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) sv[i] = __float_as_uint(__uint_as_float(sv[i]) + __uint_as_float(sw[i]));
                    tc_ld16x256_x8(tmem + lane_base + COL_S + 3 * TILE, sw);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) sv[i] = __float_as_uint(__uint_as_float(sv[i]) + __uint_as_float(sw[i]));
                    tc_fence_before();
                    mbar_arrive(bar(B_SEMPTY0));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) sv[i] = 0u;
                }
                const uint32_t valid = min(uint32_t(TILE), s.n_tok - j * TILE);
                float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
                for (int k = 0; k < 8; k++) {
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const bool in = uint32_t(8 * k + 2 * qd + e) < valid;
                        const float va = in ? __uint_as_float(sv[4 * k + e]) * scale_log2 : -INFINITY;
                        const float vb = in ? __uint_as_float(sv[4 * k + 2 + e]) * scale_log2 : -INFINITY;
                        sv[4 * k + e] = __float_as_uint(va);
                        sv[4 * k + 2 + e] = __float_as_uint(vb);
                        mx_a = fmaxf(mx_a, va);
                        mx_b = fmaxf(mx_b, vb);
                    }
                }
                mx_a = quad_max(mx_a);
                mx_b = quad_max(mx_b);
                float alpha_a = 1.0f, alpha_b = 1.0f;
                bool need = false;
                if (j == 0) {
                    m_a = mx_a;
                    m_b = mx_b;
                } else {
                    if (mx_a > m_a + RESCALE_THRESHOLD) { alpha_a = fast_ex2(m_a - mx_a); m_a = mx_a; need = true; }
                    if (mx_b > m_b + RESCALE_THRESHOLD) { alpha_b = fast_ex2(m_b - mx_b); m_b = mx_b; need = true; }
                }
                if (qd == 0) {
                    alpha_t[r_a] = alpha_a;
                    alpha_t[r_b] = alpha_b;
                }
                // one barrier on the common path; a second one only to tell failure from rescale
                bool any_need = group_or(need || fail);
                if (any_need && group_or(fail)) { stop = true; break; }
                float sum_a = 0.0f, sum_b = 0.0f;
                uint32_t pk_a[8], pk_b[8];
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const float a0 = fast_ex2(__uint_as_float(sv[4 * k]) - m_a);
                    const float a1 = fast_ex2(__uint_as_float(sv[4 * k + 1]) - m_a);
                    const float b0 = fast_ex2(__uint_as_float(sv[4 * k + 2]) - m_b);
                    const float b1 = fast_ex2(__uint_as_float(sv[4 * k + 3]) - m_b);
                    sum_a += a0 + a1;
                    sum_b += b0 + b1;
                    pk_a[k] = Elem<T>::pack2(a0, a1);
                    pk_b[k] = Elem<T>::pack2(b0, b1);
                }
                l_a = l_a * alpha_a + quad_sum(sum_a);
                l_b = l_b * alpha_b + quad_sum(sum_b);
                // PV of the previous tile must be complete: O is stable and P is free
                wait_w(bar(B_PEMPTY), (t - 1) & 1);
                if (fail) continue;            // carried to the next barrier
                tc_fence_after();
                if (any_need && j > 0) {
                    // O^T[dim lane][head column] *= alpha[head]
#pragma unroll 1
                    for (int c = 0; c < 8; c++) {
                        uint32_t o[32];
                        const uint32_t col = COL_O + c * 32;
                        tc_ld32(tmem + lane_base + col, o);
                        tc_wait_ld();
                        const int hbase = (c & 1) * 32;
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha_t[hbase + i]);
                        tc_st32(tmem + lane_base + col, o);
                    }
                    tc_wait_st();
                }
                {
                    // rows r_a, r_b of the K-major swizzled P tile; chunk k = tokens 8k..8k+7
                    unsigned char* pa = sm + OFF_P + r_a * 128 + qd * 4;
                    unsigned char* pb = sm + OFF_P + r_b * 128 + qd * 4;
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        *reinterpret_cast<uint32_t*>(pa + ((k ^ (r_a & 7)) << 4)) = pk_a[k];
                        *reinterpret_cast<uint32_t*>(pb + ((k ^ (r_b & 7)) << 4)) = pk_b[k];
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                tc_fence_before();
                mbar_arrive(bar(B_PFULL));
            }
            if (stop) break;
            // ---- epilogue of the segment: O^T -> acc[head][dim], plus (m, l)
            wait_w(bar(B_OFULL), nseg & 1);
            if (group_or(fail)) { stop = true; break; }
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 8; c++) {
                uint32_t o[32];
                tc_ld32(tmem + lane_base + COL_O + c * 32, o);
                tc_wait_ld();
                const uint32_t dim = (c / 2) * 128 + q4 * 32 + lane;
                const uint32_t hb = h0 + (c & 1) * 32;
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (hb + i < H) recs[(size_t(seg) * H + hb + i) * kPart + 2 + dim] = __uint_as_float(o[i]);
                }
            }
            if (qd == 0) {
                if (h0 + r_a < H) {
                    float* rc = recs + (size_t(seg) * H + h0 + r_a) * kPart;
                    rc[0] = m_a;
                    rc[1] = l_a;
                }
                if (h0 + r_b < H) {
                    float* rc = recs + (size_t(seg) * H + h0 + r_b) * kPart;
                    rc[0] = m_b;
                    rc[1] = l_b;
                }
            }
            tc_fence_before();
            nseg++;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

int decode_tc5_configure()
{
    cudaError_t e = cudaFuncSetAttribute(decode_tc5_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    e = cudaFuncSetAttribute(decode_tc5_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES);
    return int(e);
}

int launch_decode_tc5(int dtype, const void* tmaps, uint32_t layer, uint32_t n_pages, const StepMeta& m, float* recs,
                      uint32_t H, uint32_t* status, cudaStream_t st)
{
    if (m.ctas == 0) return 0;
    const CUtensorMap* maps = static_cast<const CUtensorMap*>(tmaps);
    const float scale_log2 = 1.4426950408889634f / sqrtf(float(kQDim));
    dim3 grid(m.ctas, (H + HG - 1) / HG);
    if (dtype == 0)
        return int(launch_pdl(decode_tc5_kernel<__half>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, maps[kMapPoolPage], maps[kMapQueries],
                              layer, n_pages, m, recs, H, scale_log2, status));
    return int(launch_pdl(decode_tc5_kernel<__nv_bfloat16>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, maps[kMapPoolPage],
                          maps[kMapQueries], layer, n_pages, m, recs, H, scale_log2, status));
}

}  // namespace mla
