// Split-KV absorbed MLA attention for narrow head counts (groups of 16 heads) on the 5th-generation tensor cores of
// sm_100a, in the transposed orientation: the tokens of a page are the M rows, the heads the N columns.
//
// With 16 heads the head-major tiles of mla_decode_tc5.cu would be three quarters padding.  Here the page tile is the
// A operand of BOTH contractions and the small matrices (queries, probabilities) are the B operands:
//
//   TMA      page tile [64 tok][576] -> shared memory as 9 swizzled sub-tiles [64 tok][64 dims]: four pairs into a ring of
//            11 pair slots and the rope sub-tile into a ring of 3, each with its own barriers (the score MMAs start while
//            the rest of the page lands, and 1.75 pages can be on their way while one is consumed); Q' of the row's head
//            group [16 heads][576] as 9 sub-tiles [16][64]
//   QK       S^T[64 tok x 16 heads] = K[64 x 576] . Q'^T          36 x tcgen05.mma  M=64  N=16 K=16
//                                     A = cache sub-tiles (K-major), B = Q' (K-major)
//   softmax  S^T keeps 16 token rows in lanes 0-15 of every TMEM sub-partition; a 16x256b load spreads them over the
//            warp (thread i: tokens i/4 and i/4 + 8, heads 2(i%4), +1, 8 + 2(i%4), +1).  The maximum of a head over
//            the 64 tokens is three shuffles and one exchange between the four warps; log2-domain online softmax with
//            lazy rescaling (threshold 2^8); the row sums stay per thread until the end of the segment
//   PV       O^T[512 dims x 16 heads] += V^T[512 x 64 tok] . P^T   16 x tcgen05.mma M=128 N=16 K=16
//                                     A = the SAME cache sub-tiles read MN-major, B = P^T [16 heads][64 tok] (K-major)
//
// Per 64-token tile the tensor core reads the page twice from shared memory and 20 KB of small operands: ~1,600 cycles
// of pipe time for 72 KB of cache, so the kernel is bound by HBM, not by padding work.
// Tensor memory: O^T in 4 x 16 columns, four partial score tiles (one per QK issuer) in 4 x 16 columns.
// Warp roles: warp 0 = TMA producer, warps 1-6 = MMA issuers (four for QK, two for PV; warp 1 also owns the TMEM
// allocation), warps 7-10 = softmax, correction and epilogue (warp w touches TMEM lanes 32*(w%4) .. +31).
// Output per (segment, head): m (reference maximum, log2 domain), l, acc[512] — 514 floats.
//
// Every mbarrier wait is bounded: after ~2 s a waiter raises ST_WAIT_TIMEOUT in the status word, sets the block's abort
// flag and every role leaves its loops; TMEM is freed on all paths.
#include "mla_launch.h"
#include "mla_tc5.cuh"

namespace mla {

namespace {

using namespace tc5;

constexpr int TILE = 64;                          // tokens per tile = one page
constexpr int HG = 16;                            // heads per block
constexpr int NSUB = kRow / 64;                   // 9 sub-tiles of 64 dims
constexpr int SUB_BYTES = TILE * 128;             // 8 KB
// A page does not sit in one stage buffer: its eight sub-tiles of latent dims are four PAIRS (one 128-dim chunk of O^T
// each, 16 KB) in a ring of 11 pair slots, its rope sub-tile goes to a ring of three.  Two whole pages plus three quarters
// of a third fit beside Q' and P, so up to 1.75 pages are on their way while one is consumed (two whole-page buffers,
// the most that fits as stages, leave one load in flight and the kernel waiting for it: 0.75 of the measured HBM peak).
constexpr int PAIR_BYTES = 2 * SUB_BYTES;         // 16 KB: sub-tiles 2i, 2i+1 of a page
constexpr int N_PAIR_SLOTS = 11, N_ROPE_SLOTS = 3;
// No L2 prefetch ahead of the loads: measured on 16 heads x 32 sequences x 8192 tokens, prefetching 4 / 8 pages ahead
// (tensor-map or linear) takes the kernel from 59 us to 77 / 88 us.
constexpr int Q_SUB = HG * 128;                   // 2,048: [16 heads][64 dims]
constexpr int Q_BYTES = NSUB * Q_SUB;             // 18,432
constexpr int P_BYTES = HG * 128;                 // 2,048: [16 heads][64 tok]
constexpr int OFF_Q = 0;
constexpr int OFF_PAIRS = OFF_Q + Q_BYTES;
constexpr int OFF_ROPE = OFF_PAIRS + N_PAIR_SLOTS * PAIR_BYTES;
constexpr int OFF_P = OFF_ROPE + N_ROPE_SLOTS * SUB_BYTES;
constexpr int OFF_MISC = OFF_P + P_BYTES;         // barriers, alpha, tmem base, abort flag
constexpr int MISC_BYTES = 1280;
constexpr int M_TMEM = 304, M_ABORT = 308, M_ALPHA = 320, M_HMAX = 384, M_LSUM = 896;   // alpha [16]; hmax [2][4][16]; lsum [4][16]
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;   // +1024: manual 1 KB alignment
static_assert(SMEM_BYTES <= 232448, "over the shared memory of one block");
static_assert(OFF_PAIRS % 1024 == 0 && OFF_ROPE % 1024 == 0 && OFF_P % 1024 == 0, "swizzled tiles need 1 KB alignment");

constexpr uint32_t TMEM_COLS = 128;
constexpr uint32_t COL_O = 0;                     // 4 chunks of 128 dims x 16 head columns
constexpr uint32_t COL_S = 64;                    // 4 partial score tiles x 16 head columns

constexpr int N_QK = 4, N_PV = 2;                 // MMA-issuing warps for QK and for PV
constexpr int NUM_THREADS = 32 * (1 + N_QK + N_PV + 4);   // producer + issuers + 4 softmax warps
constexpr int SOFTMAX_THREADS = 128;
constexpr float RESCALE_THRESHOLD = 8.0f;         // log2 units

// barrier slots inside the misc area (8 bytes each)
// one full / empty barrier per pair slot and per rope slot: QK issuer i works on pair i of a page as soon as it has landed
// (issuer 3 also on the rope sub-tile); a pair slot is free again when the PV MMAs of its chunk complete, a rope slot
// when the score MMAs on it complete
enum { B_QFULL = 0, B_QEMPTY, B_KF, B_KE = B_KF + N_PAIR_SLOTS, B_RF = B_KE + N_PAIR_SLOTS, B_RE = B_RF + N_ROPE_SLOTS,
       B_SFULL0 = B_RE + N_ROPE_SLOTS, B_SFULL1, B_SEMPTY0, B_SEMPTY1, B_PFULL, B_PEMPTY, B_OFULL, B_COUNT };
static_assert(N_QK == 4 && N_PV == 2, "the split of a page over the issuers below");
static_assert(B_COUNT * 8 <= M_TMEM, "barriers overflow their area");


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
decode_tc5_t16_kernel(const __grid_constant__ CUtensorMap map_pair, const __grid_constant__ CUtensorMap map_sub,
                      const __grid_constant__ CUtensorMap map_q,
                  uint32_t layer, uint32_t n_pages, StepMeta m, float* __restrict__ recs, uint32_t H,
                  float scale_log2, uint32_t* __restrict__ status)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = smem_raw + (base - raw);
    const uint32_t sQ = base + OFF_Q, sPairs = base + OFF_PAIRS, sRope = base + OFF_ROPE, sP = base + OFF_P;
    const uint32_t sBar = base + OFF_MISC;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC + M_TMEM);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + M_ABORT);
    float* alpha_s = reinterpret_cast<float*>(sm + OFF_MISC + M_ALPHA);
    float* hmax_s = reinterpret_cast<float*>(sm + OFF_MISC + M_HMAX);
    float* lsum_s = reinterpret_cast<float*>(sm + OFF_MISC + M_LSUM);
    auto bar = [&](int i) { return sBar + 8u * uint32_t(i); };

    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t cta = blockIdx.x, h0 = blockIdx.y * HG;
    const uint32_t seg_begin = m.cta_seg_begin[cta], seg_end = m.cta_seg_begin[cta + 1];

    grid_launch_dependents();
    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar(B_QFULL), 1);
        mbar_init(bar(B_QEMPTY), N_QK);
        for (int i = 0; i < 2 * N_PAIR_SLOTS + 2 * N_ROPE_SLOTS; i++) mbar_init(bar(B_KF + i), 1);
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
                // Q' of this row's head group: 9 sub-tiles of [16 heads][64 dims] in one box
                ok = mbar_wait(bar(B_QEMPTY), (nseg & 1) ^ 1, abort_flag, status);
                if (!ok) break;
                mbar_expect_tx(bar(B_QFULL), Q_BYTES);
                tma_load_3d(sQ, &map_q, bar(B_QFULL), 0, int(s.row * H + h0), 0);          // all 9 sub-tiles in one box
                const uint32_t* tbl = m.tables + m.seq_tbl_off[m.row_seq[s.row]];
                for (uint32_t j = 0; j < s.n_tiles && ok; j++, t++) {
                    uint32_t page = tbl[s.page_begin + j];
                    if (page >= n_pages) {
                        atomicOr(status, ST_BAD_PAGE);
                        page = 0;
                    }
#pragma unroll 1
                    for (uint32_t i = 0; i < 4 && ok; i++) {          // pair i of page t: the (4t + i)-th use of the pair ring
                        const uint32_t u = 4 * t + i, slot = u % N_PAIR_SLOTS;
                        ok = mbar_wait(bar(B_KE + slot), ((u / N_PAIR_SLOTS) & 1) ^ 1, abort_flag, status);
                        if (!ok) break;
                        mbar_expect_tx(bar(B_KF + slot), PAIR_BYTES);
                        tma_load_4d(sPairs + slot * PAIR_BYTES, &map_pair, bar(B_KF + slot), 0, int(page * kPage), int(2 * i), int(layer));
                    }
                    if (!ok) break;
                    const uint32_t rs = t % N_ROPE_SLOTS;
                    ok = mbar_wait(bar(B_RE + rs), ((t / N_ROPE_SLOTS) & 1) ^ 1, abort_flag, status);
                    if (!ok) break;
                    mbar_expect_tx(bar(B_RF + rs), SUB_BYTES);
                    tma_load_3d(sRope + rs * SUB_BYTES, &map_sub, bar(B_RF + rs), kRank, int(page * kPage), int(layer));
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
        // (sub-tile pairs 0-1, 2-3, 4-5, 6-7 + rope; the softmax adds them), warps 5-6 take two of the four
        // 128-dim chunks of O^T each.  The warp runs the loop uniformly (operands stay in uniform
        // registers) and one elected lane issues.
        constexpr uint32_t IDESC_QK = instr_desc(Fmt<T>::v, TILE, HG, 0, 0);          // M = 64 tokens, N = 16 heads
        constexpr uint32_t IDESC_PV = instr_desc(Fmt<T>::v, 128, HG, 1, 0);
        constexpr uint32_t HI = desc_hi(1024);          // every operand: 8-row groups 1024 B apart
        const bool is_qk = warp <= N_QK;
        const uint32_t part = is_qk ? warp - 1 : warp - 1 - N_QK;
        const uint32_t qk_b = desc_lo(sQ, 16);          // Q' (K-major), the B operand here
        const uint32_t pv_b = desc_lo(sP, 16);          // P (K-major)
        uint32_t t = 0, nseg = 0;
        bool ok = true;
        for (uint32_t seg = seg_begin; seg < seg_end && ok; seg++) {
            const SegInfo s = load_seg(m, seg);
            if (s.n_tiles == 0) continue;
            if (is_qk) ok = mbar_wait(bar(B_QFULL), nseg & 1, abort_flag, status);
            for (uint32_t j = 0; j < s.n_tiles && ok; j++, t++) {
                if (is_qk) {
                    // QK issuer i: pair i of the page (sub-tiles 2i, 2i+1); issuer 3 also the rope sub-tile
                    const uint32_t u = 4 * t + part, slot = u % N_PAIR_SLOTS, rs = t % N_ROPE_SLOTS;
                    ok = mbar_wait(bar(B_KF + slot), (u / N_PAIR_SLOTS) & 1, abort_flag, status) &&
                         (part != 3 || mbar_wait(bar(B_RF + rs), (t / N_ROPE_SLOTS) & 1, abort_flag, status)) &&
                         mbar_wait(bar(B_SEMPTY0), (t & 1) ^ 1, abort_flag, status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a0 = desc_lo(sPairs + slot * PAIR_BYTES, 16), ar = desc_lo(sRope + rs * SUB_BYTES, 16);
                    const uint32_t d = tmem + COL_S + part * HG;
                    if (elect_one()) {
#pragma unroll
                        for (int cc = 0; cc < 2; cc++)
#pragma unroll
                            for (int k = 0; k < 4; k++)
                                tc_mma(d, a0 + ((cc * SUB_BYTES + k * 32) >> 4), HI, qk_b + (((2 * part + cc) * Q_SUB + k * 32) >> 4),
                                       HI, IDESC_QK, (cc == 0 && k == 0) ? 0u : 1u);
                        if (part == 3) {
#pragma unroll
                            for (int k = 0; k < 4; k++)
                                tc_mma(d, ar + ((k * 32) >> 4), HI, qk_b + ((8 * Q_SUB + k * 32) >> 4), HI, IDESC_QK, 1u);
                            tc_commit(bar(B_RE + rs));
                        }
                        tc_commit(bar(B_SFULL0));
                        if (j + 1 == s.n_tiles) tc_commit(bar(B_QEMPTY));
                    }
                    __syncwarp();
                } else {
                    // PV issuer p: chunks 2p, 2p+1 of O^T = pairs 2p, 2p+1 of the page read MN-major.  The pairs have landed:
                    // P exists only after all four score issuers waited for theirs.
                    ok = mbar_wait(bar(B_PFULL), t & 1, abort_flag, status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t fresh = j == 0 ? 0u : 1u;
                    if (elect_one()) {
#pragma unroll
                        for (int cc = 0; cc < 2; cc++) {
                            const uint32_t c = part * 2 + cc, slot = (4 * t + c) % N_PAIR_SLOTS;
                            const uint32_t a0 = desc_lo(sPairs + slot * PAIR_BYTES, SUB_BYTES);
#pragma unroll
                            for (int k = 0; k < TILE / 16; k++)
                                tc_mma(tmem + COL_O + c * HG, a0 + ((k * 2048) >> 4), HI, pv_b + ((k * 32) >> 4), HI, IDESC_PV,
                                       k == 0 ? fresh : 1u);
                            tc_commit(bar(B_KE + slot));
                        }
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
        // S^T (M=64 layout) keeps token rows 16q .. 16q+15 in TMEM lanes 0-15 of sub-partition q.  A 16x256b.x2 load
        // spreads them over the warp: thread i holds tokens 16q + i/4 (registers 0, 1, 4, 5) and + 8 (registers 2, 3, 6, 7)
        // of heads 2(i%4), +1 (registers 0-3) and 8 + 2(i%4), +1 (registers 4-7).
        // The 128 threads meet at two named barriers every tile (maxima exchanged; rescale needed or not).  A failed
        // (timed-out / aborted) wait never makes a thread leave early on its own: the failure is carried to the next
        // barrier, OR-reduced there, and all 128 threads leave together.
        const uint32_t q4 = warp % 4;                         // TMEM sub-partition of this warp
        const uint32_t lane_base = (q4 * 32u) << 16;
        const uint32_t qd = lane & 3, tr = lane >> 2;         // head quad, token row within the warp's 16 (and + 8)
        auto head_of = [&](int j) { return uint32_t(8 * (j >> 1) + 2 * qd + (j & 1)); };   // this thread's four heads
        float m_ref[4], psum[4];
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
        auto rows_max = [](float v) {                         // over the 8 threads that hold the same heads
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
            return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
        };
        auto rows_sum = [](float v) {
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            return v + __shfl_xor_sync(0xffffffffu, v, 16);
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
#pragma unroll
            for (int j = 0; j < 4; j++) { m_ref[j] = -INFINITY; psum[j] = 0.0f; }
            for (uint32_t j = 0; j < s.n_tiles; j++, t++) {
                wait_w(bar(B_SFULL0), t & 1);
                float sv[8];
                if (!fail) {
                    tc_fence_after();
                    uint32_t p0[8], p1[8], p2[8], p3[8];
                    tc_ld16x256_x2(tmem + lane_base + COL_S, p0);
                    tc_ld16x256_x2(tmem + lane_base + COL_S + HG, p1);
                    tc_ld16x256_x2(tmem + lane_base + COL_S + 2 * HG, p2);
                    tc_ld16x256_x2(tmem + lane_base + COL_S + 3 * HG, p3);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 8; i++)        // the four issuers' partial sums, always in this order
                        sv[i] = ((__uint_as_float(p0[i]) + __uint_as_float(p1[i])) + __uint_as_float(p2[i])) + __uint_as_float(p3[i]);
                    tc_fence_before();
                    mbar_arrive(bar(B_SEMPTY0));
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++) sv[i] = 0.0f;
                }
                // registers: i = 4k + 2e' + e -> head 8k + 2qd + e, token 16 q4 + tr + 8 e'
                const uint32_t valid = min(uint32_t(TILE), s.n_tok - j * TILE);
                const uint32_t tok_a = 16 * q4 + tr, tok_b = tok_a + 8;
                const bool in_a = tok_a < valid, in_b = tok_b < valid;
                float mx[4];
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    const int k = jj >> 1, e = jj & 1;
                    const float va = in_a ? sv[4 * k + e] * scale_log2 : -INFINITY;
                    const float vb = in_b ? sv[4 * k + 2 + e] * scale_log2 : -INFINITY;
                    sv[4 * k + e] = va;
                    sv[4 * k + 2 + e] = vb;
                    mx[jj] = rows_max(fmaxf(va, vb));
                }
                float* hm = hmax_s + (t & 1) * 64;            // [4 warps][16 heads], two buffers by tile parity
                if (tr == 0) {
#pragma unroll
                    for (int jj = 0; jj < 4; jj++) hm[q4 * 16 + head_of(jj)] = mx[jj];
                }
                if (group_or(fail)) { stop = true; break; }
                float alpha[4];
                bool need = false;
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    const uint32_t h = head_of(jj);
                    const float mt = fmaxf(fmaxf(hm[h], hm[16 + h]), fmaxf(hm[32 + h], hm[48 + h]));
                    alpha[jj] = 1.0f;
                    if (j == 0) m_ref[jj] = mt;
                    else if (mt > m_ref[jj] + RESCALE_THRESHOLD) { alpha[jj] = fast_ex2(m_ref[jj] - mt); m_ref[jj] = mt; need = true; }
                }
                // every thread of a head quad column computes the same references; one of them publishes the factors
                const bool any_need = group_or(need);
                uint16_t pb[8];
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    const int k = jj >> 1, e = jj & 1;
                    const float mr = m_ref[jj] == -INFINITY ? 0.0f : m_ref[jj];
                    const float pa = fast_ex2(sv[4 * k + e] - mr), pbv = fast_ex2(sv[4 * k + 2 + e] - mr);
                    psum[jj] = psum[jj] * alpha[jj] + (pa + pbv);
                    const T ha = Elem<T>::from_f32(pa), hb = Elem<T>::from_f32(pbv);
                    pb[2 * jj] = *reinterpret_cast<const uint16_t*>(&ha);
                    pb[2 * jj + 1] = *reinterpret_cast<const uint16_t*>(&hb);
                }
                // PV of the previous tile must be complete: O is stable and P is free
                wait_w(bar(B_PEMPTY), (t - 1) & 1);
                if (any_need) {
                    if (q4 == 0 && tr == 0) {
#pragma unroll
                        for (int jj = 0; jj < 4; jj++) alpha_s[head_of(jj)] = alpha[jj];
                    }
                    if (group_or(fail)) { stop = true; break; }
                    if (j > 0) {
                        // O^T[dim lane][head column] *= alpha[head]: 4 chunks x 16 head columns
                        tc_fence_after();
#pragma unroll 1
                        for (int c = 0; c < 4; c++) {
                            uint32_t o[16];
                            tc_ld16(tmem + lane_base + COL_O + c * HG, o);
                            tc_wait_ld();
#pragma unroll
                            for (int i = 0; i < 16; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha_s[i]);
                            tc_st16(tmem + lane_base + COL_O + c * HG, o);
                        }
                        tc_wait_st();
                    }
                }
                if (fail) continue;            // carried to the next barrier
                {
                    // P^T [16 heads][64 tok], K-major with the 128-byte swizzle: row = head, 16-byte chunk = tok / 8
#pragma unroll
                    for (int jj = 0; jj < 4; jj++) {
                        const uint32_t h = head_of(jj);
                        unsigned char* prow = sm + OFF_P + h * 128;
                        *reinterpret_cast<uint16_t*>(prow + (((tok_a >> 3) ^ (h & 7)) << 4) + (tok_a & 7) * 2) = pb[2 * jj];
                        *reinterpret_cast<uint16_t*>(prow + (((tok_b >> 3) ^ (h & 7)) << 4) + (tok_b & 7) * 2) = pb[2 * jj + 1];
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                tc_fence_before();
                mbar_arrive(bar(B_PFULL));
            }
            if (stop) break;
            // ---- epilogue of the segment: O^T -> acc[head][dim], plus (m, l)
            wait_w(bar(B_OFULL), nseg & 1);
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                const float ls = rows_sum(psum[jj]);
                if (tr == 0) lsum_s[q4 * 16 + head_of(jj)] = ls;
            }
            if (group_or(fail)) { stop = true; break; }
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t o[16];
                tc_ld16(tmem + lane_base + COL_O + c * HG, o);
                tc_wait_ld();
                const uint32_t dim = c * 128 + q4 * 32 + lane;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    if (h0 + i < H) recs[(size_t(seg) * H + h0 + i) * kPart + 2 + dim] = __uint_as_float(o[i]);
                }
            }
            if (q4 == 0 && tr == 0) {
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    const uint32_t h = head_of(jj);
                    if (h0 + h < H) {
                        float* rc = recs + (size_t(seg) * H + h0 + h) * kPart;
                        rc[0] = m_ref[jj];
                        rc[1] = (lsum_s[h] + lsum_s[16 + h]) + (lsum_s[32 + h] + lsum_s[48 + h]);
                    }
                }
            }
            // lsum_s and the score / O columns are reused by the next segment: everyone is done reading
            if (group_or(false)) { stop = true; break; }
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

int decode_tc5_t16_configure()
{
    cudaError_t e = cudaFuncSetAttribute(decode_tc5_t16_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    e = cudaFuncSetAttribute(decode_tc5_t16_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES);
    return int(e);
}

int launch_decode_tc5_t16(int dtype, const void* tmaps, uint32_t layer, uint32_t n_pages, const StepMeta& m, float* recs,
                      uint32_t H, uint32_t* status, cudaStream_t st)
{
    if (m.ctas == 0) return 0;
    const CUtensorMap* maps = static_cast<const CUtensorMap*>(tmaps);
    const float scale_log2 = 1.4426950408889634f / sqrtf(float(kQDim));
    dim3 grid(m.ctas, (H + HG - 1) / HG);
    if (dtype == 0)
        return int(launch_pdl(decode_tc5_t16_kernel<__half>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, maps[kMapPoolV], maps[kMapPoolSub],
                              maps[kMapQueries16], layer, n_pages, m, recs, H, scale_log2, status));
    return int(launch_pdl(decode_tc5_t16_kernel<__nv_bfloat16>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, maps[kMapPoolV],
                          maps[kMapPoolSub], maps[kMapQueries16], layer, n_pages, m, recs, H, scale_log2, status));
}

}  // namespace mla
