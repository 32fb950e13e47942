// Causal attention of a prefill chunk on the 5th-generation tensor cores, sm_100a.
//
// The reference runs its absorbed routine once per chunk token with a growing length (src/core/model/
// transformer.cpp:1325-1337: token t of a chunk appended at start_position attends rows [0, start_position + t + 1)).
// Any mathematically equal form within the attention tolerance may stand in for it; for MANY query tokens over the
// same cache the cheap form is the expanded one: the latent rows are expanded ONCE per layer into per-head keys and
// values with the same weights,
//     k[t][h] = ( W_UK_h . c_kv[t]  (128 dims) , k_rope[t] (64 dims, shared by all heads) ),   v[t][h] = W_UV_h . c_kv[t],
// (two dense projections, mla_gemm_tc5.cu), and every (128 query tokens x one head) tile then runs flash attention
// over 192-dim keys and 128-dim values: 2 x (192 + 128) flops per (query, key, head) pair instead of the absorbed
// form's 2 x (576 + 512), and each staged key/value tile serves 128 query tokens instead of one.
//
// One block per (tile of 128 query tokens, head); the whole tile state lives in tensor memory:
//   Q        [128 queries][192 dims] written once into tensor memory by the softmax threads (row = lane, two dims per
//            column) and used as the A operand of every score MMA: no shared-memory reads for it
//   TMA      per step of KT = 128 keys K [128][192] (two boxes of expanded nope dims + one box of rope dims straight from
//            the gathered latent rows) and V [128][128], rings of two each; a K buffer is free as soon as the score MMAs
//            that read it complete, a V buffer one softmax later
//   QK       S[128 queries x 128 keys] = Q . K^T         12 x tcgen05.mma M128 N128 K16 (A in tensor memory), two score
//            tiles in flight (steps of 64 keys with rings of four and three score tiles measure 13 % slower: the fixed
//            cost of a step - waits, the exchange of the maxima, the hand-over to the PV issuer - is paid per step)
//   softmax  NS = 2 threads per query row, 64 keys each (the parts of a row exchange their maxima through shared memory;
//            1, 2 and 4 threads per row measure the same within 2 %, 4 slightly slower): causal mask, log2-domain online
//            softmax with lazy rescaling (threshold 2^8); P in the storage type goes back into the tensor-memory columns
//            its scores came from
//   PV       O[128 queries x 128 value dims] += P . V    8 x tcgen05.mma M128 N128 K16, A = P in tensor memory, B = the
//            staged V tile read MN-major (no transpose)
//   rescale  a row whose maximum moved rescales its own O row (its own lane) after the previous PV completes; no
//            block-wide agreement is needed
//   epilogue O / l -> out[query][head][128], rounded once to the storage type
// The tensor core reads only K and V from shared memory (6 KB per MMA step would be 2 + 4 KB with Q and P there too).
// Warps: 0 TMA producer, 1 score-MMA issuer, 2 PV-MMA issuer (two issuers keep the tensor pipe fed while one of them
// waits), 3.. softmax / correction / epilogue.  All waits are bounded.
#include <cuda.h>

#include <algorithm>

#include "mla_launch.h"
#include "mla_tc5.cuh"

namespace mla {

namespace {

using namespace tc5;

#ifndef MLA_PREFILL_KT
#define MLA_PREFILL_KT 128
#endif
constexpr int QT = 128, KT = MLA_PREFILL_KT;           // queries per block, keys per step (64 or 128)
constexpr int K_SUB = KT * 128;                        // [KT keys][64 dims]
constexpr int K_STAGE = 3 * K_SUB, V_STAGE = 2 * K_SUB;        // K: 192 dims, V: 128 dims of KT keys
constexpr int K_STAGES = KT == 64 ? 4 : 2, V_STAGES = KT == 64 ? 4 : 2;
constexpr int OFF_K = 0, OFF_V = OFF_K + K_STAGES * K_STAGE, OFF_MISC = OFF_V + V_STAGES * V_STAGE;
#ifndef MLA_PREFILL_NS
#define MLA_PREFILL_NS 2
#endif
constexpr int NS = MLA_PREFILL_NS;                     // softmax threads per query row (1, 2 or 4)
constexpr int KP = KT / NS, QP = kQDim / NS, VP = kVDim / NS;   // keys, query dims, value dims per thread of a row
// hmax: [2 step parities][NS parts][128 rows]; lsum: [NS parts][128 rows]
constexpr int M_HMAX = 256, M_LSUM = M_HMAX + 2 * NS * QT * 4, M_TMEM = M_LSUM + NS * QT * 4, M_ABORT = M_TMEM + 4, MISC_BYTES = M_TMEM + 64;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;       // + slack for 1 KB alignment
constexpr int NUM_SOFTMAX = NS * QT;
constexpr int FIRST_SOFTMAX_WARP = 3;
constexpr int NUM_THREADS = 32 * FIRST_SOFTMAX_WARP + NUM_SOFTMAX;
// tensor memory columns: Q as 16-bit pairs (96), S_BUFS score tiles (P of a step overwrites the head of each part of its
// scores), O
constexpr int S_BUFS = KT == 64 ? 3 : 2;                              // score tiles in flight: QK of step t + 1 never waits for softmax t
constexpr uint32_t TMEM_COLS = 512, COL_Q = 0, COL_S = 128, COL_O = COL_S + S_BUFS * KT;
static_assert(COL_O + kVDim <= TMEM_COLS, "tensor memory columns");
constexpr float RESCALE_THRESHOLD = 8.0f;
enum { B_QFULL = 0, B_KFULL, B_KEMPTY = B_KFULL + K_STAGES, B_VFULL = B_KEMPTY + K_STAGES, B_VEMPTY = B_VFULL + V_STAGES,
       B_SFULL = B_VEMPTY + V_STAGES, B_PFULL = B_SFULL + S_BUFS, B_PVDONE, B_OFULL = B_PVDONE + S_BUFS, B_COUNT };
static_assert(B_COUNT * 8 <= M_HMAX && B_COUNT <= 32, "barriers overflow their area");
static_assert(SMEM_BYTES <= 232448, "over the shared memory of one block");

struct ChunkArgs {
    uint32_t q_row0;        // first query row of the chunk in the q / out tensors
    uint32_t n_new;         // query tokens in the chunk
    uint32_t start;         // cache rows of the sequence before the chunk
    uint32_t H;
};

template <typename T>
__global__ void __launch_bounds__(NUM_THREADS, 1)
prefill_tc5_kernel(const T* __restrict__ q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const __grid_constant__ CUtensorMap map_r, ChunkArgs a, T* __restrict__ out, float scale_log2,
                   uint32_t* __restrict__ status)
{
    extern __shared__ unsigned char prefill_smem[];
    const uint32_t raw = smem_u32(prefill_smem);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = prefill_smem + (base - raw);
    const uint32_t sK = base + OFF_K, sV = base + OFF_V, sBar = base + OFF_MISC;
    auto bar = [&](int i) { return sBar + 8u * uint32_t(i); };
    float* hmax_s = reinterpret_cast<float*>(sm + OFF_MISC + M_HMAX);
    float* lsum_s = reinterpret_cast<float*>(sm + OFF_MISC + M_LSUM);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC + M_TMEM);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + M_ABORT);

    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    // long tiles first: the last query tile of a chunk sees the most keys
    const uint32_t n_qt = (a.n_new + QT - 1) / QT, qt = n_qt - 1 - blockIdx.x, h = blockIdx.y;
    const uint32_t q0 = qt * QT;                                   // first query token of this tile within the chunk
    const uint32_t total = a.start + a.n_new;
    const uint32_t kv_end = min(total, a.start + q0 + QT);         // keys any query of this tile may see
    const uint32_t n_kv = (kv_end + KT - 1) / KT;

    grid_launch_dependents();
    if (warp == 0 && lane < B_COUNT) {
        const int i = int(lane);
        mbar_init(bar(i), i == B_QFULL || i == B_PFULL ? uint32_t(NUM_SOFTMAX) : 1u);
    }
    if (warp == 0) mbar_init_fence();
    if (tid == 0) *abort_flag = 0;
    if (warp == 1) tc_alloc<TMEM_COLS>(tmem_slot);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    grid_dependency_wait();                 // expanded keys / values and the queries come from earlier kernels

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            for (uint32_t t = 0; t < n_kv && ok; t++) {
                const int ks = int(t % K_STAGES), vs = int(t % V_STAGES);
                ok = mbar_wait(bar(B_KEMPTY + ks), ((t / K_STAGES) & 1) ^ 1, abort_flag, status);
                if (!ok) break;
                const uint32_t kd = sK + ks * K_STAGE;
                mbar_expect_tx(bar(B_KFULL + ks), K_STAGE);
                tma_load_2d(kd, &map_k, bar(B_KFULL + ks), int(h * kNope), int(t * KT));
                tma_load_2d(kd + K_SUB, &map_k, bar(B_KFULL + ks), int(h * kNope + 64), int(t * KT));
                tma_load_2d(kd + 2 * K_SUB, &map_r, bar(B_KFULL + ks), kRank, int(t * KT));
                ok = mbar_wait(bar(B_VEMPTY + vs), ((t / V_STAGES) & 1) ^ 1, abort_flag, status);
                if (!ok) break;
                const uint32_t vd = sV + vs * V_STAGE;
                mbar_expect_tx(bar(B_VFULL + vs), V_STAGE);
                tma_load_2d(vd, &map_v, bar(B_VFULL + vs), int(h * kVDim), int(t * KT));
                tma_load_2d(vd + K_SUB, &map_v, bar(B_VFULL + vs), int(h * kVDim + 64), int(t * KT));
            }
        }
    } else if (warp == 1) {
        // ---- score MMAs.  The score buffer of step t held P(t - S_BUFS): wait for the PV MMAs that read it.
        constexpr uint32_t IDESC_QK = instr_desc(Fmt<T>::v, QT, KT, 0, 0);
        constexpr uint32_t HI = desc_hi(1024);
        bool ok = mbar_wait(bar(B_QFULL), 0, abort_flag, status);
        for (uint32_t t = 0; t < n_kv && ok; t++) {
            const int ks = int(t % K_STAGES), b = int(t % S_BUFS);
            ok = mbar_wait(bar(B_KFULL + ks), (t / K_STAGES) & 1, abort_flag, status) &&
                 (t < S_BUFS || mbar_wait(bar(B_PVDONE + b), (t / S_BUFS - 1) & 1, abort_flag, status));
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t kb = desc_lo(sK + ks * K_STAGE);
#pragma unroll
                for (int c = 0; c < 3; c++)
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        tc_mma_ts(tmem + COL_S + b * KT, tmem + COL_Q + (c * 4 + k) * 8, kb + ((c * K_SUB + k * 32) >> 4), HI,
                                  IDESC_QK, (c == 0 && k == 0) ? 0u : 1u);
                tc_commit(bar(B_SFULL + b));
                tc_commit(bar(B_KEMPTY + ks));
            }
            __syncwarp();
        }
    } else if (warp == 2) {
        // ---- O += P(t) . V(t); P(t) sits where the scores of step t were
        constexpr uint32_t IDESC_PV = instr_desc(Fmt<T>::v, QT, kVDim, 0, 1);
        constexpr uint32_t HI = desc_hi(1024);
        bool ok = true;
        for (uint32_t t = 0; t < n_kv && ok; t++) {
            const int vs = int(t % V_STAGES);
            ok = mbar_wait(bar(B_VFULL + vs), (t / V_STAGES) & 1, abort_flag, status) &&
                 mbar_wait(bar(B_PFULL), t & 1, abort_flag, status);
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t vb = desc_lo(sV + vs * V_STAGE, K_SUB), pa = tmem + COL_S + (t % S_BUFS) * KT;
#pragma unroll
                for (int k = 0; k < KT / 16; k++)    // keys 16k..: 8 columns at the head of the score columns of their part
                    tc_mma_ts(tmem + COL_O, pa + (16 * k / KP) * KP + (16 * k % KP) / 2, vb + ((k * 2048) >> 4), HI, IDESC_PV,
                              (t == 0 && k == 0) ? 0u : 1u);
                tc_commit(bar(B_VEMPTY + vs));
                tc_commit(bar(B_PVDONE + (t % S_BUFS)));
                if (t + 1 == n_kv) tc_commit(bar(B_OFULL));
            }
            __syncwarp();
        }
    } else {
        // ===== softmax / correction / epilogue: NS threads per query row; the row is this thread's tensor-memory lane =====
        static_assert(NS == 1 || NS == 2 || NS == 4, "the part sizes below");
        const uint32_t q4 = warp % 4, part = (warp - FIRST_SOFTMAX_WARP) / 4, r = q4 * 32 + lane;
        const uint32_t lane_base = (q4 * 32u) << 16;
        const uint32_t qi = q0 + r;                                      // query token within the chunk
        const bool live = qi < a.n_new;
        const uint32_t my_pos = a.start + qi;                            // last key this query may see
        {   // this thread's part of the query row: QP dims = QP / 2 columns, in three stores
            constexpr int W = QP / 6;
            const uint4* src = reinterpret_cast<const uint4*>(q + (size_t(a.q_row0 + qi) * a.H + h) * kQDim + part * QP);
#pragma unroll
            for (int c = 0; c < 3; c++) {
                uint32_t w[W];
#pragma unroll
                for (int j = 0; j < W / 4; j++) {
                    const uint4 v = live ? __ldg(src + c * (W / 4) + j) : make_uint4(0u, 0u, 0u, 0u);
                    w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
                }
                tc_stn(tmem + lane_base + COL_Q + part * (QP / 2) + c * W, w);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(B_QFULL));
        }
        float m_run = -INFINITY, l_run = 0.0f;                           // l_run: this part's share of the row sum
        bool fail = false;
        auto wait_w = [&](uint32_t b, uint32_t parity) {
            if (!fail) fail = !mbar_wait(b, parity, abort_flag, status);
            fail = __any_sync(0xffffffffu, fail);
        };
        auto group_or = [&](bool pred) -> bool {              // barrier over the softmax threads + OR
            uint32_t rr;
            asm volatile(
                "{\n.reg .pred pi, po;\n"
                "setp.ne.b32 pi, %1, 0;\n"
                "barrier.cta.red.or.pred po, 1, %2, pi;\n"
                "selp.u32 %0, 1, 0, po;\n}\n"
                : "=r"(rr) : "r"(uint32_t(pred)), "n"(NUM_SOFTMAX) : "memory");
            return rr != 0;
        };
        auto group_sync = [&]() { asm volatile("barrier.cta.sync 2, %0;\n" :: "n"(NUM_SOFTMAX) : "memory"); };
        for (uint32_t t = 0; t < n_kv; t++) {
            const uint32_t b = t % S_BUFS;
            const uint32_t s_addr = tmem + lane_base + COL_S + b * KT + part * KP;
            wait_w(bar(B_SFULL + b), (t / S_BUFS) & 1);
            uint32_t sv[KP];
            if (!fail) {
                tc_fence_after();
                tc_ldn(s_addr, sv);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < KP; i++) sv[i] = 0u;
            }
            const uint32_t k0 = t * KT + part * KP;
            if (k0 + KP > my_pos + 1 || k0 + KP > total) {               // causal / end mask (only near the diagonal)
#pragma unroll
                for (int i = 0; i < KP; i++)
                    if (k0 + uint32_t(i) > my_pos || k0 + uint32_t(i) >= total) sv[i] = __float_as_uint(-INFINITY);
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < KP; i++) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // Two buffers by step parity: another part of a row may already be one step ahead when this one reads.
            if constexpr (NS > 1) {
                float* hm = hmax_s + (t & 1) * NS * QT;
                hm[part * QT + r] = mx;
                group_sync();
#pragma unroll
                for (int p = 0; p < NS; p++) mx = fmaxf(mx, hm[p * QT + r]);
            }
            mx *= scale_log2;                                            // the same in all parts of a row
            float alpha = 1.0f;
            bool need = false;
            if (m_run == -INFINITY) { m_run = mx; }                     // nothing accumulated for this row yet
            else if (mx > m_run + RESCALE_THRESHOLD) { alpha = fast_ex2(m_run - mx); m_run = mx; need = true; }
            float sum2[2] = {0.0f, 0.0f};
            uint32_t pk[KP / 2];
            const float mref = m_run == -INFINITY ? 0.0f : m_run;         // a row whose keys so far are all masked: p = 0
#pragma unroll
            for (int i = 0; i < KP; i += 2) {
                const float p0 = fast_ex2(fmaf(__uint_as_float(sv[i]), scale_log2, -mref));
                const float p1 = fast_ex2(fmaf(__uint_as_float(sv[i + 1]), scale_log2, -mref));
                sum2[(i >> 1) & 1] += p0 + p1;
                pk[i / 2] = Elem<T>::pack2(p0, p1);
            }
            l_run = l_run * alpha + (sum2[0] + sum2[1]);
            if (t > 0) wait_w(bar(B_PVDONE + ((t - 1) % S_BUFS)), ((t - 1) / S_BUFS) & 1);   // PV of the previous step complete: this row of O is stable
            if (fail) continue;
            tc_fence_after();
            // tcgen05.ld / .st are warp-wide: the warp rescales when any of its rows needs it (the others multiply by 1)
            if (t > 0 && __any_sync(0xffffffffu, need)) {    // O[this row][this part's VP value dims] *= alpha
#pragma unroll 1
                for (uint32_t c = 0; c < VP / 32; c++) {
                    uint32_t o[32];
                    tc_ld32(tmem + lane_base + COL_O + part * VP + c * 32, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tc_st32(tmem + lane_base + COL_O + part * VP + c * 32, o);
                }
            }
            tc_stn(s_addr, pk);              // P over the first half of this thread's own score columns
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(B_PFULL));
        }
        wait_w(bar(B_OFULL), 0);
        lsum_s[part * QT + r] = l_run;
        const bool bad = group_or(fail);
        if (!bad) {
            tc_fence_after();
            float l = 0.0f;
#pragma unroll
            for (int p = 0; p < NS; p++) l += lsum_s[p * QT + r];
            const float linv = l > 0.0f ? 1.0f / l : 0.0f;
            uint4* dst = reinterpret_cast<uint4*>(out + (size_t(a.q_row0 + qi) * a.H + h) * kVDim + part * VP);
#pragma unroll 1
            for (uint32_t c = 0; c < VP / 32; c++) {
                uint32_t o[32];
                tc_ld32(tmem + lane_base + COL_O + part * VP + c * 32, o);
                tc_wait_ld();
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 16; i++)
                    w[i] = Elem<T>::pack2(__uint_as_float(o[2 * i]) * linv, __uint_as_float(o[2 * i + 1]) * linv);
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (live) dst[c * 4 + j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
            }
        }
        tc_fence_before();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tc_dealloc<TMEM_COLS>(tmem);
    }
}

// rows [0, n) of a sequence, page by page, into a contiguous [n][576] buffer
__global__ void __launch_bounds__(128)
gather_rows_kernel(const uint4* __restrict__ pool, uint64_t pool_slots, const uint32_t* __restrict__ table, uint32_t n,
                   uint4* __restrict__ dst, uint32_t* __restrict__ status)
{
    grid_launch_dependents();
    grid_dependency_wait();
    constexpr int kChunks = kRow * 2 / 16;
    const uint32_t r = blockIdx.x * 4 + threadIdx.x / 32;
    if (r >= n) return;
    const uint64_t slot = uint64_t(table[r / kPage]) * kPage + r % kPage;
    if (slot >= pool_slots) {
        if ((threadIdx.x & 31) == 0) atomicOr(status, ST_BAD_SLOT);
        return;
    }
    for (int c = threadIdx.x & 31; c < kChunks; c += 32) dst[size_t(r) * kChunks + c] = pool[slot * kChunks + c];
}

// the last 64 dims of every head of `rows` query rows rotated with their positions (NeoX pairs, the append's table and
// rounding: reference transformer.cpp:1204-1240), everything else copied: q_out = rotated copy of q_in
template <typename T>
__global__ void __launch_bounds__(192)
rotate_q_rows_kernel(const T* __restrict__ q_in, T* __restrict__ q_out, uint32_t H, uint32_t pos0, const float* __restrict__ cos_sin,
                     uint32_t cs_rows, uint32_t* __restrict__ status)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t row = blockIdx.x, h = blockIdx.y, i = threadIdx.x, pos = pos0 + row;
    const T* src = q_in + (size_t(row) * H + h) * kQDim;
    T* dst = q_out + (size_t(row) * H + h) * kQDim;
    if (i < kNope) { dst[i] = src[i]; return; }
    if (pos >= cs_rows) { if (i == kNope) atomicOr(status, ST_BAD_SLOT); return; }
    const uint32_t j = (i - kNope) % 32;
    const float cs = cos_sin[size_t(pos) * kRope + j], sn = cos_sin[size_t(pos) * kRope + 32 + j];
    const float x0 = Elem<T>::to_f32(src[kNope + j]), x1 = Elem<T>::to_f32(src[kNope + 32 + j]);
    dst[i] = i < kNope + 32 ? Elem<T>::from_f32(__fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)))
                            : Elem<T>::from_f32(__fadd_rn(__fmul_rn(x1, cs), __fmul_rn(x0, sn)));
}

using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_map(CUtensorMap* map, int dtype, const void* ptr, uint64_t rows, uint64_t cols, uint64_t pitch, uint32_t box_rows)
{
    static TensorMapEncodeFn enc = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<TensorMapEncodeFn>(p);
    }();
    if (!enc) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr),
               dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int prefill_tc5_configure()
{
    cudaError_t e = cudaFuncSetAttribute(prefill_tc5_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(prefill_tc5_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    return int(e);
}

int launch_gather_rows(const void* layer_pool, uint64_t pool_slots, const uint32_t* table, uint32_t n, void* dst, uint32_t* status,
                       cudaStream_t st)
{
    if (n == 0) return 0;
    return int(launch_pdl(gather_rows_kernel, dim3((n + 3) / 4), dim3(128), 0, st, static_cast<const uint4*>(layer_pool), pool_slots,
                          table, n, static_cast<uint4*>(dst), status));
}

int launch_rotate_q_rows(int dtype, const void* q_in, void* q_out, uint32_t rows, uint32_t H, uint32_t pos0, const float* cos_sin,
                         uint32_t cs_rows, uint32_t* status, cudaStream_t st)
{
    if (rows == 0) return 0;
    if (dtype == 0)
        return int(launch_pdl(rotate_q_rows_kernel<__half>, dim3(rows, H), dim3(192), 0, st, static_cast<const __half*>(q_in),
                              static_cast<__half*>(q_out), H, pos0, cos_sin, cs_rows, status));
    return int(launch_pdl(rotate_q_rows_kernel<__nv_bfloat16>, dim3(rows, H), dim3(192), 0, st, static_cast<const __nv_bfloat16*>(q_in),
                          static_cast<__nv_bfloat16*>(q_out), H, pos0, cos_sin, cs_rows, status));
}

// One chunk of one sequence.  q: [q_rows_total][H][192] post-RoPE (DEVICE), chunk rows start at q_row0; kx / vx: expanded keys
// (nope dims) and values [total][H][128]; latent: the gathered rows [total][576] (their last 64 dims are the shared rope
// keys); out: [q_rows_total][H][128].  Returns a cudaError_t value, or -1 when a tensor map cannot be built.
int launch_prefill_tc5(int dtype, const void* q, uint32_t q_rows_total, uint32_t q_row0, uint32_t n_new, uint32_t start,
                       const void* kx, const void* vx, const void* latent, void* out, uint32_t H, uint32_t* status, cudaStream_t st)
{
    if (n_new == 0) return 0;
    const uint32_t total = start + n_new;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15u) return int(cudaErrorMisalignedAddress);
    (void)q_rows_total;
    alignas(64) CUtensorMap mk, mv, mr;
    if (!make_map(&mk, dtype, kx, total, uint64_t(H) * kNope, uint64_t(H) * kNope, KT) ||
        !make_map(&mv, dtype, vx, total, uint64_t(H) * kVDim, uint64_t(H) * kVDim, KT) ||
        !make_map(&mr, dtype, latent, total, kRow, kRow, KT))
        return -1;
    const ChunkArgs a{q_row0, n_new, start, H};
    const float scale_log2 = 1.4426950408889634f / sqrtf(float(kQDim));
    dim3 grid((n_new + QT - 1) / QT, H);
    if (dtype == 0)
        return int(launch_pdl(prefill_tc5_kernel<__half>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, static_cast<const __half*>(q),
                              mk, mv, mr, a, static_cast<__half*>(out), scale_log2, status));
    return int(launch_pdl(prefill_tc5_kernel<__nv_bfloat16>, grid, dim3(NUM_THREADS), SMEM_BYTES, st,
                          static_cast<const __nv_bfloat16*>(q), mk, mv, mr, a, static_cast<__nv_bfloat16*>(out), scale_log2, status));
}

}  // namespace mla
