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
// One block per (tile of 128 query tokens, head):
//   TMA      Q tile [128][192] once; per 64-token step K [64][192] (two boxes of expanded nope dims + one box of rope dims
//            straight from the gathered latent rows) in a ring of three, V [64][128] in a ring of four: a K buffer is free as
//            soon as the score MMAs that read it complete, a V buffer one softmax later
//   QK       S[128 queries x 64 keys] = Q . K^T          12 x tcgen05.mma M128 N64 K16, scores double-buffered in TMEM
//   softmax  two threads per query row, 32 keys each (the two halves of a row exchange their maxima through shared
//            memory): causal mask, log2-domain online softmax with lazy rescaling (threshold 2^8), P to shared memory in
//            the storage type.  Two softmax warps per scheduler hide each other's dependent-issue latency.
//   PV       O^T[128 value dims x 128 queries] += V^T . P^T   4 x tcgen05.mma M128 N128 K16 with the V tile read MN-major
//            (the staged [64 keys][64 dims] sub-tiles serve as they are, no transpose), B = P (K-major)
//   epilogue O^T / l -> out[query][head][128], rounded once to the storage type
// Warps: 0 TMA producer, 1 MMA issuer, 2-9 softmax / correction / epilogue.  All waits are bounded.
#include <cuda.h>

#include <algorithm>

#include "mla_launch.h"
#include "mla_tc5.cuh"

namespace mla {

namespace {

using namespace tc5;

constexpr int QT = 128, KT = 64;
constexpr int Q_SUB = QT * 128;                        // 16,384: [128 queries][64 dims]
constexpr int K_SUB = KT * 128;                        // 8,192:  [64 keys][64 dims]
constexpr int Q_BYTES = 3 * Q_SUB;                     // 49,152
constexpr int K_STAGE = 3 * K_SUB, V_STAGE = 2 * K_SUB;        // K: 192 dims, V: 128 dims of 64 keys
constexpr int K_STAGES = 3, V_STAGES = 4;
constexpr int P_BYTES = QT * 128;                      // 16,384: [128 queries][64 keys]
constexpr int OFF_Q = 0, OFF_K = OFF_Q + Q_BYTES, OFF_V = OFF_K + K_STAGES * K_STAGE, OFF_P = OFF_V + V_STAGES * V_STAGE,
              OFF_MISC = OFF_P + P_BYTES;
// alpha: [2][128] by step parity; hmax / lsum: [2 halves][128 rows]
constexpr int M_ALPHA = 256, M_HMAX = M_ALPHA + 1024, M_LSUM = M_HMAX + 1024, M_LINV = M_LSUM + 1024, M_TMEM = M_LINV + 512,
              M_ABORT = M_TMEM + 4, MISC_BYTES = M_TMEM + 64;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;       // + slack for 1 KB alignment
constexpr int NUM_SOFTMAX = 256;
constexpr int NUM_THREADS = 64 + NUM_SOFTMAX;
constexpr uint32_t TMEM_COLS = 256, COL_S = 0, COL_O = 128;
constexpr float RESCALE_THRESHOLD = 8.0f;
enum { B_QFULL = 0, B_KFULL, B_KEMPTY = B_KFULL + K_STAGES, B_VFULL = B_KEMPTY + K_STAGES, B_VEMPTY = B_VFULL + V_STAGES,
       B_SFULL = B_VEMPTY + V_STAGES, B_SEMPTY = B_SFULL + 2, B_PFULL = B_SEMPTY + 2, B_PEMPTY, B_OFULL, B_COUNT };
static_assert(B_COUNT * 8 <= M_ALPHA && B_COUNT <= 32, "barriers overflow their area");
static_assert(SMEM_BYTES <= 232448, "over the shared memory of one block");

struct ChunkArgs {
    uint32_t q_row0;        // first query row of the chunk in the q / out tensors
    uint32_t n_new;         // query tokens in the chunk
    uint32_t start;         // cache rows of the sequence before the chunk
    uint32_t H;
};

template <typename T>
__global__ void __launch_bounds__(NUM_THREADS, 1)
prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_r, ChunkArgs a,
                   T* __restrict__ out, float scale_log2, uint32_t* __restrict__ status)
{
    extern __shared__ unsigned char prefill_smem[];
    const uint32_t raw = smem_u32(prefill_smem);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = prefill_smem + (base - raw);
    const uint32_t sQ = base + OFF_Q, sK = base + OFF_K, sV = base + OFF_V, sP = base + OFF_P, sBar = base + OFF_MISC;
    auto bar = [&](int i) { return sBar + 8u * uint32_t(i); };
    float* alpha_s = reinterpret_cast<float*>(sm + OFF_MISC + M_ALPHA);
    float* hmax_s = reinterpret_cast<float*>(sm + OFF_MISC + M_HMAX);
    float* lsum_s = reinterpret_cast<float*>(sm + OFF_MISC + M_LSUM);
    float* linv_s = reinterpret_cast<float*>(sm + OFF_MISC + M_LINV);
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
        const uint32_t count = (i >= B_SEMPTY && i < B_PFULL) || i == B_PFULL ? uint32_t(NUM_SOFTMAX) : 1u;
        mbar_init(bar(i), count);
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
            mbar_expect_tx(bar(B_QFULL), Q_BYTES);
#pragma unroll
            for (int c = 0; c < 3; c++)
                tma_load_2d(sQ + c * Q_SUB, &map_q, bar(B_QFULL), int(h * kQDim + 64 * c), int(a.q_row0 + q0));
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
        constexpr uint32_t IDESC_QK = instr_desc(Fmt<T>::v, QT, KT, 0, 0);
        constexpr uint32_t IDESC_PV = instr_desc(Fmt<T>::v, kVDim, QT, 1, 0);
        constexpr uint32_t HI = desc_hi(1024);
        bool ok = mbar_wait(bar(B_QFULL), 0, abort_flag, status);
        auto issue_pv = [&](uint32_t t) {           // O^T += V(t)^T . P(t)^T
            const int vs = int(t % V_STAGES);
            ok = mbar_wait(bar(B_VFULL + vs), (t / V_STAGES) & 1, abort_flag, status) &&
                 mbar_wait(bar(B_PFULL), t & 1, abort_flag, status);
            if (!ok) return;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t pa = desc_lo(sV + vs * V_STAGE, K_SUB), pb = desc_lo(sP);
#pragma unroll
                for (int k = 0; k < KT / 16; k++)
                    tc_mma(tmem + COL_O, pa + ((k * 2048) >> 4), HI, pb + ((k * 32) >> 4), HI, IDESC_PV, (t == 0 && k == 0) ? 0u : 1u);
                tc_commit(bar(B_VEMPTY + vs));
                tc_commit(bar(B_PEMPTY));
                if (t + 1 == n_kv) tc_commit(bar(B_OFULL));
            }
            __syncwarp();
        };
        for (uint32_t t = 0; t < n_kv && ok; t++) {
            const int ks = int(t % K_STAGES), b = int(t & 1);
            ok = mbar_wait(bar(B_KFULL + ks), (t / K_STAGES) & 1, abort_flag, status) &&
                 mbar_wait(bar(B_SEMPTY + b), ((t >> 1) & 1) ^ 1, abort_flag, status);
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t qa = desc_lo(sQ), kb = desc_lo(sK + ks * K_STAGE);
#pragma unroll
                for (int c = 0; c < 3; c++)
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        tc_mma(tmem + COL_S + b * KT, qa + ((c * Q_SUB + k * 32) >> 4), HI, kb + ((c * K_SUB + k * 32) >> 4), HI,
                               IDESC_QK, (c == 0 && k == 0) ? 0u : 1u);
                tc_commit(bar(B_SFULL + b));
                tc_commit(bar(B_KEMPTY + ks));
            }
            __syncwarp();
            if (t > 0) issue_pv(t - 1);
        }
        if (ok && n_kv > 0) issue_pv(n_kv - 1);
    } else {
        // ===== softmax / correction / epilogue: two threads per query row (32 keys each); for O^T: thread = value dim =====
        const uint32_t q4 = warp % 4, half = (warp - 2) / 4, r = q4 * 32 + lane;   // r: TMEM lane of this thread
        const uint32_t lane_base = (q4 * 32u) << 16;
        const uint32_t my_pos = a.start + q0 + r;                        // last key this query may see
        float m_run = -INFINITY, l_run = 0.0f;                           // l_run: this half's share of the row sum
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
        bool stop = false;
        for (uint32_t t = 0; t < n_kv; t++) {
            const uint32_t b = t & 1;
            wait_w(bar(B_SFULL + b), (t >> 1) & 1);
            uint32_t sv[32];
            if (!fail) {
                tc_fence_after();
                tc_ld32(tmem + lane_base + COL_S + b * KT + half * 32, sv);
                tc_wait_ld();
                tc_fence_before();
                mbar_arrive(bar(B_SEMPTY + b));
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) sv[i] = 0u;
            }
            const uint32_t k0 = t * KT + half * 32;
            if (k0 + 32 > my_pos + 1 || k0 + 32 > total) {               // causal / end mask (only near the diagonal)
#pragma unroll
                for (int i = 0; i < 32; i++)
                    if (k0 + uint32_t(i) > my_pos || k0 + uint32_t(i) >= total) sv[i] = __float_as_uint(-INFINITY);
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 32; i++) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            hmax_s[half * QT + r] = mx;
            group_sync();                                                // the next write of hmax_s comes after group_or below
            mx = fmaxf(mx, hmax_s[(half ^ 1u) * QT + r]) * scale_log2;   // both halves of a row now hold the same maximum
            float alpha = 1.0f;
            bool need = false;
            if (m_run == -INFINITY) { m_run = mx; }                     // nothing accumulated for this row yet
            else if (mx > m_run + RESCALE_THRESHOLD) { alpha = fast_ex2(m_run - mx); m_run = mx; need = true; }
            float* alpha_t = alpha_s + (t & 1) * QT;     // by step parity: a fast thread may be one step ahead of a slow one
            if (half == 0) alpha_t[r] = alpha;
            float sum2[2] = {0.0f, 0.0f};
            uint32_t pk[16];
            const float mref = m_run == -INFINITY ? 0.0f : m_run;         // a row whose keys so far are all masked: p = 0
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float p0 = fast_ex2(fmaf(__uint_as_float(sv[i]), scale_log2, -mref));
                const float p1 = fast_ex2(fmaf(__uint_as_float(sv[i + 1]), scale_log2, -mref));
                sum2[(i >> 1) & 1] += p0 + p1;
                pk[i / 2] = Elem<T>::pack2(p0, p1);
            }
            l_run = l_run * alpha + (sum2[0] + sum2[1]);
            const bool any_need = group_or(need || fail);
            if (any_need && group_or(fail)) { stop = true; break; }
            wait_w(bar(B_PEMPTY), (t - 1) & 1);          // PV of the previous step complete: O^T stable, P free
            if (fail) continue;
            tc_fence_after();
            if (any_need && t > 0) {
                // O^T[value dim = this thread's lane][query column] *= alpha[query]; each half takes two of the four chunks
#pragma unroll 1
                for (uint32_t c = 2 * half; c < 2 * half + 2; c++) {
                    uint32_t o[32];
                    tc_ld32(tmem + lane_base + COL_O + c * 32, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha_t[c * 32 + i]);
                    tc_st32(tmem + lane_base + COL_O + c * 32, o);
                }
                tc_wait_st();
            }
            {   // row r of the K-major swizzled P tile [128 queries][64 keys]: this half's 4 of the 8 chunks of 16 bytes
                unsigned char* prow = sm + OFF_P + r * 128;
#pragma unroll
                for (int j = 0; j < 4; j++)
                    *reinterpret_cast<uint4*>(prow + (((half * 4 + j) ^ (r & 7)) << 4)) =
                        make_uint4(pk[j * 4], pk[j * 4 + 1], pk[j * 4 + 2], pk[j * 4 + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            tc_fence_before();
            mbar_arrive(bar(B_PFULL));
        }
        if (!stop) {
            wait_w(bar(B_OFULL), 0);
            lsum_s[half * QT + r] = l_run;
            const bool bad = group_or(fail);
            if (half == 0) {
                const float l = lsum_s[r] + lsum_s[QT + r];
                linv_s[r] = l > 0.0f ? 1.0f / l : 0.0f;
            }
            group_sync();
            if (!bad) {
                tc_fence_after();
                // this thread holds value dim r of every query column: out[query][h][r] = O^T[r][query] / l[query]
#pragma unroll 1
                for (uint32_t c = 2 * half; c < 2 * half + 2; c++) {
                    uint32_t o[32];
                    tc_ld32(tmem + lane_base + COL_O + c * 32, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const uint32_t qi = q0 + c * 32 + i;
                        if (qi < a.n_new)
                            out[(size_t(a.q_row0 + qi) * a.H + h) * kVDim + r] = Elem<T>::from_f32(__uint_as_float(o[i]) * linv_s[c * 32 + i]);
                    }
                }
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
    alignas(64) CUtensorMap mq, mk, mv, mr;
    if (!make_map(&mq, dtype, q, q_rows_total, uint64_t(H) * kQDim, uint64_t(H) * kQDim, QT) ||
        !make_map(&mk, dtype, kx, total, uint64_t(H) * kNope, uint64_t(H) * kNope, KT) ||
        !make_map(&mv, dtype, vx, total, uint64_t(H) * kVDim, uint64_t(H) * kVDim, KT) ||
        !make_map(&mr, dtype, latent, total, kRow, kRow, KT))
        return -1;
    const ChunkArgs a{q_row0, n_new, start, H};
    const float scale_log2 = 1.4426950408889634f / sqrtf(float(kQDim));
    dim3 grid((n_new + QT - 1) / QT, H);
    if (dtype == 0)
        return int(launch_pdl(prefill_tc5_kernel<__half>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, mq, mk, mv, mr, a,
                              static_cast<__half*>(out), scale_log2, status));
    return int(launch_pdl(prefill_tc5_kernel<__nv_bfloat16>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, mq, mk, mv, mr, a,
                          static_cast<__nv_bfloat16*>(out), scale_log2, status));
}

}  // namespace mla
