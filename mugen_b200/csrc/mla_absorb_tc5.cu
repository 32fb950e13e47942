// q absorption (+ optionally the cache append of the same layer-step) on the 5th-generation tensor
// cores, sm_100a.
//
//   q_abs[r][h][d] = sum_{i<128} q[r][h][i] * W_UK[h*128+i][d],  d < 512;  q_abs[r][h][512..575] = q_rope
//   (reference: transformer.cpp:2563-2573; a query row gets the layout of a cache row)
//
// Absorb blocks: one per (head, group of 64 query rows).  W_UK_h^T ([512 d][128 i], contraction index
// contiguous, made once at registration) arrives by TMA as two K-major sub-tiles [512 d][64 i]
// (128 KB); the threads copy q_nope[64 rows][128] into swizzled operand rows; D[64 x 512] fills the
// 512 TMEM columns with 16 tcgen05.mma M=64 N=256 K=16; 16 warps drain TMEM into whole 256-byte
// row pieces of q_abs.
//
// Append blocks (present when the caller fuses the two steps): four new rows per block, the
// bit-exact RMSNorm + RoPE + scatter of append_kernel (mla_kernels.cu), 128 threads per row.  They
// share the launch because the append is a chain of dependent float additions that takes as long
// as the absorb itself and needs only a handful of SMs.
#include "mla_launch.h"
#include "mla_tc5.cuh"

namespace mla {

namespace {

using namespace tc5;

constexpr int MT = 64;                          // query rows per absorb block
constexpr int W_SUB = kRank * 128;              // 65,536: [512 d][64 i]
constexpr int W_BYTES = 2 * W_SUB;              // 131,072
constexpr int A_SUB = MT * 128;                 // 8,192: [64 rows][64 i]
constexpr int OFF_W = 0;
constexpr int OFF_A = OFF_W + W_BYTES;
constexpr int OFF_MISC = OFF_A + 2 * A_SUB;     // 147,456
constexpr int M_BAR = 0;                        // [0] W landed, [1] MMAs complete
constexpr int M_TMEM = 16;
constexpr int M_FAIL = 20;
constexpr int MISC_BYTES = 64;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;   // + slack to round the base up to 1 KB
constexpr int NUM_THREADS = 512;
constexpr int APPEND_ROWS = NUM_THREADS / 128;  // rows per append block
constexpr uint32_t TMEM_COLS = 512;


struct AppendArgs {          // rows == 0: no append blocks in this launch
    const void* kv_a;
    void* pool;              // this layer's slice of the cache pool
    uint64_t pool_slots;
    const void* norm_w;
    const float* cos_sin;
    uint32_t cs_rows;
    float eps;
    const uint32_t* row_pos;
    const uint64_t* row_slot;
    uint32_t rows;
    uint32_t wait_first;     // kv_a may be the output of the kernel just before this one in the stream
};

// One new cache row per 128 threads; every statement mirrors append_kernel (mla_kernels.cu), which
// documents the reference's rounding sequence.  All threads of the block reach every barrier.
template <typename T>
__device__ __forceinline__ void append_rows(const AppendArgs& a, uint32_t first_row, uint32_t* status)
{
    __shared__ __align__(16) T xin[APPEND_ROWS][kRow];
    __shared__ __align__(16) T xout[APPEND_ROWS][kRow];
    __shared__ float sq[APPEND_ROWS][kRank];
    __shared__ float rinv_s[APPEND_ROWS];
    const uint32_t g = threadIdx.x / 128, tid = threadIdx.x % 128, r = first_row + g;
    const T* kv_a = static_cast<const T*>(a.kv_a);
    const T* norm_w = static_cast<const T*>(a.norm_w);
    T* pool = static_cast<T*>(a.pool);
    bool live = r < a.rows;
    uint64_t slot = 0;
    uint32_t pos = 0;
    if (live) {
        slot = a.row_slot[r];
        pos = a.row_pos[r];
        if (slot == ~uint64_t(0)) live = false;          // a query-only row: nothing to append
        else if (slot >= a.pool_slots || pos >= a.cs_rows) {
            if (tid == 0) atomicOr(status, ST_BAD_SLOT);
            live = false;
        }
    }
    constexpr int kChunks = kRow * 2 / 16;   // 72 x 16 bytes
    // Every global load of the row is issued here, before the first barrier: the row itself, the rotation's cos/sin
    // and this thread's four norm weights.  Left where they are used they would form a chain of three dependent
    // round trips to memory (~1 us each) in a kernel whose whole budget is a few microseconds.
    uint4 row_chunk = make_uint4(0, 0, 0, 0);
    float cs = 0.0f, sn = 0.0f, nw[kRank / 128];
#pragma unroll
    for (int k = 0; k < kRank / 128; k++) nw[k] = 0.0f;
    if (live) {
        if (tid < kChunks) row_chunk = reinterpret_cast<const uint4*>(kv_a + size_t(r) * kRow)[tid];
        if (tid >= 32 && tid < 64) {
            cs = a.cos_sin[size_t(pos) * kRope + (tid - 32)];
            sn = a.cos_sin[size_t(pos) * kRope + 32 + (tid - 32)];
        }
#pragma unroll
        for (int k = 0; k < kRank / 128; k++) nw[k] = Elem<T>::to_f32(norm_w[tid + 128 * k]);
    }
    if (live && tid < kChunks) reinterpret_cast<uint4*>(xin[g])[tid] = row_chunk;
    __syncthreads();
    if (live) {
        for (int i = tid; i < kRank; i += 128) {
            const float v = Elem<T>::to_f32(xin[g][i]);
            sq[g][i] = __fmul_rn(v, v);
        }
        if (tid >= 32 && tid < 64) {
            const int i = tid - 32;
            const float x0 = Elem<T>::to_f32(xin[g][kRank + i]);
            const float x1 = Elem<T>::to_f32(xin[g][kRank + 32 + i]);
            xout[g][kRank + i]      = Elem<T>::from_f32(__fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)));
            xout[g][kRank + 32 + i] = Elem<T>::from_f32(__fadd_rn(__fmul_rn(x1, cs), __fmul_rn(x0, sn)));
        }
    }
    __syncthreads();
    if (live && tid == 0) {
        float ss = 0.0f;
#pragma unroll 16
        for (int i = 0; i < kRank; i++) ss = __fadd_rn(ss, sq[g][i]);
        rinv_s[g] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, float(kRank)), a.eps)));
    }
    __syncthreads();
    if (live) {
        const float rinv = rinv_s[g];
#pragma unroll
        for (int k = 0; k < kRank / 128; k++) {
            const int i = tid + 128 * k;
            const float v = __fmul_rn(Elem<T>::to_f32(xin[g][i]), rinv);
            xout[g][i] = Elem<T>::from_f32(__fmul_rn(v, nw[k]));
        }
    }
    __syncthreads();
    if (live && tid < kChunks)
        reinterpret_cast<uint4*>(pool + slot * kRow)[tid] = reinterpret_cast<const uint4*>(xout[g])[tid];
}

template <typename T>
__global__ void __launch_bounds__(NUM_THREADS, 1)
absorb_tc5_kernel(const __grid_constant__ CUtensorMap map_w, const T* __restrict__ q, T* __restrict__ q_abs, uint32_t rows,
                  uint32_t H, uint32_t absorb_blocks, const AppendArgs app, const float* __restrict__ q_cos_sin,
                  const uint32_t* __restrict__ q_pos, const uint32_t* __restrict__ att_row, uint32_t cs_rows,
                  uint32_t* __restrict__ status)
{
    grid_launch_dependents();
    if (blockIdx.x >= absorb_blocks) {
        // Apart from kv_a the append touches nothing that an earlier kernel of the stream still reads or writes:
        // constant tables, the step metadata (uploaded before the step's first kernel), and slots of this layer's
        // pool, last read by this layer's attention in the PREVIOUS step.  Where the host knows that kv_a was complete
        // before the kernel ahead of this one started (the later layers of a multi-layer call, whose kv_a the caller
        // handed over with the first layer's), the append works first and waits last; the wait then only keeps "this
        // kernel completes after its predecessors", which the kernels behind it rely on.
        if (app.wait_first) grid_dependency_wait();
        append_rows<T>(app, (blockIdx.x - absorb_blocks) * APPEND_ROWS, status);
        if (!app.wait_first) grid_dependency_wait();
        return;
    }
    extern __shared__ unsigned char absorb_tc5_smem[];
    const uint32_t raw = smem_u32(absorb_tc5_smem);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = absorb_tc5_smem + (base - raw);
    const uint32_t sW = base + OFF_W, sA = base + OFF_A;
    const uint32_t bar_w = base + OFF_MISC + M_BAR, bar_mma = bar_w + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC + M_TMEM);
    volatile int* fail_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + M_FAIL);
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t h = blockIdx.x % H, r0 = (blockIdx.x / H) * MT;

    if (tid == 0) {
        *fail_flag = 0;
        mbar_init(bar_w, 1);
        mbar_init(bar_mma, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        mbar_expect_tx(bar_w, W_BYTES);                      // W_UK_h^T: four boxes of 64 i x 256 d
#pragma unroll 1
        for (int bx = 0; bx < 4; bx++)
            tma_load_2d(sW + (bx / 2) * W_SUB + (bx % 2) * (W_SUB / 2), &map_w, bar_w, 64 * (bx / 2), int(h) * kRank + 256 * (bx % 2));
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    // the weights are constant; everything below reads or writes what earlier kernels of the stream touch
    grid_dependency_wait();
    // q_nope tile -> two swizzled K-major sub-tiles; q_rope -> behind the absorbed dims
    for (uint32_t c = tid; c < MT * 16; c += NUM_THREADS) {                 // 16 chunks of 16 bytes per row
        const uint32_t rr = c / 16, ch = c % 16, r = r0 + rr;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = reinterpret_cast<const uint4*>(q + (size_t(att_row ? att_row[r] : r) * H + h) * kQDim)[ch];
        *reinterpret_cast<uint4*>(sm + OFF_A + (ch / 8) * A_SUB + rr * 128 + (((ch % 8) ^ (rr & 7)) << 4)) = v;
    }
    if (q_cos_sin == nullptr) {
        for (uint32_t c = tid; c < MT * 8; c += NUM_THREADS) {              // rope part, already rotated: 8 chunks per row
            const uint32_t rr = c / 8, ch = c % 8, r = r0 + rr;
            if (r < rows)
                reinterpret_cast<uint4*>(q_abs + (size_t(r) * H + h) * kRow + kRank)[ch] =
                    reinterpret_cast<const uint4*>(q + (size_t(att_row ? att_row[r] : r) * H + h) * kQDim + kNope)[ch];
        }
    } else {
        // q-side RoPE (reference: transformer.cpp:3882-3921, NeoX pairs (i, i+32), YaRN frequencies): the same
        // table and the same separately rounded products as the k_rope rotation of the append
        for (uint32_t c = tid; c < MT * (kRope / 2); c += NUM_THREADS) {
            const uint32_t rr = c / (kRope / 2), i = c % (kRope / 2), r = r0 + rr;
            if (r >= rows) continue;
            const uint32_t pos = q_pos[r];
            if (pos >= cs_rows) {
                if (i == 0) atomicOr(status, ST_BAD_SLOT);
                continue;
            }
            const T* src = q + (size_t(att_row ? att_row[r] : r) * H + h) * kQDim + kNope;
            T* dst = q_abs + (size_t(r) * H + h) * kRow + kRank;
            const float cs = q_cos_sin[size_t(pos) * kRope + i], sn = q_cos_sin[size_t(pos) * kRope + 32 + i];
            const float x0 = Elem<T>::to_f32(src[i]), x1 = Elem<T>::to_f32(src[32 + i]);
            dst[i]      = Elem<T>::from_f32(__fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)));
            dst[32 + i] = Elem<T>::from_f32(__fadd_rn(__fmul_rn(x1, cs), __fmul_rn(x0, sn)));
        }
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    bool ok = true;
    if (warp == 0) {
        ok = mbar_wait(bar_w, 0, fail_flag, status);
        tc_fence_after();
        if (ok && elect_one()) {
            constexpr uint32_t IDESC = instr_desc(Fmt<T>::v, MT, 256);
#pragma unroll
            for (int half = 0; half < 2; half++) {
#pragma unroll
                for (int s = 0; s < 2; s++) {
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        tc_mma(tmem + half * 256, desc_lo(sA + s * A_SUB + k * 32), desc_hi(1024),
                               desc_lo(sW + s * W_SUB + half * (W_SUB / 2) + k * 32), desc_hi(1024), IDESC, (s == 0 && k == 0) ? 0u : 1u);
                }
            }
            tc_commit(bar_mma);
        }
        __syncwarp();
    }
    // D (M=64): rows 16*q .. 16*q+15 sit in lanes 0-15 of TMEM sub-partition q; warp w drains the
    // 128 columns 128*(w/4) .. of sub-partition w%4
    ok = mbar_wait(bar_mma, 0, fail_flag, status) && ok;
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
        tc_fence_after();
        const uint32_t qp = warp % 4, cg = warp / 4;
        const uint32_t row = r0 + 16 * qp + lane;
#pragma unroll 1
        for (int c = 0; c < 4; c++) {
            uint32_t o[32];
            tc_ld32(tmem + ((qp * 32u) << 16) + cg * 128 + c * 32, o);
            tc_wait_ld();
            if (lane < 16 && row < rows) {
                uint4* dst = reinterpret_cast<uint4*>(q_abs + (size_t(row) * H + h) * kRow + cg * 128 + c * 32);
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    uint32_t pk[4];
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        pk[i] = Elem<T>::pack2(__uint_as_float(o[8 * x + 2 * i]), __uint_as_float(o[8 * x + 2 * i + 1]));
                    dst[x] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

int absorb_tc5_configure()
{
    cudaError_t e = cudaFuncSetAttribute(absorb_tc5_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    e = cudaFuncSetAttribute(absorb_tc5_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    // every kernel of a layer-step asks for the same (maximal) shared-memory carve-out, so the SMs are not
    // re-partitioned between consecutive launches
    e = cudaFuncSetAttribute(absorb_tc5_kernel<__half>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return int(e);
    e = cudaFuncSetAttribute(absorb_tc5_kernel<__nv_bfloat16>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return int(e);
}

// w_map: host CUtensorMap over this layer's W_UK^T ([H*512 d][128 i], box 64 i x 256 d, 128-byte swizzle).
// With kv_a != nullptr the launch also appends the step's new rows to the layer's cache pool.  With rotate_q the
// last 64 dims of every query head are rotated with the row's position (m.row_pos) before they are stored.
int launch_absorb_tc5(int dtype, const void* q, const void* w_map, void* q_abs, uint32_t rows, uint32_t H, const void* kv_a,
                      void* layer_pool, uint64_t pool_slots, const void* norm_w, const float* cos_sin, uint32_t cs_rows,
                      float eps, const StepMeta& m, bool rotate_q, bool append_waits, uint32_t* status, cudaStream_t st)
{
    if (rows == 0) return 0;
    const CUtensorMap* map = static_cast<const CUtensorMap*>(w_map);
    AppendArgs app{};
    if (kv_a) app = AppendArgs{kv_a, layer_pool, pool_slots, norm_w, cos_sin, cs_rows, eps, m.app_pos, m.app_slot, m.app_rows, append_waits ? 1u : 0u};
    const uint32_t absorb_blocks = H * ((rows + MT - 1) / MT);
    const uint32_t append_blocks = (app.rows + APPEND_ROWS - 1) / APPEND_ROWS;
    // append blocks carry the trailing indices; for decode batches all blocks are resident at once (H + rows/4 <= SMs)
    dim3 grid(absorb_blocks + append_blocks);
    if (dtype == 0)
        return int(launch_pdl(absorb_tc5_kernel<__half>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, *map, static_cast<const __half*>(q),
                              static_cast<__half*>(q_abs), rows, H, absorb_blocks, app, rotate_q ? cos_sin : nullptr, m.row_pos, m.att_row, cs_rows, status));
    return int(launch_pdl(absorb_tc5_kernel<__nv_bfloat16>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, *map,
                          static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(q_abs), rows, H, absorb_blocks, app,
                          rotate_q ? cos_sin : nullptr, m.row_pos, m.att_row, cs_rows, status));
}

}  // namespace mla
