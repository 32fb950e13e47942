// Merge of split-KV partial states + W_UV projection on the 5th-generation tensor cores, sm_100a.
//
//   o_c[row][512] = sum_p 2^(m_p - M) acc_p / sum_p 2^(m_p - M) l_p        (float, per head)
//   out[row][128] = o_c . W_UV_h^T
//
// One block per (head, group of 64 query rows).  W_UV_h (128 x 512, 128 KB) lands in shared memory
// by TMA as eight K-major sub-tiles [128 outputs][64 dims] with the 128-byte swizzle, while the
// threads reduce the partial states.  o_c is split into hi = T(o) and lo = T(o - hi) (together ~16
// mantissa bits for bf16, ~22 for fp16, so the float state is not rounded to the storage type
// before the projection) and written to shared memory in the same swizzled K-major layout; the
// projection is 2 x 32 tcgen05.mma M=64 N=128 K=16 (hi and lo against the same W sub-tiles) into
// 128 TMEM columns.  The 512 dims are processed in two halves so that the second half's reduction
// (global loads) overlaps the first half's MMAs and the operand buffers stay at 64 KB.  The
// reduction itself is one running-maximum sweep over a row's parts with whole-line warp accesses.
//
// The mma.sync version of this step (merge_outproj_mma_kernel) re-reads the operands from shared
// memory once per warp and spends ~40 us per layer at batch 64; here every operand byte is read
// once by the tensor core.
#include "mla_launch.h"
#include "mla_tc5.cuh"

namespace mla {

namespace {

using namespace tc5;

constexpr int MT = 64;                         // query rows per block
constexpr int W_SUB = kVDim * 128;             // 16,384: [128 outputs][64 dims]
constexpr int W_BYTES = (kRank / 64) * W_SUB;  // 131,072
constexpr int A_SUB = MT * 128;                // 8,192: [64 rows][64 dims]
constexpr int A_HALF = 4 * A_SUB;              // 32,768: 256 dims of hi (or lo)
constexpr int OFF_W = 0;
constexpr int OFF_AHI = OFF_W + W_BYTES;
constexpr int OFF_ALO = OFF_AHI + A_HALF;
constexpr int OFF_MISC = OFF_ALO + A_HALF;     // 196,608
constexpr int M_BAR = 0;                       // [0] W landed, [1] MMAs complete
constexpr int M_TMEM = 16;
constexpr int M_FAIL = 20;
constexpr int MISC_BYTES = 64;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;   // + slack to round the base up to 1 KB
constexpr int NUM_THREADS = 512;
constexpr uint32_t TMEM_COLS = 128;


template <typename T, bool kSmall>
__global__ void __launch_bounds__(NUM_THREADS, 1)
merge_outproj_tc5_kernel(const __grid_constant__ CUtensorMap map_w, const float* __restrict__ recs,
                         const uint32_t* __restrict__ row_seg_begin, uint32_t n_parts, T* __restrict__ out,
                         uint32_t rows, uint32_t H, const uint32_t* __restrict__ att_row, uint32_t* __restrict__ status)
{
    extern __shared__ unsigned char merge_tc5_smem[];
    const uint32_t raw = smem_u32(merge_tc5_smem);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = merge_tc5_smem + (base - raw);
    const uint32_t sW = base + OFF_W, sAhi = base + OFF_AHI, sAlo = base + OFF_ALO;
    const uint32_t bar_w = base + OFF_MISC + M_BAR, bar_mma = bar_w + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC + M_TMEM);
    volatile int* fail_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + M_FAIL);

    const uint32_t h = blockIdx.x, tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t r0 = blockIdx.y * (kSmall ? 16u : uint32_t(MT));    // small form: 16 rows per block, one per warp
    auto rec_of = [&](uint32_t r, uint32_t p) -> const float* {
        const size_t idx = row_seg_begin ? (size_t(p) * H + h) : ((size_t(p) * rows + r) * H + h);
        return recs + idx * kPart;
    };

    grid_launch_dependents();
    if (tid == 0) {
        *fail_flag = 0;
        mbar_init(bar_w, 1);
        mbar_init(bar_mma, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (tid == 0) {                                       // W_UV_h: eight boxes of 64 dims x 128 outputs
        mbar_expect_tx(bar_w, W_BYTES);
#pragma unroll 1
        for (int s = 0; s < kRank / 64; s++) tma_load_2d(sW + s * W_SUB, &map_w, bar_w, 64 * s, int(h) * kVDim);
    }

    // Reduction of the partial states, one warp per four rows (16 apart), two rows at a time.  A lane owns dims
    // 64*k + 2*lane (+1), k = 0..3, of the current half: a warp load covers 256 contiguous bytes of
    // a state record and a warp store one whole 128-byte operand row.  Parts are taken four at a
    // time with the usual running-maximum update, so the (m, l) pass and the accumulation are one
    // sweep and a row with up to four parts costs a single round trip to memory.
    constexpr uint32_t IDESC = instr_desc(Fmt<T>::v, MT, kVDim);
    bool ok = true;
    grid_dependency_wait();          // W_UV is constant and already on its way; the partial states are not
    // A warp's four rows are warp, warp+16, warp+32, warp+48 of the block's 64: with a small batch (8 sequences
    // per GPU when the batch is sharded over 8) every row then has a warp of its own instead of two warps
    // walking all of them; a row of such a batch is cut into ~10 parts, three round trips to memory each half.
    uint32_t pb4[4], pe4[4];                              // part ranges of this warp's four rows
#pragma unroll
    for (int x = 0; x < 4; x++) {
        const uint32_t rw = r0 + warp + 16 * x;
        pb4[x] = pe4[x] = 0;
        if (rw < rows) {
            if (row_seg_begin) { pb4[x] = row_seg_begin[rw]; pe4[x] = row_seg_begin[rw + 1]; }
            else               { pb4[x] = 0; pe4[x] = n_parts; }
        }
    }
    // Small batches (at most 16 rows in this block, e.g. 8 sequences per GPU): a warp has one row and sweeps its parts
    // ONCE for all 512 dims (a lane owns dims 64*k + 2*lane (+1), k = 0..7), so a row of ~10 parts costs three round
    // trips to memory instead of six; the two halves of the projection then only differ in which eight of the lane's
    // sixteen sums they write as operands.
    constexpr bool small = kSmall;                        // chosen at launch: few rows, or few heads (see the launcher)
    float acc_s[kSmall ? 16 : 1], inv_s = 0.0f;
    if constexpr (kSmall) {
        // With fewer than nine rows the idle warps share a row's parts: G warps per row sweep a slice each and one of
        // them folds the G partial sums afterwards (one sequence cut into 74 segments: 3 round trips to memory, not 19)
        // (only when a row has many parts: with ~10 parts per row, 8 sequences per GPU, the exchange costs more than the
        // shorter sweep saves: 56.5 against 55.9 us per layer-step)
        const uint32_t nrows = min(rows - r0, 16u);
        uint32_t max_parts = n_parts;
        if (row_seg_begin) {
            max_parts = 0;
            for (uint32_t i = 0; i < nrows; i++) max_parts = max(max_parts, row_seg_begin[r0 + i + 1] - row_seg_begin[r0 + i]);
        }
        uint32_t G = 1;
        while (2 * G * nrows <= 16u && max_parts >= 12u * G) G *= 2;     // at least six parts per warp
        const uint32_t myrow = warp / G, g = warp % G, rw = r0 + myrow;
        uint32_t pb = 0, pe = 0;
        if (myrow < nrows) {
            if (row_seg_begin) { pb = row_seg_begin[rw]; pe = row_seg_begin[rw + 1]; }
            else               { pe = n_parts; }
            const uint32_t chunk = (pe - pb + G - 1) / G;
            pb = min(pe, pb + g * chunk);
            pe = min(pe, pb + chunk);
        }
        float M = -INFINITY, L = 0.0f;
#pragma unroll
        for (int k = 0; k < 16; k++) acc_s[k] = 0.0f;
        for (uint32_t p = pb; p < pe; p += 4) {
            float2 ml[4], v[4][8];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const bool on = p + i < pe;
                const float* rc = rec_of(rw, on ? p + i : pb);
                ml[i] = on ? *reinterpret_cast<const float2*>(rc) : make_float2(-INFINITY, 0.0f);
#pragma unroll
                for (int k = 0; k < 8; k++)
                    v[i][k] = on ? *reinterpret_cast<const float2*>(rc + 2 + 64 * k + 2 * lane) : make_float2(0.0f, 0.0f);
            }
            const float Mn = fmaxf(fmaxf(M, ml[0].x), fmaxf(fmaxf(ml[1].x, ml[2].x), ml[3].x));
            if (Mn > -INFINITY) {
                const float sc = exp2f(M - Mn);
                L *= sc;
#pragma unroll
                for (int k = 0; k < 16; k++) acc_s[k] *= sc;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float w = exp2f(ml[i].x - Mn);
                    L = fmaf(w, ml[i].y, L);
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        acc_s[2 * k] = fmaf(w, v[i][k].x, acc_s[2 * k]);
                        acc_s[2 * k + 1] = fmaf(w, v[i][k].y, acc_s[2 * k + 1]);
                    }
                }
                M = Mn;
            }
        }
        if (G > 1) {        // block-uniform.  The operand buffers are free until the sums are written there below.
            float* scratch = reinterpret_cast<float*>(sm + OFF_AHI);
            float* mine = scratch + (size_t(warp) * 32 + lane) * 18;
            mine[0] = M;
            mine[1] = L;
#pragma unroll
            for (int k = 0; k < 16; k++) mine[2 + k] = acc_s[k];
            __syncthreads();
            M = -INFINITY;
            L = 0.0f;
#pragma unroll
            for (int k = 0; k < 16; k++) acc_s[k] = 0.0f;
            if (warp < nrows) {                          // from here on warp w stands for row w, as the operand writes expect
                for (uint32_t j = 0; j < G; j++) {
                    const float* o = scratch + (size_t(warp * G + j) * 32 + lane) * 18;
                    const float Mj = o[0];
                    if (Mj == -INFINITY) continue;       // warp-uniform: a slice without parts
                    const float Mn = fmaxf(M, Mj), sc = exp2f(M - Mn), w = exp2f(Mj - Mn);
                    L = fmaf(w, o[1], L * sc);
#pragma unroll
                    for (int k = 0; k < 16; k++) acc_s[k] = fmaf(w, o[2 + k], acc_s[k] * sc);
                    M = Mn;
                }
            }
            __syncthreads();
        }
        inv_s = L > 0.0f ? 1.0f / L : 0.0f;
    }
#pragma unroll 1
    for (int kh = 0; kh < 2; kh++) {
        if constexpr (kSmall) {
            // the first half's MMAs read the operand buffers until they complete
            if (kh == 1) ok = mbar_wait(bar_mma, 0, fail_flag, status);
            const uint32_t rr = warp;
            const uint32_t off = rr * 128 + (((lane / 4) ^ (rr & 7)) << 4) + (lane % 4) * 4;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float o0 = (kh == 0 ? acc_s[2 * k] : acc_s[8 + 2 * k]) * inv_s;
                const float o1 = (kh == 0 ? acc_s[2 * k + 1] : acc_s[8 + 2 * k + 1]) * inv_s;
                const T h0 = Elem<T>::from_f32(o0), h1 = Elem<T>::from_f32(o1);
                *reinterpret_cast<uint32_t*>(sm + OFF_AHI + k * A_SUB + off) = Elem<T>::pack2(o0, o1);
                *reinterpret_cast<uint32_t*>(sm + OFF_ALO + k * A_SUB + off) =
                    Elem<T>::pack2(o0 - Elem<T>::to_f32(h0), o1 - Elem<T>::to_f32(h1));
            }
        }
#pragma unroll 1
        for (int pr = 0; pr < 2 && !small; pr++) {
            uint32_t p[2], pe[2], rw[2];
            float M[2], L[2], acc[2][8];
#pragma unroll
            for (int x = 0; x < 2; x++) {
                rw[x] = r0 + warp + 16 * (2 * pr + x);
                p[x] = pr == 0 ? pb4[x] : pb4[2 + x];
                pe[x] = pr == 0 ? pe4[x] : pe4[2 + x];
                M[x] = -INFINITY;
                L[x] = 0.0f;
#pragma unroll
                for (int k = 0; k < 8; k++) acc[x][k] = 0.0f;
            }
            while (p[0] < pe[0] || p[1] < pe[1]) {
                float2 ml[2][4], v[2][4][4];
#pragma unroll
                for (int x = 0; x < 2; x++) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const bool on = p[x] + i < pe[x];
                        const float* rc = rec_of(rw[x], on ? p[x] + i : 0);
                        ml[x][i] = on ? *reinterpret_cast<const float2*>(rc) : make_float2(-INFINITY, 0.0f);
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            v[x][i][k] = on ? *reinterpret_cast<const float2*>(rc + 2 + kh * 256 + 64 * k + 2 * lane)
                                            : make_float2(0.0f, 0.0f);
                        // pull the record's second half towards L2 while the first is reduced
                        if (kh == 0 && on && lane < 8)
                            asm volatile("prefetch.global.L2 [%0];\n" ::"l"(rc + 2 + 256 + 32 * lane));
                    }
                }
#pragma unroll
                for (int x = 0; x < 2; x++) {
                    const float Mn = fmaxf(fmaxf(M[x], ml[x][0].x), fmaxf(fmaxf(ml[x][1].x, ml[x][2].x), ml[x][3].x));
                    if (Mn > -INFINITY) {
                        const float s = exp2f(M[x] - Mn);
                        L[x] *= s;
#pragma unroll
                        for (int k = 0; k < 8; k++) acc[x][k] *= s;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const float w = exp2f(ml[x][i].x - Mn);
                            L[x] = fmaf(w, ml[x][i].y, L[x]);
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                acc[x][2 * k] = fmaf(w, v[x][i][k].x, acc[x][2 * k]);
                                acc[x][2 * k + 1] = fmaf(w, v[x][i][k].y, acc[x][2 * k + 1]);
                            }
                        }
                        M[x] = Mn;
                    }
                    p[x] += 4;
                }
            }
            // the first half's MMAs read the operand buffers until they complete
            if (kh == 1 && pr == 0) ok = mbar_wait(bar_mma, 0, fail_flag, status);
#pragma unroll
            for (int x = 0; x < 2; x++) {
                const float inv = L[x] > 0.0f ? 1.0f / L[x] : 0.0f;
                const uint32_t rr = warp + 16 * (2 * pr + x);
                const uint32_t off = rr * 128 + (((lane / 4) ^ (rr & 7)) << 4) + (lane % 4) * 4;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float o0 = acc[x][2 * k] * inv, o1 = acc[x][2 * k + 1] * inv;
                    const T h0 = Elem<T>::from_f32(o0), h1 = Elem<T>::from_f32(o1);
                    *reinterpret_cast<uint32_t*>(sm + OFF_AHI + k * A_SUB + off) = Elem<T>::pack2(o0, o1);
                    *reinterpret_cast<uint32_t*>(sm + OFF_ALO + k * A_SUB + off) =
                        Elem<T>::pack2(o0 - Elem<T>::to_f32(h0), o1 - Elem<T>::to_f32(h1));
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        tc_fence_before();
        __syncthreads();
        if (warp == 0) {
            if (kh == 0) ok = mbar_wait(bar_w, 0, fail_flag, status) && ok;
            tc_fence_after();
            if (ok && elect_one()) {
#pragma unroll
                for (int s = 0; s < 4; s++) {
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const uint32_t b = desc_lo(sW + (kh * 4 + s) * W_SUB + k * 32);
                        tc_mma(tmem, desc_lo(sAhi + s * A_SUB + k * 32), desc_hi(1024), b, desc_hi(1024), IDESC,
                               (kh == 0 && s == 0 && k == 0) ? 0u : 1u);
                        tc_mma(tmem, desc_lo(sAlo + s * A_SUB + k * 32), desc_hi(1024), b, desc_hi(1024), IDESC, 1u);
                    }
                }
                tc_commit(bar_mma);
            }
            __syncwarp();
        }
    }

    if (warp < 4) {
        // D (M=64): rows 16*warp .. 16*warp+15 sit in lanes 0-15 of the warp's TMEM sub-partition
        ok = mbar_wait(bar_mma, 1, fail_flag, status) && ok;
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            const uint32_t row = r0 + 16 * warp + lane;
            const uint32_t row_end = kSmall ? min(rows, r0 + 16u) : rows;       // small form: rows 16.. of the tile are not this block's
#pragma unroll 1
            for (int c = 0; c < kVDim / 32; c++) {
                uint32_t o[32];
                tc_ld32(tmem + ((warp * 32u) << 16) + c * 32, o);
                tc_wait_ld();
                if (lane < 16 && row < row_end) {
                    uint4* dst = reinterpret_cast<uint4*>(out + (size_t(att_row ? att_row[row] : row) * H + h) * kVDim + c * 32);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint32_t pk[4];
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            pk[i] = Elem<T>::pack2(__uint_as_float(o[8 * q + 2 * i]), __uint_as_float(o[8 * q + 2 * i + 1]));
                        dst[q] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
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

template <typename K>
static cudaError_t configure_one(K kernel)
{
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    // every kernel of a layer-step asks for the same (maximal) shared-memory carve-out, so the SMs are not
    // re-partitioned between consecutive launches
    return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

int merge_tc5_configure()
{
    cudaError_t e = configure_one(merge_outproj_tc5_kernel<__half, false>);
    if (e == cudaSuccess) e = configure_one(merge_outproj_tc5_kernel<__half, true>);
    if (e == cudaSuccess) e = configure_one(merge_outproj_tc5_kernel<__nv_bfloat16, false>);
    if (e == cudaSuccess) e = configure_one(merge_outproj_tc5_kernel<__nv_bfloat16, true>);
    return int(e);
}

// w_map: host CUtensorMap over this layer's W_UV ([H*128 outputs][512 dims], box 64 dims x 128 outputs, 128-byte swizzle)
int launch_merge_tc5(int dtype, const float* recs, const uint32_t* row_seg_begin, uint32_t n_parts, const void* w_map,
                     void* out, uint32_t rows, uint32_t H, const uint32_t* att_row, uint32_t* status, cudaStream_t st)
{
    if (rows == 0) return 0;
    const CUtensorMap* map = static_cast<const CUtensorMap*>(w_map);
    // The small form (16 rows per block, a warp per row, one sweep over a row's parts for all 512 dims) serves steps of at
    // most 16 rows and head counts so small that tiles of 64 rows would leave most SMs idle (16 heads x 32 rows: 16 blocks
    // of 64 rows against 32 of 16), as long as its blocks still fit one wave.
    const bool small = rows <= 16 || H * ((rows + 15) / 16) <= 128;
    dim3 grid(H, small ? (rows + 15) / 16 : (rows + MT - 1) / MT);
    auto go = [&](auto kernel, auto* o) {
        return int(launch_pdl(kernel, grid, dim3(NUM_THREADS), SMEM_BYTES, st, *map, recs, row_seg_begin, n_parts, o, rows, H, att_row, status));
    };
    if (dtype == 0)
        return small ? go(merge_outproj_tc5_kernel<__half, true>, static_cast<__half*>(out))
                     : go(merge_outproj_tc5_kernel<__half, false>, static_cast<__half*>(out));
    return small ? go(merge_outproj_tc5_kernel<__nv_bfloat16, true>, static_cast<__nv_bfloat16*>(out))
                 : go(merge_outproj_tc5_kernel<__nv_bfloat16, false>, static_cast<__nv_bfloat16*>(out));
}

}  // namespace mla
