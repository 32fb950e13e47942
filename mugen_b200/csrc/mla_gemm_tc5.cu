// Dense projections around the attention op on the 5th-generation tensor cores, sm_100a:
//
//   C[M][N] = A[M][K] . W[N][K]^T        A = activations (row-major, K contiguous), W = a weight matrix exactly as the
//                                        reference keeps it for its matvec kernels (one output per row, K contiguous:
//                                        src/metal/kernel_sources.h:55-98), 16-bit operands, float accumulation in TMEM.
//
// Used for the steps of the reference's MLA decode driver that surround the attention (src/core/model/transformer.cpp:
// 3849-3929, 4002-4015): q_a / q_b (or full q), kv_a_mqa, Wo — M is the step's row count there, so the op streams the
// weight once and is HBM-bound — and for the expansion of latent rows into per-head keys and values in the chunked
// prefill path (M = tokens, K = 512).
//
// One block per 128 x 128 output tile and K slice: warp 0 = TMA producer (A and W tiles of 128 rows x 64 values, 128-byte
// swizzle, four or two stages), warp 1 = MMA issuer (tcgen05.mma M128 N128 K16, cta_group::1), warps 2-5 = epilogue (TMEM ->
// registers -> shared memory -> TMA tile store for storage-type output; TMEM -> registers -> global for float partials).  Rows and columns beyond M / N / K are zero-filled by TMA and never stored.  With split-K
// (few output tiles, long K: the decode-time projections) every slice writes float partial sums and a second kernel
// adds them and applies what follows the projection in the reference: rounding to the storage type, then optionally
// RMSNorm with a weight (q_a_norm) or the residual add.
#include <cuda.h>

#include <algorithm>

#include "mla_launch.h"
#include "mla_tc5.cuh"

namespace mla {

namespace {

using namespace tc5;

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int TILE_BYTES = BM * BK * 2;                  // 16,384 (A and W tiles alike)
// Two shapes of the same kernel.  Four stages, one block per SM: long K (the decode-time projections, split-K).  Two
// stages, three blocks per SM: short K and many output tiles (the prefill expansion, K = 512): a tile is then a chain
// load -> 32 MMAs -> epilogue of a few microseconds with nothing to overlap inside one block, and three blocks per SM take
// turns on the tensor pipe (12288 x 16384 x 512: 502 us with one block per SM).
constexpr int off_misc(int stages) { return stages * 2 * TILE_BYTES; }
constexpr int smem_bytes(int stages) { return off_misc(stages) + 128 + 1024; }      // barriers + slack for 1 KB alignment
constexpr int MAX_STAGES = 4;
constexpr int NUM_THREADS = 32 * 6;
constexpr uint32_t TMEM_COLS = 128;

// out_f32 != nullptr: float partials [z][M][N]; else storage-type output [M][N]
template <typename T, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, STAGES == 2 ? 3 : 1)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                const __grid_constant__ CUtensorMap map_c, uint32_t tile_store, T* __restrict__ out,
                float* __restrict__ out_f32, uint32_t M, uint32_t N, uint32_t K, uint32_t k_blocks_per_split,
                uint32_t* __restrict__ status)
{
    extern __shared__ unsigned char gemm_smem[];
    const uint32_t raw = smem_u32(gemm_smem);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char* sm = gemm_smem + (base - raw);
    constexpr int OFF_MISC = off_misc(STAGES);
    static_assert(STAGES <= MAX_STAGES, "barrier slots");
    const uint32_t bar0 = base + OFF_MISC;                       // full[STAGES], empty[STAGES], done
    auto full = [&](int s) { return bar0 + 8u * uint32_t(s); };
    auto empty = [&](int s) { return bar0 + 8u * uint32_t(STAGES + s); };
    const uint32_t done = bar0 + 8u * uint32_t(2 * STAGES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC + 96);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 100);
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const uint32_t kb_total = (K + BK - 1) / BK;
    const uint32_t kb_begin = blockIdx.z * k_blocks_per_split, kb_end = min(kb_total, kb_begin + k_blocks_per_split);

    grid_launch_dependents();
    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; s++) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        mbar_init(done, 1);
        mbar_init_fence();
    }
    if (warp == 1) tc_alloc<TMEM_COLS>(tmem_slot);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    grid_dependency_wait();              // the activations come from an earlier kernel of the stream

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            for (uint32_t kb = kb_begin, i = 0; kb < kb_end && ok; kb++, i++) {
                const int s = int(i % STAGES);
                ok = mbar_wait(empty(s), ((i / STAGES) & 1) ^ 1, abort_flag, status);
                if (!ok) break;
                mbar_expect_tx(full(s), 2 * TILE_BYTES);
                tma_load_2d(base + s * 2 * TILE_BYTES, &map_a, full(s), int(kb * BK), int(m0));
                tma_load_2d(base + s * 2 * TILE_BYTES + TILE_BYTES, &map_w, full(s), int(kb * BK), int(n0));
            }
        }
    } else if (warp == 1) {
        constexpr uint32_t IDESC = instr_desc(Fmt<T>::v, BM, BN);
        bool ok = true;
        for (uint32_t kb = kb_begin, i = 0; kb < kb_end && ok; kb++, i++) {
            const int s = int(i % STAGES);
            ok = mbar_wait(full(s), (i / STAGES) & 1, abort_flag, status);
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t a = desc_lo(base + s * 2 * TILE_BYTES), b = desc_lo(base + s * 2 * TILE_BYTES + TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; k++)
                    tc_mma(tmem, a + ((k * 32) >> 4), desc_hi(1024), b + ((k * 32) >> 4), desc_hi(1024), IDESC, (i == 0 && k == 0) ? 0u : 1u);
                tc_commit(empty(s));
                if (kb + 1 == kb_end) tc_commit(done);
            }
            __syncwarp();
        }
    } else {
        // epilogue: warp w reads TMEM lanes 32*(w%4) .. +31 = output rows m0 + that
        const uint32_t q4 = warp % 4, row = m0 + q4 * 32 + lane;
        bool ok = kb_end > kb_begin ? mbar_wait(done, 0, abort_flag, status) : true;
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                uint32_t v[32];
                if (kb_end > kb_begin) {
                    tc_ld32(tmem + ((q4 * 32u) << 16) + c * 32, v);
                    tc_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = 0u;              // an empty K slice contributes zeros
                }
                const uint32_t col = n0 + c * 32;
                if (tile_store) {
                    // The tile goes out through shared memory (the pipeline buffers are free: every MMA has completed) as two
                    // boxes of 64 columns x 128 rows in the 128-byte swizzle, and TMA writes whole rows of a box; a thread
                    // storing its own 64 bytes per row piece reaches a third of that rate on 400 MB of output.
                    const uint32_t r = q4 * 32 + lane;
                    unsigned char* box = sm + (c / 2) * TILE_BYTES + r * 128;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint32_t pk[4];
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            pk[j] = Elem<T>::pack2(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                        *reinterpret_cast<uint4*>(box + ((((c % 2) * 4 + i) ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                    continue;
                }
                if (row >= M || col >= N) continue;
                if (out_f32) {
                    float* dst = out_f32 + (size_t(blockIdx.z) * M + row) * N + col;
                    if (col + 32 <= N && (N % 4) == 0) {
#pragma unroll
                        for (int i = 0; i < 8; i++)
                            reinterpret_cast<float4*>(dst)[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                                            __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                    } else {
                        for (int i = 0; i < 32 && col + i < N; i++) dst[i] = __uint_as_float(v[i]);
                    }
                } else {
                    T* dst = out + size_t(row) * N + col;
                    if (col + 32 <= N && (N % 8) == 0) {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            uint32_t pk[4];
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                pk[j] = Elem<T>::pack2(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                            reinterpret_cast<uint4*>(dst)[i] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        }
                    } else {
                        for (int i = 0; i < 32 && col + i < N; i++) dst[i] = Elem<T>::from_f32(__uint_as_float(v[i]));
                    }
                }
            }
        }
        if (tile_store) {                        // outside the test of `ok`: the barrier is for all four epilogue warps
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            asm volatile("barrier.cta.sync 1, 128;\n" ::: "memory");
            if (warp == 2 && ok && *abort_flag == 0 && elect_one()) {
                tma_store_2d(&map_c, base, int(n0), int(m0));
                tma_store_2d(&map_c, base + TILE_BYTES, int(n0 + 64), int(m0));
                tma_store_commit_and_wait_read();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tc_dealloc<TMEM_COLS>(tmem);
    }
}

// Adds the K slices of one output row, rounds to the storage type (the reference's projections store half,
// src/metal/kernel_sources.h:93-95), then
//   mode 0: stores it
//   mode 1: RMSNorm over the row with weight w, as the reference's rms_norm kernel computes it from the ROUNDED
//           projection: y = T(float(x) * rsqrt(mean(x^2) + eps) * float(w))   (kernel_sources.h:264-312)
//   mode 2: residual add, y = T(float(res) + float(x))                         (elementwise_add, :357-366)
template <typename T>
__global__ void __launch_bounds__(256)
gemm_finalize_kernel(const float* __restrict__ partial, uint32_t splits, uint32_t M, uint32_t N, int mode,
                     const T* __restrict__ w, float eps, const T* __restrict__ res, T* __restrict__ out)
{
    __shared__ float red[8];
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    float ss = 0.0f;
    for (uint32_t c = tid; c < N; c += 256) {
        float acc = 0.0f;
        for (uint32_t z = 0; z < splits; z++) acc += partial[(size_t(z) * M + row) * N + c];
        const T x = Elem<T>::from_f32(acc);
        const float xf = Elem<T>::to_f32(x);
        if (mode == 1) ss += xf * xf;
        if (mode == 2) out[size_t(row) * N + c] = Elem<T>::from_f32(Elem<T>::to_f32(res[size_t(row) * N + c]) + xf);
        else out[size_t(row) * N + c] = x;                    // mode 1 rescales below
    }
    if (mode != 1) return;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (tid % 32 == 0) red[tid / 32] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    const float inv = rsqrtf(tot / float(N) + eps);
    for (uint32_t c = tid; c < N; c += 256) {
        const float xf = Elem<T>::to_f32(out[size_t(row) * N + c]);      // this thread's own earlier store
        out[size_t(row) * N + c] = Elem<T>::from_f32(xf * inv * Elem<T>::to_f32(w[c]));
    }
}

// y = T(float(x) * rsqrt(mean(x^2) + eps) * float(w)) per row (the reference's rms_norm kernel; step A of the driver)
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, uint32_t N, float eps)
{
    __shared__ float red[8];
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    float ss = 0.0f;
    for (uint32_t c = tid; c < N; c += 256) {
        const float v = Elem<T>::to_f32(x[size_t(row) * N + c]);
        ss += v * v;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (tid % 32 == 0) red[tid / 32] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    const float inv = rsqrtf(tot / float(N) + eps);
    for (uint32_t c = tid; c < N; c += 256)
        y[size_t(row) * N + c] = Elem<T>::from_f32(Elem<T>::to_f32(x[size_t(row) * N + c]) * inv * Elem<T>::to_f32(w[c]));
}

using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

TensorMapEncodeFn encoder()
{
    static TensorMapEncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<TensorMapEncodeFn>(p);
    }();
    return fn;
}

// rows x K matrix of 16-bit values, K contiguous, row pitch ld elements: box 64 values x 128 rows, 128-byte swizzle
bool make_map(CUtensorMap* map, int dtype, const void* ptr, uint64_t rows, uint64_t K, uint64_t ld)
{
    TensorMapEncodeFn enc = encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {BK, BM};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr),
               dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int gemm_tc5_configure()
{
    cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<__half, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(4));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc5_kernel<__nv_bfloat16, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(4));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc5_kernel<__half, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(2));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc5_kernel<__nv_bfloat16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(2));
    return int(e);
}

uint32_t gemm_tc5_splits(uint32_t M, uint32_t N, uint32_t K, uint32_t sm_count)
{
    const uint32_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN), kb = (K + BK - 1) / BK;
    if (tiles >= sm_count || kb <= 4) return 1;
    const uint32_t want = (sm_count + tiles - 1) / tiles;                 // enough blocks to occupy every SM once
    return std::max(1u, std::min(want, kb / 4));                          // at least four k-blocks per slice
}

// C = A . W^T.  A [M][K] (pitch lda), W [N][K] (pitch ldw), both DEVICE, 16-bit of `dtype`.  splits == 1 and
// partial == nullptr: C is written in the storage type to `out` [M][N]; otherwise float partials go to `partial`
// [splits][M][N] (finish with launch_gemm_finalize).  Returns a cudaError_t value, or -1 when the tensor map cannot
// be built (pointers must be 16-byte aligned, pitches multiples of 8 elements).
int launch_gemm_tc5(int dtype, const void* A, uint32_t lda, const void* W, uint32_t ldw, uint32_t M, uint32_t N, uint32_t K,
                    void* out, float* partial, uint32_t splits, uint32_t* status, cudaStream_t st)
{
    if (M == 0 || N == 0) return 0;
    alignas(64) CUtensorMap ma, mw, mc;
    if (!make_map(&ma, dtype, A, M, K, lda) || !make_map(&mw, dtype, W, N, K, ldw)) return -1;
    // storage-type output with rows that TMA can address: the epilogue stores tiles (see the kernel)
    const uint32_t tile_store = (!partial && out && N % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0 &&
                                 make_map(&mc, dtype, out, M, N, N)) ? 1u : 0u;
    if (!tile_store) mc = ma;
    const uint32_t kb = (K + BK - 1) / BK;
    splits = std::max(1u, std::min(splits, kb));
    const uint32_t per = (kb + splits - 1) / splits;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, splits);
    const bool many_short = per <= 8 && size_t(grid.x) * grid.y * grid.z >= 1024;      // see the note on the two shapes
    auto go = [&](auto kernel, int stages, auto* o) {
        return int(launch_pdl(kernel, grid, dim3(NUM_THREADS), size_t(smem_bytes(stages)), st, ma, mw, mc, tile_store, o, partial, M, N, K,
                              per, status));
    };
    if (dtype == 0)
        return many_short ? go(gemm_tc5_kernel<__half, 2>, 2, static_cast<__half*>(out))
                          : go(gemm_tc5_kernel<__half, 4>, 4, static_cast<__half*>(out));
    return many_short ? go(gemm_tc5_kernel<__nv_bfloat16, 2>, 2, static_cast<__nv_bfloat16*>(out))
                      : go(gemm_tc5_kernel<__nv_bfloat16, 4>, 4, static_cast<__nv_bfloat16*>(out));
}

// mode 0 store, 1 RMSNorm(w, eps), 2 residual add (res); see gemm_finalize_kernel
int launch_gemm_finalize(int dtype, const float* partial, uint32_t splits, uint32_t M, uint32_t N, int mode, const void* w,
                         float eps, const void* res, void* out, cudaStream_t st)
{
    if (M == 0 || N == 0) return 0;
    if (dtype == 0)
        return int(launch_pdl(gemm_finalize_kernel<__half>, dim3(M), dim3(256), 0, st, partial, splits, M, N, mode,
                              static_cast<const __half*>(w), eps, static_cast<const __half*>(res), static_cast<__half*>(out)));
    return int(launch_pdl(gemm_finalize_kernel<__nv_bfloat16>, dim3(M), dim3(256), 0, st, partial, splits, M, N, mode,
                          static_cast<const __nv_bfloat16*>(w), eps, static_cast<const __nv_bfloat16*>(res),
                          static_cast<__nv_bfloat16*>(out)));
}

int launch_rmsnorm_rows(int dtype, const void* x, const void* w, void* y, uint32_t rows, uint32_t N, float eps, cudaStream_t st)
{
    if (rows == 0) return 0;
    if (dtype == 0)
        return int(launch_pdl(rmsnorm_rows_kernel<__half>, dim3(rows), dim3(256), 0, st, static_cast<const __half*>(x),
                              static_cast<const __half*>(w), static_cast<__half*>(y), N, eps));
    return int(launch_pdl(rmsnorm_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x),
                          static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), N, eps));
}

}  // namespace mla
