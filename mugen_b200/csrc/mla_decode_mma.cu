// Split-KV absorbed MLA attention on the legacy tensor path (mma.sync.m16n8k16), sm_100a.
//
// One block = one KV segment (a run of pages of one query row) x one group of 16 heads.
// It is the general-shape kernel: any head count (groups are zero-padded), fp16 or bf16, any
// segment length; the tcgen05 kernel takes over for the wide-head shapes it is built for.
//
// Per 32-token tile (half a page, 36 KB, one contiguous run in HBM, staged by cp.async):
//   scores   S[16 x 32]  = Q'[16 x 576] . K^T        the 576-long contraction is split over the 4
//                                                     warps (9 k-steps each, Q' fragments stay in
//                                                     registers), partial sums meet in shared memory
//   softmax  online, log2 domain, one running (m, l) per head
//   PV       O[16 x 512] += P[16 x 32] . V[32 x 512]  warp w owns latent columns [128w, 128w+128)
// Every cache element is read from shared memory exactly once per use (no operand
// amplification), and from HBM exactly once per head group.
// Output: un-normalised partial state per (segment, head): m, l, acc[512] (514 floats).
#include "mla_launch.h"

namespace mla {

namespace {

constexpr int TT = 32;                 // tokens per tile
constexpr int KV_PITCH = kRow + 8;     // elements; 1168 B rows keep ldmatrix conflict-free
constexpr int NS = 2;                  // cp.async stages
constexpr int SP_PITCH = TT + 4;       // floats
constexpr int PS_PITCH = TT + 8;       // elements
constexpr int KS_PER_WARP = 9;         // 36 k-steps of 16 over 4 warps

constexpr size_t SMEM_KV = size_t(NS) * TT * KV_PITCH * 2;
constexpr size_t SMEM_SP = size_t(4) * 16 * SP_PITCH * 4;
constexpr size_t SMEM_PS = size_t(16) * PS_PITCH * 2;
constexpr size_t SMEM_TOTAL = SMEM_KV + SMEM_SP + SMEM_PS + 16 * 4;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// copies 16 bytes, or writes 16 zero bytes without touching `src` when `live` is false
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool live) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(live ? 16u : 0u));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__global__ void __launch_bounds__(128, 2)
decode_mma_kernel(const T* __restrict__ q_abs, const T* __restrict__ pool, uint32_t n_pages,
                  StepMeta m, float* __restrict__ recs, uint32_t H, float scale_log2,
                  uint32_t* __restrict__ status)
{
    extern __shared__ __align__(16) unsigned char smem[];
    T* kv = reinterpret_cast<T*>(smem);
    float* Sp = reinterpret_cast<float*>(smem + SMEM_KV);
    T* Ps = reinterpret_cast<T*>(smem + SMEM_KV + SMEM_SP);
    float* alpha_s = reinterpret_cast<float*>(smem + SMEM_KV + SMEM_SP + SMEM_PS);

    const uint32_t seg = blockIdx.x, h0 = blockIdx.y * 16;
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t g = lane / 4, t4 = lane % 4;

    const uint32_t row = m.seg_row[seg];
    const uint32_t pb = m.seg_page_begin[seg], pe = m.seg_page_end[seg];
    const uint32_t len = m.row_len[row];
    const uint32_t* tbl = m.tables + m.seq_tbl_off[m.row_seq[row]];
    const uint32_t tok_begin = pb * kPage;
    const uint32_t tok_end = min(len, pe * kPage);
    const uint32_t n_tok = tok_end > tok_begin ? tok_end - tok_begin : 0;
    const uint32_t n_tiles = (n_tok + TT - 1) / TT;

    // Q' fragments of this warp's 9 k-steps (A operand, row-major 16 x 16 per step).
    uint32_t qa[KS_PER_WARP][4];
    {
        const T* qrow0 = q_abs + (size_t(row) * H + h0 + g) * kRow;
        const T* qrow1 = qrow0 + size_t(8) * kRow;
        const bool v0 = h0 + g < H, v1 = h0 + g + 8 < H;
#pragma unroll
        for (int j = 0; j < KS_PER_WARP; j++) {
            const int col = (warp * KS_PER_WARP + j) * 16 + t4 * 2;
            qa[j][0] = v0 ? *reinterpret_cast<const uint32_t*>(qrow0 + col) : 0u;
            qa[j][1] = v1 ? *reinterpret_cast<const uint32_t*>(qrow1 + col) : 0u;
            qa[j][2] = v0 ? *reinterpret_cast<const uint32_t*>(qrow0 + col + 8) : 0u;
            qa[j][3] = v1 ? *reinterpret_cast<const uint32_t*>(qrow1 + col + 8) : 0u;
        }
    }

    auto issue_tile = [&](uint32_t tile) {
        if (tile < n_tiles) {
            const uint32_t tok = tok_begin + tile * TT;
            uint32_t page = tbl[tok / kPage];
            if (page >= n_pages) {
                if (tid == 0) atomicOr(status, ST_BAD_PAGE);
                page = 0;
            }
            const T* src = pool + (size_t(page) * kPage + tok % kPage) * kRow;
            T* dst = kv + size_t(tile % NS) * TT * KV_PITCH;
            constexpr int kChunksPerRow = kRow / 8;   // 72
            // rows at or past the segment's end are zero-filled, not read: a caller's cache may end with its last
            // row, and whatever lies behind a sequence's end need not be finite (P = 0 times NaN is NaN)
            const uint32_t live_rows = n_tok - tile * TT;            // > 0 here; >= TT for all but the last tile
#pragma unroll
            for (int k = 0; k < TT * kChunksPerRow / 128; k++) {
                const int c = tid + 128 * k;
                const int r = c / kChunksPerRow, cc = c % kChunksPerRow;
                const bool live = uint32_t(r) < live_rows;
                cp_async16(smem_u32(dst + r * KV_PITCH + cc * 8), src + (live ? size_t(r) * kRow + cc * 8 : 0), live);
            }
        }
        cp_async_commit();
    };

    float oacc[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;   // kept by the softmax-phase owner of row tid/8

    issue_tile(0);
    for (uint32_t tile = 0; tile < n_tiles; tile++) {
        cp_async_wait<0>();
        __syncthreads();              // tile landed; everyone is done with the previous tile
        issue_tile(tile + 1);
        const T* kvt = kv + size_t(tile % NS) * TT * KV_PITCH;

        // ---- partial scores over this warp's slice of the contraction
        float sacc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.0f;
        {
            const int mi = lane / 8, rr = lane % 8;
#pragma unroll
            for (int j = 0; j < KS_PER_WARP; j++) {
                const int kcol = (warp * KS_PER_WARP + j) * 16 + (mi % 2) * 8;
#pragma unroll
                for (int np = 0; np < 2; np++) {
                    uint32_t b[4];
                    ldsm_x4(b, smem_u32(kvt + (np * 16 + (mi / 2) * 8 + rr) * KV_PITCH + kcol));
                    mma16816<T>(sacc[np * 2], qa[j], b[0], b[1]);
                    mma16816<T>(sacc[np * 2 + 1], qa[j], b[2], b[3]);
                }
            }
            float* sp = Sp + size_t(warp) * 16 * SP_PITCH;
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                *reinterpret_cast<float2*>(sp + g * SP_PITCH + nt * 8 + t4 * 2) = make_float2(sacc[nt][0], sacc[nt][1]);
                *reinterpret_cast<float2*>(sp + (g + 8) * SP_PITCH + nt * 8 + t4 * 2) = make_float2(sacc[nt][2], sacc[nt][3]);
            }
        }
        __syncthreads();

        // ---- online softmax: thread -> (head row tid/8, 4 tokens)
        {
            const int r = tid / 8, c4 = (tid % 8) * 4;
            float s[4];
            float mx = -INFINITY;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                float v = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; w++) v += Sp[(w * 16 + r) * SP_PITCH + c4 + k];
                v *= scale_log2;
                if (tile * TT + c4 + k >= n_tok) v = -INFINITY;
                s[k] = v;
                mx = fmaxf(mx, v);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            const float m_new = fmaxf(m_run, mx);
            const float alpha = exp2f(m_run - m_new);
            float p[4], sum = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                p[k] = exp2f(s[k] - m_new);
                sum += p[k];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            l_run = l_run * alpha + sum;
            m_run = m_new;
            uint2 pk;
            pk.x = Elem<T>::pack2(p[0], p[1]);
            pk.y = Elem<T>::pack2(p[2], p[3]);
            *reinterpret_cast<uint2*>(Ps + r * PS_PITCH + c4) = pk;
            if (tid % 8 == 0) alpha_s[r] = alpha;
        }
        __syncthreads();

        // ---- O = O*alpha + P.V on this warp's 128 latent columns
        {
            const float a0 = alpha_s[g], a1 = alpha_s[g + 8];
#pragma unroll
            for (int i = 0; i < 16; i++) {
                oacc[i][0] *= a0; oacc[i][1] *= a0;
                oacc[i][2] *= a1; oacc[i][3] *= a1;
            }
            const int mi = lane / 8, rr = lane % 8;
#pragma unroll
            for (int kk = 0; kk < TT / 16; kk++) {
                uint32_t pa[4];
                ldsm_x4(pa, smem_u32(Ps + ((mi % 2) * 8 + rr) * PS_PITCH + kk * 16 + (mi / 2) * 8));
#pragma unroll
                for (int np = 0; np < 8; np++) {
                    uint32_t b[4];
                    ldsm_x4_t(b, smem_u32(kvt + (kk * 16 + (mi % 2) * 8 + rr) * KV_PITCH +
                                          warp * 128 + np * 16 + (mi / 2) * 8));
                    mma16816<T>(oacc[np * 2], pa, b[0], b[1]);
                    mma16816<T>(oacc[np * 2 + 1], pa, b[2], b[3]);
                }
            }
        }
    }
    cp_async_wait<0>();

    // ---- partial state out
    {
        const uint32_t ha = h0 + g, hb = h0 + g + 8;
        if (ha < H) {
            float* rc = recs + (size_t(seg) * H + ha) * kPart + 2 + warp * 128 + t4 * 2;
#pragma unroll
            for (int nt = 0; nt < 16; nt++)
                *reinterpret_cast<float2*>(rc + nt * 8) = make_float2(oacc[nt][0], oacc[nt][1]);
        }
        if (hb < H) {
            float* rc = recs + (size_t(seg) * H + hb) * kPart + 2 + warp * 128 + t4 * 2;
#pragma unroll
            for (int nt = 0; nt < 16; nt++)
                *reinterpret_cast<float2*>(rc + nt * 8) = make_float2(oacc[nt][2], oacc[nt][3]);
        }
        if (tid % 8 == 0 && h0 + tid / 8 < H) {
            float* rc = recs + (size_t(seg) * H + h0 + tid / 8) * kPart;
            rc[0] = m_run;
            rc[1] = l_run;
        }
    }
}

}  // namespace

// Function attributes belong to a device: called once per device (context creation, first use of the
// no-allocation entry point on a device), with that device current.
int decode_mma_configure()
{
    cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_TOTAL));
    if (e != cudaSuccess) return int(e);
    e = cudaFuncSetAttribute(decode_mma_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_TOTAL));
    return int(e);
}

int launch_decode_mma(int dtype, const void* q_abs, const void* layer_pool, uint32_t n_pages,
                      const StepMeta& m, float* recs, uint32_t H, uint32_t* status, cudaStream_t st)
{
    if (m.segs == 0) return 0;
    const float scale_log2 = 1.4426950408889634f / sqrtf(float(kQDim));
    dim3 grid(m.segs, (H + 15) / 16);
    if (dtype == 0)
        decode_mma_kernel<__half><<<grid, 128, SMEM_TOTAL, st>>>(
            static_cast<const __half*>(q_abs), static_cast<const __half*>(layer_pool), n_pages, m, recs,
            H, scale_log2, status);
    else
        decode_mma_kernel<__nv_bfloat16><<<grid, 128, SMEM_TOTAL, st>>>(
            static_cast<const __nv_bfloat16*>(q_abs), static_cast<const __nv_bfloat16*>(layer_pool),
            n_pages, m, recs, H, scale_log2, status);
    return int(cudaGetLastError());
}

}  // namespace mla
