// Small kernels around the attention core: latent-row append, q absorption, partial merge +
// W_UV projection, bulk row copy.  sm_100a.
#include "mla_launch.h"

namespace mla {

// ------------------------------------------------------------------------------------------
// Append: RMSNorm(c_kv)*w, NeoX RoPE(k_rope) and the scatter of the 576-value row into its
// page slot.  Follows the reference's statements one by one so that the stored bits equal the
// CPU path's (src/core/model/transformer.cpp:3935-3948 and :3964-3975):
//   ss = sum_i x_i*x_i            sequential, float, multiply and add rounded separately
//   r  = 1 / sqrt(ss/512 + eps)
//   c_kv[i] = T( (x_i*r) * w_i )  two multiplies, one final rounding
//   k[i]    = T( x0*cos - x1*sin ),  k[i+32] = T( x1*cos + x0*sin )   from the original x0, x1
// cos/sin come from a host-built table (the host evaluates them with the same libm calls as
// the CPU path; device cosf/sinf are not bit-identical to glibc's).
// One block per row; the squares are formed in parallel, thread 0 adds them in order.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
append_kernel(const T* __restrict__ kv_a, T* __restrict__ pool, uint64_t pool_slots,
              const T* __restrict__ norm_w, const float* __restrict__ cos_sin, uint32_t cs_rows,
              float eps, const uint32_t* __restrict__ row_pos,
              const uint64_t* __restrict__ row_slot, uint32_t* __restrict__ status)
{
    __shared__ __align__(16) T xin[kRow];
    __shared__ __align__(16) T xout[kRow];
    __shared__ float sq[kRank];
    __shared__ float rinv_s;
    const uint32_t r = blockIdx.x, tid = threadIdx.x;
    const uint64_t slot = row_slot[r];
    const uint32_t pos = row_pos[r];
    if (slot == ~uint64_t(0)) return;          // a query-only row: nothing to append
    if (slot >= pool_slots || pos >= cs_rows) {
        if (tid == 0) atomicOr(status, ST_BAD_SLOT);
        return;
    }
    constexpr int kChunks = kRow * 2 / 16;   // 72 x 16 bytes
    if (tid < kChunks)
        reinterpret_cast<uint4*>(xin)[tid] =
            reinterpret_cast<const uint4*>(kv_a + size_t(r) * kRow)[tid];
    __syncthreads();
    // squares in parallel (each product is rounded on its own, as in the reference), then ONE
    // thread adds them in index order: the sum's rounding sequence is the reference's
    for (int i = tid; i < kRank; i += 128) {
        const float v = Elem<T>::to_f32(xin[i]);
        sq[i] = __fmul_rn(v, v);
    }
    if (tid >= 32 && tid < 64) {
        const int i = tid - 32;
        const float c = cos_sin[size_t(pos) * kRope + i];
        const float s = cos_sin[size_t(pos) * kRope + 32 + i];
        const float x0 = Elem<T>::to_f32(xin[kRank + i]);
        const float x1 = Elem<T>::to_f32(xin[kRank + 32 + i]);
        xout[kRank + i]      = Elem<T>::from_f32(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
        xout[kRank + 32 + i] = Elem<T>::from_f32(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s)));
    }
    __syncthreads();
    if (tid == 0) {
        float ss = 0.0f;
#pragma unroll 16
        for (int i = 0; i < kRank; i++) ss = __fadd_rn(ss, sq[i]);
        rinv_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, float(kRank)), eps)));
    }
    __syncthreads();
    const float rinv = rinv_s;
    for (int i = tid; i < kRank; i += 128) {
        const float v = __fmul_rn(Elem<T>::to_f32(xin[i]), rinv);
        xout[i] = Elem<T>::from_f32(__fmul_rn(v, Elem<T>::to_f32(norm_w[i])));
    }
    __syncthreads();
    if (tid < kChunks)
        reinterpret_cast<uint4*>(pool + slot * kRow)[tid] = reinterpret_cast<const uint4*>(xout)[tid];
}

void launch_append(int dtype, const void* kv_a, void* layer_pool, uint64_t pool_slots,
                   const void* norm_w, const float* cos_sin, uint32_t cs_rows, float eps,
                   const StepMeta& m, uint32_t* status, cudaStream_t st)
{
    if (m.app_rows == 0) return;
    if (dtype == 0)
        append_kernel<__half><<<m.app_rows, 128, 0, st>>>(
            static_cast<const __half*>(kv_a), static_cast<__half*>(layer_pool), pool_slots,
            static_cast<const __half*>(norm_w), cos_sin, cs_rows, eps, m.app_pos, m.app_slot, status);
    else
        append_kernel<__nv_bfloat16><<<m.app_rows, 128, 0, st>>>(
            static_cast<const __nv_bfloat16*>(kv_a), static_cast<__nv_bfloat16*>(layer_pool),
            pool_slots, static_cast<const __nv_bfloat16*>(norm_w), cos_sin, cs_rows, eps, m.app_pos,
            m.app_slot, status);
}

// ------------------------------------------------------------------------------------------
// Bulk copy of ready-made latent rows into a sequence's pages (cache fill / restore).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
write_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ pool, uint64_t pool_slots,
                  const uint32_t* __restrict__ table, uint32_t row_begin, uint32_t n,
                  uint32_t* __restrict__ status)
{
    constexpr int kChunks = kRow * 2 / 16;
    const uint32_t r = blockIdx.x * 4 + threadIdx.x / 32;   // one warp per row
    if (r >= n) return;
    const uint32_t row = row_begin + r;
    const uint64_t slot = uint64_t(table[row / kPage]) * kPage + row % kPage;
    if (slot >= pool_slots) {
        if ((threadIdx.x & 31) == 0) atomicOr(status, ST_BAD_SLOT);
        return;
    }
    for (int c = threadIdx.x & 31; c < kChunks; c += 32)
        pool[slot * kChunks + c] = src[size_t(r) * kChunks + c];
}

void launch_write_rows(const void* src, void* layer_pool, uint64_t pool_slots, const uint32_t* table,
                       uint32_t row_begin, uint32_t n, uint32_t* status, cudaStream_t st)
{
    if (n == 0) return;
    write_rows_kernel<<<(n + 3) / 4, 128, 0, st>>>(static_cast<const uint4*>(src),
                                                    static_cast<uint4*>(layer_pool), pool_slots,
                                                    table, row_begin, n, status);
}

// ------------------------------------------------------------------------------------------
// q absorption (reference: transformer.cpp:2563-2573):
//   q_abs[r][h][d] = sum_{i<128} q[r][h][i] * W_UK[h*128+i][d],   d < 512
// and q_rope copied behind it, so that a query row has the layout of a cache row
// (512 latent dims, then 64 rope dims) and the score is one 576-long dot product.
// ------------------------------------------------------------------------------------------
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

// Block = (head, quarter of the 512 output columns, group of up to 8 row tiles of 16 query rows);
// C[16 x 128] = q_nope[16 x 128] . W_UK_h[128 x 128 cols] per row tile on the warp-level tensor path
// (m16n8k16, f32 accumulate).  The weight is read from its transposed copy W_UK^T[h][d][i] (made
// once at registration), so B fragments are 16-byte loads with the contraction index contiguous;
// a warp loads the fragments of its 32 output columns ONCE and reuses them for every row tile of
// the block, so W_UK crosses L2 once per 128 query rows.
// 16-byte operand loads: within each block of 32 contraction indices, thread t4 takes indices
// 8*t4 .. 8*t4+7 of its row, for A and for B alike.  The pairs (0,1),(2,3) feed one MMA as
// (k, k+8) and (4,5),(6,7) the next: a fixed permutation of the contraction index applied to both
// operands, which leaves the product unchanged.
constexpr int kAbsorbTilesPerBlock = 8;
template <typename T>
__global__ void __launch_bounds__(128)
absorb_kernel(const T* __restrict__ q, const T* __restrict__ w_uk_t, T* __restrict__ q_abs,
              uint32_t rows, uint32_t H)
{
    const uint32_t h = blockIdx.x, nq = blockIdx.z, tid = threadIdx.x;
    const uint32_t warp = tid / 32, lane = tid % 32, g = lane / 4, t4 = lane % 4;
    const uint32_t rt_begin = blockIdx.y * kAbsorbTilesPerBlock;
    const uint32_t rt_end = min(rt_begin + kAbsorbTilesPerBlock, (rows + 15) / 16);
    const int col0 = nq * 128 + warp * 32;                     // this warp's 32 output columns
    uint4 b[4][kNope / 32];
#pragma unroll
    for (int nt = 0; nt < 4; nt++) {
        const T* wrow = w_uk_t + (size_t(h) * kRank + col0 + nt * 8 + g) * kNope + t4 * 8;
#pragma unroll
        for (int kb = 0; kb < kNope / 32; kb++) b[nt][kb] = *reinterpret_cast<const uint4*>(wrow + kb * 32);
    }
    for (uint32_t rt = rt_begin; rt < rt_end; rt++) {
        const uint32_t r0 = rt * 16;
        if (nq == 0) {
            for (int idx = tid; idx < 16 * (kRope / 2); idx += 128) {        // rope part: straight copy
                const uint32_t rr = idx / (kRope / 2), k = idx % (kRope / 2), r = r0 + rr;
                if (r < rows)
                    reinterpret_cast<uint32_t*>(q_abs + (size_t(r) * H + h) * kRow + kRank)[k] =
                        reinterpret_cast<const uint32_t*>(q + (size_t(r) * H + h) * kQDim + kNope)[k];
            }
        }
        uint4 a0[kNope / 32], a1[kNope / 32];
        const bool v0 = r0 + g < rows, v1 = r0 + g + 8 < rows;
        const T* q0 = q + (size_t(r0 + g) * H + h) * kQDim + t4 * 8;
        const T* q1 = q + (size_t(r0 + g + 8) * H + h) * kQDim + t4 * 8;
#pragma unroll
        for (int kb = 0; kb < kNope / 32; kb++) {
            a0[kb] = v0 ? *reinterpret_cast<const uint4*>(q0 + kb * 32) : make_uint4(0, 0, 0, 0);
            a1[kb] = v1 ? *reinterpret_cast<const uint4*>(q1 + kb * 32) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int kb = 0; kb < kNope / 32; kb++) {
                const uint32_t f0[4] = {a0[kb].x, a1[kb].x, a0[kb].y, a1[kb].y};
                const uint32_t f1[4] = {a0[kb].z, a1[kb].z, a0[kb].w, a1[kb].w};
                mma16816<T>(c, f0, b[nt][kb].x, b[nt][kb].y);
                mma16816<T>(c, f1, b[nt][kb].z, b[nt][kb].w);
            }
            const int col = col0 + nt * 8 + t4 * 2;
            if (v0) *reinterpret_cast<uint32_t*>(q_abs + (size_t(r0 + g) * H + h) * kRow + col) = Elem<T>::pack2(c[0], c[1]);
            if (v1) *reinterpret_cast<uint32_t*>(q_abs + (size_t(r0 + g + 8) * H + h) * kRow + col) = Elem<T>::pack2(c[2], c[3]);
        }
    }
}

void launch_absorb(int dtype, const void* q, const void* w_uk_t, void* q_abs, uint32_t rows,
                   uint32_t H, cudaStream_t st)
{
    if (rows == 0) return;
    const uint32_t row_tiles = (rows + 15) / 16;
    dim3 grid(H, (row_tiles + kAbsorbTilesPerBlock - 1) / kAbsorbTilesPerBlock, 4);
    if (dtype == 0)
        absorb_kernel<__half><<<grid, 128, 0, st>>>(static_cast<const __half*>(q), static_cast<const __half*>(w_uk_t),
                                                    static_cast<__half*>(q_abs), rows, H);
    else
        absorb_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(
            static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(w_uk_t),
            static_cast<__nv_bfloat16*>(q_abs), rows, H);
}

// ------------------------------------------------------------------------------------------
// Merge of partial softmax states + W_UV projection (reference: transformer.cpp:2610-2620).
// A partial record is 514 floats per (part, head): m (log2 domain), l, acc[512].
//   M = max m_p ;  w_p = 2^(m_p - M) ;  o_c = sum w_p*acc_p / sum w_p*l_p
//   out[r][h][j] = T( sum_d o_c[d] * W_UV[h*128+j][d] )
// Parts of row r are either the row's split-KV segments (records seg*H + h, segments
// row_seg_begin[r] .. row_seg_begin[r+1]) or the shards of a KV-range-sharded sequence (records
// (p*rows + r)*H + h, p < n_parts).
// ------------------------------------------------------------------------------------------

// The merged, still un-normalised state of every (row, head) written out (the per-GPU partial of a KV-range-sharded
// sequence): one block per (head, row); the 16 warps take a slice of the row's parts each (a lane owns dims
// 64*k + 2*lane (+1), k = 0..7, so a warp load covers whole lines of a record), their sums meet in shared memory and
// warp 0 folds them.  One sequence cut into 74 segments costs two round trips to memory.
__global__ void __launch_bounds__(512)
export_partial_kernel(const float* __restrict__ recs, const uint32_t* __restrict__ row_seg_begin, uint32_t n_parts,
                      float* __restrict__ exported, uint32_t rows, uint32_t H)
{
    __shared__ float scratch[16][32][18];
    const uint32_t h = blockIdx.x, r = blockIdx.y, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    uint32_t pb = 0, pe = n_parts;
    if (row_seg_begin) { pb = row_seg_begin[r]; pe = row_seg_begin[r + 1]; }
    auto rec_of = [&](uint32_t p) -> const float* {
        const size_t idx = row_seg_begin ? (size_t(p) * H + h) : ((size_t(p) * rows + r) * H + h);
        return recs + idx * kPart;
    };
    const uint32_t chunk = (pe - pb + 15) / 16;
    pb = min(pe, pb + warp * chunk);
    pe = min(pe, pb + chunk);
    float M = -INFINITY, L = 0.0f, acc[16];
#pragma unroll
    for (int k = 0; k < 16; k++) acc[k] = 0.0f;
    for (uint32_t p = pb; p < pe; p += 4) {
        float2 ml[4], v[4][8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const bool on = p + i < pe;
            const float* rc = rec_of(on ? p + i : pb);
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
            for (int k = 0; k < 16; k++) acc[k] *= sc;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float w = exp2f(ml[i].x - Mn);
                L = fmaf(w, ml[i].y, L);
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    acc[2 * k] = fmaf(w, v[i][k].x, acc[2 * k]);
                    acc[2 * k + 1] = fmaf(w, v[i][k].y, acc[2 * k + 1]);
                }
            }
            M = Mn;
        }
    }
    float* mine = scratch[warp][lane];
    mine[0] = M;
    mine[1] = L;
#pragma unroll
    for (int k = 0; k < 16; k++) mine[2 + k] = acc[k];
    __syncthreads();
    if (warp != 0) return;
    M = -INFINITY;
    L = 0.0f;
#pragma unroll
    for (int k = 0; k < 16; k++) acc[k] = 0.0f;
    for (int j = 0; j < 16; j++) {
        const float* o = scratch[j][lane];
        const float Mj = o[0];
        if (Mj == -INFINITY) continue;
        const float Mn = fmaxf(M, Mj), sc = exp2f(M - Mn), w = exp2f(Mj - Mn);
        L = fmaf(w, o[1], L * sc);
#pragma unroll
        for (int k = 0; k < 16; k++) acc[k] = fmaf(w, o[2 + k], acc[k] * sc);
        M = Mn;
    }
    float* ex = exported + (size_t(r) * H + h) * kPart;
    if (lane == 0) { ex[0] = M; ex[1] = L; }
#pragma unroll
    for (int k = 0; k < 8; k++) *reinterpret_cast<float2*>(ex + 2 + 64 * k + 2 * lane) = make_float2(acc[2 * k], acc[2 * k + 1]);
}

// Same merge, projection on the warp-level tensor path.  Block = (head, group of up to 4 row tiles
// of 16 query rows), 16 warps.  W_UV_h (128 x 512, 128 KB) is staged ONCE per block in shared
// memory with 16-byte loads and serves every row tile of the block.  Per row tile:
//   1. warp r finds row r's M and 1/L: its lanes take the row's parts in parallel;
//   2. the merged, normalised o_c[16 x 512] is built in shared memory as TWO 16-bit matrices,
//      hi = T(o) and lo = T(o - hi): together they carry ~16 (bf16) / 22 (fp16) mantissa bits, so
//      the float state is not rounded to the storage type before W_UV; thread -> (row, 16 dims);
//   3. out[16 x 128] = (hi + lo)[16 x 512] . W_UV_h^T, m16n8k16 with f32 accumulate; warp w owns
//      outputs [8w, 8w+8), all fragments come from shared memory through ldmatrix.
constexpr int kMergeTilesPerBlock = 4;
constexpr int kMergePitch = kRank + 8;               // elements; keeps ldmatrix rows on distinct banks
constexpr size_t kMergeSmem = size_t(kVDim + 32) * kMergePitch * 2 + 16 * 4 * 4;
template <typename T>
__global__ void __launch_bounds__(512)
merge_outproj_mma_kernel(const float* __restrict__ recs, const uint32_t* __restrict__ row_seg_begin,
                         uint32_t n_parts, const T* __restrict__ w_uv, T* __restrict__ out, uint32_t rows,
                         uint32_t H, const uint32_t* __restrict__ att_row)
{
    constexpr int PITCH = kMergePitch;
    extern __shared__ __align__(16) unsigned char merge_smem[];
    T* w_s = reinterpret_cast<T*>(merge_smem);                       // [128][PITCH]
    T* a_hi = w_s + size_t(kVDim) * PITCH;                           // [16][PITCH]
    T* a_lo = a_hi + 16 * PITCH;                                     // [16][PITCH]
    float* row_m = reinterpret_cast<float*>(a_lo + 16 * PITCH);
    float* row_inv = row_m + 16;
    uint32_t* row_pb = reinterpret_cast<uint32_t*>(row_inv + 16);
    uint32_t* row_pe = row_pb + 16;
    const uint32_t h = blockIdx.x, tid = threadIdx.x;
    const uint32_t warp = tid / 32, lane = tid % 32, g = lane / 4, t4 = lane % 4;
    const uint32_t rt_begin = blockIdx.y * kMergeTilesPerBlock;
    const uint32_t rt_end = min(rt_begin + kMergeTilesPerBlock, (rows + 15) / 16);
    auto rec_of = [&](uint32_t r, uint32_t p) -> const float* {
        const size_t idx = row_seg_begin ? (size_t(p) * H + h) : ((size_t(p) * rows + r) * H + h);
        return recs + idx * kPart;
    };
    {   // stage W_UV_h: 128 rows x 64 chunks of 16 bytes, 16 chunks per thread, all in flight at once
        const uint4* src = reinterpret_cast<const uint4*>(w_uv + size_t(h) * kVDim * kRank);
        uint4 v[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = src[tid + 512 * i];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int c = tid + 512 * i, row = c / 64, ch = c % 64;
            *reinterpret_cast<uint4*>(w_s + size_t(row) * PITCH + ch * 8) = v[i];
        }
    }
    const int mi = lane / 8, lr = lane % 8;
    const uint32_t hi_addr = static_cast<uint32_t>(__cvta_generic_to_shared(a_hi + ((mi % 2) * 8 + lr) * PITCH + (mi / 2) * 8));
    const uint32_t lo_addr = static_cast<uint32_t>(__cvta_generic_to_shared(a_lo + ((mi % 2) * 8 + lr) * PITCH + (mi / 2) * 8));
    // B fragments of outputs [8w, 8w+8) for two k-steps per ldmatrix.x4: matrices (k0-7, k8-15) of step s, then of step s+1
    const uint32_t w_addr = static_cast<uint32_t>(__cvta_generic_to_shared(w_s + size_t(warp * 8 + lr) * PITCH + mi * 8));
    for (uint32_t rt = rt_begin; rt < rt_end; rt++) {
        const uint32_t r0 = rt * 16;
        {
            const uint32_t r = r0 + warp;                // warp <-> row
            uint32_t pb = 0, pe = 0;
            if (r < rows) {
                if (row_seg_begin) { pb = row_seg_begin[r]; pe = row_seg_begin[r + 1]; }
                else               { pb = 0; pe = n_parts; }
            }
            float M = -INFINITY;
            for (uint32_t p = pb + lane; p < pe; p += 32) M = fmaxf(M, rec_of(r, p)[0]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
            float L = 0.0f;
            if (M > -INFINITY)
                for (uint32_t p = pb + lane; p < pe; p += 32) {
                    const float* rc = rec_of(r, p);
                    L = fmaf(exp2f(rc[0] - M), rc[1], L);
                }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
            if (lane == 0) {
                row_m[warp] = M;
                row_inv[warp] = L > 0.0f ? 1.0f / L : 0.0f;
                row_pb[warp] = pb;
                row_pe[warp] = pe;
            }
        }
        __syncthreads();                                 // also: W_UV staged (first tile), previous tile's MMAs done
        {   // thread -> row tid/32, dims (tid%32)*16 .. +15
            const uint32_t rr = tid / 32, r = r0 + rr, d0 = (tid % 32) * 16;
            const float M = row_m[rr], inv = row_inv[rr];
            const uint32_t pb = row_pb[rr], pe = row_pe[rr];
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = 0.0f;
            if (inv > 0.0f)
                for (uint32_t p = pb; p < pe; p++) {
                    const float* rc = rec_of(r, p);
                    const float w = exp2f(rc[0] - M);
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const float2 v = *reinterpret_cast<const float2*>(rc + 2 + d0 + 2 * i);
                        acc[2 * i] = fmaf(w, v.x, acc[2 * i]);
                        acc[2 * i + 1] = fmaf(w, v.y, acc[2 * i + 1]);
                    }
                }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float o0 = acc[2 * i] * inv, o1 = acc[2 * i + 1] * inv;
                const T h0 = Elem<T>::from_f32(o0), h1 = Elem<T>::from_f32(o1);
                *reinterpret_cast<uint32_t*>(a_hi + rr * PITCH + d0 + 2 * i) = Elem<T>::pack2(o0, o1);
                *reinterpret_cast<uint32_t*>(a_lo + rr * PITCH + d0 + 2 * i) =
                    Elem<T>::pack2(o0 - Elem<T>::to_f32(h0), o1 - Elem<T>::to_f32(h1));
            }
        }
        __syncthreads();
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
        for (int ks = 0; ks < kRank / 16; ks += 2) {
            uint32_t bw[4];
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                         : "=r"(bw[0]), "=r"(bw[1]), "=r"(bw[2]), "=r"(bw[3]) : "r"(w_addr + ks * 32));
#pragma unroll
            for (int u = 0; u < 2; u++) {
                uint32_t ah[4], al[4];
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(ah[0]), "=r"(ah[1]), "=r"(ah[2]), "=r"(ah[3]) : "r"(hi_addr + (ks + u) * 32));
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(al[0]), "=r"(al[1]), "=r"(al[2]), "=r"(al[3]) : "r"(lo_addr + (ks + u) * 32));
                mma16816<T>(c, ah, bw[2 * u], bw[2 * u + 1]);
                mma16816<T>(c, al, bw[2 * u], bw[2 * u + 1]);
            }
        }
        const int col = warp * 8 + t4 * 2;
        if (r0 + g < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t(att_row ? att_row[r0 + g] : r0 + g) * H + h) * kVDim + col) = Elem<T>::pack2(c[0], c[1]);
        if (r0 + g + 8 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t(att_row ? att_row[r0 + g + 8] : r0 + g + 8) * H + h) * kVDim + col) = Elem<T>::pack2(c[2], c[3]);
        __syncthreads();                                 // a_hi / a_lo / row_* are rewritten by the next tile
    }
}

// Once per device, with that device current (function attributes are per device).
int merge_mma_configure()
{
    cudaError_t e = cudaFuncSetAttribute(merge_outproj_mma_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kMergeSmem));
    if (e != cudaSuccess) return int(e);
    e = cudaFuncSetAttribute(merge_outproj_mma_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kMergeSmem));
    return int(e);
}

void launch_merge(int dtype, const float* recs, const uint32_t* row_seg_begin, uint32_t n_parts,
                  const void* w_uv, void* out, float* exported, uint32_t rows, uint32_t H,
                  cudaStream_t st, const uint32_t* att_row)
{
    if (rows == 0) return;
    if (!exported) {
        const uint32_t row_tiles = (rows + 15) / 16;
        dim3 grid16(H, (row_tiles + kMergeTilesPerBlock - 1) / kMergeTilesPerBlock);
        if (dtype == 0)
            merge_outproj_mma_kernel<__half><<<grid16, 512, kMergeSmem, st>>>(
                recs, row_seg_begin, n_parts, static_cast<const __half*>(w_uv), static_cast<__half*>(out), rows, H, att_row);
        else
            merge_outproj_mma_kernel<__nv_bfloat16><<<grid16, 512, kMergeSmem, st>>>(
                recs, row_seg_begin, n_parts, static_cast<const __nv_bfloat16*>(w_uv),
                static_cast<__nv_bfloat16*>(out), rows, H, att_row);
        return;
    }
    export_partial_kernel<<<dim3(H, rows), 512, 0, st>>>(recs, row_seg_begin, n_parts, exported, rows, H);
}

}  // namespace mla
