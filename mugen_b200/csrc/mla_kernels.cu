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
// One block per row; thread 0 owns the sequential sum, warp 1 does the rotation meanwhile.
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
    if (tid == 0) {
        float ss = 0.0f;
#pragma unroll 8
        for (int i = 0; i < kRank; i++) {
            const float v = Elem<T>::to_f32(xin[i]);
            ss = __fadd_rn(ss, __fmul_rn(v, v));
        }
        rinv_s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, float(kRank)), eps)));
    } else if (tid >= 32 && tid < 64) {
        const int i = tid - 32;
        const float c = cos_sin[size_t(pos) * kRope + i];
        const float s = cos_sin[size_t(pos) * kRope + 32 + i];
        const float x0 = Elem<T>::to_f32(xin[kRank + i]);
        const float x1 = Elem<T>::to_f32(xin[kRank + 32 + i]);
        xout[kRank + i]      = Elem<T>::from_f32(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
        xout[kRank + 32 + i] = Elem<T>::from_f32(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s)));
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
    if (m.rows == 0) return;
    if (dtype == 0)
        append_kernel<__half><<<m.rows, 128, 0, st>>>(
            static_cast<const __half*>(kv_a), static_cast<__half*>(layer_pool), pool_slots,
            static_cast<const __half*>(norm_w), cos_sin, cs_rows, eps, m.row_pos, m.row_slot, status);
    else
        append_kernel<__nv_bfloat16><<<m.rows, 128, 0, st>>>(
            static_cast<const __nv_bfloat16*>(kv_a), static_cast<__nv_bfloat16*>(layer_pool),
            pool_slots, static_cast<const __nv_bfloat16*>(norm_w), cos_sin, cs_rows, eps, m.row_pos,
            m.row_slot, status);
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
// Grid (head, row tile); W_UK_h is streamed once per block and reused for RT rows.
// ------------------------------------------------------------------------------------------
template <typename T, int RT>
__global__ void __launch_bounds__(256)
absorb_kernel(const T* __restrict__ q, const T* __restrict__ w_uk, T* __restrict__ q_abs,
              uint32_t rows, uint32_t H)
{
    __shared__ float qs[RT][kNope];
    const uint32_t h = blockIdx.x, r0 = blockIdx.y * RT, tid = threadIdx.x;
    for (int idx = tid; idx < RT * kNope; idx += 256) {
        const uint32_t rr = idx / kNope, i = idx % kNope, r = r0 + rr;
        qs[rr][i] = r < rows ? Elem<T>::to_f32(q[(size_t(r) * H + h) * kQDim + i]) : 0.0f;
    }
    for (int idx = tid; idx < RT * kRope; idx += 256) {
        const uint32_t rr = idx / kRope, k = idx % kRope, r = r0 + rr;
        if (r < rows)
            q_abs[(size_t(r) * H + h) * kRow + kRank + k] = q[(size_t(r) * H + h) * kQDim + kNope + k];
    }
    __syncthreads();
    const int d0 = tid * 2;
    float acc[RT][2];
#pragma unroll
    for (int rr = 0; rr < RT; rr++) acc[rr][0] = acc[rr][1] = 0.0f;
    const T* wp = w_uk + size_t(h) * kNope * kRank + d0;
#pragma unroll 4
    for (int i = 0; i < kNope; i++) {
        const typename Elem<T>::pair w2 = *reinterpret_cast<const typename Elem<T>::pair*>(wp + size_t(i) * kRank);
        const float w0 = Elem<T>::to_f32(w2.x), w1 = Elem<T>::to_f32(w2.y);
#pragma unroll
        for (int rr = 0; rr < RT; rr++) {
            const float qv = qs[rr][i];
            acc[rr][0] = fmaf(qv, w0, acc[rr][0]);
            acc[rr][1] = fmaf(qv, w1, acc[rr][1]);
        }
    }
#pragma unroll
    for (int rr = 0; rr < RT; rr++) {
        const uint32_t r = r0 + rr;
        if (r < rows)
            *reinterpret_cast<uint32_t*>(q_abs + (size_t(r) * H + h) * kRow + d0) =
                Elem<T>::pack2(acc[rr][0], acc[rr][1]);
    }
}

void launch_absorb(int dtype, const void* q, const void* w_uk, void* q_abs, uint32_t rows,
                   uint32_t H, cudaStream_t st)
{
    if (rows == 0) return;
    constexpr int RT = 8;
    dim3 grid(H, (rows + RT - 1) / RT);
    if (dtype == 0)
        absorb_kernel<__half, RT><<<grid, 256, 0, st>>>(static_cast<const __half*>(q),
                                                        static_cast<const __half*>(w_uk),
                                                        static_cast<__half*>(q_abs), rows, H);
    else
        absorb_kernel<__nv_bfloat16, RT><<<grid, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(w_uk),
            static_cast<__nv_bfloat16*>(q_abs), rows, H);
}

// ------------------------------------------------------------------------------------------
// Merge of partial softmax states + W_UV projection (reference: transformer.cpp:2610-2620).
// A partial record is 514 floats per (part, head): m (log2 domain), l, acc[512].
//   M = max m_p ;  w_p = 2^(m_p - M) ;  o_c = sum w_p*acc_p / sum w_p*l_p
//   out[r][h][j] = T( sum_d o_c[d] * W_UV[h*128+j][d] )
// Parts of row r are either the row's split-KV segments (records seg*H + h, segments
// row_seg_begin[r] .. row_seg_begin[r+1]) or the shards of a KV-range-sharded sequence (records
// (p*rows + r)*H + h, p < n_parts).  With `exported` non-null the merged, still un-normalised
// state is written out instead of being projected.
// o_c stays in float through the projection (the W_UV product is done on the FP32 pipe): the
// bf16 error budget has no room for another rounding here.
// ------------------------------------------------------------------------------------------
template <typename T, int RT>
__global__ void __launch_bounds__(256)
merge_outproj_kernel(const float* __restrict__ recs, const uint32_t* __restrict__ row_seg_begin,
                     uint32_t n_parts, const T* __restrict__ w_uv, T* __restrict__ out,
                     float* __restrict__ exported, uint32_t rows, uint32_t H)
{
    __shared__ __align__(16) float oc[RT][kRank];
    const uint32_t h = blockIdx.x, r0 = blockIdx.y * RT, tid = threadIdx.x;
    const int d0 = tid * 2;
    for (int rr = 0; rr < RT; rr++) {
        const uint32_t r = r0 + rr;
        float a0 = 0.0f, a1 = 0.0f, L = 0.0f, M = -INFINITY;
        if (r < rows) {
            uint32_t pb, pe;
            if (row_seg_begin) { pb = row_seg_begin[r]; pe = row_seg_begin[r + 1]; }
            else               { pb = 0; pe = n_parts; }
            auto rec_of = [&](uint32_t p) -> const float* {
                const size_t idx = row_seg_begin ? (size_t(p) * H + h)
                                                 : ((size_t(p) * rows + r) * H + h);
                return recs + idx * kPart;
            };
            for (uint32_t p = pb; p < pe; p++) M = fmaxf(M, rec_of(p)[0]);
            if (M > -INFINITY) {
                for (uint32_t p = pb; p < pe; p++) {
                    const float* rc = rec_of(p);
                    const float w = exp2f(rc[0] - M);
                    L = fmaf(w, rc[1], L);
                    const float2 a = *reinterpret_cast<const float2*>(rc + 2 + d0);
                    a0 = fmaf(w, a.x, a0);
                    a1 = fmaf(w, a.y, a1);
                }
            }
            if (exported) {
                float* ex = exported + (size_t(r) * H + h) * kPart;
                if (tid == 0) { ex[0] = M; ex[1] = L; }
                *reinterpret_cast<float2*>(ex + 2 + d0) = make_float2(a0, a1);
            }
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
        oc[rr][d0] = a0 * inv;
        oc[rr][d0 + 1] = a1 * inv;
    }
    if (exported) return;
    __syncthreads();
    const int warp = tid / 32, lane = tid % 32;
    for (int jj = 0; jj < kVDim / 8; jj++) {
        const int j = warp * (kVDim / 8) + jj;
        const T* wrow = w_uv + (size_t(h) * kVDim + j) * kRank;
        float s[RT];
#pragma unroll
        for (int rr = 0; rr < RT; rr++) s[rr] = 0.0f;
#pragma unroll
        for (int k = 0; k < kRank / 64; k++) {
            const typename Elem<T>::pair w2 =
                *reinterpret_cast<const typename Elem<T>::pair*>(wrow + k * 64 + lane * 2);
            const float w0 = Elem<T>::to_f32(w2.x), w1 = Elem<T>::to_f32(w2.y);
#pragma unroll
            for (int rr = 0; rr < RT; rr++) {
                const float2 o = *reinterpret_cast<const float2*>(&oc[rr][k * 64 + lane * 2]);
                s[rr] = fmaf(o.x, w0, s[rr]);
                s[rr] = fmaf(o.y, w1, s[rr]);
            }
        }
#pragma unroll
        for (int rr = 0; rr < RT; rr++) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) s[rr] += __shfl_xor_sync(0xffffffffu, s[rr], off);
        }
        if (lane < RT && r0 + lane < rows) {
            float v = 0.0f;
#pragma unroll
            for (int rr = 0; rr < RT; rr++) v = (lane == rr) ? s[rr] : v;
            out[(size_t(r0 + lane) * H + h) * kVDim + j] = Elem<T>::from_f32(v);
        }
    }
}

void launch_merge(int dtype, const float* recs, const uint32_t* row_seg_begin, uint32_t n_parts,
                  const void* w_uv, void* out, float* exported, uint32_t rows, uint32_t H,
                  cudaStream_t st)
{
    if (rows == 0) return;
    constexpr int RT = 8;
    dim3 grid(H, (rows + RT - 1) / RT);
    if (dtype == 0)
        merge_outproj_kernel<__half, RT><<<grid, 256, 0, st>>>(
            recs, row_seg_begin, n_parts, static_cast<const __half*>(w_uv),
            static_cast<__half*>(out), exported, rows, H);
    else
        merge_outproj_kernel<__nv_bfloat16, RT><<<grid, 256, 0, st>>>(
            recs, row_seg_begin, n_parts, static_cast<const __nv_bfloat16*>(w_uv),
            static_cast<__nv_bfloat16*>(out), exported, rows, H);
}

}  // namespace mla
