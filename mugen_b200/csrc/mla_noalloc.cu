// mla_attention_noalloc: the absorbed MLA attention of ONE query row over ONE contiguous latent
// cache, for callers that may not allocate device memory.
//
// Who cannot allocate: code running under a framework that owns all device memory through its
// own pool or arena (an allocation behind its back fragments or deadlocks it), code that runs
// inside a latency-critical serving loop where cudaMalloc's implicit device synchronisation
// stalls every other stream, and plug-ins that are only handed device pointers and a stream.
// Every other entry point of this library works on an mla_ctx whose creation allocates the
// page pool and the workspaces; this one needs no context.  The caller passes inputs and the
// output; the intermediate buffers (absorbed query, per-segment partial softmax states, the
// small segment table) live in the file-scope array below, which every process that loads the
// library holds on each GPU it touches until it exits.
//
// Consequences of the shared array: calls that overlap on one GPU (two streams, two threads)
// race on it and must be serialised by the caller; it keeps the previous call's contents, and
// nothing in it needs to start at zero — every word that is read was written earlier in the same
// call (this is checked by the test that runs two different problems back to back).
#include <cstring>
#include <string>

#include "../../include/mugen_mla.h"
#include "mla_launch.h"

namespace {

constexpr uint32_t kMaxHeads = 128;
constexpr uint32_t kMaxSeqLen = 65536;                    // tokens
constexpr uint32_t kMaxSegs = 32;                         // split-KV segments per call
constexpr size_t kMetaBytes = 8192;                       // segment table, block table (<= 1024 pages)
constexpr size_t kQAbsBytes = size_t(kMaxHeads) * mla::kRow * 2;
constexpr size_t kRecBytes = size_t(kMaxSegs) * kMaxHeads * mla::kPart * sizeof(float);
constexpr size_t kOffQAbs = kMetaBytes;
constexpr size_t kOffRecs = kOffQAbs + ((kQAbsBytes + 255) & ~size_t(255));
constexpr size_t kScratchBytes = kOffRecs + kRecBytes;    // 8,577,024 B, about 8.2 MiB
static_assert(kScratchBytes == 8577024, "the size quoted in the public header");

// The call's bookkeeping at the start of the scratch array, in the form the attention kernels read.
struct Meta {
    uint32_t row_seq, row_len, tbl_off, row_seg_begin[2];
    uint32_t seg_row[kMaxSegs], seg_pb[kMaxSegs], seg_pe[kMaxSegs];
    uint32_t table[kMaxSeqLen / mla::kPage];
};
static_assert(sizeof(Meta) <= kMetaBytes - 4, "metadata region too small (its last word is the status word)");

// In host code this name is only a stand-in for the symbol, not a device address: the address a
// kernel can use comes from cudaGetSymbolAddress (see scratch_for_current_device).
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

thread_local std::string g_noalloc_error;

int fail(int code, std::string msg)
{
    g_noalloc_error = std::move(msg);
    return code;
}

// q_abs[h][d] = sum_i q[h][i] * W_UK[h*128+i][d] with W_UK in the caller's (reference) layout,
// (n_heads*128) x 512 row-major; q_rope copied behind it.  One block per head.
template <typename T>
__global__ void __launch_bounds__(256)
absorb_one_row_kernel(const T* __restrict__ q, const T* __restrict__ w_uk, T* __restrict__ q_abs)
{
    __shared__ float qs[mla::kNope];
    const uint32_t h = blockIdx.x, tid = threadIdx.x;
    if (tid < mla::kNope) qs[tid] = mla::Elem<T>::to_f32(q[size_t(h) * mla::kQDim + tid]);
    if (tid < mla::kRope) q_abs[size_t(h) * mla::kRow + mla::kRank + tid] = q[size_t(h) * mla::kQDim + mla::kNope + tid];
    __syncthreads();
    float a0 = 0.0f, a1 = 0.0f;
    const T* wp = w_uk + size_t(h) * mla::kNope * mla::kRank + tid * 2;
#pragma unroll 8
    for (int i = 0; i < mla::kNope; i++) {
        const typename mla::Elem<T>::pair w2 = *reinterpret_cast<const typename mla::Elem<T>::pair*>(wp + size_t(i) * mla::kRank);
        a0 = fmaf(qs[i], mla::Elem<T>::to_f32(w2.x), a0);
        a1 = fmaf(qs[i], mla::Elem<T>::to_f32(w2.y), a1);
    }
    *reinterpret_cast<uint32_t*>(q_abs + size_t(h) * mla::kRow + tid * 2) = mla::Elem<T>::pack2(a0, a1);
}

// The split-KV plan (equal page ranges), the identity block table of the contiguous cache and a cleared
// status word, written by the device itself: the host passes two integers, so a call copies nothing from
// host memory.
__global__ void __launch_bounds__(256)
noalloc_plan_kernel(unsigned char* scratch, uint32_t seq_len, uint32_t pages, uint32_t segs)
{
    Meta* mt = reinterpret_cast<Meta*>(scratch);
    const uint32_t tid = threadIdx.x;
    if (tid == 0) {
        mt->row_seq = 0;
        mt->row_len = seq_len;
        mt->tbl_off = 0;
        mt->row_seg_begin[0] = 0;
        mt->row_seg_begin[1] = segs;
        *reinterpret_cast<uint32_t*>(scratch + kMetaBytes - 4) = 0;
    }
    if (tid < segs) {
        mt->seg_row[tid] = 0;
        mt->seg_pb[tid] = uint32_t(uint64_t(pages) * tid / segs);
        mt->seg_pe[tid] = uint32_t(uint64_t(pages) * (tid + 1) / segs);
    }
    for (uint32_t p = tid; p < pages; p += blockDim.x) mt->table[p] = p;
}

// Device address of the scratch array on the CURRENT device.  The first call on a device resolves it and
// sets the two kernels' shared-memory attributes there (both are per-device state).
int scratch_for_current_device(unsigned char** out)
{
    static unsigned char* ptrs[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(MLA_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(MLA_ERR_UNSUPPORTED, "device ordinal beyond 63");
    if (!ptrs[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return fail(MLA_ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
        if (int ce = mla::decode_mma_configure())
            return fail(MLA_ERR_CUDA, std::string("attention kernel attributes: ") + cudaGetErrorString(cudaError_t(ce)));
        if (int ce = mla::merge_mma_configure())
            return fail(MLA_ERR_CUDA, std::string("merge kernel attributes: ") + cudaGetErrorString(cudaError_t(ce)));
        ptrs[dev] = static_cast<unsigned char*>(p);
    }
    *out = ptrs[dev];
    return MLA_OK;
}

}  // namespace

extern "C" {

const char* mla_noalloc_last_error(void) { return g_noalloc_error.c_str(); }

int mla_attention_noalloc(uint32_t dtype, uint32_t n_heads, uint32_t seq_len, const void* q, const void* cache,
                          const void* w_uk, const void* w_uv, void* out, void* stream)
{
    if (dtype > MLA_DTYPE_BF16) return fail(MLA_ERR_INVALID, "dtype must be MLA_DTYPE_F16 or MLA_DTYPE_BF16");
    if (!q || !cache || !w_uk || !w_uv || !out) return fail(MLA_ERR_INVALID, "null argument");
    if (n_heads == 0 || n_heads > kMaxHeads)
        return fail(MLA_ERR_CAPACITY, "n_heads " + std::to_string(n_heads) + " is outside 1.." + std::to_string(kMaxHeads) +
                                          " (limit of the built-in scratch)");
    if (seq_len > kMaxSeqLen)
        return fail(MLA_ERR_CAPACITY, "seq_len " + std::to_string(seq_len) + " exceeds " + std::to_string(kMaxSeqLen) +
                                          " (limit of the built-in scratch)");
    auto st = static_cast<cudaStream_t>(stream);
    unsigned char* scratch = nullptr;
    if (int rc = scratch_for_current_device(&scratch)) return rc;

    // ---- segment plan, identity block table and status word: written on the device
    const uint32_t pages = (seq_len + mla::kPage - 1) / mla::kPage;
    const uint32_t segs = pages == 0 ? 1 : (pages < kMaxSegs ? pages : kMaxSegs);
    noalloc_plan_kernel<<<1, 256, 0, st>>>(scratch, seq_len, pages, segs);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MLA_ERR_CUDA, std::string("plan launch: ") + cudaGetErrorString(e));

    mla::StepMeta m{};
    auto at = [&](size_t off) { return reinterpret_cast<const uint32_t*>(scratch + off); };
    m.row_seq = at(offsetof(Meta, row_seq));
    m.row_len = at(offsetof(Meta, row_len));
    m.row_pos = nullptr;
    m.row_slot = nullptr;
    m.seq_tbl_off = at(offsetof(Meta, tbl_off));
    m.tables = at(offsetof(Meta, table));
    m.seg_row = at(offsetof(Meta, seg_row));
    m.seg_page_begin = at(offsetof(Meta, seg_pb));
    m.seg_page_end = at(offsetof(Meta, seg_pe));
    m.row_seg_begin = at(offsetof(Meta, row_seg_begin));
    m.cta_seg_begin = nullptr;
    m.rows = 1;
    m.segs = segs;
    m.ctas = segs;

    void* q_abs = scratch + kOffQAbs;
    float* recs = reinterpret_cast<float*>(scratch + kOffRecs);
    // The kernels want a status word to report into; this path has no call that reads it back (the only bit
    // they can raise here, a bad page id, cannot occur with the identity table built above).
    uint32_t* status = reinterpret_cast<uint32_t*>(scratch + kMetaBytes - 4);   // last word of the metadata region
    if (dtype == MLA_DTYPE_F16)
        absorb_one_row_kernel<__half><<<n_heads, 256, 0, st>>>(static_cast<const __half*>(q), static_cast<const __half*>(w_uk),
                                                               static_cast<__half*>(q_abs));
    else
        absorb_one_row_kernel<__nv_bfloat16><<<n_heads, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(w_uk), static_cast<__nv_bfloat16*>(q_abs));
    // the cache is addressed as pages of 64 rows with the identity table
    if (int rc = mla::launch_decode_mma(int(dtype), q_abs, cache, pages ? pages : 1, m, recs, n_heads, status, st))
        return fail(MLA_ERR_CUDA, std::string("attention launch: ") + cudaGetErrorString(cudaError_t(rc)));
    mla::launch_merge(int(dtype), recs, m.row_seg_begin, 0, w_uv, out, nullptr, 1, n_heads, st);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MLA_ERR_CUDA, std::string("launch: ") + cudaGetErrorString(e));
    return MLA_OK;
}

}  // extern "C"
