// Shared definitions of the sm_100a MLA decode kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mla {

constexpr int kRank  = 512;   // kv_lora_rank: width of c_kv
constexpr int kRope  = 64;    // qk_rope_head_dim
constexpr int kNope  = 128;   // qk_nope_head_dim
constexpr int kVDim  = 128;   // v_head_dim
constexpr int kRow   = kRank + kRope;   // 576 values per latent cache row
constexpr int kQDim  = kNope + kRope;   // 192 values per head of q
constexpr int kPage  = 64;    // tokens per page
constexpr int kPart  = kRank + 2;       // floats per head of an exported partial (m, l, acc)

// Bits of the device status word (kernels set these instead of trapping).
enum : uint32_t {
    ST_BAD_SLOT      = 1u << 0,   // append: destination slot outside the pool
    ST_BAD_PAGE      = 1u << 1,   // attend: block-table entry outside the pool
    ST_WAIT_TIMEOUT  = 1u << 2,   // a bounded mbarrier wait gave up
    ST_BAD_SEGMENT   = 1u << 3,   // segment descriptor inconsistent
    ST_BAD_ALIGNMENT = 1u << 4,   // dynamic shared memory did not start on the 1 KB boundary a kernel relies on
};

// Programmatic dependent launch: a kernel launched with launch_pdl() may become resident while the
// previous kernel of the stream is still draining.  It must call grid_dependency_wait() before its
// first access to memory that any earlier kernel of the stream reads or writes (the wait returns
// once the previous grid has completed and flushed; completion is transitive because every kernel
// of the chain waits before it completes).  grid_launch_dependents() lets the next kernel's blocks
// start as soon as this kernel's blocks have all begun.  Both are no-ops in a plain launch.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

template <typename K, typename... Args>
inline cudaError_t launch_pdl(K kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <typename T> struct Elem;
template <> struct Elem<__half> {
    using pair = __half2;
    static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};
template <> struct Elem<__nv_bfloat16> {
    using pair = __nv_bfloat162;
    static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ uint32_t pack2(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

// Per-step metadata resident on the device (one upload per step, shared by all layers).
struct StepMeta {
    // query rows
    const uint32_t* row_seq;        // [rows]  index into the step's sequence list
    const uint32_t* row_len;        // [rows]  rows of the sequence this query attends
    const uint32_t* row_pos;        // [rows]  global position of the appended token (RoPE)
    const uint64_t* row_slot;       // [rows]  destination token slot of the appended token
    // block tables
    const uint32_t* seq_tbl_off;    // [seqs]  offset of the sequence's block table in `tables`
    const uint32_t* tables;         // physical page ids
    // split-KV segments
    const uint32_t* seg_row;        // [segs]
    const uint32_t* seg_page_begin; // [segs]
    const uint32_t* seg_page_end;   // [segs]
    const uint32_t* row_seg_begin;  // [rows+1]  a row's segments are contiguous
    const uint32_t* cta_seg_begin;  // [ctas+1]  a persistent block's segments are contiguous
    uint32_t rows, segs, ctas;
    // The step's new tokens, in the caller's row order (kv_a rows): what the append writes.  Usually the same rows as
    // the query rows above; a step that routes long chunks to the prefill path keeps them here but not among the
    // query rows, which then carry the index of their row in the caller's q / out tensors.
    uint32_t app_rows;
    const uint32_t* app_pos;        // [app_rows]  global position (RoPE)
    const uint64_t* app_slot;       // [app_rows]  destination token slot
    const uint32_t* att_row;        // [rows]  query row -> row of the caller's q / out (nullptr: the same index)
};

}  // namespace mla
