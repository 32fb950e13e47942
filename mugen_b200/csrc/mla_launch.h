// Host-callable launchers of the MLA kernels (internal to the library; the public surface is
// include/mugen_mla.h).
#pragma once

#include "mla_common.cuh"

namespace mla {

void launch_append(int dtype, const void* kv_a, void* layer_pool, uint64_t pool_slots,
                   const void* norm_w, const float* cos_sin, uint32_t cs_rows, float eps,
                   const StepMeta& m, uint32_t* status, cudaStream_t st);

void launch_write_rows(const void* src, void* layer_pool, uint64_t pool_slots, const uint32_t* table,
                       uint32_t row_begin, uint32_t n, uint32_t* status, cudaStream_t st);

// w_uk_t: W_UK transposed per head, [H][512][128].
void launch_absorb(int dtype, const void* q, const void* w_uk_t, void* q_abs, uint32_t rows,
                   uint32_t H, cudaStream_t st);

// Split-KV attention, legacy tensor path (mma.sync m16n8k16): grid (segments, ceil(H/16)).
// Returns a cudaError_t-compatible code from the launch configuration.
int launch_decode_mma(int dtype, const void* q_abs, const void* layer_pool, uint32_t n_pages,
                      const StepMeta& m, float* recs, uint32_t H, uint32_t* status, cudaStream_t st);
int decode_mma_configure();   // the *_configure() functions set kernel attributes on the CURRENT device: once per device

// Split-KV attention on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM,
// cache tiles staged by TMA): grid (persistent blocks, ceil(H/64)).  tmaps points at the context's
// host CUtensorMap array (kMap* below); this kernel uses kMapPoolPage and kMapQueries.
int launch_decode_tc5(int dtype, const void* tmaps, uint32_t layer, uint32_t n_pages, const StepMeta& m,
                      float* recs, uint32_t H, uint32_t* status, cudaStream_t st);
int decode_tc5_configure();   // sets the kernel's attributes on the current device

// The transposed form for narrow head counts (mla_decode_tc5_t16.cu): tokens are the M rows, groups of 16 heads the N
// columns; grid (persistent blocks, ceil(H/16)).  Uses kMapPoolV, kMapPoolSub and kMapQueries16.
int launch_decode_tc5_t16(int dtype, const void* tmaps, uint32_t layer, uint32_t n_pages, const StepMeta& m, float* recs,
                          uint32_t H, uint32_t* status, cudaStream_t st);
int decode_tc5_t16_configure();

// Tensor maps a context builds once (mla_api.cu, make_tensor_maps), by index into its array.
enum : int {
    kMapPoolSub = 0,      // cache pool [layers][slots][576]: box 64 values x 64 tokens (one K sub-tile)
    kMapPoolV = 1,        // cache pool, whole-row view (64 values, slots, 9 chunks, layers): box 64 tokens x 2 chunks
    kMapQueries = 2,      // absorbed queries, whole-row view: box 64 head rows x 9 chunks
    kMapPoolPage = 3,     // cache pool, whole-row view: box 64 tokens x 9 chunks (one page in one instruction)
    kMapQueries16 = 4,    // absorbed queries, whole-row view: box 16 head rows x 9 chunks
    kMapCount = 5
};

// The same on a pair of SMs (cluster of 2, tcgen05.mma.cta_group::2), 128-token tiles (two pages per score
// MMA series): grid (2 x persistent pairs, ceil(H/128)).  Uses kMapPoolSub, kMapPoolV, kMapQueries and the
// layer's pool slice.
int launch_decode_tc5_pair128(int dtype, const void* tmaps, const void* layer_pool, uint32_t layer, uint32_t n_pages,
                              const StepMeta& m, float* recs, uint32_t H, uint32_t prefetch_tiles, const void* next_weights,
                              uint32_t next_weights_bytes, uint32_t* status, cudaStream_t st);
int decode_tc5_pair128_configure();

void launch_merge(int dtype, const float* recs, const uint32_t* row_seg_begin, uint32_t n_parts,
                  const void* w_uv, void* out, float* exported, uint32_t rows, uint32_t H,
                  cudaStream_t st, const uint32_t* att_row = nullptr);
int merge_mma_configure();

// Absorb on tcgen05 (one block per head and 64 rows); w_map: host CUtensorMap over the layer's W_UK^T,
// [H*512 d][128 i], box 64 i x 256 d, 128-byte swizzle.  With kv_a != nullptr the same launch appends the step's
// new rows (launch_append's arguments) in extra blocks.  rotate_q: q arrives before its RoPE; the kernel rotates
// the last 64 dims of every head with the row's position (m.row_pos) and the cos/sin table.  append_waits: kv_a may
// have been written by the kernel launched just before this one (the append blocks then wait for it before reading).
int launch_absorb_tc5(int dtype, const void* q, const void* w_map, void* q_abs, uint32_t rows, uint32_t H, const void* kv_a,
                      void* layer_pool, uint64_t pool_slots, const void* norm_w, const float* cos_sin, uint32_t cs_rows,
                      float eps, const StepMeta& m, bool rotate_q, bool append_waits, uint32_t* status, cudaStream_t st);
int absorb_tc5_configure();

// The same merge + projection on tcgen05 (one block per head and 64 rows); w_map: host CUtensorMap over the
// layer's W_UV, [H*128 outputs][512 dims], box 64 dims x 128 outputs, 128-byte swizzle.
int launch_merge_tc5(int dtype, const float* recs, const uint32_t* row_seg_begin, uint32_t n_parts, const void* w_map,
                     void* out, uint32_t rows, uint32_t H, const uint32_t* att_row, uint32_t* status, cudaStream_t st);
int merge_tc5_configure();

// Dense projection C = A . W^T on tcgen05 (mla_gemm_tc5.cu).  A [M][K] pitch lda, W [N][K] pitch ldw (the reference's
// matvec weight layout), 16-bit DEVICE operands.  partial == nullptr: C in the storage type to `out`; else float
// partials [splits][M][N] to be finished by launch_gemm_finalize (mode 0 store, 1 RMSNorm with w / eps, 2 residual
// add of res).  Return: cudaError_t value, or -1 when a tensor map cannot be built.
int launch_gemm_tc5(int dtype, const void* A, uint32_t lda, const void* W, uint32_t ldw, uint32_t M, uint32_t N, uint32_t K,
                    void* out, float* partial, uint32_t splits, uint32_t* status, cudaStream_t st);
int launch_gemm_finalize(int dtype, const float* partial, uint32_t splits, uint32_t M, uint32_t N, int mode, const void* w,
                         float eps, const void* res, void* out, cudaStream_t st);
int launch_rmsnorm_rows(int dtype, const void* x, const void* w, void* y, uint32_t rows, uint32_t N, float eps, cudaStream_t st);
uint32_t gemm_tc5_splits(uint32_t M, uint32_t N, uint32_t K, uint32_t sm_count);   // K slices that fill the SMs once
int gemm_tc5_configure();

// Chunked prefill (mla_prefill_tc5.cu): gather of a sequence's latent rows into a contiguous buffer, rotation of a
// chunk's query rows, and causal flash attention of one chunk over expanded keys / values (see the file's header).
int launch_gather_rows(const void* layer_pool, uint64_t pool_slots, const uint32_t* table, uint32_t n, void* dst, uint32_t* status,
                       cudaStream_t st);
int launch_rotate_q_rows(int dtype, const void* q_in, void* q_out, uint32_t rows, uint32_t H, uint32_t pos0, const float* cos_sin,
                         uint32_t cs_rows, uint32_t* status, cudaStream_t st);
int launch_prefill_tc5(int dtype, const void* q, uint32_t q_rows_total, uint32_t q_row0, uint32_t n_new, uint32_t start,
                       const void* kx, const void* vx, const void* latent, void* out, uint32_t H, uint32_t* status, cudaStream_t st);
int prefill_tc5_configure();

// One block that waits `limit_cycles` on a barrier nothing completes, raises ST_WAIT_TIMEOUT in *status, frees its
// tensor memory and returns; report[0] = 0 when the wait gave up, report[1] = cycles waited.
void launch_wait_timeout_selftest(long long limit_cycles, uint32_t* status, uint32_t* report, cudaStream_t st);

}  // namespace mla
