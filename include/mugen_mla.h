/*
 * mugen_mla.h — C ABI of the B200 (sm_100a) implementation of Mugen's MLA absorbed-attention
 * decode path over its compressed latent KV cache.
 *
 * This is the drop-in boundary.  The reference has no FFI layer for this path: it is private
 * C++ inside mugen::TransformerModel::Impl.  Each entry point below therefore cites the piece
 * of reference code whose job it takes over (paths relative to the reference tree).  Plain
 * pointers and sizes only; a CUDA stream travels as void* (cudaStream_t).  All functions
 * return MLA_OK (0) or an error code; mla_last_error() gives the text.  There is no CPU
 * fallback: without a CUDA device mla_create fails.
 *
 * Element types: the latent cache, q, kv_a and the output use one storage type per context,
 * IEEE half (the reference's mugen::f16, include/mugen/core/types.h:10) or bfloat16.
 *
 * Latent cache row (src/core/model/transformer.cpp:3396-3400): 576 values per token per layer
 * = c_kv[512] (RMS-normalised) followed by k_rope[64] (RoPE applied).  Rows live in fixed
 * pages of 64 tokens; a page id names the same slot range in every layer.
 *
 * Threading: one host thread per context; calls are stream-ordered and asynchronous.
 */
#ifndef MUGEN_MLA_H
#define MUGEN_MLA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mla_ctx mla_ctx;

enum {
    MLA_OK = 0,
    MLA_ERR_INVALID = 1,      /* bad argument */
    MLA_ERR_CUDA = 2,         /* a CUDA runtime/driver call failed */
    MLA_ERR_NO_PAGES = 3,     /* page pool exhausted */
    MLA_ERR_CAPACITY = 4,     /* position beyond max_seq_len, or too many rows/sequences */
    MLA_ERR_STATE = 5,        /* call out of order (e.g. decode without step_begin) */
    MLA_ERR_DEVICE = 6,       /* a kernel reported a fault through the status word */
    MLA_ERR_UNSUPPORTED = 7   /* shape or type this build does not handle */
};

enum { MLA_DTYPE_F16 = 0, MLA_DTYPE_BF16 = 1 };

/* Weight encodings accepted by mla_set_layer_weights: GGML type ids as the reference's
 * dequant_weight_row understands them (src/core/model/transformer.cpp:2489-2534,
 * src/model/ggml_types.h:12-40), plus BF16. */
enum { MLA_W_F16 = 1, MLA_W_Q4_0 = 2, MLA_W_Q8_0 = 8, MLA_W_BF16 = 30 };

/* Split-KV attention kernel family (mla_config.kernel).  AUTO picks PAIR128 when n_heads is a multiple of
 * 128 (SM pairs, tcgen05.mma.cta_group::2, 128-token tiles), TCGEN05_T16 up to 16 heads (tcgen05 in the
 * transposed form: the tokens of a page are the rows of the tile, groups of 16 heads its columns) and TCGEN05 for
 * every other head count (one SM per group of up to 64 heads).  MMA (mma.sync m16n8k16, any head count) stays selectable.  All give
 * the same results within the attention tolerance; each is bit-reproducible from run to run. */
enum { MLA_KERNEL_AUTO = 0, MLA_KERNEL_MMA = 1, MLA_KERNEL_TCGEN05 = 2, MLA_KERNEL_TCGEN05_PAIR128 = 3,
       MLA_KERNEL_TCGEN05_T16 = 4 };

/* Shape contract: the MLA fields of mugen::ModelConfig (src/core/model/transformer.h:65-79)
 * plus the paged-pool geometry the reference lacks (it keeps one contiguous
 * [max_seq_len][576] buffer per layer, transformer.cpp:3396-3407). */
typedef struct mla_config {
    uint32_t n_layers;
    uint32_t n_heads;
    uint32_t kv_lora_rank;        /* must be 512 */
    uint32_t qk_nope_head_dim;    /* must be 128 */
    uint32_t qk_rope_head_dim;    /* must be 64  */
    uint32_t v_head_dim;          /* must be 128 */
    float    rope_theta;
    float    rms_norm_eps;
    float    rope_scaling_factor; /* YaRN factor; <= 1 means plain RoPE */
    uint32_t rope_original_ctx;
    uint32_t max_seq_len;         /* per-sequence capacity in tokens */
    uint32_t page_tokens;         /* must be 64 */
    uint32_t n_pages;             /* pages in the pool (each page spans all layers) */
    uint32_t max_seqs;            /* live sequences */
    uint32_t max_rows;            /* query rows (new tokens) per step; 0 -> max_seqs */
    uint32_t dtype;               /* MLA_DTYPE_* */
    int32_t  device;              /* CUDA device ordinal */
    uint32_t kernel;              /* MLA_KERNEL_* */
    uint32_t max_position;        /* highest global position + 1 (rotary table rows);
                                     0 -> max_seq_len.  Larger than max_seq_len only for
                                     KV-range shards, whose rows start at a base position */
} mla_config;

/* ---- lifetime ------------------------------------------------------------------------- */

/* Replaces model-init steps: KVCache::create (src/core/memory/kv_cache.cpp:146-159; same
 * validation messages), the per-layer latent buffer allocation (transformer.cpp:3396-3407)
 * and the score scratch (transformer.cpp:3411-3412). */
int mla_create(const mla_config* cfg, mla_ctx** out);
void mla_destroy(mla_ctx* ctx);
/* Text of the last error on this context (or of the last failed mla_create when ctx is NULL). */
const char* mla_last_error(const mla_ctx* ctx);
/* Reads and clears the device status word that kernels set instead of trapping
 * (0 = clean).  Synchronises the given stream. */
int mla_status(mla_ctx* ctx, void* stream, uint32_t* device_status);

/* Registers W_UK and W_UV, each (n_heads*128) x 512 row-major in `w_type`, and the c_kv
 * RMSNorm weight [512] in the context dtype, all HOST pointers.  Replaces the k_b / v_b /
 * kv_a_norm loading and split (transformer.cpp:3148-3221) and the per-call
 * dequant_weight_row (:2489-2534): quantised rows are decoded once, here. Unknown types are
 * rejected (the reference zero-fills them with a warning, :2529-2533). */
int mla_set_layer_weights(mla_ctx* ctx, uint32_t layer, const void* w_uk, const void* w_uv,
                          uint32_t w_type, const void* kv_norm);

/* ---- sequences: the KVCache bookkeeping contract ---------------------------------------- */
/* The reference cache holds ONE implicit sequence and, for MLA, is only a length counter
 * (kv_cache.h:20-47; kv_cache.cpp:281-285, 313-321, 343-357).  Here every call names a
 * sequence. */
int mla_seq_create(mla_ctx* ctx, uint32_t* seq_id);
int mla_seq_free(mla_ctx* ctx, uint32_t seq_id);
/* KVCache::seq_len (kv_cache.cpp:281-285). */
int mla_seq_len(const mla_ctx* ctx, uint32_t seq_id, uint32_t* len);
/* KVCache::advance_seq_len (kv_cache.cpp:355-357); rows must have been appended. */
int mla_advance(mla_ctx* ctx, uint32_t seq_id, uint32_t n);
/* KVCache::truncate (kv_cache.cpp:313-321): frees whole pages past new_len, keeps stale rows
 * inside the last page.  Unlike the reference it never grows: new_len > seq_len is an error. */
int mla_truncate(mla_ctx* ctx, uint32_t seq_id, uint32_t new_len);
/* The rollback of a speculative-decode step for many sequences at once (reference: USPPScheduler::decode_step,
 * src/core/scheduler/uspp_scheduler.cpp:222-237, and the CLI loop, src/cli/main.cpp:658-684): the verify pass
 * appended K+1 rows per sequence (a step with n_new = K+1); of these only the accepted ones stay.  For every listed
 * sequence whose seq_len exceeds keep_lens[i] the length is cut to keep_lens[i] (whole pages past it go back to
 * the pool); a sequence already at or below its keep length is left alone, as the reference's guard
 * `seq_len() > keep_len` does.  All-or-nothing: unknown ids are reported before anything is cut. */
int mla_rollback(mla_ctx* ctx, uint32_t n_seq, const uint32_t* seq_ids, const uint32_t* keep_lens);
/* KVCache::clear (kv_cache.cpp:343-353): returns every page of the sequence. */
int mla_clear(mla_ctx* ctx, uint32_t seq_id);
/* Global position of the sequence's local row 0 (default 0).  A KV-range shard of a long
 * sequence stores rows [base, base+n) locally; RoPE still uses the global position. */
int mla_seq_set_base(mla_ctx* ctx, uint32_t seq_id, uint32_t base_pos);
/* Number of free pages in the pool. */
int mla_free_pages(const mla_ctx* ctx, uint32_t* n);
/* Test/bench aid: permute the free list with a seeded shuffle so block tables come out as a
 * random permutation of physical pages. */
int mla_shuffle_free_pages(mla_ctx* ctx, uint64_t seed);
/* Copies the block table (physical page ids) of a sequence to `pages` (capacity `cap`). */
int mla_seq_pages(const mla_ctx* ctx, uint32_t seq_id, uint32_t* pages, uint32_t cap,
                  uint32_t* n_pages);

/* ---- explicit-position calls: the reference's own call shapes, batched ------------------- */

/* Steps G+H of the decode driver (transformer.cpp:3930-3987; batched twin :1263-1323):
 * RMSNorm(c_kv)*w, YaRN/NeoX RoPE(k_rope, positions[r]) and the scatter of row r to
 * (seq_ids[r], positions[r]) of `layer`.  kv_a: DEVICE [n][576].  seq_ids/positions: HOST.
 * Bit-exact with the reference arithmetic.  Allocates pages on demand; does not move seq_len. */
int mla_append_rows(mla_ctx* ctx, uint32_t layer, uint32_t n, const uint32_t* seq_ids,
                    const uint32_t* positions, const void* kv_a, void* stream);

/* cpu_mla_attention (transformer.cpp:2539-2623) for n query rows at once: row r attends rows
 * [0, attend_lens[r]) of sequence seq_ids[r].  q: DEVICE [n][n_heads][192] (post-RoPE, nope
 * first), out: DEVICE [n][n_heads][128].  seq_ids/attend_lens: HOST. */
int mla_attend_rows(mla_ctx* ctx, uint32_t layer, uint32_t n, const uint32_t* seq_ids,
                    const uint32_t* attend_lens, const void* q, void* out, void* stream);

/* ---- decode-step scheduler ------------------------------------------------------------- */
/* One step = for every listed sequence, n_new[i] new tokens (NULL = 1 each: plain decode;
 * >1: a prefill chunk, causal; 0: the sequence takes no token here but still answers the step's
 * query with one row attending its seq_len rows — a KV-range shard that does not own the tail;
 * its kv_a row is ignored) at positions seq_len .. seq_len+n_new-1.  step_begin reserves
 * pages, balances the KV ranges over the SMs and uploads the step's metadata once; the
 * per-layer calls then take only data pointers.  Ordering contract of the reference driver
 * (transformer.cpp:3702, 3980-3996, 4401-4403): per layer append THEN attend over
 * seq_len + (row's offset) + 1 rows; counters advance once, after all layers (step_end). */
int mla_step_begin(mla_ctx* ctx, uint32_t n_seq, const uint32_t* seq_ids, const uint32_t* n_new,
                   void* stream);
/* kv_a: DEVICE [rows][576], rows ordered by sequence then position. */
int mla_step_append(mla_ctx* ctx, uint32_t layer, const void* kv_a, void* stream);
/* q: DEVICE [rows][n_heads][192]; out: DEVICE [rows][n_heads][128]. */
int mla_step_attend(mla_ctx* ctx, uint32_t layer, const void* q, void* out, void* stream);
/* append + attend for `n_layers` consecutive layers in one call (an attention stack with nothing
 * between its layers, or a caller that has all layers' inputs ready): kv_a DEVICE
 * [n_layers][rows][576], q DEVICE [n_layers][rows][n_heads][192], out DEVICE
 * [n_layers][rows][n_heads][128].  Same kernels and order as the per-layer calls. */
int mla_step_layers(mla_ctx* ctx, uint32_t layer_begin, uint32_t n_layers, const void* kv_a,
                    const void* q, void* out, void* stream);
/* Same two calls with HOST buffers: copies kv_a and q in, runs append + attend on `stream`, copies
 * out back.  Page-locked caller buffers are copied directly on two copy streams of the context, so
 * the next layer's inputs and the previous layer's outputs move while a layer computes; the call
 * returns without waiting, the host buffers must hold their data when it is made, and out_host is
 * complete when mla_step_end returns.  Pageable buffers are staged through page-locked memory
 * inside the context and the call returns when out_host is filled. */
int mla_step_layer_host(mla_ctx* ctx, uint32_t layer, const void* kv_a_host, const void* q_host,
                        void* out_host, void* stream);
int mla_step_end(mla_ctx* ctx);
/* Rows in the current step and the number of KV segments they were split into. */
int mla_step_info(const mla_ctx* ctx, uint32_t* rows, uint32_t* segments);

/* How the planner spread the last planned step over the persistent attention workers (SM pairs or SMs): their
 * number and the fewest / most cache pages any of them walks.  A balanced ragged batch has max - min <= one tile. */
int mla_step_balance(const mla_ctx* ctx, uint32_t* workers, uint32_t* min_pages, uint32_t* max_pages);

/* ---- KV-range sharding of one long sequence ----------------------------------------------- */
/* Per-head partial softmax state of this shard for every row of the current step:
 * partial DEVICE float [rows][n_heads][514] = (m, l, acc[512]) with m the running maximum of
 * score*log2(e)/sqrt(192), l = sum 2^(s-m), acc = sum 2^(s-m) * c_kv.  A shard with no rows
 * to attend emits (-inf, 0, 0). */
int mla_step_attend_partial(mla_ctx* ctx, uint32_t layer, const void* q, float* partial,
                            void* stream);
/* The same with the append of the step's new rows done by the same launch that absorbs q (the fused form of
 * mla_step_append + mla_step_attend_partial, as mla_step_layer is for the unsharded step).  kv_a may be NULL on a
 * GPU whose shard takes no new row in this step (only the owner of the tail range appends: reference
 * transformer.cpp:3930-3987 writes one row per layer and step). */
int mla_step_layer_partial(mla_ctx* ctx, uint32_t layer, const void* kv_a, const void* q, float* partial,
                           void* stream);
/* Log-sum-exp merge of n_parts such partials (DEVICE float [n_parts][rows][n_heads][514],
 * e.g. the result of an all-gather) followed by the W_UV projection
 * (transformer.cpp:2610-2620).  out: DEVICE [rows][n_heads][128]. */
int mla_merge_partials(mla_ctx* ctx, uint32_t layer, uint32_t n_parts, uint32_t rows,
                       const float* partials, void* out, void* stream);

/* q-side RoPE (reference: step E of the decode driver, transformer.cpp:3882-3921, a CPU loop between two GPU
 * round trips).  in_kernel = 1: q is passed as the W_q projection left it and the absorb kernel rotates the last
 * 64 dims of every head with the row's position (NeoX pairs, YaRN frequencies, the same table and rounding as the
 * k_rope rotation of the append; bit-exact against the reference loop).  in_kernel = 0 (default): q arrives
 * rotated, which is cpu_mla_attention's own contract.  Rows of a step take the position of their new token,
 * mla_attend_rows rows the last attended position; steps with query-only rows (n_new = 0) are refused while on. */
int mla_set_q_rope(mla_ctx* ctx, int in_kernel);

/* ---- introspection used by benchmarks --------------------------------------------------- */
/* Kernel launches issued by this context since creation. */
int mla_launch_count(const mla_ctx* ctx, uint64_t* n);
/* Device timing of the split-KV attention kernel alone: while enabled, launches of that kernel
 * are bracketed by CUDA events on the launching stream (up to 8192 launches are kept).  on = 1
 * brackets every launch, on = N > 1 every N-th one: an event between two kernels keeps the second
 * from becoming resident while the first drains (the kernels of a step are launched as programmatic
 * dependents), so a sparse sample disturbs the step it measures less.
 * mla_profile_read synchronises those events and returns launches and their summed duration,
 * then clears the record. */
int mla_profile_enable(mla_ctx* ctx, int on);
int mla_profile_read(mla_ctx* ctx, uint32_t* launches, float* total_ms);
/* Name of the attention kernel family in use ("mma", "tcgen05", "tcgen05-pair128"). */
const char* mla_kernel_name(const mla_ctx* ctx);
/* Reads `n` latent rows [row_begin, row_begin+n) of (layer, seq) back to HOST memory. */
int mla_read_rows(mla_ctx* ctx, uint32_t layer, uint32_t seq_id, uint32_t row_begin, uint32_t n,
                  void* host_out, void* stream);
/* Writes `n` ready-made latent rows (already normalised / rotated) from DEVICE memory into
 * (layer, seq) starting at row_begin, allocating pages: bulk cache fill for benchmarks and
 * for restoring a saved cache. */
int mla_write_rows(mla_ctx* ctx, uint32_t layer, uint32_t seq_id, uint32_t row_begin, uint32_t n,
                   const void* dev_rows, void* stream);

/* ---- the projections around the attention: a whole attention block, hidden in -> hidden out ---------------- */
/* Replaces steps A-D, F, J and K of the reference's MLA decode driver (src/core/model/transformer.cpp:3849-3929,
 * 4002-4015; kernels rms_norm, matvec_f16, elementwise_add, src/metal/kernel_sources.h:55-98, 264-312, 357-366):
 *   hidden2 = RMSNorm(hidden) * attn_norm
 *   q       = W_q_b . RMSNorm(W_q_a . hidden2) * q_a_norm        (q_lora_rank > 0: DeepSeek-V3)
 *           = W_q . hidden2                                       (q_lora_rank = 0: V2-Lite)
 *   kv_a    = W_kv_a_mqa . hidden2                                (feeds the append)
 *   hidden += W_o . attention output
 * Every projection stores 16-bit results with float accumulation, as the reference's kernels do.  All weights are
 * HOST pointers in the context's storage type, row-major as GGUF holds them (one output per row):
 *   attn_norm [E], q_a [q_lora_rank][E], q_a_norm [q_lora_rank], q_b [n_heads*192][q_lora_rank] (or q [n_heads*192][E]
 *   with q_lora_rank = 0; unused pointers NULL), kv_a_mqa [576][E], wo [E][n_heads*128]. */
typedef struct mla_block_weights {
    uint32_t embedding_length;     /* E, a multiple of 8 */
    uint32_t q_lora_rank;          /* 0: full q projection */
    const void* attn_norm;
    const void* q_a;
    const void* q_a_norm;
    const void* q_b;
    const void* q;
    const void* kv_a_mqa;
    const void* wo;
} mla_block_weights;
int mla_set_block_weights(mla_ctx* ctx, uint32_t layer, const mla_block_weights* w);
/* Steps A-D and F for `rows` tokens: hidden DEVICE [rows][E] -> q DEVICE [rows][n_heads][192] (BEFORE its RoPE: pass it
 * to the attention with mla_set_q_rope(ctx, 1), or rotate it yourself) and kv_a DEVICE [rows][576]. */
int mla_block_project_in(mla_ctx* ctx, uint32_t layer, uint32_t rows, const void* hidden, void* q, void* kv_a, void* stream);
/* Steps J and K: hidden DEVICE [rows][E] += W_o . attn_out (DEVICE [rows][n_heads][128]). */
int mla_block_project_out(mla_ctx* ctx, uint32_t layer, uint32_t rows, const void* attn_out, void* hidden, void* stream);
/* The whole attention block of one layer for the rows of the open step: project in, append + attend (the kernels of
 * mla_step_layers), project out; hidden DEVICE [rows][E] is updated in place.  Needs mla_set_q_rope(ctx, 1). */
int mla_step_block(mla_ctx* ctx, uint32_t layer, void* hidden, void* stream);

/* ---- weight ingestion from a GGUF model file --------------------------------------------------------- */
/* Replaces, for this path, the reference's GGUF loading: the MLA metadata keys (src/core/model/transformer.cpp:
 * 2951-3011; parser src/model/gguf_parser.cpp:158-330) and the per-layer attn_k_b / attn_v_b tensors or the split
 * of a merged attn_kv_b whose rows per head are [qk_nope rows | v_head_dim rows] (transformer.cpp:3178-3221);
 * F32 norm weights become 16-bit at load as in the reference (:2850-2869).  The file is memory-mapped; no CUDA
 * call is made until mla_gguf_register.  Errors: mla_gguf_last_error() (per thread). */
typedef struct mla_gguf mla_gguf;
typedef struct mla_gguf_info {
    uint32_t n_layers, n_heads, embedding_length, context_length;
    uint32_t kv_lora_rank, q_lora_rank, qk_nope_head_dim, qk_rope_head_dim, v_head_dim, rope_original_ctx;
    float rope_theta, rope_scaling_factor, rms_norm_eps;
} mla_gguf_info;
int mla_gguf_open(const char* path, mla_gguf** out);
void mla_gguf_close(mla_gguf* g);
const char* mla_gguf_last_error(void);
int mla_gguf_get_info(const mla_gguf* g, mla_gguf_info* info);
/* Copies the model's shape, RoPE and epsilon fields into cfg (max_seq_len too when it is 0: the file's
 * context_length, or 8192 as the reference defaults); pool geometry, dtype and kernel stay the caller's. */
int mla_gguf_fill_config(const mla_gguf* g, mla_config* cfg);
/* One layer's W_UK and W_UV ((n_heads*128) x 512 each, after the split of a merged tensor) in their MLA_W_*
 * encoding, as HOST bytes, and optionally its kv_a norm as half bits.  w_uk / w_uv may be NULL to query bytes_each. */
int mla_gguf_layer_weights(mla_gguf* g, uint32_t layer, void* w_uk, void* w_uv, size_t capacity_each, uint32_t* w_type,
                           size_t* bytes_each, uint16_t* kv_norm_f16);
/* mla_set_layer_weights for every layer of the file (ctx_dtype = the context's MLA_DTYPE_*, for the norm weights). */
int mla_gguf_register(mla_ctx* ctx, mla_gguf* g, uint32_t ctx_dtype);

/* Failure-path self-test (no reference counterpart).  Launches one block whose threads wait on a barrier that
 * nothing completes: after `limit_cycles` SM cycles (e.g. 1,000,000: about half a millisecond) the wait gives up,
 * raises the ST_WAIT_TIMEOUT bit (value 4) in the context's device status word, the block frees its tensor memory
 * and returns.  This is the mechanism every kernel here uses instead of hanging or trapping; a following
 * mla_status() returns MLA_ERR_DEVICE with device_status = 4 and clears the word, and the context stays usable.
 * waited_cycles (HOST pointer, may be NULL) receives how long the block waited.  Synchronises the stream. */
int mla_selftest_wait_timeout(mla_ctx* ctx, uint64_t limit_cycles, void* stream, uint32_t* waited_cycles);

/* ---- for callers that may not allocate ------------------------------------------------------ */
/* No counterpart in the reference.  Absorbed MLA attention of one query row over one CONTIGUOUS
 * latent cache, without a context and without any allocation: no cudaMalloc, cudaFree or
 * allocating library routine is called, now or later, and nothing is copied from host memory.
 * For callers whose device memory is owned by someone else's pool, or that must not trigger
 * cudaMalloc's device-wide synchronisation.  Intermediates live in an 8.2 MiB array built into the
 * library (held on every GPU the process uses until exit), hence the limits n_heads <= 128 and
 * seq_len <= 65536; larger sizes return MLA_ERR_CAPACITY.  All pointers are DEVICE pointers in `dtype`:
 *   q     [n_heads][192]  post-RoPE query (nope first)     out  [n_heads][128]
 *   cache [seq_len][576]  exactly seq_len rows: nothing behind the last row is read
 *   w_uk, w_uv  (n_heads*128) x 512 row-major, as the reference keeps them (transformer.cpp:3178-3221)
 * The first call on a device resolves the array's address (cudaGetSymbolAddress) and sets kernel
 * attributes on that device; make that first call outside any stream capture.  Calls that overlap
 * on one GPU race on the shared array: serialise them.  Asynchronous on `stream`.  The device status
 * word of the context entry points has no reader here: a fault inside a kernel of this path is not
 * reported (argument errors are, through the return code).  mla_noalloc_last_error() gives the text
 * of the calling thread's last failure. */
int mla_attention_noalloc(uint32_t dtype, uint32_t n_heads, uint32_t seq_len, const void* q,
                          const void* cache, const void* w_uk, const void* w_uv, void* out,
                          void* stream);
const char* mla_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* MUGEN_MLA_H */
