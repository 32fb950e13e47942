// Split-KV absorbed MLA attention for 128-head groups on a PAIR of SMs, 128-token super-tiles
// (thread-block cluster of 2, tcgen05.mma.cta_group::2), sm_100a.
//
// Same division of labour as mla_decode_tc5_pair.cu (each block: 64 heads, its 256 latent dims of
// V, O^T for its dims x all 128 heads), but a tile is TWO pages and the pair's score MMA has
// N = 128: block r stages the whole K of page r (the B operand's rows 64r .. 64r+63).  Measured on
// B200 with four issuing warps, a cta_group::2 M128 N64 K16 MMA occupies the tensor pipe for 33
// cycles and the N128 one for 44, so the 72 score MMAs of two pages (2,380 cycles) become 36
// (1,580); with the 16 value MMAs (M256 N128 K16, 77 cycles each) a 128-token tile needs ~2,800
// pipe cycles instead of ~3,600, which is below the time HBM needs to deliver it.
//
// Shared memory is exactly full (Q' 72 KB, K 72 KB, V 64 KB, P 16 KB, 3 KB of barriers and
// scratch), so K and V are not double-buffered as a whole.  Every K sub-tile [64 tokens][64 dims]
// and every V buffer [page][128-dim chunk] has its own "full" barrier and is re-loaded as soon as
// the MMAs that read it have completed; the "empty" side is signalled per release round (K
// sub-tiles {0-3}, {4-7}, {8}; V per page) so that a producer thread pays one shared-memory round
// trip (~300 cycles while the MMAs stream their operands) per round, not per buffer.  The dynamic
// shared segment must start 1 KB-aligned because there is no slack to round up (checked; the
// status word says so if not).
//
// TMEM: O^T 2 x 128 columns; four partial score tiles of 64 columns, one per issuing warp (a warp
// waits ~50-100 cycles per MMA it issues, so four of them are needed to keep the pipe busy).  Each
// accumulator has ONE issuing thread and the softmax adds the partials in a fixed order, so the
// result is bit-reproducible from run to run and under any page permutation.  (A variant with two
// partials shared by two issuers each and the score tile double-buffered took the same time and
// lost that property: the order of the accumulations then depends on timing.)
//
// Warps: 0 K producer, 1-4 score issuers (sub-tiles {0,4,8} {1,5} {2,6} {3,7}), 5-6 value issuers
// (one per chunk), 7 V producer (+ optional linear L2 prefetch of later pages), 8-15 softmax.  The
// softmax computes its exponentials optimistically against the current reference maximum while the
// cluster round that tells whether any head of the pair must move its maximum is in flight; only
// in that rare case they are redone and O^T rescaled.  Waiting threads sleep in the barrier unit
// (try_wait with a time hint) rather than re-poll: shared-memory bandwidth is what the MMA operand
// fetches and the TMA fills compete for.  All waits are bounded.
//
// What bounds it, measured with clock64 and %globaltimer inside a traced build of the kernel: about
// 400k SM cycles per launch at batch 64 x ctx 16384 at an effective SM clock of 1.55 GHz, although
// nvidia-smi reports 1.97 GHz around a short run: the clock is throttled within the kernel, and
// variants of this kernel that need fewer or more cycles (prefetch on or off, polling hints, score
// double-buffering, producer layouts) all take the same 260-275 us.
#include "mla_launch.h"
#include "mla_tc5.cuh"

namespace mla {

namespace {

using namespace tc5;

constexpr int PAGES = 2;                            // pages per super-tile
constexpr int TILE = PAGES * kPage;                 // 128 tokens
constexpr int HG = 64;                              // heads per block (128 per pair)
constexpr int NSUB = kRow / 64;                     // 9
constexpr int SUB_BYTES = kPage * 128;              // 8,192: [64 tokens or heads][64 values]
constexpr int Q_BYTES = NSUB * SUB_BYTES;           // 73,728
constexpr int K_BYTES = NSUB * SUB_BYTES;           // 73,728: the whole K of this block's page
constexpr int VBUF_BYTES = 2 * SUB_BYTES;           // 16,384: 64 tokens x 128 dims (one page, one chunk)
constexpr int P_BYTES = HG * 128;                   // 8,192 per page
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + Q_BYTES;
constexpr int OFF_V = OFF_K + K_BYTES;                      // [page][chunk]
constexpr int OFF_P = OFF_V + PAGES * 2 * VBUF_BYTES;       // [page]
constexpr int OFF_MISC = OFF_P + PAGES * P_BYTES;
constexpr int MISC_BYTES = 3072;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES;           // 232,448 = all of it: no alignment slack
static_assert(SMEM_BYTES == 232448, "shared-memory plan must fill the 227 KB exactly");

// misc area layout (bytes from OFF_MISC)
constexpr int M_BAR = 0;          // mbarriers, 8 B each
constexpr int M_TMEM = 384;       // tmem base
constexpr int M_ABORT = 388;
constexpr int M_FLAG = 392;       // [2] "some head of the pair must move its maximum", by tile parity
constexpr int M_ALPHA = 512;      // [2][128] floats: scale factor per head of the pair, by tile parity
constexpr int M_HMAX = 1536;      // [4][64] floats: tile maximum of each token quarter per head
constexpr int M_LSUM = 1536;      // [3][64] floats: the other quarters' partial sums at the epilogue (the same
                                  // bytes as M_HMAX: a barrier of the softmax group separates the two uses)

constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_O = 0;       // 2 chunks x 128 head columns
constexpr uint32_t COL_S = 256;     // 4 partial score tiles x 64 columns

constexpr int N_QK = 4, N_PV = 2;
constexpr int NUM_THREADS = 32 * (2 + N_QK + N_PV + 8);   // 512
constexpr int SOFTMAX_THREADS = 256;
constexpr int PAIR_SOFTMAX_WARPS = 16;
constexpr float RESCALE_THRESHOLD = 8.0f;

// L2 prefetch (kernel argument prefetch_tiles, 0 = off): every block pulls "its" whole page towards L2 that many
// tiles ahead as ONE linear request of 73,728 contiguous bytes.  Each K sub-tile buffer is re-loaded as soon as the
// MMAs that read it complete and is needed again one tile later, so the re-load's latency sits on the tile loop:
// with few sequences per GPU (HBM far from saturated) turning an HBM miss into an L2 hit shortens the tile period
// (8 sequences: 47.7 -> 45.3 us per launch at distance 1; distances 2 and 4 queue more requests in front of the
// demand loads and lose again), while at batch 64, where HBM bandwidth is the co-limit, it changes nothing
// (267 -> 268 us), so the host turns it on only for short work lists.
constexpr int K_ROUNDS = (NSUB + N_QK - 1) / N_QK;   // 3: the issuers free sub-tiles {0-3}, {4-7}, {8} together
enum { B_QFULL = 0, B_QEMPTY, B_KFULL, B_KEMPTY = B_KFULL + NSUB, B_VFULL = B_KEMPTY + K_ROUNDS, B_VEMPTY = B_VFULL + 4,
       B_SFULL = B_VEMPTY + PAGES, B_SEMPTY, B_PFULL, B_PEMPTY, B_OFULL, B_SYNCA0, B_SYNCA1, B_SYNCB0, B_SYNCB1, B_COUNT };
static_assert(B_COUNT * 8 <= M_TMEM, "barriers overflow their area");


struct SegInfo {
    uint32_t row, page_begin, n_pages, n_tiles, n_tok;
};
__device__ __forceinline__ SegInfo load_seg(const StepMeta& m, uint32_t seg) {
    SegInfo s;
    s.row = m.seg_row[seg];
    s.page_begin = m.seg_page_begin[seg];
    const uint32_t pe = m.seg_page_end[seg];
    const uint32_t len = m.row_len[s.row];
    const uint32_t tb = s.page_begin * kPage, te = min(len, pe * kPage);
    s.n_tok = te > tb ? te - tb : 0;
    s.n_pages = (s.n_tok + kPage - 1) / kPage;
    s.n_tiles = (s.n_pages + PAGES - 1) / PAGES;      // super-tiles
    return s;
}

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
decode_tc5_pair128_kernel(const __grid_constant__ CUtensorMap map_sub, const __grid_constant__ CUtensorMap map_kv64,
                          const __grid_constant__ CUtensorMap map_q, const unsigned char* __restrict__ pool_layer,
                          uint32_t layer, uint32_t n_pages, StepMeta m, float* __restrict__ recs, uint32_t H,
                          float scale_log2, uint32_t prefetch_tiles, const unsigned char* __restrict__ next_weights,
                          uint32_t next_weights_bytes, uint32_t* __restrict__ status)
{
    extern __shared__ __align__(1024) unsigned char sm[];
    const uint32_t base = smem_u32(sm);
    const uint32_t sQ = base + OFF_Q, sK = base + OFF_K, sV = base + OFF_V, sP = base + OFF_P;
    const uint32_t sBar = base + OFF_MISC + M_BAR;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC + M_TMEM);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + M_ABORT);
    volatile uint32_t* need_flag = reinterpret_cast<volatile uint32_t*>(sm + OFF_MISC + M_FLAG);
    float* alpha_all = reinterpret_cast<float*>(sm + OFF_MISC + M_ALPHA);
    float* half_max = reinterpret_cast<float*>(sm + OFF_MISC + M_HMAX);
    float* l_other = reinterpret_cast<float*>(sm + OFF_MISC + M_LSUM);
    auto bar = [&](int i) { return sBar + 8u * uint32_t(i); };

    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t rank = cluster_rank();                 // 0 = pair leader (issues the MMAs)
    const uint32_t worker = blockIdx.x / 2;
    const uint32_t hpair = blockIdx.y * (2 * HG);        // first head of the pair's 128
    const uint32_t h0 = hpair + rank * HG;               // first head of this block's 64
    const uint32_t seg_begin = m.cta_seg_begin[worker], seg_end = m.cta_seg_begin[worker + 1];

    // The swizzled operand tiles need 1 KB alignment and the plan leaves no room to round up.
    // Both blocks of a pair see the same offset, so they take this exit together.
    grid_launch_dependents();
    if ((base & 1023u) != 0) {
        grid_dependency_wait();          // also this exit keeps the stream's "every kernel waits before it completes" chain
        if (tid == 0) atomicOr(status, ST_BAD_ALIGNMENT);
        return;
    }

    // one barrier per thread of warp 0 (31 of them): initialised in one step instead of 31 by a single thread
    if (warp == 0) {
        if (lane == 0) {
            *abort_flag = 0;
            need_flag[0] = 0;
            need_flag[1] = 0;
        }
        if (lane < B_COUNT) {
            const int i = int(lane);
            const uint32_t count = i == B_QFULL ? 1u
                                 : i == B_QEMPTY ? uint32_t(N_QK)
                                 : i < B_KEMPTY ? 1u                                                          // KFULL
                                 : i < B_VFULL ? uint32_t(min(N_QK, NSUB - N_QK * (i - B_KEMPTY)))           // KEMPTY rounds
                                 : i < B_VEMPTY ? 1u                                                          // VFULL
                                 : i < B_SFULL ? uint32_t(N_PV)                                               // VEMPTY
                                 : i == B_SFULL ? uint32_t(N_QK)
                                 : (i == B_PEMPTY || i == B_OFULL) ? uint32_t(N_PV)
                                 : uint32_t(PAIR_SOFTMAX_WARPS);                    // SEMPTY, PFULL, SYNCA0/1, SYNCB0/1
            mbar_init(bar(i), count);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    static_assert(B_COUNT <= 32, "one barrier per lane of the initialising warp");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    // both blocks' barriers must exist before either sends a remote arrive or a TMA completion
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    // The step's metadata was uploaded by a copy that the stream ordered before the step's first kernel, so it may be
    // read ahead of the wait: the chain of dependent loads that describes the first segment (segment -> row -> table
    // offset -> page ids) then overlaps the previous kernel's tail instead of delaying the first TMA.
    SegInfo seg0{};
    const uint32_t* tbl0 = nullptr;
    uint32_t page0[PAGES] = {0, 0};
    if (seg_begin < seg_end) {
        seg0 = load_seg(m, seg_begin);
        tbl0 = m.tables + m.seq_tbl_off[m.row_seq[seg0.row]] + seg0.page_begin;
        if (seg0.n_tiles) {
#pragma unroll
            for (int r = 0; r < PAGES; r++) page0[r] = tbl0[min(uint32_t(r), seg0.n_pages - 1)];
        }
    }
    auto seg_info = [&](uint32_t seg) -> SegInfo { return seg == seg_begin ? seg0 : load_seg(m, seg); };
    auto seg_table = [&](uint32_t seg, const SegInfo& si) -> const uint32_t* {
        return seg == seg_begin ? tbl0 : m.tables + m.seq_tbl_off[m.row_seq[si.row]] + si.page_begin;
    };
    // L2 is the point of coherence, so pulling cache lines towards it ahead of the wait is safe even for the page
    // that the append of this layer-step is still writing: the first tiles' loads then find their pages in L2.
    if (warp == N_QK + N_PV + 1 && lane == 0 && seg_begin < seg_end) {
        for (uint32_t jj = 0; jj < min(2u, seg0.n_tiles); jj++) {
            const uint32_t pgid = tbl0[min(PAGES * jj + rank, seg0.n_pages - 1)];
            if (pgid < n_pages) bulk_prefetch_l2(pool_layer + size_t(pgid) * (kPage * kRow * 2), kPage * kRow * 2);
        }
    }
    grid_dependency_wait();          // queries, new cache rows and the state records belong to earlier kernels until here

    // Page of super-tile j that block `r` stages as K (and whose tokens are columns 64r .. 64r+63 of
    // the score tile).  A segment with an odd page count repeats its last page in the second half:
    // finite data whose scores the softmax masks.
    auto page_of = [&](const uint32_t* tbl, const SegInfo& s, uint32_t j, uint32_t r) -> uint32_t {
        if (tbl == tbl0 && j == 0) return page0[r];
        const uint32_t i = min(PAGES * j + r, s.n_pages - 1);
        return tbl[i];
    };

    if (warp == 0) {
        // ===================== TMA producer for Q' and K =====================
        if (lane == 0) {
            const uint32_t leader_qfull = map_to_rank(bar(B_QFULL), 0);
            const uint32_t leader_kfull = map_to_rank(bar(B_KFULL), 0);
            uint32_t t = 0, nseg = 0;
            bool ok = true;
            for (uint32_t seg = seg_begin; seg < seg_end && ok; seg++) {
                const SegInfo s = seg_info(seg);
                if (s.n_tiles == 0) continue;
                const uint32_t* tbl = seg_table(seg, s);
                ok = mbar_wait<kSleep>(bar(B_QEMPTY), (nseg & 1) ^ 1, abort_flag, status);
                if (!ok) break;
                if (rank == 0) mbar_expect_tx(bar(B_QFULL), 2 * Q_BYTES);
                tma_load_3d_pair(sQ, &map_q, leader_qfull, 0, int(s.row * H + h0), 0);      // all 9 sub-tiles at once
                for (uint32_t j = 0; j < s.n_tiles && ok; j++, t++) {
                    uint32_t page = page_of(tbl, s, j, rank);
                    if (page >= n_pages) {
                        atomicOr(status, ST_BAD_PAGE);
                        page = 0;
                    }
                    const int slot0 = int(page * kPage);
                    // The score issuers release the sub-tiles in rounds ({0-3}, {4-7}, {8}); one wait per round
                    // instead of one per sub-tile: a shared-memory round trip costs this thread ~300 cycles while
                    // the MMAs stream their operands, and nine of them per tile made it the slowest stage.
#pragma unroll 1
                    for (int rd = 0; rd < K_ROUNDS && ok; rd++) {
                        ok = mbar_wait<kSleep>(bar(B_KEMPTY + rd), (t & 1) ^ 1, abort_flag, status);
                        if (!ok) break;
#pragma unroll 1
                        for (int c = N_QK * rd; c < min(N_QK * (rd + 1), NSUB); c++) {
                            if (rank == 0) mbar_expect_tx(bar(B_KFULL + c), 2 * SUB_BYTES);
                            tma_load_3d_pair(sK + c * SUB_BYTES, &map_sub, leader_kfull + 8 * c, 64 * c, slot0, int(layer));
                        }
                    }
                }
                nseg++;
            }
        }
    } else if (warp == N_QK + N_PV + 1) {
        // ===================== TMA producer for V =====================
        if (lane == 0) {
            const uint32_t leader_vfull = map_to_rank(bar(B_VFULL), 0);
            uint32_t t = 0;
            bool ok = true;
            for (uint32_t seg = seg_begin; seg < seg_end && ok; seg++) {
                const SegInfo s = seg_info(seg);
                if (s.n_tiles == 0) continue;
                const uint32_t* tbl = seg_table(seg, s);
                // tile 0 is demand-loaded right now; tiles 1 .. prefetch_tiles-1 have no earlier tile to ride on
                for (uint32_t jj = 1; jj < min(prefetch_tiles, s.n_tiles); jj++) {
                    const uint32_t pgid = page_of(tbl, s, jj, rank);
                    if (pgid < n_pages) bulk_prefetch_l2(pool_layer + size_t(pgid) * (kPage * kRow * 2), kPage * kRow * 2);
                }
                for (uint32_t j = 0; j < s.n_tiles && ok; j++, t++) {
                    if (prefetch_tiles > 0 && j + prefetch_tiles < s.n_tiles) {
                        const uint32_t pgid = page_of(tbl, s, j + prefetch_tiles, rank);
                        if (pgid < n_pages) bulk_prefetch_l2(pool_layer + size_t(pgid) * (kPage * kRow * 2), kPage * kRow * 2);
                    }
#pragma unroll 1
                    for (uint32_t pg = 0; pg < uint32_t(PAGES) && ok; pg++) {     // both chunk issuers release a page together
                        uint32_t page = page_of(tbl, s, j, pg);
                        if (page >= n_pages) page = 0;           // flagged by the K producer
                        ok = mbar_wait<kSleep>(bar(B_VEMPTY + pg), (t & 1) ^ 1, abort_flag, status);
                        if (!ok) break;
#pragma unroll 1
                        for (uint32_t ch = 0; ch < 2; ch++) {
                            const uint32_t v = 2 * pg + ch;
                            if (rank == 0) mbar_expect_tx(bar(B_VFULL + v), 2 * VBUF_BYTES);
                            // all 64 tokens of the page, this block's 128 dims of chunk ch = sub-tiles 4*ch + 2r, +1
                            tma_load_4d_pair(sV + v * VBUF_BYTES, &map_kv64, leader_vfull + 8 * v, 0, int(page * kPage),
                                             4 * int(ch) + 2 * int(rank), int(layer));
                        }
                    }
                }
            }
            // This thread's loads are all issued about a tile before the block finishes.  The next kernel but one of
            // the stream (the following layer's absorb) starts by streaming that layer's W_UK from HBM; pulling this
            // block's share of it towards L2 now turns that stream into L2 hits (the bytes move while the last tiles
            // compute and the partial states are merged).  Any thread of the grid could do it; this one is idle.
            if (next_weights != nullptr) {
                const uint32_t nblk = gridDim.x * gridDim.y, me = blockIdx.y * gridDim.x + blockIdx.x;
                const uint32_t share = ((next_weights_bytes + nblk - 1) / nblk + 15u) & ~15u;
                const uint32_t off = me * share;
                if (off < next_weights_bytes) bulk_prefetch_l2(next_weights + off, min(share, next_weights_bytes - off) & ~15u);
            }
        }
    } else if (warp <= N_QK + N_PV) {
        // ===================== MMA issuers (pair leader only) =====================
        if (rank == 0) {
            constexpr uint32_t IDESC_QK = instr_desc(Fmt<T>::v, 128, TILE, 0, 0);        // 64 head rows, 64 tokens per block
            constexpr uint32_t IDESC_PV = instr_desc(Fmt<T>::v, 256, 2 * HG, 1, 0);      // 128 dims per block
            constexpr uint32_t HI = desc_hi(1024);
            const bool is_qk = warp <= N_QK;
            const uint32_t part = is_qk ? warp - 1 : warp - 1 - N_QK;
            const uint32_t qk_a = desc_lo(sQ, 16), qk_b = desc_lo(sK, 16);
            const uint32_t pv_a = desc_lo(sV, SUB_BYTES), pv_b = desc_lo(sP, 16);
            uint32_t t = 0, nseg = 0;
            bool ok = true;
            for (uint32_t seg = seg_begin; seg < seg_end && ok; seg++) {
                const SegInfo s = seg_info(seg);
                if (s.n_tiles == 0) continue;
                if (is_qk) ok = mbar_wait<kSleepCluster>(bar(B_QFULL), nseg & 1, abort_flag, status);
                for (uint32_t j = 0; j < s.n_tiles && ok; j++, t++) {
                    if (is_qk) {
                        // sub-tiles part, part+4 (, part+8): partial scores into this warp's own 64 columns
                        ok = mbar_wait<kSleepCluster>(bar(B_SEMPTY), (t & 1) ^ 1, abort_flag, status);
                        if (!ok) break;
                        const uint32_t d = tmem + COL_S + part * (TILE / 2);
#pragma unroll 1
                        for (uint32_t c = part; c < uint32_t(NSUB); c += N_QK) {
                            ok = mbar_wait<kSleepCluster>(bar(B_KFULL + c), t & 1, abort_flag, status);
                            if (!ok) break;
                            tc_fence_after();
                            if (elect_one()) {
#pragma unroll
                                for (int k = 0; k < 4; k++)
                                    tc_mma_pair(d, qk_a + ((c * SUB_BYTES + k * 32) >> 4), HI, qk_b + ((c * SUB_BYTES + k * 32) >> 4),
                                                HI, IDESC_QK, (c == part && k == 0) ? 0u : 1u);
                                tc_commit_pair(bar(B_KEMPTY + c / N_QK));
                                if (c + N_QK >= uint32_t(NSUB)) {      // same thread as the MMAs it covers
                                    tc_commit_pair(bar(B_SFULL));
                                    if (j + 1 == s.n_tiles) tc_commit_pair(bar(B_QEMPTY));
                                }
                            }
                            __syncwarp();
                        }
                    } else {
                        // chunk `part` of O^T += V^T P^T over the tile's two pages
                        ok = mbar_wait<kSleepCluster>(bar(B_PFULL), t & 1, abort_flag, status);
#pragma unroll 1
                        for (uint32_t pg = 0; pg < uint32_t(PAGES) && ok; pg++) {
                            const uint32_t v = 2 * pg + part;
                            ok = mbar_wait<kSleepCluster>(bar(B_VFULL + v), t & 1, abort_flag, status);
                            if (!ok) break;
                            tc_fence_after();
                            const uint32_t fresh = (j == 0 && pg == 0) ? 0u : 1u;
                            if (elect_one()) {
#pragma unroll
                                for (int k = 0; k < kPage / 16; k++)
                                    tc_mma_pair(tmem + COL_O + part * (2 * HG), pv_a + ((v * VBUF_BYTES + k * 2048) >> 4), HI,
                                                pv_b + ((pg * P_BYTES + k * 32) >> 4), HI, IDESC_PV, k == 0 ? fresh : 1u);
                                tc_commit_pair(bar(B_VEMPTY + pg));
                                if (pg + 1 == uint32_t(PAGES)) {
                                    tc_commit_pair(bar(B_PEMPTY));
                                    if (j + 1 == s.n_tiles) tc_commit_pair(bar(B_OFULL));
                                }
                            }
                            __syncwarp();
                        }
                    }
                }
                nseg++;
            }
        }
    } else {
        // ===================== softmax / correction / epilogue (both blocks, 8 warps) =====================
        // S of a pair MMA with 64 rows per block: head row r sits in TMEM lane r (tokens of the first
        // page) and lane 64+r (second page), 64 columns each.  Two warps share each lane quarter and
        // split its columns, so a thread owns (head, 32 tokens): token quarter tq = 2*page + group.
        const uint32_t sw_id = warp - (2 + N_QK + N_PV);      // 0..7
        const uint32_t grp = sw_id / 4;                       // column group within the lane quarter
        const uint32_t q4 = warp % 4;
        const uint32_t lane_base = (q4 * 32u) << 16;
        const uint32_t half = q4 / 2;                         // page within the tile
        const uint32_t tq = 2 * half + grp;                   // tokens 32*tq .. 32*tq+31 of the tile
        const uint32_t hl = 32 * (q4 % 2) + lane;             // head within this block's 64
        const uint32_t st_id = tid - (NUM_THREADS - SOFTMAX_THREADS);
        const uint32_t peer = rank ^ 1;
        const uint32_t r_sempty = map_to_rank(bar(B_SEMPTY), 0);
        const uint32_t r_pfull = map_to_rank(bar(B_PFULL), 0);
        const uint32_t r_synca[2] = {map_to_rank(bar(B_SYNCA0), peer), map_to_rank(bar(B_SYNCA1), peer)};
        const uint32_t r_syncb[2] = {map_to_rank(bar(B_SYNCB0), peer), map_to_rank(bar(B_SYNCB1), peer)};
        const uint32_t r_flag = map_to_rank(base + OFF_MISC + M_FLAG, peer);
        const uint32_t r_alpha = map_to_rank(base + OFF_MISC + M_ALPHA, peer);
        float m_used = -INFINITY, l_part = 0.0f;
        uint32_t t = 0, nseg = 0, na[2] = {0, 0}, nb[2] = {0, 0};   // na / nb: uses of SYNCA[par] / SYNCB[par] so far
        bool fail = false;
        auto wait_w = [&](uint32_t b, uint32_t parity) {              // completion of tensor-core / TMA work
            if (!fail) fail = !mbar_wait<kSleep>(b, parity, abort_flag, status);
            fail = __any_sync(0xffffffffu, fail);
        };
        auto wait_x = [&](uint32_t b, uint32_t parity) {              // rounds that carry the twin's DSMEM writes
            if (!fail) fail = !mbar_wait<kSleepCluster>(b, parity, abort_flag, status);
            fail = __any_sync(0xffffffffu, fail);
        };
        auto group_or = [&](bool pred) -> bool {              // barrier over this block's softmax threads + OR
            uint32_t r;
            asm volatile(
                "{\n.reg .pred pi, po;\n"
                "setp.ne.b32 pi, %1, 0;\n"
                "barrier.cta.red.or.pred po, 1, 256, pi;\n"
                "selp.u32 %0, 1, 0, po;\n}\n"
                : "=r"(r) : "r"(uint32_t(pred)) : "memory");
            return r != 0;
        };
        bool stop = false;
        for (uint32_t seg = seg_begin; seg < seg_end && !stop; seg++) {
            const SegInfo s = seg_info(seg);
            if (s.n_tiles == 0) {
                // nothing to attend: each block writes its 256 dims of every head, and (m, l) of its own heads
                for (uint32_t h = 0; h < 2 * HG; h++) {
                    if (hpair + h >= H) break;
                    float* rc = recs + (size_t(seg) * H + hpair + h) * kPart;
                    const uint32_t dim = (st_id / 128) * 256 + rank * 128 + (st_id % 128);
                    rc[2 + dim] = 0.0f;
                    if (st_id == 0 && h / HG == rank) { rc[0] = -INFINITY; rc[1] = 0.0f; }
                }
                continue;
            }
            m_used = -INFINITY;
            l_part = 0.0f;
            for (uint32_t j = 0; j < s.n_tiles; j++, t++) {
                const uint32_t par = t & 1;
                wait_w(bar(B_SFULL), t & 1);
                uint32_t sv[32];
                if (!fail) {
                    tc_fence_after();
                    {
                        uint32_t sw[32];
                        tc_ld32(tmem + lane_base + COL_S + grp * 32, sv);
                        tc_ld32(tmem + lane_base + COL_S + (TILE / 2) + grp * 32, sw);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) sv[i] = __float_as_uint(__uint_as_float(sv[i]) + __uint_as_float(sw[i]));
                    }
#pragma unroll 1
                    for (int p = 2; p < N_QK; p++) {
                        uint32_t sw[32];
                        tc_ld32(tmem + lane_base + COL_S + p * (TILE / 2) + grp * 32, sw);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) sv[i] = __float_as_uint(__uint_as_float(sv[i]) + __uint_as_float(sw[i]));
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {                       // orders only TMEM reads: no memory release needed
                        if (rank == 0) mbar_arrive(bar(B_SEMPTY));
                        else mbar_arrive_cluster_relaxed(r_sempty);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) sv[i] = 0u;
                }
                // Scores stay unscaled in registers: the scale rides in the FMA in front of each exponential, and
                // the mask pass runs only on a segment's last, partly filled tile.
                const uint32_t valid = min(uint32_t(TILE), s.n_tok - j * TILE);
                if (valid < uint32_t(TILE)) {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (tq * 32 + uint32_t(i) >= valid) sv[i] = __float_as_uint(-INFINITY);
                }
                float mx = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; i++) mx = fmaxf(mx, __uint_as_float(sv[i]));
                mx *= scale_log2;
                // The first tile of a segment sets every head's reference maximum, but there is no O^T to rescale yet
                // (its PV starts a fresh accumulation), so the twin block has nothing to learn from it: the four
                // token quarters of a head meet inside the block and the two cluster rounds are skipped.  Both blocks
                // of a pair walk the same segments, so they skip the same rounds.
                const bool first = j == 0;
                if (first) {
                    half_max[tq * HG + hl] = mx;
                    if (group_or(fail)) { stop = true; break; }
                    m_used = fmaxf(fmaxf(half_max[hl], half_max[HG + hl]), fmaxf(half_max[2 * HG + hl], half_max[3 * HG + hl]));
                }
                // does any head of the pair have to move its reference maximum on this tile?
                const bool need = !first && (mx > m_used + RESCALE_THRESHOLD);
                const bool warp_need = __any_sync(0xffffffffu, need);
                if (lane == 0 && !fail && !first) {
                    if (warp_need) {
                        atomicOr(const_cast<uint32_t*>(&need_flag[par]), 1u);
                        asm volatile("red.relaxed.cluster.shared::cluster.or.b32 [%0], %1;\n" ::"r"(r_flag + 4 * par), "r"(1u) : "memory");
                        mbar_arrive_local_release_cluster(bar(B_SYNCA0 + par));
                        mbar_arrive_cluster(r_synca[par]);
                    } else {
                        mbar_arrive(bar(B_SYNCA0 + par));
                        mbar_arrive_cluster_relaxed(r_synca[par]);
                    }
                }
                // optimistic: exponentials against the current maximum while the cluster round is in
                // flight; they stand unless some head of the pair raised the flag
                float sum = 0.0f;
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = fast_ex2(fmaf(__uint_as_float(sv[i]), scale_log2, -m_used));
                    const float p1 = fast_ex2(fmaf(__uint_as_float(sv[i + 1]), scale_log2, -m_used));
                    sum += p0 + p1;
                    pk[i / 2] = Elem<T>::pack2(p0, p1);
                }
                bool slow = false;
                if (!first) {
                    wait_x(bar(B_SYNCA0 + par), na[par] & 1);
                    na[par]++;
                    if (group_or(fail)) { stop = true; break; }
                    slow = need_flag[par] != 0;
                }
                if (slow) {
                    // exchange the token quarters' maxima inside the block, decide per head, publish the
                    // scale factors to both blocks, and redo the exponentials
                    float alpha = 1.0f;
                    half_max[tq * HG + hl] = mx;
                    group_or(false);
                    const float mrow = fmaxf(fmaxf(half_max[hl], half_max[HG + hl]), fmaxf(half_max[2 * HG + hl], half_max[3 * HG + hl]));
                    if (mrow > m_used + RESCALE_THRESHOLD) { alpha = fast_ex2(m_used - mrow); m_used = mrow; }
                    if (tq == 0) {
                        alpha_all[par * 128 + rank * HG + hl] = alpha;
                        asm volatile("st.relaxed.cluster.shared::cluster.f32 [%0], %1;\n"
                                     ::"r"(r_alpha + 4 * (par * 128 + rank * HG + hl)), "f"(alpha) : "memory");
                    }
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive_local_release_cluster(bar(B_SYNCB0 + par));
                        mbar_arrive_cluster(r_syncb[par]);
                    }
                    wait_x(bar(B_SYNCB0 + par), nb[par] & 1);
                    nb[par]++;
                    l_part *= alpha;
                    sum = 0.0f;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = fast_ex2(fmaf(__uint_as_float(sv[i]), scale_log2, -m_used));
                        const float p1 = fast_ex2(fmaf(__uint_as_float(sv[i + 1]), scale_log2, -m_used));
                        sum += p0 + p1;
                        pk[i / 2] = Elem<T>::pack2(p0, p1);
                    }
                }
                l_part += sum;
                // PV of the previous tile must be complete: O is stable and P is free
                wait_w(bar(B_PEMPTY), (t - 1) & 1);
                if (fail) continue;            // carried to the next barrier
                tc_fence_after();
                if (slow) {
                    // O^T[this block's dims][128 heads] *= alpha[head]; each warp group takes one chunk
#pragma unroll 1
                    for (int c = 0; c < 4; c++) {
                        uint32_t o[32];
                        const uint32_t col = COL_O + grp * 128 + c * 32;
                        tc_ld32(tmem + lane_base + col, o);
                        tc_wait_ld();
                        const float* al = alpha_all + par * 128 + c * 32;
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * al[i]);
                        tc_st32(tmem + lane_base + col, o);
                    }
                    tc_wait_st();
                }
                {
                    // row hl of the page's K-major swizzled P tile, this thread's 32 tokens = 16-byte chunks 4*grp .. 4*grp+3
                    unsigned char* prow = sm + OFF_P + half * P_BYTES + hl * 128;
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        const uint4 v = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
                        *reinterpret_cast<uint4*>(prow + (((4 * grp + ch) ^ (hl & 7)) << 4)) = v;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (rank == 0) mbar_arrive(bar(B_PFULL));
                    else mbar_arrive_remote(r_pfull);
                }
                // the flag of this parity is next written two tiles from now: clear it once every
                // thread of the block has read it (they all passed the barrier of the slow path)
                if (st_id == 0 && slow) need_flag[par] = 0;
            }
            if (stop) break;
            // ---- epilogue: O^T (this block's 256 dims x 128 heads) -> acc[head][dim]; (m, l) of own heads
            wait_w(bar(B_OFULL), nseg & 1);
            group_or(false);                   // the maxima scratch is free: its bytes now carry the partial sums
            if (tq != 0) l_other[(tq - 1) * HG + hl] = l_part;
            if (group_or(fail)) { stop = true; break; }
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 4; c++) {                      // warp group `grp` owns chunk `grp`
                uint32_t o[32];
                tc_ld32(tmem + lane_base + COL_O + grp * 128 + c * 32, o);
                tc_wait_ld();
                const uint32_t dim = grp * 256 + rank * 128 + q4 * 32 + lane;
                const uint32_t hb = hpair + c * 32;
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (hb + i < H) recs[(size_t(seg) * H + hb + i) * kPart + 2 + dim] = __uint_as_float(o[i]);
                }
            }
            if (tq == 0 && h0 + hl < H) {
                float* rc = recs + (size_t(seg) * H + h0 + hl) * kPart;
                rc[0] = m_used;
                rc[1] = l_part + l_other[hl] + l_other[HG + hl] + l_other[2 * HG + hl];
            }
            tc_fence_before();
            group_or(false);                   // the scratch is reused by the next segment
            nseg++;
        }
    }

    // Neither block may leave while its twin can still signal its barriers, write its scratch or
    // feed a pair MMA from its shared memory.
    tc_fence_before();
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}
}  // namespace

int decode_tc5_pair128_configure()
{
    cudaError_t e = cudaFuncSetAttribute(decode_tc5_pair128_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    e = cudaFuncSetAttribute(decode_tc5_pair128_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    // every kernel of a layer-step asks for the same (maximal) shared-memory carve-out, so the SMs are not
    // re-partitioned between consecutive launches
    e = cudaFuncSetAttribute(decode_tc5_pair128_kernel<__half>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return int(e);
    e = cudaFuncSetAttribute(decode_tc5_pair128_kernel<__nv_bfloat16>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    return int(e);
}

// tmaps: the context's tensor-map array (kMapPoolSub = one K sub-tile, kMapPoolV = V boxes, kMapQueries = Q').
// layer_pool: the layer's slice of the cache pool (linear L2 prefetch).
int launch_decode_tc5_pair128(int dtype, const void* tmaps, const void* layer_pool, uint32_t layer, uint32_t n_pages,
                              const StepMeta& m, float* recs, uint32_t H, uint32_t prefetch_tiles, const void* next_weights,
                              uint32_t next_weights_bytes, uint32_t* status, cudaStream_t st)
{
    if (m.ctas == 0) return 0;
    const CUtensorMap* maps = static_cast<const CUtensorMap*>(tmaps);
    const float scale_log2 = 1.4426950408889634f / sqrtf(float(kQDim));
    dim3 grid(2 * m.ctas, (H + 2 * HG - 1) / (2 * HG));          // clusters of 2 along x
    if (dtype == 0)
        return int(launch_pdl(decode_tc5_pair128_kernel<__half>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, maps[kMapPoolSub], maps[kMapPoolV], maps[kMapQueries],
                              static_cast<const unsigned char*>(layer_pool), layer, n_pages, m, recs, H, scale_log2, prefetch_tiles,
                              static_cast<const unsigned char*>(next_weights), next_weights_bytes, status));
    return int(launch_pdl(decode_tc5_pair128_kernel<__nv_bfloat16>, grid, dim3(NUM_THREADS), SMEM_BYTES, st, maps[kMapPoolSub], maps[kMapPoolV],
                          maps[kMapQueries], static_cast<const unsigned char*>(layer_pool), layer, n_pages, m, recs, H, scale_log2, prefetch_tiles,
                              static_cast<const unsigned char*>(next_weights), next_weights_bytes, status));
}

}  // namespace mla
