// Host-side bookkeeping of the paged latent KV cache: sequences, block tables, the free list.
// Pure C++ (no CUDA) so it can be unit-tested without a device.
//
// It keeps the contract of the reference's mugen::KVCache as the MLA model uses it — a
// per-sequence length counter with advance / truncate / clear
// (src/core/memory/kv_cache.h:20-47, kv_cache.cpp:281-285, 313-321, 343-357) — and adds what
// the reference lacks: many sequences, fixed-size pages, capacity checks with error returns
// (the reference writes row pos*576 unchecked, src/core/model/transformer.cpp:3982-3985), and a
// truncate that never grows (the reference's does, kv_cache.cpp:316-321).
#pragma once

#include <algorithm>
#include <cstdint>
#include <random>
#include <string>
#include <vector>

namespace mugen::mla {

enum : int { PT_OK = 0, PT_INVALID = 1, PT_NO_PAGES = 3, PT_CAPACITY = 4 };

class PageTable {
public:
    struct Seq {
        bool live = false;
        uint32_t len = 0;        // tokens counted (seq_len)
        uint32_t base_pos = 0;   // global position of local row 0
        std::vector<uint32_t> pages;
    };

    PageTable(uint32_t page_tokens, uint32_t n_pages, uint32_t max_seqs, uint32_t max_seq_len)
        : page_tokens_(page_tokens), n_pages_(n_pages), max_seq_len_(max_seq_len), seqs_(max_seqs)
    {
        free_.resize(n_pages);
        // LIFO stack: page 0 is handed out first.
        for (uint32_t i = 0; i < n_pages; i++) free_[i] = n_pages - 1 - i;
    }

    uint32_t page_tokens() const { return page_tokens_; }
    uint32_t free_pages() const { return uint32_t(free_.size()); }
    uint32_t max_seqs() const { return uint32_t(seqs_.size()); }
    const std::string& error() const { return err_; }

    void shuffle_free(uint64_t seed) {
        std::mt19937_64 rng(seed);
        std::shuffle(free_.begin(), free_.end(), rng);
    }

    int seq_create(uint32_t* id) {
        for (uint32_t i = 0; i < seqs_.size(); i++) {
            if (!seqs_[i].live) {
                seqs_[i] = Seq{};
                seqs_[i].live = true;
                *id = i;
                return PT_OK;
            }
        }
        return fail(PT_CAPACITY, "no free sequence slot (max_seqs reached)");
    }

    int seq_free(uint32_t id) {
        if (int e = check(id)) return e;
        release_from(seqs_[id], 0);
        seqs_[id].live = false;
        return PT_OK;
    }

    const Seq* seq(uint32_t id) const {
        return (id < seqs_.size() && seqs_[id].live) ? &seqs_[id] : nullptr;
    }

    int seq_len(uint32_t id, uint32_t* len) const {
        if (id >= seqs_.size() || !seqs_[id].live) return PT_INVALID;
        *len = seqs_[id].len;
        return PT_OK;
    }

    int set_base(uint32_t id, uint32_t base) {
        if (int e = check(id)) return e;
        if (seqs_[id].len != 0 || !seqs_[id].pages.empty())
            return fail(PT_INVALID, "base position can only be set on an empty sequence");
        seqs_[id].base_pos = base;
        return PT_OK;
    }

    // Makes local rows [0, n_rows) addressable.  All-or-nothing.
    int reserve(uint32_t id, uint32_t n_rows) {
        if (int e = check(id)) return e;
        if (n_rows > max_seq_len_)
            return fail(PT_CAPACITY, "row " + std::to_string(n_rows - 1) + " is beyond max_seq_len " +
                                         std::to_string(max_seq_len_));
        Seq& s = seqs_[id];
        const uint32_t need = (n_rows + page_tokens_ - 1) / page_tokens_;
        if (need <= s.pages.size()) return PT_OK;
        const uint32_t extra = need - uint32_t(s.pages.size());
        if (extra > free_.size())
            return fail(PT_NO_PAGES, "page pool exhausted: need " + std::to_string(extra) +
                                         " more pages, " + std::to_string(free_.size()) + " free");
        for (uint32_t i = 0; i < extra; i++) {
            s.pages.push_back(free_.back());
            free_.pop_back();
        }
        return PT_OK;
    }

    // seq_len += n; the rows must already be backed by pages.
    int advance(uint32_t id, uint32_t n) {
        if (int e = check(id)) return e;
        Seq& s = seqs_[id];
        const uint64_t nl = uint64_t(s.len) + n;
        if (nl > uint64_t(s.pages.size()) * page_tokens_)
            return fail(PT_INVALID, "advance past appended rows");
        s.len = uint32_t(nl);
        return PT_OK;
    }

    int truncate(uint32_t id, uint32_t new_len) {
        if (int e = check(id)) return e;
        Seq& s = seqs_[id];
        if (new_len > s.len)
            return fail(PT_INVALID, "truncate cannot grow a sequence (" + std::to_string(new_len) +
                                        " > " + std::to_string(s.len) + ")");
        s.len = new_len;
        release_from(s, (new_len + page_tokens_ - 1) / page_tokens_);
        return PT_OK;
    }

    int clear(uint32_t id) {
        if (int e = check(id)) return e;
        seqs_[id].len = 0;
        release_from(seqs_[id], 0);
        return PT_OK;
    }

    // Token slot (page*page_tokens + offset) of a local row, which must be reserved.
    uint64_t slot(uint32_t id, uint32_t row) const {
        const Seq& s = seqs_[id];
        return uint64_t(s.pages[row / page_tokens_]) * page_tokens_ + row % page_tokens_;
    }

private:
    int check(uint32_t id) {
        if (id >= seqs_.size() || !seqs_[id].live)
            return fail(PT_INVALID, "unknown sequence id " + std::to_string(id));
        return PT_OK;
    }
    int fail(int code, std::string msg) {
        err_ = std::move(msg);
        return code;
    }
    void release_from(Seq& s, uint32_t keep_pages) {
        while (s.pages.size() > keep_pages) {
            free_.push_back(s.pages.back());
            s.pages.pop_back();
        }
    }

    uint32_t page_tokens_, n_pages_, max_seq_len_;
    std::vector<Seq> seqs_;
    std::vector<uint32_t> free_;
    std::string err_;
};

// ---- split-KV planning --------------------------------------------------------------------
// A query row attends pages [0, ceil(len/page)) of its sequence.  Laid end to end, the rows'
// pages form one line of P pages; it is cut into `workers` equal shares (worker c owns line
// positions [P*c/workers, P*(c+1)/workers)), and every share is further cut at row boundaries.
// The resulting pieces are the segments: each is a run of whole pages of one row, and each
// yields one partial softmax state.  Segments come out ordered by row, then by page, so a
// row's segments and a worker's segments are both contiguous index ranges.  A row of length 0
// still gets one (empty) segment so that its state is written.
struct Segment {
    uint32_t row;
    uint32_t page_begin;
    uint32_t page_end;
};

// granule_pages > 1: the attention kernel walks a segment in tiles of that many pages, so shares are
// counted and cut in tiles (a cut inside a tile would leave two half-empty tiles that cost full ones).
inline void plan_balanced(const std::vector<uint32_t>& attend_lens, uint32_t page_tokens,
                          uint32_t workers, std::vector<Segment>& segs,
                          std::vector<uint32_t>& row_seg_begin,
                          std::vector<uint32_t>& worker_seg_begin, uint32_t granule_pages = 1)
{
    if (granule_pages > 1) {
        plan_balanced(attend_lens, page_tokens * granule_pages, workers, segs, row_seg_begin, worker_seg_begin, 1);
        for (Segment& sg : segs) {
            const uint32_t pages = (attend_lens[sg.row] + page_tokens - 1) / page_tokens;
            sg.page_begin = std::min(pages, sg.page_begin * granule_pages);
            sg.page_end = std::min(pages, sg.page_end * granule_pages);
        }
        return;
    }
    const uint32_t rows = uint32_t(attend_lens.size());
    segs.clear();
    row_seg_begin.assign(rows + 1, 0);
    uint64_t total = 0;
    for (uint32_t l : attend_lens) total += (l + page_tokens - 1) / page_tokens;
    workers = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>(workers, total)));
    std::vector<uint32_t> seg_worker;
    auto bound = [&](uint32_t c) { return total * c / workers; };   // first line position of worker c
    uint64_t cursor = 0;
    uint32_t w = 0;
    for (uint32_t r = 0; r < rows; r++) {
        row_seg_begin[r] = uint32_t(segs.size());
        const uint32_t pages = (attend_lens[r] + page_tokens - 1) / page_tokens;
        if (pages == 0) {
            segs.push_back({r, 0, 0});
            seg_worker.push_back(std::min(w, workers - 1));
            continue;
        }
        uint32_t done = 0;
        while (done < pages) {
            while (w + 1 < workers && bound(w + 1) <= cursor) w++;
            const uint64_t share_end = (w + 1 < workers) ? bound(w + 1) : total;
            const uint32_t take = uint32_t(std::min<uint64_t>(pages - done, share_end - cursor));
            segs.push_back({r, done, done + take});
            seg_worker.push_back(w);
            done += take;
            cursor += take;
        }
    }
    row_seg_begin[rows] = uint32_t(segs.size());
    worker_seg_begin.assign(workers + 1, uint32_t(segs.size()));
    worker_seg_begin[0] = 0;
    uint32_t s = 0;
    for (uint32_t c = 0; c < workers; c++) {
        worker_seg_begin[c] = s;
        while (s < segs.size() && seg_worker[s] == c) s++;
    }
    worker_seg_begin[workers] = uint32_t(segs.size());
}

// The same plan with a price on every segment.  A worker pays a fixed cost each time it starts a segment (load the
// row's queries, fill the pipeline, drain the partial state: about four tiles' worth of time on the SM-pair kernel),
// so equal shares of PAGES are not equal shares of TIME: with 8 rows over 74 workers the equal-share plan hands the
// workers that straddle a row boundary two segments for the price of a worker with one.  Here the makespan
// T = max over workers of sum(seg_overhead + units of the segment) is minimised by bisection: for a trial T the rows
// are poured into the workers in order, a worker closing when another unit (plus the overhead, if it would have to
// start a segment for it) no longer fits.  Units are `granule_pages` pages (the kernel's tile); cuts inside a row
// fall on unit boundaries.  seg_overhead = 0 reproduces equal shares up to rounding.
inline void plan_min_makespan(const std::vector<uint32_t>& attend_lens, uint32_t page_tokens, uint32_t workers,
                              std::vector<Segment>& segs, std::vector<uint32_t>& row_seg_begin,
                              std::vector<uint32_t>& worker_seg_begin, uint32_t granule_pages, uint32_t seg_overhead)
{
    const uint32_t rows = uint32_t(attend_lens.size());
    std::vector<uint32_t> pages(rows), units(rows);
    uint64_t total = 0;
    for (uint32_t r = 0; r < rows; r++) {
        pages[r] = (attend_lens[r] + page_tokens - 1) / page_tokens;
        units[r] = (pages[r] + granule_pages - 1) / granule_pages;
        total += units[r];
    }
    workers = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>(workers, total)));
    std::vector<uint32_t> seg_worker;
    // pours the rows into workers of capacity T; returns the number of workers used (emit: also records the plan)
    auto pour = [&](uint64_t T, bool emit) -> uint64_t {
        uint64_t used = 1, cur = 0;
        if (emit) { segs.clear(); seg_worker.clear(); row_seg_begin.assign(rows + 1, 0); }
        for (uint32_t r = 0; r < rows; r++) {
            if (emit) row_seg_begin[r] = uint32_t(segs.size());
            if (units[r] == 0) {
                if (emit) { segs.push_back({r, 0, 0}); seg_worker.push_back(uint32_t(used - 1)); }
                continue;
            }
            uint32_t done = 0;
            while (done < units[r]) {
                if (cur + seg_overhead + 1 > T && cur > 0) { used++; cur = 0; }      // no room to start a segment here
                const uint64_t room = T > cur + seg_overhead ? T - cur - seg_overhead : 1;
                const uint32_t take = uint32_t(std::min<uint64_t>(units[r] - done, room));
                if (emit) {
                    segs.push_back({r, std::min(pages[r], done * granule_pages), std::min(pages[r], (done + take) * granule_pages)});
                    seg_worker.push_back(uint32_t(used - 1));
                }
                done += take;
                cur += seg_overhead + take;
            }
        }
        return used;
    };
    uint64_t lo = 1, hi = total + uint64_t(seg_overhead) * (rows + workers) + 1;
    while (lo < hi) {
        const uint64_t mid = (lo + hi) / 2;
        if (pour(mid, false) <= workers) hi = mid; else lo = mid + 1;
    }
    const uint64_t used = total ? pour(lo, true) : pour(1, true);
    row_seg_begin[rows] = uint32_t(segs.size());
    const uint32_t W = total ? uint32_t(std::max<uint64_t>(used, 1)) : workers;
    worker_seg_begin.assign(W + 1, uint32_t(segs.size()));
    uint32_t s = 0;
    for (uint32_t c = 0; c < W; c++) {
        worker_seg_begin[c] = s;
        while (s < segs.size() && seg_worker[s] == c) s++;
    }
    worker_seg_begin[W] = uint32_t(segs.size());
}

}  // namespace mugen::mla
