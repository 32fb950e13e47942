// Host-side tests in the reference's own test style (one executable, local CHECK macro that
// prints and exits: tests/unit/test_kv_cache.cpp:10-17 of the reference).
//   test_host units            page table, planner and C++ wrapper checks that need no GPU
//   test_host rope f c th p..  prints cos/sin bits of the rotary table rows for positions p..
//   test_host decode in out    GPU: runs decode steps through the C++23 wrapper with host buffers
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <numeric>

#include "../../mugen_b200/host/mla_host.hpp"
#include "../../mugen_b200/host/page_table.hpp"
#include "../../mugen_b200/host/rope_table.hpp"

#define CHECK(cond)                                                              \
    do {                                                                         \
        if (!(cond)) {                                                           \
            std::fprintf(stderr, "CHECK failed %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                        \
        }                                                                        \
    } while (0)

using namespace mugen::mla;

static void test_page_table()
{
    PageTable pt(64, 8, 3, 300);
    uint32_t a, b, c, d;
    CHECK(pt.seq_create(&a) == PT_OK && pt.seq_create(&b) == PT_OK && pt.seq_create(&c) == PT_OK);
    CHECK(pt.seq_create(&d) == PT_CAPACITY);
    CHECK(pt.reserve(a, 130) == PT_OK && pt.free_pages() == 5);     // 3 pages
    CHECK(pt.advance(a, 130) == PT_OK);
    CHECK(pt.advance(a, 63) == PT_INVALID);                         // beyond the reserved rows (192)
    CHECK(pt.reserve(b, 301) == PT_CAPACITY);                       // beyond max_seq_len
    CHECK(pt.reserve(b, 64 * 6) == PT_CAPACITY);
    CHECK(pt.reserve(b, 300) == PT_OK && pt.free_pages() == 0);     // 5 pages
    CHECK(pt.reserve(c, 1) == PT_NO_PAGES);
    uint32_t n = 0;
    CHECK(pt.seq_len(a, &n) == PT_OK && n == 130);
    CHECK(pt.truncate(a, 131) == PT_INVALID);                       // never grows
    CHECK(pt.truncate(a, 65) == PT_OK && pt.free_pages() == 1);     // keeps the partial page
    CHECK(pt.truncate(a, 64) == PT_OK && pt.free_pages() == 2);
    CHECK(pt.clear(a) == PT_OK && pt.free_pages() == 3);
    CHECK(pt.seq_len(a, &n) == PT_OK && n == 0);
    CHECK(pt.set_base(b, 10) == PT_INVALID);                        // only on an empty sequence
    CHECK(pt.set_base(a, 4096) == PT_OK);
    CHECK(pt.seq_free(b) == PT_OK && pt.free_pages() == 8);
    CHECK(pt.seq_len(b, &n) == PT_INVALID);
    // slots: distinct pages, offset within page
    CHECK(pt.reserve(c, 200) == PT_OK);
    CHECK(pt.slot(c, 0) % 64 == 0 && pt.slot(c, 63) == pt.slot(c, 0) + 63);
    CHECK(pt.slot(c, 64) / 64 != pt.slot(c, 0) / 64);
    // a shuffled free list still hands out every page exactly once
    PageTable p2(64, 100, 1, 6400);
    p2.shuffle_free(7);
    uint32_t s;
    CHECK(p2.seq_create(&s) == PT_OK && p2.reserve(s, 6400) == PT_OK);
    std::vector<int> seen(100, 0);
    for (uint32_t pg : p2.seq(s)->pages) seen[pg]++;
    for (int v : seen) CHECK(v == 1);
}

static void test_planner()
{
    std::vector<Segment> segs;
    std::vector<uint32_t> rsb, wsb;
    // uniform batch: equal shares, every page covered exactly once, in order
    std::vector<uint32_t> lens(64, 16384);
    plan_balanced(lens, 64, 74, segs, rsb, wsb);
    CHECK(wsb.size() == 75 && rsb.size() == 65);
    uint64_t covered = 0;
    for (uint32_t r = 0; r < 64; r++) {
        uint32_t next = 0;
        for (uint32_t g = rsb[r]; g < rsb[r + 1]; g++) {
            CHECK(segs[g].row == r && segs[g].page_begin == next && segs[g].page_end > next);
            next = segs[g].page_end;
        }
        CHECK(next == 256);
        covered += next;
    }
    CHECK(covered == 64 * 256);
    for (uint32_t w = 0; w < 74; w++) {
        uint64_t pages = 0;
        for (uint32_t g = wsb[w]; g < wsb[w + 1]; g++) pages += segs[g].page_end - segs[g].page_begin;
        CHECK(pages == 221 || pages == 222);
    }
    // ragged batch with empty rows; fewer pages than workers
    lens = {0, 1, 64, 65, 0, 1000, 0};
    plan_balanced(lens, 64, 148, segs, rsb, wsb);
    CHECK(rsb[1] - rsb[0] == 1 && segs[rsb[0]].page_begin == segs[rsb[0]].page_end);   // empty row keeps a segment
    uint64_t total = 0;
    for (auto& g : segs) total += g.page_end - g.page_begin;
    CHECK(total == 0 + 1 + 1 + 2 + 0 + 16 + 0);
    CHECK(wsb.back() == segs.size());
    for (size_t w = 0; w + 1 < wsb.size(); w++) CHECK(wsb[w] <= wsb[w + 1]);
    // one long row over many workers: one segment per worker
    lens = {131072};
    plan_balanced(lens, 64, 148, segs, rsb, wsb);
    CHECK(segs.size() == 148 && rsb[1] == 148);
    // two-page tiles: every cut inside a row falls on an even page, pages are still covered once, shares are
    // equal in tiles; a row with an odd page count keeps its last single page
    lens.assign(64, 16385);                                   // 257 pages = 129 tiles per row
    plan_balanced(lens, 64, 74, segs, rsb, wsb, 2);
    for (uint32_t r = 0; r < 64; r++) {
        uint32_t next = 0;
        for (uint32_t g = rsb[r]; g < rsb[r + 1]; g++) {
            CHECK(segs[g].row == r && segs[g].page_begin == next && segs[g].page_end > next);
            CHECK(segs[g].page_begin % 2 == 0);
            CHECK(segs[g].page_end % 2 == 0 || segs[g].page_end == 257);
            next = segs[g].page_end;
        }
        CHECK(next == 257);
    }
    for (uint32_t w = 0; w < 74; w++) {
        uint64_t tiles = 0;
        for (uint32_t g = wsb[w]; g < wsb[w + 1]; g++) tiles += (segs[g].page_end - segs[g].page_begin + 1) / 2;
        CHECK(tiles == 111 || tiles == 112);
    }
    lens = {0, 1, 64, 65, 0, 1000, 0};
    plan_balanced(lens, 64, 148, segs, rsb, wsb, 2);
    total = 0;
    for (auto& g : segs) total += g.page_end - g.page_begin;
    CHECK(total == 0 + 1 + 1 + 2 + 0 + 16 + 0);
    // nothing at all
    lens.clear();
    plan_balanced(lens, 64, 148, segs, rsb, wsb);
    CHECK(segs.empty() && rsb.size() == 1 && wsb.back() == 0);

    // ---- the plan that prices segments: coverage, order, cuts on tile boundaries, and a makespan no worse than
    // the equal-share plan's under the same price
    auto cost_of = [&](const std::vector<Segment>& sg, const std::vector<uint32_t>& ws, uint32_t ovh) {
        uint64_t worst = 0;
        for (size_t w = 0; w + 1 < ws.size(); w++) {
            uint64_t c = 0;
            for (uint32_t g = ws[w]; g < ws[w + 1]; g++) {
                const uint32_t n = sg[g].page_end - sg[g].page_begin;
                if (n) c += ovh + (n + 1) / 2;
            }
            worst = std::max(worst, c);
        }
        return worst;
    };
    for (auto cfg : std::vector<std::pair<std::vector<uint32_t>, uint32_t>>{
             {std::vector<uint32_t>(8, 16384), 74}, {std::vector<uint32_t>(64, 16384), 74}, {std::vector<uint32_t>(1, 131072), 74},
             {{0, 1, 64, 65, 0, 1000, 0, 32768, 300}, 74}, {std::vector<uint32_t>(3, 100), 148}, {{}, 74}}) {
        const auto& ls = cfg.first;
        std::vector<Segment> s2, s1;
        std::vector<uint32_t> r2, w2, r1, w1;
        plan_min_makespan(ls, 64, cfg.second, s2, r2, w2, 2, 4);
        CHECK(r2.size() == ls.size() + 1 && w2.back() == s2.size() && w2.size() <= cfg.second + 1u);
        for (uint32_t r = 0; r < ls.size(); r++) {
            uint32_t next = 0;
            CHECK(r2[r + 1] > r2[r]);                                   // every row keeps at least one segment
            for (uint32_t g = r2[r]; g < r2[r + 1]; g++) {
                CHECK(s2[g].row == r && s2[g].page_begin == next && s2[g].page_begin % 2 == 0);
                CHECK(s2[g].page_end > next || ls[r] == 0);
                next = s2[g].page_end;
            }
            CHECK(next == (ls[r] + 63) / 64);
        }
        for (size_t w = 0; w + 1 < w2.size(); w++) CHECK(w2[w] <= w2[w + 1]);
        if (!ls.empty()) {
            plan_balanced(ls, 64, cfg.second, s1, r1, w1, 2);
            CHECK(cost_of(s2, w2, 4) <= cost_of(s1, w1, 4));
        }
    }
    {   // 8 rows of 128 tiles over 74 workers: nobody gets two segments for the price of one
        std::vector<Segment> s2;
        std::vector<uint32_t> r2, w2;
        plan_min_makespan(std::vector<uint32_t>(8, 16384), 64, 74, s2, r2, w2, 2, 4);
        CHECK(cost_of(s2, w2, 4) <= 19);
    }
}

static void test_wrapper_without_gpu()
{
    LatentKVCacheConfig cfg;
    cfg.n_layers = 0;
    auto bad = LatentKVCache::create(cfg);
    CHECK(!bad && bad.error() == "n_layers must be > 0");    // KVCache::create's message
}

static std::vector<char> slurp(const char* path)
{
    std::ifstream f(path, std::ios::binary);
    return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

// Input file: u32 header {H, L, B, T, bf16} then weights per layer (w_uk, w_uv as 16-bit values,
// norm[512]) then per step per layer kv_a[B][576], q[B][H][192].  Output: out[T][L][B][H][128].
static int run_decode(const char* in_path, const char* out_path)
{
    auto buf = slurp(in_path);
    const auto* hdr = reinterpret_cast<const uint32_t*>(buf.data());
    const uint32_t H = hdr[0], L = hdr[1], B = hdr[2], T = hdr[3], bf16 = hdr[4];
    const uint16_t* p = reinterpret_cast<const uint16_t*>(buf.data() + 20);
    LatentKVCacheConfig cfg;
    cfg.n_layers = L; cfg.n_heads = H; cfg.max_seq_len = 256; cfg.n_pages = 4 * B; cfg.max_seqs = B;
    cfg.bf16 = bf16 != 0; cfg.rope_scaling_factor = 40.0f; cfg.rope_original_ctx = 4096; cfg.rms_norm_eps = 1e-6f;
    auto cache = LatentKVCache::create(cfg);
    if (!cache) { std::fprintf(stderr, "create: %s\n", cache.error().c_str()); return 2; }
    MlaAttention attn(**cache);
    const size_t wn = size_t(H) * 128 * 512;
    for (uint32_t l = 0; l < L; l++) {
        auto r = attn.set_layer_weights(l, p, p + wn, bf16 ? MLA_W_BF16 : MLA_W_F16, p + 2 * wn);
        if (!r) { std::fprintf(stderr, "weights: %s\n", r.error().c_str()); return 2; }
        p += 2 * wn + 512;
    }
    std::vector<uint32_t> seqs(B);
    for (auto& s : seqs) s = (*cache)->new_sequence().value();
    std::vector<uint16_t> out(size_t(T) * L * B * H * 128);
    uint16_t* o = out.data();
    for (uint32_t t = 0; t < T; t++) {
        if (auto r = attn.step_begin(seqs); !r) { std::fprintf(stderr, "begin: %s\n", r.error().c_str()); return 2; }
        for (uint32_t l = 0; l < L; l++) {
            const uint16_t* kv = p;
            const uint16_t* q = p + size_t(B) * 576;
            p += size_t(B) * 576 + size_t(B) * H * 192;
            if (auto r = attn.step_layer_host(l, kv, q, o); !r) { std::fprintf(stderr, "layer: %s\n", r.error().c_str()); return 2; }
            o += size_t(B) * H * 128;
        }
        if (auto r = attn.step_end(); !r) return 2;
        CHECK((*cache)->seq_len(seqs[0]) == t + 1);
    }
    if (auto r = attn.check_device(); !r) { std::fprintf(stderr, "device: %s\n", r.error().c_str()); return 2; }
    CHECK((*cache)->truncate(seqs[0], T + 1).has_value() == false);
    std::ofstream f(out_path, std::ios::binary);
    f.write(reinterpret_cast<const char*>(out.data()), out.size() * 2);
    return 0;
}

int main(int argc, char** argv)
{
    if (argc >= 2 && !std::strcmp(argv[1], "units")) {
        test_page_table();
        test_planner();
        test_wrapper_without_gpu();
        std::puts("host units ok");
        return 0;
    }
    if (argc >= 6 && !std::strcmp(argv[1], "rope")) {
        const float factor = std::strtof(argv[2], nullptr);
        const uint32_t ctx = uint32_t(std::strtoul(argv[3], nullptr, 10));
        const float theta = std::strtof(argv[4], nullptr);
        for (int i = 5; i < argc; i++) {
            const uint32_t pos = uint32_t(std::strtoul(argv[i], nullptr, 10));
            float row[64];
            fill_rope_rows(row, pos, pos + 1, factor, ctx, theta);
            for (int k = 0; k < 64; k++) {
                uint32_t u;
                std::memcpy(&u, &row[k], 4);
                std::printf("%08x%c", u, k == 63 ? '\n' : ' ');
            }
        }
        return 0;
    }
    if (argc >= 4 && !std::strcmp(argv[1], "decode")) return run_decode(argv[2], argv[3]);
    std::fprintf(stderr, "usage: test_host units | rope factor ctx theta pos... | decode in out\n");
    return 64;
}
