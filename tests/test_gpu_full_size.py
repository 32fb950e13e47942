"""GPU parity at the benchmark's full shapes (128 heads, bf16; contexts of 16384 and 131072 tokens; 16 heads, fp16, ctx 8192),
through the C ABI.  The CPU checker is too slow for whole batches at these sizes, so most checks are
properties that do not depend on the size — the same logical cache under two page permutations, a
KV-range split against the unsplit sequence, a prefill chunk against single decode rows — with
checker spot-checks on a few heads or sequences.  Inputs are generated on the device from a seed."""
from __future__ import annotations

import os

import numpy as np
import pytest

from mugen_b200 import capi, synth

pytestmark = pytest.mark.gpu

MAX_ABS, REL_L2 = 2e-2, 5e-3
YARN = dict(rope_theta=10000.0, rope_scaling_factor=40.0, rope_original_ctx=4096, rms_norm_eps=1e-6)
H, DT = 128, synth.DT_BF16


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch


@pytest.fixture(scope="module")
def oracle():
    from oracle import binding
    return binding.oracle()


def _bits(t) -> np.ndarray:
    return t.cpu().numpy().view(np.uint16)


def _rand_bf16(torch, shape, seed, scale=1.0):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    x = torch.randn(shape, device="cuda", dtype=torch.float32, generator=g) * scale
    return x.to(torch.bfloat16).view(torch.int16)


def _weights(seed):
    rng = np.random.default_rng(seed)
    wk = synth.to_bits(rng.standard_normal((H * 128, 512), np.float32) * np.float32(0.02), DT)
    wv = synth.to_bits(rng.standard_normal((H * 128, 512), np.float32) * np.float32(0.02), DT)
    nw = synth.to_bits((1.0 + 0.1 * rng.standard_normal(512)).astype(np.float32), DT)
    return wk, wv, nw


def _close(got, want, what):
    mx, rl = synth.error_norms(got, want, DT, DT)
    assert mx <= MAX_ABS and rl <= REL_L2, f"{what}: max-abs {mx:.3e}, rel-L2 {rl:.3e}"


def test_ctx16384_decode_step_page_permutation_and_checker(torch, oracle):
    """configs[2] shape, 4 of its 64 sequences: one decode step at ctx 16384 through mla_step_layers.
    (a) two contexts holding the same logical caches under different page permutations give
    bit-identical outputs and appended rows; (b) appended rows equal the checker's bit for bit;
    (c) all four sequences, all 128 heads, agree with the CPU attention within the tolerance."""
    from mugen_b200.mla import MlaContext
    B, S = 4, 16383
    wk, wv, nw = _weights(1)
    cache = _rand_bf16(torch, (B, S, 576), 11)
    kv = _rand_bf16(torch, (B, 576), 12)
    q = _rand_bf16(torch, (B, H, 192), 13, 0.9)
    outs, rows = [], []
    for shuffle in (3, 77):
        ctx = MlaContext(n_layers=1, n_heads=H, dtype=DT, n_pages=B * 257 + 16, max_seqs=B, max_seq_len=S + 65,
                         kernel=capi.KERNEL_AUTO, **YARN)
        ctx.shuffle_free_pages(shuffle)
        ctx.set_layer_weights(0, wk, wv, synth.W_BF16, nw)
        seqs = []
        for b in range(B):
            s = ctx.seq_create()
            ctx.write_rows(0, s, 0, cache[b])
            ctx.advance_seq_len(s, S)
            seqs.append(s)
        out = torch.zeros((B, H, 128), dtype=torch.int16, device="cuda")
        ctx.step_begin(seqs)
        ctx.step_layers(0, 1, kv[None], q[None], out[None])
        ctx.step_end()
        assert ctx.status() == 0 and ctx.kernel_name() == "tcgen05-pair128"
        outs.append(_bits(out).copy())
        rows.append(np.stack([ctx.read_rows(0, seqs[b], S, 1)[0] for b in range(B)]))
        ctx.close()
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(rows[0], rows[1])
    want_rows = oracle.append_rows(_bits(kv), [S] * B, nw, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, DT)
    assert np.array_equal(rows[0], want_rows)
    qh, ch = _bits(q), _bits(cache)
    fulls = [np.concatenate([ch[b], want_rows[b:b + 1]]) for b in range(B)]
    want = oracle.attention_batch(qh, fulls, [S + 1] * B, wk, wv, synth.W_BF16, H, DT, min(B, os.cpu_count() or 1))
    for b in range(B):                                       # every sequence, all 128 heads
        _close(outs[0][b], want[b], f"sequence {b} at ctx {S + 1}")


def test_v2lite_shape_decode_step_at_size_all_sequences_against_the_checker(torch, oracle):
    """configs[1] shape: 16 heads, 32 sequences of ctx 8192, fp16 cache, pages in a random permutation, one decode step
    through mla_step_layers (the 16-column tcgen05 kernel).  Every sequence and head against the CPU attention; the
    appended rows bit for bit; the same logical caches under a second page permutation give identical bits."""
    from mugen_b200.mla import MlaContext
    Hs, dt, B, S = 16, synth.DT_F16, 32, 8191
    rng = np.random.default_rng(21)
    wk = synth.to_bits(rng.standard_normal((Hs * 128, 512), np.float32) * np.float32(0.02), dt)
    wv = synth.to_bits(rng.standard_normal((Hs * 128, 512), np.float32) * np.float32(0.02), dt)
    nw = synth.to_bits((1.0 + 0.1 * rng.standard_normal(512)).astype(np.float32), dt)
    g = torch.Generator(device="cuda")
    g.manual_seed(2121)
    f16 = lambda shape, scale=1.0: (torch.randn(shape, device="cuda", dtype=torch.float32, generator=g) * scale).to(torch.float16).view(torch.int16)
    cache, kv, q = f16((B, S, 576)), f16((B, 576)), f16((B, Hs, 192), 0.9)
    outs, rows = [], []
    for shuffle in (5, 91):
        ctx = MlaContext(n_layers=1, n_heads=Hs, dtype=dt, n_pages=B * 129 + 16, max_seqs=B, max_seq_len=S + 65,
                         kernel=capi.KERNEL_AUTO, **YARN)
        ctx.shuffle_free_pages(shuffle)
        ctx.set_layer_weights(0, wk, wv, synth.W_F16, nw)
        seqs = []
        for b in range(B):
            sq = ctx.seq_create()
            ctx.write_rows(0, sq, 0, cache[b])
            ctx.advance_seq_len(sq, S)
            seqs.append(sq)
        out = torch.zeros((B, Hs, 128), dtype=torch.int16, device="cuda")
        ctx.step_begin(seqs)
        ctx.step_layers(0, 1, kv[None], q[None], out[None])
        ctx.step_end()
        assert ctx.status() == 0 and ctx.kernel_name() == "tcgen05-t16"
        outs.append(_bits(out).copy())
        rows.append(np.stack([ctx.read_rows(0, seqs[b], S, 1)[0] for b in range(B)]))
        ctx.close()
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(rows[0], rows[1])
    want_rows = oracle.append_rows(_bits(kv), [S] * B, nw, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, dt)
    assert np.array_equal(rows[0], want_rows)
    qh, ch = _bits(q), _bits(cache)
    fulls = [np.concatenate([ch[b], want_rows[b:b + 1]]) for b in range(B)]
    want = oracle.attention_batch(qh, fulls, [S + 1] * B, wk, wv, synth.W_F16, Hs, dt, min(B, os.cpu_count() or 1))
    for b in range(B):
        mx, rl = synth.error_norms(outs[0][b], want[b], dt, dt)
        assert mx <= MAX_ABS and rl <= REL_L2, f"sequence {b}: max-abs {mx:.3e}, rel-L2 {rl:.3e}"


def test_ctx131072_kv_range_split_equals_whole(torch, oracle):
    """configs[3] shape: one sequence of 131072 tokens (after the append), 128 heads.  The sequence held by
    one context, and cut into 4 page-aligned KV ranges held by 4 contexts whose partial states are merged,
    give the same output within the tolerance; the first 32 heads are checked against the CPU attention."""
    from mugen_b200.mla import MlaContext
    S, G = 131071, 4
    wk, wv, nw = _weights(2)
    cache = _rand_bf16(torch, (S, 576), 21)
    kv = _rand_bf16(torch, (1, 576), 22)
    q = _rand_bf16(torch, (1, H, 192), 23, 0.9)

    whole = MlaContext(n_layers=1, n_heads=H, dtype=DT, n_pages=2050, max_seqs=1, max_seq_len=S + 65,
                       kernel=capi.KERNEL_AUTO, **YARN)
    whole.shuffle_free_pages(5)
    whole.set_layer_weights(0, wk, wv, synth.W_BF16, nw)
    s = whole.seq_create()
    whole.write_rows(0, s, 0, cache)
    whole.advance_seq_len(s, S)
    out_whole = torch.zeros((1, H, 128), dtype=torch.int16, device="cuda")
    whole.step_begin([s])
    whole.step_layers(0, 1, kv[None], q[None], out_whole[None])
    whole.step_end()
    assert whole.status() == 0
    new_row = whole.read_rows(0, s, S, 1)
    want_row = oracle.append_rows(_bits(kv), [S], nw, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, DT)
    assert np.array_equal(new_row, want_row)

    cuts = [0, 32768, 65536, 98304, S]                      # page-aligned ranges; the last one owns the tail
    parts = torch.zeros((G, 1, H, 514), dtype=torch.float32, device="cuda")
    shards = []
    for g in range(G):
        n = cuts[g + 1] - cuts[g]
        c = MlaContext(n_layers=1, n_heads=H, dtype=DT, n_pages=n // 64 + 4, max_seqs=1, max_seq_len=n + 65,
                       max_position=S + 65, kernel=capi.KERNEL_AUTO, **YARN)
        c.set_layer_weights(0, wk, wv, synth.W_BF16, nw)
        sg = c.seq_create()
        c.seq_set_base(sg, cuts[g])
        c.write_rows(0, sg, 0, cache[cuts[g]:cuts[g + 1]])
        c.advance_seq_len(sg, n)
        c.step_begin([sg], [1 if g == G - 1 else 0])
        c.step_append(0, kv)
        c.step_attend_partial(0, q, parts[g])
        c.step_end()
        assert c.status() == 0
        shards.append(c)
    out_split = torch.zeros((1, H, 128), dtype=torch.int16, device="cuda")
    shards[0].merge_partials(0, G, 1, parts, out_split)
    assert shards[0].status() == 0
    _close(_bits(out_split)[0], _bits(out_whole)[0], "4 KV ranges against the whole sequence")

    hs = 32                                                  # heads are independent: check the first 32 on the CPU
    full = np.concatenate([_bits(cache), want_row])
    want = oracle.attention(_bits(q)[0, :hs], full, S + 1, wk[:hs * 128], wv[:hs * 128], synth.W_BF16, hs, DT)
    _close(_bits(out_whole)[0, :hs], want, "whole sequence, heads 0-31")
    _close(_bits(out_split)[0, :hs], want, "merged ranges, heads 0-31")
    for c in shards:
        c.close()
    whole.close()


def test_prefill_chunk_on_existing_context_with_ragged_decode_rows(torch, oracle):
    """configs[4] shape in small: a 512-token chunk appended at start_position 8192 next to ragged decode
    rows in ONE step, 128 heads.  Chunk token t must see exactly [0, 8192+t+1) (transformer.cpp:1325-1337):
    its output equals an explicit-length call at that length, and the CPU attention on 8 heads."""
    from mugen_b200.mla import MlaContext
    start, N = 8192, 512
    dec_lens = [int(n) for n in synth.ragged_lengths(42, 3, 256, 32768)]
    wk, wv, nw = _weights(3)
    lens = dec_lens + [start]
    n_new = [1] * len(dec_lens) + [N]
    R = sum(n_new)
    caches = [_rand_bf16(torch, (n, 576), 31 + i) for i, n in enumerate(lens)]
    kv = _rand_bf16(torch, (R, 576), 41)
    q = _rand_bf16(torch, (R, H, 192), 42, 0.9)
    pages = sum((n + m + 63) // 64 + 1 for n, m in zip(lens, n_new)) + 8
    ctx = MlaContext(n_layers=1, n_heads=H, dtype=DT, n_pages=pages, max_seqs=len(lens), max_seq_len=max(lens) + N + 64,
                     max_rows=R, kernel=capi.KERNEL_AUTO, **YARN)
    ctx.shuffle_free_pages(8)
    ctx.set_layer_weights(0, wk, wv, synth.W_BF16, nw)
    seqs = []
    for c_, n in zip(caches, lens):
        s = ctx.seq_create()
        ctx.write_rows(0, s, 0, c_)
        ctx.advance_seq_len(s, n)
        seqs.append(s)
    out = torch.zeros((R, H, 128), dtype=torch.int16, device="cuda")
    ctx.step_begin(seqs, n_new)
    ctx.step_layers(0, 1, kv[None], q[None], out[None])
    ctx.step_end()
    assert ctx.status() == 0
    assert [ctx.seq_len(s) for s in seqs] == [n + m for n, m in zip(lens, n_new)]
    got = _bits(out)
    r0 = len(dec_lens)                                       # first row of the chunk
    pos = dec_lens + [start + t for t in range(N)]
    want_rows = oracle.append_rows(_bits(kv), pos, nw, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, DT)
    assert np.array_equal(ctx.read_rows(0, seqs[-1], start, N), want_rows[r0:])
    # the same queries through the explicit-length call: other split points, same visible rows
    ts = [0, 1, 63, 64, 300, N - 1]
    out2 = torch.zeros((len(ts), H, 128), dtype=torch.int16, device="cuda")
    ctx.attend_rows(0, [seqs[-1]] * len(ts), [start + t + 1 for t in ts], q[[r0 + t for t in ts]].contiguous(), out2)
    assert ctx.status() == 0
    got2 = _bits(out2)
    for k, t in enumerate(ts):
        _close(got[r0 + t], got2[k], f"chunk token {t} against the explicit-length call")
    hs = 8
    chunk_cache = np.concatenate([_bits(caches[-1]), want_rows[r0:]])
    for t in (0, N - 1):
        want = oracle.attention(_bits(q)[r0 + t, :hs], chunk_cache, start + t + 1, wk[:hs * 128], wv[:hs * 128],
                                synth.W_BF16, hs, DT)
        _close(got[r0 + t, :hs], want, f"chunk token {t}, heads 0-7")
    b = int(np.argmax(dec_lens))                             # the longest decode row
    full = np.concatenate([_bits(caches[b]), want_rows[b:b + 1]])
    want = oracle.attention(_bits(q)[b, :hs], full, dec_lens[b] + 1, wk[:hs * 128], wv[:hs * 128], synth.W_BF16, hs, DT)
    _close(got[b, :hs], want, f"decode row of length {dec_lens[b] + 1}, heads 0-7")
    ctx.close()


@pytest.mark.parametrize("start", [0, 8192])
def test_config5_at_size_ragged_decode_rows_and_four_4096_token_chunks_in_one_step(torch, oracle, start):
    """BASELINE.json configs[4] at its stated size, one layer, ONE scheduler step: 128 decode sequences with
    log-uniform lengths 256..32768 plus 4 sequences that each append a 4096-token chunk at start_position 0 or 8192,
    128 heads, bf16.  Chunk token t attends [0, start+t+1) (transformer.cpp:1325-1337).  Checked: every appended row
    bit-equal to the checker; chunk tokens at the first, last and page-edge positions of two chunks, and the
    longest and shortest decode rows, against the CPU attention on 8 heads; sequence counters moved by n_new."""
    from mugen_b200.mla import MlaContext
    N, n_chunks = 4096, 4
    dec_lens = [int(n) for n in synth.ragged_lengths(42, 128, 256, 32768)]
    wk, wv, nw = _weights(5 + start)
    lens = dec_lens + [start] * n_chunks
    n_new = [1] * len(dec_lens) + [N] * n_chunks
    R = sum(n_new)
    caches = [_rand_bf16(torch, (n, 576), 500 + i) if n else None for i, n in enumerate(lens)]
    kv = _rand_bf16(torch, (R, 576), 61)
    q = _rand_bf16(torch, (R, H, 192), 62, 0.9)
    pages = sum((n + m + 63) // 64 + 1 for n, m in zip(lens, n_new)) + 8
    ctx = MlaContext(n_layers=1, n_heads=H, dtype=DT, n_pages=pages, max_seqs=len(lens), max_seq_len=max(lens) + N + 64,
                     max_rows=R, kernel=capi.KERNEL_AUTO, **YARN)
    ctx.shuffle_free_pages(9)
    ctx.set_layer_weights(0, wk, wv, synth.W_BF16, nw)
    seqs = []
    for c_, n in zip(caches, lens):
        s = ctx.seq_create()
        if n:
            ctx.write_rows(0, s, 0, c_)
        ctx.advance_seq_len(s, n)
        seqs.append(s)
    out = torch.zeros((R, H, 128), dtype=torch.int16, device="cuda")
    ctx.step_begin(seqs, n_new)
    ctx.step_layers(0, 1, kv[None], q[None], out[None])
    ctx.step_end()
    torch.cuda.synchronize()
    assert ctx.status() == 0
    assert [ctx.seq_len(s) for s in seqs] == [n + m for n, m in zip(lens, n_new)]
    got, qh, kvh = _bits(out), _bits(q), _bits(kv)
    # ---- appended rows: all 16,512 of them, bit for bit
    pos = list(dec_lens)
    for _ in range(n_chunks):
        pos += [start + t for t in range(N)]
    want_rows = oracle.append_rows(kvh, pos, nw, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, DT)
    nd = len(dec_lens)
    for b in range(nd):
        assert np.array_equal(ctx.read_rows(0, seqs[b], dec_lens[b], 1)[0], want_rows[b]), f"decode row {b}"
    for c in range(n_chunks):
        r0 = nd + c * N
        assert np.array_equal(ctx.read_rows(0, seqs[nd + c], start, N), want_rows[r0:r0 + N]), f"chunk {c}"
    # ---- attention: sampled chunk tokens and decode rows against the CPU on 8 heads
    hs = 8
    for c in (0, n_chunks - 1):
        r0 = nd + c * N
        rows_c = want_rows[r0:r0 + N]
        chunk_cache = rows_c if start == 0 else np.concatenate([_bits(caches[nd + c]), rows_c])
        for t in (0, 1, 63, 64, 65, 2047, N - 65, N - 1):
            want = oracle.attention(qh[r0 + t, :hs].copy(), chunk_cache, start + t + 1, wk[:hs * 128], wv[:hs * 128],
                                    synth.W_BF16, hs, DT)
            _close(got[r0 + t, :hs], want, f"chunk {c} token {t} (start {start}), heads 0-7")
    for b in (int(np.argmax(dec_lens)), int(np.argmin(dec_lens)), 17):
        full = np.concatenate([_bits(caches[b]), want_rows[b:b + 1]])
        want = oracle.attention(qh[b, :hs].copy(), full, dec_lens[b] + 1, wk[:hs * 128], wv[:hs * 128], synth.W_BF16, hs, DT)
        _close(got[b, :hs], want, f"decode row {b} of length {dec_lens[b] + 1}, heads 0-7")
    ctx.close()


def test_speculative_verify_steps_with_rollback_at_batch_64(torch, oracle):
    """The request-level contract of the reference's speculative decoding at scale (USPPScheduler::decode_step,
    uspp_scheduler.cpp:176-298; verify :550-580): every step verifies K+1 = 5 positions per sequence as one small
    causal chunk, then keeps ctx + n_accepted + 1 rows and rolls the rest back (truncate), and the next step appends
    over the rolled-back rows.  64 sequences of ragged lengths, 128 heads, bf16, 4 steps with seeded acceptance counts.
    Checked: counters after every rollback; after the last step, for sampled sequences, the surviving cache rows
    equal the checker's append of the accepted tokens only (rolled-back rows were overwritten or dropped), and the
    outputs of the last verify chunk match the CPU attention over exactly those rows on 8 heads."""
    from mugen_b200.mla import MlaContext
    B, K1, steps = 64, 5, 4
    rng = np.random.default_rng(99)
    lens0 = [int(n) for n in synth.ragged_lengths(7, B, 300, 6000)]
    wk, wv, nw = _weights(9)
    caches = [_rand_bf16(torch, (n, 576), 900 + i) for i, n in enumerate(lens0)]
    pages = sum((n + steps * K1 + 63) // 64 + 1 for n in lens0) + 8
    ctx = MlaContext(n_layers=1, n_heads=H, dtype=DT, n_pages=pages, max_seqs=B, max_seq_len=max(lens0) + steps * K1 + 64,
                     max_rows=B * K1, kernel=capi.KERNEL_AUTO, **YARN)
    ctx.shuffle_free_pages(4)
    ctx.set_layer_weights(0, wk, wv, synth.W_BF16, nw)
    seqs = []
    for c_, n in zip(caches, lens0):
        s = ctx.seq_create()
        ctx.write_rows(0, s, 0, c_)
        ctx.advance_seq_len(s, n)
        seqs.append(s)
    cur = list(lens0)
    kept = [[] for _ in range(B)]            # per sequence: (position, kv_a bits) of every row that survived
    for step in range(steps):
        kv = _rand_bf16(torch, (B * K1, 576), 2000 + step)
        q = _rand_bf16(torch, (B * K1, H, 192), 3000 + step, 0.9)
        out = torch.zeros((B * K1, H, 128), dtype=torch.int16, device="cuda")
        ctx.step_begin(seqs, [K1] * B)
        ctx.step_layers(0, 1, kv[None], q[None], out[None])
        ctx.step_end()
        assert [ctx.seq_len(s) for s in seqs] == [n + K1 for n in cur]
        n_acc = rng.integers(0, K1, B)       # accepted drafts 0..K; the re-evaluated token always stays
        keep = [cur[b] + int(n_acc[b]) + 1 for b in range(B)]
        ctx.rollback(seqs, keep)
        assert [ctx.seq_len(s) for s in seqs] == keep
        kvh = _bits(kv)
        for b in range(B):
            for t in range(int(n_acc[b]) + 1):
                kept[b].append((cur[b] + t, kvh[b * K1 + t]))
        last = (list(cur), kvh, _bits(q), _bits(out), n_acc.copy())
        cur = keep
    assert ctx.status() == 0
    ctx.rollback(seqs, [n + 10 for n in cur])                    # keep length above seq_len: left alone (the reference's guard)
    assert [ctx.seq_len(s) for s in seqs] == cur
    start, kvh, qh, outh, n_acc = last
    hs = 8
    for b in (0, 17, int(np.argmax(lens0)), B - 1):
        pos = [p for p, _ in kept[b]]
        assert pos == list(range(lens0[b], cur[b]))               # contiguous: rollbacks left no holes
        want_rows = oracle.append_rows(np.stack([r for _, r in kept[b]]), pos, nw, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, DT)
        assert np.array_equal(ctx.read_rows(0, seqs[b], lens0[b], cur[b] - lens0[b]), want_rows), f"sequence {b}"
        # the last verify chunk saw the surviving rows below its start plus its own K+1 appended rows
        chunk_rows = oracle.append_rows(kvh[b * K1:(b + 1) * K1], list(range(start[b], start[b] + K1)), nw,
                                        YARN["rms_norm_eps"], 40.0, 4096, 10000.0, DT)
        below = want_rows[:start[b] - lens0[b]]
        full = np.concatenate([_bits(caches[b]), below, chunk_rows])
        for t in (0, K1 - 1):
            want = oracle.attention(qh[b * K1 + t, :hs].copy(), full, start[b] + t + 1, wk[:hs * 128], wv[:hs * 128],
                                    synth.W_BF16, hs, DT)
            _close(outh[b * K1 + t, :hs], want, f"sequence {b}, verify position {t}")
    ctx.close()
