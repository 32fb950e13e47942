"""Parity of the CUDA path (through the C ABI) with the CPU checker.

Bars: the append is bit-exact; attention outputs stay within max-abs 2e-2 and relative-L2 5e-3
of the CPU result on the same seeded inputs (the tolerance the task states for fp16/bf16
caches).  Every test runs once per attention kernel family the library offers.
"""
import base64
import os

import numpy as np
import pytest

from mugen_b200 import capi, synth

pytestmark = pytest.mark.gpu

MAX_ABS, REL_L2 = 2e-2, 5e-3
YARN = dict(rope_theta=10000.0, rope_scaling_factor=40.0, rope_original_ctx=4096, rms_norm_eps=1e-6)

KERNELS = [capi.KERNEL_MMA, capi.KERNEL_TCGEN05, capi.KERNEL_TCGEN05_PAIR128, capi.KERNEL_TCGEN05_T16]
if os.environ.get("MLA_TEST_KERNELS"):
    KERNELS = [int(k) for k in os.environ["MLA_TEST_KERNELS"].split(",")]


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch


def _dev(torch, bits: np.ndarray):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()


def _host(t) -> np.ndarray:
    return t.cpu().numpy().view(np.uint16)


def make_ctx(case: synth.LayerCase, kernel, n_layers=1, extra_pages=8, max_rows=0, shuffle=None, **kw):
    from mugen_b200.mla import MlaContext
    pages = sum((s + 63) // 64 + 1 for s in case.seq_lens) + extra_pages
    args = dict(n_layers=n_layers, n_heads=case.n_heads, dtype=case.dt, n_pages=pages,
                max_seqs=max(len(case.seq_lens), 1) + 2, max_seq_len=max(case.seq_lens + [64]) + 256,
                max_rows=max_rows, kernel=kernel, **YARN)
    args.update(kw)
    ctx = MlaContext(**args)
    if shuffle is not None:
        ctx.shuffle_free_pages(shuffle)
    for layer in range(n_layers):
        ctx.set_layer_weights(layer, case.w_uk, case.w_uv, case.w_type, case.norm_w)
    return ctx


def fill(torch, ctx, case, layer=0, upto=None):
    seqs = []
    for b, cache in enumerate(case.caches):
        s = ctx.seq_create()
        n = case.seq_lens[b] if upto is None else upto[b]
        if n:
            ctx.write_rows(layer, s, 0, _dev(torch, cache[:n]))
        ctx.advance_seq_len(s, n)
        seqs.append(s)
    return seqs


def check_close(got_bits, want_bits, dt, what=""):
    mx, rl = synth.error_norms(got_bits, want_bits, dt, dt)
    assert mx <= MAX_ABS and rl <= REL_L2, f"{what}: max-abs {mx:.3e}, rel-L2 {rl:.3e}"
    return mx, rl


def oracle_out(oracle, case, b, seq_len=None, q=None):
    n = case.seq_lens[b] if seq_len is None else seq_len
    return oracle.attention(case.q[b] if q is None else q, case.caches[b], n, case.w_uk, case.w_uv,
                            case.w_type, case.n_heads, case.dt)


# ---------------------------------------------------------------------------------------------
# append: bit-exact
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", [synth.DT_F16, synth.DT_BF16])
@pytest.mark.parametrize("factor,ctx_len", [(40.0, 4096), (0.0, 0)])
def test_append_bit_exact(torch, oracle, dt, factor, ctx_len):
    positions = [0, 1, 31, 32, 63, 64, 65, 127, 128, 1000, 4095, 4096, 8191, 20000, 40000]
    case = synth.make_layer_case(11, 4, [1] * len(positions), dt)
    kw = dict(YARN, rope_scaling_factor=factor, rope_original_ctx=ctx_len)
    from mugen_b200.mla import MlaContext
    ctx = MlaContext(n_layers=2, n_heads=4, dtype=dt, n_pages=640, max_seqs=4,
                     max_seq_len=40064, max_rows=len(positions), kernel=capi.KERNEL_MMA, **kw)
    for layer in range(2):
        ctx.set_layer_weights(layer, case.w_uk, case.w_uv, case.w_type, case.norm_w)
    s = ctx.seq_create()
    ctx.append_rows(1, [s] * len(positions), positions, _dev(torch, case.kv_a))
    want = oracle.append_rows(case.kv_a, positions, case.norm_w, kw["rms_norm_eps"], factor, ctx_len,
                              kw["rope_theta"], dt)
    for i, p in enumerate(positions):
        got = ctx.read_rows(1, s, p, 1)[0]
        assert np.array_equal(got, want[i]), f"position {p}"
    # the other layer's slots were not touched
    assert not ctx.read_rows(0, s, 0, 64).any()
    assert ctx.status() == 0
    ctx.close()


def test_append_reproduces_the_rows_of_the_reference_forward(torch, golden):
    """Golden rows written by the reference's own inline append (RMSNorm + NeoX/YaRN RoPE + scatter inside
    forward(), transformer.cpp:3930-3987, run on a tiny deepseek2 GGUF file): the append kernel, fed the kv_a the
    reference's code read, must store the very bits the reference stored."""
    import base64
    from mugen_b200.mla import MlaContext
    unb = lambda t: np.frombuffer(base64.b64decode(t), np.uint16).copy()
    groups = {}
    for c in golden["append"]:
        groups.setdefault((c["model"], c["layer"]), []).append(c)
    assert len(groups) >= 4
    dummy_w = np.zeros((128, 512), np.uint16)
    for (model, layer), entries in groups.items():
        c0 = entries[0]
        assert c0["source"].startswith("reference forward()") and c0["dt"] == synth.DT_F16
        top = max(c["position"] for c in entries)
        ctx = MlaContext(n_layers=1, n_heads=1, dtype=synth.DT_F16, n_pages=len(entries) + 1, max_seqs=1,
                         max_seq_len=64, max_position=top + 1, max_rows=len(entries), kernel=capi.KERNEL_MMA, rope_theta=c0["theta"],
                         rope_scaling_factor=c0["factor"], rope_original_ctx=c0["orig_ctx"], rms_norm_eps=c0["eps"])
        ctx.set_layer_weights(0, dummy_w, dummy_w, synth.W_F16, unb(c0["norm_w"]))
        # one sequence per entry would need a page table per position; instead place each row at its position
        # modulo the page size (the rotation uses the true position through a base offset)
        for c in entries:
            s = ctx.seq_create()
            ctx.seq_set_base(s, c["position"] - c["position"] % 64)
            ctx.append_rows(0, [s], [c["position"]], _dev(torch, unb(c["kv_a"])[None]))
            got = ctx.read_rows(0, s, c["position"] % 64, 1)[0]
            assert np.array_equal(got, unb(c["row"])), (model, layer, c["position"])
            ctx.seq_free(s)
        assert ctx.status() == 0
        ctx.close()


def test_append_many_rows_bit_exact(torch, oracle):
    """A 300-row chunk appended in one call (the batched twin, transformer.cpp:1263-1323)."""
    n = 300
    case = synth.make_layer_case(12, 2, [1] * n, synth.DT_F16)
    from mugen_b200.mla import MlaContext
    ctx = MlaContext(n_layers=1, n_heads=2, dtype=synth.DT_F16, n_pages=8, max_seqs=2, max_seq_len=512,
                     max_rows=n, kernel=capi.KERNEL_MMA, **YARN)
    ctx.set_layer_weights(0, case.w_uk, case.w_uv, case.w_type, case.norm_w)
    s = ctx.seq_create()
    pos = list(range(7, 7 + n))
    ctx.append_rows(0, [s] * n, pos, _dev(torch, case.kv_a))
    want = oracle.append_rows(case.kv_a, pos, case.norm_w, YARN["rms_norm_eps"], 40.0, 4096, 10000.0,
                              synth.DT_F16)
    assert np.array_equal(ctx.read_rows(0, s, 7, n), want)
    ctx.close()


# ---------------------------------------------------------------------------------------------
# attention vs the CPU checker
# ---------------------------------------------------------------------------------------------
ATTN_CASES = [
    # heads, seq_lens, dtype, w_type, q_scale
    (16, [1], synth.DT_F16, synth.W_F16, 1.0),
    (16, [63, 64, 65], synth.DT_F16, synth.W_F16, 1.0),
    (16, [2048], synth.DT_F16, synth.W_F16, 1.0),            # configs[0] shape
    (16, [700, 33, 1500, 256], synth.DT_BF16, synth.W_BF16, 1.0),
    (128, [513, 100], synth.DT_BF16, synth.W_BF16, 1.0),      # V3 head count
    (128, [300], synth.DT_F16, synth.W_F16, 6.0),             # peaky softmax: rescaling exercised
    (64, [1000, 31], synth.DT_BF16, synth.W_BF16, 8.0),
    (5, [129, 1], synth.DT_F16, synth.W_F16, 1.0),            # head count not a tile multiple
    (16, [384], synth.DT_F16, synth.W_Q8_0, 1.0),
    (16, [384], synth.DT_F16, synth.W_Q4_0, 1.0),
]


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("n_heads,seq_lens,dt,w_type,q_scale", ATTN_CASES)
def test_attend_matches_cpu(torch, oracle, kernel, n_heads, seq_lens, dt, w_type, q_scale):
    case = synth.make_layer_case(500 + n_heads + sum(seq_lens), n_heads, seq_lens, dt, w_type, q_scale)
    ctx = make_ctx(case, kernel, shuffle=3)
    seqs = fill(torch, ctx, case)
    out = torch.zeros((len(seq_lens), n_heads, 128), dtype=torch.int16, device="cuda")
    ctx.attend_rows(0, seqs, seq_lens, _dev(torch, case.q), out)
    got = _host(out)
    assert ctx.status() == 0
    for b in range(len(seq_lens)):
        check_close(got[b], oracle_out(oracle, case, b), dt, f"seq {b} len {seq_lens[b]}")
    ctx.close()


@pytest.mark.parametrize("kernel", KERNELS)
def test_golden_reference_outputs(torch, golden, kernel):
    """Against fixtures produced by the reference's own cpu_mla_attention."""
    for c in golden["attention"]:
        case = synth.make_layer_case(c["seed"], c["n_heads"], [c["seq_len"]], synth.DT_F16, c["w_type"],
                                     c["q_scale"], c["exact_in_both"])
        assert case.digest() == c["inputs_sha256"]
        ctx = make_ctx(case, kernel)
        seqs = fill(torch, ctx, case)
        out = torch.zeros((1, c["n_heads"], 128), dtype=torch.int16, device="cuda")
        ctx.attend_rows(0, seqs, [c["seq_len"]], _dev(torch, case.q), out)
        want = np.frombuffer(base64.b64decode(c["out_f16"]), np.uint16).reshape(c["n_heads"], 128)
        check_close(_host(out)[0], want, synth.DT_F16, f"golden seed {c['seed']}")
        ctx.close()


@pytest.mark.parametrize("kernel", KERNELS)
def test_bf16_cache_against_f16_reference_values(torch, oracle, kernel):
    """bf16 context on numbers exact in both formats, checked against the f16 CPU result."""
    c16 = synth.make_layer_case(77, 32, [900], synth.DT_F16, synth.W_F16, 1.0, True)
    want = oracle_out(oracle, c16, 0)
    tobf = lambda b: synth.to_bits(synth.from_bits(b, synth.DT_F16), synth.DT_BF16)
    cbf = synth.LayerCase(32, synth.DT_BF16, synth.W_BF16, [900], tobf(c16.q), [tobf(c16.caches[0])],
                          tobf(c16.w_uk), tobf(c16.w_uv), c16.w_uk_f32, c16.w_uv_f32, tobf(c16.norm_w),
                          tobf(c16.kv_a))
    ctx = make_ctx(cbf, kernel)
    seqs = fill(torch, ctx, cbf)
    out = torch.zeros((1, 32, 128), dtype=torch.int16, device="cuda")
    ctx.attend_rows(0, seqs, [900], _dev(torch, cbf.q), out)
    mx, rl = synth.error_norms(_host(out)[0], want, synth.DT_BF16, synth.DT_F16)
    assert mx <= MAX_ABS and rl <= REL_L2, (mx, rl)
    ctx.close()


@pytest.mark.parametrize("kernel", KERNELS)
def test_attend_shorter_than_cache_and_empty(torch, oracle, kernel):
    """attend_len is the caller's (cpu_mla_attention's seq_len argument), not the cache length;
    a zero-length row yields zeros."""
    case = synth.make_layer_case(91, 16, [500, 200], synth.DT_F16)
    ctx = make_ctx(case, kernel)
    seqs = fill(torch, ctx, case)
    lens = [131, 0]
    out = torch.full((2, 16, 128), 7, dtype=torch.int16, device="cuda")
    ctx.attend_rows(0, seqs, lens, _dev(torch, case.q), out)
    got = _host(out)
    check_close(got[0], oracle_out(oracle, case, 0, 131), synth.DT_F16)
    assert not got[1].any()
    ctx.close()


# ---------------------------------------------------------------------------------------------
# the decode-step scheduler
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("dt", [synth.DT_F16, synth.DT_BF16])
def test_decode_steps_multi_layer(torch, oracle, kernel, dt):
    """3 decode steps over 2 layers and 3 ragged sequences: append-then-attend ordering,
    counters moving once per step, truncate rollback and re-append (speculative-decode contract)."""
    H, L = 16, 2
    lens0 = [130, 64, 5]
    cases = [synth.make_layer_case(300 + l, H, [n + 8 for n in lens0], dt) for l in range(L)]
    from mugen_b200.mla import MlaContext
    ctx = MlaContext(n_layers=L, n_heads=H, dtype=dt, n_pages=16, max_seqs=4, max_seq_len=512,
                     kernel=kernel, **YARN)
    ctx.shuffle_free_pages(9)
    host = [[None] * 3 for _ in range(L)]   # the CPU-side mirror of each (layer, seq) cache
    seqs = [ctx.seq_create() for _ in lens0]
    for l in range(L):
        ctx.set_layer_weights(l, cases[l].w_uk, cases[l].w_uv, cases[l].w_type, cases[l].norm_w)
        for b, s in enumerate(seqs):
            host[l][b] = cases[l].caches[b].copy()
            ctx.write_rows(l, s, 0, _dev(torch, host[l][b][:lens0[b]]))
    for b, s in enumerate(seqs):
        ctx.advance_seq_len(s, lens0[b])
    rng = np.random.default_rng(5)

    def one_step(expect_len):
        ctx.step_begin(seqs)
        for l in range(L):
            kv_a = synth.to_bits(rng.standard_normal((3, 576), np.float32), dt)
            q = synth.to_bits(rng.standard_normal((3, H, 192), np.float32) * np.float32(0.9), dt)
            out = torch.zeros((3, H, 128), dtype=torch.int16, device="cuda")
            ctx.step_append(l, _dev(torch, kv_a))
            ctx.step_attend(l, _dev(torch, q), out)
            got = _host(out)
            pos = [expect_len[b] for b in range(3)]
            rows = oracle.append_rows(kv_a, pos, cases[l].norm_w, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, dt)
            for b in range(3):
                host[l][b][pos[b]] = rows[b]
                assert np.array_equal(ctx.read_rows(l, seqs[b], pos[b], 1)[0], rows[b])
                want = oracle.attention(q[b], host[l][b], pos[b] + 1, cases[l].w_uk, cases[l].w_uv,
                                        cases[l].w_type, H, dt)
                check_close(got[b], want, dt, f"layer {l} seq {b}")
            # counters do not move inside the step
            assert [ctx.seq_len(s) for s in seqs] == expect_len
        ctx.step_end()
        return [n + 1 for n in expect_len]

    cur = list(lens0)
    cur = one_step(cur)
    cur = one_step(cur)
    assert [ctx.seq_len(s) for s in seqs] == [n + 2 for n in lens0]
    # roll back one token on sequence 0 (rejected draft), then continue: the row is rewritten
    ctx.truncate(seqs[0], cur[0] - 1)
    cur[0] -= 1
    cur = one_step(cur)
    assert ctx.status() == 0
    ctx.close()


@pytest.mark.parametrize("kernel", KERNELS)
def test_step_layers_equals_per_layer_calls(torch, kernel):
    """The multi-layer call runs the append inside the absorb launch (same arithmetic, other blocks):
    outputs and appended rows are bit-identical to the per-layer calls with their separate append kernel."""
    H, L, dt, lens = 64, 3, synth.DT_BF16, [200, 65]
    case = synth.make_layer_case(333, H, [n + 1 for n in lens], dt)
    rng = np.random.default_rng(4)
    kv = _dev(torch, synth.to_bits(rng.standard_normal((L, 2, 576), np.float32), dt))
    q = _dev(torch, synth.to_bits(rng.standard_normal((L, 2, H, 192), np.float32) * np.float32(0.9), dt))
    outs, rows = [], []
    for mode in (0, 1):
        ctx = make_ctx(case, kernel, n_layers=L)
        seqs = []
        for b, n in enumerate(lens):
            s_ = ctx.seq_create()
            for l in range(L):
                ctx.write_rows(l, s_, 0, _dev(torch, case.caches[b][:n]))
            ctx.advance_seq_len(s_, n)
            seqs.append(s_)
        out = torch.zeros((L, 2, H, 128), dtype=torch.int16, device="cuda")
        ctx.step_begin(seqs)
        if mode == 0:
            for l in range(L):
                ctx.step_append(l, kv[l])
                ctx.step_attend(l, q[l], out[l])
        else:
            ctx.step_layers(0, L, kv, q, out)
        ctx.step_end()
        outs.append(_host(out).copy())
        rows.append(np.stack([ctx.read_rows(l, seqs[b], lens[b], 1) for l in range(L) for b in range(2)]))
        assert ctx.status() == 0
        ctx.close()
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(rows[0], rows[1])


@pytest.mark.parametrize("dt", [synth.DT_F16, synth.DT_BF16])
def test_q_rope_inside_the_absorb_kernel(torch, oracle, dt):
    """Step E of the reference's decode driver (transformer.cpp:3882-3921) folded into the absorb
    kernel: queries passed before their RoPE give bit-identical outputs to queries the checker
    rotated at the same positions, for decode rows, a prefill chunk (one position per row) and the
    explicit-length call; and they agree with the CPU attention over the rotated queries."""
    H, lens, chunk = 64, [130, 64], 5
    case = synth.make_layer_case(777, H, [n + chunk for n in lens], dt)
    rng = np.random.default_rng(12)
    n_new = [1, chunk]
    R = sum(n_new)
    kv = synth.to_bits(rng.standard_normal((R, 576), np.float32), dt)
    q_raw = synth.to_bits(rng.standard_normal((R, H, 192), np.float32) * np.float32(0.9), dt)
    pos = [lens[0]] + [lens[1] + t for t in range(chunk)]
    q_rot = q_raw.copy()
    for r in range(R):
        q_rot[r] = oracle.q_rope(q_raw[r], pos[r], 40.0, 4096, 10000.0, dt)
    assert not np.array_equal(q_rot, q_raw)
    outs = []
    for in_kernel in (False, True):
        ctx = make_ctx(case, capi.KERNEL_AUTO, max_rows=R)
        seqs = fill(torch, ctx, case, upto=lens)
        ctx.set_q_rope(in_kernel)
        out = torch.zeros((R, H, 128), dtype=torch.int16, device="cuda")
        ctx.step_begin(seqs, n_new)
        ctx.step_layers(0, 1, _dev(torch, kv)[None], _dev(torch, q_raw if in_kernel else q_rot)[None], out[None])
        ctx.step_end()
        got = [_host(out).copy()]
        # explicit-length call: the query stands at the last attended position
        out2 = torch.zeros((2, H, 128), dtype=torch.int16, device="cuda")
        sel = [0, R - 1]
        ctx.attend_rows(0, seqs, [lens[0] + 1, lens[1] + chunk],
                        _dev(torch, (q_raw if in_kernel else q_rot)[sel]), out2)
        got.append(_host(out2).copy())
        assert ctx.status() == 0
        if in_kernel:                      # refused where a row has no position of its own
            with pytest.raises(Exception):
                ctx.step_begin(seqs, [0, 1])
        outs.append(got)
        if not in_kernel:
            rows = oracle.append_rows(kv, pos, case.norm_w, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, dt)
            cache1 = np.concatenate([case.caches[1][:lens[1]], rows[1:]])
            want = oracle.attention(q_rot[R - 1], cache1, lens[1] + chunk, case.w_uk, case.w_uv, case.w_type, H, dt)
            check_close(got[0][R - 1], want, dt, "last chunk row")
        ctx.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    for k, r in enumerate([0, R - 1]):    # other split points, so equal only within the tolerance
        check_close(outs[0][1][k], outs[0][0][r], dt, "explicit-length call")


@pytest.mark.parametrize("kernel", KERNELS)
def test_prefill_chunk_is_causal(torch, oracle, kernel):
    """A 70-token chunk appended at start_position 50 next to a plain decode row: token t attends
    [0, start+t+1) (transformer.cpp:1325-1337)."""
    H, dt = 16, synth.DT_F16
    case = synth.make_layer_case(61, H, [50 + 70, 33 + 1], dt)
    from mugen_b200.mla import MlaContext
    ctx = MlaContext(n_layers=1, n_heads=H, dtype=dt, n_pages=8, max_seqs=2, max_seq_len=256, max_rows=80,
                     kernel=kernel, **YARN)
    ctx.set_layer_weights(0, case.w_uk, case.w_uv, case.w_type, case.norm_w)
    s0, s1 = ctx.seq_create(), ctx.seq_create()
    ctx.write_rows(0, s0, 0, _dev(torch, case.caches[0][:50])); ctx.advance_seq_len(s0, 50)
    ctx.write_rows(0, s1, 0, _dev(torch, case.caches[1][:33])); ctx.advance_seq_len(s1, 33)
    rng = np.random.default_rng(8)
    kv_a = synth.to_bits(rng.standard_normal((71, 576), np.float32), dt)
    q = synth.to_bits(rng.standard_normal((71, H, 192), np.float32) * np.float32(0.9), dt)
    out = torch.zeros((71, H, 128), dtype=torch.int16, device="cuda")
    ctx.step_begin([s0, s1], [70, 1])
    assert ctx.step_info()[0] == 71
    ctx.step_append(0, _dev(torch, kv_a))
    ctx.step_attend(0, _dev(torch, q), out)
    ctx.step_end()
    got = _host(out)
    pos = list(range(50, 120)) + [33]
    rows = oracle.append_rows(kv_a, pos, case.norm_w, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, dt)
    c0 = np.concatenate([case.caches[0][:50], rows[:70]])
    c1 = np.concatenate([case.caches[1][:33], rows[70:]])
    for t in (0, 1, 13, 14, 69):
        want = oracle.attention(q[t], c0, 50 + t + 1, case.w_uk, case.w_uv, case.w_type, H, dt)
        check_close(got[t], want, dt, f"chunk token {t}")
    check_close(got[70], oracle.attention(q[70], c1, 34, case.w_uk, case.w_uv, case.w_type, H, dt), dt)
    assert ctx.seq_len(s0) == 120 and ctx.seq_len(s1) == 34
    ctx.close()


@pytest.mark.parametrize("H,dt,spec,q_rope", [
    (16, synth.DT_F16, [(50, 70), (33, 1)], False),                  # one chunk next to a decode row
    (5, synth.DT_BF16, [(0, 64), (0, 129)], False),                  # chunks from empty sequences, odd head count
    (128, synth.DT_BF16, [(100, 1), (200, 300), (64, 2), (77, 128)], False),   # chunks, a decode row and a 2-token verify row
    (32, synth.DT_F16, [(130, 200), (40, 1)], True),                 # queries arrive before their RoPE
])
def test_prefill_chunks_take_the_expanded_path(torch, oracle, H, dt, spec, q_rope):
    """Sequences that take >= 64 new tokens in a step are routed, by mla_step_layers, through the prefill kernels
    (latent rows expanded into per-head keys / values, causal flash attention), the other rows of the same step through
    the decode kernels.  Chunk token t must see exactly [0, start + t + 1) (transformer.cpp:1325-1337): sampled tokens
    of every chunk, and every other row, against the CPU attention; appended rows bit-equal to the checker's."""
    from mugen_b200.mla import MlaContext
    starts, n_new = [a for a, _ in spec], [b for _, b in spec]
    R = sum(n_new)
    case = synth.make_layer_case(4000 + H, H, [a + b for a, b in spec], dt)
    ctx = MlaContext(n_layers=1, n_heads=H, dtype=dt, n_pages=sum((a + b) // 64 + 2 for a, b in spec), max_seqs=len(spec),
                     max_seq_len=max(a + b for a, b in spec) + 64, max_rows=R, kernel=capi.KERNEL_AUTO, **YARN)
    ctx.shuffle_free_pages(3)
    ctx.set_layer_weights(0, case.w_uk, case.w_uv, case.w_type, case.norm_w)
    seqs = fill(torch, ctx, case, upto=starts)
    rng = np.random.default_rng(77)
    kv = synth.to_bits(rng.standard_normal((R, 576), np.float32), dt)
    q_raw = synth.to_bits(rng.standard_normal((R, H, 192), np.float32) * np.float32(0.9), dt)
    pos, row0 = [], []
    for a, b in spec:
        row0.append(len(pos))
        pos += [a + t for t in range(b)]
    q_rot = q_raw
    if q_rope:
        q_rot = q_raw.copy()
        for r in range(R):
            q_rot[r] = oracle.q_rope(q_raw[r], pos[r], 40.0, 4096, 10000.0, dt)
        ctx.set_q_rope(True)
    out = torch.zeros((R, H, 128), dtype=torch.int16, device="cuda")
    ctx.step_begin(seqs, n_new)
    ctx.step_layers(0, 1, _dev(torch, kv)[None], _dev(torch, q_raw)[None], out[None])
    ctx.step_end()
    assert ctx.status() == 0
    got = _host(out)
    rows = oracle.append_rows(kv, pos, case.norm_w, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, dt)
    for i, (a, b) in enumerate(spec):
        assert ctx.seq_len(seqs[i]) == a + b
        assert np.array_equal(ctx.read_rows(0, seqs[i], a, b), rows[row0[i]:row0[i] + b]), f"appended rows of sequence {i}"
        cache = np.concatenate([case.caches[i][:a], rows[row0[i]:row0[i] + b]])
        ts = sorted(set(t for t in (0, 1, 62, 63, 64, 65, 127, 128, b // 2, b - 2, b - 1) if 0 <= t < b))
        for t in ts:
            want = oracle.attention(q_rot[row0[i] + t], cache, a + t + 1, case.w_uk, case.w_uv, case.w_type, H, dt)
            check_close(got[row0[i] + t], want, dt, f"sequence {i} (start {a}, {b} new), token {t}")
    ctx.close()


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("kernel", KERNELS)
def test_kv_range_shards_merge(torch, oracle, kernel, fused):
    """One sequence cut into 3 KV ranges held by 3 contexts (stand-ins for 3 GPUs): each emits
    (m, l, acc) partials; the merged + projected result equals the unsharded CPU result.  `fused`: the append rides in
    the launch that absorbs q (mla_step_layer_partial; the shards without a new row pass no kv_a)."""
    H, dt, S = 32, synth.DT_BF16, 64 * 9 + 17
    case = synth.make_layer_case(71, H, [S], dt)
    cuts = [0, 64 * 3, 64 * 6, S]
    from mugen_b200.mla import MlaContext
    parts = torch.zeros((3, 1, H, 514), dtype=torch.float32, device="cuda")
    ctxs = []
    rng = np.random.default_rng(3)
    kv_a = synth.to_bits(rng.standard_normal((1, 576), np.float32), dt)
    new_row = oracle.append_rows(kv_a, [S], case.norm_w, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, dt)
    full = np.concatenate([case.caches[0], new_row])
    q = _dev(torch, case.q)
    for g in range(3):
        ctx = MlaContext(n_layers=1, n_heads=H, dtype=dt, n_pages=8, max_seqs=1, max_seq_len=512,
                         max_position=4096, kernel=kernel, **YARN)
        ctx.set_layer_weights(0, case.w_uk, case.w_uv, case.w_type, case.norm_w)
        s = ctx.seq_create()
        ctx.seq_set_base(s, cuts[g])
        n = cuts[g + 1] - cuts[g]
        ctx.write_rows(0, s, 0, _dev(torch, case.caches[0][cuts[g]:cuts[g + 1]]))
        ctx.advance_seq_len(s, n)
        # the shard owning the tail takes the appended token; the others only answer the query
        ctx.step_begin([s], [1 if g == 2 else 0])
        if fused:
            ctx.step_layer_partial(0, _dev(torch, kv_a) if g == 2 else None, q, parts[g])
        else:
            ctx.step_append(0, _dev(torch, kv_a))
            ctx.step_attend_partial(0, q, parts[g])
        ctx.step_end()
        if g == 2:
            assert np.array_equal(ctx.read_rows(0, s, n, 1)[0], new_row[0])
            assert ctx.seq_len(s) == n + 1
        else:
            assert ctx.seq_len(s) == n
        ctxs.append(ctx)
    out = torch.zeros((1, H, 128), dtype=torch.int16, device="cuda")
    ctxs[0].merge_partials(0, 3, 1, parts, out)
    want = oracle.attention(case.q[0], full, S + 1, case.w_uk, case.w_uv, case.w_type, H, dt)
    check_close(_host(out)[0], want, dt, "merged shards")
    # the exported state itself: m is a log2-domain maximum, l and acc follow it
    p = parts.cpu().numpy()
    for g in range(3):
        end = cuts[g + 1] + (1 if g == 2 else 0)
        ref = oracle.partial(case.q[0], full, cuts[g], end, case.w_uk, case.w_type, H, dt)
        o_gpu = p[g, 0, :, 2:] / p[g, 0, :, 1:2]
        o_ref = ref[:, 2:] / ref[:, 1:2]
        assert np.abs(o_gpu - o_ref).max() < 2e-2
        np.testing.assert_allclose(p[g, 0, :, 0], ref[:, 0] * np.log2(np.e), rtol=2e-2, atol=5e-2)
    for ctx in ctxs:
        assert ctx.status() == 0
        ctx.close()


@pytest.mark.parametrize("kernel", KERNELS)
def test_host_buffer_entry_point(torch, oracle, kernel):
    H, dt = 16, synth.DT_F16
    case = synth.make_layer_case(81, H, [200, 77], dt)
    ctx = make_ctx(case, kernel)
    seqs = fill(torch, ctx, case, upto=[199, 76])
    out = np.zeros((2, H, 128), np.uint16)
    ctx.step_begin(seqs)
    ctx.step_layer_host(0, case.kv_a, case.q, out)
    ctx.step_end()
    rows = oracle.append_rows(case.kv_a, [199, 76], case.norm_w, YARN["rms_norm_eps"], 40.0, 4096, 10000.0, dt)
    for b, n in enumerate([200, 77]):
        cache = np.concatenate([case.caches[b][:n - 1], rows[b:b + 1]])
        want = oracle.attention(case.q[b], cache, n, case.w_uk, case.w_uv, case.w_type, H, dt)
        check_close(out[b], want, dt)
    ctx.close()


def test_host_buffer_entry_point_page_locked_overlaps_and_matches_device_path(torch):
    """Page-locked caller buffers: copies run on the context's own copy streams (inputs of the next
    layer and outputs of the previous one move while a layer computes).  Two steps over three
    layers must give, bit for bit, what the device-buffer call gives, and the outputs must be in
    the host buffers when step_end returns."""
    H, L, dt, lens = 128, 3, synth.DT_BF16, [300, 65]
    case = synth.make_layer_case(91, H, [n + 2 for n in lens], dt)
    rng = np.random.default_rng(6)
    kv = [synth.to_bits(rng.standard_normal((L, 2, 576), np.float32), dt) for _ in range(2)]
    q = [synth.to_bits(rng.standard_normal((L, 2, H, 192), np.float32) * np.float32(0.9), dt) for _ in range(2)]
    results = []
    for mode in ("device", "host"):
        ctx = make_ctx(case, capi.KERNEL_AUTO, n_layers=L)
        seqs = []
        for b, n in enumerate(lens):
            s_ = ctx.seq_create()
            for l in range(L):
                ctx.write_rows(l, s_, 0, _dev(torch, case.caches[b][:n]))
            ctx.advance_seq_len(s_, n)
            seqs.append(s_)
        outs = []
        for step in range(2):
            if mode == "device":
                out = torch.zeros((L, 2, H, 128), dtype=torch.int16, device="cuda")
                ctx.step_begin(seqs)
                ctx.step_layers(0, L, _dev(torch, kv[step]), _dev(torch, q[step]), out)
                ctx.step_end()
                outs.append(_host(out).copy())
            else:
                hkv = torch.from_numpy(kv[step].view(np.int16)).pin_memory()
                hq = torch.from_numpy(q[step].view(np.int16)).pin_memory()
                hout = torch.zeros((L, 2, H, 128), dtype=torch.int16).pin_memory()
                ctx.step_begin(seqs)
                for l in range(L):
                    ctx.step_layer_host(l, hkv[l], hq[l], hout[l])
                ctx.step_end()                      # no stream synchronisation: step_end waits for the copies
                outs.append(hout.numpy().view(np.uint16).copy())
        assert ctx.status() == 0
        results.append(outs)
        ctx.close()
    for step in range(2):
        assert results[1][step].any()
        assert np.array_equal(results[0][step], results[1][step])


# ---------------------------------------------------------------------------------------------
# bookkeeping and error behaviour on the device-backed context
# ---------------------------------------------------------------------------------------------
def test_cache_bookkeeping_and_errors(torch):
    from mugen_b200.mla import MlaContext
    case = synth.make_layer_case(1, 2, [1], synth.DT_F16)
    ctx = MlaContext(n_layers=1, n_heads=2, dtype=synth.DT_F16, n_pages=4, max_seqs=2, max_seq_len=200,
                     kernel=capi.KERNEL_MMA, **YARN)
    ctx.set_layer_weights(0, case.w_uk, case.w_uv, case.w_type, case.norm_w)
    a, b = ctx.seq_create(), ctx.seq_create()
    with pytest.raises(capi.MlaError) as e:
        ctx.seq_create()
    assert e.value.code == 4
    rows = torch.zeros((130, 576), dtype=torch.int16, device="cuda")
    ctx.write_rows(0, a, 0, rows)
    assert ctx.free_pages() == 1
    ctx.advance_seq_len(a, 130)
    with pytest.raises(capi.MlaError):          # advancing past appended rows
        ctx.advance_seq_len(a, 100)
    with pytest.raises(capi.MlaError) as e:     # pool exhausted (needs 2 pages, 1 free)
        ctx.write_rows(0, b, 0, rows[:100])
    assert e.value.code == 3
    with pytest.raises(capi.MlaError) as e:     # beyond max_seq_len
        ctx.append_rows(0, [a], [200], rows[:1])
    assert e.value.code == 4
    with pytest.raises(capi.MlaError):          # truncate never grows
        ctx.truncate(a, 131)
    ctx.truncate(a, 64)
    assert ctx.seq_len(a) == 64 and ctx.free_pages() == 3
    ctx.truncate(a, 1)
    assert ctx.free_pages() == 3                # partial last page is kept
    ctx.clear(a)
    assert ctx.seq_len(a) == 0 and ctx.free_pages() == 4
    with pytest.raises(capi.MlaError) as e:     # out-of-order scheduler calls
        ctx.step_end()
    assert e.value.code == 5
    ctx.step_begin([a, b])
    with pytest.raises(capi.MlaError):
        ctx.step_begin([a])
    ctx.step_end()
    assert ctx.seq_len(a) == 1 and ctx.seq_len(b) == 1
    assert ctx.status() == 0
    ctx.close()


def test_a_wait_that_runs_out_raises_the_status_bit_and_leaves_the_context_usable(torch, oracle):
    """Failure detection on the device, without faulting it: the self-test block waits on a barrier nothing
    completes, with a limit of a million cycles; the wait must give up (never hang, never trap), raise
    ST_WAIT_TIMEOUT (4) in the status word, free its tensor memory and return.  The host reads the bit through
    mla_status, which clears it, and the same context then computes a correct attention."""
    case = synth.make_layer_case(4242, 128, [200], synth.DT_BF16)
    ctx = make_ctx(case, capi.KERNEL_AUTO)
    seqs = fill(torch, ctx, case)
    assert ctx.status() == 0
    waited = ctx.selftest_wait_timeout(1_000_000)
    assert 1_000_000 <= waited < 400_000_000, waited          # gave up after the limit, within a fraction of a second
    with pytest.raises(capi.MlaError) as ei:
        ctx.status()
    assert ei.value.code == 6 and "= 4" in str(ei.value)          # MLA_ERR_DEVICE, ST_WAIT_TIMEOUT
    assert ctx.status() == 0                                   # reading cleared it
    out = torch.zeros((1, 128, 128), dtype=torch.int16, device="cuda")
    ctx.attend_rows(0, seqs, [200], _dev(torch, case.q), out)
    check_close(_host(out)[0], oracle_out(oracle, case, 0), case.dt, "after the timed-out wait")
    assert ctx.status() == 0
    with pytest.raises(capi.MlaError):                         # limits beyond about a second are refused
        ctx.selftest_wait_timeout(3_000_000_000)
    ctx.close()


def test_block_tables_are_permuted_pages(torch):
    from mugen_b200.mla import MlaContext
    ctx = MlaContext(n_layers=1, n_heads=2, dtype=synth.DT_F16, n_pages=64, max_seqs=2, max_seq_len=4096,
                     kernel=capi.KERNEL_MMA, **YARN)
    ctx.shuffle_free_pages(42)
    s = ctx.seq_create()
    ctx.write_rows(0, s, 0, torch.zeros((64 * 40, 576), dtype=torch.int16, device="cuda"))
    pages = ctx.seq_pages(s)
    assert len(pages) == 40 and len(set(pages.tolist())) == 40
    assert not np.array_equal(pages, np.sort(pages))
    ctx.close()
