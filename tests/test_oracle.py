"""The CPU checker against (a) the committed fixtures that the reference's own code produced
and (b) that code itself wherever its build is present.  Bit-exact throughout."""
import base64

import os

import numpy as np
import pytest

from mugen_b200 import synth


def _unb64(s, dtype):
    return np.frombuffer(base64.b64decode(s), dtype=dtype)


def _attn_case(c):
    return synth.make_layer_case(c["seed"], c["n_heads"], [c["seq_len"]], synth.DT_F16,
                                 c["w_type"], c["q_scale"], c["exact_in_both"])


def test_golden_attention_bit_exact(oracle, golden):
    assert len(golden["attention"]) >= 8
    for c in golden["attention"]:
        case = _attn_case(c)
        assert case.digest() == c["inputs_sha256"], "synthetic input generator drifted"
        got = oracle.attention(case.q[0], case.caches[0], c["seq_len"], case.w_uk, case.w_uv,
                               c["w_type"], c["n_heads"], synth.DT_F16)
        want = _unb64(c["out_f16"], np.uint16).reshape(c["n_heads"], synth.VDIM)
        assert np.array_equal(got, want), f"case seed={c['seed']}"


def test_golden_yarn_freq_bit_exact(oracle, golden):
    for c in golden["yarn"]:
        want = _unb64(c["freq_f32"], np.float32)
        got = np.array([oracle.yarn_rope_freq(i, 64, c["factor"], c["orig_ctx"], c["theta"])
                        for i in range(32)], np.float32)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_golden_counter_trace(oracle, golden):
    import ctypes as C
    L = oracle.L

    class Counter(C.Structure):
        _fields_ = [("phantom", C.c_uint32)]

    L.oracle_counter_seq_len.restype = C.c_uint32
    for entry in golden["counter"]:
        c = Counter(0)
        for (op, n), want in zip(entry["trace"], entry["seq_len_after"]):
            if op == "advance":
                L.oracle_counter_advance(C.byref(c), C.c_uint32(n))
            elif op == "truncate":
                L.oracle_counter_truncate(C.byref(c), C.c_uint32(n))
            else:
                L.oracle_counter_clear(C.byref(c))
            assert L.oracle_counter_seq_len(C.byref(c)) == want


def test_golden_append_regression(oracle, golden):
    assert len(golden["append"]) >= 12
    for c in golden["append"]:
        # inputs and outputs of the reference's own inline append, recorded from its forward()
        assert c["source"].startswith("reference forward()")
        got = oracle.append_rows(_unb64(c["kv_a"], np.uint16), [c["position"]], _unb64(c["norm_w"], np.uint16), c["eps"],
                                 c["factor"], c["orig_ctx"], c["theta"], c["dt"])
        assert np.array_equal(got[0], _unb64(c["row"], np.uint16)), (c["model"], c["layer"], c["position"])
    for c in golden["q_rope"]:
        got = oracle.q_rope(_unb64(c["q_in"], np.uint16), c["position"], c["factor"], c["orig_ctx"], c["theta"], c["dt"])
        assert np.array_equal(got.reshape(-1), _unb64(c["q_out"], np.uint16)), (c["model"], c["position"])
    for c in golden["append_restated"]:
        case = synth.make_layer_case(c["seed"], 1, [1] * c["n"], c["dt"])
        assert case.digest() == c["inputs_sha256"]
        got = oracle.append_rows(case.kv_a, c["positions"], case.norm_w, c["eps"], c["factor"],
                                 c["orig_ctx"], c["theta"], c["dt"])
        want = _unb64(c["rows"], np.uint16).reshape(c["n"], synth.ROW)
        assert np.array_equal(got, want)


def test_append_matches_plain_numpy_formula(oracle):
    """Independent float32 numpy evaluation of the append statements, operation by operation."""
    case = synth.make_layer_case(7, 1, [1] * 6, synth.DT_F16)
    pos = [0, 3, 64, 1000, 8191, 40000]
    factor, ctx, theta, eps = 40.0, 4096, 10000.0, 1e-6
    got = oracle.append_rows(case.kv_a, pos, case.norm_w, eps, factor, ctx, theta, synth.DT_F16)
    x = synth.from_bits(case.kv_a, synth.DT_F16)
    w = synth.from_bits(case.norm_w, synth.DT_F16)
    for r in range(6):
        ss = np.float32(0)
        for v in x[r, :512]:
            ss = np.float32(ss + np.float32(v * v))
        rinv = np.float32(1) / np.sqrt(np.float32(ss / np.float32(512) + np.float32(eps)))
        c_kv = (np.float32(x[r, :512] * rinv) * w).astype(np.float16)
        cs, sn = oracle.rope_cos_sin(pos[r], factor, ctx, theta)
        x0, x1 = x[r, 512:544], x[r, 544:576]
        lo = (np.float32(x0 * cs) - np.float32(x1 * sn)).astype(np.float16)
        hi = (np.float32(x1 * cs) + np.float32(x0 * sn)).astype(np.float16)
        want = np.concatenate([c_kv, lo, hi]).view(np.uint16)
        assert np.array_equal(got[r], want), f"row {r}"


def test_bf16_mode_differs_from_f16_only_in_final_rounding(oracle):
    """On inputs exact in both formats, the bf16 path must equal the f16 path up to the one
    rounding of the output (the reference is f16-only; this ties the bf16 checker to it)."""
    c16 = synth.make_layer_case(31, 4, [150], synth.DT_F16, synth.W_F16, 1.0, True)
    vals = lambda b: synth.to_bits(synth.from_bits(b, synth.DT_F16), synth.DT_BF16)
    out16 = oracle.attention(c16.q[0], c16.caches[0], 150, c16.w_uk, c16.w_uv, synth.W_F16, 4,
                             synth.DT_F16)
    outbf = oracle.attention(vals(c16.q[0]), vals(c16.caches[0]), 150, vals(c16.w_uk),
                             vals(c16.w_uv), synth.W_BF16, 4, synth.DT_BF16)
    a = synth.from_bits(out16, synth.DT_F16)
    b = synth.from_bits(outbf, synth.DT_BF16)
    assert np.all(np.abs(a - b) <= np.abs(a) * 2.0 ** -8 + 1e-7)


def test_partial_states_merge_to_full(oracle):
    """KV-range partials (max, sum, acc) merged by log-sum-exp reproduce the full softmax·V."""
    case = synth.make_layer_case(41, 4, [300], synth.DT_F16)
    q, cache = case.q[0], case.caches[0]
    full = oracle.partial(q, cache, 0, 300, case.w_uk, synth.W_F16, 4, synth.DT_F16)
    parts = [oracle.partial(q, cache, a, b, case.w_uk, synth.W_F16, 4, synth.DT_F16)
             for a, b in [(0, 128), (128, 192), (192, 300)]]
    m = np.max([p[:, 0] for p in parts], axis=0)
    w = [np.exp(p[:, 0] - m) for p in parts]
    l = sum(wi * p[:, 1] for wi, p in zip(w, parts))
    acc = sum(wi[:, None] * p[:, 2:] for wi, p in zip(w, parts))
    np.testing.assert_allclose(acc / l[:, None], full[:, 2:] / full[:, 1:2], rtol=2e-5, atol=1e-6)


# ---- against the reference's own compiled code (skipped where it cannot be built) ----

@pytest.mark.parametrize("w_type", [synth.W_F16, synth.W_Q8_0, synth.W_Q4_0])
@pytest.mark.parametrize("n_heads,seq_len,q_scale", [(1, 1, 1.0), (5, 190, 1.0), (16, 512, 6.0)])
def test_restatement_equals_reference(oracle, reference, w_type, n_heads, seq_len, q_scale):
    if reference is None:
        pytest.skip("reference build not present")
    case = synth.make_layer_case(1000 + n_heads + seq_len, n_heads, [seq_len], synth.DT_F16,
                                 w_type, q_scale)
    want = reference.attention(case.q[0], case.caches[0], seq_len, case.w_uk, case.w_uv, w_type,
                               n_heads)
    got = oracle.attention(case.q[0], case.caches[0], seq_len, case.w_uk, case.w_uv, w_type,
                           n_heads, synth.DT_F16)
    assert np.array_equal(got, want)


def test_restatement_yarn_equals_reference(oracle, reference):
    if reference is None:
        pytest.skip("reference build not present")
    rng = np.random.default_rng(5)
    for _ in range(200):
        factor = float(rng.choice([0.0, 0.5, 1.0, 2.0, 40.0, 64.0]))
        ctx = int(rng.choice([1024, 4096, 32768, 163840]))
        theta = float(rng.choice([10000.0, 50000.0, 1e6]))
        i = int(rng.integers(0, 32))
        a = oracle.yarn_rope_freq(i, 64, factor, ctx, theta)
        b = reference.yarn_rope_freq(i, 64, factor, ctx, theta)
        assert a.view(np.uint32) == b.view(np.uint32)


@pytest.mark.parametrize("variant", ["lora_yarn", "full_q_merged_kv_b_plain_rope", "q8_0_kv_b"])
def test_append_and_q_rope_restatements_equal_reference_forward(oracle, reference, tmp_path, variant):
    """The reference's append (steps G+H) and q RoPE (step E) are inline in forward(): run the real from_gguf +
    forward() on a tiny synthetic deepseek2 GGUF file and compare, bit for bit, every cache row it writes and
    every rotated q it hands to the attention with the restatements fed the same kv_a / q."""
    if reference is None:
        pytest.skip("reference build not present")
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import tiny_gguf
    model = {"lora_yarn": dict(seed=21),
             "full_q_merged_kv_b_plain_rope": dict(seed=22, q_lora_rank=0, merged_kv_b=True, rope_factor=0.5, eps=1e-5,
                                                   context_length=4096, n_heads=3),
             "q8_0_kv_b": dict(seed=23, kv_b_type=tiny_gguf.GGML_Q8_0, n_layers=1, rope_factor=4.0, rope_orig_ctx=128)}[variant]
    path = str(tmp_path / "tiny.gguf")
    tiny_gguf.write(path, tiny_gguf.TinyModel(**model))
    mod = reference.load_model(path)
    c = mod.cfg
    assert (c["kv_lora_rank"], c["qk_nope"], c["qk_rope"], c["v_head_dim"]) == (512, 128, 64, 128)
    rope = (c["rope_scaling_factor"], c["rope_original_ctx"], c["rope_theta"])
    positions = list(range(70)) if variant != "full_q_merged_kv_b_plain_rope" else [0, 1, 63, 64, 65, 1000, 4095]
    for n, pos in enumerate(positions):
        taps = mod.forward(n % c["vocab"], pos)
        for L in range(c["n_layers"]):
            norm_w = mod.weight(L, "kv_a_norm", 1024)[1].view(np.uint16)
            want = mod.cache_rows(L, pos, 1)[0]
            got = oracle.append_rows(taps["kv_a_pre"][L][None], [pos], norm_w, c["rms_norm_eps"], *rope, synth.DT_F16)[0]
            assert np.array_equal(got, want), (variant, L, pos)
            q = oracle.q_rope(taps["q_pre"][L], pos, *rope, synth.DT_F16)
            assert np.array_equal(q.reshape(-1), taps["q_post"][L].reshape(-1)), (variant, L, pos)
            # the attention the driver ran on its own cache is the routine the other tests pin
            seq_len = mod.seq_len()          # counter moved once, after all layers
            if pos + 1 == seq_len:
                cache = mod.cache_rows(L, 0, seq_len)
                nb = c["n_heads"] * 128 * 512 * 2 if variant != "q8_0_kv_b" else c["n_heads"] * 128 * 16 * 34
                wt, w_uk = mod.weight(L, "w_uk", nb)
                _, w_uv = mod.weight(L, "w_uv", nb)
                att = oracle.attention(taps["q_post"][L], cache, seq_len, w_uk, w_uv, wt, c["n_heads"], synth.DT_F16)
                assert np.array_equal(att, taps["attn_out"][L]), (variant, L, pos)
    assert mod.seq_len() == len(positions)       # advance_seq_len(1) once per token (transformer.cpp:4401-4403)
    mod.close()


def test_quant_pack_roundtrip():
    rng = np.random.default_rng(3)
    w = rng.standard_normal((8, 512), np.float32) * np.float32(0.02)
    assert np.abs(synth.unpack_q8_0(synth.pack_q8_0(w)) - w).max() < 0.02 * 4 / 127 * 1.01
    assert np.abs(synth.unpack_q4_0(synth.pack_q4_0(w)) - w).max() < 0.02 * 5 / 8
