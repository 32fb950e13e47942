"""GGUF ingestion (mla_gguf_*): the MLA metadata keys and the per-layer W_UK / W_UV / kv_a-norm tensors of a
deepseek2 model file.  The files are tiny synthetic models written by tests/golden/tiny_gguf.py.  Checked on the CPU
against what the writer put in and, where the reference tree is mounted, against what the reference's own
from_gguf holds after loading the same file (src/core/model/transformer.cpp:2951-3011, 3178-3221); on the GPU a
context configured and registered from the file must attend like one fed the same tensors by hand."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

from mugen_b200 import capi, synth

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import tiny_gguf  # noqa: E402

VARIANTS = {
    "separate_f16": dict(seed=31),
    "merged_f16_no_q_lora": dict(seed=32, merged_kv_b=True, q_lora_rank=0, n_heads=3, rope_factor=1.0, eps=1e-5),
    "merged_q8_0": dict(seed=33, merged_kv_b=True, kv_b_type=tiny_gguf.GGML_Q8_0, n_layers=1),
    "separate_q4_0": dict(seed=34, kv_b_type=tiny_gguf.GGML_Q4_0, n_layers=1, context_length=0),
}


def _open(path):
    lib = capi.load()
    h = C.c_void_p()
    rc = lib.mla_gguf_open(path.encode(), C.byref(h))
    assert rc == 0, lib.mla_gguf_last_error().decode()
    return lib, h


def _layer(lib, h, layer, n_heads):
    wt, nb = C.c_uint32(), C.c_size_t()
    assert lib.mla_gguf_layer_weights(h, layer, None, None, 0, C.byref(wt), C.byref(nb), None) == 0
    k, v = np.zeros(nb.value, np.uint8), np.zeros(nb.value, np.uint8)
    norm = np.zeros(512, np.uint16)
    rc = lib.mla_gguf_layer_weights(h, layer, k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p), nb.value,
                                    C.byref(wt), C.byref(nb), norm.ctypes.data_as(C.c_void_p))
    assert rc == 0, lib.mla_gguf_last_error().decode()
    return wt.value, k, v, norm


@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_metadata_and_tensors_match_the_file_and_the_reference_loader(tmp_path, reference, variant):
    m = tiny_gguf.TinyModel(**VARIANTS[variant])
    path = str(tmp_path / "tiny.gguf")
    tiny_gguf.write(path, m)
    lib, h = _open(path)
    info = capi.GgufInfo()
    assert lib.mla_gguf_get_info(h, C.byref(info)) == 0
    assert (info.n_layers, info.n_heads, info.embedding_length) == (m.n_layers, m.n_heads, m.embed)
    assert (info.kv_lora_rank, info.qk_nope_head_dim, info.qk_rope_head_dim, info.v_head_dim) == (512, 128, 64, 128)
    assert info.q_lora_rank == m.q_lora_rank and info.context_length == m.context_length
    assert np.float32(info.rope_theta) == np.float32(m.rope_theta) and np.float32(info.rms_norm_eps) == np.float32(m.eps)
    assert np.float32(info.rope_scaling_factor) == np.float32(m.rope_factor) and info.rope_original_ctx == m.rope_orig_ctx
    cfg = capi.MlaConfig()
    assert lib.mla_gguf_fill_config(h, C.byref(cfg)) == 0
    assert cfg.max_seq_len == (m.context_length or 8192) and cfg.n_heads == m.n_heads and cfg.kv_lora_rank == 512
    ref_model = reference.load_model(path) if reference is not None else None
    if ref_model is not None:
        rc = ref_model.cfg
        assert (rc["n_layers"], rc["n_heads"], rc["q_lora_rank"], rc["max_seq_len"]) == (info.n_layers, info.n_heads,
                                                                                        info.q_lora_rank, cfg.max_seq_len)
        assert np.float32(rc["rms_norm_eps"]) == np.float32(info.rms_norm_eps)
    H = m.n_heads
    for layer in range(m.n_layers):
        wt, k, v, norm = _layer(lib, h, layer, H)
        assert wt == {tiny_gguf.GGML_F16: synth.W_F16, tiny_gguf.GGML_Q8_0: synth.W_Q8_0, tiny_gguf.GGML_Q4_0: synth.W_Q4_0}[m.kv_b_type]
        blk = f"blk.{layer}."
        bpr = len(k) // (H * 128)
        if m.merged_kv_b:                     # per head [128 nope rows | 128 v rows]
            raw = np.frombuffer(m.tensors[blk + "attn_kv_b.weight"][2], np.uint8).reshape(H, 256, bpr)
            want_k, want_v = raw[:, :128].reshape(-1), raw[:, 128:].reshape(-1)
        else:
            want_k = np.frombuffer(m.tensors[blk + "attn_k_b.weight"][2], np.uint8)
            want_v = np.frombuffer(m.tensors[blk + "attn_v_b.weight"][2], np.uint8)
        assert np.array_equal(k, want_k) and np.array_equal(v, want_v)
        want_norm = m.tensors[blk + "attn_kv_a_norm.weight"][3].astype(np.float16).view(np.uint16)
        assert np.array_equal(norm, want_norm)
        if ref_model is not None:             # what the reference's loader holds for the same file
            rt, rk = ref_model.weight(layer, "w_uk", len(k))
            _, rv = ref_model.weight(layer, "w_uv", len(v))
            _, rn = ref_model.weight(layer, "kv_a_norm", 1024)
            assert rt == wt and np.array_equal(rk, k) and np.array_equal(rv, v) and np.array_equal(rn.view(np.uint16), norm)
    if ref_model is not None:
        ref_model.close()
    lib.mla_gguf_close(h)


def test_errors_are_reported_not_crashed(tmp_path):
    lib = capi.load()
    h = C.c_void_p()
    assert lib.mla_gguf_open(str(tmp_path / "absent.gguf").encode(), C.byref(h)) == 1
    assert b"cannot open" in lib.mla_gguf_last_error()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUX" + b"\0" * 64)
    assert lib.mla_gguf_open(str(bad).encode(), C.byref(h)) == 1 and b"magic" in lib.mla_gguf_last_error()
    good = tiny_gguf.build(tiny_gguf.TinyModel(seed=35, n_layers=1))
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(good[:len(good) // 2])      # tensor data missing
    rc = lib.mla_gguf_open(str(cut).encode(), C.byref(h))
    if rc == 0:
        wt, nb = C.c_uint32(), C.c_size_t()
        k = np.zeros(1 << 20, np.uint8)
        assert lib.mla_gguf_layer_weights(h, 0, k.ctypes.data_as(C.c_void_p), k.ctypes.data_as(C.c_void_p), 0,
                                          C.byref(wt), C.byref(nb), None) != 0
        lib.mla_gguf_close(h)
    m = tiny_gguf.TinyModel(seed=36, n_layers=1)
    full = tmp_path / "ok.gguf"
    tiny_gguf.write(str(full), m)
    lib2, h2 = _open(str(full))
    wt, nb = C.c_uint32(), C.c_size_t()
    assert lib2.mla_gguf_layer_weights(h2, 5, None, None, 0, C.byref(wt), C.byref(nb), None) == 1     # layer out of range
    lib2.mla_gguf_close(h2)


@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["separate_f16", "merged_q8_0"])
def test_context_built_from_a_gguf_file_attends_like_the_checker(tmp_path, oracle, variant):
    import torch
    from mugen_b200.mla import MlaContext
    m = tiny_gguf.TinyModel(**VARIANTS[variant])
    path = str(tmp_path / "tiny.gguf")
    tiny_gguf.write(path, m)
    lib, h = _open(path)
    info = capi.GgufInfo()
    lib.mla_gguf_get_info(h, C.byref(info))
    dt, H, S = synth.DT_F16, m.n_heads, 200
    ctx = MlaContext(n_layers=info.n_layers, n_heads=info.n_heads, dtype=dt, n_pages=8, max_seqs=1, max_seq_len=256,
                     rope_theta=info.rope_theta, rope_scaling_factor=info.rope_scaling_factor,
                     rope_original_ctx=info.rope_original_ctx, rms_norm_eps=info.rms_norm_eps)
    assert lib.mla_gguf_register(ctx.h, h, dt) == 0, lib.mla_gguf_last_error().decode()
    rng = np.random.default_rng(1)
    cache = synth.to_bits(rng.standard_normal((S, 576), np.float32), dt)
    q = synth.to_bits(rng.standard_normal((1, H, 192), np.float32) * np.float32(0.9), dt)
    dev = lambda b: torch.from_numpy(np.ascontiguousarray(b).view(np.int16)).cuda()
    for layer in range(info.n_layers):
        s = ctx.seq_create()
        ctx.write_rows(layer, s, 0, dev(cache))
        out = torch.zeros((1, H, 128), dtype=torch.int16, device="cuda")
        ctx.attend_rows(layer, [s], [S], dev(q), out)
        wt, k, v, _ = _layer(lib, h, layer, H)
        want = oracle.attention(q[0], cache, S, k, v, wt, H, dt)
        mx, rl = synth.error_norms(out.cpu().numpy().view(np.uint16)[0], want, dt, dt)
        assert mx <= 2e-2 and rl <= 5e-3, (layer, mx, rl)
        ctx.seq_free(s)
    assert ctx.status() == 0
    ctx.close()
    lib.mla_gguf_close(h)
