"""mla_attention_noalloc — the entry point for callers that are not allowed to allocate device
memory (their memory belongs to another allocator, or a cudaMalloc would stall their other
streams).  It keeps its intermediates in an array built into the library instead of a context's
workspaces, so the check is simple: through the C ABI, its output must agree with what the
context-based entry point (mla_attend_rows) returns for the same query, cache and weights — on
two different problems run back to back, because the built-in array is shared between calls and
still holds the first call's data when the second one starts.  This file sorts last on purpose:
a run that stops at the first failure has then already exercised every other test."""
import ctypes as C

import numpy as np
import pytest

from mugen_b200 import capi, synth

pytestmark = pytest.mark.gpu
ROPE = dict(rope_theta=10000.0, rope_scaling_factor=40.0, rope_original_ctx=4096, rms_norm_eps=1e-6)


def _dev(torch, bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()


def _both_ways(torch, seed, n_heads, seq_len, dt):
    """(output of the context-based entry point, output of the no-allocation entry point)."""
    from mugen_b200.mla import MlaContext
    lib = capi.load()
    case = synth.make_layer_case(seed, n_heads, [seq_len], dt)
    ctx = MlaContext(n_layers=1, n_heads=n_heads, dtype=dt, n_pages=seq_len // 64 + 4, max_seqs=1,
                     max_seq_len=seq_len + 128, kernel=capi.KERNEL_MMA, **ROPE)
    ctx.set_layer_weights(0, case.w_uk, case.w_uv, case.w_type, case.norm_w)
    s = ctx.seq_create()
    ctx.write_rows(0, s, 0, _dev(torch, case.caches[0]))
    ctx.advance_seq_len(s, seq_len)
    want = torch.zeros((1, n_heads, 128), dtype=torch.int16, device="cuda")
    ctx.attend_rows(0, [s], [seq_len], _dev(torch, case.q), want)
    torch.cuda.synchronize()
    ctx.close()
    # the caller's own buffers: a contiguous cache of exactly seq_len rows.  The allocation continues with
    # rows of NaN bit patterns: the entry point promises to read nothing behind the last row, and if it did
    # and multiplied them by a zero probability, the NaNs would show in the output.
    padded = np.full((seq_len + 64, 576), 0x7FC0 if dt == synth.DT_BF16 else 0x7E00, np.uint16)
    padded[:seq_len] = case.caches[0]
    d_cache, d_q = _dev(torch, padded), _dev(torch, case.q[0])
    d_wk, d_wv = _dev(torch, case.w_uk), _dev(torch, case.w_uv)
    got = torch.full((n_heads, 128), 0x7E00, dtype=torch.int16, device="cuda")
    rc = lib.mla_attention_noalloc(dt, n_heads, seq_len, C.c_void_p(d_q.data_ptr()), C.c_void_p(d_cache.data_ptr()),
                                   C.c_void_p(d_wk.data_ptr()), C.c_void_p(d_wv.data_ptr()),
                                   C.c_void_p(got.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.mla_noalloc_last_error().decode()
    torch.cuda.synchronize()
    return want.cpu().numpy().view(np.uint16)[0], got.cpu().numpy().view(np.uint16), case


def test_noalloc_matches_context_entry_point_twice_in_a_row(oracle):
    import torch
    assert torch.cuda.is_available()
    # two calls in a row on different shapes and dtypes: the second one finds the first one's
    # leftovers in the shared array
    for seed, heads, seq_len, dt in [(4101, 128, 3000, synth.DT_BF16), (4102, 16, 257, synth.DT_F16)]:
        want, got, case = _both_ways(torch, seed, heads, seq_len, dt)
        mx, rl = synth.error_norms(got, want, dt, dt)
        assert mx <= 2e-2 and rl <= 5e-3, (heads, seq_len, mx, rl)
        # and, like every other attention test here, against the CPU result
        cpu = oracle.attention(case.q[0], case.caches[0], seq_len, case.w_uk, case.w_uv, case.w_type, heads, dt)
        mx, rl = synth.error_norms(got, cpu, dt, dt)
        assert mx <= 2e-2 and rl <= 5e-3, (heads, seq_len, mx, rl)


def test_noalloc_rejects_sizes_beyond_its_built_in_scratch():
    import torch
    lib = capi.load()
    t = torch.zeros(64, dtype=torch.int16, device="cuda")
    p = C.c_void_p(t.data_ptr())
    assert lib.mla_attention_noalloc(0, 129, 64, p, p, p, p, p, None) == 4
    assert b"n_heads" in lib.mla_noalloc_last_error()
    assert lib.mla_attention_noalloc(1, 16, 65537, p, p, p, p, p, None) == 4
    assert b"seq_len" in lib.mla_noalloc_last_error()
    assert lib.mla_attention_noalloc(2, 16, 64, p, p, p, p, p, None) == 1
