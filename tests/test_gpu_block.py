"""The projections around the attention op (mla_set_block_weights, mla_block_project_in / _out, mla_step_block):
steps A-D, F, J, K of the reference's MLA decode driver (src/core/model/transformer.cpp:3849-3929, 4002-4015).

Two oracles.  (1) The recorded trace of the reference's own forward() on a tiny deepseek2 model (tests/golden, "block"
entries; the model is re-created here from its seed): what went into and came out of every layer's attention block at
every position.  (2) A plain numpy restatement of the reference's kernels for the DeepSeek-V3 projection shapes:
matvec = float accumulation rounded once to the storage type, rms_norm = x * rsqrt(mean(x^2) + eps) * w rounded once,
residual = sum rounded once (src/metal/kernel_sources.h:55-98, 264-312, 357-366).  The tensor core adds the products
in another order than the reference's lanes, so results are compared within a tolerance, stated below."""
import base64
import os
import sys

import numpy as np
import pytest

from mugen_b200 import capi, synth

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import tiny_gguf  # noqa: E402

pytestmark = pytest.mark.gpu
# a projection output is one rounding of a float sum: two correct implementations differ by at most one unit in the last
# place of a few elements.  max-abs is relative to the tensor's largest magnitude.
REL_L2, MAX_REL = 2e-3, 1.6e-2


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def _dev(torch, bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()


def _bits(t):
    return t.cpu().numpy().view(np.uint16)


def _close(got, want, dt, what):
    g, w = synth.from_bits(got, dt).astype(np.float64).ravel(), synth.from_bits(want, dt).astype(np.float64).ravel()
    rl = np.sqrt(((g - w) ** 2).sum()) / max(np.sqrt((w ** 2).sum()), 1e-30)
    mx = np.abs(g - w).max() / max(np.abs(w).max(), 1e-30)
    assert rl <= REL_L2 and mx <= MAX_REL, f"{what}: rel-L2 {rl:.2e}, max/peak {mx:.2e}"


def _unb(t):
    return np.frombuffer(base64.b64decode(t), np.uint16).copy()


def test_block_trace_of_the_reference_forward(torch, golden):
    from mugen_b200.mla import MlaContext
    blk = golden["block"]
    m = tiny_gguf.TinyModel(**blk["model"])
    tiny_gguf.build(m)
    f16 = lambda name: np.frombuffer(m.tensors[name][2], np.float16 if m.tensors[name][0] == 1 else np.float32).astype(np.float16).view(np.uint16).reshape(m.tensors[name][1][::-1])
    H, E, L, dt = m.n_heads, m.embed, m.n_layers, synth.DT_F16
    ctx = MlaContext(n_layers=L, n_heads=H, dtype=dt, n_pages=4, max_seqs=L, max_seq_len=64, rope_theta=m.rope_theta,
                     rope_scaling_factor=m.rope_factor, rope_original_ctx=m.rope_orig_ctx, rms_norm_eps=m.eps)
    for l in range(L):
        b = f"blk.{l}."
        ctx.set_layer_weights(l, f16(b + "attn_k_b.weight"), f16(b + "attn_v_b.weight"), synth.W_F16, f16(b + "attn_kv_a_norm.weight"))
        ctx.set_block_weights(l, attn_norm=f16(b + "attn_norm.weight"), q_a=f16(b + "attn_q_a.weight"),
                              q_a_norm=f16(b + "attn_q_a_norm.weight"), q_b=f16(b + "attn_q_b.weight"),
                              kv_a_mqa=f16(b + "attn_kv_a_mqa.weight"), wo=f16(b + "attn_output.weight"))
    ctx.set_q_rope(True)
    # one sequence per layer: the layers of the reference share a position counter but not a cache, and here every
    # layer is replayed from its own recorded input (the FFN between the blocks is not part of this library)
    seqs = [ctx.seq_create() for _ in range(L)]
    for pos, step in enumerate(blk["steps"]):
        taps = {k: _unb(v) for k, v in step.items()}
        for l in range(L):
            hidden_in = taps["hidden_in"].reshape(L, E)[l]
            # the pieces
            q = torch.zeros((1, H, 192), dtype=torch.int16, device="cuda")
            kv = torch.zeros((1, 576), dtype=torch.int16, device="cuda")
            ctx.block_project_in(l, _dev(torch, hidden_in[None]), q, kv)
            _close(_bits(q)[0], taps["q_pre"].reshape(L, H, 192)[l], dt, f"q, layer {l}, position {pos}")
            _close(_bits(kv)[0], taps["kv_a_pre"].reshape(L, 576)[l], dt, f"kv_a, layer {l}, position {pos}")
            h2 = _dev(torch, hidden_in[None].copy())
            ctx.block_project_out(l, _dev(torch, taps["attn_out"].reshape(L, 1, H, 128)[l]), h2)
            _close(_bits(h2)[0], taps["hidden_mid"].reshape(L, E)[l], dt, f"Wo + residual, layer {l}, position {pos}")
            # the whole block through the step interface: hidden in -> hidden out, cache growing by one row per position
            h = _dev(torch, hidden_in[None].copy())
            ctx.step_begin([seqs[l]])
            ctx.step_block(l, h)
            ctx.step_end()
            _close(_bits(h)[0], taps["hidden_mid"].reshape(L, E)[l], dt, f"whole block, layer {l}, position {pos}")
    assert ctx.status() == 0 and [ctx.seq_len(s) for s in seqs] == [len(blk["steps"])] * L
    ctx.close()


def _np_project(x_bits, w_bits, dt):
    y = synth.from_bits(x_bits, dt).astype(np.float32) @ synth.from_bits(w_bits, dt).astype(np.float32).T
    return synth.to_bits(y, dt)


def _np_rmsnorm(x_bits, w_bits, eps, dt):
    x = synth.from_bits(x_bits, dt).astype(np.float32)
    inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + np.float32(eps))
    return synth.to_bits(x * inv * synth.from_bits(w_bits, dt).astype(np.float32), dt)


@pytest.mark.parametrize("dt,rows,H,E,R", [(synth.DT_BF16, 64, 128, 7168, 1536),      # DeepSeek-V3 attention block, batch 64
                                           (synth.DT_F16, 32, 16, 2048, 0),           # V2-Lite: full q projection
                                           (synth.DT_BF16, 5, 8, 264, 72)])           # ragged sizes: tiles cut by M, N and K
def test_projection_shapes_against_numpy_restatement(torch, dt, rows, H, E, R):
    from mugen_b200.mla import MlaContext
    rng = np.random.default_rng(E + R)
    rnd = lambda shape, s: synth.to_bits((rng.standard_normal(shape) * s).astype(np.float32), dt)
    w = dict(attn_norm=synth.to_bits((1 + 0.1 * rng.standard_normal(E)).astype(np.float32), dt), kv_a_mqa=rnd((576, E), E ** -0.5),
             wo=rnd((E, H * 128), (H * 128) ** -0.5))
    if R:
        w.update(q_a=rnd((R, E), E ** -0.5), q_a_norm=synth.to_bits((1 + 0.1 * rng.standard_normal(R)).astype(np.float32), dt),
                 q_b=rnd((H * 192, R), R ** -0.5))
    else:
        w.update(q=rnd((H * 192, E), E ** -0.5))
    ctx = MlaContext(n_layers=1, n_heads=H, dtype=dt, n_pages=2, max_seqs=1, max_seq_len=64, rms_norm_eps=1e-6)
    ctx.set_block_weights(0, **w)
    hidden = rnd((rows, E), 1.0)
    q = torch.zeros((rows, H, 192), dtype=torch.int16, device="cuda")
    kv = torch.zeros((rows, 576), dtype=torch.int16, device="cuda")
    ctx.block_project_in(0, _dev(torch, hidden), q, kv)
    h2 = _np_rmsnorm(hidden, w["attn_norm"], 1e-6, dt)
    if R:
        want_q = _np_project(_np_rmsnorm(_np_project(h2, w["q_a"], dt), w["q_a_norm"], 1e-6, dt), w["q_b"], dt)
    else:
        want_q = _np_project(h2, w["q"], dt)
    _close(_bits(q).reshape(rows, -1), want_q, dt, "q")
    _close(_bits(kv), _np_project(h2, w["kv_a_mqa"], dt), dt, "kv_a")
    attn = rnd((rows, H, 128), 0.05)
    hid = _dev(torch, hidden.copy())
    ctx.block_project_out(0, _dev(torch, attn), hid)
    wo_out = synth.from_bits(_np_project(attn.reshape(rows, -1), w["wo"], dt), dt)
    want_h = synth.to_bits(synth.from_bits(hidden, dt).astype(np.float32) + wo_out, dt)
    _close(_bits(hid), want_h, dt, "Wo + residual")
    assert ctx.status() == 0
    ctx.close()
