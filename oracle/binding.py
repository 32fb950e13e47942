"""ctypes bindings of the CPU checker.

TEST INFRASTRUCTURE ONLY.  Importers allowed: tests/, __graft_entry__.smoke() and
the cpu_baseline / --impl reference legs of bench.py.  The product package
(mugen_b200) never imports this module.

Two libraries live here:
  * libmla_oracle.so       — this repository's restatement (oracle/mla_oracle.cpp);
  * _ref/libmugen_ref.so   — the reference's own sources compiled in place
                             (oracle/ref_harness.cpp); present only where it was
                             built, i.e. where the reference tree was mounted.
All array arguments are C-contiguous numpy arrays; half and bfloat16 values
travel as their uint16 bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
DT_F16, DT_BF16 = 0, 1
W_F16, W_Q4_0, W_Q8_0, W_BF16 = 1, 2, 8, 30
ROW, QDIM, VDIM, RANK, ROPE, NOPE = 576, 192, 128, 512, 64, 128

_u32, _f32, _vp = C.c_uint32, C.c_float, C.c_void_p


def build(ref: bool | None = None) -> None:
    """Compile the checker libraries (and the reference build when its tree is present)."""
    targets = ["all"]
    ref_root = os.environ.get("MUGEN_REF_ROOT", "/root/reference")
    if ref is None:
        ref = os.path.isdir(os.path.join(ref_root, "src", "core", "model"))
    if ref:
        targets.append("ref")
    subprocess.run(["make", "-C", _HERE, f"REF_ROOT={ref_root}", *targets], check=True,
                   stdout=subprocess.DEVNULL)


def _ptr(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(_vp)


class _Oracle:
    def __init__(self) -> None:
        path = os.path.join(_HERE, "libmla_oracle.so")
        if not os.path.exists(path):
            build(ref=False)
        L = C.CDLL(path)
        L.oracle_yarn_rope_freq.restype = _f32
        L.oracle_yarn_rope_freq.argtypes = [_u32, _u32, _f32, _u32, _f32]
        L.oracle_rope_cos_sin.argtypes = [_u32, _f32, _u32, _f32, _vp, _vp]
        L.oracle_append_rows.argtypes = [_vp, _u32, _vp, _vp, _f32, _f32, _u32, _f32, _u32, _vp]
        L.oracle_q_rope.argtypes = [_vp, _u32, _u32, _f32, _u32, _f32, _u32]
        L.oracle_mla_attention.argtypes = [_vp, _vp, _u32, _vp, _vp, _u32, _u32, _vp, _u32]
        L.oracle_mla_partial.argtypes = [_vp, _vp, _u32, _u32, _vp, _u32, _u32, _u32, _vp]
        L.oracle_mla_attention_batch.argtypes = [_vp, _vp, _vp, _u32, _vp, _vp, _u32, _u32, _vp,
                                                 _u32, _u32]
        self.L = L

    def yarn_rope_freq(self, pair, rope_dim, factor, orig_ctx, theta) -> np.float32:
        return np.float32(self.L.oracle_yarn_rope_freq(pair, rope_dim, factor, orig_ctx, theta))

    def rope_cos_sin(self, pos, factor, orig_ctx, theta):
        c = np.empty(32, np.float32)
        s = np.empty(32, np.float32)
        self.L.oracle_rope_cos_sin(pos, factor, orig_ctx, theta, _ptr(c), _ptr(s))
        return c, s

    def append_rows(self, kv_a, positions, norm_w, eps, factor, orig_ctx, theta, dt):
        kv_a = np.ascontiguousarray(kv_a, np.uint16).reshape(-1, ROW)
        positions = np.ascontiguousarray(positions, np.uint32)
        out = np.empty_like(kv_a)
        self.L.oracle_append_rows(_ptr(kv_a), kv_a.shape[0], _ptr(positions),
                                  _ptr(np.ascontiguousarray(norm_w, np.uint16)), eps, factor,
                                  orig_ctx, theta, dt, _ptr(out))
        return out

    def q_rope(self, q, pos, factor, orig_ctx, theta, dt):
        q = np.array(q, np.uint16, copy=True).reshape(-1, QDIM)
        self.L.oracle_q_rope(_ptr(q), q.shape[0], pos, factor, orig_ctx, theta, dt)
        return q

    def attention(self, q, cache, seq_len, w_uk, w_uv, w_type, n_heads, dt):
        out = np.empty((n_heads, VDIM), np.uint16)
        self.L.oracle_mla_attention(_ptr(q), _ptr(cache), seq_len, _ptr(w_uk), _ptr(w_uv),
                                    w_type, n_heads, _ptr(out), dt)
        return out

    def partial(self, q, cache, row_begin, row_end, w_uk, w_type, n_heads, dt):
        p = np.empty((n_heads, RANK + 2), np.float32)
        self.L.oracle_mla_partial(_ptr(q), _ptr(cache), row_begin, row_end, _ptr(w_uk), w_type,
                                  n_heads, dt, _ptr(p))
        return p

    def attention_batch(self, q, caches, seq_lens, w_uk, w_uv, w_type, n_heads, dt, n_threads):
        n = len(caches)
        ptrs = (C.c_void_p * n)(*[c.ctypes.data for c in caches])
        lens = np.ascontiguousarray(seq_lens, np.uint32)
        out = np.empty((n, n_heads, VDIM), np.uint16)
        self.L.oracle_mla_attention_batch(_ptr(q), ptrs, _ptr(lens), n, _ptr(w_uk), _ptr(w_uv),
                                          w_type, n_heads, _ptr(out), dt, n_threads)
        return out


class _Reference:
    """The reference's own code (f16 only, as the reference is)."""

    def __init__(self, path: str) -> None:
        L = C.CDLL(path)
        L.ref_yarn_rope_freq.restype = _f32
        L.ref_yarn_rope_freq.argtypes = [_u32, _u32, _f32, _u32, _f32]
        L.ref_mla_attention.argtypes = [_vp, _vp, _u32, _vp, _vp, _u32, _u32, _vp]
        L.ref_mla_attention_batch.argtypes = [_vp, _vp, _vp, _u32, _vp, _vp, _u32, _u32, _vp, _u32]
        L.ref_kvcache_create.restype = _vp
        L.ref_kvcache_create.argtypes = [_u32, _u32]
        L.ref_kvcache_destroy.argtypes = [_vp]
        L.ref_kvcache_seq_len.restype = _u32
        L.ref_kvcache_seq_len.argtypes = [_vp]
        L.ref_kvcache_advance.argtypes = [_vp, _u32]
        L.ref_kvcache_truncate.argtypes = [_vp, _u32]
        L.ref_kvcache_clear.argtypes = [_vp]
        for f in ("ref_ggml_f16", "ref_ggml_q8_0", "ref_ggml_q4_0"):
            getattr(L, f).restype = _u32
        assert (L.ref_ggml_f16(), L.ref_ggml_q4_0(), L.ref_ggml_q8_0()) == (W_F16, W_Q4_0, W_Q8_0)
        self.L = L

    def yarn_rope_freq(self, pair, rope_dim, factor, orig_ctx, theta) -> np.float32:
        return np.float32(self.L.ref_yarn_rope_freq(pair, rope_dim, factor, orig_ctx, theta))

    def attention(self, q, cache, seq_len, w_uk, w_uv, w_type, n_heads):
        out = np.empty((n_heads, VDIM), np.uint16)
        self.L.ref_mla_attention(_ptr(q), _ptr(cache), seq_len, _ptr(w_uk), _ptr(w_uv), w_type,
                                 n_heads, _ptr(out))
        return out

    def attention_batch(self, q, caches, seq_lens, w_uk, w_uv, w_type, n_heads, n_threads):
        n = len(caches)
        ptrs = (C.c_void_p * n)(*[c.ctypes.data for c in caches])
        lens = np.ascontiguousarray(seq_lens, np.uint32)
        out = np.empty((n, n_heads, VDIM), np.uint16)
        self.L.ref_mla_attention_batch(_ptr(q), ptrs, _ptr(lens), n, _ptr(w_uk), _ptr(w_uv),
                                       w_type, n_heads, _ptr(out), n_threads)
        return out


_oracle: _Oracle | None = None
_reference: _Reference | None | bool = False


def oracle() -> _Oracle:
    global _oracle
    if _oracle is None:
        _oracle = _Oracle()
    return _oracle


def reference() -> _Reference | None:
    """The compiled reference, or None where it was never built (e.g. on a GPU box whose
    snapshot did not carry oracle/_ref)."""
    global _reference
    if _reference is False:
        path = os.path.join(_HERE, "_ref", "libmugen_ref.so")
        _reference = _Reference(path) if os.path.exists(path) else None
    return _reference
