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
        L.ref_model_load.restype = _vp
        L.ref_model_load.argtypes = [C.c_char_p]
        L.ref_model_free.argtypes = [_vp]
        L.ref_model_last_error.restype = C.c_char_p
        L.ref_model_config.argtypes = [_vp, _vp, _vp]
        L.ref_model_weight.restype = _u32
        L.ref_model_weight.argtypes = [_vp, _u32, _u32, _vp, C.c_size_t]
        L.ref_model_forward.restype = C.c_int
        L.ref_model_forward.argtypes = [_vp, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp]
        L.ref_model_cache_rows.argtypes = [_vp, _u32, _u32, _u32, _vp]
        L.ref_model_seq_len.restype = _u32
        L.ref_model_seq_len.argtypes = [_vp]
        L.ref_model_truncate.argtypes = [_vp, _u32]
        self.L = L

    def load_model(self, gguf_path: str) -> "_RefModel":
        """The reference's from_gguf on a GGUF file (see _RefModel)."""
        return _RefModel(self.L, gguf_path)

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


class _RefModel:
    """The reference's TransformerModel built by its own from_gguf from a GGUF file, driven through its own
    forward() on host stand-ins of the Metal layer (oracle/ref_harness.cpp).  forward() returns what the
    decode driver's host code read and wrote per layer."""
    WEIGHTS = dict(w_uk=0, w_uv=1, kv_a_norm=2, kv_a_mqa=3, q_a=4, q_a_norm=5, q_b=6, q=7, wo=8, attn_norm=9)

    def __init__(self, L, path: str) -> None:
        self.L = L
        self.h = L.ref_model_load(path.encode())
        if not self.h:
            raise RuntimeError(L.ref_model_last_error().decode())
        cfg = np.zeros(12, np.uint32)
        fcfg = np.zeros(3, np.float32)
        L.ref_model_config(self.h, _ptr(cfg), _ptr(fcfg))
        names = ["n_layers", "n_heads", "embed", "kv_lora_rank", "q_lora_rank", "qk_nope", "qk_rope", "v_head_dim",
                 "rope_original_ctx", "max_seq_len", "vocab", "ffn"]
        self.cfg = {k: int(v) for k, v in zip(names, cfg)}
        self.cfg.update(rope_theta=float(fcfg[0]), rope_scaling_factor=float(fcfg[1]), rms_norm_eps=float(fcfg[2]))

    def close(self) -> None:
        if self.h:
            self.L.ref_model_free(self.h)
            self.h = None

    def weight(self, layer: int, which: str, n_bytes: int):
        """(GGML type, raw bytes) of a layer's weight as the loaded model holds it, or None when absent."""
        buf = np.zeros(n_bytes, np.uint8)
        t = self.L.ref_model_weight(self.h, layer, self.WEIGHTS[which], _ptr(buf), n_bytes)
        return None if t == 0xFFFFFFFF else (int(t), buf)

    def forward(self, token: int, pos: int) -> dict:
        c = self.cfg
        Lr, H, E = c["n_layers"], c["n_heads"], c["embed"]
        t = dict(hidden_in=np.zeros((Lr, E), np.uint16), q_pre=np.zeros((Lr, H, QDIM), np.uint16),
                 q_post=np.zeros((Lr, H, QDIM), np.uint16), kv_a_pre=np.zeros((Lr, ROW), np.uint16),
                 attn_out=np.zeros((Lr, H, VDIM), np.uint16), hidden_mid=np.zeros((Lr, E), np.uint16))
        rc = self.L.ref_model_forward(self.h, token, pos, _ptr(t["hidden_in"]), _ptr(t["q_pre"]), _ptr(t["q_post"]),
                                      _ptr(t["kv_a_pre"]), _ptr(t["attn_out"]), _ptr(t["hidden_mid"]))
        if rc:
            raise RuntimeError(self.L.ref_model_last_error().decode())
        return t

    def cache_rows(self, layer: int, row_begin: int, n: int) -> np.ndarray:
        out = np.zeros((n, ROW), np.uint16)
        self.L.ref_model_cache_rows(self.h, layer, row_begin, n, _ptr(out))
        return out

    def seq_len(self) -> int:
        return int(self.L.ref_model_seq_len(self.h))


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
