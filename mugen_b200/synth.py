"""Seeded synthetic inputs with the shapes and value distributions of DeepSeek-style MLA layers.

The reference is measured on real GGUF chat models that are not available offline, so
every test and benchmark draws inputs from here instead: latent cache rows ~N(0,1), W_UK and
W_UV ~N(0,0.02), queries ~N(0,0.9) (the spread of W_q·x for W_q~N(0,0.02), x~N(0,1), hidden 2048).
Half and bfloat16 tensors are carried as uint16 bit patterns so that numpy can hold them.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass

import numpy as np

ROW, QDIM, VDIM, RANK, ROPE, NOPE = 576, 192, 128, 512, 64, 128
DT_F16, DT_BF16 = 0, 1
W_F16, W_Q4_0, W_Q8_0, W_BF16 = 1, 2, 8, 30


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_bits(x: np.ndarray, dt: int) -> np.ndarray:
    """float32 values -> storage bit patterns (round to nearest even)."""
    if dt == DT_F16:
        return np.ascontiguousarray(x, np.float32).astype(np.float16).view(np.uint16)
    return f32_to_bf16_bits(x)


def from_bits(b: np.ndarray, dt: int) -> np.ndarray:
    if dt == DT_F16:
        return np.ascontiguousarray(b, np.uint16).view(np.float16).astype(np.float32)
    return bf16_bits_to_f32(b)


def both_representable(x: np.ndarray) -> np.ndarray:
    """Round to bfloat16 and flush magnitudes below 2**-14 to zero, so that the value is
    exact in bfloat16 AND in IEEE half: the f16-only reference can then be run on the very
    numbers a bf16 cache holds."""
    y = bf16_bits_to_f32(f32_to_bf16_bits(x))
    y[np.abs(y) < 2.0 ** -14] = 0.0
    return y


def pack_q8_0(w: np.ndarray) -> np.ndarray:
    """float32 [rows][512] -> GGML Q8_0 bytes (34-byte blocks: f16 scale + 32 int8)."""
    rows = w.shape[0]
    blk = w.reshape(rows, -1, 32)
    amax = np.abs(blk).max(axis=2)
    d = (amax / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df > 0, 1.0 / np.where(df > 0, df, 1), 0.0)
    q = np.clip(np.rint(blk * inv[..., None]), -127, 127).astype(np.int8)
    out = np.empty((rows, blk.shape[1], 34), np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, -1, 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(rows, -1)


def pack_q4_0(w: np.ndarray) -> np.ndarray:
    """float32 [rows][512] -> GGML Q4_0 bytes (18-byte blocks: f16 scale + 16 nibble bytes;
    low nibbles hold elements 0..15, high nibbles 16..31, value = (n - 8) * scale)."""
    rows = w.shape[0]
    blk = w.reshape(rows, -1, 32)
    idx = np.abs(blk).argmax(axis=2)
    mx = np.take_along_axis(blk, idx[..., None], axis=2)[..., 0]
    d = (mx / -8.0).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, 1.0 / np.where(df != 0, df, 1), 0.0)
    q = np.clip(np.floor(blk * inv[..., None] + 8.5), 0, 15).astype(np.uint8)
    out = np.empty((rows, blk.shape[1], 18), np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, -1, 2)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(rows, -1)


@dataclass
class LayerCase:
    """Inputs of one attention layer call over a batch of sequences."""
    n_heads: int
    dt: int
    w_type: int
    seq_lens: list[int]
    q: np.ndarray            # [B][H][192] bits (post-RoPE, as the attention op receives it)
    caches: list[np.ndarray]  # per sequence [S_b][576] bits (the last row is the appended one)
    w_uk: np.ndarray          # raw weight bytes in w_type
    w_uv: np.ndarray
    w_uk_f32: np.ndarray      # the values those bytes decode to
    w_uv_f32: np.ndarray
    norm_w: np.ndarray        # [512] bits
    kv_a: np.ndarray          # [B][576] bits, pre-norm / pre-RoPE rows for the appended token

    def digest(self) -> str:
        h = hashlib.sha256()
        for a in (self.q, *self.caches, self.w_uk, self.w_uv, self.norm_w, self.kv_a):
            h.update(np.ascontiguousarray(a).tobytes())
        return h.hexdigest()


def make_layer_case(seed: int, n_heads: int, seq_lens, dt: int = DT_F16, w_type: int | None = None,
                    q_scale: float = 1.0, exact_in_both: bool = False,
                    norm_random: bool = True) -> LayerCase:
    """Draw order: cache rows, q, W_UK, W_UV, norm weight, kv_a."""
    rng = np.random.default_rng(seed)
    if w_type is None:
        w_type = W_F16 if dt == DT_F16 else W_BF16
    fix = both_representable if exact_in_both else (lambda a: a)
    caches = [to_bits(fix(rng.standard_normal((s, ROW), np.float32)), dt) for s in seq_lens]
    q = to_bits(fix(rng.standard_normal((len(seq_lens), n_heads, QDIM), np.float32)
                    * np.float32(0.9 * q_scale)), dt)
    wk = fix(rng.standard_normal((n_heads * NOPE, RANK), np.float32) * np.float32(0.02))
    wv = fix(rng.standard_normal((n_heads * VDIM, RANK), np.float32) * np.float32(0.02))
    if w_type == W_F16:
        w_uk, w_uv = to_bits(wk, DT_F16), to_bits(wv, DT_F16)
        wk_f, wv_f = from_bits(w_uk, DT_F16), from_bits(w_uv, DT_F16)
    elif w_type == W_BF16:
        w_uk, w_uv = to_bits(wk, DT_BF16), to_bits(wv, DT_BF16)
        wk_f, wv_f = from_bits(w_uk, DT_BF16), from_bits(w_uv, DT_BF16)
    elif w_type == W_Q8_0:
        w_uk, w_uv = pack_q8_0(wk), pack_q8_0(wv)
        wk_f, wv_f = unpack_q8_0(w_uk), unpack_q8_0(w_uv)
    elif w_type == W_Q4_0:
        w_uk, w_uv = pack_q4_0(wk), pack_q4_0(wv)
        wk_f, wv_f = unpack_q4_0(w_uk), unpack_q4_0(w_uv)
    else:
        raise ValueError(f"unsupported weight type {w_type}")
    nw = 1.0 + 0.1 * rng.standard_normal(RANK, np.float32) if norm_random else np.ones(RANK, np.float32)
    norm_w = to_bits(fix(nw.astype(np.float32)), dt)
    kv_a = to_bits(fix(rng.standard_normal((len(seq_lens), ROW), np.float32)), dt)
    return LayerCase(n_heads, dt, w_type, list(seq_lens), q, caches, w_uk, w_uv, wk_f, wv_f,
                     norm_w, kv_a)


def unpack_q8_0(b: np.ndarray) -> np.ndarray:
    rows = b.shape[0]
    blk = b.reshape(rows, -1, 34)
    d = np.ascontiguousarray(blk[..., 0:2]).view(np.float16).astype(np.float32)
    q = np.ascontiguousarray(blk[..., 2:]).view(np.int8).astype(np.float32)
    return (d * q).reshape(rows, -1)


def unpack_q4_0(b: np.ndarray) -> np.ndarray:
    rows = b.shape[0]
    blk = b.reshape(rows, -1, 18)
    d = np.ascontiguousarray(blk[..., 0:2]).view(np.float16).astype(np.float32)
    qs = blk[..., 2:]
    lo = (qs & 0x0F).astype(np.float32) - 8.0
    hi = (qs >> 4).astype(np.float32) - 8.0
    return (np.concatenate([lo, hi], axis=2) * d).reshape(rows, -1)


def ragged_lengths(seed: int, n: int, lo: int, hi: int) -> list[int]:
    """Lengths ~ log-uniform in [lo, hi]."""
    rng = np.random.default_rng(seed)
    return [int(round(float(np.exp(u)))) for u in rng.uniform(np.log(lo), np.log(hi), n)]


def error_norms(got_bits: np.ndarray, want_bits: np.ndarray, dt_got: int, dt_want: int):
    """(max-abs error, relative L2 error) between two bit-pattern tensors."""
    g = from_bits(got_bits, dt_got).astype(np.float64).ravel()
    w = from_bits(want_bits, dt_want).astype(np.float64).ravel()
    den = float(np.sqrt((w * w).sum()))
    return float(np.abs(g - w).max()), float(np.sqrt(((g - w) ** 2).sum()) / max(den, 1e-30))
