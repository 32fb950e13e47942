"""Writer of a tiny synthetic `deepseek2` GGUF file (version 3) with seeded random weights.

Test infrastructure.  Two users: `make_golden.py` / `tests/test_oracle.py` drive the reference's own
`from_gguf` + `forward()` on such a file (where the reference tree is mounted), and the GGUF-ingestion
tests hand the same file to this library's loader.  The layout follows the GGUF specification: header,
key/value pairs, tensor infos (dimensions innermost first, so an (M_out x K_in) matrix has dims [K_in, M_out]),
padding to 32 bytes, tensor data.  The MLA dimensions are the ones the kernels are built for
(kv_lora_rank 512, rope 64, nope 128, v 128); everything around them is kept small.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

GGUF_MAGIC = 0x46554747
T_U32, T_F32, T_STRING = 4, 6, 8
GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0 = 0, 1, 2, 8


@dataclass
class TinyModel:
    n_layers: int = 2
    n_heads: int = 4
    embed: int = 128
    q_lora_rank: int = 96          # 0: a full attn_q tensor instead of the LoRA pair
    merged_kv_b: bool = False      # True: one attn_kv_b tensor with per-head [128 nope rows | 128 v rows]
    vocab: int = 16
    ffn: int = 64
    context_length: int = 256
    rope_theta: float = 10000.0
    rope_factor: float = 40.0      # <= 1: plain RoPE
    rope_orig_ctx: int = 4096
    eps: float = 1e-6
    seed: int = 7
    kv_b_type: int = GGML_F16      # F16, Q8_0 or Q4_0 for attn_k_b / attn_v_b / attn_kv_b
    tensors: dict = field(default_factory=dict)   # name -> (ggml type, dims innermost-first, raw bytes, float32 values or None)


def _str(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, vtype: int, value) -> bytes:
    out = _str(key) + struct.pack("<I", vtype)
    if vtype == T_U32:
        return out + struct.pack("<I", value)
    if vtype == T_F32:
        return out + struct.pack("<f", value)
    if vtype == T_STRING:
        return out + _str(value)
    raise ValueError(vtype)


def build(m: TinyModel) -> bytes:
    """Fills m.tensors and returns the file's bytes."""
    from mugen_b200 import synth
    rng = np.random.default_rng(m.seed)
    H, E = m.n_heads, m.embed

    def f16(name, rows, cols, scale):
        w = (rng.standard_normal((rows, cols)) * scale).astype(np.float32).astype(np.float16)
        m.tensors[name] = (GGML_F16, [cols, rows], w.tobytes(), w.astype(np.float32))

    def norm(name, n, as_f32=True):
        w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        if as_f32:
            m.tensors[name] = (GGML_F32, [n], w.tobytes(), w)
        else:
            m.tensors[name] = (GGML_F16, [n], w.astype(np.float16).tobytes(), w.astype(np.float16).astype(np.float32))

    def kv_b(name, rows):
        w = (rng.standard_normal((rows, 512)) * 0.05).astype(np.float32)
        if m.kv_b_type == GGML_F16:
            h = w.astype(np.float16)
            m.tensors[name] = (GGML_F16, [512, rows], h.tobytes(), h.astype(np.float32))
        elif m.kv_b_type == GGML_Q8_0:
            m.tensors[name] = (GGML_Q8_0, [512, rows], synth.pack_q8_0(w).tobytes(), None)
        else:
            m.tensors[name] = (GGML_Q4_0, [512, rows], synth.pack_q4_0(w).tobytes(), None)

    f16("token_embd.weight", m.vocab, E, 1.0)
    norm("output_norm.weight", E)
    for L in range(m.n_layers):
        b = f"blk.{L}."
        norm(b + "attn_norm.weight", E)
        norm(b + "ffn_norm.weight", E, as_f32=False)
        if m.q_lora_rank:
            f16(b + "attn_q_a.weight", m.q_lora_rank, E, 1.0 / np.sqrt(E))
            norm(b + "attn_q_a_norm.weight", m.q_lora_rank)
            f16(b + "attn_q_b.weight", H * 192, m.q_lora_rank, 1.0 / np.sqrt(m.q_lora_rank))
        else:
            f16(b + "attn_q.weight", H * 192, E, 1.0 / np.sqrt(E))
        f16(b + "attn_kv_a_mqa.weight", 576, E, 1.0 / np.sqrt(E))
        norm(b + "attn_kv_a_norm.weight", 512)
        if m.merged_kv_b:
            kv_b(b + "attn_kv_b.weight", H * 256)
        else:
            kv_b(b + "attn_k_b.weight", H * 128)
            kv_b(b + "attn_v_b.weight", H * 128)
        f16(b + "attn_output.weight", E, H * 128, 1.0 / np.sqrt(H * 128))
        f16(b + "ffn_gate.weight", m.ffn, E, 1.0 / np.sqrt(E))
        f16(b + "ffn_up.weight", m.ffn, E, 1.0 / np.sqrt(E))
        f16(b + "ffn_down.weight", E, m.ffn, 1.0 / np.sqrt(m.ffn))

    a = "deepseek2."
    kvs = [
        _kv("general.architecture", T_STRING, "deepseek2"),
        _kv("general.name", T_STRING, "tiny synthetic MLA model"),
        _kv(a + "block_count", T_U32, m.n_layers),
        _kv(a + "vocab_size", T_U32, m.vocab),
        _kv(a + "embedding_length", T_U32, E),
        _kv(a + "attention.head_count", T_U32, H),
        _kv(a + "context_length", T_U32, m.context_length),
        _kv(a + "feed_forward_length", T_U32, m.ffn),
        _kv(a + "attention.kv_lora_rank", T_U32, 512),
        _kv(a + "rope.dimension_count", T_U32, 64),
        _kv(a + "attention.key_length", T_U32, 192),
        _kv(a + "attention.value_length", T_U32, 128),
        _kv(a + "rope.freq_base", T_F32, m.rope_theta),
        _kv(a + "rope.scaling.factor", T_F32, m.rope_factor),
        _kv(a + "rope.scaling.original_context_length", T_U32, m.rope_orig_ctx),
        _kv(a + "attention.layer_norm_rms_epsilon", T_F32, m.eps),
    ]
    if m.q_lora_rank:
        kvs.append(_kv(a + "attention.q_lora_rank", T_U32, m.q_lora_rank))

    infos, blobs, off = b"", [], 0
    for name, (ttype, dims, raw, _) in m.tensors.items():
        infos += _str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", ttype, off)
        pad = (-len(raw)) % 32
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    head = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(m.tensors), len(kvs)) + b"".join(kvs) + infos
    head += b"\0" * ((-len(head)) % 32)
    return head + b"".join(blobs)


def write(path: str, m: TinyModel) -> TinyModel:
    with open(path, "wb") as f:
        f.write(build(m))
    return m
