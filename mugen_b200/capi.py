"""ctypes binding of libmugen_mla.so — the C ABI declared in include/mugen_mla.h.

Every call goes to the CUDA library; there is no Python or CPU implementation behind these
names.  If the shared object is missing it is built with nvcc; if that is impossible the
import of the library fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

u32, u64, i32, f32, vp = C.c_uint32, C.c_uint64, C.c_int32, C.c_float, C.c_void_p

OK = 0
ERR_NAMES = {1: "INVALID", 2: "CUDA", 3: "NO_PAGES", 4: "CAPACITY", 5: "STATE", 6: "DEVICE",
             7: "UNSUPPORTED"}
DTYPE_F16, DTYPE_BF16 = 0, 1
W_F16, W_Q4_0, W_Q8_0, W_BF16 = 1, 2, 8, 30
KERNEL_AUTO, KERNEL_MMA, KERNEL_TCGEN05, KERNEL_TCGEN05_PAIR128, KERNEL_TCGEN05_T16 = 0, 1, 2, 3, 4


class MlaConfig(C.Structure):
    _fields_ = [("n_layers", u32), ("n_heads", u32), ("kv_lora_rank", u32),
                ("qk_nope_head_dim", u32), ("qk_rope_head_dim", u32), ("v_head_dim", u32),
                ("rope_theta", f32), ("rms_norm_eps", f32), ("rope_scaling_factor", f32),
                ("rope_original_ctx", u32), ("max_seq_len", u32), ("page_tokens", u32),
                ("n_pages", u32), ("max_seqs", u32), ("max_rows", u32), ("dtype", u32),
                ("device", i32), ("kernel", u32), ("max_position", u32)]


class GgufInfo(C.Structure):
    _fields_ = [(n, u32) for n in ("n_layers", "n_heads", "embedding_length", "context_length", "kv_lora_rank",
                                   "q_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim",
                                   "rope_original_ctx")] + [(n, f32) for n in ("rope_theta", "rope_scaling_factor",
                                                                               "rms_norm_eps")]


class BlockWeights(C.Structure):
    _fields_ = [("embedding_length", u32), ("q_lora_rank", u32)] + [(n, vp) for n in (
        "attn_norm", "q_a", "q_a_norm", "q_b", "q", "kv_a_mqa", "wo")]


# name -> (restype, argtypes); must list every symbol include/mugen_mla.h declares
SIGNATURES = {
    "mla_create": (C.c_int, [C.POINTER(MlaConfig), C.POINTER(vp)]),
    "mla_destroy": (None, [vp]),
    "mla_last_error": (C.c_char_p, [vp]),
    "mla_status": (C.c_int, [vp, vp, C.POINTER(u32)]),
    "mla_set_layer_weights": (C.c_int, [vp, u32, vp, vp, u32, vp]),
    "mla_seq_create": (C.c_int, [vp, C.POINTER(u32)]),
    "mla_seq_free": (C.c_int, [vp, u32]),
    "mla_seq_len": (C.c_int, [vp, u32, C.POINTER(u32)]),
    "mla_advance": (C.c_int, [vp, u32, u32]),
    "mla_truncate": (C.c_int, [vp, u32, u32]),
    "mla_clear": (C.c_int, [vp, u32]),
    "mla_seq_set_base": (C.c_int, [vp, u32, u32]),
    "mla_free_pages": (C.c_int, [vp, C.POINTER(u32)]),
    "mla_shuffle_free_pages": (C.c_int, [vp, u64]),
    "mla_seq_pages": (C.c_int, [vp, u32, vp, u32, C.POINTER(u32)]),
    "mla_append_rows": (C.c_int, [vp, u32, u32, vp, vp, vp, vp]),
    "mla_attend_rows": (C.c_int, [vp, u32, u32, vp, vp, vp, vp, vp]),
    "mla_step_begin": (C.c_int, [vp, u32, vp, vp, vp]),
    "mla_step_append": (C.c_int, [vp, u32, vp, vp]),
    "mla_step_attend": (C.c_int, [vp, u32, vp, vp, vp]),
    "mla_step_layers": (C.c_int, [vp, u32, u32, vp, vp, vp, vp]),
    "mla_step_layer_host": (C.c_int, [vp, u32, vp, vp, vp, vp]),
    "mla_step_end": (C.c_int, [vp]),
    "mla_step_info": (C.c_int, [vp, C.POINTER(u32), C.POINTER(u32)]),
    "mla_step_attend_partial": (C.c_int, [vp, u32, vp, vp, vp]),
    "mla_step_layer_partial": (C.c_int, [vp, u32, vp, vp, vp, vp]),
    "mla_merge_partials": (C.c_int, [vp, u32, u32, u32, vp, vp, vp]),
    "mla_launch_count": (C.c_int, [vp, C.POINTER(u64)]),
    "mla_kernel_name": (C.c_char_p, [vp]),
    "mla_set_q_rope": (C.c_int, [vp, C.c_int]),
    "mla_profile_enable": (C.c_int, [vp, C.c_int]),
    "mla_set_block_weights": (C.c_int, [vp, u32, C.POINTER(BlockWeights)]),
    "mla_block_project_in": (C.c_int, [vp, u32, u32, vp, vp, vp, vp]),
    "mla_block_project_out": (C.c_int, [vp, u32, u32, vp, vp, vp]),
    "mla_step_block": (C.c_int, [vp, u32, vp, vp]),
    "mla_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(vp)]),
    "mla_gguf_close": (None, [vp]),
    "mla_gguf_last_error": (C.c_char_p, []),
    "mla_gguf_get_info": (C.c_int, [vp, C.POINTER(GgufInfo)]),
    "mla_gguf_fill_config": (C.c_int, [vp, C.POINTER(MlaConfig)]),
    "mla_gguf_layer_weights": (C.c_int, [vp, u32, vp, vp, C.c_size_t, C.POINTER(u32), C.POINTER(C.c_size_t), vp]),
    "mla_gguf_register": (C.c_int, [vp, vp, u32]),
    "mla_rollback": (C.c_int, [vp, u32, vp, vp]),
    "mla_step_balance": (C.c_int, [vp, C.POINTER(u32), C.POINTER(u32), C.POINTER(u32)]),
    "mla_selftest_wait_timeout": (C.c_int, [vp, C.c_uint64, vp, C.POINTER(u32)]),
    "mla_profile_read": (C.c_int, [vp, C.POINTER(u32), C.POINTER(f32)]),
    "mla_read_rows": (C.c_int, [vp, u32, u32, u32, u32, vp, vp]),
    "mla_write_rows": (C.c_int, [vp, u32, u32, u32, u32, vp, vp]),
    "mla_attention_noalloc": (C.c_int, [u32, u32, u32, vp, vp, vp, vp, vp, vp]),
    "mla_noalloc_last_error": (C.c_char_p, []),
}

_lib = None


def lib_path() -> str:
    return _build.LIB


def load() -> C.CDLL:
    """Loads (building first if needed) the CUDA library and types every exported symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_build.LIB):
        _build.build_library()
    lib = C.CDLL(_build.LIB)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError = a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class MlaError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"MLA_ERR_{ERR_NAMES.get(code, code)}: {text}")
        self.code = code
