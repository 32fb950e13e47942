"""Host-side mirror of the reference's attention-op / KV-cache interface over the C ABI.

`MlaContext` owns one `mla_ctx` (one GPU).  Method names follow the reference's vocabulary:
`seq_len / advance_seq_len / truncate / clear` are mugen::KVCache's (src/core/memory/kv_cache.h:
22-41) with a sequence id added; `append_rows` is steps G+H of the decode driver
(src/core/model/transformer.cpp:3930-3987); `attend_rows` is cpu_mla_attention (:2539-2623)
batched; `step_*` is the decode-step scheduler.  Device buffers are torch CUDA tensors (torch is
plumbing here: memory and streams); every computation happens in libmugen_mla.so.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi

ROW, QDIM, VDIM, RANK = 576, 192, 128, 512


def _np_ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


class MlaContext:
    def __init__(self, *, n_layers: int, n_heads: int, dtype: int, n_pages: int, max_seqs: int,
                 max_seq_len: int, max_rows: int = 0, rope_theta: float = 10000.0,
                 rope_scaling_factor: float = 40.0, rope_original_ctx: int = 4096,
                 rms_norm_eps: float = 1e-6, device: int = 0, kernel: int = capi.KERNEL_AUTO,
                 max_position: int = 0):
        self.lib = capi.load()
        self.cfg = capi.MlaConfig(n_layers, n_heads, 512, 128, 64, 128, rope_theta, rms_norm_eps,
                                  rope_scaling_factor, rope_original_ctx, max_seq_len, 64, n_pages,
                                  max_seqs, max_rows, dtype, device, kernel, max_position)
        self.n_heads, self.n_layers, self.dtype, self.device = n_heads, n_layers, dtype, device
        h = C.c_void_p()
        rc = self.lib.mla_create(C.byref(self.cfg), C.byref(h))
        if rc != capi.OK:
            raise capi.MlaError(rc, self.lib.mla_last_error(None).decode())
        self.h = h

    # ---- plumbing ---------------------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc != capi.OK:
            raise capi.MlaError(rc, self.lib.mla_last_error(self.h).decode())

    @staticmethod
    def _stream():
        import torch
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    @staticmethod
    def _dev(t):
        assert t.is_cuda and t.is_contiguous()
        return C.c_void_p(t.data_ptr())

    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.mla_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- weights ----------------------------------------------------------------------
    def set_layer_weights(self, layer: int, w_uk: np.ndarray, w_uv: np.ndarray, w_type: int,
                          norm_w: np.ndarray) -> None:
        w_uk, w_uv = np.ascontiguousarray(w_uk), np.ascontiguousarray(w_uv)
        norm_w = np.ascontiguousarray(norm_w, np.uint16)
        self._check(self.lib.mla_set_layer_weights(self.h, layer, _np_ptr(w_uk), _np_ptr(w_uv), w_type,
                                                   _np_ptr(norm_w)))

    # ---- sequences (KVCache contract) -------------------------------------------------
    def seq_create(self) -> int:
        v = C.c_uint32()
        self._check(self.lib.mla_seq_create(self.h, C.byref(v)))
        return v.value

    def seq_free(self, seq: int) -> None:
        self._check(self.lib.mla_seq_free(self.h, seq))

    def seq_len(self, seq: int) -> int:
        v = C.c_uint32()
        self._check(self.lib.mla_seq_len(self.h, seq, C.byref(v)))
        return v.value

    def advance_seq_len(self, seq: int, n: int = 1) -> None:
        self._check(self.lib.mla_advance(self.h, seq, n))

    # ---- the projections around the op (steps A-D, F, J, K of the decode driver) -------------------
    def set_block_weights(self, layer: int, *, attn_norm, kv_a_mqa, wo, q=None, q_a=None, q_a_norm=None, q_b=None) -> None:
        """All arrays: uint16 bit patterns in the context dtype, row-major [outputs][inputs] as GGUF holds them."""
        arrs = dict(attn_norm=attn_norm, q_a=q_a, q_a_norm=q_a_norm, q_b=q_b, q=q, kv_a_mqa=kv_a_mqa, wo=wo)
        arrs = {k: (None if v is None else np.ascontiguousarray(v, np.uint16)) for k, v in arrs.items()}
        w = capi.BlockWeights(int(arrs["attn_norm"].size), 0 if q_a is None else int(arrs["q_a"].shape[0]),
                              *[None if arrs[k] is None else _np_ptr(arrs[k]) for k in
                                ("attn_norm", "q_a", "q_a_norm", "q_b", "q", "kv_a_mqa", "wo")])
        self._check(self.lib.mla_set_block_weights(self.h, layer, C.byref(w)))

    def block_project_in(self, layer: int, hidden, q, kv_a) -> None:
        self._check(self.lib.mla_block_project_in(self.h, layer, hidden.shape[0], self._dev(hidden), self._dev(q),
                                                  self._dev(kv_a), self._stream()))

    def block_project_out(self, layer: int, attn_out, hidden) -> None:
        self._check(self.lib.mla_block_project_out(self.h, layer, hidden.shape[0], self._dev(attn_out), self._dev(hidden),
                                                   self._stream()))

    def step_block(self, layer: int, hidden) -> None:
        self._check(self.lib.mla_step_block(self.h, layer, self._dev(hidden), self._stream()))

    def rollback(self, seq_ids, keep_lens) -> None:
        """Speculative-decode rollback for many sequences: cut every listed sequence longer than its keep length
        (uspp_scheduler.cpp:222-237)."""
        s, k = _u32(seq_ids), _u32(keep_lens)
        self._check(self.lib.mla_rollback(self.h, len(s), _np_ptr(s), _np_ptr(k)))

    def truncate(self, seq: int, new_len: int) -> None:
        self._check(self.lib.mla_truncate(self.h, seq, new_len))

    def clear(self, seq: int) -> None:
        self._check(self.lib.mla_clear(self.h, seq))

    def seq_set_base(self, seq: int, base_pos: int) -> None:
        self._check(self.lib.mla_seq_set_base(self.h, seq, base_pos))

    def free_pages(self) -> int:
        v = C.c_uint32()
        self._check(self.lib.mla_free_pages(self.h, C.byref(v)))
        return v.value

    def shuffle_free_pages(self, seed: int) -> None:
        self._check(self.lib.mla_shuffle_free_pages(self.h, seed))

    def seq_pages(self, seq: int) -> np.ndarray:
        n = C.c_uint32()
        self._check(self.lib.mla_seq_pages(self.h, seq, None, 0, C.byref(n)))
        out = np.empty(n.value, np.uint32)
        self._check(self.lib.mla_seq_pages(self.h, seq, _np_ptr(out), n.value, C.byref(n)))
        return out

    # ---- explicit-position calls ------------------------------------------------------
    def append_rows(self, layer: int, seq_ids, positions, kv_a) -> None:
        s, p = _u32(seq_ids), _u32(positions)
        self._check(self.lib.mla_append_rows(self.h, layer, len(s), _np_ptr(s), _np_ptr(p), self._dev(kv_a),
                                             self._stream()))

    def attend_rows(self, layer: int, seq_ids, attend_lens, q, out) -> None:
        s, a = _u32(seq_ids), _u32(attend_lens)
        self._check(self.lib.mla_attend_rows(self.h, layer, len(s), _np_ptr(s), _np_ptr(a), self._dev(q),
                                             self._dev(out), self._stream()))

    # ---- decode-step scheduler --------------------------------------------------------
    def step_begin(self, seq_ids, n_new=None) -> None:
        s = _u32(seq_ids)
        nn = _u32(n_new) if n_new is not None else None
        self._check(self.lib.mla_step_begin(self.h, len(s), _np_ptr(s), _np_ptr(nn) if nn is not None else None,
                                            self._stream()))

    def step_append(self, layer: int, kv_a) -> None:
        self._check(self.lib.mla_step_append(self.h, layer, self._dev(kv_a), self._stream()))

    def step_attend(self, layer: int, q, out) -> None:
        self._check(self.lib.mla_step_attend(self.h, layer, self._dev(q), self._dev(out), self._stream()))

    def step_layers(self, layer_begin: int, n_layers: int, kv_a, q, out) -> None:
        """append + attend for consecutive layers in one call; tensors are [n_layers][rows]..."""
        self._check(self.lib.mla_step_layers(self.h, layer_begin, n_layers, self._dev(kv_a), self._dev(q),
                                             self._dev(out), self._stream()))

    def step_layer_host(self, layer: int, kv_a_host, q_host, out_host) -> None:
        """kv_a_host / q_host / out_host: host torch tensors or numpy arrays (contiguous)."""
        def hp(x):
            return C.c_void_p(x.ctypes.data if isinstance(x, np.ndarray) else x.data_ptr())
        self._check(self.lib.mla_step_layer_host(self.h, layer, hp(kv_a_host), hp(q_host), hp(out_host),
                                                 self._stream()))

    def step_end(self) -> None:
        self._check(self.lib.mla_step_end(self.h))

    def step_info(self) -> tuple[int, int]:
        r, g = C.c_uint32(), C.c_uint32()
        self._check(self.lib.mla_step_info(self.h, C.byref(r), C.byref(g)))
        return r.value, g.value

    def step_attend_partial(self, layer: int, q, partial) -> None:
        self._check(self.lib.mla_step_attend_partial(self.h, layer, self._dev(q), self._dev(partial),
                                                     self._stream()))

    def step_layer_partial(self, layer: int, kv_a, q, partial) -> None:
        """Append (kv_a may be None on a GPU whose shard takes no new row) and partial attend in one call."""
        self._check(self.lib.mla_step_layer_partial(self.h, layer, self._dev(kv_a) if kv_a is not None else None,
                                                    self._dev(q), self._dev(partial), self._stream()))

    def merge_partials(self, layer: int, n_parts: int, rows: int, partials, out) -> None:
        self._check(self.lib.mla_merge_partials(self.h, layer, n_parts, rows, self._dev(partials),
                                                self._dev(out), self._stream()))

    # ---- introspection ----------------------------------------------------------------
    def status(self) -> int:
        """Device status word (0 = clean); raises MlaError when a kernel flagged a fault."""
        v = C.c_uint32()
        self._check(self.lib.mla_status(self.h, self._stream(), C.byref(v)))
        return v.value

    def launch_count(self) -> int:
        v = C.c_uint64()
        self._check(self.lib.mla_launch_count(self.h, C.byref(v)))
        return v.value

    def set_q_rope(self, in_kernel: bool) -> None:
        """True: q is passed before its RoPE and the absorb kernel rotates it with the row's position."""
        self._check(self.lib.mla_set_q_rope(self.h, int(in_kernel)))

    def profile_enable(self, on) -> None:
        """False/0: off; True/1: time every attention launch; N > 1: every N-th launch."""
        self._check(self.lib.mla_profile_enable(self.h, int(on)))

    def profile_read(self) -> tuple[int, float]:
        """(launches, summed milliseconds) of the attention kernel since the last read."""
        n, ms = C.c_uint32(), C.c_float()
        self._check(self.lib.mla_profile_read(self.h, C.byref(n), C.byref(ms)))
        return n.value, ms.value

    def kernel_name(self) -> str:
        return self.lib.mla_kernel_name(self.h).decode()

    def step_balance(self) -> tuple[int, int, int]:
        """(workers, fewest pages, most pages) of the last planned step."""
        w, lo, hi = C.c_uint32(), C.c_uint32(), C.c_uint32()
        self._check(self.lib.mla_step_balance(self.h, C.byref(w), C.byref(lo), C.byref(hi)))
        return w.value, lo.value, hi.value

    def selftest_wait_timeout(self, limit_cycles: int = 1_000_000) -> int:
        """Runs the bounded-wait self-test; returns the SM cycles the block waited before giving up."""
        waited = C.c_uint32()
        self._check(self.lib.mla_selftest_wait_timeout(self.h, limit_cycles, self._stream(), C.byref(waited)))
        return waited.value

    def read_rows(self, layer: int, seq: int, row_begin: int, n: int) -> np.ndarray:
        out = np.empty((n, ROW), np.uint16)
        self._check(self.lib.mla_read_rows(self.h, layer, seq, row_begin, n, _np_ptr(out), self._stream()))
        return out

    def write_rows(self, layer: int, seq: int, row_begin: int, rows_dev) -> None:
        n = rows_dev.shape[0]
        self._check(self.lib.mla_write_rows(self.h, layer, seq, row_begin, n, self._dev(rows_dev),
                                            self._stream()))
