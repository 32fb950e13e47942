"""CPU-side checks of the C-ABI library: it builds, loads, exports every declared symbol, and
refuses to run without a GPU (no compute call is made here)."""
import ctypes as C
import os
import re
import subprocess

import pytest

from mugen_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "mugen_mla.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mla_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    names = _declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/mugen_mla.h but not exported"
    assert sorted(capi.SIGNATURES) == names, "ctypes binding and header disagree"


def test_exported_symbols_are_dynamic():
    out = subprocess.run(["nm", "-D", "--defined-only", capi.lib_path()], capture_output=True, text=True,
                         check=True).stdout
    for n in _declared_symbols():
        assert re.search(rf"\bT {n}\b", out), n


def test_create_validates_like_the_reference_cache():
    """Same messages as KVCache::create (src/core/memory/kv_cache.cpp:146-159)."""
    lib = capi.load()
    h = C.c_void_p()
    cfg = capi.MlaConfig(0, 16, 512, 128, 64, 128, 1e4, 1e-6, 40.0, 4096, 128, 64, 8, 2, 0, 0, 0, 0, 0)
    assert lib.mla_create(C.byref(cfg), C.byref(h)) == 1
    assert lib.mla_last_error(None) == b"n_layers must be > 0"
    cfg.n_layers, cfg.max_seq_len = 1, 0
    assert lib.mla_create(C.byref(cfg), C.byref(h)) == 1
    assert lib.mla_last_error(None) == b"max_seq_len must be > 0"
    cfg.max_seq_len, cfg.kv_lora_rank = 128, 256
    assert lib.mla_create(C.byref(cfg), C.byref(h)) == 7


def test_no_cpu_fallback():
    """Without a CUDA device the library must refuse, not compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = capi.load()
    h = C.c_void_p()
    cfg = capi.MlaConfig(1, 16, 512, 128, 64, 128, 1e4, 1e-6, 40.0, 4096, 128, 64, 8, 2, 0, 0, 0, 0, 0)
    rc = lib.mla_create(C.byref(cfg), C.byref(h))
    assert rc == 2 and b"no CUDA device" in lib.mla_last_error(None)
    assert not h.value
