"""Builds tests/host/test_host.cpp (C++23, g++) against libmugen_mla.so and runs it: page table and
planner units and the rotary table against the CPU checker here; one decode run through the C++23
wrapper on the GPU."""
import os
import subprocess

import numpy as np
import pytest

from mugen_b200 import capi, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "host", "test_host")


@pytest.fixture(scope="module")
def exe():
    capi.load()
    src = os.path.join(ROOT, "tests", "host", "test_host.cpp")
    libdir = os.path.dirname(capi.lib_path())
    subprocess.run(["g++", "-std=c++23", "-O1", "-ffp-contract=off", "-Wall", "-o", EXE, src, f"-L{libdir}",
                    "-l:libmugen_mla.so", f"-Wl,-rpath,{libdir}"], check=True)
    return EXE


def test_host_units(exe):
    out = subprocess.run([exe, "units"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert "host units ok" in out.stdout


def test_host_units_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """The CPU-only host logic (page table, free list, split-KV planner, rotary table) once more, compiled
    with -fsanitize=address,undefined: an out-of-bounds table access, a use after free in the page
    bookkeeping or a signed overflow in the planner's arithmetic would abort the run."""
    capi.load()
    src = os.path.join(ROOT, "tests", "host", "test_host.cpp")
    libdir = os.path.dirname(capi.lib_path())
    exe_san = str(tmp_path / "test_host_san")
    subprocess.run(["g++", "-std=c++23", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
                    "-fno-omit-frame-pointer", "-ffp-contract=off", "-Wall", "-o", exe_san, src, f"-L{libdir}",
                    "-l:libmugen_mla.so", f"-Wl,-rpath,{libdir}"], check=True)
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    out = subprocess.run([exe_san, "units"], capture_output=True, text=True, env=env)
    assert out.returncode == 0, out.stderr[-3000:]
    assert "host units ok" in out.stdout
    out = subprocess.run([exe_san, "rope", "40.0", "4096", "10000.0", "0", "63", "64", "131071"], capture_output=True,
                         text=True, env=env)
    assert out.returncode == 0 and len(out.stdout.strip().splitlines()) == 4, out.stderr[-3000:]


@pytest.mark.parametrize("factor,ctx,theta", [(40.0, 4096, 10000.0), (0.0, 0, 10000.0), (4.0, 32768, 1e6)])
def test_rope_table_matches_checker_bit_for_bit(exe, oracle, factor, ctx, theta):
    """The library's host-built cos/sin rows (what the append kernel consumes) equal the values the
    reference arithmetic produces, for small, page-boundary and very large positions."""
    positions = [0, 1, 2, 63, 64, 4095, 4096, 8191, 16383, 65535, 131071]
    out = subprocess.run([exe, "rope", str(factor), str(ctx), repr(theta), *map(str, positions)],
                         capture_output=True, text=True, check=True).stdout.strip().splitlines()
    assert len(out) == len(positions)
    for line, pos in zip(out, positions):
        got = np.array([int(x, 16) for x in line.split()], np.uint32)
        c, s = oracle.rope_cos_sin(pos, factor, ctx, theta)
        assert np.array_equal(got[:32], c.view(np.uint32)) and np.array_equal(got[32:], s.view(np.uint32)), pos


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [synth.DT_F16, synth.DT_BF16])
def test_cpp_wrapper_decodes_like_the_checker(exe, oracle, tmp_path, dt):
    H, L, B, T = 16, 2, 3, 5
    rng = np.random.default_rng(17)
    case = [synth.make_layer_case(900 + l, H, [1], dt) for l in range(L)]
    blobs = [np.array([H, L, B, T, int(dt == synth.DT_BF16)], np.uint32).tobytes()]
    for l in range(L):
        blobs += [case[l].w_uk.tobytes(), case[l].w_uv.tobytes(), case[l].norm_w.tobytes()]
    kv = synth.to_bits(rng.standard_normal((T, L, B, 576), np.float32), dt)
    q = synth.to_bits(rng.standard_normal((T, L, B, H, 192), np.float32) * np.float32(0.9), dt)
    for t in range(T):
        for l in range(L):
            blobs += [kv[t, l].tobytes(), q[t, l].tobytes()]
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    fin.write_bytes(b"".join(blobs))
    r = subprocess.run([exe, "decode", str(fin), str(fout)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = np.frombuffer(fout.read_bytes(), np.uint16).reshape(T, L, B, H, 128)
    caches = [[np.zeros((0, 576), np.uint16) for _ in range(B)] for _ in range(L)]
    for t in range(T):
        for l in range(L):
            rows = oracle.append_rows(kv[t, l], [t] * B, case[l].norm_w, 1e-6, 40.0, 4096, 10000.0, dt)
            for b in range(B):
                caches[l][b] = np.concatenate([caches[l][b], rows[b:b + 1]])
                want = oracle.attention(q[t, l, b], caches[l][b], t + 1, case[l].w_uk, case[l].w_uv,
                                        case[l].w_type, H, dt)
                mx, rl = synth.error_norms(got[t, l, b], want, dt, dt)
                assert mx <= 2e-2 and rl <= 5e-3, (t, l, b, mx, rl)
