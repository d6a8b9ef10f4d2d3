"""The C-ABI library without a GPU: it loads, exports every function that
include/h3q8.h declares (in the spirit of h3cli's tests/test_gpu_contract.c and
tests/check_gpu_contract.py), its host packer reproduces the reference's golden
vectors, and the GPU operators refuse to run instead of falling back."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def lib():
    from h3cli_b200 import build
    build.build()
    import h3cli_b200
    return h3cli_b200.library()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "h3q8.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"typedef\s+(struct|enum)\s*\{.*?\}\s*\w+\s*;", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(h3q?8?_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_functions()
    assert len(names) >= 60
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/h3q8.h but not exported"
        assert name in lib._signatures, f"{name} has no ctypes signature in h3cli_b200/api.py"
    assert set(lib._signatures) <= set(names), "the binding names a function the header does not declare"


def test_host_packer_known_answers(lib):
    # tests/metal_q8.c:21-34 through the library's own h3_q8_* symbols
    g = np.load(os.path.join(GOLDEN, "q8_pack.npz"))
    src = np.ascontiguousarray(g["known_src"])
    q = np.empty((1, 65), np.int8)
    s = np.empty((1, 2), np.float32)
    assert lib.h3_q8_pack_rows(src.ctypes.data, q.ctypes.data, s.ctypes.data, 1, 65)
    assert q[0, :8].tolist() == [127, -127, 0, 2, 2, 0, -2, -2] and (s == 1).all() and q[0, 64] == 0
    off, total = ctypes.c_size_t(), ctypes.c_size_t()
    assert lib.h3_q8_layout(1, 65, ctypes.byref(off), ctypes.byref(total)) and (off.value, total.value) == (68, 76)
    assert not lib.h3_q8_layout(0, 65, ctypes.byref(off), ctypes.byref(total))
    assert not lib.h3_q8_layout(0xFFFFFFFF, 0xFFFFFFFF, ctypes.byref(off), ctypes.byref(total))
    assert not lib.h3_q8_layout(1, 0xFFFFFFFF - 31, ctypes.byref(off), ctypes.byref(total))
    for bad in (0x7FC0, 0x7F80):
        src[0, 64] = bad
        assert not lib.h3_q8_pack_rows(src.ctypes.data, q.ctypes.data, s.ctypes.data, 1, 65)
    src[0, 64] = 1
    assert lib.h3_q8_pack_rows(src.ctypes.data, q.ctypes.data, s.ctypes.data, 1, 65) and np.isfinite(s).all()


def test_host_packer_matches_reference_fixtures(lib, oracle):
    g = np.load(os.path.join(GOLDEN, "q8_pack.npz"))
    for i in range(4):
        src = np.ascontiguousarray(g[f"src{i}"])
        rows, cols = src.shape
        q = np.empty((rows, cols), np.int8)
        s = np.empty(g[f"s{i}"].shape, np.float32)
        assert lib.h3_q8_pack_rows(src.ctypes.data, q.ctypes.data, s.ctypes.data, rows, cols)
        assert (q == g[f"q{i}"]).all() and (s.view(np.uint32) == g[f"s{i}"].view(np.uint32)).all()
    rng = np.random.default_rng(3)
    w = oracle.f32_to_bf16(rng.standard_normal((12, 400)).astype(np.float32)).reshape(12, 400)
    for group in (0, 64, 128):
        want_q, want_s = oracle.q8_pack_rows(w, group)
        q = np.empty_like(want_q)
        s = np.empty_like(want_s)
        assert lib.h3q8_q8_pack_rows(w.ctypes.data, q.ctypes.data, s.ctypes.data, 12, 400, group)
        assert (q == want_q).all() and (s.view(np.uint32) == want_s.view(np.uint32)).all()


def test_no_cpu_fallback(lib):
    import h3cli_b200
    buf = ctypes.create_string_buffer(256)
    handle = lib.h3_gpu_create(b"", buf, len(buf))
    if handle:  # a GPU is present: nothing to refuse
        lib.h3_gpu_free(handle)
        pytest.skip("a CUDA device is present")
    assert b"no CPU path" in buf.value or b"sm_100a" in buf.value
    with pytest.raises(h3cli_b200.H3Error):
        h3cli_b200.Gpu()
    d = h3cli_b200.LinearDesc(mode=1, rows=4, input_dim=16, output_dim=8)
    assert lib.h3q8_linear(ctypes.byref(d), None) == 0 and lib.h3q8_last_error()
