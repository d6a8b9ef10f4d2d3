"""Residency planner: known answers of the reference's tests/weight_residency.c and a seeded
sweep against the reference's src/weights/residency.c compiled as-is (oracle/_ref)."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle
from h3cli_b200 import api
from h3cli_b200.api import WeightOptions, WeightPlan

AUTO, RESIDENT, STREAM = 0, 1, 2
FIELDS = [n for n, _ in WeightPlan._fields_ if n != "options"]


def build(lib, options, mask, block, available, live, future, reserve):
    plan, err = WeightPlan(), C.create_string_buffer(256)
    ok = lib.h3_weight_plan_build(C.byref(plan), options, mask, block, available, live, future, reserve, err, 256)
    return ok, plan, err.value.decode()


def opts(mode=AUTO, cap=-1, capacity=0, allocation=0):
    return WeightOptions(mode, cap, capacity, allocation)


def test_known_answers():
    lib = api.library()
    mask = (1 << 3) - 1
    ok, p, _ = build(lib, opts(), mask, 100, 400, 900, 40, 60)
    assert ok and p.resident_mask == mask and p.resident_bytes == 300 and p.effective_mode == RESIDENT and p.slot_bytes == 0
    ok, p, _ = build(lib, opts(), mask, 100, 399, 0, 40, 60)  # one byte short: two slots, 0 resident
    assert ok and p.slot_bytes == 200 and p.resident_count == 0 and p.effective_mode == STREAM
    ok, p, _ = build(lib, opts(), (1 << 10) - 1, 100, 700, 0, 50, 50)  # budget 600: slots 200 + 4 blocks
    assert ok and p.resident_count == 4 and p.resident_mask == 0xF and p.effective_mode == AUTO
    ok, p, _ = build(lib, opts(cap=2), (1 << 10) - 1, 100, 5000, 0, 0, 0)
    assert ok and p.resident_count == 2 and p.slot_bytes == 200
    ok, p, _ = build(lib, opts(mode=STREAM), mask, 100, 5000, 0, 0, 0)
    assert ok and p.resident_count == 0 and p.effective_mode == STREAM
    ok, _, why = build(lib, opts(mode=RESIDENT), mask, 100, 299, 0, 0, 0)
    assert not ok and "resident weights need more capacity" in why
    ok, _, why = build(lib, opts(), mask, 100, 199, 0, 0, 0)
    assert not ok and "two-slot streaming" in why
    ok, _, why = build(lib, opts(), 1 << 50, 100, 199, 0, 0, 0)
    assert not ok and "invalid weight planner input" in why
    ok, _, why = build(lib, opts(), mask, 1 << 63, 1 << 62, 0, 0, 0)
    assert not ok and "overflow" in why
    ok, p, _ = build(lib, opts(capacity=1000), mask, 100, 5000, 900, 0, 0)  # capacity covers live bytes
    assert not ok or p.free_bytes == 100


def test_retry_cap_reaches_zero():
    lib = api.library()
    cap, steps = 50, 0
    while cap > 0:
        cap = lib.h3_weight_retry_cap(cap)
        steps += 1
    assert cap == 0 and steps <= 7
    assert lib.h3_weight_retry_cap(0) == -1
    assert [lib.h3_weight_mode_name(m) for m in (0, 1, 2)] == [b"auto", b"resident", b"stream"]


def reference_library():
    oracle.build()
    path = os.path.join(os.path.dirname(oracle.__file__), "_ref", "libh3_residency_ref.so")
    if not os.path.exists(path):
        pytest.skip("reference residency.c was not compiled on this machine")
    ref = C.CDLL(path)
    u64 = C.c_uint64
    ref.h3_weight_plan_build.restype = C.c_int
    ref.h3_weight_plan_build.argtypes = [C.POINTER(WeightPlan), WeightOptions, u64, u64, u64, u64, u64, u64, C.c_char_p, C.c_size_t]
    ref.h3_weight_retry_cap.restype = C.c_int
    ref.h3_weight_retry_cap.argtypes = [C.c_uint]
    ref.h3_weight_options_read.restype = C.c_int
    ref.h3_weight_options_read.argtypes = [C.POINTER(WeightOptions), C.c_int, C.c_char_p, C.c_size_t]
    return ref


def test_sweep_against_reference():
    ref, lib = reference_library(), api.library()
    rng = np.random.default_rng(7)
    accepted = 0
    for _ in range(20000):
        bits = int(rng.integers(1, 51))
        mask = int(rng.integers(0, 1 << bits)) if rng.random() < 0.9 else int(rng.integers(0, 1 << 52))
        block = int(rng.integers(0, 400)) if rng.random() < 0.95 else int(rng.integers(1 << 60, 1 << 63))
        available = int(rng.integers(0, 30000))
        live, future, reserve = (int(rng.integers(0, 3000)) for _ in range(3))
        if rng.random() < 0.02:
            future = (1 << 64) - 1 - int(rng.integers(0, 100))
        o = opts(int(rng.integers(-1, 4)), int(rng.integers(-2, 53)) if rng.random() < 0.5 else -1,
                 int(rng.integers(0, 20000)) if rng.random() < 0.3 else 0, int(rng.integers(0, 5)))
        a_ok, a, a_why = build(lib, o, mask, block, available, live, future, reserve)
        b_ok, b, b_why = build(ref, o, mask, block, available, live, future, reserve)
        assert a_ok == b_ok and a_why == b_why, (mask, block, available, live, future, reserve, a_why, b_why)
        if a_ok:
            accepted += 1
            assert all(getattr(a, f) == getattr(b, f) for f in FIELDS), [(f, getattr(a, f), getattr(b, f)) for f in FIELDS]
    assert accepted > 5000
    for count in range(0, 60):
        assert lib.h3_weight_retry_cap(count) == ref.h3_weight_retry_cap(count)


def test_options_from_environment(monkeypatch):
    ref, lib = reference_library(), api.library()
    cases = [({}, 0), ({"H3_CUDA_WEIGHT_MODE": "stream"}, 0), ({"H3_CUDA_WEIGHT_MODE": "resident"}, 1),
             ({"H3_CUDA_WEIGHT_MODE": "auto"}, 1), ({"H3_CUDA_WEIGHT_MODE": "bogus"}, 0),
             ({"H3_TEST_CUDA_RESIDENT_BLOCKS": "7"}, 0), ({"H3_TEST_CUDA_RESIDENT_BLOCKS": "51"}, 0),
             ({"H3_TEST_CUDA_RESIDENT_BLOCKS": "-1"}, 0), ({"H3_TEST_CUDA_CAPACITY_BYTES": "123456789012"}, 0),
             ({"H3_CUDA_TEST_MEMORY_BUDGET": "99x"}, 0), ({"H3_CUDA_TEST_MEMORY_BUDGET": "4096"}, 1)]
    names = ["H3_CUDA_WEIGHT_MODE", "H3_TEST_CUDA_RESIDENT_BLOCKS", "H3_TEST_CUDA_CAPACITY_BYTES", "H3_CUDA_TEST_MEMORY_BUDGET"]
    for env, force in cases:
        for n in names:
            monkeypatch.delenv(n, raising=False)
        for k, v in env.items():
            monkeypatch.setenv(k, v)
        results = []
        for l in (lib, ref):
            o, err = WeightOptions(), C.create_string_buffer(256)
            ok = l.h3_weight_options_read(C.byref(o), force, err, 256)
            results.append((ok, err.value, (o.mode, o.max_resident, o.capacity_limit, o.allocation_limit) if ok else None))
        assert results[0] == results[1], (env, force, results)
