"""CPU checks that pin the oracle (oracle/h3q8_oracle.c) before it is trusted:
the reference's golden vectors, the reference's own packer compiled as-is, and
the committed fixtures.  Mirrors the host half of h3cli's tests/metal_q8.c."""
import ctypes
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_bf16_round_to_nearest_even(oracle):
    # src/metal/shaders.metal:15-19
    cases = {1.0: 0x3F80, 1.00390625: 0x3F80, 1.01171875: 0x3F82, -2.5: 0xC020, 0.0: 0, 3.3895313892515355e38: 0x7F7F}
    for value, bits in cases.items():
        assert oracle.lib().h3o_f32_to_bf16(value) == bits
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    bits = oracle.f32_to_bf16(x)
    assert all(oracle.lib().h3o_f32_to_bf16(float(v)) == b for v, b in zip(x[:256], bits[:256]))
    assert (oracle.f32_to_bf16(oracle.bf16_to_f32(bits)) == bits).all()


def test_packer_known_answers(oracle):
    # tests/metal_q8.c:21-34
    values = np.zeros((1, 65), np.float32)
    values[0, :8] = [127, -127, .5, 1.5, 2.5, -.5, -1.5, -2.5]
    src = oracle.f32_to_bf16(values).reshape(1, 65)
    q, s = oracle.q8_pack_rows(src, 64)
    assert q[0, :8].tolist() == [127, -127, 0, 2, 2, 0, -2, -2]
    assert (s == 1.0).all() and q[0, 64] == 0
    assert oracle.q8_layout(1, 65, 64) == (68, 76)
    assert oracle.q8_layout(0, 65, 64) is None
    assert oracle.q8_layout(0xFFFFFFFF, 0xFFFFFFFF, 64) is None
    assert oracle.q8_layout(1, 0xFFFFFFFF - 31, 64) is None
    for bad in (0x7FC0, 0x7F80):  # NaN, Inf
        src[0, 64] = bad
        assert oracle.q8_pack_rows(src, 64) is None
    src[0, 64] = 1  # subnormal accepted, scale stays finite and normal
    q, s = oracle.q8_pack_rows(src, 64)
    assert np.isfinite(s).all() and s[0, 1] >= np.finfo(np.float32).tiny


def test_packer_matches_reference_build(oracle):
    ref = oracle.reference_q8()
    if ref is None:
        pytest.skip("oracle/_ref was not built (no reference tree); the committed fixtures cover this")
    rng = np.random.default_rng(5)
    for rows, cols in [(1, 1), (3, 63), (17, 65), (67, 129), (33, 256), (8, 1000)]:
        w = oracle.f32_to_bf16((rng.standard_normal((rows, cols)) * 0.125).astype(np.float32)).reshape(rows, cols)
        w[0, 0] = 0
        if cols > 64:
            w[rows - 1, :64] = 0  # an all-zero group: scale 1
        q, s = oracle.q8_pack_rows(w, 64)
        q2 = np.empty_like(q)
        s2 = np.empty_like(s)
        assert ref.h3_q8_pack_rows(w.ctypes.data, q2.ctypes.data, s2.ctypes.data, rows, cols)
        assert (q == q2).all() and (s.view(np.uint32) == s2.view(np.uint32)).all()
        off, total = ctypes.c_size_t(), ctypes.c_size_t()
        assert ref.h3_q8_layout(rows, cols, ctypes.byref(off), ctypes.byref(total))
        assert oracle.q8_layout(rows, cols, 64) == (off.value, total.value)


def test_packer_matches_committed_fixtures(oracle):
    g = np.load(os.path.join(GOLDEN, "q8_pack.npz"))
    q, s = oracle.q8_pack_rows(g["known_src"], 64)
    assert (q == g["known_q"]).all() and (s == g["known_s"]).all()
    for i in range(4):
        q, s = oracle.q8_pack_rows(g[f"src{i}"], 64)
        assert (q == g[f"q{i}"]).all()
        assert (s.view(np.uint32) == g[f"s{i}"].view(np.uint32)).all()


def test_group_parameter(oracle):
    rng = np.random.default_rng(6)
    w = oracle.f32_to_bf16(rng.standard_normal((9, 384)).astype(np.float32)).reshape(9, 384)
    for group, groups in [(0, 1), (64, 6), (128, 3), (256, 2)]:
        q, s = oracle.q8_pack_rows(w, group)
        assert s.shape == (9, groups)
        width = group or 384
        wf = oracle.bf16_to_f32(w).reshape(9, 384)
        for g in range(groups):
            peak = np.abs(wf[:, g * width:(g + 1) * width]).max(axis=1)
            assert np.array_equal(s[:, g], np.maximum(peak / np.float32(127.0), np.finfo(np.float32).tiny).astype(np.float32))
        assert np.abs(q).max() <= 127
        deq = oracle.bf16_to_f32(oracle.q8_dequant(q, s, group)).reshape(9, 384)
        assert np.abs(deq - wf).max() <= s.max() * 0.51 + np.abs(wf).max() * 2 ** -8


def test_row_quantiser(oracle):
    # src/metal/shaders.metal:1391-1460
    rng = np.random.default_rng(7)
    x = rng.standard_normal((6, 130)).astype(np.float32)
    x[1] = 0.0
    x[2, 5] *= 20
    xb = oracle.f32_to_bf16(x).reshape(6, 130)
    q, s = oracle.quantize_rows(xb, dispatch_rows=8)
    xf = oracle.bf16_to_f32(xb).reshape(6, 130)
    peak = np.abs(xf).max(axis=1)
    assert s[1] == np.float32(1.0) / np.float32(127.0) and (q[1] == 0).all()     # zero row
    assert (s[6:] == 1.0).all() and (q[6:] == 0).all()                           # padding rows
    live = [0, 2, 3, 4, 5]
    assert np.array_equal(s[live], (peak[live] / np.float32(127.0)).astype(np.float32))
    inverse = (np.float32(127.0) / peak[live]).astype(np.float32)
    expect = np.clip(np.rint((xf[live] * inverse[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    assert (q[live] == expect).all()
    assert np.abs(q[live]).max(axis=1).tolist() == [127] * 5
    # ties go to even: x = 2.5 * max/127 ... use exact powers of two
    t = np.array([[127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 63.5]], np.float32)
    q, s = oracle.quantize_rows(oracle.f32_to_bf16(t).reshape(1, 8))
    assert s[0] == 1.0 and q[0].tolist() == [127, 0, 2, 2, 0, -2, -2, 64]


def test_epilogue_operators(oracle):
    lib = oracle.lib()
    # src/cuda/cuda_kernels.cuh:883-893: saturation guards and the tanh branch
    for v in (-40.0, -12.0, 12.0, 40.0, 0.0, 1.0, -1.0, 3.0):
        b = int(oracle.f32_to_bf16(np.float32(v))[()] if np.ndim(oracle.f32_to_bf16(np.float32(v))) == 0 else oracle.f32_to_bf16(np.array([v], np.float32))[0])
        got = oracle.bf16_to_f32(np.array([lib.h3o_gelu_tanh_bf16(b)], np.uint16))[0]
        x = oracle.bf16_to_f32(np.array([b], np.uint16))[0].astype(np.float64)
        want = 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
        assert abs(got - want) <= abs(want) * 2 ** -8 + 1e-30
    # src/cuda/cuda_kernels.cuh:979-984
    r, b, g = (int(oracle.f32_to_bf16(np.array([v], np.float32))[0]) for v in (0.75, -1.5, 1.125))
    got = oracle.bf16_to_f32(np.array([lib.h3o_gate_residual_bf16(r, b, g)], np.uint16))[0]
    assert got == oracle.bf16_to_f32(oracle.f32_to_bf16(np.array([0.75 + (-1.5 * 1.125)], np.float32)))[0]


def test_linear_fixture_and_fast_path(oracle):
    pack = np.load(os.path.join(GOLDEN, "q8_pack.npz"))
    lin = np.load(os.path.join(GOLDEN, "linear.npz"))
    for i in range(4):
        out = oracle.linear(oracle.MODE_W8A16, lin[f"x{i}"], pack[f"q{i}"], pack[f"s{i}"], 64, bias=lin[f"bias{i}"])
        assert (out == lin[f"out{i}"]).all()
        fast = oracle.linear(oracle.MODE_W8A16, lin[f"x{i}"], pack[f"q{i}"], pack[f"s{i}"], 64, bias=lin[f"bias{i}"], fast=True)
        a, e = oracle.bf16_to_f32(fast).astype(np.float64), oracle.bf16_to_f32(out).astype(np.float64)
        assert np.sqrt(((a - e) ** 2).sum() / max((e ** 2).sum(), 1e-30)) < 2e-3


def test_w8a8_fixture(oracle):
    g = np.load(os.path.join(GOLDEN, "w8a8.npz"))
    for i in range(3):
        xq, xs = oracle.quantize_rows(g[f"x{i}"])
        assert (xq == g[f"xq{i}"]).all() and (xs.view(np.uint32) == g[f"xs{i}"].view(np.uint32)).all()
        for fast in (False, True):
            out, acc = oracle.linear(oracle.MODE_W8A8, xq, g[f"wq{i}"], g[f"ws{i}"], 0, x_scales=xs, want_acc=True, fast=fast)
            assert (acc == g[f"acc{i}"]).all() and (out == g[f"out{i}"]).all()
        # epilogue order: (float(acc) * in_scale) * w_scale, src/metal/shaders.metal:2463-2464
        want = (g[f"acc{i}"].astype(np.float32) * xs[:, None]).astype(np.float32) * g[f"ws{i}"][None, :]
        assert (oracle.f32_to_bf16(want.astype(np.float32)).reshape(out.shape) == out).all()


def test_w8a8_grouped_combine_order(oracle):
    rng = np.random.default_rng(9)
    xq = rng.integers(-127, 128, (7, 512)).astype(np.int8)
    wq = rng.integers(-127, 128, (5, 512)).astype(np.int8)
    xs = rng.uniform(0.01, 0.05, 7).astype(np.float32)
    ws = rng.uniform(0.005, 0.02, (5, 4)).astype(np.float32)
    out = oracle.linear(oracle.MODE_W8A8, xq, wq, ws, 128, x_scales=xs)
    total = None
    for gidx in range(4):  # src/metal/shaders.metal:2727-2735: first group assigns, later groups add, in order
        acc = xq[:, gidx * 128:(gidx + 1) * 128].astype(np.int32) @ wq[:, gidx * 128:(gidx + 1) * 128].astype(np.int32).T
        value = ((acc.astype(np.float32) * xs[:, None]).astype(np.float32) * ws[None, :, gidx]).astype(np.float32)
        total = value if total is None else (total + value).astype(np.float32)
    assert (oracle.f32_to_bf16(total).reshape(7, 5) == out).all()
    assert (oracle.linear(oracle.MODE_W8A8, xq, wq, ws, 128, x_scales=xs, fast=True) == out).all()


def test_w8a8_activation_group_scales(oracle):
    """Per-row, per-1024-K-group activation scales of the reference's FC2 path
    (quantiser src/metal/shaders.metal:1552-1598, GEMM :2663-2742)."""
    rng = np.random.default_rng(10)
    x = oracle.f32_to_bf16(rng.standard_normal((5, 2048)).astype(np.float32)).reshape(5, 2048)
    x[3, :1024] = 0
    xq, xs = oracle.quantize_rows_grouped(x, 1024, dispatch_rows=6)
    assert xs.shape == (6, 2) and (xs[5] == 1.0).all() and (xq[5] == 0).all()
    assert xs[3, 0] == np.float32(1.0) / np.float32(127.0) and (xq[3, :1024] == 0).all()
    for g in range(2):
        q, s = oracle.quantize_rows(np.ascontiguousarray(x[:, g * 1024:(g + 1) * 1024]))
        assert (q == xq[:5, g * 1024:(g + 1) * 1024]).all() and (s == xs[:5, g]).all()
    wq = rng.integers(-127, 128, (7, 2048)).astype(np.int8)
    ws = rng.uniform(0.005, 0.02, 7).astype(np.float32)
    out = oracle.linear(oracle.MODE_W8A8, xq[:5], wq, ws, 0, x_scales=xs[:5], input_group=1024)
    total = None
    for g in range(2):
        acc = xq[:5, g * 1024:(g + 1) * 1024].astype(np.int32) @ wq[:, g * 1024:(g + 1) * 1024].astype(np.int32).T
        value = ((acc.astype(np.float32) * xs[:5, g:g + 1]).astype(np.float32) * ws[None, :]).astype(np.float32)
        total = value if total is None else (total + value).astype(np.float32)
    assert (oracle.f32_to_bf16(total).reshape(5, 7) == out).all()
    assert (oracle.linear(oracle.MODE_W8A8, xq[:5], wq, ws, 0, x_scales=xs[:5], input_group=1024, fast=True) == out).all()


def test_restatement_against_reference_cuda_kernel_outputs(oracle):
    """tests/golden/reference_kernels.npz holds outputs of the reference's OWN CUDA element kernels
    (src/cuda/cuda_kernels.cuh compiled unmodified, run on a B200 by tests/golden/make_reference_kernel_golden.py).
    The CPU restatement is held to them here with the bounds the GPU tests use beside the live kernels: gate, add-style
    IEEE steps and the v stream bit for bit; tanhf / expf / rsqrtf results within one bf16 step (a CPU's libm and
    1/sqrt against the GPU's)."""
    g = np.load(os.path.join(GOLDEN, "reference_kernels.npz"))
    f32 = lambda bits: oracle.bf16_to_f32(np.asarray(bits, np.uint16))

    def steps_apart(a, b):
        ordered = lambda bits: np.where(bits.astype(np.int32) & 0x8000, -(bits.astype(np.int32) & 0x7FFF), bits.astype(np.int32))
        return np.abs(ordered(np.asarray(a)) - ordered(np.asarray(b)))

    def within_one_step(a, b, floor):
        x, y = f32(a).astype(np.float64), f32(b).astype(np.float64)
        step = 2.0 ** (np.floor(np.log2(np.maximum(np.maximum(np.abs(x), np.abs(y)), floor))) - 7)
        return bool((np.abs(x - y) <= step).all())

    # GELU-tanh over every bf16 input (src/cuda/cuda_kernels.cuh:879-902)
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    finite = np.isfinite(f32(bits))
    apart = steps_apart(oracle.gelu_tanh_bf16(bits)[finite], g["gelu_out"][finite])
    assert apart.max() <= 1 and (apart != 0).mean() < 2e-3
    # gate * branch + residual (:973-986): separate IEEE multiply and add, bit for bit
    for i in range(2):
        res, branch, mod, row_map = g[f"gate{i}_res"], g[f"gate{i}_branch"], g[f"gate{i}_mod"], g[f"gate{i}_map"]
        product = f32(branch) * f32(mod[row_map, 2, :])
        assert (oracle.f32_to_bf16(f32(res) + product) == g[f"gate{i}_out"]).all()
    # SwiGLU on a stored [rows, 2 * width] tensor (:1047-1059)
    fused = g["swiglu_in"]
    width = fused.shape[1] // 2
    gate, up = f32(fused[:, :width]), f32(fused[:, width:])
    apart = steps_apart(oracle.f32_to_bf16(gate / (np.float32(1) + np.exp(-gate, dtype=np.float32)) * up), g["swiglu_out"])
    assert apart.max() <= 1 and (apart != 0).mean() < 5e-3
    # grouped QKV: per-head RMS norm + rotary embedding (:988-1045)
    for i, (heads, half) in enumerate([(2, 48), (3, 64)]):
        got = oracle.grouped_qkv_rope(g[f"rope{i}_qkv"], g[f"rope{i}_qn"], g[f"rope{i}_kn"], g[f"rope{i}_cos"], g[f"rope{i}_sin"],
                                      heads, 128, half, 1e-5)
        for mine, theirs in zip(got, (g[f"rope{i}_q"], g[f"rope{i}_k"], g[f"rope{i}_v"])):
            assert within_one_step(mine, theirs, 1.0)
        assert (got[2] == g[f"rope{i}_v"]).all()
    # gate -> AdaLN -> per-row int8 (:973-986, 936-971; src/metal/shaders.metal:1434-1459)
    for i in range(3):
        res, branch, mod, norm_w, row_map = (g[f"chain{i}_{k}"] for k in ("res", "branch", "mod", "norm", "map"))
        rows = res.shape[0]
        padded = (rows + 127) // 128 * 128
        o_gated, o_norm, o_q, _ = oracle.gate_adaln_quantize(res, branch, mod, norm_w, mod, row_map, padded, 6, 2, 3, 4, 1e-5)
        assert (o_gated == g[f"chain{i}_gated"]).all()
        assert within_one_step(o_norm, g[f"chain{i}_adaln"], 0.25)
        want_q, _ = oracle.quantize_rows(g[f"chain{i}_adaln"], padded)
        assert np.abs(o_q.astype(np.int32) - want_q.astype(np.int32)).max() <= 1
    # the reference's small bf16 linear (:762-794): fp32 fmaf chain against the FP64-dot restatement
    from parity import check_bf16
    for i in range(3):
        bias = g[f"linear{i}_bias"]
        check_bf16(oracle.linear(oracle.MODE_BF16, g[f"linear{i}_x"], g[f"linear{i}_w"], bias=bias if bias.size else None), g[f"linear{i}_out"])
