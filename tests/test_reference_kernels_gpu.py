"""The reference's OWN CUDA element kernels as the checker (needs a B200).

`oracle/_ref/libh3_cuda_kernels_ref.so` is greg31337/h3cli's src/cuda/cuda_kernels.cuh compiled
unmodified with the reference's nvcc flags (oracle/ref_cuda_kernels.cu, oracle/Makefile).  Each test
runs one reference kernel on the same GPU and the same seeded inputs and compares it with

  * this library's operator for the same step (through the C-ABI), bit for bit wherever both
    sides use the same instructions, and
  * the CPU restatement under oracle/, so that the restatement itself is pinned by reference
    output and not only by a reading of the reference's source.

Where the reference calls rsqrtf / tanhf / expf the GPU and a CPU cannot agree in every last bit
(rsqrtf is the hardware's approximate instruction, the others are different libm implementations);
those comparisons state the measured bound.
"""
import numpy as np
import pytest

import h3cli_b200 as h
from h3cli_b200 import synth
from parity import bf16_to_f32, check_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(oracle):
    kernels = oracle.reference_cuda()
    if kernels is None:
        pytest.skip("oracle/_ref/libh3_cuda_kernels_ref.so was not built (no reference tree at build time)")
    return kernels


def bf(a):
    a = np.asarray(a, np.float32)
    return synth.to_bf16(a).reshape(a.shape)


def within_one_step(a_bits, b_bits, floor):
    """|a - b| <= one bf16 step taken at max(|a|, |b|, floor): for results that are differences of larger terms
    (a rotation, a shifted product) the step of the terms, not of the tiny result, is the honest unit."""
    a, b = bf16_to_f32(a_bits).astype(np.float64), bf16_to_f32(b_bits).astype(np.float64)
    step = 2.0 ** (np.floor(np.log2(np.maximum(np.maximum(np.abs(a), np.abs(b)), floor))) - 7)
    return bool((np.abs(a - b) <= step).all())


def steps_apart(a_bits, b_bits):
    """Distance in bf16 steps between two arrays of finite bf16 bit patterns (sign-magnitude -> ordered ints)."""
    def ordered(bits):
        v = bits.astype(np.int32)
        return np.where(v & 0x8000, -(v & 0x7FFF), v)
    return np.abs(ordered(np.asarray(a_bits)) - ordered(np.asarray(b_bits)))


def test_gelu_tanh_against_the_reference_kernel(gpu, oracle, ref):
    """h3_gelu_bf16 (src/cuda/cuda_kernels.cuh:879-902) over every bf16 input.

    CPU restatement: same formula with glibc's tanhf instead of CUDA's: at most one bf16 step apart, rarely.
    h3_gpu_gelu_bf16 / the fused epilogue: evaluated as v / (1 + exp(-2u)) with the hardware exponential, a
    documented deviation: at most one bf16 step from the reference kernel outside the cancellation region
    (|v| * 2^-23 absolute inside it)."""
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    v = bf16_to_f32(bits).astype(np.float64)
    finite = np.isfinite(v)
    want = ref.gelu(bits, 1)
    restated = oracle.gelu_tanh_bf16(bits)
    apart = steps_apart(restated[finite], want[finite])
    assert apart.max() <= 1 and (apart != 0).mean() < 2e-3
    tin, tout = gpu.tensor_from_bf16(bits), gpu.tensor_new_bf16(65536)
    gpu.begin()
    gpu.gelu_bf16(tout, tin, 65536, 1)
    gpu.submit()
    got = tout.read()
    g, w = bf16_to_f32(got).astype(np.float64), bf16_to_f32(want).astype(np.float64)
    with np.errstate(divide="ignore", invalid="ignore"):
        ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(w), 1e-300))) - 7)
    allowed = np.maximum(ulp, np.abs(v) * 2.0 ** -23)
    assert (np.abs(g - w)[finite] <= allowed[finite]).all()
    plain = finite & (np.abs(v) < 3.0)
    assert (got[plain] != want[plain]).mean() < 2e-3
    tin.free(), tout.free()


@pytest.mark.parametrize("rows,width,classes", [(5, 256, 1), (130, 3072, 2), (33, 5376, 3), (7, 1000, 2)])
def test_gate_against_the_reference_kernel(gpu, oracle, ref, rows, width, classes):
    """h3_gate_bf16 (src/cuda/cuda_kernels.cuh:973-986): bit-exact, operator and restatement."""
    rng = np.random.default_rng(rows)
    slots, slot = 6, 2
    res, branch = bf(rng.standard_normal((rows, width))), bf(rng.standard_normal((rows, width)) * 3)
    mod = bf(1 + 0.1 * rng.standard_normal((classes, slots, width)))
    row_map = (np.arange(rows) % classes).astype(np.uint32)
    want = ref.gate(res, branch, mod, row_map, slots, slot)
    gate_rows = bf16_to_f32(mod[row_map, slot, :])
    product = bf16_to_f32(branch) * gate_rows                       # float32 numpy: separate IEEE multiply and add
    restated = oracle.f32_to_bf16(bf16_to_f32(res) + product)
    assert (restated == want).all()
    one = np.array([oracle.lib().h3o_gate_residual_bf16(int(res[0, c]), int(branch[0, c]), int(mod[row_map[0], slot, c]))
                    for c in range(min(width, 64))], np.uint16)
    assert (one == want[0, :one.size]).all()
    t_res, t_br, t_mod = (gpu.tensor_from_bf16(a) for a in (res, branch, mod))
    t_map, out = gpu.tensor_from_u32(row_map), gpu.tensor_new_bf16(rows * width)
    gpu.begin()
    gpu.gate_bf16(out, t_res, t_br, t_mod, t_map, rows, width, slots, slot)
    gpu.submit()
    assert (out.read().reshape(rows, width) == want).all()
    for t in (t_res, t_br, t_mod, t_map, out):
        t.free()


@pytest.mark.parametrize("rows,width", [(3, 64), (129, 1792), (40, 14336)])
def test_swiglu_against_the_reference_kernel(gpu, oracle, ref, rows, width):
    """h3_swiglu_bf16 (src/cuda/cuda_kernels.cuh:1047-1059) on a stored [rows, 2 * width] fc1 output.
    h3_gpu_swiglu_bf16 uses the hardware exponential and reciprocal: at most one bf16 step apart."""
    rng = np.random.default_rng(width)
    fused = bf(rng.standard_normal((rows, 2 * width)) * 2.5)
    want = ref.swiglu(fused)
    gate, up = bf16_to_f32(fused[:, :width]), bf16_to_f32(fused[:, width:])
    restated = oracle.f32_to_bf16(gate / (np.float32(1) + np.exp(-gate, dtype=np.float32)) * up)
    apart = steps_apart(restated, want)
    assert apart.max() <= 1 and (apart != 0).mean() < 2e-3
    t_in, out = gpu.tensor_from_bf16(fused), gpu.tensor_new_bf16(rows * width)
    gpu.begin()
    gpu.swiglu_bf16(out, t_in, rows, width)
    gpu.submit()
    apart = steps_apart(out.read().reshape(rows, width), want)
    assert apart.max() <= 1 and (apart != 0).mean() < 5e-3
    t_in.free(), out.free()


@pytest.mark.parametrize("rows,heads,half", [(37, 3, 48), (130, 5, 64), (9, 56, 48)])
def test_qkv_norm_rope_against_the_reference_kernel(gpu, oracle, ref, rows, heads, half):
    """h3_qkv_rope_bf16, grouped columns (src/cuda/cuda_kernels.cuh:988-1045): h3_gpu_grouped_qkv_rope_bf16
    is bit-equal (same rsqrtf instruction on the same GPU, same operation order); the CPU restatement uses
    a correctly rounded 1/sqrt and stays within the bf16 bar."""
    dim = 128
    rng = np.random.default_rng(rows)
    qkv = bf(rng.standard_normal((rows, heads * 3 * dim)) * 4)
    q_norm, k_norm = bf(1 + 0.1 * rng.standard_normal(dim)), bf(1 + 0.1 * rng.standard_normal(dim))
    angle = rng.uniform(0, 6.28, (rows, half))
    cos, sin = bf(np.cos(angle)), bf(np.sin(angle))
    want = ref.qkv_rope(qkv, q_norm, k_norm, cos, sin, heads, dim, half, 1e-5, grouped=1)
    restated = oracle.grouped_qkv_rope(qkv, q_norm, k_norm, cos, sin, heads, dim, half, 1e-5)
    for r, w in zip(restated, want):
        assert within_one_step(r, w, 1.0)          # inputs are N(0, 4^2) normalised to unit RMS
        check_bf16(r.ravel(), w.ravel())
    assert (restated[2] == want[2]).all()
    t_qkv, t_qn, t_kn, t_c, t_s = (gpu.tensor_from_bf16(a) for a in (qkv, q_norm, k_norm, cos, sin))
    outs = [gpu.tensor_new_bf16(rows * heads * dim) for _ in range(3)]
    gpu.begin()
    gpu.grouped_qkv_rope_bf16(*outs, t_qkv, t_qn, t_kn, t_c, t_s, rows, heads, dim, half, 1e-5)
    gpu.submit()
    for o, w in zip(outs, want):
        assert (o.read() == w.ravel()).all()
    for t in [t_qkv, t_qn, t_kn, t_c, t_s] + outs:
        t.free()


@pytest.mark.parametrize("rows,width", [(5, 256), (130, 5376), (300, 3072), (7, 1000), (9, 7168), (6, 248), (6, 250)])
def test_gate_adaln_quantize_against_the_reference_chain(oracle, ref, rows, width):
    """h3_gpu_gate_adaln_quantize_int8 against the reference's own chain on this GPU:
    h3_gate_bf16 -> h3_adaln_bf16 (src/cuda/cuda_kernels.cuh:973-986, 936-971) -> the per-row int8 recipe
    (src/metal/shaders.metal:1434-1459, exact IEEE arithmetic).  Bytes, scales and the gated residual are
    bit-exact.  The CPU restatement differs only through rsqrt: at most one bf16 step in the normalised row."""
    slots, padded = 6, (rows + 127) // 128 * 128
    rng = np.random.default_rng(width)
    res, branch = bf(rng.standard_normal((rows, width))), bf(rng.standard_normal((rows, width)))
    mod = bf(rng.standard_normal((2, slots, width)) * 0.1)
    norm_w = bf(1 + 0.1 * rng.standard_normal(width))
    row_map = (np.arange(rows) % 2).astype(np.uint32)
    gated = ref.gate(res, branch, mod, row_map, slots, 2)
    normalized = ref.adaln(gated, norm_w, mod, row_map, slots, 3, 4, 1e-5)
    want_q, want_s = oracle.quantize_rows(normalized, padded)
    o_gated, o_norm, o_q, o_s = oracle.gate_adaln_quantize(res, branch, mod, norm_w, mod, row_map, padded, slots, 2, 3, 4, 1e-5)
    assert (o_gated == gated).all()
    assert within_one_step(o_norm, normalized, 0.25)
    assert np.abs(o_q.astype(np.int32) - want_q.astype(np.int32)).max() <= 1
    gpu = h.Gpu()
    t_res, t_br, t_mod, t_nw = (gpu.tensor_from_bf16(a) for a in (res, branch, mod, norm_w))
    t_map = gpu.tensor_from_u32(row_map)
    q, sc = gpu.tensor_new_i8(padded * width), gpu.tensor_new_f32(padded)
    gpu.begin()
    gpu.gate_adaln_quantize_int8(t_res, q, sc, t_res, t_br, t_nw, t_mod, t_mod, t_map, rows, padded, width, slots, 2, 3, 4, 1e-5)
    gpu.submit()
    assert (t_res.read().reshape(rows, width) == gated).all()
    assert (q.read().reshape(padded, width) == want_q).all()
    assert (sc.read() == want_s).all()
    gpu.free()


@pytest.mark.parametrize("rows,k,n,with_bias", [(1, 16, 8, True), (17, 128, 24, False), (31, 320, 40, True)])
def test_small_linear_against_the_reference_kernel(gpu, oracle, ref, rows, k, n, with_bias):
    """h3_linear_bf16 (src/cuda/cuda_kernels.cuh:762-794), the reference's own bf16 linear for small
    problems (fp32 fmaf chain, bias seeded into the accumulator): h3_gpu_linear_bf16 and the FP64-dot
    restatement are within the bf16 bar of it."""
    x = synth.activations(3, 1, rows, k).reshape(rows, k)
    w = bf(np.random.default_rng(n).standard_normal((n, k)) * 0.05)
    bias = synth.bf16_normal(3, 4, 1, n, 0, 0.02)[0] if with_bias else None
    want = ref.linear(x, w, bias)
    check_bf16(oracle.linear(oracle.MODE_BF16, x, w, bias=bias), want)
    tx, tw = gpu.tensor_from_bf16(x), gpu.tensor_from_bf16(w)
    tb = gpu.tensor_from_bf16(bias) if with_bias else None
    out = gpu.tensor_new_bf16(rows * n)
    gpu.begin()
    gpu.linear_bf16(out, tx, tw, tb, rows, k, n)
    gpu.submit()
    check_bf16(out.read().reshape(rows, n), want)
    for t in (tx, tw, tb, out):
        if t is not None:
            t.free()


def test_add_against_the_reference_kernel(gpu, ref):
    rng = np.random.default_rng(1)
    a, b = bf(rng.standard_normal(5000)), bf(rng.standard_normal(5000))
    ta, tb, out = gpu.tensor_from_bf16(a), gpu.tensor_from_bf16(b), gpu.tensor_new_bf16(5000)
    gpu.begin()
    gpu.add_bf16(out, ta, tb, 5000)
    gpu.submit()
    assert (out.read() == ref.add(a, b)).all()
    for t in (ta, tb, out):
        t.free()
