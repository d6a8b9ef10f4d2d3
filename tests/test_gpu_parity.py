"""Parity of the CUDA path with the oracle, through the C-ABI (ctypes), on a B200.

The bar: bit-exact for integer work (quantised bytes, scales, int32
accumulators) and for exactly representable patterns; bf16 outputs within
rel-L2 <= 2e-3 and max |delta| <= 2 bf16 ulp (ulp floor: see tests/parity.py).
Cases follow h3cli's own operator tests (tests/metal_q8.c, tests/quant_native.c)
and the benchmark configurations.
"""
import os
import tempfile

import numpy as np
import pytest

import h3cli_b200 as h
from h3cli_b200 import synth
from parity import bf16_to_f32, check_bf16, rel_l2

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TC_KERNELS = [h.KERNEL_TCGEN05, h.KERNEL_TCGEN05_M256, h.KERNEL_TCGEN05_N128]
PAIR = [h.KERNEL_TCGEN05_PAIR]   # two-CTA kernels (bf16, int8, and W8A16 with main-loop dequantisation)
GUARD = 64


def upload(gpu, **arrays):
    out = {}
    for name, a in arrays.items():
        if a is None:
            continue
        a = np.ascontiguousarray(a)
        out[name] = (gpu.tensor_from_bf16(a) if a.dtype == np.uint16 else gpu.tensor_from_i8(a) if a.dtype == np.int8
                     else gpu.tensor_from_f32(a))
    return out


def raw_linear(gpu, mode, x, w, ws=None, group=0, xs=None, bias=None, gate=None, residual=None, activation=0,
               kernel=h.KERNEL_AUTO, want_acc=False):
    """One h3q8_linear call on fresh tensors; returns bf16 bits [M,N] (and int32 accumulators)."""
    M, K = x.shape
    N = w.shape[0]
    t = upload(gpu, input=x, weight=w, weight_scales=ws, input_scales=xs, bias=bias, gate=gate, residual=residual)
    out = gpu.tensor_from_bf16(np.full(M * N + GUARD, 0x3F80, np.uint16))
    fields = dict(mode=mode, rows=M, input_dim=K, output_dim=N, weight_group=group, activation=activation, kernel=kernel,
                  output=out, **t)
    acc = None
    if want_acc:
        acc = gpu.tensor_alloc(M * N, 3)
        fields["accumulators"] = acc
    gpu.raw_linear(**fields)
    assert gpu.raw_status() == 0
    got = out.read()
    assert (got[M * N:] == 0x3F80).all(), "wrote past the end of the output"
    result = got[:M * N].reshape(M, N)
    accv = acc.read(dtype=3).view(np.int32).reshape(M, N) if want_acc else None
    for tensor in list(t.values()) + [out] + ([acc] if acc else []):
        tensor.free()
    return (result, accv) if want_acc else result


def operands(seed, M, N, K, group, outliers=False):
    width = group or K
    x = synth.activations(seed, 1, M, K, outliers=synth.outlier_channels(seed, K) if outliers else None).reshape(M, K)
    wq = synth.int8_weights(seed, 2, N, K)
    ws = synth.lognormal_scales(seed, 3, N, (K + width - 1) // width)
    return x, wq, ws


def epilogue_operands(seed, M, N, spec):
    bias = synth.bf16_normal(seed, 4, 1, N, 0, 0.02)[0] if "b" in spec else None
    gate = synth.bf16_normal(seed, 5, 1, N, 1, 0.1)[0] if "g" in spec else None
    res = synth.bf16_normal(seed, 6, M, N, 0, 1).reshape(M, N) if "r" in spec else None
    return bias, gate, res, (1 if "a" in spec else 0)


# --------------------------------------------------------------------------- quantisers
@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (33, 100), (130, 128), (300, 3072), (17, 5000), (5, 12288), (9, 1000), (70, 4096), (11, 3080)])
def test_row_quantiser_bit_exact(gpu, oracle, rows, cols):
    x = synth.activations(11, 1, rows, cols, outliers=synth.outlier_channels(11, cols)).reshape(rows, cols)
    x[0] = 0  # zero row: scale 1/127
    padded = (rows + 127) // 128 * 128
    tx, q, s = gpu.tensor_from_bf16(x), gpu.tensor_new_i8(padded * cols), gpu.tensor_new_f32(padded)
    lib = h.library()
    assert lib.h3q8_quantize_rows(tx.device_pointer, q.device_pointer, s.device_pointer, rows, padded, cols, 1.0, gpu.stream)
    gpu.synchronize()
    want_q, want_s = oracle.quantize_rows(x, padded)
    assert (q.read().reshape(padded, cols) == want_q).all()
    assert (s.read().view(np.uint32) == want_s.view(np.uint32)).all()
    assert not lib.h3q8_quantize_rows(tx.device_pointer, q.device_pointer, s.device_pointer, rows, rows - 1, cols, 1.0, gpu.stream)
    for t in (tx, q, s):
        t.free()


@pytest.mark.parametrize("group", [0, 64, 128])
@pytest.mark.parametrize("rows,cols", [(1, 1), (35, 65), (67, 129), (256, 256), (96, 3072)])
def test_device_packer_and_dequant_bit_exact(gpu, oracle, rows, cols, group):
    w = synth.bf16_normal(13, 2, rows, cols, 0, 0.125).reshape(rows, cols)
    w[0, 0] = 0
    want_q, want_s = oracle.q8_pack_rows(w, group)
    tw, q, s = gpu.tensor_from_bf16(w), gpu.tensor_new_i8(rows * cols), gpu.tensor_new_f32(want_s.size)
    lib = h.library()
    assert lib.h3q8_q8_pack_rows_device(tw.device_pointer, q.device_pointer, s.device_pointer, rows, cols, group, gpu.stream)
    gpu.synchronize()
    assert (q.read().reshape(rows, cols) == want_q).all()
    assert (s.read().view(np.uint32) == want_s.ravel().view(np.uint32)).all()
    d = gpu.tensor_new_bf16(rows * cols)
    assert lib.h3q8_q8_dequant(q.device_pointer, s.device_pointer, d.device_pointer, rows, cols, group, gpu.stream)
    gpu.synchronize()
    assert (d.read().reshape(rows, cols) == oracle.q8_dequant(want_q, want_s, group)).all()
    for t in (tw, q, s, d):
        t.free()


def test_gelu_operator_all_bf16_inputs(gpu, oracle):
    """Every finite bf16 input through h3_gpu_gelu_bf16 against the oracle's tanh-GELU
    (src/cuda/cuda_kernels.cuh:883-893).

    The device evaluates 0.5 v (1 + tanh u) as v / (1 + exp(-2u)).  Where tanh u is
    within 2^-24 of -1 the reference's own fp32 expression 1 + tanhf(u) cancels to
    noise of about 2^-25 |v| (it returns exactly 0 below u = -8.7), so outputs there
    are compared on that absolute scale; everywhere else within one bf16 step."""
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    v = bf16_to_f32(bits).astype(np.float64)
    finite = np.isfinite(v)
    tin, tout = gpu.tensor_from_bf16(bits), gpu.tensor_new_bf16(65536)
    gpu.begin()
    gpu.gelu_bf16(tout, tin, 65536, 1)
    gpu.submit()
    got_bits, want_bits = tout.read(), oracle.gelu_tanh_bf16(bits)
    got, want = bf16_to_f32(got_bits).astype(np.float64), bf16_to_f32(want_bits).astype(np.float64)
    with np.errstate(divide="ignore", invalid="ignore"):
        ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(want), 1e-300))) - 7)
    allowed = np.maximum(ulp, np.abs(v) * 2.0 ** -23)
    error = np.abs(got - want)
    assert (error[finite] <= allowed[finite]).all()
    assert (got_bits[finite] != want_bits[finite]).mean() < 0.02
    exact = np.abs(v) < 3.0          # away from the cancellation region the stored bits agree almost always
    assert (got_bits[finite & exact] != want_bits[finite & exact]).mean() < 2e-3
    tin.free(), tout.free()


# --------------------------------------------------------------------------- the reference's operator test
@pytest.mark.parametrize("index", [0, 1, 2, 3])
def test_q8_load_and_linear_like_the_reference(oracle, index):
    """tests/metal_q8.c:89-175: load bf16 from a file into Q8, stored bytes equal
    the CPU packer's, linear + bias against the FP64 oracle, guard words, rejects,
    dispatch counters."""
    pack, lin = np.load(os.path.join(GOLDEN, "q8_pack.npz")), np.load(os.path.join(GOLDEN, "linear.npz"))
    src, want_q, want_s = pack[f"src{index}"], pack[f"q{index}"], pack[f"s{index}"]
    x, bias, want = lin[f"x{index}"], lin[f"bias{index}"], lin[f"out{index}"]
    n, k = src.shape
    m = x.shape[0]
    gpu = h.Gpu()
    with tempfile.NamedTemporaryFile(suffix=".bf16") as f:
        f.write(src.tobytes())
        f.flush()
        w = gpu.q8_load(f.name, 0, n, k)
        with pytest.raises(h.H3Error):
            gpu.q8_load(f.name, 1, n, k)
        with pytest.raises(h.H3Error):
            gpu.q8_load(f.name, 0, 0xFFFFFFFF, 0xFFFFFFFF)
        with pytest.raises(h.H3Error):
            gpu.q8_load(f.name, 2, n, k)  # short read
    offset = ((n * k + 3) & ~3) + 15 & ~15
    blob = w.read(offset + want_s.size * 4, dtype=2)
    assert (blob[:n * k].reshape(n, k) == want_q).all()
    assert (blob[offset:].view(np.float32).view(np.uint32) == want_s.ravel().view(np.uint32)).all()
    tx, tb = gpu.tensor_from_bf16(x), gpu.tensor_from_bf16(bias)
    out = gpu.tensor_from_bf16(np.full(m * n + GUARD, 0x3F80, np.uint16))
    for repeat in range(2):
        gpu.begin()
        gpu.linear_bf16(out, tx, w, tb, m, k, n)
        gpu.submit()
    got = out.read()
    assert (got[m * n:] == 0x3F80).all()
    assert rel_l2(got[:m * n], want.ravel()) < 0.006          # the reference's own gate
    check_bf16(got[:m * n], want.ravel())
    gpu.begin()
    with pytest.raises(h.H3Error):
        gpu.linear_bf16(out, tx, w, None, m, k, n + 1)
    with pytest.raises(h.H3Error):
        gpu.linear_bf16(tx, tx, w, None, m, k, n)
    gpu.cancel()
    assert (tx.read() == x.ravel()).all()
    stats = gpu.stats()
    assert stats.q8_weights == 1 and stats.q8_dispatches == 2
    gpu.free()


@pytest.mark.parametrize("scratch_rows", [0, 1])
def test_queued_linears_share_scratch(scratch_rows):
    """tests/metal_q8.c:42-87: distinct diagonal matrices queued in one command
    scope; with the dequant-to-scratch policy they share one scratch buffer, so a
    missing producer/consumer dependency would show as a wrong (exact) answer."""
    gpu = h.Gpu()
    gpu.set_w8a16_scratch_rows(scratch_rows)
    with tempfile.NamedTemporaryFile(suffix=".bf16") as f:
        for j in range(2):
            f.write(synth.to_bf16(np.eye(64, dtype=np.float32) * (j + 1)).tobytes())
        f.flush()
        w = [gpu.q8_load(f.name, j * 64 * 64 * 2, 64, 64) for j in range(2)]
    x = synth.to_bf16(np.arange(3 * 64, dtype=np.float32) - 100.0)
    tx = gpu.tensor_from_bf16(x)
    outs = [gpu.tensor_new_bf16(3 * 64) for _ in range(6)]
    warm = None
    for repeat in range(3):
        gpu.begin()
        for j in range(6):
            gpu.linear_bf16(outs[j], tx, w[(j + repeat) % 2], None, 3, 64, 64)
            if repeat and j % 2:
                gpu.continue_()
        gpu.submit()
        for j in range(6):
            want = synth.to_bf16(synth.from_bf16(x) * np.float32(1 + (j + repeat) % 2))
            assert (outs[j].read() == want).all()
        stats = gpu.stats()
        if not repeat:
            warm = stats
        else:
            assert stats.tensor_allocations == warm.tensor_allocations
            assert stats.native_scratch_bytes == warm.native_scratch_bytes
            if scratch_rows:
                assert stats.native_scratch_reuses > warm.native_scratch_reuses
    assert gpu.stats().q8_weights == 2 and gpu.stats().q8_dispatches == 18
    gpu.free()


# --------------------------------------------------------------------------- exact patterns
def exact_pattern(M, N, K):
    """Operands whose products and sums are exactly representable (the design of
    tests/quant_native.c:30-52): powers of two by row/column bands."""
    r, c, k = np.arange(M)[:, None], np.arange(N)[:, None], np.arange(K)[None, :]
    x = (2.0 ** ((r + k) % 3 - 1)) * np.where((r + k) % 2, -1.0, 1.0)
    wq = (2 ** ((c + k) % 4)).astype(np.int8) * np.where((c + 2 * k) % 3 == 0, -1, 1).astype(np.int8)
    ws = (2.0 ** (-(np.arange(N) % 3) - 4)).astype(np.float32)[:, None]
    return synth.to_bf16(x.astype(np.float32)).reshape(M, K), wq, ws


@pytest.mark.parametrize("rows", [1, 3, 17, 129, 300])
@pytest.mark.parametrize("kernel", [h.KERNEL_PLAIN] + TC_KERNELS + PAIR)
def test_exact_patterns_bit_exact(gpu, oracle, rows, kernel):
    N, K = 256, 512
    x, wq, ws = exact_pattern(rows, N, K)
    want = oracle.linear(oracle.MODE_W8A16, x, wq, ws, 0)
    assert (raw_linear(gpu, h.MODE_W8A16, x, wq, ws, 0, kernel=kernel) == want).all()
    wb = oracle.q8_dequant(wq, ws, 0)
    assert (raw_linear(gpu, h.MODE_BF16, x, wb, kernel=kernel) == want).all()
    xq, xs = oracle.quantize_rows(x)
    want8, acc8 = oracle.linear(oracle.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, x_scales=xs, want_acc=True)
    got8, gacc = raw_linear(gpu, h.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, xs=xs, kernel=kernel, want_acc=True)
    assert (gacc == acc8).all() and (got8 == want8).all()


def test_all_zero_input(gpu, oracle):
    x = np.zeros((129, 256), np.uint16)
    _, wq, ws = operands(3, 129, 128, 256, 0)
    for kernel in (h.KERNEL_PLAIN, h.KERNEL_TCGEN05):
        assert (raw_linear(gpu, h.MODE_W8A16, x, wq, ws, 0, kernel=kernel) == 0).all()


# --------------------------------------------------------------------------- randomised parity, ragged shapes
SHAPES = [(1, 8, 16), (17, 40, 80), (129, 256, 256), (300, 520, 512), (128, 256, 64), (257, 264, 1040), (64, 3072, 3072)]


@pytest.mark.parametrize("kernel", [h.KERNEL_PLAIN] + TC_KERNELS + PAIR)
@pytest.mark.parametrize("M,N,K", SHAPES + [(1000, 776, 1024), (513, 1032, 3072)])
@pytest.mark.parametrize("group,spec", [(0, ""), (64, "b"), (128, "ba"), (0, "gr"), (64, "bgra")])
def test_w8a16_parity(gpu, oracle, M, N, K, group, spec, kernel):
    x, wq, ws = operands(21, M, N, K, group)
    bias, gate, res, act = epilogue_operands(21, M, N, spec)
    want = oracle.linear(oracle.MODE_W8A16, x, wq, ws, group, bias=bias, gate=gate, residual=res, activation=act)
    got = raw_linear(gpu, h.MODE_W8A16, x, wq, ws, group, bias=bias, gate=gate, residual=res, activation=act, kernel=kernel)
    check_bf16(got, want)


@pytest.mark.parametrize("kernel", [h.KERNEL_PLAIN] + TC_KERNELS + PAIR)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_bf16_parity(gpu, oracle, M, N, K, kernel):
    x, wq, ws = operands(22, M, N, K, 64)
    wb = oracle.q8_dequant(wq, ws, 64)
    bias, gate, res, act = epilogue_operands(22, M, N, "bgr")
    want = oracle.linear(oracle.MODE_BF16, x, wb, bias=bias, gate=gate, residual=res)
    check_bf16(raw_linear(gpu, h.MODE_BF16, x, wb, bias=bias, gate=gate, residual=res, kernel=kernel), want)


@pytest.mark.parametrize("kernel", [h.KERNEL_PLAIN] + TC_KERNELS + PAIR)
@pytest.mark.parametrize("M,N,K", [(1, 8, 16), (40, 24, 128), (130, 128, 256), (300, 520, 512), (257, 264, 1040), (64, 3072, 3072)])
@pytest.mark.parametrize("spec", ["", "ba", "gr"])
def test_w8a8_int32_exact_and_epilogue(gpu, oracle, M, N, K, spec, kernel):
    x, wq, ws = operands(23, M, N, K, 0, outliers=True)
    xq, xs = oracle.quantize_rows(x)
    bias, gate, res, act = epilogue_operands(23, M, N, spec)
    want, acc = oracle.linear(oracle.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, x_scales=xs, bias=bias, gate=gate, residual=res,
                              activation=act, want_acc=True, fast=True)
    got, gacc = raw_linear(gpu, h.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, xs=xs, bias=bias, gate=gate, residual=res,
                           activation=act, kernel=kernel, want_acc=True)
    assert (gacc == acc).all(), "int32 accumulators differ"
    if act:
        check_bf16(got, want)           # tanhf may differ in its last fp32 bit
    else:
        assert (got == want).all()      # identical accumulators and identical fp32 epilogue: identical bits


@pytest.mark.parametrize("kernel", [h.KERNEL_PLAIN, h.KERNEL_TCGEN05, h.KERNEL_TCGEN05_PAIR])
@pytest.mark.parametrize("M,N,K", [(40, 24, 256), (130, 128, 256), (300, 520, 512), (64, 3072, 3072)])
def test_w8a8_group128_weight_scales(gpu, oracle, M, N, K, kernel):
    """Config 3(b): per-group-128 weight scales.  No reference implementation
    exists; pinned by exact int32 group sums combined in fp32 in ascending group
    order (the order of src/metal/shaders.metal:2701-2741)."""
    x, wq, ws = operands(24, M, N, K, 128, outliers=True)
    xq, xs = oracle.quantize_rows(x)
    bias = synth.bf16_normal(24, 4, 1, N, 0, 0.02)[0]
    want = oracle.linear(oracle.MODE_W8A8, xq, wq, ws, 128, x_scales=xs, bias=bias, fast=True)
    got = raw_linear(gpu, h.MODE_W8A8, xq, wq, ws, 128, xs=xs, bias=bias, kernel=kernel)
    assert (got == want).all()


@pytest.mark.parametrize("kernel", [h.KERNEL_TCGEN05_SPLITK, h.KERNEL_AUTO])
@pytest.mark.parametrize("M,N,K", [(1, 3072, 3072), (16, 3072, 3072), (100, 520, 1536), (128, 1536, 12288), (77, 256, 1000 * 16)])
@pytest.mark.parametrize("mode", ["bf16", "w8a16", "w8a16g128", "w8a8"])
def test_skinny_split_k(gpu, oracle, mode, M, N, K, kernel):
    """At most 128 rows: the K range of every 128 x 128 tile is split over several CTAs (partial sums in a
    caller-provided workspace, summed in a fixed order by a finishing kernel that owns the epilogue).
    int32 partial sums are exact, so W8A8 stays bit-equal to the oracle; bf16 / W8A16 change the fp32 order."""
    group = 128 if mode == "w8a16g128" else 0
    if group and K % 128:
        pytest.skip("group width must divide K")
    x, wq, ws = operands(61, M, N, K, group, outliers=mode == "w8a8")
    bias, gate, res, act = epilogue_operands(61, M, N, "bgr" if M % 2 else "ba")
    lib = h.library()
    mode_id = {"bf16": h.MODE_BF16, "w8a16": h.MODE_W8A16, "w8a16g128": h.MODE_W8A16, "w8a8": h.MODE_W8A8}[mode]
    nbytes = lib.h3q8_linear_workspace_bytes(mode_id, M, K, N)
    assert lib.h3q8_linear_workspace_bytes(mode_id, 129, K, N) == 0
    if not nbytes:                                   # too few k-blocks to split (int8 k-blocks are 128 wide)
        assert mode == "w8a8" and K < 2048
        pytest.skip("K too short for split-K in this mode")
    assert nbytes >= 2 * M * N * 4
    workspace = gpu.tensor_alloc(nbytes + 64, 2)
    if mode == "bf16":
        wb = oracle.q8_dequant(wq, ws, 0)
        want = oracle.linear(oracle.MODE_BF16, x, wb, bias=bias, gate=gate, residual=res, activation=act)
        t = upload(gpu, input=x, weight=wb, bias=bias, gate=gate, residual=res)
    elif mode == "w8a8":
        xq, xs = oracle.quantize_rows(x)
        want = oracle.linear(oracle.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, x_scales=xs, bias=bias, gate=gate, residual=res, activation=act, fast=True)
        t = upload(gpu, input=xq, weight=wq, weight_scales=ws[:, 0].copy(), input_scales=xs, bias=bias, gate=gate, residual=res)
    else:
        want = oracle.linear(oracle.MODE_W8A16, x, wq, ws, group, bias=bias, gate=gate, residual=res, activation=act)
        t = upload(gpu, input=x, weight=wq, weight_scales=ws, bias=bias, gate=gate, residual=res)
    out = gpu.tensor_from_bf16(np.full(M * N + GUARD, 0x3F80, np.uint16))
    launches = lib.h3q8_kernel_launches()
    gpu.raw_linear(mode=mode_id, rows=M, input_dim=K, output_dim=N, weight_group=group, activation=act, kernel=kernel, output=out,
                   workspace=workspace, workspace_bytes=nbytes, **t)
    # split GEMM + finishing kernel; AUTO prefers the one-launch weight-streaming kernel
    assert gpu.raw_status() == 0 and lib.h3q8_kernel_launches() - launches == (1 if kernel == h.KERNEL_AUTO else 2)
    got = out.read()
    assert (got[M * N:] == 0x3F80).all(), "wrote past the end of the output"
    if mode == "w8a8" and not act:
        assert (got[:M * N].reshape(M, N) == want).all()
    else:
        check_bf16(got[:M * N].reshape(M, N), want)
    with pytest.raises(h.H3Error):
        gpu.raw_linear(mode=mode_id, rows=M, input_dim=K, output_dim=N, weight_group=group, activation=act,
                       kernel=h.KERNEL_TCGEN05_SPLITK, output=out, workspace=workspace, workspace_bytes=M * N * 4, **t)
    for tensor in list(t.values()) + [out, workspace]:
        tensor.free()


def test_gemm_as_programmatic_dependent_of_its_dequantiser(gpu, oracle):
    """h3q8_linear_desc.after_producer: the dequantiser writes the bf16 weight into ONE scratch buffer and the two-CTA
    GEMM enqueued right behind it is launched as a programmatic dependent.  Two weight sets alternate through the same
    scratch for 40 calls; if the GEMM's first load did not wait for the dequantiser it would multiply by the other set
    (or a mixture), so every output is compared with the ordinary-launch result bit for bit."""
    M, N, K = 1024, 768, 1024
    lib = h.library()
    sets, wants, outs = [], [], []
    x = synth.activations(81, 1, M, K).reshape(M, K)
    tx = gpu.tensor_from_bf16(x)
    scratch = gpu.tensor_new_bf16(N * K)
    for i in range(2):
        wq, ws = synth.int8_weights(82 + i, 2, N, K), synth.lognormal_scales(82 + i, 3, N, 1)
        sets.append(upload(gpu, weight=wq, weight_scales=ws))
        wants.append(raw_linear(gpu, h.MODE_BF16, x, oracle.q8_dequant(wq, ws, 0), kernel=h.KERNEL_TCGEN05_PAIR))
        check_bf16(wants[i], oracle.linear(oracle.MODE_W8A16, x, wq, ws, 0))
    outs = [gpu.tensor_new_bf16(M * N) for _ in range(40)]
    for i, out in enumerate(outs):
        t = sets[i % 2]
        assert lib.h3q8_q8_dequant(t["weight"].device_pointer, t["weight_scales"].device_pointer, scratch.device_pointer, N, K, 0, gpu.stream)
        gpu.raw_linear(mode=h.MODE_BF16, rows=M, input_dim=K, output_dim=N, input=tx, weight=scratch, output=out,
                       kernel=h.KERNEL_TCGEN05_PAIR, after_producer=1)
    assert gpu.raw_status() == 0
    for i, out in enumerate(outs):
        assert (out.read().reshape(M, N) == wants[i % 2]).all(), i
    for tensor in outs + [tx, scratch] + [v for t in sets for v in t.values()]:
        tensor.free()


@pytest.mark.parametrize("M,N,K", [(1, 3072, 3072), (16, 3072, 3072), (16, 12288, 3072), (16, 3072, 12288), (33, 520, 1536),
                                   (64, 1536, 12288), (47, 256, 16000), (5, 136, 1040), (17, 128, 128), (64, 8, 4096),
                                   (65, 3072, 3072), (100, 520, 1536), (128, 1536, 12288), (128, 3072, 3072)])
@pytest.mark.parametrize("mode", ["bf16", "w8a16", "w8a16g64", "w8a16g128", "w8a8"])
def test_skinny_weight_streaming(gpu, oracle, mode, M, N, K):
    """At most 128 rows: the weight is the MMA's wide operand, K is split over a thread-block cluster and the partial
    sums are reduced through distributed shared memory in ascending split order -- one launch, no workspace.
    int32 partial sums are exact, so W8A8 stays bit-equal to the oracle; ragged N, K tails and every epilogue term."""
    group = {"w8a16g64": 64, "w8a16g128": 128}.get(mode, 0)
    if group and K % group:
        pytest.skip("group width must divide K")
    x, wq, ws = operands(67, M, N, K, group, outliers=mode == "w8a8")
    bias, gate, res, act = epilogue_operands(67, M, N, "bgr" if M % 2 else "ba")
    lib = h.library()
    mode_id = h.MODE_BF16 if mode == "bf16" else h.MODE_W8A8 if mode == "w8a8" else h.MODE_W8A16
    if mode == "bf16":
        wb = oracle.q8_dequant(wq, ws, 0)
        want = oracle.linear(oracle.MODE_BF16, x, wb, bias=bias, gate=gate, residual=res, activation=act)
        t = upload(gpu, input=x, weight=wb, bias=bias, gate=gate, residual=res)
    elif mode == "w8a8":
        xq, xs = oracle.quantize_rows(x)
        want = oracle.linear(oracle.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, x_scales=xs, bias=bias, gate=gate, residual=res, activation=act, fast=True)
        t = upload(gpu, input=xq, weight=wq, weight_scales=ws[:, 0].copy(), input_scales=xs, bias=bias, gate=gate, residual=res)
    else:
        want = oracle.linear(oracle.MODE_W8A16, x, wq, ws, group, bias=bias, gate=gate, residual=res, activation=act)
        t = upload(gpu, input=x, weight=wq, weight_scales=ws, bias=bias, gate=gate, residual=res)
    out = gpu.tensor_from_bf16(np.full(M * N + GUARD, 0x3F80, np.uint16))
    launches = lib.h3q8_kernel_launches()
    gpu.raw_linear(mode=mode_id, rows=M, input_dim=K, output_dim=N, weight_group=group, activation=act,
                   kernel=h.KERNEL_TCGEN05_SKINNY, output=out, **t)
    assert gpu.raw_status() == 0 and lib.h3q8_kernel_launches() - launches == 1
    got = out.read()
    assert (got[M * N:] == 0x3F80).all(), "wrote past the end of the output"
    if mode == "w8a8" and not act:
        assert (got[:M * N].reshape(M, N) == want).all()
    else:
        check_bf16(got[:M * N].reshape(M, N), want)
    with pytest.raises(h.H3Error):                   # more rows than the kernel's token operand holds
        gpu.raw_linear(mode=mode_id, rows=129, input_dim=K, output_dim=N, weight_group=group, activation=act,
                       kernel=h.KERNEL_TCGEN05_SKINNY, output=out, **t)
    for tensor in list(t.values()) + [out]:
        tensor.free()


@pytest.mark.parametrize("spec", ["", "bgr", "ba"])
@pytest.mark.parametrize("M,N,K,group,both", [(1000, 776, 1024, 128, False), (513, 256, 3072, 256, True), (700, 1032, 2048, 512, False),
                                              (2100, 3072, 1536, 128, True)])
def test_w8a8_grouped_two_cta_kernel(gpu, oracle, M, N, K, group, both, spec):
    """Per-K-group weight scales (and, with `both`, per-group activation scales of the same width) on the
    two-CTA kernel: group sums leave TMEM per group and are combined in fp32 registers, bit-equal to the
    oracle's ascending-group sum; groups <= 256 take the exact bias-trick conversion, wider ones cvt."""
    x, wq, ws = operands(31, M, N, K, group, outliers=True)
    bias, gate, res, act = epilogue_operands(31, M, N, spec)
    if both:
        xq, xs = oracle.quantize_rows_grouped(x, group)
    else:
        xq, xs = oracle.quantize_rows(x)
    want = oracle.linear(oracle.MODE_W8A8, xq, wq, ws, group, x_scales=xs, bias=bias, gate=gate, residual=res, activation=act,
                         input_group=group if both else 0, fast=True)
    t = upload(gpu, input=xq, weight=wq, weight_scales=ws, input_scales=np.ascontiguousarray(xs), bias=bias, gate=gate, residual=res)
    out = gpu.tensor_from_bf16(np.full(M * N + GUARD, 0x3F80, np.uint16))
    launches = h.library().h3q8_kernel_launches()
    gpu.raw_linear(mode=h.MODE_W8A8, rows=M, input_dim=K, output_dim=N, weight_group=group, input_group=group if both else 0,
                   activation=act, kernel=h.KERNEL_AUTO, output=out, **t)
    assert gpu.raw_status() == 0 and h.library().h3q8_kernel_launches() - launches == 1
    got = out.read()
    assert (got[M * N:] == 0x3F80).all(), "wrote past the end of the output"
    if act:
        check_bf16(got[:M * N].reshape(M, N), want)
    else:
        assert (got[:M * N].reshape(M, N) == want).all()
    for tensor in list(t.values()) + [out]:
        tensor.free()


@pytest.mark.parametrize("kernel", [h.KERNEL_PLAIN, h.KERNEL_AUTO])
@pytest.mark.parametrize("M,N,K,group", [(40, 24, 2048, 1024), (300, 520, 2048, 1024), (130, 128, 512, 128), (64, 5376, 14336, 1024)])
def test_w8a8_activation_group_scales(gpu, oracle, M, N, K, group, kernel):
    """The reference's FC2 recipe: per-row, per-1024-K-group activation scales, per-channel
    weight scales, group sums combined in fp32 (src/metal/shaders.metal:1552-1598, 2663-2742)."""
    x, wq, ws = operands(26, M, N, K, 0, outliers=True)
    want_q, want_s = oracle.quantize_rows_grouped(x, group)
    tx, q, sc = gpu.tensor_from_bf16(x), gpu.tensor_new_i8(M * K), gpu.tensor_new_f32(M * (K // group))
    lib = h.library()
    assert lib.h3q8_quantize_rows_grouped(tx.device_pointer, q.device_pointer, sc.device_pointer, M, M, K, group, gpu.stream)
    gpu.synchronize()
    assert (q.read().reshape(M, K) == want_q).all() and (sc.read().reshape(M, -1).view(np.uint32) == want_s.view(np.uint32)).all()
    want = oracle.linear(oracle.MODE_W8A8, want_q, wq, ws[:, 0].copy(), 0, x_scales=want_s, input_group=group, fast=True)
    tw, tws, out = gpu.tensor_from_i8(wq), gpu.tensor_from_f32(ws[:, 0].copy()), gpu.tensor_new_bf16(M * N)
    gpu.raw_linear(mode=h.MODE_W8A8, rows=M, input_dim=K, output_dim=N, input=q, input_scales=sc, input_group=group,
                   weight=tw, weight_scales=tws, output=out, kernel=kernel)
    assert gpu.raw_status() == 0
    assert (out.read().reshape(M, N) == want).all()
    for t in (tx, q, sc, tw, tws, out):
        t.free()


@pytest.mark.parametrize("kernel", [h.KERNEL_PLAIN, h.KERNEL_AUTO])
@pytest.mark.parametrize("M,N,K", [(40, 24, 128), (300, 520, 512), (257, 1000, 320), (129, 14336 // 8, 5376 // 4)])
@pytest.mark.parametrize("mode", ["bf16", "w8a16", "w8a8"])
def test_swiglu_projection(gpu, oracle, mode, M, N, K, kernel):
    """fc1 + SwiGLU in one kernel: weight [gate N | up N] rows, out = bf16(silu(bf16(gate)) * up)
    (src/metal/shaders.metal:2209-2317 for int8, linear + src/cuda/cuda_kernels.cuh:1047-1059 otherwise)."""
    x, wq, ws = operands(27, M, 2 * N, K, 0)
    ws = (ws * np.float32(0.2)).astype(np.float32)       # keep silu(gate) * up in a sane range
    bias = synth.bf16_normal(27, 4, 1, 2 * N, 0, 0.02)[0]
    if mode == "w8a8":
        xq, xs = oracle.quantize_rows(x)
        want = oracle.linear(oracle.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, x_scales=xs, bias=bias, activation=2, fast=True)
        got = raw_swiglu(gpu, h.MODE_W8A8, xq, wq, ws[:, 0].copy(), xs, bias, M, N, K, kernel)
    elif mode == "w8a16":
        want = oracle.linear(oracle.MODE_W8A16, x, wq, ws, 0, bias=bias, activation=2)
        got = raw_swiglu(gpu, h.MODE_W8A16, x, wq, ws, None, bias, M, N, K, kernel)
    else:
        wb = oracle.q8_dequant(wq, ws, 0)
        want = oracle.linear(oracle.MODE_BF16, x, wb, bias=bias, activation=2)
        got = raw_swiglu(gpu, h.MODE_BF16, x, wb, None, None, bias, M, N, K, kernel)
    check_bf16(got, want)


def raw_swiglu(gpu, mode, x, w, ws, xs, bias, M, N, K, kernel):
    t = upload(gpu, input=x, weight=w, weight_scales=ws, input_scales=xs, bias=bias)
    out = gpu.tensor_from_bf16(np.full(M * N + GUARD, 0x3F80, np.uint16))
    gpu.raw_linear(mode=mode, rows=M, input_dim=K, output_dim=N, activation=h.ACT_SWIGLU, kernel=kernel, output=out, **t)
    assert gpu.raw_status() == 0
    got = out.read()
    assert (got[M * N:] == 0x3F80).all()
    for tensor in list(t.values()) + [out]:
        tensor.free()
    return got[:M * N].reshape(M, N)


@pytest.mark.parametrize("quant_mode", [0, 1])
def test_swiglu_fused_equals_unfused_chain(oracle, quant_mode):
    """h3_gpu_linear_bf16 over the [gate | up] weight followed by h3_gpu_swiglu_bf16 (what
    src/denoise/dit.c:2489-2491 does) gives the same bits as the fused projection."""
    M, N, K = 300, 512, 256
    x, wq, ws = operands(28, M, 2 * N, K, 64)
    ws = (ws * np.float32(0.2)).astype(np.float32)
    gpu = h.Gpu()
    if quant_mode:
        gpu.quant_configure(1)
        gpu.set_w8a16_scratch_rows(1)
        w = gpu.q8_from_host(wq, ws, 64)
    else:
        w = gpu.tensor_from_bf16(oracle.q8_dequant(wq, ws, 64))
    tx, wide, chain, fused = gpu.tensor_from_bf16(x), gpu.tensor_new_bf16(M * 2 * N), gpu.tensor_new_bf16(M * N), gpu.tensor_new_bf16(M * N)
    gpu.begin()
    gpu.linear_bf16(wide, tx, w, None, M, K, 2 * N)
    gpu.swiglu_bf16(chain, wide, M, N)
    gpu.linear_fused_bf16(fused, tx, w, None, None, None, M, K, N, h.ACT_SWIGLU)
    gpu.submit()
    assert (chain.read() == fused.read()).all()
    check_bf16(fused.read().reshape(M, N), oracle.linear(oracle.MODE_W8A16, x, wq, ws, 64, activation=2))
    gpu.free()


def test_fixture_w8a8(gpu):
    g = np.load(os.path.join(GOLDEN, "w8a8.npz"))
    for i in range(3):
        got, acc = raw_linear(gpu, h.MODE_W8A8, g[f"xq{i}"], g[f"wq{i}"], g[f"ws{i}"], 0, xs=g[f"xs{i}"], want_acc=True)
        assert (acc == g[f"acc{i}"]).all() and (got == g[f"out{i}"]).all()


# --------------------------------------------------------------------------- properties at benchmark size
def sample_rows(M, count, seed):
    rows = np.unique(np.concatenate([[0, M - 1, M // 2, 127, 128], np.random.default_rng(seed).integers(0, M, count)]))
    return rows[rows < M]


def test_config1_single_w8a16(gpu, oracle):
    """X bf16 [4096,3072] N(0,1), W int8 [3072,3072], per-channel log-normal scales,
    bf16 bias: sampled rows against the FP64 oracle, the whole output against the
    plain kernel, and exact properties (doubling the input, row sharding)."""
    M = N = K = 3072
    M = 4096
    x, wq, ws = operands(1, M, N, K, 0)
    bias = synth.bf16_normal(1, 4, 1, N, 0, 0.02)[0]
    got = raw_linear(gpu, h.MODE_W8A16, x, wq, ws, 0, bias=bias, kernel=h.KERNEL_TCGEN05)
    rows = sample_rows(M, 48, 1)
    want = oracle.linear(oracle.MODE_W8A16, x[rows], wq, ws, 0, bias=bias)
    check_bf16(got[rows], want)
    plain = raw_linear(gpu, h.MODE_W8A16, x, wq, ws, 0, bias=bias, kernel=h.KERNEL_PLAIN)
    check_bf16(got, plain)
    # doubling a bf16 input is exact, so without bias the output doubles exactly
    base = raw_linear(gpu, h.MODE_W8A16, x[:512], wq, ws, 0, kernel=h.KERNEL_TCGEN05)
    twice = raw_linear(gpu, h.MODE_W8A16, synth.to_bf16(synth.from_bf16(x[:512]) * np.float32(2)).reshape(512, K), wq, ws, 0,
                       kernel=h.KERNEL_TCGEN05)
    assert (synth.to_bf16(synth.from_bf16(base) * np.float32(2)).reshape(base.shape) == twice).all()
    # token-row sharding: any split of the rows gives the same bits as the whole
    for shards in (2, 8):
        bounds = [M * i // shards for i in range(shards + 1)]
        parts = [raw_linear(gpu, h.MODE_W8A16, x[a:b], wq, ws, 0, bias=bias, kernel=h.KERNEL_TCGEN05) for a, b in zip(bounds, bounds[1:])]
        assert (np.concatenate(parts) == got).all()


def test_config3_w8a8_outliers(oracle):
    """W8A8 variant of config 1 through the operator layer: activation outliers,
    per-token quantisation in a fused call, (a) per-channel and (b) group-128
    weight scales, bias + GELU in the epilogue."""
    M, N, K = 4096, 3072, 3072
    x, wq, ws_group = operands(3, M, N, K, 128, outliers=True)
    ws_channel = synth.lognormal_scales(3, 7, N, 1)
    bias = synth.bf16_normal(3, 4, 1, N, 0, 0.02)[0]
    xq, xs = oracle.quantize_rows(x)
    for ws, group in ((ws_channel, 0), (ws_group, 128)):
        gpu = h.Gpu()
        gpu.quant_configure(2)
        w = gpu.q8_from_host(wq, ws, group)
        tx, tb, out = gpu.tensor_from_bf16(x), gpu.tensor_from_bf16(bias), gpu.tensor_new_bf16(M * N)
        gpu.begin()
        gpu.linear_fused_bf16(out, tx, w, tb, None, None, M, K, N, h.ACT_GELU_TANH)
        gpu.submit()
        got = out.read().reshape(M, N)
        want = oracle.linear(oracle.MODE_W8A8, xq, wq, ws if group else ws[:, 0].copy(), group, x_scales=xs, bias=bias,
                             activation=1, fast=True)
        check_bf16(got, want)
        # identical int32 sums and dequantisation: away from GELU's cancellation region
        # (negative inputs, outputs near zero) the stored bits agree almost everywhere
        clear = bf16_to_f32(want) > 0.5
        assert (got[clear] != want[clear]).mean() < 1e-3
        gpu.free()


def test_config2_block_stack(oracle):
    """One DiT block's four linears at M = 32,400 (hidden 3072, FFN 12288), W8A16
    per-channel, fused epilogues, through the operator layer; sampled rows against
    the oracle and both W8A16 policies against each other."""
    M, H, F = 32400, 3072, 12288
    rng = np.random.default_rng(2)
    bf = lambda shape, mean=0.0, std=1.0: synth.to_bf16((rng.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean))).reshape(shape)
    x, hidden, res = bf((M, H)), bf((M, F)), bf((M, H))
    gate = bf((H,), 1.0, 0.1)
    layers = [("qkv", x, 3 * H, None, None, 0), ("out", x, H, gate, res, 0), ("up", x, F, None, None, 1), ("down", hidden, H, gate, res, 0)]
    rows = sample_rows(M, 24, 2)
    results = {}
    for policy_rows in (0, 1):
        gpu = h.Gpu()
        gpu.set_w8a16_scratch_rows(policy_rows)
        for name, inp, n, g, r, act in layers:
            k = inp.shape[1]
            wq = rng.integers(-127, 128, (n, k), dtype=np.int8) if policy_rows == 0 else results[name][1]
            ws = synth.lognormal_scales(2, hash(name) % 1000, n, 1) if policy_rows == 0 else results[name][2]
            w = gpu.q8_from_host(wq, ws, 0)
            tx, out = gpu.tensor_from_bf16(inp), gpu.tensor_new_bf16(M * n)
            tg = gpu.tensor_from_bf16(g) if g is not None else None
            tr = gpu.tensor_from_bf16(r) if r is not None else None
            gpu.begin()
            gpu.linear_fused_bf16(out, tx, w, None, tg, tr, M, k, n, act)
            gpu.submit()
            got = out.read().reshape(M, n)
            # each policy on its own against the oracle (policy 1, dequantise-to-scratch + two-CTA bf16 kernel, is the
            # one the benchmark times), then the two policies against each other over the whole output
            want = oracle.linear(oracle.MODE_W8A16, inp[rows], wq, ws, 0, gate=g, residual=None if r is None else r[rows], activation=act)
            check_bf16(got[rows], want)
            if policy_rows == 0:
                results[name] = (got, wq, ws)
            else:
                check_bf16(got, results[name][0])
            for t in (w, tx, out, tg, tr):
                if t is not None:
                    t.free()
        gpu.free()


@pytest.mark.parametrize("shape", ["proj", "qkv", "ffn_up"])
@pytest.mark.parametrize("quant_mode", [1, 2])
def test_config4_grouped_call(oracle, quant_mode, shape):
    """Video (M = 2 x 32 400, K=N=3072) and audio (M = 2 x 1 152, K=N=1536) problems with separate
    weight sets in ONE GEMM launch, at the configuration's full row counts: after the per-problem
    conversion kernels exactly one more kernel is launched; sampled rows against the oracle.
    "qkv" and "ffn_up" are the same launch with the QKV (N = 3 x hidden) and FFN-up (N = 4 x hidden)
    widths of both streams."""
    factor = {"proj": 1, "qkv": 3, "ffn_up": 4}[shape]
    specs = [(2 * 32400, factor * 3072, 3072), (2 * 1152, factor * 1536, 1536)]
    gpu = h.Gpu()
    gpu.quant_configure(quant_mode)
    gpu.set_w8a16_scratch_rows(1)
    problems, wants = [], []
    for i, (M, N, K) in enumerate(specs):
        rng = np.random.default_rng(40 + i)
        x = synth.to_bf16(rng.standard_normal((M, K), dtype=np.float32)).reshape(M, K)
        wq, ws = synth.int8_weights(40 + i, 2, N, K), synth.lognormal_scales(40 + i, 3, N, 1)
        w = gpu.q8_from_host(wq, ws, 0)
        tx, out = gpu.tensor_from_bf16(x), gpu.tensor_new_bf16(M * N)
        problems.append(dict(output=out, input=tx, weight=w, rows=M, input_dim=K, output_dim=N))
        rows = sample_rows(M, 24, i)
        if quant_mode == 1:
            wants.append((rows, oracle.linear(oracle.MODE_W8A16, x[rows], wq, ws, 0), M, N))
        else:
            xq, xs = oracle.quantize_rows(x[rows])
            wants.append((rows, oracle.linear(oracle.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, x_scales=xs), M, N))
    before = h.library().h3q8_kernel_launches()
    gpu.begin()
    gpu.linear_grouped_bf16(problems)
    gpu.submit()
    assert h.library().h3q8_kernel_launches() - before == 3      # two conversion kernels + ONE GEMM launch
    for p, (rows, want, M, N) in zip(problems, wants):
        got = p["output"].read().reshape(M, N)[rows]
        if quant_mode == 2:
            assert (got == want).all()
        else:
            check_bf16(got, want)
        for key in ("output", "input", "weight"):
            p[key].free()
    gpu.free()


def test_grouped_launch_equals_separate_launches(gpu, oracle):
    """Four bf16 problems of different shapes (ragged rows, N and K tails) through
    h3q8_linear_grouped: one launch, and the same bits as four separate launches."""
    import ctypes
    shapes = [(300, 520, 512), (129, 264, 1040), (1000, 256, 64), (257, 3072, 128)]
    lib = h.library()
    descs, keep, separate = (h.LinearDesc * len(shapes))(), [], []
    for i, (M, N, K) in enumerate(shapes):
        x, wq, ws = operands(45 + i, M, N, K, 64)
        wb = oracle.q8_dequant(wq, ws, 64)
        bias, gate, res, act = epilogue_operands(45 + i, M, N, "bgra" if i % 2 else "b")
        separate.append(raw_linear(gpu, h.MODE_BF16, x, wb, bias=bias, gate=gate, residual=res, activation=act,
                                   kernel=h.KERNEL_TCGEN05_PAIR))
        t = upload(gpu, input=x, weight=wb, bias=bias, gate=gate, residual=res)
        t["output"] = gpu.tensor_new_bf16(M * N)
        keep.append(t)
        d = descs[i]
        d.mode, d.rows, d.input_dim, d.output_dim, d.activation, d.kernel = h.MODE_BF16, M, K, N, act, h.KERNEL_TCGEN05_PAIR
        for name, tensor in t.items():
            setattr(d, name, tensor.device_pointer)
    before = lib.h3q8_kernel_launches()
    assert lib.h3q8_linear_grouped(descs, len(shapes), gpu.stream), lib.h3q8_last_error()
    assert gpu.raw_status() == 0
    assert lib.h3q8_kernel_launches() - before == 1
    for (M, N, K), t, want in zip(shapes, keep, separate):
        assert (t["output"].read().reshape(M, N) == want).all()
        for tensor in t.values():
            tensor.free()


@pytest.mark.parametrize("quant_mode", [0, 1])
@pytest.mark.parametrize("rows,N,K", [(300, 520, 1024), (1000, 3072, 2048), (64, 264, 512)])
def test_partial_sums_of_two_k_slices_meet_the_bar(oracle, quant_mode, rows, N, K):
    """A linear cut along K the way the tensor-parallel FFN cuts FFN-down across GPUs: two half-K calls
    store fp32 partial sums (h3q8_gpu_linear_partial_f32), the sums are added in fp32 (what an all-reduce
    does) and h3q8_gpu_linear_finish_bf16 applies gate + residual with the single bf16 rounding.  The result
    meets the same bar against the oracle as the unsplit fused call (rel-L2 <= 2e-3, <= 2 bf16 ulp)."""
    x, wq, ws = operands(61, rows, N, K, 0)
    bias, gate, res, act = epilogue_operands(61, rows, N, "bgr")
    want = oracle.linear(oracle.MODE_W8A16, x, wq, ws, 0, bias=bias, gate=gate, residual=res)
    gpu = h.Gpu()
    if quant_mode:
        gpu.quant_configure(1)
    half = K // 2
    total = np.zeros(rows * N, np.float32)
    for k0, k1 in ((0, half), (half, K)):
        xs = np.ascontiguousarray(x[:, k0:k1])
        w = (gpu.q8_from_host(np.ascontiguousarray(wq[:, k0:k1]), ws, 0) if quant_mode
             else gpu.tensor_from_bf16(oracle.q8_dequant(np.ascontiguousarray(wq[:, k0:k1]), ws, 0)))
        tx, sums = gpu.tensor_from_bf16(xs), gpu.tensor_from_f32(np.full(rows * N + GUARD, 7.0, np.float32))
        gpu.begin()
        gpu.linear_partial_f32(sums, tx, w, rows, k1 - k0, N)
        gpu.submit()
        got = sums.read()
        assert (got[rows * N:] == 7.0).all(), "wrote past the end of the partial sums"
        total += got[:rows * N]                       # fp32 addition, as NCCL's sum does
        for t in (tx, w, sums):
            t.free()
    t_sum, out = gpu.tensor_from_f32(total), gpu.tensor_new_bf16(rows * N)
    tb, tg, tr = (gpu.tensor_from_bf16(a) for a in (bias, gate, res))
    gpu.begin()
    gpu.linear_finish_bf16(out, t_sum, tb, tg, tr, rows, N, 0)
    gpu.submit()
    check_bf16(out.read().reshape(rows, N), want)
    with pytest.raises(h.H3Error):
        gpu.begin()
        gpu.linear_partial_f32(out, tb, tg, rows, K, N)      # sums must be an fp32 tensor
    gpu.cancel()
    gpu.free()


def test_fused_equals_unfused_chain(gpu):
    """linear -> gelu and linear -> gate as separate operators give the same bits
    as the fused projection (the fused epilogue rounds where the chain rounds)."""
    M, N, K = 300, 520, 512
    x, wq, ws = operands(50, M, N, K, 64)
    bias, gate, res, _ = epilogue_operands(50, M, N, "bgr")
    w = gpu.q8_from_host(wq, ws, 64)
    tx, tb, tg, tr = (gpu.tensor_from_bf16(a) for a in (x, bias, gate, res))
    lin, act, chain, fused = (gpu.tensor_new_bf16(M * N) for _ in range(4))
    gpu.begin()
    gpu.linear_bf16(lin, tx, w, tb, M, K, N)
    gpu.gelu_bf16(act, lin, M * N, 1)
    gpu.gate_bf16(chain, tr, act, tg, None, M, N, 1, 0)
    gpu.linear_fused_bf16(fused, tx, w, tb, tg, tr, M, K, N, h.ACT_GELU_TANH)
    gpu.submit()
    assert (chain.read() == fused.read()).all()
    for t in (w, tx, tb, tg, tr, lin, act, chain, fused):
        t.free()


# --------------------------------------------------------------------------- producer-side quantiser fusion
@pytest.mark.parametrize("rows,width", [(5, 256), (130, 5376), (300, 3072), (7, 1000), (9, 7168), (6, 250)])
def test_gate_adaln_quantize_feeds_the_int8_gemm(oracle, rows, width):
    """h3_gpu_gate_adaln_quantize_int8 (src/gpu.h:630-642, src/metal/shaders.metal:3390-3473) and the int8
    projection that consumes its output without re-reading bf16 activations.  gated_residual is bit-exact;
    the normalised row passes through rsqrt (approximate on the GPU), so int8 bytes may differ by one step."""
    slots, padded = 6, (rows + 127) // 128 * 128
    rng = np.random.default_rng(rows)
    bf = lambda a: synth.to_bf16(a.astype(np.float32)).reshape(a.shape)
    res, branch = bf(rng.standard_normal((rows, width))), bf(rng.standard_normal((rows, width)))
    mod = bf(rng.standard_normal((2, slots, width)) * 0.1)
    norm_w = bf(1 + 0.1 * rng.standard_normal(width))
    row_map = (np.arange(rows) % 2).astype(np.uint32)
    want_g, want_n, want_q, want_s = oracle.gate_adaln_quantize(res, branch, mod, norm_w, mod, row_map, padded, slots, 2, 3, 4, 1e-5)
    gpu = h.Gpu()
    t_res, t_br, t_mod, t_nw = (gpu.tensor_from_bf16(a) for a in (res, branch, mod, norm_w))
    t_map = gpu.tensor_from_u32(row_map)
    q, sc = gpu.tensor_new_i8(padded * width), gpu.tensor_new_f32(padded)
    gpu.begin()
    gpu.gate_adaln_quantize_int8(t_res, q, sc, t_res, t_br, t_nw, t_mod, t_mod, t_map, rows, padded, width, slots, 2, 3, 4, 1e-5)
    gpu.submit()
    assert (t_res.read().reshape(rows, width) == want_g).all()          # in place, bit-exact
    got_q, got_s = q.read().reshape(padded, width).astype(np.int32), sc.read()
    assert np.abs(got_q - want_q.astype(np.int32)).max() <= 1 and (got_q != want_q).mean() < 0.02
    assert np.allclose(got_s, want_s, rtol=1e-2) and (got_s[rows:] == 1.0).all() and (got_q[rows:] == 0).all()
    # the int8 projection on exactly these bytes/scales is then bit-exact against the oracle
    N = 256
    wq, ws = synth.int8_weights(7, 2, N, width), synth.lognormal_scales(7, 3, N, 1)
    w = gpu.q8_from_host(wq, ws, 0)
    out = gpu.tensor_new_bf16(rows * N)
    gpu.begin()
    gpu.linear_fused_int8_bf16(out, q, sc, 0, w, None, None, None, rows, width, N, h.ACT_GELU_TANH)
    gpu.submit()
    want = oracle.linear(oracle.MODE_W8A8, got_q[:rows].astype(np.int8), wq, ws[:, 0].copy(), 0, x_scales=got_s[:rows], activation=1, fast=True)
    check_bf16(out.read().reshape(rows, N), want)
    with pytest.raises(h.H3Error):
        gpu.begin()
        gpu.gate_adaln_quantize_int8(t_res, q, sc, t_res, t_br, t_nw, t_mod, t_mod, t_map, rows, padded, width, slots, 9, 3, 4, 1e-5)
    gpu.cancel()
    gpu.free()


@pytest.mark.parametrize("quant_mode", [0, 1, 2])
@pytest.mark.parametrize("rows,heads,width,half", [(300, 4, 512, 48), (129, 3, 256, 64), (1000, 7, 384, 48)])
def test_qkv_projection_with_norm_and_rope(oracle, quant_mode, rows, heads, width, half):
    """h3_gpu_grouped_qkv_linear_rope_bf16 (src/gpu.h:665-683): the QKV projection with per-head RMS
    norm + rotary embedding in its epilogue, grouped [head, q|k|v, 128] columns, head-major outputs.
    Checked bit for bit against the two-call route (projection stored, then h3_gpu_grouped_qkv_rope_bf16,
    formulas of src/cuda/cuda_kernels.cuh:988-1045) and within tolerance against the CPU oracle."""
    dim, n = 128, heads * 3 * 128
    rng = np.random.default_rng(rows)
    bf = lambda a: synth.to_bf16(a.astype(np.float32)).reshape(a.shape)
    x, wq, ws = operands(33, rows, n, width, 0)
    q_norm, k_norm = bf(1 + 0.1 * rng.standard_normal(dim)), bf(1 + 0.1 * rng.standard_normal(dim))
    angle = rng.uniform(0, 6.28, (rows, half))
    cos, sin = bf(np.cos(angle)), bf(np.sin(angle))
    gpu = h.Gpu()
    if quant_mode:
        gpu.quant_configure(quant_mode)
        w = gpu.q8_from_host(wq, ws, 0)
    else:
        w = gpu.tensor_from_bf16(oracle.q8_dequant(wq, ws, 0))
    tx, tqn, tkn, tc, ts = (gpu.tensor_from_bf16(a) for a in (x, q_norm, k_norm, cos, sin))
    fused = [gpu.tensor_new_bf16(rows * heads * dim) for _ in range(3)]
    chain = [gpu.tensor_new_bf16(rows * heads * dim) for _ in range(3)]
    qkv_fused, qkv_chain = gpu.tensor_new_bf16(rows * n), gpu.tensor_new_bf16(rows * n)
    before = h.library().h3q8_kernel_launches()
    gpu.begin()
    gpu.grouped_qkv_linear_rope_bf16(*fused, qkv_fused, tx, w, tqn, tkn, tc, ts, rows, width, heads, dim, half, 1e-5)
    gpu.submit()
    assert h.library().h3q8_kernel_launches() - before == (2 if quant_mode else 1)   # (conversion +) ONE fused kernel
    gpu.begin()
    gpu.linear_fused_bf16(qkv_chain, tx, w, None, None, None, rows, width, n, 0)
    gpu.grouped_qkv_rope_bf16(*chain, qkv_chain, tqn, tkn, tc, ts, rows, heads, dim, half, 1e-5)
    gpu.submit()
    stored = qkv_fused.read()
    assert (stored == qkv_chain.read()).all()
    for a, b in zip(fused, chain):
        assert (a.read() == b.read()).all()
    want = oracle.grouped_qkv_rope(stored.reshape(rows, n), q_norm, k_norm, cos, sin, heads, dim, half, 1e-5)
    for a, e in zip(fused, want):
        check_bf16(a.read(), e.ravel())
    # without a qkv tensor the fused route still works; shapes it cannot fuse need one
    gpu.begin()
    gpu.grouped_qkv_linear_rope_bf16(*chain, None, tx, w, tqn, tkn, tc, ts, rows, width, heads, dim, half, 1e-5)
    gpu.submit()
    assert (chain[0].read() == fused[0].read()).all()
    gpu.free()


def test_quant_load_uses_the_artifact_cache(oracle, tmp_path):
    """h3_gpu_quant_configure(cache) + h3_gpu_quant_load (src/cuda/cuda_quant.cuh:292-333): the first load
    packs on the device and publishes an artifact, the second one is a cache hit with identical bytes."""
    rows, cols, group = 256, 384, 128
    w = synth.bf16_normal(90, 2, rows, cols, 0, 0.05).reshape(rows, cols)
    source = tmp_path / "weights.bf16"
    source.write_bytes(b"\0" * 64 + w.tobytes())
    want_q, want_s = oracle.q8_pack_rows(w, group)
    blobs = []
    for attempt in range(2):
        gpu = h.Gpu()
        gpu.set_group(group)
        gpu.quant_configure(1, cache=str(tmp_path / "cache" / "nested"))
        t = gpu.quant_load(str(source), 64, rows, cols)
        stats = gpu.stats()
        assert (stats.quant_cache_misses, stats.quant_cache_hits) == ((1, 0) if attempt == 0 else (0, 1))
        offset = (rows * cols + 15) & ~15
        blob = t.read(offset + want_s.size * 4, dtype=2)
        assert (blob[:rows * cols].reshape(rows, cols) == want_q).all()
        assert (blob[offset:].view(np.float32).view(np.uint32) == want_s.ravel().view(np.uint32)).all()
        blobs.append(blob)
        x = synth.activations(91, 1, 130, cols).reshape(130, cols)
        tx, out = gpu.tensor_from_bf16(x), gpu.tensor_new_bf16(130 * rows)
        gpu.begin()
        gpu.linear_bf16(out, tx, t, None, 130, cols, rows)
        gpu.submit()
        check_bf16(out.read().reshape(130, rows), oracle.linear(oracle.MODE_W8A16, x, want_q, want_s, group))
        with pytest.raises(h.H3Error):
            gpu.quant_load(str(source), 64, rows + 1, cols)        # shapes must be multiples of 128
        gpu.free()
    assert (blobs[0] == blobs[1]).all()
    assert len([f for f in os.listdir(tmp_path / "cache" / "nested") if f.endswith(".h3q8")]) == 1


def test_prepare_tool_builds_every_artifact(oracle, tmp_path):
    """h3q8_prepare (the job of src/weights/quant_prepare.c): walks a safetensors directory, publishes one
    artifact per DiT projection, and a second run finds all of them; a context then loads from the cache."""
    import subprocess
    from h3cli_b200 import build
    from safetensors_fixture import write_directory
    model, cache = tmp_path / "transformer", tmp_path / "cache"
    model.mkdir()
    written = write_directory(model)
    first = subprocess.run([build.PREPARE, "w8a16", str(model), str(cache), "64"], capture_output=True, text=True)
    assert first.returncode == 0, first.stderr
    assert "8 weights, 8 prepared, 0 already cached" in first.stderr
    assert len([f for f in os.listdir(cache) if f.endswith(".h3q8")]) == 8
    second = subprocess.run([build.PREPARE, "w8a16", str(model), str(cache), "64"], capture_output=True, text=True)
    assert second.returncode == 0 and "8 weights, 0 prepared, 8 already cached" in second.stderr
    gpu = h.Gpu()
    gpu.set_group(64)
    gpu.quant_configure(1, cache=str(cache))
    for name, (path, offset, w) in sorted(written.items())[:3]:
        rows, cols = w.shape
        t = gpu.quant_load(path, offset, rows, cols)
        want_q, want_s = oracle.q8_pack_rows(w, 64)
        blob = t.read(((rows * cols + 15) & ~15) + want_s.size * 4, dtype=2)
        assert (blob[:rows * cols].reshape(rows, cols) == want_q).all()
        assert (blob[(rows * cols + 15) & ~15:].view(np.float32).view(np.uint32) == want_s.ravel().view(np.uint32)).all()
    assert gpu.stats().quant_cache_hits == 3 and gpu.stats().quant_cache_misses == 0
    gpu.free()
    other = subprocess.run([build.PREPARE, "w8a16", str(model), str(cache), "128"], capture_output=True, text=True)
    assert other.returncode == 0 and "8 prepared" in other.stderr      # another scale group is another artifact


def test_profile_report_lines(oracle, monkeypatch, capfd):
    """H3_PROFILE: h3_gpu_profile_mark prints the placement / quant / transfer / category lines
    (src/cuda/gpu_cuda.cu:497-524), fed by the event categories 0, 4, 5 and 7; silent without the variable."""
    rows, cols, n = 512, 256, 384
    x = synth.activations(77, 1, rows, cols).reshape(rows, cols)
    w = synth.bf16_normal(78, 2, n, cols, 0, 0.05).reshape(n, cols)
    wq, ws = oracle.q8_pack_rows(w, 0)

    def run():
        gpu = h.Gpu()
        gpu.quant_configure(1)
        gpu.set_w8a16_scratch_rows(1)                  # the conversion category needs the dequantise-to-scratch policy
        h.library().h3_gpu_profile_set_label(gpu.handle, b"unit")
        weight = gpu.q8_from_host(wq, ws, 0)
        tx, out = gpu.tensor_new_bf16(rows * cols), gpu.tensor_new_bf16(rows * n)
        host = np.ascontiguousarray(x)
        back = np.zeros(rows * n, dtype=np.uint16)
        tx.upload_async(host.ctypes.data, host.nbytes)
        gpu.begin()
        gpu.linear_bf16(out, tx, weight, None, rows, cols, n)
        gpu.continue_()
        out.download_async(back.ctypes.data, back.nbytes)
        out.wait()
        gpu.submit()
        gpu.synchronize()
        gpu.plan_bf16_weights(0xFF, 1 << 20)
        gpu.begin()
        gpu.submit()                                   # harvests the copy events that finished after the first submit
        h.library().h3_gpu_profile_mark(gpu.handle, b"after block")
        stats = gpu.stats()
        check_bf16(back.reshape(rows, n), oracle.linear(oracle.MODE_W8A16, x, wq, ws, 0))
        gpu.free()
        return stats

    monkeypatch.delenv("H3_PROFILE", raising=False)
    capfd.readouterr()
    quiet = run()
    assert capfd.readouterr().err == "" and quiet.linear_seconds == 0
    monkeypatch.setenv("H3_PROFILE", "1")
    stats = run()
    err = capfd.readouterr().err
    assert "h3cli: weight placement after block: resident=8/8" in err
    assert "h3cli: quant profile unit / after block: mode=w8a16" in err
    assert "h3cli: CUDA profile unit / after block: wall" in err and "GEMM 1," in err
    assert "h3cli: CUDA category seconds: GEMM 0.0" in err and "h3cli: CUDA transfer events: H2D" in err
    assert stats.linear_seconds > 0 and stats.h2d_seconds > 0 and stats.d2h_seconds > 0 and stats.quant_conversion_seconds > 0


@pytest.mark.parametrize("rows,heads,dim,N", [(130, 3, 128, 256), (300, 6, 64, 384)])
def test_int8_head_major_projection(oracle, rows, heads, dim, N):
    """h3_gpu_linear_int8_head_major_bf16 (src/gpu.h:536-546): SDPA's [head, row, dimension] output is quantised per
    token straight into row-major int8 (no bf16 transpose) and projected; bit-equal to transposing on the host."""
    K, padded = heads * dim, (rows + 127) // 128 * 128
    x = synth.activations(71, 1, rows, K, outliers=synth.outlier_channels(71, K)).reshape(rows, K)
    head_major = np.ascontiguousarray(x.reshape(rows, heads, dim).transpose(1, 0, 2))
    wq, ws = synth.int8_weights(71, 2, N, K), synth.lognormal_scales(71, 3, N, 1)
    want_q, want_s = oracle.quantize_rows(x)
    want = oracle.linear(oracle.MODE_W8A8, want_q, wq, ws[:, 0].copy(), 0, x_scales=want_s, fast=True)
    gpu = h.Gpu()
    t_in, t_w, t_ws = gpu.tensor_from_bf16(head_major), gpu.tensor_from_i8(wq), gpu.tensor_from_f32(ws[:, 0].copy())
    q, sc, out = gpu.tensor_new_i8(padded * K), gpu.tensor_new_f32(padded), gpu.tensor_new_bf16(rows * N)
    gpu.begin()
    gpu.linear_int8_head_major_bf16(out, q, sc, t_in, t_w, t_ws, rows, heads, dim, N)
    gpu.submit()
    got_q = q.read().reshape(padded, K)
    assert (got_q[:rows] == want_q).all() and (got_q[rows:] == 0).all()
    assert (sc.read()[:rows].view(np.uint32) == want_s.view(np.uint32)).all() and (sc.read()[rows:] == 1.0).all()
    assert (out.read().reshape(rows, N) == want).all()
    with pytest.raises(h.H3Error):
        gpu.begin()
        gpu.linear_int8_head_major_bf16(out, q, sc, t_in, t_w, t_ws, 64, heads, dim, N)     # fewer than 128 rows
    gpu.cancel()
    gpu.free()


@pytest.mark.parametrize("row_fc2", [0, 1])
@pytest.mark.parametrize("rows,K,hidden,N", [(130, 256, 1024, 384), (300, 384, 2048, 256)])
def test_int8_mlp_operator(oracle, rows, K, hidden, N, row_fc2):
    """h3_gpu_mlp_int8_bf16 (src/gpu.h:547-563, src/metal/gpu.m:3281-3490): per-row int8 of the input, fc1 + SwiGLU,
    int8 of the activation per row and per 1024 features (or per row), fc2.  Each stage is checked against the oracle
    on the bytes the previous stage actually produced, so every comparison after the SwiGLU is bit-exact."""
    padded = (rows + 127) // 128 * 128
    x = synth.activations(81, 1, rows, K).reshape(rows, K)
    w1, s1 = synth.int8_weights(81, 2, 2 * hidden, K), synth.lognormal_scales(81, 3, 2 * hidden, 1) * np.float32(0.2)
    w2, s2 = synth.int8_weights(81, 4, N, hidden), synth.lognormal_scales(81, 5, N, 1)
    gpu = h.Gpu()
    t_x, t_w1, t_s1 = gpu.tensor_from_bf16(x), gpu.tensor_from_i8(w1), gpu.tensor_from_f32(s1[:, 0].copy())
    t_w2, t_s2 = gpu.tensor_from_i8(w2), gpu.tensor_from_f32(s2[:, 0].copy())
    q = gpu.tensor_new_i8(padded * max(K, hidden))
    sc = gpu.tensor_new_f32(padded * max(hidden // 1024, 1))
    act, out = gpu.tensor_new_bf16(rows * hidden), gpu.tensor_new_bf16(rows * N)
    before = h.library().h3q8_kernel_launches()
    gpu.begin()
    gpu.mlp_int8_bf16(out, act, q, sc, t_x, t_w1, t_s1, t_w2, t_s2, rows, K, hidden, N, use_int8_row_fc2=row_fc2)
    gpu.submit()
    assert h.library().h3q8_kernel_launches() - before == 4          # quantise, fc1 + SwiGLU, quantise, fc2
    xq, xs = oracle.quantize_rows(x)
    want_act = oracle.linear(oracle.MODE_W8A8, xq, w1, s1[:, 0].copy(), 0, x_scales=xs, activation=2, fast=True)
    got_act = act.read().reshape(rows, hidden)
    check_bf16(got_act, want_act)
    assert (got_act != want_act).mean() < 2e-3
    if row_fc2:
        aq, a_s = oracle.quantize_rows(got_act)
        want = oracle.linear(oracle.MODE_W8A8, aq, w2, s2[:, 0].copy(), 0, x_scales=a_s, fast=True)
        assert (q.read()[:rows * hidden].reshape(rows, hidden) == aq).all()
    else:
        aq, a_s = oracle.quantize_rows_grouped(got_act, 1024)
        want = oracle.linear(oracle.MODE_W8A8, aq, w2, s2[:, 0].copy(), 0, x_scales=a_s, input_group=1024, fast=True)
        assert (q.read()[:rows * hidden].reshape(rows, hidden) == aq).all()
        assert (sc.read()[:rows * (hidden // 1024)].view(np.uint32) == a_s.ravel().view(np.uint32)).all()
    assert (out.read().reshape(rows, N) == want).all()
    gpu.free()


def test_int8_qkv_projection_with_rope(oracle):
    """h3_gpu_grouped_qkv_linear_rope_int8 (src/gpu.h:682-702): per-row int8 of the input, int8 projection, per-head
    RMS norm and rotary embedding in the epilogue; equal bit for bit to the q8-descriptor route of the same weights,
    with and without a pre-quantised input."""
    rows, heads, width, half, dim = 300, 4, 512, 48, 128
    n, padded = heads * 3 * dim, 384
    rng = np.random.default_rng(5)
    bf = lambda a: synth.to_bf16(a.astype(np.float32)).reshape(a.shape)
    x, wq, ws = operands(91, rows, n, width, 0)
    q_norm, k_norm = bf(1 + 0.1 * rng.standard_normal(dim)), bf(1 + 0.1 * rng.standard_normal(dim))
    angle = rng.uniform(0, 6.28, (rows, half))
    cos, sin = bf(np.cos(angle)), bf(np.sin(angle))
    gpu = h.Gpu()
    gpu.quant_configure(2)
    tx, tqn, tkn, tc, ts = (gpu.tensor_from_bf16(a) for a in (x, q_norm, k_norm, cos, sin))
    w_desc = gpu.q8_from_host(wq, ws, 0)
    t_w, t_ws = gpu.tensor_from_i8(wq), gpu.tensor_from_f32(ws[:, 0].copy())
    reference = [gpu.tensor_new_bf16(rows * heads * dim) for _ in range(3)]
    first = [gpu.tensor_new_bf16(rows * heads * dim) for _ in range(3)]
    second = [gpu.tensor_new_bf16(rows * heads * dim) for _ in range(3)]
    qin, sc = gpu.tensor_new_i8(padded * width), gpu.tensor_new_f32(padded)
    gpu.begin()
    gpu.grouped_qkv_linear_rope_bf16(*reference, None, tx, w_desc, tqn, tkn, tc, ts, rows, width, heads, dim, half, 1e-5)
    gpu.grouped_qkv_linear_rope_int8(*first, qin, sc, tx, t_w, t_ws, tqn, tkn, tc, ts, rows, width, heads, dim, half, 1e-5)
    gpu.grouped_qkv_linear_rope_int8(*second, qin, sc, None, t_w, t_ws, tqn, tkn, tc, ts, rows, width, heads, dim, half, 1e-5,
                                     input_is_quantized=1)
    gpu.submit()
    want_q, want_s = oracle.quantize_rows(x)
    assert (qin.read()[:rows * width].reshape(rows, width) == want_q).all()
    for a, b, c in zip(reference, first, second):
        assert (a.read() == b.read()).all() and (a.read() == c.read()).all()
    linear = oracle.linear(oracle.MODE_W8A8, want_q, wq, ws[:, 0].copy(), 0, x_scales=want_s, fast=True)
    for got, want in zip(first, oracle.grouped_qkv_rope(linear, q_norm, k_norm, cos, sin, heads, dim, half, 1e-5)):
        check_bf16(got.read(), want.ravel())
    with pytest.raises(h.H3Error):
        gpu.begin()
        gpu.grouped_qkv_linear_rope_int8(*first, qin, sc, tx, t_w, t_ws, tqn, tkn, tc, ts, rows, width, heads, 64, 32, 1e-5)
    gpu.cancel()
    gpu.free()


def test_residency_plan_on_the_device(monkeypatch):
    """h3_gpu_plan_bf16_weights (src/cuda/gpu_cuda.cu:559-578): free memory and reserve come from the device;
    the test-only block ceiling and capacity turn the same request into partial and streamed plans."""
    block, mask = 64 << 20, (1 << 48) - 1
    gpu = h.Gpu()
    plan = gpu.plan_bf16_weights(mask, block, future_bytes=1 << 30)
    stats = gpu.stats()
    assert plan.effective_mode == 1 and plan.resident_count == 48 and plan.slot_bytes == 0
    assert (stats.resident_blocks, stats.active_weight_blocks, stats.resident_block_mask) == (48, 48, mask)
    assert stats.resident_weight_bytes == 48 * block and plan.reserve_bytes >= 1 << 30
    partial = gpu.plan_bf16_weights(mask, block, retry_cap=5)
    assert partial.effective_mode == 0 and partial.resident_mask == 0x1F and partial.slot_bytes == 2 * block
    streamed = gpu.plan_bf16_weights(mask, block, force_stream=1)
    assert streamed.effective_mode == 2 and streamed.resident_count == 0 and gpu.stats().stream_slot_bytes == 2 * block
    assert not h.library().h3_gpu_should_retry_streaming(gpu.handle)
    with pytest.raises(h.H3Error, match="two-slot streaming"):
        gpu.plan_bf16_weights(mask, 1 << 40)
    assert h.library().h3_gpu_weight_plan_compatible(gpu.handle, 0) == 0   # last accepted plan was constrained
    gpu.free()
    capacity = plan.reserve_bytes + 40 * block   # the visible capacity has to cover the reserve first
    monkeypatch.setenv("H3_TEST_CUDA_RESIDENT_BLOCKS", "3")
    monkeypatch.setenv("H3_TEST_CUDA_CAPACITY_BYTES", str(capacity))
    gpu = h.Gpu()
    plan = gpu.plan_bf16_weights(mask, block)
    assert plan.resident_count == 3 and plan.free_bytes <= capacity and plan.options.max_resident == 3
    monkeypatch.setenv("H3_TEST_CUDA_RESIDENT_BLOCKS", "50")
    roomy = h.Gpu()
    assert roomy.plan_bf16_weights(mask, block).resident_count in (37, 38)   # 40 blocks of budget minus two slots (minus live bytes)
    roomy.free()
    monkeypatch.setenv("H3_TEST_CUDA_RESIDENT_BLOCKS", "3")
    assert h.library().h3_gpu_weight_plan_compatible(gpu.handle, 0) == 0
    monkeypatch.setenv("H3_TEST_CUDA_RESIDENT_BLOCKS", "4")
    assert h.library().h3_gpu_weight_plan_compatible(gpu.handle, 0) == 0   # options differ from the context's
    gpu.free()
    monkeypatch.setenv("H3_CUDA_WEIGHT_MODE", "bogus")
    with pytest.raises(h.H3Error, match="auto, resident, or stream"):
        h.Gpu()


# --------------------------------------------------------------------------- weight streaming
def pinned_bytes(gpu, count):
    import ctypes
    host = gpu.tensor_alloc(count, 2, 2)   # int8, H3_GPU_HOST_PINNED
    pointer = h.library().h3_gpu_tensor_contents(host.handle)
    view = np.ctypeslib.as_array((ctypes.c_uint8 * count).from_address(pointer))
    return host, pointer, view


def test_weight_stream_slots_filled_by_the_callers_stream(oracle):
    """h3q8_gpu_weight_stream_reserve / _publish: a producer stream of the caller (here torch copies standing in
    for an all-gather of per-rank slices) fills the slots; compute waits for publish, the producer for release."""
    import torch
    M, K, N, group, layers = 200, 256, 384, 128, 7
    gpu = h.Gpu()
    gpu.quant_configure(1)
    x = synth.activations(40, 1, M, K).reshape(M, K)
    weights = [(synth.int8_weights(40 + l, 2, N, K), synth.lognormal_scales(40 + l, 3, N, K // group)) for l in range(layers)]
    blobs = [torch.from_numpy(h.q8_blob(wq, ws, group)).pin_memory() for wq, ws in weights]
    slot_bytes = blobs[0].numel()
    ring = gpu.weight_stream(slot_bytes, 2)
    producer = torch.cuda.Stream()

    class Bytes:
        def __init__(self, pointer, count):
            self.__cuda_array_interface__ = {"shape": (count,), "typestr": "|u1", "data": (pointer, False), "version": 2}

    def fill(layer):
        with torch.cuda.stream(producer):
            slot, address = ring.reserve(producer.cuda_stream)
            half = slot_bytes // 2 // 256 * 256                        # two "slices" written separately
            target = torch.as_tensor(Bytes(address, slot_bytes), device="cuda")
            target[:half].copy_(blobs[layer][:half], non_blocking=True)
            target[half:].copy_(blobs[layer][half:], non_blocking=True)
            ring.publish(slot, producer.cuda_stream, slot_bytes)
        return slot

    tx = gpu.tensor_from_bf16(x)
    outs = [gpu.tensor_new_bf16(M * N) for _ in range(layers)]
    views = []
    slot = fill(0)
    gpu.begin()
    for layer in range(layers):
        upcoming = fill(layer + 1) if layer + 1 < layers else None
        ring.acquire(slot)
        views.append(ring.view(slot, 0, N, K, group))
        gpu.linear_fused_bf16(outs[layer], tx, views[-1], None, None, None, M, K, N, 0)
        ring.release(slot)
        gpu.continue_()
        slot = upcoming
    gpu.submit()
    torch.cuda.synchronize()
    for layer, (wq, ws) in enumerate(weights):
        check_bf16(outs[layer].read().reshape(M, N), oracle.linear(oracle.MODE_W8A16, x, wq, ws, group))
    assert gpu.stats().streamed_bytes == layers * slot_bytes
    with pytest.raises(h.H3Error):
        ring.publish(0, producer.cuda_stream, slot_bytes + 1)
    gpu.free()


def test_weight_streaming_double_buffered(oracle):
    """Config 5 in miniature: packed group-128 layers streamed from pinned host memory
    through two device slots, one layer prefetched while the previous one computes
    (slot handoffs as in the reference's tests/test_cuda_runtime.c)."""
    M, K, N1, N2, group, layers = 300, 256, 512, 256, 128, 9
    gpu = h.Gpu()
    gpu.quant_configure(1)
    x = synth.activations(30, 1, M, K).reshape(M, K)
    weights, blobs = [], []
    for layer in range(layers):
        wq1, ws1 = synth.int8_weights(30 + layer, 2, N1, K), synth.lognormal_scales(30 + layer, 3, N1, K // group)
        wq2, ws2 = synth.int8_weights(30 + layer, 4, N2, N1), synth.lognormal_scales(30 + layer, 5, N2, N1 // group)
        first, second = h.q8_blob(wq1, ws1, group), h.q8_blob(wq2, ws2, group)
        weights.append((wq1, ws1, wq2, ws2, first.size))
        blobs.append(np.concatenate([first, second]))
    slot_bytes = blobs[0].size
    host, pointer, view = pinned_bytes(gpu, layers * slot_bytes)
    for layer, blob in enumerate(blobs):
        view[layer * slot_bytes:(layer + 1) * slot_bytes] = blob
    stream = gpu.weight_stream(slot_bytes, 2)
    with pytest.raises(h.H3Error):
        stream.prefetch(pointer, slot_bytes + 1)
    tx = gpu.tensor_from_bf16(x)
    mids = [gpu.tensor_new_bf16(M * N1) for _ in range(layers)]
    outs = [gpu.tensor_new_bf16(M * N2) for _ in range(layers)]
    views = []
    slot = stream.prefetch(pointer, slot_bytes)
    gpu.begin()
    for layer in range(layers):
        upcoming = stream.prefetch(pointer + (layer + 1) * slot_bytes, slot_bytes) if layer + 1 < layers else None
        stream.acquire(slot)
        w1 = stream.view(slot, 0, N1, K, group)
        w2 = stream.view(slot, weights[layer][4], N2, N1, group)
        gpu.linear_fused_bf16(mids[layer], tx, w1, None, None, None, M, K, N1, h.ACT_GELU_TANH)
        gpu.linear_fused_bf16(outs[layer], mids[layer], w2, None, None, None, M, N1, N2, 0)
        stream.release(slot)
        gpu.continue_()
        views += [w1, w2]
        slot = upcoming
    gpu.submit()
    for layer in range(layers):
        wq1, ws1, wq2, ws2, _ = weights[layer]
        mid = mids[layer].read().reshape(M, N1)
        check_bf16(mid, oracle.linear(oracle.MODE_W8A16, x, wq1, ws1, group, activation=1))
        check_bf16(outs[layer].read().reshape(M, N2), oracle.linear(oracle.MODE_W8A16, mid, wq2, ws2, group))
    stats = gpu.stats()
    assert stats.streamed_bytes == layers * slot_bytes and stats.stream_slot_bytes == 2 * slot_bytes
    for t in views + mids + outs + [tx]:
        t.free()
    stream.free()
    assert gpu.stats().stream_slot_bytes == 0
    host.free()
    gpu.free()


def test_config5_full_rows_streamed_layers(oracle):
    """Config 5 at its full row count: M = 219 600 tokens, hidden 3072, FFN 12288, W8A16 group-128 weights streamed
    layer by layer from pinned host memory through two device slots (two layers here: attention output with gate and
    residual, then FFN-up with GELU and FFN-down with gate and residual).  24 sampled rows per projection against the
    oracle; the concatenation property of row sharding is covered by test_config1_single_w8a16."""
    M, H, F, group = 219600, 3072, 12288, 128
    gpu = h.Gpu()
    gpu.quant_configure(1)
    rng = np.random.default_rng(55)
    def bf16(shape, mean=0.0, std=1.0):
        return synth.to_bf16(rng.standard_normal(shape, dtype=np.float32) * np.float32(std) + np.float32(mean)).reshape(shape)
    x, res, gate = bf16((M, H)), bf16((M, H)), bf16((H,), 1.0, 0.1)
    specs = [[(H, H)], [(F, H), (H, F)]]                    # layer 0: out projection; layer 1: FFN-up, FFN-down
    blobs, weights = [], []
    for layer, shapes in enumerate(specs):
        parts, kept = [], []
        for i, (n, k) in enumerate(shapes):
            wq, ws = synth.int8_weights(60 + layer, 2 + i, n, k), synth.lognormal_scales(60 + layer, 6 + i, n, k // group)
            blob = h.q8_blob(wq, ws, group)
            kept.append((wq, ws, sum(part.size for part in parts)))
            parts.append(np.concatenate([blob, np.zeros(-blob.size % 256, np.uint8)]))
        blobs.append(np.concatenate(parts))
        weights.append(kept)
    slot_bytes = max(blob.size for blob in blobs)
    host, pointer, view = pinned_bytes(gpu, len(blobs) * slot_bytes)
    for layer, blob in enumerate(blobs):
        view[layer * slot_bytes:layer * slot_bytes + blob.size] = blob
    stream = gpu.weight_stream(slot_bytes, 2)
    tx, tres, tgate = gpu.tensor_from_bf16(x), gpu.tensor_from_bf16(res), gpu.tensor_from_bf16(gate)
    attn, hidden, down = gpu.tensor_new_bf16(M * H), gpu.tensor_new_bf16(M * F), gpu.tensor_new_bf16(M * H)
    views = []
    slot = stream.prefetch(pointer, slot_bytes)
    gpu.begin()
    upcoming = stream.prefetch(pointer + slot_bytes, slot_bytes)
    stream.acquire(slot)
    w_out = stream.view(slot, weights[0][0][2], H, H, group)
    gpu.linear_fused_bf16(attn, tx, w_out, None, tgate, tres, M, H, H, 0)
    stream.release(slot)
    gpu.continue_()
    stream.acquire(upcoming)
    w_up = stream.view(upcoming, weights[1][0][2], F, H, group)
    w_down = stream.view(upcoming, weights[1][1][2], H, F, group)
    gpu.linear_fused_bf16(hidden, attn, w_up, None, None, None, M, H, F, h.ACT_GELU_TANH)
    gpu.linear_fused_bf16(down, hidden, w_down, None, tgate, attn, M, F, H, 0)
    stream.release(upcoming)
    gpu.submit()
    views += [w_out, w_up, w_down]
    rows = sample_rows(M, 24, 5)
    got_attn, got_hidden, got_down = (t.read().reshape(M, -1)[rows] for t in (attn, hidden, down))
    check_bf16(got_attn, oracle.linear(oracle.MODE_W8A16, x[rows], weights[0][0][0], weights[0][0][1], group, gate=gate, residual=res[rows]))
    check_bf16(got_hidden, oracle.linear(oracle.MODE_W8A16, got_attn, weights[1][0][0], weights[1][0][1], group, activation=1))
    check_bf16(got_down, oracle.linear(oracle.MODE_W8A16, got_hidden, weights[1][1][0], weights[1][1][1], group, gate=gate, residual=got_attn))
    assert gpu.stats().streamed_bytes == 2 * slot_bytes
    for t in views + [tx, tres, tgate, attn, hidden, down]:
        t.free()
    stream.free()
    host.free()
    gpu.free()


# --------------------------------------------------------------------------- interface behaviour
def test_int8_operator_family_like_the_reference(oracle):
    """h3_gpu_quantize_weight_int8 + h3_gpu_linear_int8_bf16 (src/metal/gpu.m:3174-3249):
    per-channel weight scales from the row quantiser, caller-owned scratch padded
    to 128 rows, rejects rows < 128 and K/N not multiples of 128."""
    M, N, K = 200, 256, 384
    x = synth.activations(60, 1, M, K).reshape(M, K)
    wb = synth.bf16_normal(60, 2, N, K, 0, 0.05).reshape(N, K)
    gpu = h.Gpu()
    tw, wq, wsc = gpu.tensor_from_bf16(wb), gpu.tensor_new_i8(N * K), gpu.tensor_new_f32(N)
    tx, out = gpu.tensor_from_bf16(x), gpu.tensor_new_bf16(M * N)
    qin, qs = gpu.tensor_new_i8(256 * K), gpu.tensor_new_f32(256)
    gpu.begin()
    gpu.quantize_weight_int8(wq, wsc, tw, N, K)
    gpu.linear_int8_bf16(out, qin, qs, tx, wq, wsc, M, K, N)
    gpu.submit()
    want_wq, want_ws = oracle.quantize_rows(wb)
    assert (wq.read().reshape(N, K) == want_wq).all() and (wsc.read() == want_ws).all()
    want_xq, want_xs = oracle.quantize_rows(x, 256)
    assert (qin.read().reshape(256, K) == want_xq).all() and (qs.read() == want_xs).all()
    want = oracle.linear(oracle.MODE_W8A8, want_xq[:M], want_wq, want_ws, 0, x_scales=want_xs[:M])
    assert (out.read().reshape(M, N) == want).all()
    gpu.begin()
    for bad in ((100, K, N), (M, K + 64, N), (M, K, N + 64)):
        with pytest.raises(h.H3Error):
            gpu.linear_int8_bf16(out, qin, qs, tx, wq, wsc, *bad)
    gpu.cancel()
    gpu.free()


def test_command_scope_and_errors():
    gpu = h.Gpu()
    assert gpu.backend_name() == "cuda-b200-q8"
    x = gpu.tensor_from_bf16(np.zeros(64, np.uint16))
    w = gpu.tensor_from_bf16(np.zeros(64 * 64, np.uint16))
    out = gpu.tensor_new_bf16(64)
    with pytest.raises(h.H3Error, match="requires h3_gpu_begin"):
        gpu.linear_bf16(out, x, w, None, 1, 64, 64)
    gpu.begin()
    with pytest.raises(h.H3Error, match="already active"):
        gpu.begin()
    gpu.linear_bf16(out, x, w, None, 1, 64, 64)
    gpu.submit()
    other = h.Gpu()
    foreign = other.tensor_new_bf16(64)
    gpu.begin()
    with pytest.raises(h.H3Error, match="another context"):
        gpu.linear_bf16(foreign, x, w, None, 1, 64, 64)
    with pytest.raises(h.H3Error):
        gpu.linear_bf16(out, x, w, None, 0, 64, 64)
    gpu.cancel()
    gpu.begin()          # the context is reusable after cancel
    gpu.submit()
    other.free()
    gpu.free()


@pytest.mark.parametrize("poison", [0x7FC0, 0x7F80, 0xFF80, 0xFFC1])
def test_nonfinite_activation_reported_at_submit(oracle, poison):
    """tests/quant_native.c:64-74 (which injects 0x7fc0, a NaN): a non-finite input, NaN or Inf of either sign,
    fails at submit, and cancel recovers."""
    M, N, K = 128, 128, 128
    x, wq, ws = operands(70, M, N, K, 0)
    gpu = h.Gpu()
    gpu.quant_configure(2)
    w = gpu.q8_from_host(wq, ws, 0)
    bad = x.copy()
    bad[5, 7] = poison
    tx, out = gpu.tensor_from_bf16(bad), gpu.tensor_new_bf16(M * N)
    gpu.begin()
    gpu.linear_fused_bf16(out, tx, w, None, None, None, M, K, N, 0)
    with pytest.raises(h.H3Error, match="non-finite"):
        gpu.submit()
    gpu.cancel()
    tx.write(x)
    gpu.begin()
    gpu.linear_fused_bf16(out, tx, w, None, None, None, M, K, N, 0)
    gpu.submit()
    xq, xs = oracle.quantize_rows(x)
    assert (out.read().reshape(M, N) == oracle.linear(oracle.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, x_scales=xs)).all()
    gpu.free()


@pytest.mark.parametrize("poison", [0x7FC0, 0x7F80])
def test_nonfinite_weight_is_rejected_and_never_cached(poison, tmp_path):
    """src/weights/q8.c:38-41 rejects NaN and Inf weights alike: h3_gpu_q8_load and h3_gpu_quant_load fail on
    either, no artifact is published, and the raw device packer / row quantiser report it in the status word."""
    rows, cols = 128, 256
    w = synth.bf16_normal(95, 2, rows, cols, 0, 0.05).reshape(rows, cols)
    w[77, 130] = poison
    source = tmp_path / "poisoned.bf16"
    source.write_bytes(w.tobytes())
    gpu = h.Gpu()
    with pytest.raises(h.H3Error, match="non-finite"):
        gpu.q8_load(str(source), 0, rows, cols)
    gpu.quant_configure(1, cache=str(tmp_path / "cache"))
    with pytest.raises(h.H3Error, match="non-finite"):
        gpu.quant_load(str(source), 0, rows, cols)
    assert not [f for f in os.listdir(tmp_path / "cache") if f.endswith(".h3q8")] if os.path.isdir(tmp_path / "cache") else True
    lib = h.library()
    src, q, sc = gpu.tensor_from_bf16(w), gpu.tensor_new_i8(rows * cols), gpu.tensor_new_f32(rows * 4)
    assert gpu.raw_status() == 0
    assert lib.h3q8_q8_pack_rows_device(src.device_pointer, q.device_pointer, sc.device_pointer, rows, cols, 64, gpu.stream)
    assert gpu.raw_status() & 0x80000000 and b"non-finite" in lib.h3q8_last_error()
    assert gpu.raw_status() == 0                                            # reading clears it
    assert lib.h3q8_quantize_rows(src.device_pointer, q.device_pointer, sc.device_pointer, rows, rows, cols, 1.0, gpu.stream)
    assert gpu.raw_status() & 0x80000000
    gpu.free()


def test_quant_diagnostics_and_activation_clip(oracle, monkeypatch):
    """H3_QUANT_DIAGNOSTICS=1 (src/cuda/cuda_quant.cuh:72-87, 156; counters of src/gpu.h:131) counts values the quantiser
    clipped and non-zero values it turned into 0; H3_INT8_ACTIVATION_CLIP (src/metal/gpu.m:3379-3384) shrinks the range
    of the MLP's row quantisers, which is what makes clipping possible at all."""
    rows, K, hidden, N = 130, 256, 1024, 256
    x = synth.activations(83, 1, rows, K, outliers=synth.outlier_channels(83, K)).reshape(rows, K)
    w1, s1 = synth.int8_weights(83, 2, 2 * hidden, K), synth.lognormal_scales(83, 3, 2 * hidden, 1) * np.float32(0.2)
    w2, s2 = synth.int8_weights(83, 4, N, hidden), synth.lognormal_scales(83, 5, N, 1)
    padded = 256

    def run(clip):
        if clip is None:
            monkeypatch.delenv("H3_INT8_ACTIVATION_CLIP", raising=False)
        else:
            monkeypatch.setenv("H3_INT8_ACTIVATION_CLIP", str(clip))
        gpu = h.Gpu()
        t_x, t_w1, t_s1 = gpu.tensor_from_bf16(x), gpu.tensor_from_i8(w1), gpu.tensor_from_f32(s1[:, 0].copy())
        t_w2, t_s2 = gpu.tensor_from_i8(w2), gpu.tensor_from_f32(s2[:, 0].copy())
        q, sc = gpu.tensor_new_i8(padded * hidden), gpu.tensor_new_f32(padded)
        act, out = gpu.tensor_new_bf16(rows * hidden), gpu.tensor_new_bf16(rows * N)
        gpu.begin()
        gpu.mlp_int8_bf16(out, act, q, sc, t_x, t_w1, t_s1, t_w2, t_s2, rows, K, hidden, N, use_int8_row_fc2=1)
        gpu.submit()
        stats, scales = gpu.stats(), sc.read()[:rows].copy()
        gpu.free()
        return stats, scales

    monkeypatch.setenv("H3_QUANT_DIAGNOSTICS", "1")
    plain, plain_scales = run(None)
    assert plain.quant_clipped_values == 0 and plain.quant_zeroed_values > 0           # outlier rows push small values to 0
    clipped, clipped_scales = run(0.5)
    assert clipped.quant_clipped_values > 0
    # what is left in the scale buffer are the fc2-input scales = clip * max|activated| / 127; the activations themselves
    # moved a little because the fc1 input was clipped too, so the halving is approximate
    ratio = clipped_scales / plain_scales
    assert 0.3 < np.median(ratio) < 0.7
    xq, _ = oracle.quantize_rows(x)
    assert plain.quant_zeroed_values >= int(((xq == 0) & (synth.from_bf16(x) != 0)).sum())   # at least the MLP input's
    monkeypatch.delenv("H3_QUANT_DIAGNOSTICS")
    quiet, _ = run(None)
    assert quiet.quant_clipped_values == 0 and quiet.quant_zeroed_values == 0           # off: no scan, no counts


def test_allocation_budget_fault_injection(monkeypatch):
    """Host-side fault injection as in the reference (H3_CUDA_TEST_MEMORY_BUDGET,
    src/weights/residency.c:31-32): allocations beyond the budget fail cleanly and
    the planner answers 'streamed' or 'insufficient' without touching the device."""
    monkeypatch.setenv("H3_CUDA_TEST_MEMORY_BUDGET", str(1 << 20))
    gpu = h.Gpu()
    small = gpu.tensor_new_bf16(1024)
    with pytest.raises(h.H3Error, match="out of memory"):
        gpu.tensor_new_bf16(1 << 20)
    lib = h.library()
    assert lib.h3_gpu_plan_weights(gpu.handle, 1 << 10, 1 << 10) == 0
    assert lib.h3_gpu_plan_weights(gpu.handle, 1 << 30, 1 << 10) == 1
    assert lib.h3_gpu_plan_weights(gpu.handle, 1 << 10, 1 << 30) == -1
    small.free()
    gpu.free()


def test_launch_counter_moves(gpu):
    before = h.library().h3q8_kernel_launches()
    x, wq, ws = operands(80, 128, 128, 128, 0)
    raw_linear(gpu, h.MODE_W8A16, x, wq, ws, 0, kernel=h.KERNEL_TCGEN05)
    assert h.library().h3q8_kernel_launches() == before + 1
