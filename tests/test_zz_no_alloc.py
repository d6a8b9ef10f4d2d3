"""h3q8_linear_w8a8_static -- the projection for callers that are not allowed to
allocate GPU memory (see include/h3q8.h).  Collected last on purpose: a run that
stops at the first failure has then already run every other test.

The entry point must give the same bits as the regular route (h3q8_quantize_rows
into caller-owned scratch, then h3q8_linear in W8A8 mode), call after call, even
though all calls share one built-in scratch array that keeps whatever the
previous call left in it; both are also held against the CPU checker.
"""
import ctypes

import numpy as np
import pytest

import h3cli_b200 as h
from h3cli_b200 import synth
from parity import check_bf16

pytestmark = pytest.mark.gpu


def regular_route(gpu, lib, x, wq, ws, bias, gate, res, activation):
    M, K = x.shape
    N = wq.shape[0]
    t = dict(x=gpu.tensor_from_bf16(x), w=gpu.tensor_from_i8(wq), ws=gpu.tensor_from_f32(ws), b=gpu.tensor_from_bf16(bias),
             g=gpu.tensor_from_bf16(gate), r=gpu.tensor_from_bf16(res), q=gpu.tensor_new_i8(M * K), s=gpu.tensor_new_f32(M),
             out=gpu.tensor_new_bf16(M * N))
    assert lib.h3q8_quantize_rows(t["x"].device_pointer, t["q"].device_pointer, t["s"].device_pointer, M, M, K, 1.0, gpu.stream)
    gpu.raw_linear(mode=h.MODE_W8A8, rows=M, input_dim=K, output_dim=N, input=t["q"], input_scales=t["s"], weight=t["w"],
                   weight_scales=t["ws"], bias=t["b"], gate=t["g"], residual=t["r"], activation=activation, output=t["out"],
                   kernel=h.KERNEL_TCGEN05)
    assert gpu.raw_status() == 0
    out = t["out"].read().reshape(M, N)
    for tensor in t.values():
        tensor.free()
    return out


def static_route(gpu, lib, x, wq, ws, bias, gate, res, activation):
    M, K = x.shape
    N = wq.shape[0]
    t = dict(x=gpu.tensor_from_bf16(x), w=gpu.tensor_from_i8(wq), ws=gpu.tensor_from_f32(ws), b=gpu.tensor_from_bf16(bias),
             g=gpu.tensor_from_bf16(gate), r=gpu.tensor_from_bf16(res), out=gpu.tensor_from_bf16(np.full(M * N + 64, 0x3F80, np.uint16)),
             status=gpu.tensor_from_u32(np.zeros(1, np.uint32)))
    d = h.LinearDesc(mode=h.MODE_W8A8, rows=M, input_dim=K, output_dim=N, input=t["x"].device_pointer,
                     weight=t["w"].device_pointer, weight_scales=t["ws"].device_pointer, bias=t["b"].device_pointer,
                     gate=t["g"].device_pointer, residual=t["r"].device_pointer, activation=activation,
                     output=t["out"].device_pointer)
    assert lib.h3q8_linear_w8a8_static(ctypes.byref(d), t["status"].device_pointer, gpu.stream), lib.h3q8_last_error()
    gpu.synchronize()
    assert t["status"].read(dtype=3)[0] == 0
    got = t["out"].read()
    assert (got[M * N:] == 0x3F80).all()
    for tensor in t.values():
        tensor.free()
    return got[:M * N].reshape(M, N)


def test_static_scratch_entry_point_matches_regular_route(oracle):
    gpu = h.Gpu()
    lib = h.library()
    # two calls in a row: the second is smaller and uses different data, so anything the
    # first call left in the shared scratch would show up as a difference
    for seed, (M, N, K), activation in ((91, (300, 520, 512), h.ACT_GELU_TANH), (92, (129, 264, 256), h.ACT_NONE)):
        x = synth.activations(seed, 1, M, K, outliers=synth.outlier_channels(seed, K)).reshape(M, K)
        wq = synth.int8_weights(seed, 2, N, K)
        ws = synth.lognormal_scales(seed, 3, N, 1)[:, 0].copy()
        bias = synth.bf16_normal(seed, 4, 1, N, 0, 0.02)[0]
        gate = synth.bf16_normal(seed, 5, 1, N, 1, 0.1)[0]
        res = synth.bf16_normal(seed, 6, M, N).reshape(M, N)
        want = regular_route(gpu, lib, x, wq, ws, bias, gate, res, activation)
        got = static_route(gpu, lib, x, wq, ws, bias, gate, res, activation)
        assert (got == want).all(), f"{(got != want).sum()} of {got.size} outputs differ"
        # and against the CPU restatement of the reference's arithmetic: the fp32 epilogue is deterministic, so
        # without GELU the bits are equal; with GELU (hardware exponential) within the bf16 bar
        xq, xs = oracle.quantize_rows(x)
        expected = oracle.linear(oracle.MODE_W8A8, xq, wq, ws, 0, x_scales=xs, bias=bias, gate=gate, residual=res,
                                 activation=activation, fast=True)
        if activation == h.ACT_NONE:
            assert (got == expected).all()
        else:
            check_bf16(got, expected)
    # operands this entry point does not take are refused, not ignored
    scratch = gpu.tensor_new_bf16(16)
    for field, value in (("workspace", scratch.device_pointer), ("kernel", h.KERNEL_TCGEN05_PAIR)):
        bad = h.LinearDesc(mode=h.MODE_W8A8, rows=16, input_dim=16, output_dim=8, input=scratch.device_pointer,
                           weight=scratch.device_pointer, weight_scales=scratch.device_pointer, output=scratch.device_pointer)
        setattr(bad, field, value)
        assert lib.h3q8_linear_w8a8_static(ctypes.byref(bad), None, gpu.stream) == 0
    scratch.free()
    assert gpu.raw_status() == 0      # also reads the status word inside the built-in array
    # beyond the built-in scratch: refused with a clear message, nothing launched
    before = lib.h3q8_kernel_launches()
    dummy = gpu.tensor_new_bf16(16)
    too_big = h.LinearDesc(mode=h.MODE_W8A8, rows=8192, input_dim=4096, output_dim=256, input=dummy.device_pointer,
                           weight=dummy.device_pointer, weight_scales=dummy.device_pointer, output=dummy.device_pointer)
    assert lib.h3q8_linear_w8a8_static(ctypes.byref(too_big), None, gpu.stream) == 0
    assert b"exceed the built-in scratch" in lib.h3q8_last_error()
    too_many_rows = h.LinearDesc(mode=h.MODE_W8A8, rows=20000, input_dim=16, output_dim=256, input=dummy.device_pointer,
                                 weight=dummy.device_pointer, weight_scales=dummy.device_pointer, output=dummy.device_pointer)
    assert lib.h3q8_linear_w8a8_static(ctypes.byref(too_many_rows), None, gpu.stream) == 0
    assert lib.h3q8_kernel_launches() == before
    dummy.free()
    gpu.free()
