"""Generates the committed golden fixtures (run in the build container, where the
reference tree and oracle/_ref exist):

  q8_pack.npz   inputs and the outputs of the REFERENCE's own packer
                (src/weights/q8.c compiled unmodified into oracle/_ref) for the
                shapes and input generator of tests/metal_q8.c:89-141, plus the
                known-answer vector of tests/metal_q8.c:21-34.
  linear.npz    W8A16 group-64 linear outputs for the same shapes computed the
                way tests/metal_q8.c:124-133 computes its expectation (FP64 dot
                over bf16(q*scale), + bias, rounded to bf16), by oracle/h3q8_oracle.c
                on weights packed by the reference packer.
  w8a8.npz      per-token quantiser outputs and exact int32 accumulators for
                small W8A8 cases (pure integer arithmetic; numpy cross-checks
                the oracle before anything is written).

usage: python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle as o  # noqa: E402


def xorshift_floats(count, state, scale):
    """The input generator of tests/metal_q8.c:15 (xorshift32 -> [-1, 1] in steps of 1/4096)."""
    out = np.empty(count, np.float32)
    s = state
    for i in range(count):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        out[i] = np.float32((int(s % 8193) - 4096) / 4096.0) * np.float32(scale)
    return out, s


def main():
    ref = o.reference_q8()
    if ref is None:
        raise SystemExit("oracle/_ref/libh3q8_ref.so is missing: run `make -C oracle` where the reference tree exists")
    pack, linear = {}, {}
    # known-answer vector, tests/metal_q8.c:21-34
    values = np.zeros((1, 65), np.float32)
    values[0, :8] = [127, -127, .5, 1.5, 2.5, -.5, -1.5, -2.5]
    src = o.f32_to_bf16(values).reshape(1, 65)
    q = np.empty((1, 65), np.int8)
    s = np.empty((1, 2), np.float32)
    assert ref.h3_q8_pack_rows(src.ctypes.data, q.ctypes.data, s.ctypes.data, 1, 65)
    assert q[0, :8].tolist() == [127, -127, 0, 2, 2, 0, -2, -2] and (s == 1).all() and q[0, 64] == 0
    pack["known_src"], pack["known_q"], pack["known_s"] = src, q, s
    # operator shapes, tests/metal_q8.c:179-180: (m, n, k, large)
    for idx, (m, n, k, large) in enumerate([(1, 3, 1, 0), (17, 35, 65, 0), (65, 67, 129, 1), (129, 256, 256, 0)]):
        x, state = xorshift_floats(m * k, 12467, 262144.0 if large else 1.0)
        w, state = xorshift_floats(n * k, state, 0.125)
        xb = o.f32_to_bf16(x).reshape(m, k)
        wb = o.f32_to_bf16(w).reshape(n, k)
        groups = (k + 63) // 64
        q = np.empty((n, k), np.int8)
        s = np.empty((n, groups), np.float32)
        assert ref.h3_q8_pack_rows(wb.ctypes.data, q.ctypes.data, s.ctypes.data, n, k)
        bias = o.f32_to_bf16((np.arange(n) % 5).astype(np.float32) * 0.125)
        out = o.linear(o.MODE_W8A16, xb, q, s, 64, bias=bias)
        pack[f"src{idx}"], pack[f"q{idx}"], pack[f"s{idx}"] = wb, q, s
        linear[f"x{idx}"], linear[f"bias{idx}"], linear[f"out{idx}"] = xb, bias, out
    np.savez_compressed(os.path.join(HERE, "q8_pack.npz"), **pack)
    np.savez_compressed(os.path.join(HERE, "linear.npz"), **linear)
    # W8A8: quantiser + exact accumulators
    w8a8 = {}
    rng = np.random.default_rng(20251125)
    for idx, (m, n, k) in enumerate([(5, 16, 128), (130, 128, 256), (64, 24, 384)]):
        x = rng.standard_normal((m, k)).astype(np.float32)
        x[:, rng.integers(0, k, 2)] *= 20.0
        if idx == 0:
            x[2] = 0.0
        xb = o.f32_to_bf16(x).reshape(m, k)
        wq = rng.integers(-127, 128, (n, k)).astype(np.int8)
        ws = np.exp(rng.normal(np.log(0.01), 0.3, n)).astype(np.float32)
        xq, xs = o.quantize_rows(xb)
        out, acc = o.linear(o.MODE_W8A8, xq, wq, ws, 0, x_scales=xs, want_acc=True)
        assert (acc == xq.astype(np.int64) @ wq.astype(np.int64).T).all()
        for name, value in (("x", xb), ("wq", wq), ("ws", ws), ("xq", xq), ("xs", xs), ("acc", acc), ("out", out)):
            w8a8[f"{name}{idx}"] = value
    np.savez_compressed(os.path.join(HERE, "w8a8.npz"), **w8a8)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    main()
