"""Generates tests/golden/reference_kernels.npz: inputs and the outputs of the REFERENCE's own CUDA element
kernels (greg31337/h3cli src/cuda/cuda_kernels.cuh, compiled unmodified into oracle/_ref/libh3_cuda_kernels_ref.so
by oracle/Makefile) on small seeded cases.  Needs a CUDA GPU and that library; run once where both exist:

    python tests/golden/make_reference_kernel_golden.py

The CPU test suite then holds the CPU restatement under oracle/ to these outputs without a GPU
(tests/test_oracle_cpu.py::test_restatement_against_reference_cuda_kernel_outputs), with the same bounds the GPU
tests use next to the live kernels.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle as o  # noqa: E402
from h3cli_b200 import synth  # noqa: E402


def bf(a):
    a = np.asarray(a, np.float32)
    return synth.to_bf16(a).reshape(a.shape)


def main():
    ref = o.reference_cuda()
    if ref is None:
        raise SystemExit("oracle/_ref/libh3_cuda_kernels_ref.so is missing: make -C oracle REFERENCE=<tree>")
    out = {}
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    out["gelu_out"] = ref.gelu(bits, 1)
    for i, (rows, width, classes) in enumerate([(5, 256, 1), (7, 1000, 2)]):
        rng = np.random.default_rng(100 + i)
        res, branch = bf(rng.standard_normal((rows, width))), bf(rng.standard_normal((rows, width)) * 3)
        mod = bf(1 + 0.1 * rng.standard_normal((classes, 6, width)))
        row_map = (np.arange(rows) % classes).astype(np.uint32)
        out.update({f"gate{i}_res": res, f"gate{i}_branch": branch, f"gate{i}_mod": mod, f"gate{i}_map": row_map,
                    f"gate{i}_out": ref.gate(res, branch, mod, row_map, 6, 2)})
    rng = np.random.default_rng(110)
    fused = bf(rng.standard_normal((9, 2 * 192)) * 2.5)
    out.update({"swiglu_in": fused, "swiglu_out": ref.swiglu(fused)})
    for i, (rows, heads, half) in enumerate([(11, 2, 48), (6, 3, 64)]):
        rng = np.random.default_rng(120 + i)
        qkv = bf(rng.standard_normal((rows, heads * 3 * 128)) * 4)
        q_norm, k_norm = bf(1 + 0.1 * rng.standard_normal(128)), bf(1 + 0.1 * rng.standard_normal(128))
        angle = rng.uniform(0, 6.28, (rows, half))
        cos, sin = bf(np.cos(angle)), bf(np.sin(angle))
        q, k, v = ref.qkv_rope(qkv, q_norm, k_norm, cos, sin, heads, 128, half, 1e-5, grouped=1)
        out.update({f"rope{i}_qkv": qkv, f"rope{i}_qn": q_norm, f"rope{i}_kn": k_norm, f"rope{i}_cos": cos, f"rope{i}_sin": sin,
                    f"rope{i}_q": q, f"rope{i}_k": k, f"rope{i}_v": v})
    for i, (rows, width) in enumerate([(5, 256), (7, 1000), (6, 250)]):
        rng = np.random.default_rng(130 + i)
        res, branch = bf(rng.standard_normal((rows, width))), bf(rng.standard_normal((rows, width)))
        mod = bf(rng.standard_normal((2, 6, width)) * 0.1)
        norm_w = bf(1 + 0.1 * rng.standard_normal(width))
        row_map = (np.arange(rows) % 2).astype(np.uint32)
        gated = ref.gate(res, branch, mod, row_map, 6, 2)
        out.update({f"chain{i}_res": res, f"chain{i}_branch": branch, f"chain{i}_mod": mod, f"chain{i}_norm": norm_w,
                    f"chain{i}_map": row_map, f"chain{i}_gated": gated,
                    f"chain{i}_adaln": ref.adaln(gated, norm_w, mod, row_map, 6, 3, 4, 1e-5)})
    for i, (rows, k, n, with_bias) in enumerate([(1, 16, 8, True), (17, 128, 24, False), (31, 320, 40, True)]):
        x = synth.activations(3, 1, rows, k).reshape(rows, k)
        w = bf(np.random.default_rng(n).standard_normal((n, k)) * 0.05)
        bias = synth.bf16_normal(3, 4, 1, n, 0, 0.02)[0] if with_bias else np.zeros(0, np.uint16)
        out.update({f"linear{i}_x": x, f"linear{i}_w": w, f"linear{i}_bias": bias,
                    f"linear{i}_out": ref.linear(x, w, bias if with_bias else None)})
    path = os.path.join(HERE, "reference_kernels.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
