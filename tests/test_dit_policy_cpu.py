"""h3_quant_projection / h3_quant_projection_policy (src/weights/quant.c:22-40) without a GPU: pinned against the
reference's own quant.c compiled unmodified (oracle/_ref/libh3_quant_ref.so) on every name shape that matters."""
import ctypes
import itertools
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAMES = [None, b"", b"blocks", b"blocks.", b"blocks..attn.qkv_proj.weight", b"blocks.x.attn.qkv_proj.weight", b"block.3.attn.qkv_proj.weight",
         b"blocks.0.attn.qkv_proj.weight", b"blocks.0.attn.out_proj.weight", b"blocks.0.mlp.fc1.weight", b"blocks.0.mlp.fc2.weight",
         b"blocks.7.attn.qkv_proj.weight", b"blocks.49.mlp.fc2.weight", b"blocks.007.mlp.fc1.weight", b"blocks.12.mlp.fc1.weight.extra",
         b"blocks.12.mlp.fc1.bias", b"blocks.12.norm1.weight", b"blocks.12.attn.q_norm.weight", b"blocks.3attn.qkv_proj.weight",
         b"blocks.3.attn.qkv_proj.weight ", b"final.attn.qkv_proj.weight", b"blocks.00.mlp.fc2.weight", b"blocks.0.", b"blocks.01.attn.out_proj.weight"]


@pytest.fixture(scope="module")
def lib():
    from h3cli_b200 import build
    build.build()
    import h3cli_b200
    return h3cli_b200.library()


def test_projection_policy_known_answers(lib):
    assert lib.h3_quant_projection(b"blocks.3.attn.qkv_proj.weight", 2) == 2
    assert lib.h3_quant_projection(b"blocks.3.mlp.fc2.weight", 1) == 1
    assert lib.h3_quant_projection(b"blocks.3.norm1.weight", 1) == 0
    assert lib.h3_quant_projection(None, 1) == 0
    assert lib.h3_quant_projection_policy(b"blocks.0.mlp.fc1.weight", 1, 1) == 0      # adaptive cache keeps block 0 in bf16
    assert lib.h3_quant_projection_policy(b"blocks.0.mlp.fc1.weight", 1, 0) == 1
    assert lib.h3_quant_projection_policy(b"blocks.10.mlp.fc1.weight", 1, 1) == 1


def test_projection_policy_equals_the_reference_build(lib):
    path = os.path.join(ROOT, "oracle", "_ref", "libh3_quant_ref.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libh3_quant_ref.so was not built (no reference tree at build time)")
    ref = ctypes.CDLL(path)
    for f in (ref.h3_quant_projection, ref.h3_quant_projection_policy):
        f.restype = ctypes.c_int
    ref.h3_quant_projection.argtypes = [ctypes.c_char_p, ctypes.c_int]
    ref.h3_quant_projection_policy.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
    for name, requested in itertools.product(NAMES, (0, 1, 2)):
        assert lib.h3_quant_projection(name, requested) == ref.h3_quant_projection(name, requested), name
        for adaptive in (0, 1):
            assert lib.h3_quant_projection_policy(name, requested, adaptive) == ref.h3_quant_projection_policy(name, requested, adaptive), name
