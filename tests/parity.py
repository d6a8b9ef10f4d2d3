"""Shared comparison helpers for the parity tests."""
import numpy as np


def bf16_to_f32(bits):
    return (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def rel_l2(actual_bits, expected_bits):
    a, e = bf16_to_f32(actual_bits).astype(np.float64), bf16_to_f32(expected_bits).astype(np.float64)
    return float(np.sqrt(((a - e) ** 2).sum() / max((e ** 2).sum(), 1e-30)))


def ulp_errors(actual_bits, expected_bits, floor):
    """|actual - expected| in bf16 ulps, the ulp taken at max(|expected|, floor).

    Outputs that are sums with cancellation can be far smaller than the terms
    that formed them; a different fp32 summation order then moves them by many
    of their own ulps although the sum is as accurate as it can be.  `floor` is
    the magnitude below which the ulp stops shrinking (the root-mean-square of
    the expected output unless a test states otherwise)."""
    a, e = bf16_to_f32(actual_bits).astype(np.float64), bf16_to_f32(expected_bits).astype(np.float64)
    magnitude = np.maximum(np.abs(e), floor)
    ulp = 2.0 ** (np.floor(np.log2(magnitude)) - 7)
    return np.abs(a - e) / ulp


def check_bf16(actual_bits, expected_bits, rel_limit=2e-3, ulp_limit=2.0, floor=None):
    """The parity bar for bf16 outputs: rel-L2 <= 2e-3 and max |delta| <= 2 bf16 ulp."""
    e = bf16_to_f32(expected_bits).astype(np.float64)
    if floor is None:
        floor = float(np.sqrt((e ** 2).mean())) or 1.0
    rel = rel_l2(actual_bits, expected_bits)
    worst = float(ulp_errors(actual_bits, expected_bits, floor).max())
    assert np.isfinite(bf16_to_f32(actual_bits)).all(), "non-finite output"
    assert rel <= rel_limit, f"rel-L2 {rel:.3e} > {rel_limit}"
    assert worst <= ulp_limit, f"max error {worst:.2f} bf16 ulp > {ulp_limit} (floor {floor:.3g})"
    return rel, worst
