"""Seeded synthetic operands for the DiT linear configurations.

Counter-based: element (row, column) of tensor `tensor_id` depends only on
(seed, tensor_id, row, column), so any rank regenerates exactly its own rows and
a checker regenerates any sampled row.  These tensors stand in for MiniMax-H3
activations and weights: bf16 N(0,1) activations, int8 weights uniform in
[-127,127], log-normal fp32 scales (median 0.01, sigma 0.3), bf16 N(0,0.02)
bias, bf16 N(1,0.1) gate.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix(x):
    """splitmix64 finaliser on uint64 arrays."""
    x = x.astype(np.uint64)
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return x ^ (x >> np.uint64(31))


def _counters(seed, tensor_id, rows, columns, row0, lane):
    with np.errstate(over="ignore"):
        key = _mix(np.array([seed], np.uint64) ^ _mix(np.array([tensor_id * 4 + lane + 1], np.uint64)))
        r = (np.arange(rows, dtype=np.uint64) + np.uint64(row0))[:, None]
        c = np.arange(columns, dtype=np.uint64)[None, :]
        return _mix((r * np.uint64(0x100000001B3) + c) ^ key)


def uniform(seed, tensor_id, rows, columns, row0=0, lane=0):
    """float64 in (0, 1)."""
    bits = _counters(seed, tensor_id, rows, columns, row0, lane)
    return ((bits >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def normal(seed, tensor_id, rows, columns, row0=0):
    """Box-Muller on two counter streams."""
    u1 = uniform(seed, tensor_id, rows, columns, row0, 0)
    u2 = uniform(seed, tensor_id, rows, columns, row0, 1)
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def to_bf16(values):
    """fp32 -> bf16 bits, round to nearest even on the raw bits."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + np.uint64(0x7FFF) + ((bits >> np.uint64(16)) & np.uint64(1))) & np.uint64(0xFFFFFFFF)
    return (bits >> np.uint64(16)).astype(np.uint16)


def from_bf16(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_normal(seed, tensor_id, rows, columns, mean=0.0, std=1.0, row0=0):
    return to_bf16((normal(seed, tensor_id, rows, columns, row0) * std + mean).astype(np.float32))


def int8_weights(seed, tensor_id, rows, columns):
    return (np.floor(uniform(seed, tensor_id, rows, columns) * 255.0) - 127.0).astype(np.int8)


def lognormal_scales(seed, tensor_id, rows, groups, median=0.01, sigma=0.3):
    return np.exp(normal(seed, tensor_id, rows, groups) * sigma + np.log(median)).astype(np.float32)


def outlier_channels(seed, columns, fraction=0.001):
    """Indices of the activation channels scaled x20 in the W8A8 configuration."""
    count = int(np.ceil(fraction * columns))
    order = np.argsort(_counters(seed, 9999, 1, columns, 0, 0)[0], kind="stable")
    return np.sort(order[:count])


def activations(seed, tensor_id, rows, columns, row0=0, outliers=None, factor=20.0):
    x = normal(seed, tensor_id, rows, columns, row0).astype(np.float32)
    if outliers is not None:
        x[:, outliers] *= factor
    return to_bf16(x)
