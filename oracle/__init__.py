"""TEST INFRASTRUCTURE ONLY: ctypes binding of the CPU checker.

`oracle/h3q8_oracle.c` restates the reference's q8 linear arithmetic on the CPU;
`oracle/_ref/libh3q8_ref.so` is the reference's own `src/weights/q8.c` compiled
unmodified.  Only the test-suite, the smoke check and the benchmark's CPU
baseline may import this package; the shipped library never does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libh3q8_oracle.so")
_REF = os.path.join(_HERE, "_ref", "libh3q8_ref.so")

MODE_BF16, MODE_W8A16, MODE_W8A8 = 0, 1, 2
ACT_NONE, ACT_GELU_TANH, ACT_SWIGLU = 0, 1, 2


def _reference_tree():
    """Where the reference sources lie on this machine, or None: $H3_REFERENCE, else a `reference`
    directory beside the repository (the layout of the build container)."""
    for candidate in (os.environ.get("H3_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if candidate and os.path.isfile(os.path.join(candidate, "src", "weights", "q8.c")):
            return candidate
    return None


def build():
    """Compile the checker (and, when the reference tree is present, `_ref`)."""
    tree = _reference_tree()
    subprocess.run(["make", "-s", "-C", _HERE] + ([f"REFERENCE={tree}"] if tree else []), check=True,
                   stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL if not os.environ.get("H3_ORACLE_VERBOSE") else None)


class _Args(ctypes.Structure):
    _fields_ = [
        ("mode", ctypes.c_uint32), ("rows", ctypes.c_uint32),
        ("input_dim", ctypes.c_uint32), ("output_dim", ctypes.c_uint32),
        ("input", ctypes.c_void_p), ("weight", ctypes.c_void_p),
        ("weight_scales", ctypes.c_void_p), ("weight_group", ctypes.c_uint32),
        ("input_scales", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("gate", ctypes.c_void_p), ("residual", ctypes.c_void_p),
        ("activation", ctypes.c_uint32),
        ("output", ctypes.c_void_p), ("accumulators", ctypes.c_void_p),
        ("fast", ctypes.c_int), ("input_group", ctypes.c_uint32),
    ]


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            build()
        _lib = ctypes.CDLL(_LIB)
        _lib.h3o_q8_layout.argtypes = [ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
                                       ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
        _lib.h3o_q8_pack_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32]
        _lib.h3o_q8_dequant.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32]
        _lib.h3o_quantize_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_float]
        _lib.h3o_gelu_tanh_bf16.argtypes = [ctypes.c_uint16]
        _lib.h3o_gelu_tanh_bf16.restype = ctypes.c_uint16
        _lib.h3o_gate_residual_bf16.argtypes = [ctypes.c_uint16] * 3
        _lib.h3o_gate_residual_bf16.restype = ctypes.c_uint16
        _lib.h3o_f32_to_bf16.argtypes = [ctypes.c_float]
        _lib.h3o_f32_to_bf16.restype = ctypes.c_uint16
        _lib.h3o_bf16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.h3o_bf16_to_f32.restype = ctypes.c_float
        _lib.h3o_linear.argtypes = [ctypes.POINTER(_Args)]
    return _lib


def reference_q8():
    """The reference's own packer (src/weights/q8.c), or None if it was never built."""
    global _ref
    if _ref is None and os.path.exists(_REF):
        _ref = ctypes.CDLL(_REF)
        _ref.h3_q8_layout.argtypes = [ctypes.c_uint32, ctypes.c_uint32,
                                      ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
        _ref.h3_q8_pack_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                         ctypes.c_uint32, ctypes.c_uint32]
    return _ref


def _ptr(a):
    return None if a is None else a.ctypes.data


def f32_to_bf16(x):
    """Vectorised src/metal/shaders.metal:15-19."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFFFFFF
    return (bits >> 16).astype(np.uint16)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def q8_layout(rows, cols, group):
    off, total = ctypes.c_size_t(), ctypes.c_size_t()
    ok = lib().h3o_q8_layout(rows, cols, group, ctypes.byref(off), ctypes.byref(total))
    return (off.value, total.value) if ok else None


def q8_pack_rows(src_bf16, group):
    rows, cols = src_bf16.shape
    width = group or cols
    groups = (cols + width - 1) // width
    src = np.ascontiguousarray(src_bf16, dtype=np.uint16)
    q = np.empty((rows, cols), np.int8)
    s = np.empty((rows, groups), np.float32)
    if not lib().h3o_q8_pack_rows(_ptr(src), _ptr(q), _ptr(s), rows, cols, group):
        return None
    return q, s


def q8_dequant(q, s, group):
    rows, cols = q.shape
    out = np.empty((rows, cols), np.uint16)
    lib().h3o_q8_dequant(_ptr(np.ascontiguousarray(q)), _ptr(np.ascontiguousarray(s)), _ptr(out), rows, cols, group)
    return out


def quantize_rows(x_bf16, dispatch_rows=None, clip=1.0):
    rows, cols = x_bf16.shape
    dispatch_rows = dispatch_rows or rows
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    q = np.empty((dispatch_rows, cols), np.int8)
    s = np.empty((dispatch_rows,), np.float32)
    lib().h3o_quantize_rows(_ptr(x), _ptr(q), _ptr(s), rows, dispatch_rows, cols, clip)
    return q, s


def gate_adaln_quantize(residual, branch, gate_modulation, norm_weight, norm_modulation, row_map, padded_rows,
                        slots, gate_slot, shift_slot, scale_slot, epsilon):
    """Returns (gated_residual bf16 [M,W], normalized bf16 [M,W], int8 [padded,W], scales [padded])."""
    rows, width = residual.shape
    f = lib().h3o_gate_adaln_quantize
    f.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_uint32] * 7 + [ctypes.c_float]
    f.restype = None
    keep = [np.ascontiguousarray(a) if a is not None else None
            for a in (residual, branch, gate_modulation, row_map, norm_weight, norm_modulation)]
    gated, normalized = np.empty((rows, width), np.uint16), np.empty((rows, width), np.uint16)
    q, s = np.empty((padded_rows, width), np.int8), np.empty(padded_rows, np.float32)
    f(*[_ptr(a) for a in keep], _ptr(gated), _ptr(normalized), _ptr(q), _ptr(s), rows, padded_rows, width, slots,
      gate_slot, shift_slot, scale_slot, epsilon)
    return gated, normalized, q, s


def grouped_qkv_rope(qkv, q_weight, k_weight, rope_cos, rope_sin, heads, head_dim, rope_half, epsilon):
    rows = qkv.shape[0]
    f = lib().h3o_grouped_qkv_rope
    f.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_uint32] * 4 + [ctypes.c_float]
    f.restype = None
    keep = [np.ascontiguousarray(a) for a in (qkv, q_weight, k_weight, rope_cos, rope_sin)]
    out = [np.empty((rows, heads, head_dim), np.uint16) for _ in range(3)]
    f(*[_ptr(a) for a in keep], *[_ptr(a) for a in out], rows, heads, head_dim, rope_half, epsilon)
    return out


def gelu_tanh_bf16(b):
    f = lib().h3o_gelu_tanh_bf16
    return np.array([f(int(v)) for v in np.asarray(b, np.uint16).ravel()], np.uint16).reshape(np.shape(b))


def quantize_rows_grouped(x_bf16, group, dispatch_rows=None):
    """src/metal/shaders.metal:1552-1598: the row recipe on every `group` columns; scales [rows, K/group]."""
    rows, cols = x_bf16.shape
    dispatch_rows = dispatch_rows or rows
    groups = cols // group
    q, s = quantize_rows(np.ascontiguousarray(x_bf16).reshape(rows * groups, group), dispatch_rows * groups)
    return q.reshape(dispatch_rows, cols), s.reshape(dispatch_rows, groups)


def linear(mode, x, w, w_scales=None, group=0, x_scales=None, bias=None, gate=None,
           residual=None, activation=ACT_NONE, fast=False, want_acc=False, input_group=0):
    """out[M,N] (bf16 bits) = epilogue(x . w^T); see h3o_linear_args."""
    M, K = x.shape
    N = w.shape[0] // 2 if activation == ACT_SWIGLU else w.shape[0]
    keep = [np.ascontiguousarray(a) if a is not None else None
            for a in (x, w, w_scales, x_scales, bias, gate, residual)]
    out = np.empty((M, N), np.uint16)
    acc = np.empty((M, N), np.int32) if want_acc else None
    a = _Args(mode, M, K, N, _ptr(keep[0]), _ptr(keep[1]), _ptr(keep[2]), group, _ptr(keep[3]),
              _ptr(keep[4]), _ptr(keep[5]), _ptr(keep[6]), activation, _ptr(out), _ptr(acc), int(fast), input_group)
    if not lib().h3o_linear(ctypes.byref(a)):
        raise ValueError("oracle rejected the arguments")
    return (out, acc) if want_acc else out


# --------------------------------------------------------------------------- the reference's own CUDA element kernels
_REF_CUDA = os.path.join(_HERE, "_ref", "libh3_cuda_kernels_ref.so")
_ref_cuda = None


class ReferenceCuda:
    """src/cuda/cuda_kernels.cuh of the reference, compiled unmodified with its own flags
    (oracle/ref_cuda_kernels.cu), run on the current CUDA device.  Arrays in and out are numpy."""

    def __init__(self, library):
        self._lib = library
        for name in ("gelu_bf16", "gate_bf16", "adaln_bf16", "rms_norm_bf16", "qkv_rope_bf16", "swiglu_bf16", "add_bf16", "linear_bf16"):
            getattr(library, "h3ref_" + name).restype = ctypes.c_int

    @staticmethod
    def _check(ok, what):
        if not ok:
            raise RuntimeError(f"reference CUDA kernel {what} failed")

    def gelu(self, bits, approximate=1):
        bits = np.ascontiguousarray(bits, np.uint16)
        out = np.empty_like(bits)
        self._lib.h3ref_gelu_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32]
        self._check(self._lib.h3ref_gelu_bf16(_ptr(bits), _ptr(out), bits.size, approximate), "h3_gelu_bf16")
        return out

    def gate(self, residual, branch, modulation, row_map, slots, gate_slot):
        rows, width = residual.shape
        keep = [np.ascontiguousarray(a) for a in (residual, branch, modulation, np.asarray(row_map, np.uint32))]
        out = np.empty((rows, width), np.uint16)
        f = self._lib.h3ref_gate_bf16
        f.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_uint32] * 5
        self._check(f(*[_ptr(a) for a in keep], _ptr(out), rows, width, slots, gate_slot, keep[2].size // (slots * width)), "h3_gate_bf16")
        return out

    def adaln(self, x, norm_weight, modulation, row_map, slots, shift_slot, scale_slot, epsilon):
        rows, width = x.shape
        keep = [np.ascontiguousarray(a) for a in (x, norm_weight, modulation, np.asarray(row_map, np.uint32))]
        out = np.empty((rows, width), np.uint16)
        f = self._lib.h3ref_adaln_bf16
        f.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_uint32] * 5 + [ctypes.c_float, ctypes.c_uint32]
        self._check(f(*[_ptr(a) for a in keep], _ptr(out), rows, width, slots, shift_slot, scale_slot, epsilon,
                      keep[2].size // (slots * width)), "h3_adaln_bf16")
        return out

    def rms_norm(self, x, weight, epsilon):
        rows, width = x.shape
        keep = [np.ascontiguousarray(a) for a in (x, weight)]
        out = np.empty((rows, width), np.uint16)
        f = self._lib.h3ref_rms_norm_bf16
        f.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_uint32] * 2 + [ctypes.c_float]
        self._check(f(_ptr(keep[0]), _ptr(keep[1]), _ptr(out), rows, width, epsilon), "h3_rms_norm_bf16")
        return out

    def qkv_rope(self, qkv, q_weight, k_weight, rope_cos, rope_sin, heads, head_dim, rope_half, epsilon, grouped=1):
        rows = qkv.shape[0]
        keep = [np.ascontiguousarray(a) for a in (qkv, q_weight, k_weight, rope_cos, rope_sin)]
        out = [np.empty((rows, heads, head_dim), np.uint16) for _ in range(3)]
        f = self._lib.h3ref_qkv_rope_bf16
        f.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_uint32] * 5 + [ctypes.c_float]
        self._check(f(*[_ptr(a) for a in keep], *[_ptr(a) for a in out], rows, heads, head_dim, rope_half, grouped, epsilon),
                    "h3_qkv_rope_bf16")
        return out

    def swiglu(self, fused):
        rows, width = fused.shape[0], fused.shape[1] // 2
        fused = np.ascontiguousarray(fused, np.uint16)
        out = np.empty((rows, width), np.uint16)
        f = self._lib.h3ref_swiglu_bf16
        f.argtypes = [ctypes.c_void_p] * 2 + [ctypes.c_uint32] * 2
        self._check(f(_ptr(fused), _ptr(out), rows, width), "h3_swiglu_bf16")
        return out

    def add(self, left, right):
        keep = [np.ascontiguousarray(a, np.uint16) for a in (left, right)]
        out = np.empty_like(keep[0])
        f = self._lib.h3ref_add_bf16
        f.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_uint32]
        self._check(f(_ptr(keep[0]), _ptr(keep[1]), _ptr(out), out.size), "h3_add_bf16")
        return out

    def linear(self, x, w, bias=None):
        rows, k = x.shape
        n = w.shape[0]
        keep = [np.ascontiguousarray(a) if a is not None else None for a in (x, w, bias)]
        out = np.empty((rows, n), np.uint16)
        f = self._lib.h3ref_linear_bf16
        f.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_uint32] * 3
        self._check(f(*[_ptr(a) for a in keep], _ptr(out), rows, k, n), "h3_linear_bf16")
        return out


def reference_cuda():
    """The reference's CUDA element kernels (needs a GPU), or None if `_ref` was never built."""
    global _ref_cuda
    if _ref_cuda is None and os.path.exists(_REF_CUDA):
        _ref_cuda = ReferenceCuda(ctypes.CDLL(_REF_CUDA))
    return _ref_cuda
