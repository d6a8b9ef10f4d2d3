"""ctypes binding of include/h3q8.h.

`Gpu` mirrors the reference's operator interface (src/gpu.h): the same operator
names without the `h3_gpu_` prefix, the same argument order and meaning, the
same 1/0 result convention turned into `H3Error` carrying `h3_gpu_error()`.
"""
import ctypes as C
import os

import numpy as np

MODE_BF16, MODE_W8A16, MODE_W8A8 = 0, 1, 2
ACT_NONE, ACT_GELU_TANH, ACT_SWIGLU = 0, 1, 2
KERNEL_AUTO, KERNEL_PLAIN, KERNEL_TCGEN05, KERNEL_TCGEN05_M256, KERNEL_TCGEN05_N128, KERNEL_TCGEN05_PAIR = 0, 1, 2, 3, 4, 5
KERNEL_TCGEN05_SPLITK = 6
KERNEL_TCGEN05_SKINNY = 7
F32, BF16, I8, U32, F16 = 0, 1, 2, 3, 4
HOST_VISIBLE, DEVICE_ONLY, HOST_PINNED = 0, 1, 2

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libh3q8.so")
_lib = None


class H3Error(RuntimeError):
    pass


class LinearDesc(C.Structure):
    """h3q8_linear_desc"""
    _fields_ = [
        ("mode", C.c_uint32), ("rows", C.c_uint32), ("input_dim", C.c_uint32), ("output_dim", C.c_uint32),
        ("input", C.c_void_p), ("weight", C.c_void_p), ("weight_scales", C.c_void_p), ("weight_group", C.c_uint32),
        ("input_scales", C.c_void_p), ("bias", C.c_void_p), ("gate", C.c_void_p), ("residual", C.c_void_p),
        ("activation", C.c_uint32), ("output", C.c_void_p), ("accumulators", C.c_void_p), ("kernel", C.c_uint32),
        ("input_group", C.c_uint32), ("rope", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("after_producer", C.c_uint32),
    ]


def _u64(*names):
    return [(n, C.c_uint64) for n in names]


def _f64(*names):
    return [(n, C.c_double) for n in names]


class Stats(C.Structure):
    """h3_gpu_stats: the reference's layout (src/gpu.h:99-142), field for field."""
    _fields_ = (_u64("q8_weights", "q8_source_bytes", "q8_storage_bytes", "q8_dispatches") + _f64("q8_load_seconds") +
                _u64("layout_prepares", "layout_inplace_packs", "layout_scan_replaced_bytes", "layout_partial_bytes",
                     "allocated_bytes", "live_bytes", "peak_live_bytes", "tensor_allocations", "direct_dispatches",
                     "mps_linear_dispatches", "mps_conv_dispatches", "mps_sdpa_dispatches", "native_attention_dispatches",
                     "metal_current_allocated_bytes", "blit_copies", "submissions") +
                _f64("command_encode_seconds", "command_wait_seconds", "gpu_seconds") +
                _u64("linear_dispatches", "conv_dispatches", "attention_dispatches", "h2d_bytes", "d2h_bytes", "d2d_bytes",
                     "streamed_bytes", "resident_weight_bytes", "stream_slot_bytes", "resident_block_mask") +
                [("resident_blocks", C.c_uint), ("active_weight_blocks", C.c_uint)] +
                _u64("device_bytes", "managed_bytes", "pinned_bytes", "peak_pinned_bytes", "stream_stalls") +
                _f64("transfer_seconds", "stream_wait_seconds", "linear_seconds", "attention_seconds", "conv_seconds",
                     "h2d_seconds", "d2h_seconds", "slot_wait_seconds", "normalization_seconds") +
                _u64("weight_cache_bytes", "weight_cache_hits", "weight_cache_hit_bytes", "weight_cache_misses",
                     "weight_cache_evictions") + _f64("quant_conversion_seconds") +
                _u64("quant_clipped_values", "quant_zeroed_values", "quant_projection_dispatches", "quant_cache_hits",
                     "quant_cache_misses", "sage2_attention_dispatches", "sage3_attention_dispatches",
                     "attention_workspace_bytes", "inflight_peak", "command_retirements", "bounded_waits", "pressure_drains",
                     "native_scratch_bytes", "native_scratch_allocations", "native_scratch_reuses", "native_pipeline_count",
                     "main_dense_calls", "subblock_calls", "subblock_bypass", "subblock_protected_calls", "subblock_selected",
                     "subblock_possible", "subblock_router_calls", "attention_timing_samples", "attention_timing_missed") +
                _f64("main_attention_seconds", "subblock_router_seconds", "subblock_kernel_seconds"))


class Profile(C.Structure):
    """h3q8_gpu_profile"""
    _fields_ = _u64("linear_kernel_launches", "conversion_kernel_launches")


class WeightOptions(C.Structure):
    """h3_weight_options"""
    _fields_ = [("mode", C.c_int), ("max_resident", C.c_int), ("capacity_limit", C.c_uint64), ("allocation_limit", C.c_uint64)]


class WeightPlan(C.Structure):
    """h3_weight_plan"""
    _fields_ = [("options", WeightOptions)] + [(n, C.c_uint64) for n in (
        "active_mask", "resident_mask", "free_bytes", "live_bytes", "reserve_bytes", "future_bytes", "block_bytes",
        "resident_bytes", "slot_bytes")] + [("active_count", C.c_uint), ("resident_count", C.c_uint), ("effective_mode", C.c_int)]


class DitPolicy(C.Structure):
    """h3q8_dit_linear_policy"""
    _fields_ = [(n, C.c_int) for n in ("int8_qkv", "int8_attention_out", "int8_mlp", "head_major_attention_out",
                                       "fuse_int8_mlp_input", "fuse_int8_qkv_input", "int8_row_fc2")]


class DitShape(C.Structure):
    """h3q8_dit_shape"""
    _fields_ = [(n, C.c_uint32) for n in ("rows", "hidden", "heads", "head_dim", "rope_half", "ffn", "slots")] + [("epsilon", C.c_float)]


class DitWeights(C.Structure):
    """h3q8_dit_block_weights"""
    _fields_ = [(n, C.c_void_p) for n in ("qkv", "out", "fc1", "fc2", "qkv_int8", "qkv_scales", "out_int8", "out_scales", "fc1_int8",
                                          "fc1_scales", "fc2_int8", "fc2_scales", "q_norm", "k_norm", "norm1", "norm2")]


class DitBuffers(C.Structure):
    """h3q8_dit_block_buffers"""
    _fields_ = [(n, C.c_void_p) for n in ("hidden", "mod_attention", "qkv", "query", "key", "value", "attention_heads", "attention_output",
                                          "mod_mlp", "mlp_output", "activated", "int8_activation", "int8_activation_scales")]


class Problem(C.Structure):
    """h3_gpu_linear_problem"""
    _fields_ = [("output", C.c_void_p), ("input", C.c_void_p), ("weight", C.c_void_p), ("bias", C.c_void_p),
                ("gate", C.c_void_p), ("residual", C.c_void_p), ("rows", C.c_uint32), ("input_dim", C.c_uint32),
                ("output_dim", C.c_uint32), ("activation", C.c_int)]


def library():
    """Loads the in-tree libh3q8.so; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise H3Error(f"{_LIB_PATH} is missing: run `python -m h3cli_b200.build` (needs nvcc); there is no CPU fallback")
    lib = C.CDLL(_LIB_PATH)
    vp, u32, u64, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t
    sig = {
        "h3_q8_layout": (C.c_int, [u32, u32, C.POINTER(sz), C.POINTER(sz)]),
        "h3_q8_pack_rows": (C.c_int, [vp, vp, vp, u32, u32]),
        "h3q8_q8_layout": (C.c_int, [u32, u32, u32, C.POINTER(sz), C.POINTER(sz)]),
        "h3q8_q8_pack_rows": (C.c_int, [vp, vp, vp, u32, u32, u32]),
        "h3_gpu_profile_set_label": (None, [vp, C.c_char_p]),
        "h3_gpu_profile_mark": (None, [vp, C.c_char_p]),
        "h3_gpu_plan_bf16_weights": (C.c_int, [vp, u64, u64, u64, C.c_int, C.c_int, C.POINTER(WeightPlan)]),
        "h3_gpu_weight_plan_compatible": (C.c_int, [vp, C.c_int]),
        "h3_gpu_should_retry_streaming": (C.c_int, [vp]),
        "h3_weight_mode_name": (C.c_char_p, [C.c_int]),
        "h3_weight_options_read": (C.c_int, [C.POINTER(WeightOptions), C.c_int, C.c_char_p, sz]),
        "h3_weight_options_equal": (C.c_int, [C.POINTER(WeightOptions), C.POINTER(WeightOptions)]),
        "h3_weight_plan_build": (C.c_int, [C.POINTER(WeightPlan), WeightOptions, u64, u64, u64, u64, u64, u64, C.c_char_p, sz]),
        "h3_weight_retry_cap": (C.c_int, [C.c_uint]),
        "h3q8_cache_open": (vp, [C.c_char_p, C.c_char_p, u64, u32, u32, u32, C.c_char_p, sz]),
        "h3q8_cache_open_content": (vp, [C.c_char_p, C.c_char_p, u64, u32, u32, u32, C.c_char_p, sz]),
        "h3q8_sha256": (None, [vp, sz, vp]),
        "h3q8_cache_read": (C.c_int, [vp, vp, C.c_char_p, sz]),
        "h3q8_cache_write": (C.c_int, [vp, vp, C.c_char_p, sz]),
        "h3q8_cache_unchanged": (C.c_int, [vp, C.c_char_p, sz]),
        "h3q8_cache_payload_bytes": (sz, [vp]),
        "h3q8_cache_artifact": (C.c_char_p, [vp]),
        "h3q8_cache_close": (None, [vp]),
        "h3q8_linear": (C.c_int, [C.POINTER(LinearDesc), vp]),
        "h3q8_linear_workspace_bytes": (sz, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
        "h3q8_linear_grouped": (C.c_int, [C.POINTER(LinearDesc), u32, vp]),
        "h3q8_linear_w8a8_static": (C.c_int, [C.POINTER(LinearDesc), vp, vp]),
        "h3q8_quantize_rows": (C.c_int, [vp, vp, vp, u32, u32, u32, C.c_float, vp]),
        "h3q8_quantize_rows_grouped": (C.c_int, [vp, vp, vp, u32, u32, u32, u32, vp]),
        "h3q8_q8_pack_rows_device": (C.c_int, [vp, vp, vp, u32, u32, u32, vp]),
        "h3q8_q8_dequant": (C.c_int, [vp, vp, vp, u32, u32, u32, vp]),
        "h3q8_device_status": (u32, [vp]),
        "h3q8_last_error": (C.c_char_p, []),
        "h3q8_kernel_launches": (u64, []),
        "h3q8_fault_injection": (None, [u64, u32]),
        "h3_gpu_create": (vp, [C.c_char_p, C.c_char_p, sz]),
        "h3_gpu_free": (None, [vp]), "h3_gpu_cancel": (None, [vp]),
        "h3_gpu_error": (C.c_char_p, [vp]),
        "h3_gpu_get_stats": (C.c_int, [vp, C.POINTER(Stats)]),
        "h3q8_gpu_get_profile": (C.c_int, [vp, C.POINTER(Profile)]),
        "h3_weight_packed_size": (C.c_int, [u32, u32, C.c_int, C.POINTER(u64), C.POINTER(u64), C.POINTER(u64)]),
        "h3q8_linear_finish": (C.c_int, [vp, u32, u32, vp, vp, vp, u32, vp, vp]),
        "h3_gpu_adaln_bf16": (C.c_int, [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, C.c_float]),
        "h3_gpu_gate_adaln_bf16": (C.c_int, [vp] * 9 + [u32] * 6 + [C.c_float]),
        "h3_gpu_mlp_bf16": (C.c_int, [vp, vp, vp, vp, vp, u32, u32, u32, u32]),
        "h3_quant_projection": (C.c_int, [C.c_char_p, C.c_int]),
        "h3_quant_projection_policy": (C.c_int, [C.c_char_p, C.c_int, C.c_int]),
        "h3q8_dit_linear_policy_resolve": (C.c_int, [vp, u32, C.c_int, C.POINTER(DitPolicy)]),
        "h3q8_dit_block_attention_input": (C.c_int, [vp, C.POINTER(DitPolicy), C.POINTER(DitShape), C.POINTER(DitWeights),
                                                     C.POINTER(DitBuffers), vp, vp, vp, vp, C.c_int, C.c_int]),
        "h3q8_dit_block_after_attention": (C.c_int, [vp, C.POINTER(DitPolicy), C.POINTER(DitShape), C.POINTER(DitWeights), vp,
                                                     C.POINTER(DitBuffers), vp, vp, vp, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
        "h3q8_gpu_linear_partial_f32": (C.c_int, [vp, vp, vp, vp, u32, u32, u32]),
        "h3q8_gpu_linear_finish_bf16": (C.c_int, [vp, vp, vp, vp, vp, vp, u32, u32, C.c_int]),
        "h3_gpu_backend_name": (C.c_char_p, [vp]), "h3_gpu_has_int8_mlp": (C.c_int, [vp]),
        "h3_gpu_begin": (C.c_int, [vp]), "h3_gpu_continue": (C.c_int, [vp]),
        "h3_gpu_submit": (C.c_int, [vp]), "h3_gpu_synchronize": (C.c_int, [vp]),
        "h3_gpu_tensor_alloc": (vp, [vp, sz, C.c_int, C.c_int]),
        "h3_gpu_tensor_contents": (vp, [vp]),
        "h3_gpu_tensor_new_f32": (vp, [vp, sz]), "h3_gpu_tensor_new_bf16": (vp, [vp, sz]), "h3_gpu_tensor_new_i8": (vp, [vp, sz]),
        "h3_gpu_tensor_from_f32": (vp, [vp, vp, sz]), "h3_gpu_tensor_from_bf16": (vp, [vp, vp, sz]),
        "h3_gpu_tensor_from_u32": (vp, [vp, vp, sz]),
        "h3_gpu_tensor_free": (None, [vp]), "h3_gpu_tensor_elements": (sz, [vp]), "h3_gpu_tensor_dtype": (C.c_int, [vp]),
        "h3_gpu_tensor_read_f32": (C.c_int, [vp, vp, sz]), "h3_gpu_tensor_read_bf16": (C.c_int, [vp, vp, sz]),
        "h3_gpu_tensor_read_u32": (C.c_int, [vp, vp, sz]), "h3_gpu_tensor_read_i8": (C.c_int, [vp, vp, sz]),
        "h3_gpu_tensor_write_f32": (C.c_int, [vp, vp, sz]), "h3_gpu_tensor_write_bf16": (C.c_int, [vp, vp, sz]),
        "h3_gpu_tensor_write_i8": (C.c_int, [vp, vp, sz]),
        "h3_gpu_tensor_write_bf16_range": (C.c_int, [vp, sz, vp, sz]),
        "h3_gpu_event_new": (vp, [vp]), "h3_gpu_event_record": (C.c_int, [vp, vp]),
        "h3_gpu_event_wait": (C.c_int, [vp, vp]), "h3_gpu_event_free": (None, [vp]),
        "h3_gpu_tensor_load_bf16": (vp, [vp, C.c_char_p, u64, sz]),
        "h3_gpu_tensor_read_file_bf16": (C.c_int, [vp, C.c_char_p, u64, sz, C.c_char_p, sz]),
        "h3_gpu_tensor_stream_file_bf16": (C.c_int, [vp, C.c_char_p, u64, sz, C.c_char_p, sz]),
        "h3_gpu_plan_weights": (C.c_int, [vp, u64, u64]), "h3_gpu_release_weight_cache": (C.c_int, [vp]),
        "h3_gpu_linear_bf16": (C.c_int, [vp, vp, vp, vp, vp, u32, u32, u32]),
        "h3_gpu_quant_configure": (C.c_int, [vp, C.c_int, C.c_char_p, u64, u64, C.c_int]),
        "h3_gpu_quant_load": (vp, [vp, C.c_char_p, u64, u32, u32]),
        "h3_gpu_q8_load": (vp, [vp, C.c_char_p, u64, u32, u32]),
        "h3q8_gpu_set_group": (C.c_int, [vp, u32]),
        "h3q8_gpu_tensor_device_pointer": (vp, [vp]), "h3q8_gpu_compute_stream": (vp, [vp]),
        "h3q8_gpu_set_w8a16_scratch_rows": (C.c_int, [vp, u32]),
        "h3q8_gpu_set_profiling": (C.c_int, [vp, C.c_int]),
        "h3q8_gpu_tensor_upload_async": (C.c_int, [vp, vp, sz]),
        "h3q8_gpu_tensor_download_async": (C.c_int, [vp, vp, sz]),
        "h3q8_gpu_tensor_wait": (C.c_int, [vp]),
        "h3q8_gpu_q8_from_host": (vp, [vp, vp, vp, u32, u32, u32]),
        "h3q8_gpu_weight_stream_create": (vp, [vp, sz, u32]),
        "h3q8_gpu_weight_stream_prefetch": (C.c_int, [vp, vp, sz]),
        "h3q8_gpu_weight_stream_acquire": (C.c_int, [vp, C.c_int]),
        "h3q8_gpu_weight_stream_reserve": (C.c_int, [vp, vp, C.POINTER(vp)]),
        "h3q8_gpu_weight_stream_publish": (C.c_int, [vp, C.c_int, vp, sz]),
        "h3q8_gpu_weight_stream_release": (C.c_int, [vp, C.c_int]),
        "h3q8_gpu_weight_stream_view": (vp, [vp, C.c_int, sz, u32, u32, u32]),
        "h3q8_gpu_weight_stream_free": (None, [vp]),
        "h3q8_q8_blob_bytes": (sz, [u32, u32, u32, C.POINTER(sz)]),
        "h3_gpu_quantize_weight_int8": (C.c_int, [vp, vp, vp, vp, u32, u32]),
        "h3_gpu_linear_int8_bf16": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, C.c_int]),
        "h3_gpu_gate_adaln_quantize_int8": (C.c_int, [vp] * 10 + [u32] * 7 + [C.c_float]),
        "h3_gpu_linear_int8_head_major_bf16": (C.c_int, [vp] * 7 + [u32] * 4),
        "h3_gpu_mlp_int8_bf16": (C.c_int, [vp] * 12 + [u32] * 4 + [C.c_int] * 4),
        "h3_gpu_grouped_qkv_linear_rope_int8": (C.c_int, [vp] * 13 + [u32] * 5 + [C.c_float] + [C.c_int] * 4),
        "h3_gpu_linear_fused_int8_bf16": (C.c_int, [vp, vp, vp, vp, u32, vp, vp, vp, vp, u32, u32, u32, C.c_int]),
        "h3_gpu_gelu_bf16": (C.c_int, [vp, vp, vp, u32, C.c_int]),
        "h3_gpu_gate_bf16": (C.c_int, [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32]),
        "h3_gpu_add_bf16": (C.c_int, [vp, vp, vp, vp, u32]),
        "h3_gpu_swiglu_bf16": (C.c_int, [vp, vp, vp, u32, u32]),
        "h3_gpu_grouped_qkv_rope_bf16": (C.c_int, [vp] * 9 + [u32] * 4 + [C.c_float]),
        "h3_gpu_grouped_qkv_linear_rope_bf16": (C.c_int, [vp] * 11 + [u32] * 5 + [C.c_float]),
        "h3_gpu_linear_fused_bf16": (C.c_int, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, C.c_int]),
        "h3_gpu_linear_grouped_bf16": (C.c_int, [vp, C.POINTER(Problem), u32]),
    }
    for name, (restype, argtypes) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = restype, argtypes
    lib._signatures = sig
    _lib = lib
    return lib


_NP = {F32: np.float32, BF16: np.uint16, I8: np.int8, U32: np.uint32}


class Tensor:
    """An h3_gpu_tensor; bf16 travels as uint16 bit patterns."""

    def __init__(self, gpu, handle):
        if not handle:
            raise H3Error(gpu.error())
        self.gpu, self.handle = gpu, handle

    @property
    def elements(self):
        return library().h3_gpu_tensor_elements(self.handle)

    @property
    def dtype(self):
        return library().h3_gpu_tensor_dtype(self.handle)

    @property
    def device_pointer(self):
        return library().h3q8_gpu_tensor_device_pointer(self.handle)

    def read(self, elements=None, dtype=None):
        dtype = self.dtype if dtype is None else dtype
        n = self.elements if elements is None else elements
        out = np.empty(n, _NP[dtype])
        fn = {F32: "read_f32", BF16: "read_bf16", I8: "read_i8", U32: "read_u32"}[dtype]
        self.gpu._check(getattr(library(), "h3_gpu_tensor_" + fn)(self.handle, out.ctypes.data, n))
        return out

    def write(self, values):
        values = np.ascontiguousarray(values)
        fn = {F32: "write_f32", BF16: "write_bf16", I8: "write_i8"}[self.dtype]
        self.gpu._check(getattr(library(), "h3_gpu_tensor_" + fn)(self.handle, values.ctypes.data, values.size))

    def upload_async(self, host_pointer, nbytes):
        self.gpu._check(library().h3q8_gpu_tensor_upload_async(self.handle, host_pointer, nbytes))

    def download_async(self, host_pointer, nbytes):
        self.gpu._check(library().h3q8_gpu_tensor_download_async(self.handle, host_pointer, nbytes))

    def wait(self):
        self.gpu._check(library().h3q8_gpu_tensor_wait(self.handle))

    def free(self):
        if self.handle:
            library().h3_gpu_tensor_free(self.handle)
            self.handle = None


def _h(t):
    return None if t is None else t.handle


def q8_blob(weights, scales, group):
    """Packs int8 [N,K] + fp32 scales into the byte layout weight-stream views expect."""
    weights = np.ascontiguousarray(weights, np.int8)
    rows, columns = weights.shape
    offset = C.c_size_t()
    total = library().h3q8_q8_blob_bytes(rows, columns, group, C.byref(offset))
    blob = np.zeros(total, np.uint8)
    blob[:rows * columns] = weights.reshape(-1).view(np.uint8)
    s = np.ascontiguousarray(scales, np.float32).reshape(-1).view(np.uint8)
    blob[offset.value:offset.value + s.size] = s
    return blob


class WeightStream:
    """h3q8_weight_stream: device slots fed from host memory on the copy stream."""

    def __init__(self, gpu, slot_bytes, slots):
        self.gpu = gpu
        self.handle = library().h3q8_gpu_weight_stream_create(gpu.handle, slot_bytes, slots)
        if not self.handle:
            raise H3Error(gpu.error())

    def prefetch(self, host_pointer, nbytes):
        slot = library().h3q8_gpu_weight_stream_prefetch(self.handle, host_pointer, nbytes)
        if slot < 0:
            raise H3Error(self.gpu.error())
        return slot

    def reserve(self, producer_stream):
        """Next slot for a caller-filled layer: (slot, device pointer); producer_stream waits for the slot's release."""
        pointer = C.c_void_p()
        slot = library().h3q8_gpu_weight_stream_reserve(self.handle, producer_stream, C.byref(pointer))
        if slot < 0:
            raise H3Error(self.gpu.error())
        return slot, pointer.value

    def publish(self, slot, producer_stream, nbytes):
        return self.gpu._check(library().h3q8_gpu_weight_stream_publish(self.handle, slot, producer_stream, nbytes))

    def acquire(self, slot):
        return self.gpu._check(library().h3q8_gpu_weight_stream_acquire(self.handle, slot))

    def release(self, slot):
        return self.gpu._check(library().h3q8_gpu_weight_stream_release(self.handle, slot))

    def view(self, slot, offset, rows, columns, group):
        return Tensor(self.gpu, library().h3q8_gpu_weight_stream_view(self.handle, slot, offset, rows, columns, group))

    def free(self):
        if self.handle:
            library().h3q8_gpu_weight_stream_free(self.handle)
            self.handle = None


class Gpu:
    """An h3_gpu context (src/gpu.h): one per GPU, used by one thread at a time."""

    def __init__(self, shader_path=""):
        err = C.create_string_buffer(1024)
        self.handle = library().h3_gpu_create(shader_path.encode(), err, len(err))
        if not self.handle:
            raise H3Error(err.value.decode() or "h3_gpu_create failed")

    def error(self):
        return library().h3_gpu_error(self.handle).decode()

    def _check(self, ok):
        if not ok:
            raise H3Error(self.error())
        return ok

    def free(self):
        if self.handle:
            library().h3_gpu_free(self.handle)
            self.handle = None

    def cancel(self):
        library().h3_gpu_cancel(self.handle)

    def plan_bf16_weights(self, active_mask, block_bytes, future_bytes=0, force_stream=0, retry_cap=-1):
        """h3_gpu_plan_bf16_weights: returns the accepted h3_weight_plan or raises."""
        plan = WeightPlan()
        self._check(library().h3_gpu_plan_bf16_weights(self.handle, active_mask, block_bytes, future_bytes, force_stream,
                                                       retry_cap, C.byref(plan)))
        return plan

    def stats(self):
        s = Stats()
        self._check(library().h3_gpu_get_stats(self.handle, C.byref(s)))
        return s

    def profile(self):
        p = Profile()
        self._check(library().h3q8_gpu_get_profile(self.handle, C.byref(p)))
        return p

    def backend_name(self):
        return library().h3_gpu_backend_name(self.handle).decode()

    def begin(self):
        return self._check(library().h3_gpu_begin(self.handle))

    def continue_(self):
        return self._check(library().h3_gpu_continue(self.handle))

    def submit(self):
        return self._check(library().h3_gpu_submit(self.handle))

    def synchronize(self):
        return self._check(library().h3_gpu_synchronize(self.handle))

    @property
    def stream(self):
        return library().h3q8_gpu_compute_stream(self.handle)

    # tensors ------------------------------------------------------------
    def tensor_alloc(self, elements, dtype, storage=DEVICE_ONLY):
        return Tensor(self, library().h3_gpu_tensor_alloc(self.handle, elements, dtype, storage))

    def tensor_new_bf16(self, n):
        return Tensor(self, library().h3_gpu_tensor_new_bf16(self.handle, n))

    def tensor_new_i8(self, n):
        return Tensor(self, library().h3_gpu_tensor_new_i8(self.handle, n))

    def tensor_new_f32(self, n):
        return Tensor(self, library().h3_gpu_tensor_new_f32(self.handle, n))

    def tensor_from_bf16(self, bits):
        bits = np.ascontiguousarray(bits, np.uint16)
        return Tensor(self, library().h3_gpu_tensor_from_bf16(self.handle, bits.ctypes.data, bits.size))

    def tensor_from_f32(self, values):
        values = np.ascontiguousarray(values, np.float32)
        return Tensor(self, library().h3_gpu_tensor_from_f32(self.handle, values.ctypes.data, values.size))

    def tensor_from_u32(self, values):
        values = np.ascontiguousarray(values, np.uint32)
        return Tensor(self, library().h3_gpu_tensor_from_u32(self.handle, values.ctypes.data, values.size))

    def tensor_from_i8(self, values):
        values = np.ascontiguousarray(values, np.int8)
        t = self.tensor_new_i8(values.size)
        t.write(values)
        return t

    def tensor_load_bf16(self, path, offset, elements):
        return Tensor(self, library().h3_gpu_tensor_load_bf16(self.handle, path.encode(), offset, elements))

    # quantised weights --------------------------------------------------
    def quant_configure(self, mode, cache=None, bf16_weights=0, activations=0, force_stream=0):
        return self._check(library().h3_gpu_quant_configure(self.handle, mode, cache.encode() if cache else None,
                                                            bf16_weights, activations, force_stream))

    def set_group(self, group):
        return self._check(library().h3q8_gpu_set_group(self.handle, group))

    def set_w8a16_scratch_rows(self, rows):
        return self._check(library().h3q8_gpu_set_w8a16_scratch_rows(self.handle, rows))

    def set_profiling(self, enabled):
        return self._check(library().h3q8_gpu_set_profiling(self.handle, int(enabled)))

    def q8_load(self, path, offset, rows, columns):
        return Tensor(self, library().h3_gpu_q8_load(self.handle, path.encode(), offset, rows, columns))

    def quant_load(self, path, offset, rows, columns):
        return Tensor(self, library().h3_gpu_quant_load(self.handle, path.encode(), offset, rows, columns))

    def q8_from_host(self, weights, scales, group):
        weights = np.ascontiguousarray(weights, np.int8)
        scales = np.ascontiguousarray(scales, np.float32)
        rows, columns = weights.shape
        return Tensor(self, library().h3q8_gpu_q8_from_host(self.handle, weights.ctypes.data, scales.ctypes.data,
                                                            rows, columns, group))

    # packed-weight streaming ----------------------------------------------
    def weight_stream(self, slot_bytes, slots=2):
        return WeightStream(self, slot_bytes, slots)

    # operators ----------------------------------------------------------
    def linear_bf16(self, output, input, weight, bias, rows, input_dim, output_dim):
        return self._check(library().h3_gpu_linear_bf16(self.handle, _h(output), _h(input), _h(weight), _h(bias),
                                                        rows, input_dim, output_dim))

    def linear_fused_bf16(self, output, input, weight, bias, gate, residual, rows, input_dim, output_dim, activation):
        return self._check(library().h3_gpu_linear_fused_bf16(self.handle, _h(output), _h(input), _h(weight), _h(bias),
                                                              _h(gate), _h(residual), rows, input_dim, output_dim,
                                                              activation))

    def linear_partial_f32(self, sums, input, weight, rows, input_dim, output_dim):
        return self._check(library().h3q8_gpu_linear_partial_f32(self.handle, _h(sums), _h(input), _h(weight), rows, input_dim, output_dim))

    def linear_finish_bf16(self, output, sums, bias, gate, residual, rows, output_dim, activation):
        return self._check(library().h3q8_gpu_linear_finish_bf16(self.handle, _h(output), _h(sums), _h(bias), _h(gate), _h(residual),
                                                                 rows, output_dim, activation))

    def linear_grouped_bf16(self, problems):
        array = (Problem * len(problems))(*[Problem(_h(p["output"]), _h(p["input"]), _h(p["weight"]), _h(p.get("bias")),
                                                     _h(p.get("gate")), _h(p.get("residual")), p["rows"], p["input_dim"],
                                                     p["output_dim"], p.get("activation", 0)) for p in problems])
        return self._check(library().h3_gpu_linear_grouped_bf16(self.handle, array, len(problems)))

    def quantize_weight_int8(self, output, scales, input, rows, columns):
        return self._check(library().h3_gpu_quantize_weight_int8(self.handle, _h(output), _h(scales), _h(input), rows, columns))

    def linear_int8_bf16(self, output, quantized_input, input_scales, input, weight, weight_scales, rows, input_dim,
                         output_dim, use_slower_uncached_int8_scales=0):
        return self._check(library().h3_gpu_linear_int8_bf16(self.handle, _h(output), _h(quantized_input), _h(input_scales),
                                                             _h(input), _h(weight), _h(weight_scales), rows, input_dim,
                                                             output_dim, use_slower_uncached_int8_scales))

    def gate_adaln_quantize_int8(self, gated_residual, quantized_output, quantized_scales, residual, branch, norm_weight,
                                 gate_modulation, norm_modulation, row_map, rows, padded_rows, width, slots, gate_slot,
                                 shift_slot, scale_slot, epsilon):
        return self._check(library().h3_gpu_gate_adaln_quantize_int8(
            self.handle, _h(gated_residual), _h(quantized_output), _h(quantized_scales), _h(residual), _h(branch),
            _h(norm_weight), _h(gate_modulation), _h(norm_modulation), _h(row_map), rows, padded_rows, width, slots,
            gate_slot, shift_slot, scale_slot, epsilon))

    def linear_int8_head_major_bf16(self, output, quantized_input, input_scales, input, weight, weight_scales, rows, heads, head_dim,
                                    output_dim):
        return self._check(library().h3_gpu_linear_int8_head_major_bf16(
            self.handle, _h(output), _h(quantized_input), _h(input_scales), _h(input), _h(weight), _h(weight_scales), rows, heads,
            head_dim, output_dim))

    def mlp_int8_bf16(self, output, activated, quantized_activation, activation_scales, input, fc1_weight, fc1_scales, fc2_weight,
                      fc2_scales, rows, input_dim, hidden_dim, output_dim, use_int8_row_fc2=0, input_is_quantized=0):
        return self._check(library().h3_gpu_mlp_int8_bf16(
            self.handle, _h(output), _h(activated), _h(quantized_activation), _h(activation_scales), _h(input), _h(fc1_weight),
            _h(fc1_scales), _h(fc2_weight), _h(fc2_scales), None, None, rows, input_dim, hidden_dim, output_dim, 0, 0,
            use_int8_row_fc2, input_is_quantized))

    def grouped_qkv_linear_rope_int8(self, query, key, value, quantized_input, input_scales, input, weight, weight_scales, q_norm,
                                     k_norm, rope_cos, rope_sin, rows, input_dim, heads, head_dim, rope_half, epsilon,
                                     input_is_quantized=0):
        return self._check(library().h3_gpu_grouped_qkv_linear_rope_int8(
            self.handle, _h(query), _h(key), _h(value), _h(quantized_input), _h(input_scales), _h(input), _h(weight),
            _h(weight_scales), _h(q_norm), _h(k_norm), _h(rope_cos), _h(rope_sin), rows, input_dim, heads, head_dim, rope_half,
            epsilon, input_is_quantized, 0, 0, 0))

    def linear_fused_int8_bf16(self, output, quantized_input, input_scales, input_group, weight, bias, gate, residual,
                               rows, input_dim, output_dim, activation):
        return self._check(library().h3_gpu_linear_fused_int8_bf16(
            self.handle, _h(output), _h(quantized_input), _h(input_scales), input_group, _h(weight), _h(bias), _h(gate),
            _h(residual), rows, input_dim, output_dim, activation))

    def gelu_bf16(self, output, input, elements, approximate=1):
        return self._check(library().h3_gpu_gelu_bf16(self.handle, _h(output), _h(input), elements, approximate))

    def gate_bf16(self, output, residual, branch, modulation, row_map, rows, width, slots, gate_slot):
        return self._check(library().h3_gpu_gate_bf16(self.handle, _h(output), _h(residual), _h(branch), _h(modulation),
                                                      _h(row_map), rows, width, slots, gate_slot))

    def grouped_qkv_rope_bf16(self, query, key, value, qkv, q_norm, k_norm, rope_cos, rope_sin, sequence, heads, head_dim,
                              rope_half, epsilon):
        return self._check(library().h3_gpu_grouped_qkv_rope_bf16(
            self.handle, _h(query), _h(key), _h(value), _h(qkv), _h(q_norm), _h(k_norm), _h(rope_cos), _h(rope_sin),
            sequence, heads, head_dim, rope_half, epsilon))

    def grouped_qkv_linear_rope_bf16(self, query, key, value, qkv, input, weight, q_norm, k_norm, rope_cos, rope_sin, rows,
                                     input_dim, heads, head_dim, rope_half, epsilon):
        return self._check(library().h3_gpu_grouped_qkv_linear_rope_bf16(
            self.handle, _h(query), _h(key), _h(value), _h(qkv), _h(input), _h(weight), _h(q_norm), _h(k_norm),
            _h(rope_cos), _h(rope_sin), rows, input_dim, heads, head_dim, rope_half, epsilon))

    def adaln_bf16(self, output, input, norm_weight, modulation, row_map, rows, width, slots, shift_slot, scale_slot, epsilon):
        return self._check(library().h3_gpu_adaln_bf16(self.handle, _h(output), _h(input), _h(norm_weight), _h(modulation), _h(row_map),
                                                       rows, width, slots, shift_slot, scale_slot, epsilon))

    def gate_adaln_bf16(self, gated_residual, output, residual, branch, norm_weight, gate_modulation, norm_modulation, row_map, rows,
                        width, slots, gate_slot, shift_slot, scale_slot, epsilon):
        return self._check(library().h3_gpu_gate_adaln_bf16(self.handle, _h(gated_residual), _h(output), _h(residual), _h(branch),
                                                            _h(norm_weight), _h(gate_modulation), _h(norm_modulation), _h(row_map), rows,
                                                            width, slots, gate_slot, shift_slot, scale_slot, epsilon))

    def mlp_bf16(self, output, input, fc1, fc2, rows, input_dim, hidden_dim, output_dim):
        return self._check(library().h3_gpu_mlp_bf16(self.handle, _h(output), _h(input), _h(fc1), _h(fc2), rows, input_dim, hidden_dim,
                                                     output_dim))

    def swiglu_bf16(self, output, fused, rows, width):
        return self._check(library().h3_gpu_swiglu_bf16(self.handle, _h(output), _h(fused), rows, width))

    def add_bf16(self, output, left, right, elements):
        return self._check(library().h3_gpu_add_bf16(self.handle, _h(output), _h(left), _h(right), elements))

    # raw layer on this context's stream ------------------------------------
    def raw_linear(self, **fields):
        """h3q8_linear with Tensor / int fields; enqueues on the compute stream."""
        d = LinearDesc()
        for key, value in fields.items():
            setattr(d, key, value.device_pointer if isinstance(value, Tensor) else value)
        if not library().h3q8_linear(C.byref(d), self.stream):
            raise H3Error(library().h3q8_last_error().decode())

    def raw_status(self):
        return library().h3q8_device_status(self.stream)
