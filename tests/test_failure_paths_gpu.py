"""Failure paths on a B200, none of which faults or hangs the GPU.

Every wait inside the GEMM kernels is bounded.  The tests make one run out the sanctioned way -- a host-side switch
(h3q8_fault_injection) shortens the limit to about a millisecond and makes the TMA producer leave out its first
operand load, so the MMA issuer waits for a barrier that nothing completes -- and check that the kernel returns through
its normal exit, the status word carries the code, the operator layer turns it into an error at submit, cancel
recovers the context and the next linear is bit-exact again.  The second half is the reference's streaming test
(tests/test_cuda_runtime.c: 64 slot hand-offs with a prefetch thread while the owner computes)."""
import threading

import numpy as np
import pytest

import h3cli_b200 as h
from h3cli_b200 import synth

pytestmark = pytest.mark.gpu
LIMIT = 2_000_000        # clocks: about a millisecond


@pytest.fixture
def injected():
    lib = h.library()
    yield lib
    lib.h3q8_fault_injection(0, 0)


def exact_operands(rows, n, k):
    x = synth.to_bf16(np.where((np.arange(rows)[:, None] + np.arange(k)[None, :]) % 2, -1.0, 0.5).astype(np.float32)).reshape(rows, k)
    w = synth.to_bf16(np.where((np.arange(n)[:, None] + 2 * np.arange(k)[None, :]) % 3, 0.25, -2.0).astype(np.float32)).reshape(n, k)
    return x, w


@pytest.mark.parametrize("kernel,rows", [(h.KERNEL_TCGEN05_N128, 128), (h.KERNEL_TCGEN05, 128), (h.KERNEL_TCGEN05_PAIR, 256)])
def test_bounded_wait_runs_out_and_the_kernel_returns(injected, oracle, kernel, rows):
    lib = injected
    n = k = 128 if kernel == h.KERNEL_TCGEN05_N128 else 256
    x, w = exact_operands(rows, n, k)
    want = oracle.linear(oracle.MODE_BF16, x, w)
    gpu = h.Gpu()
    tx, tw, out = gpu.tensor_from_bf16(x), gpu.tensor_from_bf16(w), gpu.tensor_new_bf16(rows * n)
    call = lambda: gpu.raw_linear(mode=h.MODE_BF16, rows=rows, input_dim=k, output_dim=n, input=tx, weight=tw, output=out, kernel=kernel)
    assert gpu.raw_status() == 0
    lib.h3q8_fault_injection(LIMIT, 1)
    call()                                                     # returns: the launch itself is fine
    status = gpu.raw_status()                                  # synchronises; the kernel has come back on its own
    assert status != 0 and status != 0xFFFFFFFF and 1 <= (status & 0xFF) <= 4
    assert b"bounded wait" in lib.h3q8_last_error()
    assert gpu.raw_status() == 0                               # reading cleared it
    lib.h3q8_fault_injection(0, 0)
    call()
    assert gpu.raw_status() == 0
    assert (out.read().reshape(rows, n) == want).all()         # the context and the library are as good as new
    gpu.free()


def test_operator_layer_reports_at_submit_and_cancel_recovers(injected, oracle):
    lib = injected
    rows, n, k = 300, 256, 256
    x, w = exact_operands(rows, n, k)
    want = oracle.linear(oracle.MODE_BF16, x, w)
    gpu = h.Gpu()
    tx, tw, out = gpu.tensor_from_bf16(x), gpu.tensor_from_bf16(w), gpu.tensor_new_bf16(rows * n)
    lib.h3q8_fault_injection(LIMIT, 1)
    gpu.begin()
    gpu.linear_bf16(out, tx, tw, None, rows, k, n)
    with pytest.raises(h.H3Error, match="bounded wait"):
        gpu.submit()
    gpu.cancel()
    lib.h3q8_fault_injection(0, 0)
    gpu.begin()
    gpu.linear_bf16(out, tx, tw, None, rows, k, n)
    gpu.submit()
    assert (out.read().reshape(rows, n) == want).all()
    gpu.free()


def test_prefetch_thread_hands_over_slots_while_the_owner_computes(oracle, tmp_path):
    """tests/test_cuda_runtime.c: two device slots, an I/O thread that streams layer l + 1 from a file into the free slot
    with h3_gpu_tensor_stream_file_bf16 while the owner thread runs layer l's linear; 64 hand-offs, every result exact."""
    import ctypes
    layers, rows, n, k = 64, 130, 256, 256
    x, _ = exact_operands(rows, n, k)
    rng = np.random.default_rng(4)
    weights = [synth.to_bf16(rng.choice([-2.0, -0.5, 0.25, 1.0], (n, k)).astype(np.float32)).reshape(n, k) for _ in range(4)]
    path = tmp_path / "layers.bf16"
    path.write_bytes(b"".join(wt.tobytes() for wt in weights))
    want = [oracle.linear(oracle.MODE_BF16, x, wt) for wt in weights]
    lib = h.library()
    gpu = h.Gpu()
    slots = [gpu.tensor_new_bf16(n * k), gpu.tensor_new_bf16(n * k)]
    tx, out = gpu.tensor_from_bf16(x), gpu.tensor_new_bf16(rows * n)
    failures = []

    def prefetch(layer, slot):
        error = ctypes.create_string_buffer(256)
        if not lib.h3_gpu_tensor_stream_file_bf16(slots[slot].handle, str(path).encode(), (layer % 4) * n * k * 2, n * k, error, len(error)):
            failures.append(error.value.decode())

    prefetch(0, 0)
    gpu.begin()
    for layer in range(layers):
        worker = None
        if layer + 1 < layers:
            worker = threading.Thread(target=prefetch, args=(layer + 1, (layer + 1) % 2))
            worker.start()                                         # fills the other slot while this layer computes
        gpu.linear_bf16(out, tx, slots[layer % 2], None, rows, k, n)
        gpu.continue_()
        got = out.read().reshape(rows, n)
        assert (got == want[layer % 4]).all(), f"layer {layer}"
        if worker:
            worker.join()
        assert not failures, failures
    gpu.submit()
    stats = gpu.stats()
    assert stats.streamed_bytes == layers * n * k * 2 and stats.linear_dispatches == layers
    # a truncated file is an error from the I/O call, not a fault
    error = ctypes.create_string_buffer(256)
    assert not lib.h3_gpu_tensor_stream_file_bf16(slots[0].handle, str(path).encode(), 4 * n * k * 2 - 64, n * k, error, len(error))
    assert b"short read" in error.value
    for t in slots + [tx, out]:
        t.free()
    assert gpu.stats().live_bytes == 0
    gpu.free()
