"""The C dispatcher of a DiT block's linears (h3q8_dit_block_*, the job of run_block() in
src/denoise/dit.c:2286-2537) on a B200: for every family setting it must issue exactly the operators the
reference's block issues, with the "input already quantised" state threaded from one block's tail into the next
block's QKV projection.  Two blocks are run through the dispatcher and through the same operator calls written
out by hand (each of which has its own parity test against the oracle); every tensor must agree bit for bit.
Attention is outside this path: a fixed synthetic tensor stands in for its output."""
import ctypes

import numpy as np
import pytest

import h3cli_b200 as h
from h3cli_b200 import api, synth

pytestmark = pytest.mark.gpu
ROWS, HIDDEN, HEADS, DIM, HALF, FFN, SLOTS, EPS = 300, 256, 2, 128, 48, 1024, 6, 1e-5
INNER, PADDED = HEADS * DIM, 384


def bf(a):
    a = np.asarray(a, np.float32)
    return synth.to_bf16(a).reshape(a.shape)


class Block:
    """Weights of one block in all the forms the dispatcher may pick from."""

    def __init__(self, gpu, oracle, seed):
        rng = np.random.default_rng(seed)
        shapes = dict(qkv=(3 * INNER, HIDDEN), out=(HIDDEN, INNER), fc1=(2 * FFN, HIDDEN), fc2=(HIDDEN, FFN))
        self.t = {}
        for i, (name, (n, k)) in enumerate(shapes.items()):
            wq = synth.int8_weights(seed, 10 + i, n, k)
            ws = synth.lognormal_scales(seed, 20 + i, n, 1) * np.float32(0.3 if name == "fc1" else 1.0)
            self.t[name] = gpu.q8_from_host(wq, ws, 0)                          # quantised descriptor for the bf16-call family
            self.t[name + "_int8"], self.t[name + "_scales"] = gpu.tensor_from_i8(wq), gpu.tensor_from_f32(ws[:, 0].copy())
        for name, width in (("q_norm", DIM), ("k_norm", DIM), ("norm1", HIDDEN), ("norm2", HIDDEN)):
            self.t[name] = gpu.tensor_from_bf16(bf(1 + 0.1 * rng.standard_normal(width)))
        self.modulation = gpu.tensor_from_bf16(bf(rng.standard_normal((2, SLOTS, HIDDEN)) * 0.1 + np.array([0, 0, 1, 0, 0, 1]).reshape(1, SLOTS, 1)))

    def struct(self):
        return api.DitWeights(**{name: tensor.handle for name, tensor in self.t.items()})


def make_buffers(gpu):
    sizes = dict(hidden=ROWS * HIDDEN, mod_attention=ROWS * HIDDEN, qkv=ROWS * 3 * INNER, query=ROWS * INNER, key=ROWS * INNER,
                 value=ROWS * INNER, attention_heads=ROWS * INNER, attention_output=ROWS * HIDDEN, mod_mlp=ROWS * HIDDEN,
                 mlp_output=ROWS * HIDDEN, activated=ROWS * FFN)
    b = {name: gpu.tensor_new_bf16(n) for name, n in sizes.items()}
    b["int8_activation"] = gpu.tensor_new_i8(PADDED * max(HIDDEN, INNER, FFN))
    b["int8_activation_scales"] = gpu.tensor_new_f32(PADDED * max(FFN // 1024, 1))
    return b


def by_hand(gpu, policy, blocks, b, row_map, cos, sin, attention, head_major):
    """run_block()'s operator sequence, written out call by call."""
    ready = quantized = 0
    snapshots = []
    for index, w in enumerate(blocks):
        t, mod = w.t, w.modulation
        if not ready:
            gpu.adaln_bf16(b["mod_attention"], b["hidden"], t["norm1"], mod, row_map, ROWS, HIDDEN, SLOTS, 0, 1, EPS)
        if policy.int8_qkv:
            gpu.grouped_qkv_linear_rope_int8(b["query"], b["key"], b["value"], b["int8_activation"], b["int8_activation_scales"], b["mod_attention"],
                                             t["qkv_int8"], t["qkv_scales"], t["q_norm"], t["k_norm"], cos, sin, ROWS, HIDDEN, HEADS, DIM, HALF, EPS,
                                             input_is_quantized=1 if ready and quantized else 0)
        else:
            gpu.grouped_qkv_linear_rope_bf16(b["query"], b["key"], b["value"], b["qkv"], b["mod_attention"], t["qkv"], t["q_norm"], t["k_norm"],
                                             cos, sin, ROWS, HIDDEN, HEADS, DIM, HALF, EPS)
        gpu.continue_()
        b["attention_heads"].write(attention[index])                       # the caller's attention
        if policy.int8_attention_out and head_major:
            gpu.linear_int8_head_major_bf16(b["attention_output"], b["int8_activation"], b["int8_activation_scales"], b["attention_heads"],
                                            t["out_int8"], t["out_scales"], ROWS, HEADS, DIM, HIDDEN)
        elif policy.int8_attention_out:
            gpu.linear_int8_bf16(b["attention_output"], b["int8_activation"], b["int8_activation_scales"], b["attention_heads"], t["out_int8"],
                                 t["out_scales"], ROWS, INNER, HIDDEN)
        else:
            gpu.linear_bf16(b["attention_output"], b["attention_heads"], t["out"], None, ROWS, INNER, HIDDEN)
        fused_mlp_in = policy.int8_mlp and policy.fuse_int8_mlp_input
        if fused_mlp_in:
            gpu.gate_adaln_quantize_int8(b["hidden"], b["int8_activation"], b["int8_activation_scales"], b["hidden"], b["attention_output"], t["norm2"],
                                         mod, mod, row_map, ROWS, PADDED, HIDDEN, SLOTS, 2, 3, 4, EPS)
        else:
            gpu.gate_adaln_bf16(b["hidden"], b["mod_mlp"], b["hidden"], b["attention_output"], t["norm2"], mod, mod, row_map, ROWS, HIDDEN, SLOTS,
                                2, 3, 4, EPS)
        if policy.int8_mlp:
            gpu.mlp_int8_bf16(b["mlp_output"], b["activated"], b["int8_activation"], b["int8_activation_scales"], b["mod_mlp"], t["fc1_int8"],
                              t["fc1_scales"], t["fc2_int8"], t["fc2_scales"], ROWS, HIDDEN, FFN, HIDDEN, use_int8_row_fc2=policy.int8_row_fc2,
                              input_is_quantized=1 if fused_mlp_in else 0)
        else:
            gpu.mlp_bf16(b["mlp_output"], b["mod_mlp"], t["fc1"], t["fc2"], ROWS, HIDDEN, FFN, HIDDEN)
        if index + 1 < len(blocks):
            nxt = blocks[index + 1]
            if policy.int8_qkv and policy.fuse_int8_qkv_input:
                gpu.gate_adaln_quantize_int8(b["hidden"], b["int8_activation"], b["int8_activation_scales"], b["hidden"], b["mlp_output"],
                                             nxt.t["norm1"], mod, nxt.modulation, row_map, ROWS, PADDED, HIDDEN, SLOTS, 5, 0, 1, EPS)
                quantized = 1
            else:
                gpu.gate_adaln_bf16(b["hidden"], b["mod_attention"], b["hidden"], b["mlp_output"], nxt.t["norm1"], mod, nxt.modulation, row_map,
                                    ROWS, HIDDEN, SLOTS, 5, 0, 1, EPS)
                quantized = 0
            ready = 1
        else:
            gpu.gate_bf16(b["hidden"], b["hidden"], b["mlp_output"], mod, row_map, ROWS, HIDDEN, SLOTS, 5)
        gpu.continue_()
        snapshots.append({name: b[name].read() for name in ("query", "key", "value", "attention_output", "mlp_output", "hidden")})
    return snapshots


def dispatched(gpu, lib, policy, blocks, b, row_map, cos, sin, attention, poison):
    shape = api.DitShape(ROWS, HIDDEN, HEADS, DIM, HALF, FFN, SLOTS, EPS)
    buffers = api.DitBuffers(**{name: tensor.handle for name, tensor in b.items()})
    ready, quantized = ctypes.c_int(0), ctypes.c_int(0)
    snapshots, flags = [], []
    for index, w in enumerate(blocks):
        weights = w.struct()
        if ready.value and quantized.value and poison:
            # the next QKV must read the int8 activations the previous tail left, not this bf16 buffer
            b["mod_attention"].write(np.full(ROWS * HIDDEN, 0x7FC0, np.uint16))
        assert lib.h3q8_dit_block_attention_input(gpu.handle, ctypes.byref(policy), ctypes.byref(shape), ctypes.byref(weights),
                                                  ctypes.byref(buffers), w.modulation.handle, row_map.handle, cos.handle, sin.handle,
                                                  ready.value, quantized.value), gpu.error()
        gpu.continue_()
        b["attention_heads"].write(attention[index])
        last = index + 1 == len(blocks)
        nxt = None if last else blocks[index + 1]
        assert lib.h3q8_dit_block_after_attention(gpu.handle, ctypes.byref(policy), ctypes.byref(shape), ctypes.byref(weights),
                                                  None if last else nxt.t["norm1"].handle, ctypes.byref(buffers), w.modulation.handle,
                                                  None if last else nxt.modulation.handle, row_map.handle, 0 if last else 1,
                                                  ctypes.byref(ready), ctypes.byref(quantized)), gpu.error()
        gpu.continue_()
        flags.append((ready.value, quantized.value))
        snapshots.append({name: b[name].read() for name in ("query", "key", "value", "attention_output", "mlp_output", "hidden")})
    return snapshots, flags


SETTINGS = {
    "descriptor weights through the bf16 calls": dict(),
    "int8 everywhere, fused quantisers, head-major attention output": dict(int8_qkv=1, int8_attention_out=1, int8_mlp=1,
                                                                          head_major_attention_out=1, fuse_int8_mlp_input=1, fuse_int8_qkv_input=1),
    "int8 everywhere, separate quantisers, row-major attention output, per-row fc2": dict(int8_qkv=1, int8_attention_out=1, int8_mlp=1, int8_row_fc2=1),
    "int8 MLP only": dict(int8_mlp=1, fuse_int8_mlp_input=1),
    "int8 QKV only with the fused tail": dict(int8_qkv=1, fuse_int8_qkv_input=1),
}


@pytest.mark.parametrize("setting", list(SETTINGS))
def test_dispatcher_issues_the_reference_sequence(oracle, setting):
    policy = api.DitPolicy(**SETTINGS[setting])
    head_major = bool(policy.head_major_attention_out)
    rng = np.random.default_rng(7)
    x0 = bf(rng.standard_normal((ROWS, HIDDEN)))
    angle = rng.uniform(0, 6.28, (ROWS, HALF))
    attention = [bf(rng.standard_normal((HEADS, ROWS, DIM) if head_major else (ROWS, INNER))).ravel() for _ in range(2)]
    results = []
    for route in ("hand", "dispatcher"):
        gpu = h.Gpu()
        gpu.quant_configure(1)
        blocks = [Block(gpu, oracle, 100), Block(gpu, oracle, 200)]
        b = make_buffers(gpu)
        b["hidden"].write(x0.ravel())
        row_map = gpu.tensor_from_u32((np.arange(ROWS) % 2).astype(np.uint32))
        cos, sin = gpu.tensor_from_bf16(bf(np.cos(angle))), gpu.tensor_from_bf16(bf(np.sin(angle)))
        gpu.begin()
        if route == "hand":
            results.append(by_hand(gpu, policy, blocks, b, row_map, cos, sin, attention, head_major))
        else:
            snapshots, flags = dispatched(gpu, h.library(), policy, blocks, b, row_map, cos, sin, attention, poison=True)
            results.append(snapshots)
            assert flags[0] == (1, 1 if policy.int8_qkv and policy.fuse_int8_qkv_input else 0) and flags[1] == (0, 0)
        gpu.submit()
        gpu.free()
    for block_index, (hand, auto) in enumerate(zip(*results)):
        for name in hand:
            assert (hand[name] == auto[name]).all(), f"block {block_index}: {name} differs"
            assert np.isfinite(synth.from_bf16(auto[name])).all(), f"block {block_index}: {name} is not finite"


def test_policy_follows_the_reference_flags(monkeypatch):
    """src/denoise/dit.c:1956-1968 and the H3_DISABLE_* switches of run_block()."""
    gpu = h.Gpu()
    lib = h.library()
    policy = api.DitPolicy()
    for name in ("H3_DISABLE_INT8_MLP", "H3_DISABLE_INT8_QKV", "H3_DISABLE_INT8_ATTENTION_OUT", "H3_DISABLE_FUSED_INT8_MLP_INPUT",
                 "H3_DISABLE_FUSED_INT8_QKV_INPUT", "H3_DISABLE_HEAD_MAJOR_ATTENTION_OUTPUT", "H3_INT8_MLP_STAGE"):
        monkeypatch.delenv(name, raising=False)
    assert lib.h3q8_dit_linear_policy_resolve(gpu.handle, 32400, 0, ctypes.byref(policy))
    assert (policy.int8_qkv, policy.int8_attention_out, policy.int8_mlp, policy.head_major_attention_out, policy.fuse_int8_mlp_input,
            policy.fuse_int8_qkv_input) == (1, 1, 1, 1, 1, 1)
    assert lib.h3q8_dit_linear_policy_resolve(gpu.handle, 64, 0, ctypes.byref(policy))          # fewer than 128 rows
    assert (policy.int8_qkv, policy.int8_attention_out, policy.int8_mlp) == (0, 0, 1)
    assert lib.h3q8_dit_linear_policy_resolve(gpu.handle, 32400, 1, ctypes.byref(policy))       # streamed weights
    assert (policy.int8_qkv, policy.int8_attention_out, policy.int8_mlp) == (0, 0, 0)
    monkeypatch.setenv("H3_DISABLE_INT8_QKV", "1")
    monkeypatch.setenv("H3_DISABLE_FUSED_INT8_MLP_INPUT", "1")
    assert lib.h3q8_dit_linear_policy_resolve(gpu.handle, 32400, 0, ctypes.byref(policy))
    assert (policy.int8_qkv, policy.fuse_int8_qkv_input, policy.int8_mlp, policy.fuse_int8_mlp_input) == (0, 0, 1, 0)
    gpu.free()
