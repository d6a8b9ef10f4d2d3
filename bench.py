#!/usr/bin/env python
"""Benchmark of the q8 DiT linear stack (one DiT block's four projections).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one pass of QKV (3072->9216), attention-output (3072->3072, gate *
branch + residual), FFN-up (3072->12288, GELU-tanh) and FFN-down (12288->3072,
gate * branch + residual) over M = 32,400 tokens per GPU with int8 weights and
per-channel fp32 scales (W8A16), synthetic seeded data.  With N > 1 every rank
runs the same rows-sharded step on its own GPU (weights replicated, no
collective); the job value is total TFLOP/s with the slowest rank's device time.

Prints one JSON line (rank 0): `value` with operands resident in HBM, `e2e`
through the h3_gpu_* operator interface with host buffers, `roofline` of the
GEMM kernel from CUDA events, `cpu_baseline` = the CPU restatement on a bounded
row slab.  `--impl reference` times only that CPU restatement: the reference's
int8 linears exist as Metal shaders only, it has no CPU or CUDA implementation
of this path that could be run here.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_TOKENS, HIDDEN, FFN = 32400, 3072, 12288
# The real MiniMax-H3 DiT projections (src/denoise/dit.c:31-46, 2424-2494): hidden 5376, heads 56 x 128, FFN 14336
# SwiGLU, no bias, group-64 scales.  "s" = fc1 + SwiGLU (weight rows [gate | up]).  Measured with --case real_*.
REAL_LAYERS = [("real_qkv", 5376, 21504, ""), ("real_qkv_rope", 5376, 21504, "q"), ("real_attn_out", 7168, 5376, "gr"), ("real_fc1", 5376, 14336, "s"),
               ("real_fc2", 14336, 5376, "gr")]
# name, K, N, epilogue
LAYERS = [("qkv", HIDDEN, 3 * HIDDEN, ""), ("attn_out", HIDDEN, HIDDEN, "gr"),
          ("ffn_up", HIDDEN, FFN, "a"), ("ffn_down", FFN, HIDDEN, "gr")]
# BASELINE configs 1 and 3: one linear, K = N = 3072, bias (and GELU-tanh for config 3); --rows 4096
CONFIG_CASES = [("config1", HIDDEN, HIDDEN, "b"), ("config3", HIDDEN, HIDDEN, "ba")]
FLOP_PER_STEP = sum(2.0 * M_TOKENS * k * n for _, k, n, _ in LAYERS)
METRIC = "q8_dit_block_linear_tflops"
UNIT = "TFLOP/s"
# dram__bytes_read.sum + dram__bytes_write.sum per GEMM launch of this workload (mean of QKV, attn-out, FFN-up,
# FFN-down at M = 32,400), from a one-pass ncu capture of this same command
NCU_TRAFFIC_BYTES_PER_LAUNCH = 2.484e9


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            peaks = json.load(f)
        return float(peaks["bf16_tflops"]), float(peaks.get("bf16_tflops_sustained", 0.0)), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self.stop_flag = index, [], set(), None, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.handle = pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if not self.nv:
            return
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
        while not self.stop_flag:
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.handle, self.nv.NVML_CLOCK_SM))
                try:
                    bits = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    bits = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.reasons.update(n for b, n in names.items() if bits & b)
            except Exception:
                break
            time.sleep(0.002)

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def oracle_slab(rows, steps, warmup, mode="w8a16"):
    """Times the CPU restatement (oracle fast path, all host threads) on `rows` rows of each GEMM shape."""
    import oracle
    oracle.build()
    # every core this process may run on, whatever OMP_NUM_THREADS a launcher exported (torch.distributed.run sets 1)
    oracle.lib().h3o_set_threads(len(os.sched_getaffinity(0)))
    rng = np.random.default_rng(0)
    work = []
    for name, k, n, spec in LAYERS:
        x = oracle.f32_to_bf16(rng.standard_normal((rows, k), dtype=np.float32)).reshape(rows, k)
        wq = rng.integers(-127, 128, (n, k), dtype=np.int8)
        ws = np.exp(rng.normal(np.log(0.01), 0.3, (n, 1))).astype(np.float32)
        gate = oracle.f32_to_bf16((rng.standard_normal(n, dtype=np.float32) * np.float32(0.1) + 1)) if "g" in spec else None
        res = oracle.f32_to_bf16(rng.standard_normal((rows, n), dtype=np.float32)).reshape(rows, n) if "r" in spec else None
        work.append((x, wq, ws, gate, res, 1 if "a" in spec else 0))
    flop = sum(2.0 * rows * k * n for _, k, n, _ in LAYERS)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        for x, wq, ws, gate, res, act in work:
            if mode == "w8a8":
                xq, xs = oracle.quantize_rows(x)
                oracle.linear(oracle.MODE_W8A8, xq, wq, ws[:, 0].copy(), 0, x_scales=xs, gate=gate, residual=res, activation=act, fast=True)
            else:
                oracle.linear(oracle.MODE_W8A16, x, wq, ws, 0, gate=gate, residual=res, activation=act, fast=True)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    seconds = float(np.mean(times))
    return flop / seconds / 1e12, seconds, oracle.lib().h3o_threads()


def run_reference(args, rank):
    if rank != 0:
        return
    rows = 512
    value, seconds, cores = oracle_slab(rows, args.steps, args.warmup, args.mode)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.mode),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{rows}-row slab of each of the 4 GEMM shapes per step (the reference has no CPU linear; "
                                   "this is the CPU restatement of its shader arithmetic, blocked fp32 + OpenMP)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(mode="w8a16"):
    return {"workload": "DiT block linear stack (BASELINE config 2): M=32400 tokens per GPU, hidden 3072, FFN 12288, "
                        + ("W8A16 int8 weights with per-channel fp32 scales" if mode == "w8a16" else
                           "W8A8: int8 weights with per-channel scales, activations quantised per token in a fused kernel")
                        + "; QKV, attn-out(+gate,+residual), FFN-up(GELU-tanh), FFN-down(+gate,+residual)",
            "mode": mode,
            "rows_per_gpu": M_TOKENS, "hidden": HIDDEN, "ffn": FFN, "l2": "inputs_exceed_l2 (>= 199 MB per operand vs 126 MB L2)",
            "parallelism": "token-row sharding, weights replicated, no collective"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="h3q8")
    ap.add_argument("--case", default=None, choices=[name for name, _, _, _ in LAYERS + REAL_LAYERS + CONFIG_CASES] + ["helpers", "grouped_streams", "real_block_int8"],
                    help="profiling aid: run only this projection (with --rows) and print a short line")
    ap.add_argument("--rows", type=int, default=M_TOKENS, help="rows per GPU for --case")
    ap.add_argument("--workload", default="block", choices=["block", "stream", "tp_ffn"],
                    help="block: one DiT block stack, weights resident (default, BASELINE config 2); stream: the large render "
                         "(config 5): M=219,600 rows sharded over the GPUs, --layers layers of group-128 weights streamed "
                         "from pinned host memory through two device slots")
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--flush-l2", type=int, default=0, help="--case: write 256 MB between iterations and time each call on its own (cold L2)")
    ap.add_argument("--kernel", type=int, default=0, help="--case --graph 1: H3Q8_KERNEL_* selector of the raw call (0 = automatic)")
    ap.add_argument("--graph", type=int, default=0, help="--case: time raw h3q8_linear calls replayed from a CUDA graph (device time of skinny problems)")
    ap.add_argument("--stream-gather", type=int, default=0,
                    help="--workload stream at N > 1: each rank uploads 1/N of a layer, NCCL all-gather assembles it in the local slot")
    ap.add_argument("--group", type=int, default=-1, help="weight scale group for --case (default: 64 for real W8A16 shapes, else per channel)")
    ap.add_argument("--e2e-depth", type=int, default=4, help="end-to-end steps in flight (buffer sets)")
    ap.add_argument("--e2e-slices", type=int, default=1, help="row slices per end-to-end step (copy/compute overlap inside a step)")
    ap.add_argument("--e2e-edge-slices", type=int, default=4, help="row slices of the FIRST and LAST end-to-end step of a run: the pipeline "
                    "fills and drains a slice at a time instead of a whole batch at a time")
    ap.add_argument("--no-subrecords", action="store_true", help="default run: skip the w8a8 / config5_stream / tp_ffn sub-records")
    ap.add_argument("--mode", default="w8a16", choices=["w8a16", "w8a8"],
                    help="w8a16 (default, BASELINE config 2) or the W8A8 variant: per-token int8 activations, int8 MMAs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank)

    import torch
    import torch.distributed as dist
    os.environ["H3_CUDA_DEVICE"] = str(local)
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import h3cli_b200 as h
    from h3cli_b200 import api

    gpu = h.Gpu()
    gpu.quant_configure(2 if args.mode == "w8a8" else 1)
    stream = torch.cuda.ExternalStream(gpu.stream, device=local)
    lib = h.library()

    class _Span:
        """Zero-copy torch view of an h3_gpu tensor (CUDA array interface)."""

        def __init__(self, pointer, count):
            self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<i2", "data": (pointer, False), "version": 2}

    def device_bf16(rows, cols, mean=0.0, std=1.0, seed=0, replicated=False):
        """A resident h3_gpu bf16 tensor filled on the device with seeded normals (per rank unless replicated)."""
        gen = torch.Generator(device="cuda").manual_seed(seed if replicated else 1000 * rank + seed)
        t = gpu.tensor_new_bf16(rows * cols)
        view = torch.as_tensor(_Span(t.device_pointer, rows * cols), device=f"cuda:{local}").view(torch.bfloat16)
        chunk = 4096
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            block = torch.randn(r1 - r0, cols, generator=gen, device="cuda", dtype=torch.float32) * std + mean
            view[r0 * cols:r1 * cols].copy_(block.to(torch.bfloat16).reshape(-1))
        torch.cuda.synchronize()
        return t

    if args.case == "helpers":
        return run_helpers(args, gpu, lib, stream, device_bf16)
    if args.case == "grouped_streams":
        return run_grouped_streams(args, gpu, lib, stream, device_bf16)
    if args.case == "real_block_int8":
        return run_real_block_int8(args, gpu, lib, stream, device_bf16)
    if args.case:
        return run_case(args, gpu, lib, stream, device_bf16)
    if args.workload == "stream":
        return run_stream(args, gpu, lib, stream, device_bf16, rank, world, local)
    if args.workload == "tp_ffn":
        return run_tp_ffn(args, gpu, lib, stream, device_bf16, rank, world, local)

    # ---- the headline record (and, in the default W8A16 run, the W8A8 variant of the same step as a sub-record) ----
    dev = dict(torch=torch, dist=dist, rank=rank, world=world, local=local, lib=lib, stream=stream, device_bf16=device_bf16)
    line = measure_block(args, gpu, args.mode, dev)
    extra = {}
    if args.mode == "w8a16" and not args.no_subrecords:
        gpu.free()
        # W8A8 on the record: same step, per-token int8 activations, int8 MMAs, against a measured int8 peak
        gpu8 = h.Gpu()
        gpu8.quant_configure(2)
        dev8 = dict(dev, stream=torch.cuda.ExternalStream(gpu8.stream, device=local),
                    device_bf16=make_device_bf16(torch, gpu8, rank, local))
        sub = measure_block(args, gpu8, "w8a8", dev8, steps=max(5, args.steps // 2))
        gpu8.free()
        if sub:
            extra["w8a8"] = {k: sub[k] for k in ("value", "unit", "ms_per_step", "dtype", "roofline", "e2e", "gpu_launches", "int8_peak")}
        # the multi-GPU configuration (BASELINE config 5) strong-scaled over the ranks, and the tensor-parallel FFN:
        # short sub-records so that every N of a scaling run exercises the all-gather and the all-reduce
        gpu5 = h.Gpu()
        gpu5.quant_configure(1)
        dev5 = dict(dev, stream=torch.cuda.ExternalStream(gpu5.stream, device=local), device_bf16=make_device_bf16(torch, gpu5, rank, local))
        sub_args = argparse.Namespace(**vars(args))
        sub_args.layers, sub_args.steps, sub_args.stream_gather = 8, 10, 1
        stream_record = run_stream(sub_args, gpu5, lib, dev5["stream"], dev5["device_bf16"], rank, world, local, standalone=False)
        sub_args.steps, sub_args.warmup, sub_args.rows = 10, 3, M_TOKENS
        tp_record = run_tp_ffn(sub_args, gpu5, lib, dev5["stream"], dev5["device_bf16"], rank, world, local, standalone=False)
        gpu5.free()
        if stream_record:
            extra["config5_stream"] = {k: stream_record[k] for k in ("value", "unit", "n_gpus", "layers", "rows_total", "rows_this_rank", "scaling",
                                                                     "ms_per_layer", "seconds_per_pass", "weights_over", "allgather_ms_per_layer_comm_stream",
                                                                     "pcie_bytes_per_layer_this_rank", "stream_stalls", "slot_wait_ms_per_pass")}
            extra["config5_stream"]["note"] = "M = 219 600 rows over all ranks (strong scaling), 8 of the 48 layers, group-128 weights streamed from pinned host memory"
        if tp_record:
            extra["tp_ffn"] = {k: tp_record[k] for k in ("value", "unit", "n_gpus", "ms_per_block_ffn", "rows", "scaling", "allreduce_bytes_per_block",
                                                         "allreduce_ms_per_block_comm_stream", "parity_vs_unsharded_fused_call")}
    else:
        gpu.free()
    if rank == 0:
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def bind_to_gpu_numa_node(torch, local):
    """Runs this process (and so the threads that allocate and fill its pinned buffers) on the CPUs of the NUMA node
    the GPU hangs off: pinned memory is then first-touched next to the GPU's PCIe root.  Returns the node or None."""
    try:
        bus = torch.cuda.get_device_properties(local).pci_bus_id
        domain = torch.cuda.get_device_properties(local).pci_domain_id
        device = torch.cuda.get_device_properties(local).pci_device_id
        node = int(open(f"/sys/bus/pci/devices/{domain:04x}:{bus:02x}:{device:02x}.0/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return node
    except Exception:
        pass
    return None


_INT8_PEAK = {}


def int8_peak(torch):
    """Dense int8 tensor-core rate of this GPU, measured the way MEASURED_PEAKS.json measures bf16: torch._int_mm
    8192^3 (2 N^3 operations), best of 10 launches (burst) and back to back for about 2 s (sustained)."""
    if _INT8_PEAK:
        return _INT8_PEAK
    try:
        n = 8192
        a = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
        b = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8).t()      # column-major right operand
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None or ms < best else best
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        count = max(10, int(2000.0 / best))
        e0.record()
        for _ in range(count):
            torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        ops = 2.0 * n ** 3
        _INT8_PEAK.update({"tops": ops / best / 1e9, "tops_sustained": ops * count / e0.elapsed_time(e1) / 1e9,
                           "how": "torch._int_mm int8 8192^3 (2*N^3): best of 10 (burst) and back to back for ~2 s (sustained), CUDA events"})
        del a, b
        torch.cuda.empty_cache()
    except Exception as error:   # the library GEMM is only the yardstick; without it the bf16 figure is reported instead
        _INT8_PEAK.update({"tops": None, "tops_sustained": None, "how": f"torch._int_mm unavailable: {error}"})
    return _INT8_PEAK


def make_device_bf16(torch, gpu, rank, local):
    class _Span:
        """Zero-copy torch view of an h3_gpu tensor (CUDA array interface)."""

        def __init__(self, pointer, count):
            self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<i2", "data": (pointer, False), "version": 2}

    def device_bf16(rows, cols, mean=0.0, std=1.0, seed=0, replicated=False):
        """A resident h3_gpu bf16 tensor filled on the device with seeded normals (per rank unless replicated)."""
        gen = torch.Generator(device="cuda").manual_seed(seed if replicated else 1000 * rank + seed)
        t = gpu.tensor_new_bf16(rows * cols)
        view = torch.as_tensor(_Span(t.device_pointer, rows * cols), device=f"cuda:{local}").view(torch.bfloat16)
        chunk = 4096
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            block = torch.randn(r1 - r0, cols, generator=gen, device="cuda", dtype=torch.float32) * std + mean
            view[r0 * cols:r1 * cols].copy_(block.to(torch.bfloat16).reshape(-1))
        torch.cuda.synchronize()
        return t
    return device_bf16


def measure_block(args, gpu, mode, dev, steps=None):
    """One DiT block's four projections in `mode` on context `gpu`: resident value, roofline, end-to-end.  Returns the
    record (rank 0) or None."""
    torch, dist, rank, world, local, lib, stream, device_bf16 = (dev[k] for k in ("torch", "dist", "rank", "world", "local", "lib", "stream", "device_bf16"))
    steps = steps or args.steps
    # ---- operands (weights replicated on every rank: same seed) ----------------------------------
    weights, inputs, outputs = {}, {}, {}
    wgen = np.random.default_rng(42)
    for name, k, n, spec in LAYERS:
        wq = wgen.integers(-127, 128, (n, k), dtype=np.int8)
        ws = np.exp(wgen.normal(np.log(0.01), 0.3, (n, 1))).astype(np.float32)
        weights[name] = gpu.q8_from_host(wq, ws, 0)
        outputs[name] = gpu.tensor_new_bf16(M_TOKENS * n)
    x = device_bf16(M_TOKENS, HIDDEN, seed=1)
    hidden = device_bf16(M_TOKENS, FFN, seed=2)
    residual = device_bf16(M_TOKENS, HIDDEN, seed=3)
    gate = device_bf16(1, HIDDEN, 1.0, 0.1, seed=4)
    inputs = {"qkv": x, "attn_out": x, "ffn_up": x, "ffn_down": hidden}

    def enqueue_step():
        for name, k, n, spec in LAYERS:
            gpu.linear_fused_bf16(outputs[name], inputs[name], weights[name], None, gate if "g" in spec else None,
                                  residual if "r" in spec else None, M_TOKENS, k, n, 1 if "a" in spec else 0)
        gpu.continue_()      # commit without waiting, as the reference's block loop does between blocks

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: operands resident in HBM -----------------------------------------------------------
    gpu.begin()
    for _ in range(args.warmup):
        enqueue_step()
    gpu.submit()
    gpu.set_profiling(True)
    before = gpu.stats()
    gemm_launches_before = gpu.profile().linear_kernel_launches
    launches_before = lib.h3q8_kernel_launches()
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gpu.begin()
    start.record(stream)
    for _ in range(steps):
        enqueue_step()
    stop.record(stream)
    barrier()
    sampler.stop_flag = True
    gpu.submit()            # waits (already idle) and harvests the per-kernel events
    seconds = start.elapsed_time(stop) * 1e-3
    after = gpu.stats()
    launches = lib.h3q8_kernel_launches() - launches_before
    gpu.set_profiling(False)
    t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    job_seconds = float(t.item())
    value = world * FLOP_PER_STEP * steps / job_seconds / 1e12

    gemm_seconds = after.linear_seconds - before.linear_seconds
    gemm_launches = gpu.profile().linear_kernel_launches - gemm_launches_before
    burst, sustained, which = measured_peak()
    achieved = FLOP_PER_STEP * steps / gemm_seconds / 1e12 if gemm_seconds > 0 else None

    # ---- e2e: the same four operators, host buffers in, host buffer out ------------------------------
    # Chain as a DiT block calls them: x -> qkv; x -> attn_out (+gate, residual x) -> ffn_up (GELU) ->
    # ffn_down (+gate, residual h1).  Per step the block input crosses PCIe in and the block output out.
    # The rows are cut into E2E_CHUNKS slices with their own tensors, so that the upload of slice c+1 and the
    # download of slice c-1 (copy stream, h3q8_gpu_tensor_upload_async / _download_async) overlap the GEMMs of slice c.
    from h3cli_b200 import sharding
    numa_node = bind_to_gpu_numa_node(torch, local)    # before the pinned buffers are allocated and first touched
    host_x = torch.empty(M_TOKENS * HIDDEN, dtype=torch.int16).pin_memory()
    host_y = torch.empty(M_TOKENS * HIDDEN, dtype=torch.int16).pin_memory()
    lib.h3_gpu_tensor_read_bf16(x.handle, host_x.data_ptr(), M_TOKENS * HIDDEN)
    for tensor in list(outputs.values()) + [hidden, residual]:
        tensor.free()                                 # the resident-run tensors are no longer needed
    # DEPTH sets of slice tensors and host output buffers: steps i+1 .. i+DEPTH-1 are enqueued (their uploads start
    # at once on the upload stream) before the host waits for step i's output, so a stream of independent batches
    # keeps the upload stream, the compute stream and the download stream busy at the same time.
    E2E_CHUNKS = args.e2e_slices
    DEPTH = max(1, args.e2e_depth)
    host_out = [host_y] + [torch.empty(M_TOKENS * HIDDEN, dtype=torch.int16).pin_memory() for _ in range(DEPTH - 1)]
    def new_set(chunks):
        slices = []
        for begin, end in sharding.all_ranges(M_TOKENS, chunks):
            rows = end - begin
            slices.append(dict(rows=rows, offset=begin * HIDDEN * 2, x=gpu.tensor_new_bf16(rows * HIDDEN),
                               qkv=gpu.tensor_new_bf16(rows * 3 * HIDDEN), h1=gpu.tensor_new_bf16(rows * HIDDEN),
                               up=gpu.tensor_new_bf16(rows * FFN), y=gpu.tensor_new_bf16(rows * HIDDEN)))
        return slices

    sets = [new_set(E2E_CHUNKS) for _ in range(DEPTH)]
    # The first batch of a run cannot hide its upload behind anything and the last cannot hide its download: those two
    # batches are cut into EDGE row slices (own tensors), so compute starts after the first slice has arrived and the
    # last slice's download is all that trails the last GEMM.  Batches in between stay whole: a slice costs a second
    # pass of the weight dequantiser and smaller GEMMs, which only pays where nothing else overlaps the copy.
    EDGE = max(1, args.e2e_edge_slices)
    edge_sets = [new_set(EDGE), new_set(EDGE)] if EDGE != E2E_CHUNKS else None
    plan = {}                                         # step index -> tensor set in use

    def enqueue_e2e(index, count):
        if edge_sets and index == 0:
            slices = edge_sets[0]
        elif edge_sets and index == count - 1 and count > 1:
            slices = edge_sets[1]
        else:
            slices = sets[index % DEPTH]
        plan[index] = slices
        out = host_out[index % DEPTH]
        for c in slices:
            c["x"].upload_async(host_x.data_ptr() + c["offset"], c["rows"] * HIDDEN * 2)
        for c in slices:
            rows = c["rows"]
            gpu.linear_fused_bf16(c["qkv"], c["x"], weights["qkv"], None, None, None, rows, HIDDEN, 3 * HIDDEN, 0)
            gpu.linear_fused_bf16(c["h1"], c["x"], weights["attn_out"], None, gate, c["x"], rows, HIDDEN, HIDDEN, 0)
            gpu.linear_fused_bf16(c["up"], c["h1"], weights["ffn_up"], None, None, None, rows, HIDDEN, FFN, 1)
            gpu.linear_fused_bf16(c["y"], c["up"], weights["ffn_down"], None, gate, c["h1"], rows, FFN, HIDDEN, 0)
            gpu.continue_()
            c["y"].download_async(out.data_ptr() + c["offset"], rows * HIDDEN * 2)

    def finish_e2e(index):
        for c in plan.pop(index):
            c["y"].wait()                             # this step's block output is in host memory

    def run_e2e(count, depth):
        """depth 1: each step ends before the next is enqueued; depth d: d-1 steps in flight behind the current one."""
        begin = time.perf_counter()
        gpu.begin()                                   # one command scope; h3_gpu_continue commits each slice
        for i in range(count):
            enqueue_e2e(i, count)
            if i >= depth - 1:
                finish_e2e(i - (depth - 1))
        for i in range(max(0, count - (depth - 1)), count):
            finish_e2e(i)
        gpu.submit()                                  # surfaces deferred kernel errors; everything is already done
        return time.perf_counter() - begin

    def timed_e2e(depth):
        run_e2e(3, depth)
        gpu.synchronize()
        barrier()
        elapsed = run_e2e(steps, depth)
        barrier()
        t = torch.tensor([elapsed], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    e_serial = timed_e2e(1)
    gpu.set_profiling(True)                           # event pairs around the asynchronous copies (categories 4 and 5)
    copies_before = gpu.stats()
    e_seconds = timed_e2e(DEPTH)
    copies_after = gpu.stats()
    gpu.set_profiling(False)
    e2e_value = world * FLOP_PER_STEP * steps / e_seconds / 1e12
    h2d_seconds, d2h_seconds = copies_after.h2d_seconds - copies_before.h2d_seconds, copies_after.d2h_seconds - copies_before.d2h_seconds
    for slices in sets + (edge_sets or []):
        for c in slices:
            for key in ("x", "qkv", "h1", "up", "y"):
                c[key].free()
    for tensor in list(weights.values()) + [x, gate]:
        tensor.free()
    del host_out, host_x, host_y

    if rank != 0:
        return None
    cpu_value, cpu_seconds, cores = (None, None, None)
    if world == 1 and mode == args.mode:
        cpu_value, cpu_seconds, cores = oracle_slab(1024, 2, 1, mode)
    clocks = sampler.summary()
    step_bytes = M_TOKENS * HIDDEN * 2
    if mode == "w8a16":
        roofline = {"bound": "tensor", "kernel": "gemm_tcgen05_pair_kernel<bf16> (256x256 tile per CTA pair) after q8_dequant_kernel "
                                                 "(dequantise-to-scratch policy; the main-loop kernel gemm_tcgen05_pair_w8a16_kernel runs the same step at 0.71 of the burst peak)",
                    "achieved": achieved, "peak": burst, "unit": UNIT, "frac": achieved / burst if achieved else None,
                    "peak_source": f"bf16_tflops (burst) of {which}", "frac_of_sustained": achieved / sustained if achieved and sustained else None,
                    "launches": int(gemm_launches), "avg_launch_ms": gemm_seconds / max(gemm_launches, 1) * 1e3,
                    "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH}
        peak8 = None
    else:
        peak8 = int8_peak(torch)
        peak = peak8["tops"] or 2.0 * burst
        roofline = {"bound": "tensor", "kernel": "gemm_tcgen05_pair_kernel<int8> (256x256 tile per CTA pair) after quantize_segments_warp_kernel",
                    "achieved": achieved, "peak": peak, "unit": "TOP/s", "frac": achieved / peak if achieved else None,
                    "peak_source": "int8 dense rate measured in this run (int8_peak.tops, burst)" if peak8["tops"] else "2 x bf16_tflops (no int8 GEMM to measure with)",
                    "frac_of_sustained": achieved / peak8["tops_sustained"] if achieved and peak8["tops_sustained"] else None,
                    "launches": int(gemm_launches), "avg_launch_ms": gemm_seconds / max(gemm_launches, 1) * 1e3, "traffic": None}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT if mode == "w8a16" else "TOP/s", "n_gpus": world, "steps": steps, "warmup": args.warmup,
        "ms_per_step": job_seconds / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if mode == "w8a16" else "int8", "data": "synthetic", "config": workload_config(mode),
        "dit_block_linear_ms": job_seconds / steps * 1e3,
        "tensor_peak_fraction_per_gpu": value / world / burst,
        "e2e": {"value": e2e_value, "unit": UNIT if mode == "w8a16" else "TOP/s", "h2d_bytes_per_step": step_bytes,
                "d2h_bytes_per_step": step_bytes,
                "ms_per_step": e_seconds / steps * 1e3,
                "ms_per_step_one_at_a_time": e_serial / steps * 1e3,
                "h2d_gbs": step_bytes * steps / h2d_seconds / 1e9 if h2d_seconds > 0 else None,
                "d2h_gbs": step_bytes * steps / d2h_seconds / 1e9 if d2h_seconds > 0 else None,
                "pcie_gbs_needed_per_direction": step_bytes / (job_seconds / steps) / 1e9,
                "host_numa_node": numa_node,
                "path": "pinned host x -> h3q8_gpu_tensor_upload_async -> 4 x h3_gpu_linear_fused_bf16 per row slice (chained as "
                        "the DiT block calls them, " + str(E2E_CHUNKS) + " row slices so copies overlap compute) -> h3q8_gpu_tensor_download_async -> "
                        "pinned host y -> h3q8_gpu_tensor_wait; steps are independent batches with " + str(DEPTH) + " buffer sets: "
                        "later steps are enqueued before the host waits for step i's output (ms_per_step_one_at_a_time: no "
                        "step in flight behind the current one); the first and the last batch of the run are cut into " + str(EDGE) +
                        " row slices so that the pipeline fills and drains a slice at a time; host wall clock over all steps, max over ranks; h2d_gbs / d2h_gbs: "
                        "bytes / CUDA-event time of this rank's copies; the process is bound to the CPUs of the GPU's NUMA node "
                        "before its pinned buffers are allocated"},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
        "cpu_baseline": None if cpu_value is None else {
            "value": cpu_value, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "1024-row slab of each of the 4 GEMM shapes (0.232 TFLOP), blocked fp32 OpenMP restatement"},
    }
    if peak8:
        line["int8_peak"] = peak8
    return line


def run_tp_ffn(args, gpu, lib, stream, device_bf16, rank, world, local, standalone=True):
    """The optional tensor-parallel FFN: every rank sees all M rows; FFN-up is column-parallel (rank r owns FFN
    features [f0, f1), GELU stays local), FFN-down is row-parallel over the same features and stores fp32 partial
    sums.  The one all-reduce per block is issued as its two halves so that the bf16 rounding sits between them: a
    reduce-scatter adds the partial sums in fp32 and leaves every rank 1/N of the rows, the finishing call applies
    gate + residual and the single bf16 rounding to those rows, and an all-gather distributes the bf16 result --
    the same sums as an fp32 all-reduce, three quarters of its bytes on the wire and 1/N of the finishing work per
    rank.  The rows are cut into chunks so the communication of chunk c overlaps the GEMMs of chunk c+1."""
    import torch
    import torch.distributed as dist
    from h3cli_b200 import sharding
    rows_total, chunks = args.rows, 4
    f0, f1 = sharding.feature_range(FFN, rank, world)
    width = f1 - f0
    wgen = np.random.default_rng(42)                        # every rank draws the full weights, keeps its slices
    wup = wgen.integers(-127, 128, (FFN, HIDDEN), dtype=np.int8)
    sup = np.exp(wgen.normal(np.log(0.01), 0.3, (FFN, 1))).astype(np.float32)
    wdn = wgen.integers(-127, 128, (HIDDEN, FFN), dtype=np.int8)
    sdn = np.exp(wgen.normal(np.log(0.01), 0.3, (HIDDEN, 1))).astype(np.float32)
    up_slice = gpu.q8_from_host(np.ascontiguousarray(wup[f0:f1]), np.ascontiguousarray(sup[f0:f1]), 0)
    down_slice = gpu.q8_from_host(np.ascontiguousarray(wdn[:, f0:f1]), sdn, 0)
    gate = device_bf16(1, HIDDEN, 1.0, 0.1, seed=4, replicated=True)
    comm = torch.cuda.Stream()
    parts = []
    # chunk sizes are multiples of 8 * world rows, so that every rank's share of a chunk is whole and 16-byte aligned
    for c, (begin, end) in enumerate(sharding.reduce_chunks(rows_total, chunks, world)):
        rows = end - begin
        part = dict(rows=rows, x=device_bf16(rows, HIDDEN, seed=10 + c, replicated=True),
                    residual=device_bf16(rows, HIDDEN, seed=20 + c, replicated=True), hidden=gpu.tensor_new_bf16(rows * width),
                    partial=gpu.tensor_new_f32(rows * HIDDEN), y=gpu.tensor_new_bf16(rows * HIDDEN))
        share = rows // world                               # rows of this chunk that this rank finishes
        part["share"], part["first"] = share, rank * share
        part["view"] = torch.as_tensor(_Span32(part["partial"].device_pointer, rows * HIDDEN), device=f"cuda:{local}")
        part["y_view"] = torch.as_tensor(_Span16(part["y"].device_pointer, rows * HIDDEN), device=f"cuda:{local}").view(torch.bfloat16)
        if world > 1:
            part["reduced"] = gpu.tensor_new_f32(share * HIDDEN)
            part["reduced_view"] = torch.as_tensor(_Span32(part["reduced"].device_pointer, share * HIDDEN), device=f"cuda:{local}")
        parts.append(part)
    reduce_events = []
    comm_pointer = comm.cuda_stream

    def one_block(timed=False):
        for p in parts:
            gpu.linear_fused_bf16(p["hidden"], p["x"], up_slice, None, None, None, p["rows"], HIDDEN, width, 1)
            gpu.linear_partial_f32(p["partial"], p["hidden"], down_slice, p["rows"], width, HIDDEN)
            gpu.continue_()
            if world > 1:
                comm.wait_stream(stream)                    # this chunk's partial sums are complete
                with torch.cuda.stream(comm):
                    if timed:
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(comm)
                    dist.reduce_scatter_tensor(p["reduced_view"], p["view"])     # fp32 sums; this rank keeps its rows
                    offset = p["first"] * HIDDEN * 2
                    # gate + residual + the one bf16 rounding, on this rank's rows, on the communication stream
                    assert lib.h3q8_linear_finish(p["reduced"].device_pointer, p["share"], HIDDEN, None, gate.device_pointer,
                                                  p["residual"].device_pointer + offset, 0, p["y"].device_pointer + offset,
                                                  comm_pointer), lib.h3q8_last_error()
                    share = p["share"] * HIDDEN
                    dist.all_gather_into_tensor(p["y_view"], p["y_view"][rank * share:(rank + 1) * share])
                    if timed:
                        e1.record(comm)
                        reduce_events.append((e0, e1))
        if world > 1:
            stream.wait_stream(comm)
        else:
            for p in parts:
                gpu.linear_finish_bf16(p["y"], p["partial"], None, gate, p["residual"], p["rows"], HIDDEN, 0)
        gpu.continue_()

    gpu.begin()
    for _ in range(args.warmup):
        one_block()
    gpu.submit()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gpu.begin()
    start.record(stream)
    for _ in range(args.steps):
        one_block(timed=True)
    stop.record(stream)
    gpu.submit()
    torch.cuda.synchronize()
    seconds = torch.tensor([start.elapsed_time(stop) * 1e-3], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
    reduce_ms = sum(a.elapsed_time(b) for a, b in reduce_events) / max(args.steps, 1)
    # parity: rank 0 runs the unsharded fused FFN on the first chunk and compares
    record = None
    if rank == 0:
        p = parts[0]
        full_up, full_down = gpu.q8_from_host(wup, sup, 0), gpu.q8_from_host(wdn, sdn, 0)
        hidden, want = gpu.tensor_new_bf16(p["rows"] * FFN), gpu.tensor_new_bf16(p["rows"] * HIDDEN)
        gpu.begin()
        gpu.linear_fused_bf16(hidden, p["x"], full_up, None, None, None, p["rows"], HIDDEN, FFN, 1)
        gpu.linear_fused_bf16(want, hidden, full_down, None, gate, p["residual"], p["rows"], FFN, HIDDEN, 0)
        gpu.submit()
        f32 = lambda bits: (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)

        def ulps(got_bits, want_bits):
            got_v, want_v = f32(got_bits), f32(want_bits)
            floor = float(np.sqrt((want_v ** 2).mean()))
            ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(want_v), floor))) - 7)
            return np.abs(got_v - want_v) / ulp, float(np.sqrt(((got_v - want_v) ** 2).sum() / (want_v ** 2).sum()))

        # (a) the block output: gate * bf16(linear) + residual, rounded again; (b) the projection itself, bf16(linear)
        final_ulp, final_rel = ulps(p["y"].read(), want.read())
        plain, plain_tp = gpu.tensor_new_bf16(p["rows"] * HIDDEN), gpu.tensor_new_bf16(p["rows"] * HIDDEN)
        gpu.begin()
        gpu.linear_fused_bf16(plain, hidden, full_down, None, None, None, p["rows"], FFN, HIDDEN, 0)
        # the reduced fp32 sums this rank holds: all rows on one GPU, its share of the chunk (the first rows on rank 0) otherwise
        sums, held = (p["reduced"], p["share"]) if world > 1 else (p["partial"], p["rows"])
        gpu.linear_finish_bf16(plain_tp, sums, None, None, None, held, HIDDEN, 0)
        gpu.submit()
        linear_ulp, linear_rel = ulps(plain_tp.read()[:held * HIDDEN], plain.read()[:held * HIDDEN])
        report = {"rel_l2": final_rel, "max_bf16_ulp": float(final_ulp.max()), "fraction_beyond_2_ulp": float((final_ulp > 2.0).mean()),
                  "projection_only": {"rel_l2": linear_rel, "max_bf16_ulp": float(linear_ulp.max()),
                                      "fraction_not_bit_equal": float((linear_ulp > 0).mean())},
                  "rows_checked": p["rows"], "outputs_checked": int(final_ulp.size),
                  "bar": "rel-L2 <= 2e-3 and <= 2 bf16 ulp",
                  "note": "the fp32 sums differ from the unsharded call's only in summation order, so the projection bf16(linear) is at "
                          "most one step apart; where that step flips, gate * bf16(linear) + residual, rounded again at a smaller "
                          "exponent, can land up to three steps apart (the reference's own unfused chain does the same between any "
                          "two summation orders)"}
        for t in (full_up, full_down, hidden, want, plain, plain_tp):
            t.free()
        t = float(seconds.item())
        flop = 2.0 * rows_total * HIDDEN * FFN * 2 * args.steps
        record = {
            "metric": METRIC, "workload": "tp_ffn", "value": flop / t / 1e12, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "ms_per_block_ffn": t / args.steps * 1e3, "rows": rows_total, "ffn_features_this_rank": width, "row_chunks": chunks,
            "allreduce_bytes_per_block": rows_total * HIDDEN * (4 + 2) if world > 1 else 0, "allreduce_ms_per_block_comm_stream": reduce_ms,
            "collective": "reduce_scatter (fp32 partial sums) -> finish own rows -> all_gather (bf16 result)",
            "scaling": "strong", "dtype": "bf16", "data": "synthetic", "parity_vs_unsharded_fused_call": report,
            "config": {"workload": "tensor-parallel FFN (optional variant): FFN-up column-parallel with local GELU, FFN-down "
                                   "row-parallel into fp32 partial sums, one all-reduce per block issued as NCCL reduce-scatter (fp32) + "
                                   "all-gather (bf16) with gate + residual + the bf16 rounding between the two, chunked over rows "
                                   "and overlapped with the next chunk's GEMMs"}}
    for p in parts:
        for key in ("x", "residual", "hidden", "partial", "y", "reduced"):
            if key in p:
                p[key].free()
    for t in (up_slice, down_slice, gate):
        t.free()
    if standalone:
        if record:
            print(json.dumps(record), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        gpu.free()
    return record


class _Span32:
    """Zero-copy torch view of device fp32 words (CUDA array interface)."""

    def __init__(self, pointer, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (pointer, False), "version": 2}


class _Span16:
    """Zero-copy torch view of device 16-bit words (CUDA array interface)."""

    def __init__(self, pointer, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<i2", "data": (pointer, False), "version": 2}


class _ByteSpan:
    """Zero-copy torch view of device bytes (CUDA array interface)."""

    def __init__(self, pointer, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "|u1", "data": (pointer, False), "version": 2}


def run_stream(args, gpu, lib, stream, device_bf16, rank, world, local, standalone=True):
    """BASELINE config 5: 48 layers x 4 projections at M = 219,600 (rows sharded over the ranks, strong scaling),
    W8A16 per-group-128 weights (116.8 MB per layer) streamed from pinned host memory, two device slots, the copy
    of layer l+1 overlapping the compute of layer l."""
    import ctypes
    import torch
    import torch.distributed as dist
    from h3cli_b200 import sharding, q8_blob
    total_rows, group, unique = 219600, 128, 4
    begin, end = sharding.row_range(total_rows, rank, world)
    rows = end - begin
    shapes = [(n, k) for _, k, n, _ in LAYERS]
    sizes = [lib.h3q8_q8_blob_bytes(n, k, group, None) for n, k in shapes]
    offsets = [sum(sizes[:i]) for i in range(len(sizes))]
    align = world * 256                                                    # equal 256-byte aligned slices for --stream-gather
    slot_bytes = (sum(sizes) + align - 1) // align * align
    host = gpu.tensor_alloc(unique * slot_bytes, 2, 2)                    # int8, pinned host memory
    pointer = lib.h3_gpu_tensor_contents(host.handle)
    view = np.ctypeslib.as_array((ctypes.c_uint8 * (unique * slot_bytes)).from_address(pointer))
    wgen = np.random.default_rng(42)
    for u in range(unique):
        for (n, k), off in zip(shapes, offsets):
            wq = wgen.integers(-127, 128, (n, k), dtype=np.int8)
            ws = np.exp(wgen.normal(np.log(0.01), 0.3, (n, k // group))).astype(np.float32)
            blob = q8_blob(wq, ws, group)
            view[u * slot_bytes + off:u * slot_bytes + off + blob.size] = blob
    ring = gpu.weight_stream(slot_bytes, 2)
    views = [[ring.view(slot, off, n, k, group) for (n, k), off in zip(shapes, offsets)] for slot in range(2)]
    x, hidden, residual = device_bf16(rows, HIDDEN, seed=1), device_bf16(rows, FFN, seed=2), device_bf16(rows, HIDDEN, seed=3)
    gate = device_bf16(1, HIDDEN, 1.0, 0.1, seed=4)
    inputs = [x, x, x, hidden]
    outputs = [gpu.tensor_new_bf16(rows * n) for n, _ in shapes]

    # --stream-gather (N > 1): every rank pulls only its 1/N byte slice of the layer over PCIe into a staging buffer and
    # one NCCL all-gather over NVLink assembles the layer in each rank's local slot, on a communication stream, one layer
    # ahead of the compute stream.  The slot is local memory before any tensor map points at it.
    gather = bool(args.stream_gather) and world > 1
    gather_events = []
    if gather:
        piece = slot_bytes // world
        comm = torch.cuda.Stream()
        staging = [torch.empty(piece, dtype=torch.uint8, device="cuda") for _ in range(2)]
        host_bytes = torch.from_numpy(view)                 # the pinned host blobs as a CPU tensor (no copy)
        turn = [0]

        def fetch(layer):
            """Enqueue the fill of the next slot with layer `layer` on the communication stream; returns the slot."""
            blob = (layer % unique) * slot_bytes + rank * piece
            stage = staging[turn[0] % 2]
            turn[0] += 1
            with torch.cuda.stream(comm):
                slot, address = ring.reserve(comm.cuda_stream)
                stage.copy_(host_bytes[blob:blob + piece], non_blocking=True)
                target = torch.as_tensor(_ByteSpan(address, slot_bytes), device=f"cuda:{local}")
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(comm)
                dist.all_gather_into_tensor(target, stage)
                e1.record(comm)
                gather_events.append((e0, e1))
                ring.publish(slot, comm.cuda_stream, slot_bytes)
            return slot
    else:
        def fetch(layer):
            return ring.prefetch(pointer + (layer % unique) * slot_bytes, slot_bytes)

    def one_pass():
        slot = fetch(0)
        for layer in range(args.layers):
            upcoming = fetch(layer + 1) if layer + 1 < args.layers else None
            ring.acquire(slot)
            for i, (name, k, n, spec) in enumerate(LAYERS):
                gpu.linear_fused_bf16(outputs[i], inputs[i], views[slot][i], None, gate if "g" in spec else None,
                                      residual if "r" in spec else None, rows, k, n, 1 if "a" in spec else 0)
            ring.release(slot)
            gpu.continue_()
            slot = upcoming

    gpu.begin()
    one_pass()
    gpu.submit()
    gpu.set_profiling(True)
    before = gpu.stats()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    gather_events.clear()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    passes = max(1, args.steps // 10)
    gpu.begin()
    start.record(stream)
    for _ in range(passes):
        one_pass()
    stop.record(stream)
    gpu.submit()
    seconds = torch.tensor([start.elapsed_time(stop) * 1e-3], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
    after = gpu.stats()
    flop = sum(2.0 * total_rows * k * n for _, k, n, _ in LAYERS) * args.layers * passes
    torch.cuda.synchronize()
    gather_ms = sum(a.elapsed_time(b) for a, b in gather_events) / max(passes * args.layers, 1)
    gpu.set_profiling(False)
    record = None
    if rank == 0:
        t = float(seconds.item())
        record = {
            "metric": METRIC, "workload": "stream", "value": flop / t / 1e12, "unit": UNIT, "n_gpus": world, "passes": passes,
            "layers": args.layers, "rows_total": total_rows, "rows_this_rank": rows, "scaling": "strong",
            "ms_per_layer": t / passes / args.layers * 1e3, "seconds_per_pass": t / passes,
            "streamed_bytes_per_layer": slot_bytes, "pcie_bytes_per_layer_this_rank": slot_bytes // world if gather else slot_bytes,
            "weights_over": "pcie slice + nccl all-gather" if gather else "pcie (whole layer per rank)",
            "allgather_ms_per_layer_comm_stream": gather_ms if gather else 0.0,
            "h2d_gbs_this_rank": (after.streamed_bytes - before.streamed_bytes) / t / 1e9,
            "stream_stalls": int(after.stream_stalls - before.stream_stalls),
            "slot_wait_ms_per_pass": (after.stream_wait_seconds - before.stream_wait_seconds) / passes * 1e3, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"large render (BASELINE config 5): {args.layers}-layer DiT linear stack, M=219600 over all ranks, W8A16 "
                                   "group-128, weights streamed per layer from pinned host memory, 2 device slots"}}
    for t in views[0] + views[1] + outputs + [x, hidden, residual, gate]:
        t.free()
    ring.free()
    host.free()
    if standalone:
        if record:
            print(json.dumps(record), flush=True)
        if world > 1:
            dist.destroy_process_group()
        gpu.free()
    return record


def run_grouped_streams(args, gpu, lib, stream, device_bf16):
    """BASELINE's grouped-GEMM configuration: the video stream (M = 2 x 32 400, K = N = 3072) and the audio stream
    (M = 2 x 1 152, K = N = 1536) with separate int8 weight sets, as ONE call (one GEMM launch over both problems)
    and as two calls, same operands."""
    import torch
    specs = [("video", 2 * 32400, 3072, 3072), ("audio", 2 * 1152, 1536, 1536)]
    wgen = np.random.default_rng(42)
    problems = []
    for i, (_, rows, k, n) in enumerate(specs):
        wq = wgen.integers(-127, 128, (n, k), dtype=np.int8)
        ws = np.exp(wgen.normal(np.log(0.01), 0.3, (n, 1))).astype(np.float32)
        problems.append(dict(output=gpu.tensor_new_bf16(rows * n), input=device_bf16(rows, k, seed=30 + i), weight=gpu.q8_from_host(wq, ws, 0),
                             rows=rows, input_dim=k, output_dim=n))
    flop = sum(2.0 * rows * k * n for _, rows, k, n in specs)

    def timed(call):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        gpu.begin()
        for i in range(args.warmup + args.steps):
            if i == args.warmup:
                start.record(stream)
            call()
        stop.record(stream)
        gpu.submit()
        return start.elapsed_time(stop) / args.steps

    before = lib.h3q8_kernel_launches()
    together = timed(lambda: gpu.linear_grouped_bf16(problems))
    launches = (lib.h3q8_kernel_launches() - before) // (args.warmup + args.steps)
    separate = timed(lambda: [gpu.linear_fused_bf16(p["output"], p["input"], p["weight"], None, None, None, p["rows"], p["input_dim"],
                                                    p["output_dim"], 0) for p in problems])
    print(json.dumps({"case": "grouped_streams", "mode": args.mode, "problems": [dict(name=s[0], rows=s[1], k=s[2], n=s[3]) for s in specs],
                      "one_call_ms": together, "one_call_tflops": flop / together / 1e9, "kernels_per_call": int(launches),
                      "two_calls_ms": separate, "two_calls_tflops": flop / separate / 1e9}), flush=True)
    gpu.free()


def run_real_block_int8(args, gpu, lib, stream, device_bf16):
    """The real model's block (hidden 5376, 56 heads of 128, FFN 14336, SwiGLU) on the int8 operator family, issued by
    the C dispatcher (h3q8_dit_block_attention_input / _after_attention, the job of run_block()) with the policy the
    reference resolves on a backend with int8 operators: int8 QKV + norm + RoPE, head-major int8 attention output,
    gate + AdaLN + quantise in front of the MLP and in front of the next block's QKV.  Attention itself is outside this
    path, so its output is a resident synthetic tensor in SDPA's [head, row, dimension] layout."""
    import ctypes
    import torch
    from h3cli_b200 import api
    rows, hidden, heads, dim, half, ffn, slots = args.rows, 5376, 56, 128, 48, 14336, 6
    padded = (rows + 127) // 128 * 128
    wgen = np.random.default_rng(42)

    def weight(n, k, scale):
        w = gpu.tensor_from_i8(wgen.integers(-127, 128, (n, k), dtype=np.int8))
        return w, gpu.tensor_from_f32(np.exp(wgen.normal(np.log(scale), 0.3, n)).astype(np.float32))

    w_qkv, s_qkv = weight(3 * heads * dim, hidden, 0.01)
    w_out, s_out = weight(hidden, heads * dim, 0.01)
    w_fc1, s_fc1 = weight(2 * ffn, hidden, 0.002)
    w_fc2, s_fc2 = weight(hidden, ffn, 0.01)
    qn, kn = device_bf16(1, dim, 1.0, 0.1, seed=5), device_bf16(1, dim, 1.0, 0.1, seed=6)
    norm1, norm2 = device_bf16(1, hidden, 1.0, 0.1, seed=9), device_bf16(1, hidden, 1.0, 0.1, seed=11)
    modulation = device_bf16(1, slots * hidden, 0.0, 0.1, seed=10)
    cos, sin = device_bf16(rows, half, 0.0, 0.7, seed=7), device_bf16(rows, half, 0.0, 0.7, seed=8)
    buffers = dict(hidden=device_bf16(rows, hidden, seed=1), mod_attention=gpu.tensor_new_bf16(rows * hidden), qkv=None,
                   query=gpu.tensor_new_bf16(rows * heads * dim), key=gpu.tensor_new_bf16(rows * heads * dim),
                   value=gpu.tensor_new_bf16(rows * heads * dim), attention_heads=device_bf16(rows, heads * dim, seed=2),
                   attention_output=gpu.tensor_new_bf16(rows * hidden), mod_mlp=gpu.tensor_new_bf16(rows * hidden),
                   mlp_output=gpu.tensor_new_bf16(rows * hidden), activated=gpu.tensor_new_bf16(rows * ffn),
                   int8_activation=gpu.tensor_new_i8(padded * ffn), int8_activation_scales=gpu.tensor_new_f32(padded * (ffn // 1024)))
    c_buffers = api.DitBuffers(**{name: t.handle if t else None for name, t in buffers.items()})
    c_weights = api.DitWeights(qkv_int8=w_qkv.handle, qkv_scales=s_qkv.handle, out_int8=w_out.handle, out_scales=s_out.handle,
                               fc1_int8=w_fc1.handle, fc1_scales=s_fc1.handle, fc2_int8=w_fc2.handle, fc2_scales=s_fc2.handle,
                               q_norm=qn.handle, k_norm=kn.handle, norm1=norm1.handle, norm2=norm2.handle)
    shape = api.DitShape(rows, hidden, heads, dim, half, ffn, slots, 1e-6)
    policy = api.DitPolicy()
    assert lib.h3q8_dit_linear_policy_resolve(gpu.handle, rows, 0, ctypes.byref(policy))
    ready, quantized = ctypes.c_int(0), ctypes.c_int(0)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]

    def block(timed=False):
        """One block; its tail is fused with the next block's attention AdaLN + quantiser (same weights stand in)."""
        mark = (lambda i: marks[i].record(stream)) if timed else (lambda i: None)
        mark(0)
        if not lib.h3q8_dit_block_attention_input(gpu.handle, ctypes.byref(policy), ctypes.byref(shape), ctypes.byref(c_weights),
                                                  ctypes.byref(c_buffers), modulation.handle, None, cos.handle, sin.handle, ready.value,
                                                  quantized.value):
            raise RuntimeError(gpu.error())
        mark(1)
        if not lib.h3q8_dit_block_after_attention(gpu.handle, ctypes.byref(policy), ctypes.byref(shape), ctypes.byref(c_weights), norm1.handle,
                                                  ctypes.byref(c_buffers), modulation.handle, modulation.handle, None, 1, ctypes.byref(ready),
                                                  ctypes.byref(quantized)):
            raise RuntimeError(gpu.error())
        mark(2)
        gpu.continue_()

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gpu.begin()
    block()                                                   # the first block still runs the attention AdaLN itself
    before = lib.h3q8_kernel_launches()
    for i in range(args.warmup + args.steps):
        if i == args.warmup:
            start.record(stream)
        block()
    stop.record(stream)
    launches = lib.h3q8_kernel_launches() - before
    block(timed=True)
    gpu.submit()
    ms = start.elapsed_time(stop) / args.steps
    parts = [marks[i].elapsed_time(marks[i + 1]) for i in range(2)]
    ops = 2.0 * rows * (hidden * 3 * heads * dim + heads * dim * hidden + hidden * 2 * ffn + ffn * hidden)
    print(json.dumps({"case": "real_block_int8", "rows": rows, "hidden": hidden, "heads": heads, "ffn": ffn, "ms_per_block": ms,
                      "tops": ops / ms / 1e9, "kernels_per_block": int(launches // (args.warmup + args.steps)),
                      "policy": {name: int(getattr(policy, name)) for name, _ in api.DitPolicy._fields_},
                      "next_block_flags": {"attention_adaln_ready": ready.value, "attention_input_quantized": quantized.value},
                      "ms_per_call": dict(zip(["h3q8_dit_block_attention_input", "h3q8_dit_block_after_attention"], parts)),
                      "operators": ["h3_gpu_grouped_qkv_linear_rope_int8 (pre-quantised input)", "h3_gpu_linear_int8_head_major_bf16",
                                    "h3_gpu_gate_adaln_quantize_int8", "h3_gpu_mlp_int8_bf16",
                                    "h3_gpu_gate_adaln_quantize_int8 (MLP gate + next attention AdaLN)"]}), flush=True)
    gpu.free()


def run_helpers(args, gpu, lib, stream, device_bf16):
    """The memory-bound kernels beside the GEMM, each timed alone with CUDA events against the measured copy
    bandwidth: algorithmic bytes (what must cross HBM once) / time.  Operands exceed L2 (126 MB)."""
    import torch
    rows, hidden, ffn = args.rows, HIDDEN, FFN
    burst, _, which = measured_peak()
    try:
        hbm = float(json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))["hbm_gbs"])
        source = "measured"
    except (OSError, KeyError, ValueError):
        hbm, source = 6650.0, "fallback"
    x = device_bf16(rows, ffn, seed=1)                       # [rows, 12288] bf16 = 796 MB at 32 400 rows
    branch, residual = device_bf16(rows, hidden, seed=2), device_bf16(rows, hidden, seed=3)
    q, sc = gpu.tensor_new_i8(rows * ffn), gpu.tensor_new_f32(rows * (ffn // 1024))
    wbf = device_bf16(ffn, ffn, 0.0, 0.02, seed=4)           # [12288, 12288] bf16 weight = 302 MB
    wq, ws = gpu.tensor_new_i8(ffn * ffn), gpu.tensor_new_f32(ffn * (ffn // 128))
    wout = gpu.tensor_new_bf16(ffn * ffn)
    norm_w, mod = device_bf16(1, hidden, 1.0, 0.1, seed=5), device_bf16(1, 3 * hidden, 0.0, 0.1, seed=6)
    gated, q3, s3 = gpu.tensor_new_bf16(rows * hidden), gpu.tensor_new_i8(rows * hidden), gpu.tensor_new_f32(rows)
    wide = 5376
    branch5, residual5 = device_bf16(rows, wide, seed=12), device_bf16(rows, wide, seed=13)
    norm5, mod5 = device_bf16(1, wide, 1.0, 0.1, seed=14), device_bf16(1, 3 * wide, 0.0, 0.1, seed=15)
    gated5, q5 = gpu.tensor_new_bf16(rows * wide), gpu.tensor_new_i8(rows * wide)
    p = lambda t: t.device_pointer
    cases = [
        ("quantize_rows_kernel [M,3072]", lambda: lib.h3q8_quantize_rows(p(branch), p(q3), p(s3), rows, rows, hidden, 1.0, gpu.stream),
         rows * hidden * 3 + rows * 4),
        ("quantize_rows_kernel [M,12288]", lambda: lib.h3q8_quantize_rows(p(x), p(q), p(sc), rows, rows, ffn, 1.0, gpu.stream),
         rows * ffn * 3 + rows * 4),
        ("quantize_rows_kernel grouped 1024 [M,12288]", lambda: lib.h3q8_quantize_rows_grouped(p(x), p(q), p(sc), rows, rows, ffn, 1024, gpu.stream),
         rows * ffn * 3 + rows * (ffn // 1024) * 4),
        ("q8_pack_rows_kernel [12288,12288] group 128", lambda: lib.h3q8_q8_pack_rows_device(p(wbf), p(wq), p(ws), ffn, ffn, 128, gpu.stream),
         ffn * ffn * 3 + ffn * (ffn // 128) * 4),
        ("q8_dequant_kernel [12288,12288] group 128", lambda: lib.h3q8_q8_dequant(p(wq), p(ws), p(wout), ffn, ffn, 128, gpu.stream),
         ffn * ffn * 3 + ffn * (ffn // 128) * 4),
        ("gate_adaln_quantize_kernel [M,3072]", lambda: gpu.gate_adaln_quantize_int8(gated, q3, s3, residual, branch, norm_w, mod, mod, None, rows, rows,
                                                                                  hidden, 3, 0, 1, 2, 1e-6),
         rows * hidden * (2 + 2 + 2 + 1) + rows * 4),
        ("gate_adaln_quantize_kernel [M,5376]", lambda: gpu.gate_adaln_quantize_int8(gated5, q5, s3, residual5, branch5, norm5, mod5, mod5, None, rows,
                                                                                  rows, wide, 3, 0, 1, 2, 1e-6),
         rows * wide * (2 + 2 + 2 + 1) + rows * 4),
    ]
    out = []
    for name, call, nbytes in cases:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        gpu.begin()
        for i in range(args.warmup + args.steps):
            if i == args.warmup:
                start.record(stream)
            assert call()
        stop.record(stream)
        gpu.submit()
        ms = start.elapsed_time(stop) / args.steps
        out.append({"kernel": name, "ms": ms, "algorithmic_bytes": nbytes, "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / hbm})
    print(json.dumps({"case": "helpers", "rows": rows, "hbm_peak_gbs": hbm, "peak_source": source, "kernels": out}), flush=True)
    gpu.free()


def run_case(args, gpu, lib, stream, device_bf16):
    """One projection at --rows rows: the small workload used under ncu."""
    import torch
    name, k, n, spec = next(layer for layer in LAYERS + REAL_LAYERS + CONFIG_CASES if layer[0] == args.case)
    rows = args.rows
    real = name.startswith("real_")
    wrows = 2 * n if "s" in spec else n
    group = args.group if args.group >= 0 else 64 if real and args.mode == "w8a16" else 0
    wgen = np.random.default_rng(42)
    wq = wgen.integers(-127, 128, (wrows, k), dtype=np.int8)
    ws = np.exp(wgen.normal(np.log(0.002 if "s" in spec else 0.01), 0.3, (wrows, k // group if group else 1))).astype(np.float32)
    weight = gpu.q8_from_host(wq, ws, group)
    x, out = device_bf16(rows, k, seed=1), gpu.tensor_new_bf16(rows * n)
    residual = device_bf16(rows, n, seed=3) if "r" in spec else None
    gate = device_bf16(1, n, 1.0, 0.1, seed=4) if "g" in spec else None
    bias = device_bf16(1, n, 0.0, 0.02, seed=9) if "b" in spec else None
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if "q" in spec:   # QKV projection with per-head RMS norm + RoPE in the epilogue: 56 heads x 128, rotary half 48
        heads, half = n // 384, 48
        q, kk, v = (gpu.tensor_new_bf16(rows * heads * 128) for _ in range(3))
        qn, kn = device_bf16(1, 128, 1.0, 0.1, seed=5), device_bf16(1, 128, 1.0, 0.1, seed=6)
        cos, sin = device_bf16(rows, half, 0.0, 0.7, seed=7), device_bf16(rows, half, 0.0, 0.7, seed=8)
    if args.graph:
        # Skinny problems are shorter than a host launch: capture `steps` raw calls in a CUDA graph and time replays,
        # so the figure is device time.  W8A16 reads the int8 weight directly (main-loop dequantisation, split-K).
        import ctypes
        import h3cli_b200 as h
        from h3cli_b200.api import LinearDesc
        mode = {"w8a16": h.MODE_W8A16, "w8a8": h.MODE_W8A8}[args.mode]
        nbytes = lib.h3q8_linear_workspace_bytes(mode, rows, k, n)
        workspace = gpu.tensor_alloc(max(nbytes, 256), 2)
        # The weight is the traffic: consecutive calls read DIFFERENT copies of it, 384 MB in all (three times the L2),
        # so that every call streams its weight from HBM instead of finding the previous call's copy in L2.
        copies = max(1, min(args.steps, -(-384 * 1024 * 1024 // (wrows * k))))
        weights = [weight] + [gpu.q8_from_host(wq, ws, group) for _ in range(copies - 1)]
        descs = []
        if mode == h.MODE_W8A8:
            xq, xs = gpu.tensor_new_i8(rows * k), gpu.tensor_new_f32(rows)
            assert lib.h3q8_quantize_rows(x.device_pointer, xq.device_pointer, xs.device_pointer, rows, rows, k, 1.0, gpu.stream)
        for w in weights:
            d = LinearDesc(mode=mode, rows=rows, input_dim=k, output_dim=n, input=x.device_pointer, weight=w.device_pointer,
                           weight_scales=w.device_pointer + ((wrows * k + 15) & ~15), weight_group=group,
                           gate=gate.device_pointer if gate else None, residual=residual.device_pointer if residual else None,
                           activation=1 if "a" in spec else 0, output=out.device_pointer,
                           workspace=workspace.device_pointer if nbytes else None, workspace_bytes=nbytes, kernel=args.kernel)
            if mode == h.MODE_W8A8:
                d.input, d.input_scales = xq.device_pointer, xs.device_pointer
            descs.append(d)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(3):
                assert lib.h3q8_linear(ctypes.byref(descs[i % copies]), side.cuda_stream), lib.h3q8_last_error()
        torch.cuda.synchronize()
        before = lib.h3q8_kernel_launches()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(args.steps):
                assert lib.h3q8_linear(ctypes.byref(descs[i % copies]), side.cuda_stream), lib.h3q8_last_error()
        per_step = (lib.h3q8_kernel_launches() - before) // args.steps
        graph.replay()
        torch.cuda.synchronize()
        best = None
        for _ in range(5):
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(stop) / args.steps
            best = ms if best is None or ms < best else best
        assert lib.h3q8_device_status(None) == 0
        print(json.dumps({"case": name, "mode": args.mode, "group": group, "rows": rows, "k": k, "n": n, "timing": "cuda graph replay",
                          "l2": "calls rotate over %d copies of the weight (%d MB in all): every call reads its weight from HBM" % (copies, copies * wrows * k >> 20),
                          "kernels_per_call": int(per_step), "ms": best, "tflops": 2.0 * rows * k * wrows / best / 1e9,
                          "weight_gbs": wrows * k / best / 1e6, "workspace_bytes": int(nbytes)}), flush=True)
        gpu.free()
        return
    def call():
        if "q" in spec:
            gpu.grouped_qkv_linear_rope_bf16(q, kk, v, None, x, weight, qn, kn, cos, sin, rows, k, heads, 128, half, 1e-5)
        else:
            gpu.linear_fused_bf16(out, x, weight, bias, gate, residual, rows, k, n, 2 if "s" in spec else 1 if "a" in spec else 0)

    gpu.begin()
    for i in range(args.warmup + args.steps):
        if i == args.warmup:
            start.record(stream)
        call()
    stop.record(stream)
    gpu.submit()
    ms = start.elapsed_time(stop) / args.steps
    record = {"case": name, "mode": args.mode, "group": group, "rows": rows, "k": k, "n": n, "ms": ms, "tflops": 2.0 * rows * k * wrows / ms / 1e9,
              "weight_gbs": wrows * k / ms / 1e6, "launches": int(lib.h3q8_kernel_launches())}
    if args.flush_l2:
        # cold L2: 256 MB are written on the same stream between calls, and every call is timed on its own
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        gpu.begin()
        for first, last in pairs:
            with torch.cuda.stream(stream):
                flush.zero_()
            first.record(stream)
            call()
            last.record(stream)
        gpu.submit()
        cold = sorted(first.elapsed_time(last) for first, last in pairs)
        record.update({"ms_cold_l2_median": cold[len(cold) // 2], "ms_cold_l2_min": cold[0],
                       "tflops_cold_l2": 2.0 * rows * k * wrows / cold[len(cold) // 2] / 1e9, "l2": "256 MB written between calls"})
    print(json.dumps(record), flush=True)
    gpu.free()


if __name__ == "__main__":
    main()
