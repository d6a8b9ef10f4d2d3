"""The N > 1 host logic on CPU ranks (gloo, world size 2): the row-sharding plan,
the "concatenation of shard outputs equals the whole" property that makes the
multi-GPU path collective-free, and the max-over-ranks timing reduce that
bench.py uses.  Each rank computes its shard with the CPU oracle (the checker
stands in for the GPU here; the GPU-side version of the same property is in
test_gpu_parity.py::test_config1_single_w8a16)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from h3cli_b200 import sharding, synth  # noqa: E402


def test_row_ranges_partition_and_align():
    for rows in (1, 127, 128, 129, 4096, 32400, 219600):
        for world in (1, 2, 3, 4, 8):
            ranges = sharding.all_ranges(rows, world)
            assert ranges[0][0] == 0 and ranges[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            assert all(e >= b for b, e in ranges)
            if rows >= 128 * world * 4:
                assert all(b % 128 == 0 for b, _ in ranges)
                sizes = [e - b for b, e in ranges]
                assert max(sizes) - min(sizes) <= 256
    with pytest.raises(ValueError):
        sharding.row_range(10, 2, 2)


def _worker(rank, world, port, result_queue):
    import torch
    import torch.distributed as dist
    import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M, N, K = 517, 48, 192
    x = synth.activations(5, 1, M, K).reshape(M, K)         # every rank can regenerate any rows
    wq, ws = synth.int8_weights(5, 2, N, K), synth.lognormal_scales(5, 3, N, 3)
    begin, end = sharding.row_range(M, rank, world)
    mine = synth.activations(5, 1, end - begin, K, row0=begin).reshape(end - begin, K)
    assert (mine == x[begin:end]).all()                     # counter-based generator: shard == slice
    part = oracle.linear(oracle.MODE_W8A16, mine, wq, ws, 64, activation=1)
    padded = np.zeros((M, N), np.int32)
    padded[begin:end] = part
    gathered = torch.from_numpy(padded)
    dist.all_reduce(gathered)                               # shards are disjoint: the sum is the concatenation
    # streamed layers at N > 1: each rank holds one aligned byte slice, an all-gather assembles the blob
    blob = np.frombuffer(synth.int8_weights(6, 1, 1, 70001).tobytes(), dtype=np.uint8)
    padded, piece = sharding.blob_slices(blob.size, world)
    whole_blob = np.zeros(padded, np.uint8)
    whole_blob[:blob.size] = blob
    pieces = [torch.zeros(piece, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(pieces, torch.from_numpy(whole_blob[rank * piece:(rank + 1) * piece].copy()))
    assert piece % 256 == 0 and (torch.cat(pieces).numpy() == whole_blob).all()
    # tensor-parallel FFN: GELU(x Wup[f0:f1]^T) Wdown[:, f0:f1]^T summed over the ranks == the unsharded FFN
    F, H = 512, 64
    xin = synth.activations(7, 1, 40, H).reshape(40, H)
    wup, sup = synth.int8_weights(7, 2, F, H), synth.lognormal_scales(7, 3, F, 1)
    wdn, sdn = synth.int8_weights(7, 4, H, F), synth.lognormal_scales(7, 5, H, 1)
    f0, f1 = sharding.feature_range(F, rank, world)
    hid = oracle.linear(oracle.MODE_W8A16, xin, wup[f0:f1], sup[f0:f1], 0, activation=1)
    partial = oracle.linear(oracle.MODE_W8A16, hid, np.ascontiguousarray(wdn[:, f0:f1]), sdn, 0)
    total = torch.from_numpy((partial.astype(np.uint32) << 16).view(np.float32).copy())
    dist.all_reduce(total)                                  # fp32 sum of the bf16 partial sums
    hid_all = oracle.linear(oracle.MODE_W8A16, xin, wup, sup, 0, activation=1)
    whole_ffn = (oracle.linear(oracle.MODE_W8A16, hid_all, wdn, sdn, 0).astype(np.uint32) << 16).view(np.float32)
    ffn_error = float(np.linalg.norm(total.numpy() - whole_ffn) / np.linalg.norm(whole_ffn))
    assert ffn_error < 4e-3                                 # each partial is rounded to bf16 once: tolerance parity only
    seconds = torch.tensor([0.5 + rank], dtype=torch.float64)
    dist.all_reduce(seconds, op=dist.ReduceOp.MAX)          # job time = slowest rank
    if rank == 0:
        whole = oracle.linear(oracle.MODE_W8A16, x, wq, ws, 64, activation=1)
        result_queue.put((bool((gathered.numpy() == whole.astype(np.int32)).all()), float(seconds.item())))
    dist.barrier()
    dist.destroy_process_group()


def test_reduce_chunks_give_every_rank_a_whole_share():
    for rows in (32400, 4096, 219600, 64, 8):
        for world in (1, 2, 4, 8):
            for chunks in (1, 4):
                got = sharding.reduce_chunks(rows, chunks, world)
                assert got[0][0] == 0 and got[-1][1] == rows and all(a[1] == b[0] for a, b in zip(got, got[1:]))
                assert all((e - b) % world == 0 for b, e in got)
                assert all((e - b) % (8 * world) == 0 for b, e in got[:-1])
    with pytest.raises(ValueError):
        sharding.reduce_chunks(32401, 4, 2)


def test_blob_and_feature_splits():
    for total in (0, 1, 255, 256, 116785152, 116785153):
        for world in (1, 2, 4, 8):
            padded, piece = sharding.blob_slices(total, world)
            assert padded >= total and padded - total < world * 256 and piece * world == padded and piece % 256 == 0
    assert [sharding.feature_range(12288, r, 8) for r in (0, 7)] == [(0, 1536), (10752, 12288)]
    with pytest.raises(ValueError):
        sharding.feature_range(12288, 0, 5)


def test_two_rank_sharded_linear_equals_whole():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    same, seconds = queue.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same and seconds == 1.5
