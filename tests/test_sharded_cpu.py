"""Host logic of the sharded path on CPU: partitions, shard byte ranges, and the exchange
steps with world_size 2 over gloo.  Each rank's compute is done by the CPU oracle here;
the GPU kernels take its place in tests/test_sharded_gpu.py."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

from fortai_b200 import sharded


def test_partition_is_balanced_and_covers_everything():
    for total, parts, multiple in ((151936, 8, 1), (151936, 4, 1), (17408, 8, 32), (9728, 3, 32),
                                   (10, 4, 1), (100, 8, 32), (0, 2, 1)):
        ranges = sharded.partition(total, parts, multiple)
        assert len(ranges) == parts
        assert ranges[0][0] == 0
        for (f0, c0), (f1, _) in zip(ranges, ranges[1:]):
            assert f0 + c0 == f1
        assert ranges[-1][0] + ranges[-1][1] == total
        sizes = [c for _, c in ranges]
        full = [c for c in sizes if c % multiple == 0]
        assert max(full) - min(full) <= multiple
    assert sharded.partition(151936, 8) == [(i * 18992, 18992) for i in range(8)]
    assert sharded.partition(17408, 8, 32) == [(i * 2176, 2176) for i in range(8)]
    with pytest.raises(ValueError):
        sharded.partition(10, 0)


def test_shard_bytes_match_row_and_column_slices(oracle):
    rows, width = 12, 128
    w = oracle.make_weights(rows, width, seed=4)
    full = w.reshape(rows, width // 32, 34)
    assert np.array_equal(sharded.row_shard_bytes(w, rows, width, 3, 5).reshape(5, 4, 34),
                          full[3:8])
    assert np.array_equal(sharded.column_shard_bytes(w, rows, width, 1, 2).reshape(rows, 2, 34),
                          full[:, 1:3])
    with pytest.raises(ValueError):
        sharded.row_shard_bytes(w, rows, width, 10, 5)
    with pytest.raises(ValueError):
        sharded.column_shard_bytes(w, rows, width, 3, 2)


def _worker(rank, world, port, result_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import q8_oracle as o
    failures = []
    # ---- row-sharded matvec + all-gather (uneven split on purpose: 131 rows)
    rows, width = 131, 256
    w = o.make_weights(rows, width, seed=1)
    x = o.normal(width, seed=2)
    expected = o.matvec(w, rows, width, x)[0]
    ranges = sharded.partition(rows, world)
    first, count = ranges[rank]
    local = o.matvec(sharded.row_shard_bytes(w, rows, width, first, count), count, width, x)[0]
    full = sharded.all_gather_rows(dist, torch.from_numpy(local), [c for _, c in ranges]).numpy()
    if not np.array_equal(full, expected):
        failures.append("row-sharded matvec differs from the unsharded oracle")
    # ---- even split takes the single-tensor all-gather
    rows2 = 128
    w2 = o.make_weights(rows2, width, seed=3)
    expected2 = o.matvec(w2, rows2, width, x)[0]
    ranges2 = sharded.partition(rows2, world)
    f2, c2 = ranges2[rank]
    local2 = o.matvec(sharded.row_shard_bytes(w2, rows2, width, f2, c2), c2, width, x)[0]
    full2 = sharded.all_gather_rows(dist, torch.from_numpy(local2), [c for _, c in ranges2]).numpy()
    if not np.array_equal(full2, expected2):
        failures.append("evenly sharded matvec differs from the unsharded oracle")
    # ---- FFN: gate/up by rows, down by columns, all-reduce of the partial outputs
    hidden, inner = 64, 192
    gate, up = o.make_weights(inner, hidden, seed=5), o.make_weights(inner, hidden, seed=6)
    down = o.make_weights(hidden, inner, seed=7)
    xh = o.normal(hidden, seed=8)
    expected_ffn = o.ffn(gate, up, down, inner, hidden, hidden, xh)
    fr = sharded.partition(inner, world, multiple=32)
    ff, fc = fr[rank]
    g = sharded.row_shard_bytes(gate, inner, hidden, ff, fc)
    u = sharded.row_shard_bytes(up, inner, hidden, ff, fc)
    d = sharded.column_shard_bytes(down, hidden, inner, ff // 32, fc // 32)
    partial = o.ffn(g, u, d, fc, hidden, hidden, xh)
    total = sharded.all_reduce_sum(dist, torch.from_numpy(partial.copy()), world).numpy()
    bound = 2e-5 * float(np.linalg.norm(expected_ffn.astype(np.float64)))
    if float(np.abs(total - expected_ffn).max()) > bound:
        failures.append("sharded FFN differs from the unsharded oracle")
    # every rank must hold the same assembled vectors
    check = torch.from_numpy(full.copy())
    dist.all_reduce(check, op=dist.ReduceOp.MAX)
    if not np.array_equal(check.numpy(), full):
        failures.append("ranks disagree after the all-gather")
    with open(f"{result_path}.{rank}", "w") as f:
        f.write("\n".join(failures))
    dist.destroy_process_group()


def test_two_ranks_over_gloo_reproduce_the_unsharded_oracle(tmp_path, oracle):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    result = str(tmp_path / "result")
    mp.spawn(_worker, args=(world, port, result), nprocs=world, join=True)
    for rank in range(world):
        assert open(f"{result}.{rank}").read() == ""
