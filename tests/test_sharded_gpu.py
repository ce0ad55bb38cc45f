"""Sharded paths on real GPUs.  Single-GPU parts check the shard kernels against the
oracle; the multi-rank part spawns one process per GPU (needs >= 2 GPUs)."""
import os
import sys

import numpy as np
import pytest

from conftest import ROOT, l2_tolerance

pytestmark = pytest.mark.gpu


def test_row_shards_on_one_gpu_reproduce_the_full_matvec(backend, context, dev, oracle):
    from fortai_b200 import sharded
    rows, width, world = 1003, 2560, 4
    weights = oracle.make_weights(rows, width, seed=1)
    x = oracle.normal(width, seed=2)
    expected = oracle.matvec(weights, rows, width, x)[0]
    dx = dev.to_device(x)
    out = np.zeros(rows, np.float32)
    for rank in range(world):
        shard = sharded.RowShardedMatvec(backend, context, weights, rows, width, rank, world)
        dout = dev.buffer(4 * shard.count)
        shard.local(dx, dout)
        out[shard.first:shard.first + shard.count] = dev.floats(dout, shard.count)
        shard.destroy()
    assert float(np.abs(out - expected).max()) <= l2_tolerance(expected)


def test_peer_epilogue_writes_every_output_vector(backend, context, dev, oracle):
    rows, width = 300, 1024
    weights = oracle.make_weights(rows, width, seed=3)
    x = oracle.normal(width, seed=4)
    expected = oracle.matvec(weights, rows, width, x)[0]
    w = dev.weights(weights, rows, width)
    dx = dev.to_device(x)
    total = rows + 50
    outs = [dev.to_device(np.full(total, -7.0, np.float32)) for _ in range(3)]
    stat = backend.cuda_q8_matvec_device_f32_peers(context, w, dx, width, outs, 20, total)
    assert stat.is_ok(), stat
    for ptr in outs:
        got = dev.floats(ptr, total)
        assert (got[:20] == -7.0).all() and (got[20 + rows:] == -7.0).all()
        assert float(np.abs(got[20:20 + rows] - expected).max()) <= l2_tolerance(expected)
    # the slice must fit inside the output vectors
    assert not backend.cuda_q8_matvec_device_f32_peers(context, w, dx, width, outs, 60, total).is_ok()


def test_fused_allgather_with_a_single_rank(backend, context, dev, oracle):
    """World size 1: the flag protocol runs against this rank's own flag word."""
    rows, width = 777, 2560
    weights = oracle.make_weights(rows, width, seed=5)
    x = oracle.normal(width, seed=6)
    expected = oracle.matvec(weights, rows, width, x)[0]
    w = dev.weights(weights, rows, width)
    dx = dev.to_device(x)
    out = dev.to_device(np.zeros(rows, np.float32))
    flags = dev.to_device(np.zeros(1, np.int32))
    for call in range(3):
        stat = backend.cuda_q8_matvec_device_f32_allgather(context, w, dx, width, [out], [flags],
                                                           0, 0, rows)
        assert stat.is_ok(), stat
        assert context.synchronize().is_ok()
        assert dev.int32s(flags, 1)[0] == call + 1      # the last CTA writes the call's number
    assert float(np.abs(dev.floats(out, rows) - expected).max()) <= l2_tolerance(expected)
    # the other protocol: every launch adds exactly 2^20 to the sender's word, whatever its grid
    assert context.set_option("peer_publish_per_cta", 1).is_ok()
    flags = dev.to_device(np.zeros(1, np.int32))
    out = dev.to_device(np.zeros(rows, np.float32))
    for call in range(3):
        stat = backend.cuda_q8_matvec_device_f32_allgather(context, w, dx, width, [out], [flags],
                                                           0, 0, rows)
        assert stat.is_ok(), stat
        assert context.synchronize().is_ok()
        assert dev.int32s(flags, 1)[0] == (call + 1) << 20
    assert float(np.abs(dev.floats(out, rows) - expected).max()) <= l2_tolerance(expected)


def test_pair_allgather_with_a_single_rank(backend, context, dev, oracle):
    """World size 1: the own slice goes straight into the output; consecutive calls alternate
    the halves of the pair array and carry growing call numbers."""
    rows, width = 777, 2560
    weights = oracle.make_weights(rows, width, seed=5)
    w = dev.weights(weights, rows, width)
    pairs = dev.to_device(np.zeros(4 * rows, np.int32))      # 2 halves x rows pairs of 8 bytes
    for call in range(3):
        x = oracle.normal(width, seed=60 + call)
        expected = oracle.matvec(weights, rows, width, x)[0]
        out = dev.to_device(np.zeros(rows, np.float32))
        stat = backend.cuda_q8_matvec_device_f32_allgather_ll(context, w, dev.to_device(x), width,
                                                              [pairs], 0, 0, out, rows)
        assert stat.is_ok(), stat
        assert context.synchronize().is_ok()
        assert float(np.abs(dev.floats(out, rows) - expected).max()) <= l2_tolerance(expected)
    # refused: unaligned pair array, rank outside the list, capture
    assert not backend.cuda_q8_matvec_device_f32_allgather_ll(context, w, dev.to_device(x), width,
                                                              [pairs + 4], 0, 0, out, rows).is_ok()
    assert not backend.cuda_q8_matvec_device_f32_allgather_ll(context, w, dev.to_device(x), width,
                                                              [pairs], 1, 0, out, rows).is_ok()


def test_pair_allgather_collects_what_a_peer_sent_and_gives_up_on_what_it_did_not(
        backend, context, dev, oracle):
    """Two "ranks" on this GPU, run one after the other (their kernels do not wait for each
    other's launch: rank 1 sends first, rank 0 then finds its pairs).  Rank 0's slice comes
    from its own rows, rank 1's from the pairs rank 1 stored.  Then a call whose peer never
    sends: the wait runs out, the kernel returns by itself and the next blocking call reports
    it."""
    rows, width = 512, 1024            # two slices of 256 rows
    weights = oracle.make_weights(rows, width, seed=11)
    x = oracle.normal(width, seed=12)
    expected = oracle.matvec(weights, rows, width, x)[0]
    half = rows // 2
    flat = weights.view(np.int8).reshape(rows, -1)
    w0 = dev.weights(np.ascontiguousarray(flat[:half]).reshape(-1), half, width)
    w1 = dev.weights(np.ascontiguousarray(flat[half:]).reshape(-1), half, width)
    pairs = [dev.to_device(np.zeros(4 * rows, np.int32)) for _ in range(2)]
    outs = [dev.to_device(np.zeros(rows, np.float32)) for _ in range(2)]
    dx = dev.to_device(x)
    other = backend.cuda_q8_context_t()         # rank 1's context: its own call counters
    assert other.create(0).is_ok()
    w1b = backend.cuda_q8_weights_t()
    assert w1b.upload(other, np.ascontiguousarray(flat[half:]).reshape(-1), half * (width // 32) * 34,
                      half, width).is_ok()
    assert other.set_option("peer_wait_clocks_millions", 5).is_ok()
    assert context.set_option("peer_wait_clocks_millions", 5).is_ok()
    # rank 1 sends its slice and fails to collect rank 0's (rank 0 has not run): reported
    stat = backend.cuda_q8_matvec_device_f32_allgather_ll(other, w1b, dx, width, pairs, 1, half,
                                                          outs[1], rows)
    assert stat.is_ok(), stat
    stat = other.synchronize()
    assert not stat.is_ok() and "gave up waiting" in other.last_error()
    # rank 0 now finds rank 1's pairs and completes
    stat = backend.cuda_q8_matvec_device_f32_allgather_ll(context, w0, dx, width, pairs, 0, 0,
                                                          outs[0], rows)
    assert stat.is_ok(), stat
    assert context.synchronize().is_ok()
    assert float(np.abs(dev.floats(outs[0], rows) - expected).max()) <= l2_tolerance(expected)
    # the context that reported the timeout works again
    assert other.synchronize().is_ok()
    w1b.destroy()
    other.destroy()


def test_column_shards_sum_to_the_full_ffn(backend, context, dev, oracle):
    from fortai_b200 import sharded
    hidden, inner, world = 1024, 3840, 4
    gate = oracle.make_weights(inner, hidden, seed=1)
    up = oracle.make_weights(inner, hidden, seed=2)
    down = oracle.make_weights(hidden, inner, seed=3)
    x = oracle.normal(hidden, seed=4)
    expected = oracle.ffn(gate, up, down, inner, hidden, hidden, x)
    dx = dev.to_device(x)
    total = np.zeros(hidden, np.float64)
    for rank in range(world):
        ffn = sharded.ShardedFfn(backend, context, gate, up, down, hidden, inner, rank, world)
        dout = dev.buffer(4 * hidden)
        stat = backend.cuda_q8_ffn_device(context, ffn.gate, ffn.up, ffn.down, dx, hidden, dout,
                                          hidden)
        assert stat.is_ok(), stat
        total += dev.floats(dout, hidden)
        ffn.destroy()
    assert float(np.abs(total - expected).max()) <= 2 * l2_tolerance(expected)


@pytest.mark.parametrize("per_cta", [1, 0])
def test_fused_allgather_gives_up_when_a_peer_never_answers(backend, context, dev, oracle, per_cta):
    """Failure detection without a fault: two "ranks" whose flag arrays are ordinary buffers
    on this GPU, the second rank's flag is never raised.  The wait runs out (a few
    milliseconds here), the kernel returns by itself, the next blocking call reports it, and
    the context works again afterwards."""
    rows, width = 256, 1024
    weights = oracle.make_weights(rows, width, seed=9)
    x = oracle.normal(width, seed=10)
    expected = oracle.matvec(weights, rows, width, x)[0]
    w = dev.weights(weights, rows, width)
    dx = dev.to_device(x)
    outs = [dev.to_device(np.zeros(2 * rows, np.float32)) for _ in range(2)]
    flags = [dev.to_device(np.zeros(2, np.int32)) for _ in range(2)]
    assert context.set_option("peer_wait_clocks_millions", 5).is_ok()
    assert context.set_option("peer_publish_per_cta", per_cta).is_ok()
    stat = backend.cuda_q8_matvec_device_f32_allgather(context, w, dx, width, outs, flags, 0, 0,
                                                       2 * rows)
    assert stat.is_ok(), stat               # enqueue only: the launch itself is fine
    stat = context.synchronize()
    assert not stat.is_ok()
    assert "gave up waiting for a peer flag" in context.last_error()
    # this rank's slice was stored everywhere all the same, and its own flag was raised
    for ptr in outs:
        assert float(np.abs(dev.floats(ptr, 2 * rows)[:rows] - expected).max()) <= l2_tolerance(expected)
    assert dev.int32s(flags[1], 2)[0] != 0 and dev.int32s(flags[0], 2)[1] == 0
    # the status was cleared by reporting it; an ordinary call succeeds
    assert context.set_option("peer_wait_clocks_millions", 2000).is_ok()
    assert context.synchronize().is_ok()
    out = np.zeros(rows, np.float32)
    _, stat = backend.cuda_q8_matvec_host_f32(context, w, x, out)
    assert stat.is_ok(), stat
    assert float(np.abs(out - expected).max()) <= l2_tolerance(expected)


def test_fused_allgather_in_a_cuda_graph(backend, context, dev, oracle):
    """The per-CTA protocol takes the call's number from the flag words, so a captured launch
    can be replayed: every replay waits for its own number and adds 2^20.  The last-CTA
    protocol carries the number as a launch argument and refuses capture."""
    rows, width = 640, 2560
    weights = oracle.make_weights(rows, width, seed=1)
    x = oracle.normal(width, seed=2)
    expected = oracle.matvec(weights, rows, width, x)[0]
    w = dev.weights(weights, rows, width)
    dx = dev.to_device(x)
    out = dev.to_device(np.zeros(rows, np.float32))
    flags = dev.to_device(np.zeros(1, np.int32))
    assert context.set_option("peer_publish_per_cta", 1).is_ok()
    assert context.capture_begin().is_ok()
    stat = backend.cuda_q8_matvec_device_f32_allgather(context, w, dx, width, [out], [flags], 0,
                                                       0, rows)
    assert stat.is_ok(), stat
    assert context.capture_end().is_ok()
    for replay in range(3):
        assert context.graph_launch().is_ok()
        assert context.synchronize().is_ok()
        assert dev.int32s(flags, 1)[0] == (replay + 1) << 20
    assert float(np.abs(dev.floats(out, rows) - expected).max()) <= l2_tolerance(expected)
    other = backend.cuda_q8_context_t()
    assert other.create(0).is_ok()
    w2 = backend.cuda_q8_weights_t()
    assert w2.upload(other, weights, weights.size, rows, width).is_ok()
    assert other.capture_begin().is_ok()
    stat = backend.cuda_q8_matvec_device_f32_allgather(other, w2, dx, width, [out], [flags], 0, 0,
                                                       rows)
    assert not stat.is_ok()
    assert "cannot be captured" in other.last_error()
    assert other.capture_end().is_ok()
    w2.destroy()
    other.destroy()


def test_27b_ffn_at_its_eight_way_shard_sizes(backend, context, dev, oracle):
    """hidden 5120, inner 17408 over 8 ranks: 2176 gate/up rows and a 68-block column shard of
    the down matrix per rank (68 is not a multiple of 8: the raw GGUF rows of such a shard are
    only 8-byte aligned).  All eight shards run on this GPU; their sum is the full FFN."""
    from fortai_b200 import sharded
    hidden, inner, world = 5120, 17408, 8
    gate = oracle.make_weights(inner, hidden, seed=31)
    up = oracle.make_weights(inner, hidden, seed=32)
    down = oracle.make_weights(hidden, inner, seed=33)
    x = oracle.normal(hidden, seed=34)
    expected = oracle.ffn(gate, up, down, inner, hidden, hidden, x)
    dx = dev.to_device(x)
    total = np.zeros(hidden, np.float64)
    for rank in range(world):
        ffn = sharded.ShardedFfn(backend, context, gate, up, down, hidden, inner, rank, world)
        assert ffn.count == 2176 and ffn.count // 32 == 68
        dout = dev.buffer(4 * hidden)
        stat = backend.cuda_q8_ffn_device(context, ffn.gate, ffn.up, ffn.down, dx, hidden, dout,
                                          hidden)
        assert stat.is_ok(), stat
        total += dev.floats(dout, hidden)
        ffn.destroy()
    assert float(np.abs(total - expected).max()) <= 2 * l2_tolerance(expected)


def test_allreduce_ffn_with_a_single_rank(backend, context, dev, oracle):
    """World size 1: the exchange runs against this rank's own pair array; consecutive calls use
    its two halves."""
    hidden, inner = 1024, 3840
    gate = oracle.make_weights(inner, hidden, seed=41)
    up = oracle.make_weights(inner, hidden, seed=42)
    down = oracle.make_weights(hidden, inner, seed=43)
    wg, wu, wd = (dev.weights(m, r, c) for m, r, c in ((gate, inner, hidden), (up, inner, hidden),
                                                     (down, hidden, inner)))
    pairs = dev.to_device(np.zeros(4 * hidden, np.int32))       # 2 halves x 1 slot x hidden pairs
    for call in range(3):
        x = oracle.normal(hidden, seed=50 + call)
        expected = oracle.ffn(gate, up, down, inner, hidden, hidden, x)
        dout = dev.buffer(4 * hidden)
        stat = backend.cuda_q8_ffn_device_allreduce(context, wg, wu, wd, dev.to_device(x), hidden,
                                                    [pairs], 0, dout, hidden)
        assert stat.is_ok(), stat
        assert context.synchronize().is_ok()
        plain = dev.buffer(4 * hidden)
        assert backend.cuda_q8_ffn_device(context, wg, wu, wd, dev.to_device(x), hidden, plain,
                                          hidden).is_ok()
        got = dev.floats(dout, hidden)
        assert float(np.abs(got - expected).max()) <= 2 * l2_tolerance(expected)
        assert np.array_equal(got, dev.floats(plain, hidden))    # one slot: the sum is the slot
        # the half of the pair array this call used carries its number beside every value
        half = dev.int32s(pairs, 4 * hidden).reshape(2, hidden, 2)[call & 1]
        assert np.all(half[:, 1] == call + 1)
        assert np.array_equal(half[:, 0].view(np.float32), got)
    # refused: a rank outside the peer list, an unaligned array
    assert not backend.cuda_q8_ffn_device_allreduce(context, wg, wu, wd, dev.to_device(x), hidden,
                                                    [pairs], 1, dout, hidden).is_ok()
    assert not backend.cuda_q8_ffn_device_allreduce(context, wg, wu, wd, dev.to_device(x), hidden,
                                                    [pairs + 4], 0, dout, hidden).is_ok()


def _rank_main(rank, world, port, result_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    from fortai_b200 import backend_cuda as b, sharded
    from oracle import q8_oracle as o
    failures = []
    ctx = b.cuda_q8_context_t()
    assert ctx.create(rank, stream=torch.cuda.current_stream().cuda_stream).is_ok()
    rows, width = 4099, 2560
    weights = o.make_weights(rows, width, seed=1)
    xh = o.normal(width, seed=2)
    expected = o.matvec(weights, rows, width, xh)[0]
    x = torch.from_numpy(xh).cuda()
    shard = sharded.PeerGatherMatvec(b, ctx, weights, rows, width, rank, world)
    out = torch.zeros(rows, device="cuda")
    shard.matvec(dist, x, out)
    torch.cuda.synchronize()
    if float(np.abs(out.cpu().numpy() - expected).max()) > 1e-5 * float(np.linalg.norm(expected)):
        failures.append("all-gather path differs from the oracle")
    try:
        import torch.distributed._symmetric_memory as symm
        buf = symm.empty(rows, dtype=torch.float32, device=torch.device("cuda", rank))
        handle = symm.rendezvous(buf, dist.group.WORLD)
        buf.zero_()
        handle.barrier(channel=0)
        flags = symm.empty(world, dtype=torch.int32, device=torch.device("cuda", rank))
        flags.zero_()
        flag_handle = symm.rendezvous(flags, dist.group.WORLD)
        torch.cuda.synchronize()
        dist.barrier()
        shard.attach([int(p) for p in handle.buffer_ptrs], lambda: handle.barrier(channel=0),
                     [int(p) for p in flag_handle.buffer_ptrs])
        shard.matvec_peers(x)
        torch.cuda.synchronize()
        if float(np.abs(buf.cpu().numpy() - expected).max()) > 1e-5 * float(np.linalg.norm(expected)):
            failures.append("peer-store path differs from the oracle")
        for _ in range(3):
            buf.zero_()
            handle.barrier(channel=0)
            shard.matvec_fused(x)
            torch.cuda.synchronize()
            if not ctx.synchronize().is_ok():
                failures.append("fused all-gather reported a device-side timeout")
            if float(np.abs(buf.cpu().numpy() - expected).max()) > 1e-5 * float(np.linalg.norm(expected)):
                failures.append("fused all-gather differs from the oracle")
        # the all-gather whose data carries its own flag, three calls in a row (both halves
        # of the pair arrays), each on another activation
        pair_buffer = symm.empty(4 * rows, dtype=torch.int32, device=torch.device("cuda", rank))
        pair_buffer.zero_()
        pair_handle = symm.rendezvous(pair_buffer, dist.group.WORLD)
        torch.cuda.synchronize()
        dist.barrier()
        shard.attach_pairs([int(p) for p in pair_handle.buffer_ptrs])
        for call in range(3):
            xc = o.normal(width, seed=30 + call)
            want = o.matvec(weights, rows, width, xc)[0]
            got = torch.zeros(rows, device="cuda")
            shard.matvec_pairs(torch.from_numpy(xc).cuda(), got)
            torch.cuda.synchronize()
            if not ctx.synchronize().is_ok():
                failures.append("pair all-gather reported a device-side timeout")
            if float(np.abs(got.cpu().numpy() - want).max()) > 1e-5 * float(np.linalg.norm(want)):
                failures.append("pair all-gather differs from the oracle")
    except Exception as error:  # symmetric memory is optional; say so rather than fail
        failures.append(f"SKIP-PEERS {type(error).__name__}: {error}")
    # FFN: rows of gate/up, columns of down, all-reduce
    hidden, inner = 1024, 3840
    gate, up = o.make_weights(inner, hidden, seed=5), o.make_weights(inner, hidden, seed=6)
    down = o.make_weights(hidden, inner, seed=7)
    xf = o.normal(hidden, seed=8)
    expected_ffn = o.ffn(gate, up, down, inner, hidden, hidden, xf)
    ffn = sharded.ShardedFfn(b, ctx, gate, up, down, hidden, inner, rank, world)
    outf = torch.zeros(hidden, device="cuda")
    ffn.forward(dist, torch.from_numpy(xf).cuda(), outf)
    torch.cuda.synchronize()
    if float(np.abs(outf.cpu().numpy() - expected_ffn).max()) > 2e-5 * float(np.linalg.norm(expected_ffn)):
        failures.append("sharded FFN differs from the oracle")
    try:
        # the same with the partial vectors exchanged by the down GEMV itself, for both a
        # pipelined-width shard (3840 / world) and consecutive calls (slot parity)
        import torch.distributed._symmetric_memory as symm
        ffn_pairs = symm.empty(4 * world * hidden, dtype=torch.int32, device=torch.device("cuda", rank))
        ffn_pairs.zero_()
        ffn_pair_handle = symm.rendezvous(ffn_pairs, dist.group.WORLD)
        torch.cuda.synchronize()
        dist.barrier()
        ffn.attach([int(p) for p in ffn_pair_handle.buffer_ptrs])
        gathered = [torch.zeros(hidden, device="cuda") for _ in range(world)]
        for call in range(3):
            xc = o.normal(hidden, seed=20 + call)
            want = o.ffn(gate, up, down, inner, hidden, hidden, xc)
            fused = torch.zeros(hidden, device="cuda")
            ffn.forward_fused(torch.from_numpy(xc).cuda(), fused)
            torch.cuda.synchronize()
            if not ctx.synchronize().is_ok():
                failures.append("fused FFN reported a device-side timeout")
            if float(np.abs(fused.cpu().numpy() - want).max()) > 2e-5 * float(np.linalg.norm(want)):
                failures.append("fused sharded FFN differs from the oracle")
            dist.all_gather(gathered, fused)
            if any(not torch.equal(g, gathered[0]) for g in gathered):
                failures.append("fused sharded FFN: ranks hold different bits")
    except Exception as error:
        failures.append(f"SKIP-PEERS {type(error).__name__}: {error}")
    shard.destroy()
    ffn.destroy()
    ctx.destroy()
    with open(f"{result_path}.{rank}", "w") as f:
        f.write("\n".join(failures))
    dist.destroy_process_group()


def test_ranks_on_separate_gpus(tmp_path):
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    port = 29600 + (os.getpid() % 2000)
    result = str(tmp_path / "result")
    mp.spawn(_rank_main, args=(world, port, result), nprocs=world, join=True)
    for rank in range(world):
        lines = [l for l in open(f"{result}.{rank}").read().splitlines() if l]
        assert [l for l in lines if not l.startswith("SKIP-PEERS")] == [], lines
