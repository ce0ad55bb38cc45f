"""Row and column sharding of Q8_0 projections across the GPUs of one box.

The reference is single-GPU ("deferred", ROADMAP.md:31); its CPU matvec is already a
partition over output rows (OpenMP static loop, src/fortai_gguf_runtime.f90:457-463),
which is the partition used here across ranks.  One process per GPU
(`torch.distributed`, NCCL over NVLink on GPUs, gloo on CPU for the host-logic tests).

* Row sharding (lm_head, FFN gate/up): rank r owns rows [first, first + count); its
  slice of the GGUF bytes is contiguous.  Every rank computes its slice of the output;
  the slices are reassembled with an all-gather, or written straight into every rank's
  output vector by the GEMV epilogue (`PeerGatherMatvec`).
* Column sharding (FFN down): rank r owns blocks [first_block, first_block + n) of every
  row.  Q8_0 activation blocks are independent, so a rank quantizes just its slice of
  the hidden vector; partial outputs are summed with an all-reduce.  In an FFN the
  slice of the hidden vector a rank needs is exactly the slice its gate/up row shard
  produced, so nothing is exchanged between the two halves.

Per-rank results are bit-identical to the single-GPU kernel for row sharding (same
per-row arithmetic) and differ only in fp32 summation order for column sharding.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import numpy as np

Q8_BLOCK_ELEMS = 32
Q8_BLOCK_BYTES = 34


# --------------------------------------------------------------------------- partitions
def partition(total: int, parts: int, multiple: int = 1) -> List[Tuple[int, int]]:
    """Split `total` items into `parts` contiguous (first, count) ranges whose sizes are
    multiples of `multiple` (except that the last non-empty one takes the remainder) and
    differ by at most one multiple."""
    if total < 0 or parts <= 0 or multiple <= 0:
        raise ValueError("invalid partition request")
    units, tail = divmod(total, multiple)
    base, extra = divmod(units, parts)
    ranges = []
    first = 0
    for r in range(parts):
        count = (base + (1 if r < extra else 0)) * multiple
        ranges.append((first, count))
        first += count
    if tail:
        # the ragged remainder goes to the last rank that has any work (or rank 0)
        owner = max((r for r, (_, c) in enumerate(ranges) if c), default=0)
        f, c = ranges[owner]
        ranges[owner] = (f, c + tail)
        for r in range(owner + 1, parts):
            ranges[r] = (ranges[r][0] + tail, ranges[r][1])
    return ranges


def row_shard_bytes(weights: np.ndarray, rows: int, width: int, first: int, count: int) -> np.ndarray:
    """The contiguous GGUF byte range of rows [first, first + count)."""
    row_bytes = (width // Q8_BLOCK_ELEMS) * Q8_BLOCK_BYTES
    flat = np.ascontiguousarray(weights).view(np.int8).reshape(-1)
    if first < 0 or first + count > rows or flat.size < rows * row_bytes:
        raise ValueError("row shard out of range")
    return flat[first * row_bytes:(first + count) * row_bytes]


def column_shard_bytes(weights: np.ndarray, rows: int, width: int, first_block: int,
                       block_count: int) -> np.ndarray:
    """Host-side re-layout of a K-slice (used by the CPU tests; on the GPU the slice is
    cut at upload by fortai_cuda_q8_weights_upload_columns)."""
    blocks = width // Q8_BLOCK_ELEMS
    flat = np.ascontiguousarray(weights).view(np.int8).reshape(rows, blocks, Q8_BLOCK_BYTES)
    if first_block < 0 or first_block + block_count > blocks:
        raise ValueError("column shard out of range")
    return np.ascontiguousarray(flat[:, first_block:first_block + block_count]).reshape(-1)


# --------------------------------------------------------------------------- exchange steps
def all_gather_rows(dist, local: "torch.Tensor", counts: Sequence[int], out: "torch.Tensor" = None):
    """Reassemble a row-sharded vector.  `counts[r]` is rank r's row count."""
    import torch
    world = len(counts)
    total = int(sum(counts))
    if out is None:
        out = torch.empty(total, dtype=local.dtype, device=local.device)
    if world == 1:
        out.copy_(local)
        return out
    if len(set(counts)) == 1:
        dist.all_gather_into_tensor(out, local.contiguous())
    else:
        # collectives want equal pieces: pad every slice to the largest one
        widest = int(max(counts))
        padded = torch.zeros(widest, dtype=local.dtype, device=local.device)
        padded[:local.numel()] = local
        gathered = torch.empty(world * widest, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(gathered, padded)
        offsets = np.cumsum([0] + list(counts))
        for r in range(world):
            out[int(offsets[r]):int(offsets[r + 1])] = gathered[r * widest:r * widest + counts[r]]
    return out


def all_reduce_sum(dist, partial: "torch.Tensor", world: int):
    """Sum the partial outputs of a column-sharded projection, in place."""
    if world > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM)
    return partial


# --------------------------------------------------------------------------- GPU objects
class RowShardedMatvec:
    """One rank's share of a row-sharded Q8_0 matrix on its GPU."""

    def __init__(self, backend, context, host_weights: np.ndarray, rows: int, width: int,
                 rank: int, world: int):
        self.backend, self.context = backend, context
        self.rows, self.width, self.rank, self.world = rows, width, rank, world
        self.ranges = partition(rows, world)
        self.counts = [c for _, c in self.ranges]
        self.first, self.count = self.ranges[rank]
        self.weights = backend.cuda_q8_weights_t()
        shard = row_shard_bytes(host_weights, rows, width, self.first, self.count)
        stat = self.weights.upload(context, shard, shard.size, self.count, width)
        if not stat.is_ok():
            raise RuntimeError(f"row shard upload failed: {stat}")

    def local(self, activation_ptr: int, output_ptr: int):
        """Enqueue this rank's slice: fp32 activation in, `count` floats out."""
        stat = self.backend.cuda_q8_matvec_device_f32(self.context, self.weights, activation_ptr,
                                                      self.width, output_ptr, self.count)
        if not stat.is_ok():
            raise RuntimeError(f"sharded matvec failed: {stat}")

    def matvec(self, dist, activation: "torch.Tensor", out: "torch.Tensor"):
        """Full-length result on every rank: local slice + all-gather."""
        mine = out[self.first:self.first + self.count]
        self.local(activation.data_ptr(), mine.data_ptr())
        return all_gather_rows(dist, mine, self.counts, out)

    def destroy(self):
        self.weights.destroy()


class PeerGatherMatvec(RowShardedMatvec):
    """Row-sharded matvec whose GEMV epilogue stores the slice into every rank's output
    vector (peer pointers from symmetric memory), followed by a cross-rank barrier: one
    kernel and one barrier instead of a kernel and an all-gather."""

    def attach(self, peer_output_ptrs: Sequence[int], barrier: Callable[[], None],
               peer_flag_ptrs: Sequence[int] = None):
        # C arrays built once: the calls are made once per decoded token
        self.peer_ptrs = self.backend.pointer_array(list(peer_output_ptrs))
        self.barrier = barrier
        self.flag_ptrs = (self.backend.pointer_array(list(peer_flag_ptrs))
                          if peer_flag_ptrs is not None else None)

    def matvec_fused(self, activation: "torch.Tensor"):
        """Slice + all-gather in ONE kernel: the last CTA of every rank raises a flag in
        every rank's memory and waits (bounded) for the others' flags."""
        stat = self.backend.cuda_q8_matvec_device_f32_allgather(
            self.context, self.weights, activation.data_ptr(), self.width, self.peer_ptrs,
            self.flag_ptrs, self.rank, self.first, self.rows)
        if not stat.is_ok():
            raise RuntimeError(f"fused all-gather matvec failed: {stat}")

    def attach_pairs(self, peer_pair_ptrs: Sequence[int]):
        """Pair arrays (2 * rows pairs of 8 bytes per rank, zeroed once) that every rank can
        reach, for `matvec_pairs`."""
        self.pair_ptrs = self.backend.pointer_array(list(peer_pair_ptrs))

    def matvec_pairs(self, activation: "torch.Tensor", out: "torch.Tensor"):
        """Slice + all-gather in ONE kernel without flags: results travel as (value, call
        number) pairs and are collected into `out` (this rank's memory)."""
        stat = self.backend.cuda_q8_matvec_device_f32_allgather_ll(
            self.context, self.weights, activation.data_ptr(), self.width, self.pair_ptrs,
            self.rank, self.first, out.data_ptr(), self.rows)
        if not stat.is_ok():
            raise RuntimeError(f"all-gather matvec (pairs) failed: {stat}")

    def matvec_peers(self, activation: "torch.Tensor"):
        stat = self.backend.cuda_q8_matvec_device_f32_peers(
            self.context, self.weights, activation.data_ptr(), self.width, self.peer_ptrs,
            self.first, self.rows)
        if not stat.is_ok():
            raise RuntimeError(f"peer matvec failed: {stat}")
        self.barrier()


class ShardedFfn:
    """gate/up row-sharded, down column-sharded; the partial outputs are all-reduced."""

    def __init__(self, backend, context, gate: np.ndarray, up: np.ndarray, down: np.ndarray,
                 hidden: int, inner: int, rank: int, world: int):
        self.backend, self.context = backend, context
        self.hidden, self.inner, self.rank, self.world = hidden, inner, rank, world
        # inner rows are cut on block boundaries so that each rank re-quantizes whole blocks
        self.ranges = partition(inner, world, multiple=Q8_BLOCK_ELEMS)
        self.first, self.count = self.ranges[rank]
        if self.count == 0:
            raise ValueError("more ranks than 32-row groups in the FFN inner dimension")
        self.gate, self.up, self.down = (backend.cuda_q8_weights_t() for _ in range(3))
        g = row_shard_bytes(gate, inner, hidden, self.first, self.count)
        u = row_shard_bytes(up, inner, hidden, self.first, self.count)
        for handle, data in ((self.gate, g), (self.up, u)):
            stat = handle.upload(context, data, data.size, self.count, hidden)
            if not stat.is_ok():
                raise RuntimeError(f"FFN shard upload failed: {stat}")
        stat = self.down.upload_columns(context, down, hidden, inner,
                                        self.first // Q8_BLOCK_ELEMS,
                                        self.count // Q8_BLOCK_ELEMS)
        if not stat.is_ok():
            raise RuntimeError(f"FFN down shard upload failed: {stat}")

    def forward(self, dist, activation: "torch.Tensor", out: "torch.Tensor"):
        stat = self.backend.cuda_q8_ffn_device(self.context, self.gate, self.up, self.down,
                                               activation.data_ptr(), self.hidden, out.data_ptr(),
                                               self.hidden)
        if not stat.is_ok():
            raise RuntimeError(f"sharded FFN failed: {stat}")
        return all_reduce_sum(dist, out, self.world)

    def attach(self, peer_pair_ptrs: Sequence[int]):
        """Pair arrays (2 * world * hidden pairs of 8 bytes per rank, zeroed once) that every
        rank can reach, for `forward_fused`."""
        self.pair_ptrs = self.backend.pointer_array(list(peer_pair_ptrs))

    def forward_fused(self, activation: "torch.Tensor", out: "torch.Tensor"):
        """The same result without a collective call: partial vectors are exchanged by the
        down GEMV itself and added in rank order (the same bits on every rank)."""
        stat = self.backend.cuda_q8_ffn_device_allreduce(
            self.context, self.gate, self.up, self.down, activation.data_ptr(), self.hidden,
            self.pair_ptrs, self.rank, out.data_ptr(), self.hidden)
        if not stat.is_ok():
            raise RuntimeError(f"fused sharded FFN failed: {stat}")
        return out

    def forward_batch(self, dist, activations: "torch.Tensor", out: "torch.Tensor"):
        """`tokens` activations at once (tokens x hidden in, tokens x hidden out)."""
        tokens = int(activations.shape[0])
        stat = self.backend.cuda_q8_ffn_batch_device(self.context, self.gate, self.up, self.down,
                                                     activations.data_ptr(), tokens,
                                                     out.data_ptr(), out.numel())
        if not stat.is_ok():
            raise RuntimeError(f"sharded batched FFN failed: {stat}")
        return all_reduce_sum(dist, out, self.world)

    def destroy(self):
        for handle in (self.gate, self.up, self.down):
            handle.destroy()
