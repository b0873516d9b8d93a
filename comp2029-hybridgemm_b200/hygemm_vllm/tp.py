"""Tensor-parallel sharding of hybrid linears (one process per GPU, NCCL over NVLink).

The reference rejects tensor parallelism (quantization.py:81-83 of the
reference); this module adds it the way vLLM shards dense layers:

* column-parallel (qkv_proj, gate_up_proj): split N.  Rank r keeps rows
  `[r*size, (r+1)*size)` of every unfused projection; its high-precision set is
  the part of the selection that falls in that range, re-based to the rank's
  fused row numbering.  No communication.
* row-parallel (o_proj, down_proj): split K in multiples of 128, so every rank's
  K32 quantisation blocks are exactly the corresponding blocks of the unsharded
  tensor.  Every rank keeps all N rows and the same channel subset, scatters its
  partial sums into a full `[M,N]` buffer, and the partials are summed with one
  all-reduce.
"""
from __future__ import annotations

from typing import Mapping, Sequence

import torch
import torch.distributed as dist


def shard_bounds(size: int, rank: int, world: int) -> tuple[int, int]:
    if size % world:
        raise ValueError(f"size {size} is not divisible by tensor-parallel world {world}")
    step = size // world
    return rank * step, (rank + 1) * step


def validate_ids(ids: Sequence[int], size: int, name: str) -> None:
    """Selection rule of the reference (quantization.py:113-115): unique ids in [0, size)."""
    if len(set(ids)) != len(ids) or any(i < 0 or i >= size for i in ids):
        raise ValueError(f"Invalid channel map for {name}")


def column_parallel_rows(selection: Mapping[str, Sequence[int]], names: Sequence[str], full_sizes: Sequence[int],
                         rank: int, world: int, shard_ranks: Sequence[tuple[int, int]] | None = None) -> list[int]:
    """Fused-row ids (sorted) of the high-precision channels owned by `rank`.

    `names`/`full_sizes` list the unfused projections of the fused layer in order
    with their unsharded widths; `shard_ranks[p] = (shard, parts)` overrides the
    shard of projection p (replicated KV heads: `(rank // replicas, world // replicas)`).
    """
    rows, offset = [], 0
    for p, (name, size) in enumerate(zip(names, full_sizes)):
        if name not in selection:
            raise ValueError(f"Missing channel selection for {name}")
        ids = selection[name]
        validate_ids(ids, size, name)
        shard, parts = (rank, world) if shard_ranks is None else shard_ranks[p]
        begin, end = shard_bounds(size, shard, parts)
        rows.extend(i - begin + offset for i in ids if begin <= i < end)
        offset += end - begin
    return sorted(rows)


def row_parallel_k(k: int, rank: int, world: int) -> tuple[int, int]:
    begin, end = shard_bounds(k, rank, world)
    if (end - begin) % 128:
        raise ValueError(f"K shard {end - begin} must stay a multiple of 128")
    return begin, end


def select_by_l2norm(weight: torch.Tensor, fraction: float, multiple: int = 1,
                     group: dist.ProcessGroup | None = None, row_parallel: bool = False) -> list[int]:
    """Channels with the largest weight-row L2 norm (row = output channel).

    For a row-parallel shard the squared norms are summed over the group first so
    every rank chooses the same set.  `multiple` rounds the quota (e.g. to 128).
    """
    norms = weight.float().square().sum(dim=1)
    if row_parallel and group is not None and dist.get_world_size(group) > 1:
        dist.all_reduce(norms, group=group)
    n = weight.shape[0]
    quota = int(round(fraction * n / multiple)) * multiple
    quota = max(0, min(n, quota))
    if quota == 0:
        return []
    # Stable tie-break on the channel index keeps ranks and runs identical.
    order = torch.sort(norms, descending=True, stable=True).indices[:quota]
    return sorted(order.tolist())


def all_reduce_partial(y: torch.Tensor, group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """Sum the row-parallel partial outputs in place (NCCL on GPUs, gloo in the CPU tests)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(y, group=group)
    return y


class PeerExchange:
    """Buffers of the row-parallel GEMM + exchange (`DualLinear.run_exchange`).

    Every rank allocates, in memory mapped on all peers (torch symmetric memory over CUDA IPC), an exchange
    buffer of two halves and a flag array; the GEMM of rank r writes its partial result into one half of
    rank r's own buffer, and the all-reduce launch tells the peers, waits on the flags, loads every rank's
    partial over NVLink and sums them in rank order.  One instance serves every row-parallel layer of a model
    whose `tokens x outputs` fits `max_elems`, as the exchanges of a stream are ordered.  NVLink multicast is
    not used (plain peer loads), so the buffers are never bound to a multicast object by this class.
    Callers read `status()` at step boundaries: a peer that did not arrive in time leaves a code there and
    NaN in that exchange's result.
    """

    def __init__(self, group: dist.ProcessGroup, max_elems: int, dtype: torch.dtype, device: torch.device):
        import ctypes as C
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PeerExchange serves at most 8 ranks of one NVLink domain")
        self.dtype, self.group = dtype, group
        self.half_bytes = -(-max_elems * 2 // 256) * 256          # one half: max_elems 16-bit partial sums
        self.buffer = symm.empty(2 * self.half_bytes, dtype=torch.uint8, device=device)
        self.flags = symm.empty(64, dtype=torch.int32, device=device)
        self.buffer.zero_()
        self.flags.zero_()
        self.state = torch.zeros(4, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        self._handles = (symm.rendezvous(self.buffer, group), symm.rendezvous(self.flags, group))
        self.buffer_ptrs = (C.c_void_p * self.world)(*[int(p) for p in self._handles[0].buffer_ptrs])
        self.flag_ptrs = (C.c_void_p * self.world)(*[int(p) for p in self._handles[1].buffer_ptrs])
        if self.buffer_ptrs[self.rank] != self.buffer.data_ptr():
            raise RuntimeError("symmetric memory did not return this rank's own buffer at its rank index")
        dist.barrier(group)
        torch.cuda.synchronize(device)

    def status(self) -> int:
        """0, or 1000 + the rank whose partials never arrived within the wait limit (cleared by the read)."""
        import ctypes as C
        from . import native
        out = C.c_int(0)
        native.check(native.library().hg_tp_status(self.state.data_ptr(), torch.cuda.current_stream().cuda_stream,
                                                   C.byref(out)))
        return out.value
