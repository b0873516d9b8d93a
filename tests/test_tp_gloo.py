"""Tensor-parallel shard arithmetic on CPU ranks (gloo, world size 2): the shards of a hybrid linear,
computed per rank with the CPU oracle and combined the way the GPU path combines them, reproduce the
unsharded layer."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from hygemm_vllm import tp

OUT, K, TOKENS, WORLD = 512, 512, 5, 2
NAMES, SIZES = ["l.q_proj", "l.k_proj", "l.v_proj"], [256, 128, 128]


def _layer():
    g = torch.Generator().manual_seed(20261024)
    w = (torch.randn(OUT, K, generator=g) * 0.02).bfloat16()
    x = torch.randn(TOKENS, K, generator=g).bfloat16()
    selection = {n: sorted(torch.randperm(s, generator=g)[: s // 8].tolist()) for n, s in zip(NAMES, SIZES)}
    return w, x, selection


def _oracle_linear(w, ids, x):
    outputs = w.shape[0]
    lo, hi = oracle.partition(outputs, ids)
    w4, sf4 = oracle.pack(w[torch.from_numpy(lo).long()], fp4=True)
    w8, sf8 = oracle.pack(w[torch.from_numpy(hi).long()], fp4=False)
    xq, xsf = oracle.pack(x)
    _, yf = oracle.hybrid_linear(w4, sf4, lo, w8, sf8, hi, xq, xsf, outputs)
    return yf


def _worker(rank, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        w, x, selection = _layer()
        # column-parallel: this rank's rows of q, k, v and its share of the selection
        keep, offset = [], 0
        for size in SIZES:
            begin, end = tp.shard_bounds(size, rank, WORLD)
            keep.append(torch.arange(offset + begin, offset + end))
            offset += size
        keep = torch.cat(keep)
        rows = tp.column_parallel_rows(selection, NAMES, SIZES, rank, WORLD)
        y_col = torch.from_numpy(_oracle_linear(w[keep].contiguous(), rows, x))
        gathered = [torch.empty_like(y_col) for _ in range(WORLD)]
        dist.all_gather(gathered, y_col)
        # row-parallel: K shard, whole selection, partial sums all-reduced
        begin, end = tp.row_parallel_k(K, rank, WORLD)
        full_ids = sorted(i + o for n, o in zip(NAMES, np.cumsum([0] + SIZES[:-1])) for i in selection[n])
        y_row = torch.from_numpy(_oracle_linear(w[:, begin:end].contiguous(), full_ids, x[:, begin:end].contiguous()))
        tp.all_reduce_partial(y_row)
        # selection rule: identical on every rank after the norm all-reduce
        chosen = tp.select_by_l2norm(w[:, begin:end].contiguous(), 0.25, 128, group=dist.group.WORLD, row_parallel=True)
        if rank == 0:
            results.put((keep.numpy(), [g.numpy() for g in gathered], y_row.numpy(), chosen))
        else:
            results.put(("chosen", chosen))
    finally:
        dist.destroy_process_group()


def test_two_rank_shards_reproduce_the_unsharded_layer():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, port, results)) for r in range(WORLD)]
    for p in procs:
        p.start()
    got = [results.get(timeout=180) for _ in range(WORLD)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    main = next(g for g in got if g[0] is not None and not isinstance(g[0], str))
    other = next(g for g in got if isinstance(g[0], str))
    keep0, gathered, y_row, chosen0 = main
    assert chosen0 == other[1] and len(chosen0) == 128

    w, x, selection = _layer()
    full_ids = sorted(i + o for n, o in zip(NAMES, np.cumsum([0] + SIZES[:-1])) for i in selection[n])
    ref = _oracle_linear(w, full_ids, x)
    # column-parallel: each rank's columns are exactly the unsharded columns (same rows, same quantisation)
    y_full = np.zeros_like(ref)
    offset = 0
    for rank in range(WORLD):
        cols, off = [], 0
        for size in SIZES:
            b, e = tp.shard_bounds(size, rank, WORLD)
            cols.append(np.arange(off + b, off + e))
            off += size
        y_full[:, np.concatenate(cols)] = gathered[rank]
    assert np.array_equal(y_full, ref)
    # row-parallel: K32 blocks are never split by a 128-aligned K shard, so only the fp32 summation order differs
    err = np.linalg.norm(y_row - ref) / np.linalg.norm(ref)
    assert err < 1e-6, err
