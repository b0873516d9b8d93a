"""Every GEMM shape `bench.py --gpus N` gives a rank (N in 1, 2, 4, 8; every token count of the sweep) must have a
schedule: the uneven K128-block shards of the row-parallel layers at eight ranks (o_proj K = 512 / 384, down
K = 2432 / 2304) and the narrow column shards are the shapes no single-GPU run ever builds.  Host only: the
schedule builder needs no GPU."""
import ctypes as C

import torch

import bench
from hygemm_vllm import native


def rank_shapes(world, rank, seed=0):
    """(name, K, low rows, high rows) of the four layers as `bench.build_layer` shards them (the MXFP8 channels are
    drawn from another stream than the bench's, which only moves a few channels between ranks)."""
    g = torch.Generator().manual_seed(seed)
    for name, (k, parts) in bench.SHAPES.items():
        n = sum(parts.values())
        high = torch.randperm(n, generator=g)[: bench.high_quota(n)]
        if world == 1:
            yield name, k, n - high.numel(), high.numel()
        elif name in bench.ROW_PARALLEL:
            begin, end = bench.k_block_shard(k, rank, world)
            yield name, end - begin, n - high.numel(), high.numel()
        else:
            keep, offset = [], 0
            for width in parts.values():
                begin, end = (bench.k_block_shard(width, rank, world) if name == "gate_up"
                              else (rank * (width // world), (rank + 1) * (width // world)))
                keep.append(torch.arange(offset + begin, offset + end))
                offset += width
            keep = torch.cat(keep)
            mask = torch.zeros(n, dtype=torch.bool)
            mask[high] = True
            h = int(mask[keep].sum())
            yield name, k, keep.numel() - h, h


def test_every_rank_shape_of_the_tensor_parallel_sweep_has_a_schedule():
    lib = native.library()
    header = (C.c_int * 12)()
    seen = set()
    for world in (1, 2, 4, 8):
        covered = {name: 0 for name in bench.SHAPES}
        for rank in range(world):
            for name, k, lo, hi in rank_shapes(world, rank):
                assert k % 128 == 0 and k > 0 and lo + hi > 0, (world, rank, name, k, lo, hi)
                covered[name] += k if name in bench.ROW_PARALLEL else lo + hi
                for tokens in bench.M_SWEEP:
                    if (k, lo, hi, tokens) in seen:
                        continue
                    seen.add((k, lo, hi, tokens))
                    status = lib.hg_plan(lo, hi, tokens, k, 148, 0, header, None, 0)
                    assert status == 0, (world, rank, name, tokens, lib.hg_last_error())
                    grid, n_tile, stages, smem, tmem = header[1], header[2], header[4], header[5], header[6]
                    assert 1 <= grid <= 148 and n_tile % 16 == 0 and stages >= 2 and smem <= 232448 and tmem <= 512
        for name, (k, parts) in bench.SHAPES.items():       # the shards tile the layer exactly
            assert covered[name] == (k if name in bench.ROW_PARALLEL else sum(parts.values())), (world, name)
