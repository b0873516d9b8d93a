"""Row-parallel exchange (hg_run_partial + hg_tp_allreduce) on ONE GPU.

Ranks (two, and once eight) are emulated by one set of buffers each in the same device memory and launches in an order in
which no launch ever waits for a later one: both GEMMs write their partials first, the flag the first
all-reduce would wait for is written by the host beforehand (standing in for the other rank's publish), and
the second all-reduce finds the first one's publish already there.  The sum must equal the fp32 sum of the
two partial results rounded once (the partials themselves cross as fp32 at decode sizes and as 16-bit values
above), bit for bit, on both ranks and across three consecutive exchanges (both halves of the exchange
buffers).  The real multi-GPU path is exercised by `bench.py --gpus N`.
"""
import ctypes as C

import pytest
import torch

from helpers import bits, make_inputs
from hygemm_vllm import native

pytestmark = pytest.mark.gpu


class LocalExchange:
    """Stand-in for tp.PeerExchange with every rank's buffers on this GPU."""

    def __init__(self, world, rank, half_bytes, buffers, flags, dtype):
        self.world, self.rank, self.half_bytes, self.dtype = world, rank, half_bytes, dtype
        self.buffer = buffers[rank]
        self.buffer_ptrs = (C.c_void_p * world)(*[t.data_ptr() for t in buffers])
        self.flag_ptrs = (C.c_void_p * world)(*[t.data_ptr() for t in flags])
        self.state = torch.zeros(4, dtype=torch.int32, device="cuda")

    def status(self):
        out = C.c_int(0)
        native.check(native.library().hg_tp_status(self.state.data_ptr(), torch.cuda.current_stream().cuda_stream,
                                                   C.byref(out)))
        return out.value


def shards(tokens, k, outputs, high, world, dtype):
    x, w, ids = make_inputs(tokens, k, outputs, high, dtype)
    x, w, ids = x.cuda(), w.cuda(), ids.cuda()
    step = k // world
    layers = [native.DualLinear(w[:, r * step:(r + 1) * step].contiguous(), ids) for r in range(world)]
    xs = [x[:, r * step:(r + 1) * step].contiguous() for r in range(world)]
    return layers, xs


def buffers(world, half_bytes):
    bufs = [torch.full((2 * half_bytes,), 0xFF, dtype=torch.uint8, device="cuda") for _ in range(world)]   # NaN patterns
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(world)]
    return bufs, flags


@pytest.mark.parametrize("tokens,fused", [(1, True), (16, True), (16, False), (48, False), (100, False), (128, False), (130, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_two_emulated_ranks_sum_bit_exact(tokens, fused, dtype):
    emulated_ranks_sum_bit_exact(2, tokens, fused, dtype)


@pytest.mark.parametrize("tokens,fused", [(16, True), (128, False)])
def test_eight_emulated_ranks_sum_bit_exact(tokens, fused):
    """The widest world the exchange takes: rank r's all-reduce finds the flags of the ranks before it published by
    their kernels and those of the ranks after it written by the host ahead of time."""
    emulated_ranks_sum_bit_exact(8, tokens, fused, torch.bfloat16)


def emulated_ranks_sum_bit_exact(world, tokens, fused, dtype):
    k, outputs, high = 1024, 640, 96
    layers, xs = shards(tokens, k, outputs, high, world, dtype)
    elems = tokens * outputs
    f32 = int(tokens <= 16)
    half = -(-elems * 4 // 256) * 256
    bufs, flags = buffers(world, half)
    ex = [LocalExchange(world, r, half, bufs, flags, dtype) for r in range(world)]
    lib, stream = native.library(), torch.cuda.current_stream().cuda_stream
    for epoch in (1, 2, 3):
        packed = [native.pack(x) for x in xs]
        if f32:
            # the partial sums cross as fp32: the reference sum is built from fp32 partials too
            partial32 = []
            for r in range(world):
                layer, (q, sf) = layers[r], packed[r]
                out32 = torch.zeros(2 * half, dtype=torch.uint8, device="cuda")
                st = torch.zeros(4, dtype=torch.int32, device="cuda")
                y0 = torch.empty(tokens, outputs, dtype=dtype, device="cuda")
                low, high_p = layer.problems(q, sf, y0)
                layer.run_packed(q, sf)                                   # warms the handle
                handle = layer.handles[next(k_ for k_ in layer.handles if k_[0] == tokens)]
                native.check(lib.hg_run_partial(handle, C.byref(low), C.byref(high_p), None, 0, out32.data_ptr(), half, 1,
                                                st.data_ptr(), stream))
                partial32.append(out32[half:half + elems * 4].view(torch.float32).clone())   # exchange 1 -> second half
            total = partial32[0]
            for r in range(1, world):             # rank order, as the kernel adds
                total = total + partial32[r]
            want = total.to(dtype).view(tokens, outputs)
        else:
            partial = [layers[r].run_packed(*packed[r]) for r in range(world)]
            total = partial[0].float()
            for r in range(1, world):
                total = total + partial[r].float()
            want = total.to(dtype)
        for r in range(world):                    # the publishes of the ranks that run later, ahead of time
            flags[r][r + 1:world] = epoch
        ys = [torch.empty(tokens, outputs, dtype=dtype, device="cuda") for _ in range(world)]
        for r in range(world):                    # both GEMMs write their partials before any all-reduce runs
            layer, (q, sf) = layers[r], packed[r]
            low, high_p = layer.problems(xs[r] if fused else q, xs[r] if fused else sf, ys[r])
            if not layer.handles:
                layer.run_packed(q, sf)
            handle = layer.handles[next(k_ for k_ in layer.handles if k_[0] == tokens)]
            native.check(lib.hg_run_partial(handle, C.byref(low), C.byref(high_p), xs[r].data_ptr() if fused else None,
                                            native.DTYPES[dtype], bufs[r].data_ptr(), half, f32,
                                            ex[r].state.data_ptr(), stream))
        for r in range(world):
            native.check(lib.hg_tp_allreduce(ex[r].buffer_ptrs, ys[r].data_ptr(), elems, half, f32, world, r,
                                             ex[r].flag_ptrs, ex[r].state.data_ptr(), native.DTYPES[dtype], stream))
        torch.cuda.synchronize()
        for r in range(world):
            assert ex[r].status() == 0
            assert ex[r].state[0].item() == epoch
            assert (bits(ys[r]) == bits(want)).all(), f"rank {r} epoch {epoch}"
    assert all(layer.status()[0] == 0 for layer in layers)


def test_single_rank_exchange_equals_plain_run():
    layers, xs = shards(16, 512, 384, 40, 1, torch.bfloat16)
    half = 16 * 384 * 4
    bufs, flags = buffers(1, half)
    ex = LocalExchange(1, 0, half, bufs, flags, torch.bfloat16)
    want = layers[0](xs[0])
    for _ in range(2):
        got = layers[0].run_exchange(ex, x=xs[0])
        q, sf = native.pack(xs[0])
        got_packed = layers[0].run_exchange(ex, q=q, sf=sf)
        torch.cuda.synchronize()
        assert (bits(got) == bits(want)).all() and (bits(got_packed) == bits(want)).all()
    assert ex.status() == 0 and ex.state[0].item() == 4


def test_missing_peer_ends_the_wait_with_a_status(monkeypatch):
    """A flag that nothing sets: the all-reduce gives up after its limit (about a second), reports which rank it
    waited for, fills the output with NaN so the failure cannot pass for a result, still advances the exchange
    count and the context stays usable; the same through `DualLinear.run_exchange`."""
    world, tokens, outputs = 2, 8, 256
    half = tokens * outputs * 4
    bufs, flags = buffers(world, half)
    ex = LocalExchange(world, 0, half, bufs, flags, torch.bfloat16)
    out = torch.full((tokens, outputs), 7.0, dtype=torch.bfloat16, device="cuda")
    native.check(native.library().hg_tp_allreduce(ex.buffer_ptrs, out.data_ptr(), tokens * outputs, half, 1, world, 0,
                                                  ex.flag_ptrs, ex.state.data_ptr(), 1, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert ex.status() == 1001
    assert ex.status() == 0
    assert torch.isnan(out.float()).all() and ex.state[0].item() == 1
    layers, xs = shards(tokens, 512, outputs, 32, 1, torch.bfloat16)
    y = layers[0].run_exchange(ex, x=xs[0])                                    # rank 1 never publishes exchange 2
    torch.cuda.synchronize()
    assert ex.status() == 1001 and torch.isnan(y.float()).all() and ex.state[0].item() == 2
    assert layers[0].status()[0] == 0
    assert torch.ones(4, device="cuda").sum().item() == 4.0


def test_bench_shards_stay_consistent_at_eight_ranks():
    """The benchmark's tensor-parallel shards: gate_up keeps exactly the intermediate channels of the rank's
    K shard of down_proj (whole K128 blocks, uneven at 8 ranks), so the SwiGLU producer feeds down_proj."""
    import importlib.util
    import sys
    from pathlib import Path
    from hygemm_vllm import producer
    spec = importlib.util.spec_from_file_location("bench_module", Path(__file__).resolve().parent.parent / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(bench)
    finally:
        sys.argv = argv
    total = 0
    for rank in (0, 3, 7):
        layer = bench.build_layer(torch.device("cuda", 0), bench.SEED, rank, 8)
        assert layer["gate_up"].outputs == 2 * layer["down"].k and layer["down"].k % 128 == 0
        assert layer["o_proj"].k % 128 == 0 and layer["qkv"].outputs == 4608 // 8
        x = torch.randn(16, 3584, dtype=torch.bfloat16, device="cuda")
        q, sf = producer.silu_pack(layer["gate_up"](x), 0)
        y = layer["down"].run_packed(q, sf)
        assert y.shape == (16, 3584) and torch.isfinite(y.float()).all()
        total += layer["down"].k
        for rt in layer.values():
            rt.close()
    assert total in (2432 + 2432 + 2304, 2432 * 2 + 2304, 2432 + 2304 * 2)
