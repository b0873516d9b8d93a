"""`hg_run_static`, the entry point for callers that cannot allocate device memory where a layer runs
(an engine whose pool owns the device, a latency-critical loop, a shape met only when it must run).

Its scratch — tile schedule, split-K partial sums, arrival counters — sits in a fixed array inside the
library instead of in a handle, so the test checks through the C ABI that it produces exactly what the
handle-based `hg_create` + `hg_run` path produces, twice in a row (the second call finds the array as the
first one left it), and that a shape too large for the array is refused instead of launched.

Collected last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import dev, make_inputs, run_gemm
from hygemm_vllm import native

pytestmark = pytest.mark.gpu


def _operands(tokens, k, outputs, high, exact=False):
    if exact:
        return oracle.exact_case(outputs, tokens, k, high, "random")
    x, w, ids = make_inputs(tokens, k, outputs, high)
    layer = native.DualLinear(w.cuda(), ids.cuda())
    xq, xsf = native.pack(x.cuda())
    case = dict(w4=layer.w4.cpu().numpy(), sf4=layer.sf4.cpu().numpy(), lo=layer.lo.cpu().numpy(),
                w8=layer.w8.cpu().numpy(), sf8=layer.sf8.cpu().numpy(), hi=layer.hi.cpu().numpy(),
                xq=xq.cpu().numpy(), xsf=xsf.cpu().numpy(), outputs=outputs, tokens=tokens, k=k)
    layer.close()
    return case


def _run_static(case, schedule, dtype=torch.bfloat16, calls=2):
    lib = native.library()
    tokens, k = case["xq"].shape
    outputs = case["outputs"]
    d = {n: dev(case[n]) for n in ("w4", "sf4", "lo", "w8", "sf8", "hi", "xq", "xsf")}
    stream = torch.cuda.current_stream().cuda_stream
    results = []
    for _ in range(calls):
        y = torch.full((tokens, outputs), -1, dtype=torch.int16, device="cuda")      # 0xffff: NaN in bf16/fp16

        def ptr(t):
            return t.data_ptr() if t.numel() else None
        low = native.Problem(d["lo"].numel(), tokens, k, outputs, ptr(d["w4"]), d["xq"].data_ptr(), ptr(d["sf4"]),
                             d["xsf"].data_ptr(), ptr(d["lo"]), y.data_ptr())
        high = native.Problem(d["hi"].numel(), tokens, k, outputs, ptr(d["w8"]), d["xq"].data_ptr(), ptr(d["sf8"]),
                              d["xsf"].data_ptr(), ptr(d["hi"]), y.data_ptr())
        native.check(lib.hg_run_static(schedule, C.byref(low), C.byref(high), stream, native.DTYPES[dtype]))
        torch.cuda.synchronize()
        results.append(y.cpu().numpy().view(np.uint16))
    return results


@pytest.mark.parametrize("shape", [(7, 256, 257, 26, True), (33, 384, 511, 73, True), (16, 3584, 4608, 512, False),
                                   (1, 18944, 3584, 384, False)])
@pytest.mark.parametrize("schedule", [0, 3])
def test_static_scratch_entry_point_equals_handle_path_on_two_calls(shape, schedule):
    tokens, k, outputs, high, exact = shape
    case = _operands(tokens, k, outputs, high, exact)
    reference, guards, status = run_gemm(case, torch.bfloat16, schedule)
    assert status[0] == 0 and guards
    first, second = _run_static(case, schedule)
    # Same kernel, same schedule, fixed-order fix-up: the outputs are bit-identical (tolerance 0),
    # which is also what the other GEMM tests demand between runs.
    assert np.array_equal(first, reference)
    assert np.array_equal(second, reference)
    if exact:
        assert np.array_equal(first, case["expected"])


def test_shape_beyond_the_static_array_is_refused():
    lib = native.library()
    # 128 tokens x 4608 outputs cut by split-K needs far more than HG_STATIC_SCRATCH_BYTES of partial sums.
    case = _operands(128, 3584, 4608, 512)
    with pytest.raises(RuntimeError, match="bytes of scratch"):
        _run_static(case, 2, calls=1)
    assert b"static buffer holds" in lib.hg_last_error()
    bad = native.Problem()
    assert lib.hg_run_static(0, C.byref(bad), C.byref(bad), None, 1) == -1
    assert lib.hg_run_static(9, None, None, None, 1) == -1


def test_static_path_allocates_nothing_reports_its_status_and_refuses_capture():
    """Free device memory is the same before and after the calls (first call included: its set-up only looks
    up an address); the status words of the array have their own reader, so a bounded wait that expired on
    this path would be seen; and a capturing stream is refused, because the call copies a schedule from host
    memory that a later call rewrites."""
    lib = native.library()
    case = _operands(16, 3584, 3584, 384)
    torch.cuda.synchronize()
    status = (C.c_int * 3)()
    stream = torch.cuda.current_stream().cuda_stream
    native.check(lib.hg_static_status(stream, status))            # also performs the per-device set-up
    free_before, _ = torch.cuda.mem_get_info()
    other = _operands(4, 896, 640, 64)                              # torch allocations happen out here, not inside
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    d = {n: dev(case[n]) for n in ("w4", "sf4", "lo", "w8", "sf8", "hi", "xq", "xsf")}
    e = {n: dev(other[n]) for n in ("w4", "sf4", "lo", "w8", "sf8", "hi", "xq", "xsf")}
    y = torch.zeros(16 * 3584, dtype=torch.int16, device="cuda")
    y2 = torch.zeros(4 * 640, dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()

    def problems(t, tokens, k, outputs, out):
        low = native.Problem(t["lo"].numel(), tokens, k, outputs, t["w4"].data_ptr(), t["xq"].data_ptr(), t["sf4"].data_ptr(),
                             t["xsf"].data_ptr(), t["lo"].data_ptr(), out.data_ptr())
        high = native.Problem(t["hi"].numel(), tokens, k, outputs, t["w8"].data_ptr(), t["xq"].data_ptr(), t["sf8"].data_ptr(),
                              t["xsf"].data_ptr(), t["hi"].data_ptr(), out.data_ptr())
        return low, high
    big, small = problems(d, 16, 3584, 3584, y), problems(e, 4, 896, 640, y2)
    for low, high in (big, small, big, small):                      # alternating shapes: schedules come from the cache
        native.check(lib.hg_run_static(0, C.byref(low), C.byref(high), stream, 1))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    native.check(lib.hg_static_status(stream, status))
    tiles_big = -(-d["lo"].numel() // 128) + -(-d["hi"].numel() // 128)
    tiles_small = -(-e["lo"].numel() // 128) + -(-e["hi"].numel() // 128)
    assert status[0] == 0
    assert status[1] == 2 * (tiles_big * (3584 // 128) + tiles_small * (896 // 128))     # K128 blocks issued
    native.check(lib.hg_static_status(stream, status))
    assert list(status) == [0, 0, 0]                                                      # cleared by the read
    graph = torch.cuda.CUDAGraph()
    with pytest.raises(RuntimeError, match="cannot be captured"):
        with torch.cuda.graph(graph):
            low, high = big
            native.check(lib.hg_run_static(0, C.byref(low), C.byref(high), torch.cuda.current_stream().cuda_stream, 1))
    torch.cuda.synchronize()
    assert torch.ones(4, device="cuda").sum().item() == 4.0
