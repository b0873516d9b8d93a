"""Shared helpers of the GPU parity tests: device buffers by torch, calls through the C ABI."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

import oracle
from hygemm_vllm import native

SEED = 20261024


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def make_inputs(tokens, k, outputs, high, dtype=torch.bfloat16, seed=SEED, outliers=True):
    """Synthetic layer: x ~ N(0,1) with 1 % of K columns x20, w ~ N(0,0.02), seeded sorted high set."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, k, generator=g)
    if outliers:
        cols = torch.randperm(k, generator=g)[: max(1, -(-k // 100))]
        x[:, cols] *= 20
    w = torch.randn(outputs, k, generator=g) * 0.02
    ids = torch.sort(torch.randperm(outputs, generator=g)[:high]).values
    return x.to(dtype), w.to(dtype), ids


def run_gemm(case: dict, dtype=torch.bfloat16, schedule=0, policy=0, fill=0xFF, guard=256, runs=1):
    """hg_create_dtype + hg_run on device copies of an operand dict (w4,sf4,lo,w8,sf8,hi,xq,xsf).

    The output is pre-filled with NaN bit patterns and surrounded by guard bands
    (0x5a5a), as the reference's harness does (src/kernel/output_channel_bench.cu:115-131).
    Returns (output bits [tokens,outputs], guards_intact, status tuple).
    """
    lib = native.library()
    tokens, k = case["xq"].shape
    outputs = case["outputs"]
    d = {n: dev(case[n]) for n in ("w4", "sf4", "lo", "w8", "sf8", "hi", "xq", "xsf")}
    buf = torch.full((tokens * outputs + 2 * guard,), 0x5A5A, dtype=torch.int16, device="cuda")
    y = buf[guard: guard + tokens * outputs]
    y.fill_(-1 if fill else 0)                      # 0xffff is a NaN in fp16 and in bf16
    def ptr(t):
        return t.data_ptr() if t.numel() else None
    low = native.Problem(d["lo"].numel(), tokens, k, outputs, ptr(d["w4"]), d["xq"].data_ptr(), ptr(d["sf4"]),
                         d["xsf"].data_ptr(), ptr(d["lo"]), y.data_ptr())
    hi = native.Problem(d["hi"].numel(), tokens, k, outputs, ptr(d["w8"]), d["xq"].data_ptr(), ptr(d["sf8"]),
                        d["xsf"].data_ptr(), ptr(d["hi"]), y.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    handle = C.c_void_p()
    native.check(lib.hg_create_dtype(schedule, schedule, C.byref(low), C.byref(hi), stream, native.DTYPES[dtype],
                                     C.byref(handle)))
    try:
        for _ in range(runs):
            native.check(lib.hg_run(handle, C.byref(low), C.byref(hi), stream, policy))
        status = (C.c_int * 3)()
        native.check(lib.hg_status(handle, stream, status))
        torch.cuda.synchronize()
    finally:
        lib.hg_destroy(handle)
    host = buf.cpu().numpy().view(np.uint16)
    guards_ok = bool(np.all(host[:guard] == 0x5A5A) and np.all(host[-guard:] == 0x5A5A))
    return host[guard:-guard].reshape(tokens, outputs).copy(), guards_ok, tuple(status)


def quantised_case(tokens, k, outputs, high, dtype=torch.bfloat16, seed=SEED):
    """Operands quantised by the CPU oracle plus the oracle's fp32 and 16-bit outputs."""
    x, w, ids = make_inputs(tokens, k, outputs, high, dtype, seed)
    bf16 = dtype == torch.bfloat16
    lo, hi = oracle.partition(outputs, ids.numpy())
    w4, sf4 = oracle.pack(w[torch.from_numpy(lo).long()], fp4=True, bf16=bf16)
    w8, sf8 = oracle.pack(w[torch.from_numpy(hi).long()], fp4=False, bf16=bf16)
    xq, xsf = oracle.pack(x, fp4=False, bf16=bf16)
    y16, yf = oracle.hybrid_linear(w4, sf4, lo, w8, sf8, hi, xq, xsf, outputs, bf16=bf16)
    return dict(w4=w4, sf4=sf4, lo=lo, w8=w8, sf8=sf8, hi=hi, xq=xq, xsf=xsf, outputs=outputs, tokens=tokens, k=k,
                expected=y16, expected_f32=yf, x=x, w=w, ids=ids)


def to_float(bits16: np.ndarray, dtype) -> np.ndarray:
    t = torch.from_numpy(bits16.view(np.int16).copy())
    return t.view(dtype).float().numpy()


def rel_frobenius(got: np.ndarray, ref: np.ndarray) -> float:
    return float(np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref), 1e-30))
