"""CPU oracle for the hybrid MXFP4/MXFP8 linear layer — TEST INFRASTRUCTURE ONLY.

Thin ctypes/numpy front end over ``mx_oracle.c`` (a plain-C restatement of the
reference algorithm; every C function cites the reference file:line it
follows).  Only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may import this package; the product path never does.

Parity status: pinned (see the header of ``mx_oracle.c`` and ``tests/golden``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "libmx_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile ``mx_oracle.c`` with the Makefile beside it (gcc, no GPU needed)."""
    src = _HERE / "mx_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_SO))
        u8p, u16p, i32p, f32p = (C.POINTER(t) for t in (C.c_uint8, C.c_uint16, C.c_int32, C.c_float))
        L.hgo_scale_size.restype = C.c_int64
        L.hgo_scale_size.argtypes = [C.c_int, C.c_int]
        L.hgo_scale_index.restype = C.c_int64
        L.hgo_scale_index.argtypes = [C.c_int] * 3
        L.hgo_pack.argtypes = [u16p, u8p, u8p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.hgo_silu_pack.argtypes = [u16p, u8p, u8p, u16p, C.c_int, C.c_int, C.c_int]
        L.hgo_decode.argtypes = [u8p, u8p, f32p, C.c_int, C.c_int, C.c_int]
        L.hgo_clip_pack.argtypes = [u16p, f32p, u8p, u8p, C.c_int, C.c_int, i32p, C.c_int, C.c_int]
        L.hgo_hybrid_linear.argtypes = [u8p, u8p, i32p, C.c_int, u8p, u8p, i32p, C.c_int,
                                        u8p, u8p, C.c_int, C.c_int, C.c_int, u16p, C.c_int, f32p]
        L.hgo_exact_weights.argtypes = [i32p, C.c_int, C.c_int, C.c_int, u8p, u8p]
        L.hgo_exact_activations.argtypes = [C.c_int, C.c_int, u8p, u8p]
        L.hgo_exact_expected.argtypes = [u8p, C.c_int, C.c_int, C.c_int, u16p, C.c_int]
        L.hgo_exact_expected.restype = None
        for name, res, args in [
            ("hgo_half_to_float", C.c_float, [C.c_uint16]), ("hgo_bf16_to_float", C.c_float, [C.c_uint16]),
            ("hgo_float_to_half", C.c_uint16, [C.c_float]), ("hgo_float_to_bf16", C.c_uint16, [C.c_float]),
            ("hgo_e4m3_from_float", C.c_uint8, [C.c_float]), ("hgo_e4m3_to_float", C.c_float, [C.c_uint8]),
            ("hgo_e2m1_from_float", C.c_uint8, [C.c_float]), ("hgo_e2m1_to_float", C.c_float, [C.c_uint8]),
            ("hgo_exponent_literal", C.c_int, [C.c_float, C.c_int]),
            ("hgo_exponent_exact", C.c_int, [C.c_float, C.c_int]),
            ("hgo_exact_reference", C.c_float, [C.c_int] * 4),
            ("hgo_threads", C.c_int, []), ("hgo_set_threads", None, [C.c_int]),
        ]:
            getattr(L, name).restype = res
            getattr(L, name).argtypes = args
        _lib = L
    return _lib


def _ptr(a: np.ndarray, ctype):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.POINTER(ctype))


def as_u16(x) -> np.ndarray:
    """Bit view of a 16-bit float array/tensor (torch bf16/fp16 or numpy) as uint16."""
    try:
        import torch
        if isinstance(x, torch.Tensor):
            return x.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    except ImportError:
        pass
    x = np.ascontiguousarray(x)
    return x.view(np.uint16) if x.dtype != np.uint16 else x


def scale_size(rows: int, k: int) -> int:
    return int(lib().hgo_scale_size(rows, k))


def scale_indices(rows: int, k: int) -> np.ndarray:
    r = np.arange(rows, dtype=np.int64)[:, None]
    g = np.arange(k // 32, dtype=np.int64)[None, :]
    return ((r // 128) * (k // 128) + g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4


def pack(x, fp4: bool = False, bf16: bool = True):
    """Quantise ``[rows,k]`` 16-bit floats → (codes, padded scales)."""
    bits = as_u16(x)
    rows, k = bits.shape
    q = np.zeros((rows, k // 2 if fp4 else k), dtype=np.uint8)
    sf = np.zeros(scale_size(rows, k), dtype=np.uint8)
    if rows:
        status = lib().hgo_pack(_ptr(bits, C.c_uint16), _ptr(q, C.c_uint8), _ptr(sf, C.c_uint8),
                                rows, k, int(fp4), int(bf16))
        if status:
            raise ValueError("Invalid MX pack arguments")
    return q, sf


def silu_pack(x, bf16: bool = True, debug: bool = False):
    """``[rows, 2k]`` gate‖up → (codes ``[rows,k]``, scales[, 16-bit intermediate bits])."""
    bits = as_u16(x)
    rows, k2 = bits.shape
    k = k2 // 2
    q = np.zeros((rows, k), dtype=np.uint8)
    sf = np.zeros(scale_size(rows, k), dtype=np.uint8)
    dbg = np.zeros((rows, k), dtype=np.uint16) if debug else None
    status = lib().hgo_silu_pack(_ptr(bits, C.c_uint16), _ptr(q, C.c_uint8), _ptr(sf, C.c_uint8),
                                 _ptr(dbg, C.c_uint16), rows, k, int(bf16))
    if status:
        raise ValueError("Invalid SwiGLU pack arguments")
    return (q, sf, dbg) if debug else (q, sf)


def clip_pack(x, importance=None, offsets=(0, -1, -2), bf16: bool = True):
    """Offline MXFP4 exponent search → (packed codes ``[rows,k/2]``, logical scale bytes ``[rows,k/32]``)."""
    bits = as_u16(x)
    rows, k = bits.shape
    q4 = np.zeros((rows, k // 2), dtype=np.uint8)
    scales = np.zeros((rows, k // 32), dtype=np.uint8)
    weight = None if importance is None else np.ascontiguousarray(importance, dtype=np.float32)
    if weight is not None and weight.shape != (k,):
        raise ValueError("importance must have k entries")
    shifts = np.ascontiguousarray(offsets, dtype=np.int32)
    status = lib().hgo_clip_pack(_ptr(bits, C.c_uint16), _ptr(weight, C.c_float), _ptr(q4, C.c_uint8),
                                 _ptr(scales, C.c_uint8), rows, k, _ptr(shifts, C.c_int32), len(shifts), int(bf16))
    if status:
        raise ValueError("Invalid clipping-quantiser arguments")
    return q4, scales


def decode(q: np.ndarray, sf: np.ndarray, k: int, fp4: bool) -> np.ndarray:
    rows = q.shape[0]
    out = np.zeros((rows, k), dtype=np.float32)
    if rows:
        lib().hgo_decode(_ptr(np.ascontiguousarray(q), C.c_uint8), _ptr(np.ascontiguousarray(sf), C.c_uint8),
                         _ptr(out, C.c_float), rows, k, int(fp4))
    return out


def hybrid_linear(w4, sf4, lo, w8, sf8, hi, xq, xsf, outputs: int, bf16: bool = True):
    """Dequantise-and-matmul with scatter → (16-bit output bits, fp32 output)."""
    tokens, k = xq.shape
    y = np.zeros((tokens, outputs), dtype=np.uint16)
    yf = np.zeros((tokens, outputs), dtype=np.float32)
    lo = np.ascontiguousarray(lo, dtype=np.int32)
    hi = np.ascontiguousarray(hi, dtype=np.int32)
    dummy8 = np.zeros(1, dtype=np.uint8)
    dummyi = np.zeros(1, dtype=np.int32)
    args = []
    for a in (w4, sf4):
        args.append(np.ascontiguousarray(a) if a is not None and a.size else dummy8)
    status = lib().hgo_hybrid_linear(
        _ptr(args[0], C.c_uint8), _ptr(args[1], C.c_uint8), _ptr(lo if lo.size else dummyi, C.c_int32), lo.size,
        _ptr(np.ascontiguousarray(w8) if w8 is not None and w8.size else dummy8, C.c_uint8),
        _ptr(np.ascontiguousarray(sf8) if sf8 is not None and sf8.size else dummy8, C.c_uint8),
        _ptr(hi if hi.size else dummyi, C.c_int32), hi.size,
        _ptr(np.ascontiguousarray(xq), C.c_uint8), _ptr(np.ascontiguousarray(xsf), C.c_uint8),
        tokens, k, outputs, _ptr(y, C.c_uint16), int(bf16), _ptr(yf, C.c_float))
    if status:
        raise ValueError("Invalid hybrid linear arguments")
    return y, yf


def partition(outputs: int, high_ids) -> tuple[np.ndarray, np.ndarray]:
    """lo/hi ascending int32 row lists (integrations/vllm/hygemm_vllm/native.py:56-59)."""
    mask = np.zeros(outputs, dtype=bool)
    mask[np.asarray(high_ids, dtype=np.int64)] = True
    return np.where(~mask)[0].astype(np.int32), np.where(mask)[0].astype(np.int32)


def exact_maps(outputs: int, high: int, mapping: str):
    """Channel maps of the exact-representable cases (src/kernel/output_channel_bench.cu:74-86).

    ``random`` shuffles with a seeded numpy generator instead of the C++
    ``std::shuffle(mt19937(20261024))`` order (the shuffle algorithm of the C++
    library is implementation-defined); membership and order are still random,
    which is what the case exercises.
    """
    is_high = np.zeros(outputs, dtype=np.uint8)
    if mapping == "contiguous":
        is_high[outputs - high:] = 1
    else:
        i = np.arange(outputs, dtype=np.int64)
        is_high[:] = ((i + 1) * high // outputs) != (i * high // outputs)
    low = np.where(is_high == 0)[0].astype(np.int32)
    hi = np.where(is_high == 1)[0].astype(np.int32)
    if mapping == "random":
        perm = np.random.default_rng(20261024).permutation(outputs).astype(np.int32)
        hi, low = perm[:high].copy(), perm[high:].copy()
        is_high[:] = 0
        is_high[hi] = 1
    return low, hi, is_high


def exact_case(outputs: int, tokens: int, k: int, high: int, mapping: str = "interleaved", bf16: bool = True):
    """Inputs and bit-exact expected output of one exact-representable case."""
    low, hi, is_high = exact_maps(outputs, high, mapping)
    L = lib()
    w4 = np.zeros((low.size, k // 2), dtype=np.uint8)
    sf4 = np.zeros(scale_size(low.size, k), dtype=np.uint8)
    w8 = np.zeros((hi.size, k), dtype=np.uint8)
    sf8 = np.zeros(scale_size(hi.size, k), dtype=np.uint8)
    if low.size:
        L.hgo_exact_weights(_ptr(low, C.c_int32), low.size, k, 0, _ptr(w4, C.c_uint8), _ptr(sf4, C.c_uint8))
    if hi.size:
        L.hgo_exact_weights(_ptr(hi, C.c_int32), hi.size, k, 1, _ptr(w8, C.c_uint8), _ptr(sf8, C.c_uint8))
    xq = np.zeros((tokens, k), dtype=np.uint8)
    xsf = np.zeros(scale_size(tokens, k), dtype=np.uint8)
    L.hgo_exact_activations(tokens, k, _ptr(xq, C.c_uint8), _ptr(xsf, C.c_uint8))
    y = np.zeros((tokens, outputs), dtype=np.uint16)
    L.hgo_exact_expected(_ptr(is_high, C.c_uint8), outputs, tokens, k, _ptr(y, C.c_uint16), int(bf16))
    return dict(w4=w4, sf4=sf4, lo=low, w8=w8, sf8=sf8, hi=hi, xq=xq, xsf=xsf, expected=y,
                outputs=outputs, tokens=tokens, k=k)


def threads() -> int:
    return int(lib().hgo_threads())
