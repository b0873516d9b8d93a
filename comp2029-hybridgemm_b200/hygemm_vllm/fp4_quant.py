"""Offline MXFP4 quantisation with a per-group exponent search, and the E2M1 helpers around it.

Counterpart of the reference's `integrations/vllm/allocation/fp4_quant.py`: same
function names, arguments and return values (`unpack`, `codes_rne`, `pack_codes`,
`decode_logical`, `quantize`).  The search itself is one CUDA kernel
(`hg_clip_pack`) instead of a chain of full-tensor torch ops; the helpers are
plain torch and run on any device, which is what the CPU tests use.  Online
quantisation and the GEMM are untouched: the result only replaces the stored
MXFP4 rows of a layer (`offline_weights.replace_low_weight`).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import native
from .offline_weights import logical_scales

# Midpoints between neighbouring E2M1 magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6.
_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def unpack(q: torch.Tensor) -> torch.Tensor:
    """`[rows, k/2]` bytes -> `[rows, k]` 4-bit codes (even k in the low nibble)."""
    return torch.stack((q & 15, q >> 4), dim=-1).reshape(q.shape[0], -1)


def pack_codes(code: torch.Tensor) -> torch.Tensor:
    """`[rows, k]` 4-bit codes -> `[rows, k/2]` bytes."""
    return (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()


def codes_rne(x: torch.Tensor) -> torch.Tensor:
    """E2M1 code of every element: nearest magnitude, ties to the even code, saturating at 6, sign kept for -0."""
    mids = torch.tensor(_MIDPOINTS, dtype=x.dtype, device=x.device)
    mag = x.abs().contiguous()
    code = torch.bucketize(mag, mids, right=False)                  # first midpoint >= |x|
    on_midpoint = (code < 7) & (mag == mids[code.clamp(max=6)])
    code = code + (on_midpoint & (code % 2 == 1)).long()             # an odd code on a midpoint yields to its even neighbour
    return code.to(torch.uint8) | (torch.signbit(x).to(torch.uint8) << 3)


def decode_logical(q: torch.Tensor, scales: torch.Tensor, k: int) -> torch.Tensor:
    """fp32 values of packed codes `[rows, k/2]` under logical scale bytes `[rows, k/32]`."""
    table = torch.tensor(_MAGNITUDES + tuple(-m for m in _MAGNITUDES), dtype=torch.float32, device=q.device)
    table[8] = 0.0
    values = table[unpack(q).long()].reshape(q.shape[0], k // 32, 32)
    return (values * torch.exp2(scales.float() - 127).unsqueeze(-1)).reshape(q.shape[0], k)


def quantize(w: torch.Tensor, importance: torch.Tensor | None = None, offsets=(0, -1, -2)):
    """Search the E8M0 exponent of every K32 group of `w` `[rows, k]` (reference: fp4_quant.py:28-58).

    Returns `(q4 [rows, k/2], scales [rows, k/32], stats)`: codes and logical scale bytes that never have a
    larger importance-weighted squared error than round-to-nearest, and the same statistics dictionary as the
    reference (`groups`, `shift_groups`, `weighted_error_before/after`, `weight_error_before/after`).
    """
    if w.ndim != 2 or w.dtype not in native.DTYPES or not w.is_cuda or w.shape[1] % 128:
        raise ValueError("quantize needs a CUDA FP16/BF16 [rows, K] matrix with K % 128 == 0")
    if not torch.isfinite(w).all():
        raise ValueError("weights must be finite")
    rows, k = w.shape
    w = w.contiguous()
    weight = None
    if importance is not None:
        weight = importance.to(device=w.device, dtype=torch.float32).contiguous()
        if weight.shape != (k,) or not torch.isfinite(weight).all() or (weight < 0).any():
            raise ValueError("importance must be k finite non-negative values")
    q4 = torch.empty((rows, k // 2), dtype=torch.uint8, device=w.device)
    scales = torch.empty((rows, k // 32), dtype=torch.uint8, device=w.device)
    shifts = (C.c_int * len(offsets))(*[int(o) for o in offsets])
    lib = native.library()
    lib.hg_clip_pack.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                 C.POINTER(C.c_int), C.c_int, C.c_int, C.c_void_p]
    native.check(lib.hg_clip_pack(w.data_ptr(), weight.data_ptr() if weight is not None else None, q4.data_ptr(),
                                  scales.data_ptr(), rows, k, shifts, len(offsets), native.DTYPES[w.dtype],
                                  torch.cuda.current_stream(w.device).cuda_stream))

    # Statistics against the round-to-nearest baseline (the same kernel with no offsets is hg_pack's result).
    base_q, base_sf = native.pack(w, True)
    base_scales = logical_scales(base_sf, rows, k)
    source = w.float().reshape(rows, k // 32, 32)
    per_k = (torch.ones(k, device=w.device) if weight is None else weight).reshape(1, k // 32, 32)
    before = (decode_logical(base_q, base_scales, k).reshape_as(source) - source).square()
    after = (decode_logical(q4, scales, k).reshape_as(source) - source).square()
    weighted_before, weighted_after = (before * per_k).sum(-1), (after * per_k).sum(-1)
    if not torch.all(weighted_after <= weighted_before * (1 + 1e-6) + 1e-25):
        raise AssertionError("exponent search increased a group's weighted error")
    moved = base_scales.int() - scales.int()
    stats = {"groups": rows * (k // 32),
             "shift_groups": {str(-s): int((moved == -s).sum()) for s in offsets},
             "weighted_error_before": weighted_before.double().sum().item(),
             "weighted_error_after": weighted_after.double().sum().item(),
             "weight_error_before": before.double().sum().item(),
             "weight_error_after": after.double().sum().item()}
    return q4, scales, stats
