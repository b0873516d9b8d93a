"""Logical <-> physical E8M0 scale layout and load-time MXFP4 replacement.

Mirror of the reference's `integrations/vllm/hygemm_vllm/offline_weights.py`.
Physical layout: 512-byte atoms of 128 rows x 4 K32 groups, row r / group g at
`((r//128)*(K//128) + g//4)*512 + (r%32)*16 + ((r%128)//32)*4 + g%4`; padding 0x7f.
"""
from __future__ import annotations

import torch


def scale_indices(rows, k, device):
    r = torch.arange(rows, device=device).unsqueeze(1)
    g = torch.arange(k // 32, device=device).unsqueeze(0)
    atom = (r // 128) * (k // 128) + g // 4
    return atom * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4


def scale_size(rows, k):
    return ((rows + 127) // 128) * (k // 128) * 512 if rows > 0 else 0


def logical_scales(sf, rows, k):
    """Physical buffer -> `[rows, K/32]` bytes."""
    return sf[scale_indices(rows, k, sf.device)].contiguous()


def physical_scales(values, k):
    """`[rows, K/32]` bytes -> padded physical buffer (padding 0x7f)."""
    rows = values.shape[0]
    if values.shape != (rows, k // 32) or values.dtype != torch.uint8:
        raise ValueError("Logical scales must be uint8 [rows, K/32]")
    out = torch.full((scale_size(rows, k),), 127, dtype=torch.uint8, device=values.device)
    if rows:
        out[scale_indices(rows, k, values.device)] = values
    return out


def replace_low_weight(runtime, q4, scales, verify_native=False):
    """Swap a layer's MXFP4 rows for an offline bank `[N,K/2]` codes + `[N,K/32]` scales
    (reference: offline_weights.py:24-37).  Must run before any GEMM handle exists."""
    if runtime.handles:
        raise RuntimeError("Offline weights must be installed before any GEMM/capture")
    if q4.dtype != torch.uint8 or scales.dtype != torch.uint8:
        raise ValueError("Offline bank tensors must be uint8")
    if q4.shape != (runtime.outputs, runtime.k // 2) or scales.shape != (runtime.outputs, runtime.k // 32):
        raise ValueError("Offline bank shape does not match the layer")
    rows = runtime.lo.long()
    packed = q4.index_select(0, rows.to(q4.device)).contiguous().to(runtime.w4.device)
    logical = scales.index_select(0, rows.to(scales.device)).contiguous().to(runtime.sf4.device)
    sf = physical_scales(logical, runtime.k)
    if packed.shape != runtime.w4.shape or sf.shape != runtime.sf4.shape:
        raise ValueError("Offline bank does not cover the low partition")
    if verify_native:
        if not torch.equal(packed, runtime.w4):
            raise AssertionError("Native-RTN bank payload mismatch")
        if not torch.equal(sf, runtime.sf4):
            raise AssertionError("Native-RTN bank scale/padding mismatch")
    runtime.w4, runtime.sf4 = packed, sf
