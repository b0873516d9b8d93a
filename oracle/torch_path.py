"""PyTorch restatement of the reference's dequantise-and-matmul path — TEST/BASELINE INFRASTRUCTURE ONLY.

Port of `decode_mx` and `reference` of the reference's
`integrations/vllm/test_components.py:10-38` (vectorised torch on CPU, fp32
`dx @ w.T`), with the CUDA-only activation `pack` replaced by the C oracle's
quantiser.  It is what the benchmark times as the CPU baseline (`kind: "port"`,
all host threads through torch's intra-op pool) and a second, independent
implementation the C oracle is cross-checked against.  Never imported by the
product path.
"""
from __future__ import annotations

import numpy as np
import torch

from . import pack as oracle_pack

_E2M1 = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32)


def decode_mx(q: torch.Tensor, sf: torch.Tensor, k: int, fp4: bool) -> torch.Tensor:
    """uint8 codes + physical E8M0 scales -> fp32 `[rows,k]` (test_components.py:10-24)."""
    rows = q.shape[0]
    if rows == 0:
        return torch.empty((0, k), dtype=torch.float32)
    if fp4:
        nibbles = torch.stack((q & 15, q >> 4), dim=-1).reshape(rows, k).long()
        values = _E2M1[nibbles]
    else:
        values = q.view(torch.float8_e4m3fn).float()
    r = torch.arange(rows).unsqueeze(1)
    g = torch.arange(k // 32).unsqueeze(0)
    index = ((r // 128) * (k // 128) + g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4
    scale = torch.exp2(sf[index].float() - 127)
    return (values.view(rows, k // 32, 32) * scale.unsqueeze(-1)).reshape(rows, k)


def reference_linear(x: torch.Tensor, w4, sf4, lo, w8, sf8, hi, outputs: int, redequantise: bool = True,
                     cache: dict | None = None) -> torch.Tensor:
    """`reference(runtime, x, 'hygemm')` (test_components.py:27-38): quantise x, dequantise both operands,
    fp32 matmul, cast to x's dtype.  `redequantise=False` reuses the dequantised weights kept in `cache`
    (what a CPU deployment would do); the literal reference re-dequantises on every call."""
    k = x.shape[1]
    xq, xsf = oracle_pack(x, fp4=False, bf16=x.dtype == torch.bfloat16)
    dx = decode_mx(torch.from_numpy(xq), torch.from_numpy(xsf), k, False)
    if redequantise or cache is None or "w" not in cache:
        w = torch.empty(outputs, k)
        w[torch.as_tensor(np.asarray(lo)).long()] = decode_mx(torch.as_tensor(w4), torch.as_tensor(sf4), k, True)
        w[torch.as_tensor(np.asarray(hi)).long()] = decode_mx(torch.as_tensor(w8), torch.as_tensor(sf8), k, False)
        if cache is not None:
            cache["w"] = w
    else:
        w = cache["w"]
    return (dx @ w.t()).to(x.dtype)
