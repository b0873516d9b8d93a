"""Fused SwiGLU -> MXFP8 producer feeding down_proj.

Mirror of the reference's `integrations/vllm/hygemm_vllm/producer.py` and
`mistral_producer.py`: `silu_pack` turns the `[M, 2I]` gate||up output of the
hybrid gate_up projection straight into E4M3 codes + E8M0 scales (one kernel
instead of silu_and_mul + memset + pack), and `install()` routes Qwen2 /
Llama / Mistral MLPs through `linear_silu` for up to 128 tokens.
"""
from __future__ import annotations

import os

import torch

from .native import DTYPES, _stream, library, scale_size
from .ops import _runtimes, linear_silu  # noqa: F401  (re-exported, reference layout)

MAX_FUSED_TOKENS = 128


def silu_pack(x: torch.Tensor, math: int = 0, debug: bool = False):
    """`[rows, 2K]` gate||up -> (`q [rows,K]` uint8, `sf`) (reference: producer.py:11-24).

    math 0 = expf + IEEE division (bit-exact with SiluAndMul followed by pack),
    1/2 = fast intrinsics.  With `debug=True` also returns the 16-bit product.
    """
    if not (x.is_cuda and x.is_contiguous() and x.dtype in DTYPES and x.ndim == 2):
        raise ValueError("SwiGLU pack requires contiguous CUDA FP16/BF16 [rows, 2K]")
    rows, k = x.shape[0], x.shape[1] // 2
    if x.shape[1] != 2 * k or k % 128:
        raise ValueError("SwiGLU pack requires K divisible by 128")
    q = torch.empty((rows, k), device=x.device, dtype=torch.uint8)
    sf = torch.empty(scale_size(rows, k) if rows else 0, device=x.device, dtype=torch.uint8)
    dbg = torch.empty((rows, k), device=x.device, dtype=x.dtype) if debug else None
    if rows:
        fn = library().hg_silu_pack_bf16 if x.dtype == torch.bfloat16 else library().hg_silu_pack
        status = fn(x.data_ptr(), q.data_ptr(), sf.data_ptr(), dbg.data_ptr() if debug else None,
                    rows, k, _stream(x.device), math)
        if status:
            raise RuntimeError(f"SwiGLU MX producer CUDA status {status}")
    return (q, sf, dbg) if debug else (q, sf)


def _patch(mlp_class, method_types):
    if getattr(mlp_class, "_hygemm_producer_installed", False):
        return
    original = mlp_class.forward
    math = int(os.environ.get("HYGEMM_SILU_MATH", "0"))

    def forward(self, x):
        method = getattr(self.down_proj, "quant_method", None)
        tokens = x.numel() // x.shape[-1]
        if not isinstance(method, method_types) or tokens > MAX_FUSED_TOKENS or getattr(method, "runtime", None) is None:
            return original(self, x)
        if self.down_proj.bias is not None:
            raise ValueError("Fused SwiGLU path does not support a down_proj bias")
        gate_up, _ = self.gate_up_proj(x)
        y = linear_silu(gate_up.reshape(-1, 2 * method.k), method.handle, method.outputs, math)
        y = method.reduce(y)
        return y.reshape(*x.shape[:-1], method.outputs)

    mlp_class.forward = forward
    mlp_class._hygemm_producer_installed = True


def install(llama: bool = False):
    """Patch the MLP forward of Qwen2 (and Llama/Mistral when asked) (reference: producer.py:43-58,
    mistral_producer.py:5-27).  The reference limits the patch to its offline method; here every
    hybrid linear method qualifies."""
    from .quantization import MixedLinearMethod
    from vllm.model_executor.models.qwen2 import Qwen2MLP
    _patch(Qwen2MLP, MixedLinearMethod)
    if llama:
        from vllm.model_executor.models.llama import LlamaMLP
        _patch(LlamaMLP, MixedLinearMethod)
        try:
            from vllm.model_executor.models.mistral import MistralMLP
            _patch(MistralMLP, MixedLinearMethod)
        except ImportError:
            pass
