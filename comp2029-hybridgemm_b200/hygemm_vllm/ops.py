"""Opaque torch custom ops of the hybrid linear (no vLLM import needed).

`hygemm_vllm::linear` and `hygemm_vllm::linear_silu` keep the reference's
schemas (quantization.py:18-25, producer.py:27-40 of the reference): the layer
runtime is looked up by an integer handle in `_runtimes`, nothing is mutated,
and the fake implementations give shape/dtype for tracing.
"""
from __future__ import annotations

import torch

_runtimes: dict[int, object] = {}


def register_runtime(runtime) -> int:
    handle = id(runtime)
    _runtimes[handle] = runtime
    return handle


@torch.library.custom_op("hygemm_vllm::linear", mutates_args=())
def linear(x: torch.Tensor, handle: int, outputs: int) -> torch.Tensor:
    return _runtimes[handle](x)


@linear.register_fake
def _linear_fake(x, handle, outputs):
    return x.new_empty((x.shape[0], outputs))


@torch.library.custom_op("hygemm_vllm::linear_silu", mutates_args=())
def linear_silu(x: torch.Tensor, handle: int, outputs: int, math: int) -> torch.Tensor:
    from .producer import silu_pack
    runtime = _runtimes[handle]
    if hasattr(runtime, "profile_name") and torch.cuda.is_current_stream_capturing():
        # Same NVTX label as the reference's profiling hook (producer.py:31).
        label = (f"projection|{runtime.profile_name}|O={runtime.outputs}|K={runtime.k}"
                 f"|H={runtime.hi.numel()}|T={x.shape[0]}")
        with torch.cuda.nvtx.range(label):
            return runtime.run_packed(*silu_pack(x, math))
    return runtime.run_packed(*silu_pack(x, math))


@linear_silu.register_fake
def _linear_silu_fake(x, handle, outputs, math):
    return x.new_empty((x.shape[0], outputs))
