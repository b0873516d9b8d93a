"""The library loaded the way the reference's own Python loads it, and the MLP patch.

First half: a fresh ctypes handle on the shared object with ONLY the prototypes the reference declares
(integrations/vllm/hygemm_vllm/native.py:19-32 of the reference: hg_last_error, hg_scale_size, hg_pack,
hg_pack_mode, hg_create, hg_run, hg_destroy; IEEE half everywhere), driving the component check of
integrations/vllm/test_components.py:41-65: DualLinear-style pack of the weights, per-call activation pack
in every pack mode, two Problems, hg_create / hg_run, new pointers with the same shape, against the CPU
oracle with the reference's fp16 tolerance (atol = rtol = .002).

Second half: producer.install() (integrations/vllm/hygemm_vllm/producer.py:43-58, mistral_producer.py:12-27)
on a stand-in MLP class: the patched forward must route gate_up's output through the `linear_silu` op for up
to 128 tokens and fall back to the original forward above that or when down_proj is not a hybrid linear.
"""
import ctypes as C
import sys
import types

import numpy as np
import pytest
import torch

import oracle
from helpers import rel_frobenius, to_float
from hygemm_vllm import native

pytestmark = pytest.mark.gpu


class RefProblem(C.Structure):
    """The reference's ctypes struct, field for field (native.py:7-9 of the reference)."""
    _fields_ = [(n, C.c_int) for n in ["rows", "tokens", "k", "outputs"]] + [
        (n, C.c_void_p) for n in ["weight", "activation", "weight_scales", "activation_scales", "ids", "output"]]


def reference_style_library():
    lib = C.CDLL(str(native.library_path()))
    lib.hg_last_error.restype = C.c_char_p
    lib.hg_scale_size.argtypes = [C.c_int, C.c_int]
    lib.hg_scale_size.restype = C.c_int64
    lib.hg_pack.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3 + [C.c_void_p]
    assert hasattr(lib, "hg_pack_mode")
    lib.hg_pack_mode.argtypes = lib.hg_pack.argtypes + [C.c_int]
    lib.hg_create.argtypes = [C.c_int, C.c_int, C.POINTER(RefProblem), C.POINTER(RefProblem), C.c_void_p, C.POINTER(C.c_void_p)]
    lib.hg_run.argtypes = [C.c_void_p, C.POINTER(RefProblem), C.POINTER(RefProblem), C.c_void_p, C.c_int]
    lib.hg_destroy.argtypes = [C.c_void_p]
    return lib


def ref_pack(lib, x, fp4=False, mode=0):
    rows, k = x.shape
    q = torch.empty((rows, k // 2 if fp4 else k), dtype=torch.uint8, device=x.device)
    sf = torch.empty(lib.hg_scale_size(rows, k) if rows else 0, dtype=torch.uint8, device=x.device)
    if rows:
        params = (x.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, k, int(fp4), torch.cuda.current_stream().cuda_stream)
        status = lib.hg_pack_mode(*params, mode) if mode else lib.hg_pack(*params)
        assert status == 0, lib.hg_last_error()
    return q, sf


def test_components_through_the_reference_prototypes():
    lib = reference_style_library()
    torch.manual_seed(20261024)
    outputs = 257
    stream = torch.cuda.current_stream().cuda_stream
    for k in (256, 896):
        for high in (0, 26, outputs):
            w = (torch.randn(outputs, k, device="cuda") * .04).half()
            ids = torch.randperm(outputs, device="cuda")[:high]
            mask = torch.zeros(outputs, dtype=torch.bool, device="cuda")
            mask[ids] = True
            hi = torch.where(mask)[0].to(torch.int32)
            lo = torch.where(~mask)[0].to(torch.int32)
            w4, sf4 = ref_pack(lib, w[lo.long()].contiguous(), True)
            w8, sf8 = ref_pack(lib, w[hi.long()].contiguous(), False)
            torch.cuda.synchronize()
            ow4, osf4 = oracle.pack(w[lo.long()].cpu(), fp4=True, bf16=False)
            ow8, osf8 = oracle.pack(w[hi.long()].cpu(), fp4=False, bf16=False)
            assert np.array_equal(w4.cpu().numpy(), ow4) and np.array_equal(sf4.cpu().numpy(), osf4)
            assert np.array_equal(w8.cpu().numpy(), ow8) and np.array_equal(sf8.cpu().numpy(), osf8)
            for tokens in (1, 3, 17, 128):
                handle = C.c_void_p()
                for attempt, scale in enumerate((1.0, 0.5)):          # second round: new pointers, same shape
                    x = (torch.randn(tokens, k, device="cuda") * scale).half().contiguous()
                    packs = [ref_pack(lib, x, False, mode) for mode in (0, 1, 2, 3)]
                    for q_m, sf_m in packs[1:]:                        # every pack mode writes the same bytes
                        assert torch.equal(q_m, packs[0][0]) and torch.equal(sf_m, packs[0][1])
                    q, sf = packs[0]
                    y = torch.empty((tokens, outputs), device="cuda", dtype=torch.float16)
                    low = RefProblem(lo.numel(), tokens, k, outputs, w4.data_ptr(), q.data_ptr(), sf4.data_ptr(),
                                     sf.data_ptr(), lo.data_ptr(), y.data_ptr())
                    high_p = RefProblem(hi.numel(), tokens, k, outputs, w8.data_ptr(), q.data_ptr(), sf8.data_ptr(),
                                        sf.data_ptr(), hi.data_ptr(), y.data_ptr())
                    if attempt == 0:
                        assert lib.hg_create(0, 0, C.byref(low), C.byref(high_p), stream, C.byref(handle)) == 0, lib.hg_last_error()
                    assert lib.hg_run(handle, C.byref(low), C.byref(high_p), stream, 1) == 0, lib.hg_last_error()
                    torch.cuda.synchronize()
                    xq, xsf = oracle.pack(x.cpu(), fp4=False, bf16=False)
                    assert np.array_equal(q.cpu().numpy(), xq) and np.array_equal(sf.cpu().numpy(), xsf)
                    ref16, ref32 = oracle.hybrid_linear(ow4, osf4, lo.cpu().numpy(), ow8, osf8, hi.cpu().numpy(), xq, xsf,
                                                        outputs, bf16=False)
                    got = y.float().cpu().numpy()
                    np.testing.assert_allclose(got, to_float(ref16, torch.float16), atol=.002, rtol=.002)
                    assert rel_frobenius(got, ref32) <= 1e-2
                lib.hg_destroy(handle)


class _Linear(torch.nn.Module):
    """Stand-in for a vLLM linear layer: `forward` returns (output, bias) and carries `quant_method`."""

    def __init__(self, runtime=None, method=None, dense=None):
        super().__init__()
        self.runtime, self.quant_method, self.dense, self.bias = runtime, method, dense, None

    def forward(self, x):
        if self.runtime is not None:
            return self.runtime(x.reshape(-1, x.shape[-1]).contiguous()).reshape(*x.shape[:-1], -1), None
        return x @ self.dense.t(), None


def test_producer_install_routes_the_mlp_through_linear_silu(monkeypatch):
    pytest.importorskip("vllm")
    from hygemm_vllm import ops, producer, quantization

    class StandInMLP(torch.nn.Module):
        calls = {"original": 0}

        def __init__(self, gate_up, down):
            super().__init__()
            self.gate_up_proj, self.down_proj = gate_up, down

        def forward(self, x):
            StandInMLP.calls["original"] += 1
            gate_up, _ = self.gate_up_proj(x)
            half = gate_up.shape[-1] // 2
            act = torch.nn.functional.silu(gate_up[..., :half].float()).to(x.dtype)
            y, _ = self.down_proj((act.float() * gate_up[..., half:].float()).to(x.dtype))
            return y

    # install() imports the model classes from vLLM; give it the stand-in under that module path
    fake = types.ModuleType("vllm.model_executor.models.qwen2")
    fake.Qwen2MLP = StandInMLP
    monkeypatch.setitem(sys.modules, "vllm.model_executor.models.qwen2", fake)
    producer.install()
    assert StandInMLP._hygemm_producer_installed
    producer.install()                                                # idempotent

    torch.manual_seed(3)
    hidden, inter = 256, 384
    w_gu = (torch.randn(2 * inter, hidden) * .05).bfloat16().cuda()
    w_dn = (torch.randn(hidden, inter) * .05).bfloat16().cuda()
    gate_up_rt = native.DualLinear(w_gu, torch.randperm(2 * inter)[:77].cuda())
    down_rt = native.DualLinear(w_dn, torch.randperm(hidden)[:26].cuda())
    config = quantization.HyGEMMConfig.from_config({"selection": {}})
    method = quantization.MixedLinearMethod(config, "model.layers.0.mlp.down_proj")
    method.runtime, method.k, method.outputs = down_rt, inter, hidden
    method.handle = ops.register_runtime(down_rt)
    mlp = StandInMLP(_Linear(runtime=gate_up_rt), _Linear(runtime=down_rt, method=method))

    x = torch.randn(2, 5, hidden, device="cuda", dtype=torch.bfloat16)
    before = dict(down_rt.calls)
    y = mlp(x)                                                         # 10 tokens: the fused producer path
    assert StandInMLP.calls["original"] == 0 and y.shape == (2, 5, hidden)
    assert down_rt.calls.get(10, 0) == before.get(10, 0) + 1
    gate_up, _ = mlp.gate_up_proj(x)
    q, sf = producer.silu_pack(gate_up.reshape(-1, 2 * inter), 0)
    want = down_rt.run_packed(q, sf).reshape(2, 5, hidden)
    assert torch.equal(y, want)                                        # same launches, same bits
    # the op itself, by its registered name
    again = torch.ops.hygemm_vllm.linear_silu(gate_up.reshape(-1, 2 * inter), method.handle, hidden, 0)
    assert torch.equal(again.reshape(2, 5, hidden), want)
    # against the oracle chain
    oq, osf = oracle.silu_pack(gate_up.reshape(-1, 2 * inter).cpu(), bf16=True)
    _, ref32 = oracle.hybrid_linear(down_rt.w4.cpu().numpy(), down_rt.sf4.cpu().numpy(), down_rt.lo.cpu().numpy(),
                                    down_rt.w8.cpu().numpy(), down_rt.sf8.cpu().numpy(), down_rt.hi.cpu().numpy(),
                                    oq, osf, hidden, bf16=True)
    assert rel_frobenius(y.float().cpu().numpy().reshape(-1, hidden), ref32) <= 1e-2

    big = torch.randn(129, hidden, device="cuda", dtype=torch.bfloat16)   # above 128 tokens: the original forward
    mlp(big)
    assert StandInMLP.calls["original"] == 1
    plain = StandInMLP(_Linear(runtime=gate_up_rt), _Linear(dense=w_dn))  # down_proj is not a hybrid linear
    plain(x)
    assert StandInMLP.calls["original"] == 2
    mlp.down_proj.bias = torch.zeros(hidden, device="cuda")
    with pytest.raises(ValueError, match="bias"):
        mlp(x)
    gate_up_rt.close()
    down_rt.close()
