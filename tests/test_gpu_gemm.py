"""Hybrid GEMM through the C ABI: bit-exact on the reference's exact-representable cases,
within tolerance of the CPU oracle on random data, deterministic, guard bands intact."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import bits, dev, make_inputs, quantised_case, rel_frobenius, run_gemm, to_float
from hygemm_vllm import native

pytestmark = pytest.mark.gpu

# (outputs, tokens, k, high, mapping): scripts/run_output_channel_bench.py:66-75 and
# src/kernel/output_channel_fused_bench.cu stress shape of the reference.
EXACT = [(257, 7, 256, 0, "random"), (257, 7, 256, 1, "random"), (257, 7, 256, 26, "random"),
         (257, 7, 256, 128, "random"), (257, 7, 256, 256, "random"), (257, 7, 256, 257, "random"),
         (511, 33, 384, 73, "interleaved"), (129, 1, 128, 17, "random"), (255, 17, 128, 51, "contiguous"),
         (4096, 128, 1024, 2048, "random"), (2049, 130, 384, 300, "interleaved")]
SCHEDULES = {"auto": 0, "data_parallel": 1, "split_k": 2, "stream_k": 3}


def expected_work(case, schedule):
    """Closed-form totals the kernel's audit counters must reproduce."""
    lib = native.library()
    header = (C.c_int * 12)()
    props = torch.cuda.get_device_properties(0)
    native.check(lib.hg_plan(case["lo"].size, case["hi"].size, case["tokens"], case["k"],
                             props.multi_processor_count, schedule, header, None, 0))
    tiles = -(-case["lo"].size // 128) + -(-case["hi"].size // 128)
    return tiles * header[3] * (case["k"] // 128), header[9]


@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_exact_cases_bit_exact(schedule, dtype):
    for outputs, tokens, k, high, mapping in EXACT:
        case = oracle.exact_case(outputs, tokens, k, high, mapping, bf16=dtype == torch.bfloat16)
        got, guards, status = run_gemm(case, dtype, SCHEDULES[schedule])
        tag = (outputs, tokens, k, high, mapping, schedule)
        assert status[0] == 0, (tag, status)
        assert guards, tag
        blocks, units = expected_work(case, SCHEDULES[schedule])
        assert (status[1], status[2]) == (blocks, units), (tag, status, blocks, units)
        assert np.array_equal(got, case["expected"]), (tag, int((got != case["expected"]).sum()))


@pytest.mark.parametrize("policy", [4, 5, 6])
def test_simt_pair_policies_bit_exact(policy):
    for outputs, tokens, k, high, mapping in EXACT[:9]:
        case = oracle.exact_case(outputs, tokens, k, high, mapping)
        got, guards, _ = run_gemm(case, torch.bfloat16, 0, policy)
        assert guards and np.array_equal(got, case["expected"]), (outputs, tokens, k, high, policy)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_component_matrix_vs_oracle(dtype):
    """Matrix of integrations/vllm/test_components.py:41-65 of the reference: DualLinear(x) against the
    dequantise-and-matmul oracle, then new pointers with the same shape (stale-descriptor detector)."""
    torch.manual_seed(20261024)
    outputs = 257
    for k in (256, 896):
        for high in (0, 26, outputs):
            w = (torch.randn(outputs, k) * .04).to(dtype)
            ids = torch.randperm(outputs)[:high]
            layer = native.DualLinear(w.cuda(), ids.cuda())
            lo, hi = layer.lo.cpu().numpy(), layer.hi.cpu().numpy()
            want_lo, want_hi = oracle.partition(outputs, ids.numpy())
            assert np.array_equal(lo, want_lo) and np.array_equal(hi, want_hi)           # scatter indices bit-exact
            w4, sf4 = oracle.pack(w[torch.from_numpy(lo).long()], fp4=True, bf16=dtype == torch.bfloat16)
            w8, sf8 = oracle.pack(w[torch.from_numpy(hi).long()], fp4=False, bf16=dtype == torch.bfloat16)
            assert np.array_equal(layer.w4.cpu().numpy(), w4) and np.array_equal(layer.sf4.cpu().numpy(), sf4)
            assert np.array_equal(layer.w8.cpu().numpy(), w8) and np.array_equal(layer.sf8.cpu().numpy(), sf8)
            for tokens in (1, 3, 17, 128):
                for scale in (1.0, 0.5):
                    x = (torch.randn(tokens, k) * scale).to(dtype)
                    y = layer(x.cuda().contiguous())
                    xq, xsf = oracle.pack(x, bf16=dtype == torch.bfloat16)
                    ref16, ref32 = oracle.hybrid_linear(w4, sf4, lo, w8, sf8, hi, xq, xsf, outputs, bf16=dtype == torch.bfloat16)
                    got = y.float().cpu().numpy()
                    assert rel_frobenius(got, ref32) <= 1e-2, (k, high, tokens)      # bar of this build (bf16 out)
                    ref = to_float(ref16, dtype)
                    tol = (.002, .002) if dtype == torch.float16 else (.02, .02)       # fp16 tolerance of the reference
                    np.testing.assert_allclose(got, ref, atol=tol[0], rtol=tol[1])
            assert layer.status()[0] == 0
            layer.close()


def test_graph_replay_with_changed_input():
    """integrations/vllm/test_components.py:67-76 of the reference."""
    torch.manual_seed(5)
    outputs, k = 257, 896
    w = (torch.randn(outputs, k) * .04).bfloat16().cuda()
    layer = native.DualLinear(w, torch.randperm(outputs)[:26].cuda())
    x = torch.randn(3, k, device="cuda", dtype=torch.bfloat16)
    layer(x)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = layer(x)
    for seed in (111, 112):
        torch.manual_seed(seed)
        x.copy_(torch.randn_like(x))
        graph.replay()
        torch.cuda.synchronize()
        eager = layer(x)
        assert torch.equal(y, eager)
        xq, xsf = oracle.pack(x.cpu())
        _, ref = oracle.hybrid_linear(layer.w4.cpu().numpy(), layer.sf4.cpu().numpy(), layer.lo.cpu().numpy(),
                                      layer.w8.cpu().numpy(), layer.sf8.cpu().numpy(), layer.hi.cpu().numpy(),
                                      xq, xsf, outputs)
        assert rel_frobenius(y.float().cpu().numpy(), ref) <= 1e-2
    # an un-warmed shape must be refused while capturing
    x5 = torch.randn(5, k, device="cuda", dtype=torch.bfloat16)
    q5, sf5 = native.pack(x5)
    g2 = torch.cuda.CUDAGraph()
    with pytest.raises(RuntimeError, match="must be warmed"):
        with torch.cuda.graph(g2):
            layer.run_packed(q5, sf5)
    layer.close()


def test_rebind_to_other_shape_is_rejected():
    case = oracle.exact_case(257, 7, 256, 26, "random")
    lib = native.library()
    d = {n: dev(case[n]) for n in ("w4", "sf4", "lo", "w8", "sf8", "hi", "xq", "xsf")}
    y = torch.zeros(7 * 257, dtype=torch.int16, device="cuda")
    low = native.Problem(d["lo"].numel(), 7, 256, 257, d["w4"].data_ptr(), d["xq"].data_ptr(), d["sf4"].data_ptr(),
                         d["xsf"].data_ptr(), d["lo"].data_ptr(), y.data_ptr())
    high = native.Problem(d["hi"].numel(), 7, 256, 257, d["w8"].data_ptr(), d["xq"].data_ptr(), d["sf8"].data_ptr(),
                          d["xsf"].data_ptr(), d["hi"].data_ptr(), y.data_ptr())
    handle = C.c_void_p()
    native.check(lib.hg_create_dtype(0, 0, C.byref(low), C.byref(high), None, 1, C.byref(handle)))
    low.tokens = 6
    assert lib.hg_run(handle, C.byref(low), C.byref(high), None, 0) == -1
    assert b"shape" in lib.hg_last_error()
    info = (C.c_int * 20)()
    native.check(lib.hg_info(handle, info))
    assert info[1] == 128 and info[3] == 256 and info[11] == 128 and info[8] == 0 and info[18] == 1
    lib.hg_destroy(handle)
    bad = native.Problem(0, 7, 256, 257, None, None, None, None, None, None)
    assert lib.hg_create_dtype(0, 0, C.byref(bad), C.byref(bad), None, 1, C.byref(handle)) == -1


SHAPES_7B = {"qkv": (3584, 4608, 512), "o_proj": (3584, 3584, 384), "gate_up": (3584, 37888, 3840),
             "down": (18944, 3584, 384)}


@pytest.mark.parametrize("name", list(SHAPES_7B))
def test_7b_shapes_vs_oracle_and_determinism(name):
    """Full Qwen2.5-7B layer shapes: M=16 against the CPU oracle, every schedule bit-identical run to run,
    tensor-core and SIMT kernels agreeing, M=1/128 against the SIMT kernel."""
    k, outputs, high = SHAPES_7B[name]
    case = quantised_case(16, k, outputs, high)
    ref = case["expected_f32"]
    got, guards, status = run_gemm(case, torch.bfloat16, 0)
    assert status[0] == 0 and guards
    assert rel_frobenius(to_float(got, torch.bfloat16), ref) <= 1e-2
    mism = (got != case["expected"]).mean()
    assert mism < 0.02, mism                      # same fp32 products, different summation order
    again, _, _ = run_gemm(case, torch.bfloat16, 0, runs=3)
    assert np.array_equal(got, again)
    for schedule in (1, 2, 3):
        other, _, st = run_gemm(case, torch.bfloat16, schedule)
        assert st[0] == 0
        assert rel_frobenius(to_float(other, torch.bfloat16), ref) <= 1e-2
    simt, _, _ = run_gemm(case, torch.bfloat16, 0, policy=6)
    assert rel_frobenius(to_float(simt, torch.bfloat16), ref) <= 1e-2
    for tokens in (1, 128):
        big = quantised_case_light(tokens, k, outputs, high)
        a, g1, s1 = run_gemm(big, torch.bfloat16, 0)
        b, g2, _ = run_gemm(big, torch.bfloat16, 0, policy=6)
        assert s1[0] == 0 and g1 and g2
        assert not np.any(a == 0xFFFF)
        assert rel_frobenius(to_float(a, torch.bfloat16), to_float(b, torch.bfloat16).astype(np.float64)) <= 5e-3


def quantised_case_light(tokens, k, outputs, high):
    """Operands quantised on the device (already checked bit-exact against the oracle elsewhere)."""
    x, w, ids = make_inputs(tokens, k, outputs, high)
    layer = native.DualLinear(w.cuda(), ids.cuda())
    xq, xsf = native.pack(x.cuda())
    case = dict(w4=layer.w4.cpu().numpy(), sf4=layer.sf4.cpu().numpy(), lo=layer.lo.cpu().numpy(),
                w8=layer.w8.cpu().numpy(), sf8=layer.sf8.cpu().numpy(), hi=layer.hi.cpu().numpy(),
                xq=xq.cpu().numpy(), xsf=xsf.cpu().numpy(), outputs=outputs, tokens=tokens, k=k)
    layer.close()
    return case


def test_config0_reference_cpu_case():
    """M=8, K=896, N=4864, H=486: the reference's CPU-runnable configuration."""
    case = quantised_case(8, 896, 4864, 486)
    got, guards, status = run_gemm(case, torch.bfloat16, 0)
    assert status[0] == 0 and guards
    assert rel_frobenius(to_float(got, torch.bfloat16), case["expected_f32"]) <= 1e-2
    assert (got != case["expected"]).mean() < 0.02


def test_linearity_property_full_size():
    """Scaling the activations by 2 (exact in MX: only the E8M0 bytes move) doubles the output bit-exactly."""
    k, outputs, high = SHAPES_7B["down"]
    case = quantised_case_light(4, k, outputs, high)
    a, _, _ = run_gemm(case, torch.bfloat16, 0)
    doubled = dict(case)
    sf = case["xsf"].copy()
    idx = oracle.scale_indices(4, k)
    sf[idx] += 1
    doubled["xsf"] = sf
    b, _, _ = run_gemm(doubled, torch.bfloat16, 0)
    fa, fb = to_float(a, torch.bfloat16), to_float(b, torch.bfloat16)
    assert np.array_equal(fb, 2 * fa)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_quantisation_launch_equals_pack_then_run(dtype):
    """`hg_run_x` (decode sizes: activations quantised inside the GEMM launch) must give the bytes of
    `hg_pack` followed by `hg_run`, for odd K128 counts, both partitions empty or not, and outliers."""
    torch.manual_seed(11)
    for outputs, k, high in [(257, 256, 26), (300, 896, 0), (384, 896, 384), (4608, 3584, 512), (3584, 18944, 384)]:
        w = (torch.randn(outputs, k) * .04).to(dtype).cuda()
        layer = native.DualLinear(w, torch.randperm(outputs)[:high].cuda())
        for tokens in (1, 3, 16):
            x = torch.randn(tokens, k)
            x[:, ::97] *= 20
            x[0, :64] = 0
            x = x.to(dtype).cuda()
            fused = layer(x)                                   # hg_run_x
            q, sf = native.pack(x)
            two_step = layer.run_packed(q, sf)                 # hg_pack + hg_run
            assert torch.equal(fused.view(torch.int16), two_step.view(torch.int16)), (outputs, k, high, tokens)
        assert layer.status()[0] == 0
        layer.close()
    big = torch.randn(17, 256).to(dtype).cuda()
    layer = native.DualLinear((torch.randn(257, 256) * .04).to(dtype).cuda(), torch.arange(26).cuda())
    q, sf = native.pack(big)
    assert torch.equal(layer(big), layer.run_packed(q, sf))   # 17 tokens: two launches again
    layer.close()
