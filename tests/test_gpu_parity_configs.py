"""Parity at the sizes the benchmark configurations list, through the C ABI, against the CPU oracle.

* config 1: every Qwen2.5-7B layer shape at every listed token count (the oracle finishes each in seconds),
  so the stream-K fix-up, the 64-token tile pairs and the 128-token tile all meet the oracle at full size;
* config 2: gate_up output -> SwiGLU + MXFP8 quantisation -> down_proj as ONE chain;
* prefill buckets of the reference's plans (integrations/vllm/formal/tune.py:20): 256, 512, 2048 tokens;
* the reference's activation extremes (integrations/vllm/performance/check_extremes.py:14-22);
* the quantiser matrix of optimization/check_pack.py:17-35 / performance/check.py:19-44 at K = 18944 and
  2048 rows, with a CUDA-graph replay over a scale buffer refilled with 0xff;
* the single-kernel entry points hg_fused_* against hg_run, bit for bit (performance/check_fused.py:25).

Tolerance for GEMM outputs: relative Frobenius error <= 1e-2 against the fp32-accumulated dequantised
reference (bf16 output); codes, scales and indices bit-exact.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from helpers import bits, dev, make_inputs, rel_frobenius, run_gemm, to_float
from hygemm_vllm import native, producer

pytestmark = pytest.mark.gpu

SHAPES_7B = {"qkv": (3584, 4608, 512), "o_proj": (3584, 3584, 384), "gate_up": (3584, 37888, 3840),
             "down": (18944, 3584, 384)}
TOKENS = {"qkv": (1, 2, 4, 8, 16, 32, 64, 128), "o_proj": (1, 2, 4, 8, 16, 32, 64, 128),
          "down": (1, 2, 4, 8, 16, 32, 64, 128), "gate_up": (1, 16, 128)}


def packed_layer(k, outputs, high, dtype=torch.bfloat16, seed=20261024):
    """Weights of one layer quantised by the oracle (once per shape)."""
    _, w, ids = make_inputs(1, k, outputs, high, dtype, seed)
    bf16 = dtype == torch.bfloat16
    lo, hi = oracle.partition(outputs, ids.numpy())
    w4, sf4 = oracle.pack(w[torch.from_numpy(lo).long()], fp4=True, bf16=bf16)
    w8, sf8 = oracle.pack(w[torch.from_numpy(hi).long()], fp4=False, bf16=bf16)
    return dict(w4=w4, sf4=sf4, lo=lo, w8=w8, sf8=sf8, hi=hi, outputs=outputs, k=k)


def with_activations(layer, x, dtype=torch.bfloat16):
    bf16 = dtype == torch.bfloat16
    xq, xsf = oracle.pack(x, fp4=False, bf16=bf16)
    y16, y32 = oracle.hybrid_linear(layer["w4"], layer["sf4"], layer["lo"], layer["w8"], layer["sf8"], layer["hi"],
                                    xq, xsf, layer["outputs"], bf16=bf16)
    return dict(layer, xq=xq, xsf=xsf, tokens=x.shape[0], expected=y16, expected_f32=y32)


@pytest.mark.parametrize("name", list(SHAPES_7B))
def test_config1_every_token_count_vs_oracle(name):
    k, outputs, high = SHAPES_7B[name]
    layer = packed_layer(k, outputs, high)
    for tokens in TOKENS[name]:
        x, _, _ = make_inputs(tokens, k, 8, 1, seed=1000 + tokens)
        case = with_activations(layer, x)
        got, guards, status = run_gemm(case, torch.bfloat16, 0)
        assert status[0] == 0 and guards, (name, tokens, status)
        assert not np.any(got == 0xFFFF), (name, tokens)                       # every output written
        err = rel_frobenius(to_float(got, torch.bfloat16), case["expected_f32"])
        assert err <= 1e-2, (name, tokens, err)
        # same fp32 products in another summation order: the 16-bit results differ in rare last bits only
        assert (got != case["expected"]).mean() < 0.02, (name, tokens)


@pytest.mark.parametrize("tokens", [1, 16, 128])
def test_config2_swiglu_quant_down_chain_vs_oracle(tokens):
    """bf16 gate_up output ~N(0,2) -> silu(gate)*up -> E4M3 codes + E8M0 scales -> hybrid down_proj."""
    k, outputs, high = SHAPES_7B["down"]
    layer = packed_layer(k, outputs, high)
    g = torch.Generator().manual_seed(77 + tokens)
    gate_up = (torch.randn(tokens, 2 * k, generator=g) * 2.0).to(torch.bfloat16)
    # device chain through the library
    q, sf, product = producer.silu_pack(gate_up.cuda(), 0, debug=True)
    # (i) the quantisation of the device's own 16-bit product is bit-exact
    want_q, want_sf = oracle.pack(product.cpu(), fp4=False, bf16=True)
    assert np.array_equal(q.cpu().numpy(), want_q) and np.array_equal(sf.cpu().numpy(), want_sf)
    # (ii) the product itself against the oracle's: expf differs by at most one ulp between the libraries,
    #      so a few 16-bit neighbours are allowed, nothing else
    oq, osf, oproduct = oracle.silu_pack(gate_up, bf16=True, debug=True)
    got_bits = bits(product)
    differ = got_bits != oproduct
    assert differ.mean() < 1e-3
    assert np.all(np.abs(got_bits[differ].astype(np.int32) - oproduct[differ].astype(np.int32)) <= 1)
    # (iii) the GEMM on the device's codes against the oracle GEMM on the same codes ...
    case = dict(layer, xq=q.cpu().numpy(), xsf=sf.cpu().numpy(), tokens=tokens)
    y16, y32 = oracle.hybrid_linear(layer["w4"], layer["sf4"], layer["lo"], layer["w8"], layer["sf8"], layer["hi"],
                                    case["xq"], case["xsf"], outputs, bf16=True)
    got, guards, status = run_gemm(case, torch.bfloat16, 0)
    assert status[0] == 0 and guards
    assert rel_frobenius(to_float(got, torch.bfloat16), y32) <= 1e-2
    # ... and the whole chain against the oracle's whole chain (its own product, codes and GEMM)
    _, chain32 = oracle.hybrid_linear(layer["w4"], layer["sf4"], layer["lo"], layer["w8"], layer["sf8"], layer["hi"],
                                      oq, osf, outputs, bf16=True)
    assert rel_frobenius(to_float(got, torch.bfloat16), chain32) <= 1e-2


@pytest.mark.parametrize("tokens", [256, 512, 2048])
def test_prefill_buckets_exact_and_vs_oracle(tokens):
    """Token counts of the reference's prefill plans run as rows of 128-token tiles."""
    case = oracle.exact_case(1024, tokens, 512, 200, "interleaved")
    for schedule in (0, 1, 3):
        got, guards, status = run_gemm(case, torch.bfloat16, schedule)
        assert status[0] == 0 and guards
        assert np.array_equal(got, case["expected"]), (tokens, schedule, int((got != case["expected"]).sum()))
    if tokens == 256:
        for name in ("qkv", "down"):
            k, outputs, high = SHAPES_7B[name]
            layer = packed_layer(k, outputs, high)
            x, _, _ = make_inputs(tokens, k, 8, 1, seed=5)
            full = with_activations(layer, x)
            got, guards, status = run_gemm(full, torch.bfloat16, 0)
            assert status[0] == 0 and guards
            assert rel_frobenius(to_float(got, torch.bfloat16), full["expected_f32"]) <= 1e-2, name


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_activation_extremes(dtype):
    """integrations/vllm/performance/check_extremes.py:14-22 of the reference: tiny weights, activations scaled
    by 0, 2^-24, 2^-14, 1 and 32752 (the largest scale at which uniform(-1,1) stays finite in fp16), against the
    dequantise-and-matmul oracle with the reference's tolerance for that check (atol .01, rtol .003 in fp16;
    relative Frobenius 1e-2 for bf16 output)."""
    torch.manual_seed(20261026)
    outputs, k = 129, 896
    w = (torch.randn(outputs, k) * 1e-4).to(dtype)
    ids = torch.randperm(outputs)[:19]
    layer = native.DualLinear(w.cuda(), ids.cuda())
    bf16 = dtype == torch.bfloat16
    w4, sf4, w8, sf8 = (t.cpu().numpy() for t in (layer.w4, layer.sf4, layer.w8, layer.sf8))
    lo, hi = layer.lo.cpu().numpy(), layer.hi.cpu().numpy()
    for scale in (0.0, 2.0 ** -24, 2.0 ** -14, 1.0, 32752.0):
        x = ((torch.rand(3, k) * 2 - 1) * scale).to(dtype)
        for y in (layer(x.cuda()), layer.run_packed(*native.pack(x.cuda()))):     # fused and two-launch paths
            xq, xsf = oracle.pack(x, fp4=False, bf16=bf16)
            ref16, ref32 = oracle.hybrid_linear(w4, sf4, lo, w8, sf8, hi, xq, xsf, outputs, bf16=bf16)
            got = y.float().cpu().numpy()
            assert np.isfinite(got).all(), scale
            if scale == 0.0:
                assert not got.any()
            if bf16:
                assert rel_frobenius(got, ref32) <= 1e-2 or not ref32.any(), scale
            else:
                np.testing.assert_allclose(got, to_float(ref16, dtype), atol=.01, rtol=.003)
    assert layer.status()[0] == 0
    layer.close()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_pack_matrix_large_k_many_rows_and_graph_replay(dtype):
    """The part of the reference's quantiser matrix that the basic test leaves out: K = 18944, 2048 rows, scales
    0 / .125 / 2 / 4096, and a CUDA-graph replay after the scale buffer was filled with 0xff (every padding byte
    must be rewritten by the replayed launch), codes and all scale bytes equal to the oracle's."""
    bf16 = dtype == torch.bfloat16
    for rows, k in [(1, 18944), (17, 18944), (129, 18944), (2048, 128), (2048, 896), (2048, 3584), (257, 3584)]:
        g = torch.Generator().manual_seed(rows + k)
        base = torch.randn(rows, k, generator=g)
        for scale in (0.0, 0.125, 2.0, 4096.0):
            x = (base * scale).to(dtype)
            for fp4 in (False, True):
                q, sf = native.pack(x.cuda(), fp4)
                want_q, want_sf = oracle.pack(x, fp4=fp4, bf16=bf16)
                assert np.array_equal(q.cpu().numpy(), want_q), (rows, k, scale, fp4)
                assert np.array_equal(sf.cpu().numpy(), want_sf), (rows, k, scale, fp4)
        if rows in (1, 17, 129, 257):
            xd = (base * 0.5).to(dtype).cuda()
            native.pack(xd)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                q, sf = native.pack(xd)
            for scale in (0.0, 0.25, 32.0):
                fresh = (torch.randn(rows, k, generator=g) * scale).to(dtype)
                xd.copy_(fresh)
                sf.fill_(255)
                graph.replay()
                torch.cuda.synchronize()
                want_q, want_sf = oracle.pack(fresh, fp4=False, bf16=bf16)
                assert np.array_equal(q.cpu().numpy(), want_q) and np.array_equal(sf.cpu().numpy(), want_sf), (rows, k, scale)


def test_fused_entry_points_equal_hg_run_bitwise():
    """integrations/vllm/performance/check_fused.py:16-35 of the reference: the single-kernel path
    (hg_fused_create / update / run / info) is bitwise equal to the dual path, before and after rebinding."""
    lib = native.library()
    stream = torch.cuda.current_stream().cuda_stream
    for outputs, k, high, tokens in [(257, 384, 26, 17), (257, 896, 0, 3), (257, 128, 257, 1), (4608, 3584, 512, 8)]:
        case = oracle.exact_case(outputs, tokens, k, high, "random") if outputs == 257 else None
        if case is None:
            x, _, _ = make_inputs(tokens, k, 8, 1, seed=9)
            case = with_activations(packed_layer(k, outputs, high), x)
        want, guards, status = run_gemm(case, torch.bfloat16, 0)
        assert guards and status[0] == 0
        d = {n: dev(case[n]) for n in ("w4", "sf4", "lo", "w8", "sf8", "hi", "xq", "xsf")}

        def ptr(t):
            return t.data_ptr() if t.numel() else None

        def problems(y):
            low = native.Problem(d["lo"].numel(), tokens, k, outputs, ptr(d["w4"]), d["xq"].data_ptr(), ptr(d["sf4"]),
                                 d["xsf"].data_ptr(), ptr(d["lo"]), y.data_ptr())
            hi = native.Problem(d["hi"].numel(), tokens, k, outputs, ptr(d["w8"]), d["xq"].data_ptr(), ptr(d["sf8"]),
                                d["xsf"].data_ptr(), ptr(d["hi"]), y.data_ptr())
            return low, hi
        y1 = torch.full((tokens, outputs), -1, dtype=torch.int16, device="cuda")
        low, hi = problems(y1)
        handle = C.c_void_p()
        assert lib.hg_fused_create_dtype(0, C.byref(low), C.byref(hi), stream, 1, C.byref(handle)) == 0, lib.hg_fused_error()
        assert lib.hg_fused_run(handle, stream) == 0
        torch.cuda.synchronize()
        assert np.array_equal(y1.cpu().numpy().view(np.uint16), want)
        y2 = torch.full((tokens, outputs), -1, dtype=torch.int16, device="cuda")      # new output pointer
        low2, hi2 = problems(y2)
        assert lib.hg_fused_update(handle, C.byref(low2), C.byref(hi2)) == 0
        assert lib.hg_fused_run(handle, stream) == 0
        torch.cuda.synchronize()
        assert np.array_equal(y2.cpu().numpy().view(np.uint16), want)
        info = (C.c_int * 11)()
        assert lib.hg_fused_info(handle, info) == 0
        tiles = -(-d["lo"].numel() // 128) + -(-d["hi"].numel() // 128)
        assert info[1] == 128 and info[10] == tiles * 128 and info[9] - info[8] == 16384
        low2.tokens += 1
        assert lib.hg_fused_update(handle, C.byref(low2), C.byref(hi2)) == -1 and b"rebind" in lib.hg_fused_error()
        lib.hg_fused_destroy(handle)
