"""The CPU oracle against the golden vectors taken from the reference (no GPU)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle

ALL16 = np.arange(65536, dtype=np.uint16)


def _vec(fn, values, restype=np.int64):
    return np.array([fn(C.c_float(float(v))) for v in values], dtype=restype)


def test_float16_helpers_match_torch():
    L = oracle.lib()
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(20000) * 10 ** rng.uniform(-9, 5, 20000),
                        [0., -0., 65504., 65519.9, 65520., 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5]]).astype(np.float32)
    half = torch.from_numpy(x).half().view(torch.int16).numpy().view(np.uint16)
    bf = torch.from_numpy(x).bfloat16().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(_vec(L.hgo_float_to_half, x, np.uint16), half)
    assert np.array_equal(_vec(L.hgo_float_to_bf16, x, np.uint16), bf)
    back = np.array([L.hgo_half_to_float(int(h)) for h in ALL16[::7]], dtype=np.float32)
    want = ALL16[::7].view(np.float16).astype(np.float32)
    assert np.array_equal(back.view(np.uint32)[np.isfinite(want)], want.view(np.uint32)[np.isfinite(want)])


@pytest.mark.parametrize("src", ["half", "bf16"])
def test_element_codecs_match_cutlass_for_every_16bit_input(golden, src):
    """E4M3 / E2M1 conversion == cutlass::float_e4m3_t / float_e2m1_t (host) on all 65536 inputs."""
    L = oracle.lib()
    g = golden("cutlass_codecs.npz")
    vals = ALL16.view(np.float16).astype(np.float32) if src == "half" else (ALL16.astype(np.uint32) << 16).view(np.float32)
    vals = np.where(np.isfinite(vals), vals, 0).astype(np.float32)
    assert np.array_equal(_vec(L.hgo_e4m3_from_float, vals, np.uint8), g[f"e4m3_from_{src}"])
    assert np.array_equal(_vec(L.hgo_e2m1_from_float, vals, np.uint8), g[f"e2m1_from_{src}"])


def test_e4m3_matches_torch_float8_cast():
    L = oracle.lib()
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(50000) * 10 ** rng.uniform(-4, 2.6, 50000)).astype(np.float32)
    x = x[np.abs(x) <= 448]
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(_vec(L.hgo_e4m3_from_float, x, np.uint8), want)
    codes = np.arange(256, dtype=np.uint8)
    dec = np.array([L.hgo_e4m3_to_float(int(c)) for c in codes], dtype=np.float32)
    ref = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    ok = ~np.isnan(ref)
    assert np.array_equal(dec[ok].view(np.uint32), ref[ok].view(np.uint32))


@pytest.mark.parametrize("fp4", [0, 1])
def test_exponent_rule_literal_equals_closed_form_exhaustively(fp4):
    """ceil(log2(amax/max)) in fp32 == smallest e with amax*2^-e <= max, all fp16 and bf16 amax."""
    L = oracle.lib()
    for vals in (ALL16.view(np.float16).astype(np.float32), (ALL16.astype(np.uint32) << 16).view(np.float32)):
        vals = vals[np.isfinite(vals) & (vals > 0)]
        for v in vals[:: 1 if vals.size < 40000 else 1]:
            a = L.hgo_exponent_literal(C.c_float(float(v)), fp4)
            b = L.hgo_exponent_exact(C.c_float(float(v)), fp4)
            assert a == b, (float(v), a, b)


def test_decode_matches_reference_decode_mx(golden):
    g = golden("decode_mx.npz")
    for rows, k in [(3, 128), (130, 256), (33, 896)]:
        for fp4 in (True, False):
            tag = f"r{rows}_k{k}_{'fp4' if fp4 else 'fp8'}"
            got = oracle.decode(g[tag + "_q"], g[tag + "_sf"], k, fp4)
            assert np.array_equal(got, g[tag + "_out"]), tag


def test_scale_layout_matches_reference(golden):
    g = golden("scale_indices.npz")
    L = oracle.lib()
    for key in g.files:
        rows, k = (int(s[1:]) for s in key.split("_"))
        want = g[key]
        assert np.array_equal(oracle.scale_indices(rows, k), want)
        for r, c in [(0, 0), (rows - 1, k // 32 - 1), (rows // 2, 1)]:
            assert L.hgo_scale_index(r, c, k) == want[r, c]
        assert oracle.scale_size(rows, k) == -(-rows // 128) * (k // 128) * 512
        assert want.max() < oracle.scale_size(rows, k)


def test_fp4_codes_match_reference_codes_rne(golden):
    g = golden("codes_rne.npz")
    L = oracle.lib()
    values = g["values"]
    got = _vec(L.hgo_e2m1_from_float, values.ravel(), np.uint8).reshape(values.shape)
    assert np.array_equal(got, g["codes"])
    packed = (got[:, 0::2] | (got[:, 1::2] << 4)).astype(np.uint8)
    assert np.array_equal(packed, g["packed"])
    # decode_logical == oracle.decode through the physical layout
    rows = values.shape[0]
    sf = np.full(oracle.scale_size(rows, 128), 127, dtype=np.uint8)
    wide = np.zeros((rows, 64), dtype=np.uint8)
    wide[:, :32] = packed
    idx = oracle.scale_indices(rows, 128)
    sf[idx[:, :2]] = g["logical"]
    dec = oracle.decode(wide, sf, 128, True)[:, :64]
    assert np.array_equal(dec, g["decoded"])


def test_pack_agrees_with_golden_quantised_operands(golden):
    """oracle.pack is deterministic and reproduces the operands stored with the reference outputs."""
    g = golden("reference_linear.npz")
    tags = sorted({f.split("__")[0] for f in g.files})
    for tag in tags:
        w = torch.from_numpy(g[tag + "__w"].view(np.int16)).view(torch.bfloat16)
        x = torch.from_numpy(g[tag + "__x"].view(np.int16)).view(torch.bfloat16)
        lo, hi = g[tag + "__lo"], g[tag + "__hi"]
        w4, sf4 = oracle.pack(w[torch.from_numpy(lo).long()], fp4=True)
        w8, sf8 = oracle.pack(w[torch.from_numpy(hi).long()], fp4=False)
        xq, xsf = oracle.pack(x)
        for name, val in dict(w4=w4, sf4=sf4, w8=w8, sf8=sf8, xq=xq, xsf=xsf).items():
            assert np.array_equal(val, g[f"{tag}__{name}"]), (tag, name)


def test_hybrid_linear_matches_reference_dequant_matmul(golden):
    g = golden("reference_linear.npz")
    tags = sorted({f.split("__")[0] for f in g.files})
    assert len(tags) == 4
    for tag in tags:
        outputs = int(tag.split("_")[0][1:])
        a = {n: g[f"{tag}__{n}"] for n in ["w4", "sf4", "lo", "w8", "sf8", "hi", "xq", "xsf", "y", "y_bf16", "y_half"]}
        y16, yf = oracle.hybrid_linear(a["w4"], a["sf4"], a["lo"], a["w8"], a["sf8"], a["hi"], a["xq"], a["xsf"], outputs, bf16=True)
        # fp32 accumulation order differs (sequential vs blocked BLAS): relative Frobenius <= 1e-6
        err = np.linalg.norm(yf - a["y"]) / np.linalg.norm(a["y"])
        assert err < 1e-6, (tag, err)
        mism = np.mean(y16 != a["y_bf16"])
        assert mism < 2e-3, (tag, mism)
        h16, _ = oracle.hybrid_linear(a["w4"], a["sf4"], a["lo"], a["w8"], a["sf8"], a["hi"], a["xq"], a["xsf"], outputs, bf16=False)
        assert np.mean(h16 != a["y_half"]) < 2e-3


def _numpy_pack_fp8(x: torch.Tensor):
    """Independent vectorised restatement (torch float8 cast) used to cross-check the C oracle."""
    rows, k = x.shape
    v = x.float().reshape(rows, k // 32, 32)
    amax = v.abs().amax(-1)
    e = torch.where(amax > 0, torch.ceil(torch.log2(amax / 448.0)), torch.zeros_like(amax)).clamp(-127, 127)
    q = torch.ldexp(v, (-e).int()[..., None]).to(torch.float8_e4m3fn).view(torch.uint8).reshape(rows, k)
    sf = np.full(oracle.scale_size(rows, k), 127, dtype=np.uint8)
    sf[oracle.scale_indices(rows, k)] = (e + 127).to(torch.uint8).numpy()
    return q.numpy(), sf


@pytest.mark.parametrize("rows,k", [(1, 128), (3, 896), (33, 256), (129, 384), (257, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_pack_fp8_matches_vectorised_restatement_and_pads_with_0x7f(rows, k, dtype):
    torch.manual_seed(rows * 1000 + k)
    x = torch.randn(rows, k)
    x[:, :: 97] *= 20
    x[0, :32] = 0
    x = (x * torch.tensor([.125, 1, 64, 1e-3])[torch.arange(rows) % 4][:, None]).to(dtype)
    q, sf = oracle.pack(x, fp4=False, bf16=dtype == torch.bfloat16)
    q2, sf2 = _numpy_pack_fp8(x)
    assert np.array_equal(q, q2)
    assert np.array_equal(sf, sf2)
    valid = np.zeros(sf.size, dtype=bool)
    valid[oracle.scale_indices(rows, k).ravel()] = True
    assert np.all(sf[~valid] == 0x7f)
    assert sf[oracle.scale_indices(rows, k)[0, 0]] == 127          # zero block -> exponent 0


def test_pack_fp4_nibble_order_and_negative_zero():
    x = torch.zeros(1, 128, dtype=torch.bfloat16)
    x[0, 0], x[0, 1], x[0, 2], x[0, 3] = 6.0, -3.0, -0.0, 0.5
    q, sf = oracle.pack(x, fp4=True)
    assert sf[0] == 127                                            # amax 6 -> e = 0
    assert q[0, 0] == (7 | (13 << 4))                              # even k in the low nibble
    assert q[0, 1] == (8 | (1 << 4))                               # -0 keeps its sign bit (code 8)


@pytest.mark.parametrize("case", [(257, 7, 256, 26, "random"), (257, 7, 256, 0, "interleaved"),
                                  (257, 7, 256, 257, "interleaved"), (511, 33, 384, 73, "interleaved"),
                                  (129, 1, 128, 17, "random"), (255, 17, 128, 51, "contiguous")])
@pytest.mark.parametrize("bf16", [True, False])
def test_exact_representable_cases_are_bit_exact_through_the_oracle(case, bf16):
    """The generator of src/kernel/output_channel_bench.cu: decode+matmul must equal the closed-form loop bit for bit."""
    outputs, tokens, k, high, mapping = case
    c = oracle.exact_case(outputs, tokens, k, high, mapping, bf16=bf16)
    assert sorted(np.concatenate([c["lo"], c["hi"]]).tolist()) == list(range(outputs))
    y, _ = oracle.hybrid_linear(c["w4"], c["sf4"], c["lo"], c["w8"], c["sf8"], c["hi"], c["xq"], c["xsf"], outputs, bf16=bf16)
    assert np.array_equal(y, c["expected"])


def test_silu_pack_equals_two_step_restatement():
    torch.manual_seed(7)
    for dtype in (torch.bfloat16, torch.float16):
        bf16 = dtype == torch.bfloat16
        x = (torch.randn(5, 512) * 2).to(dtype)
        q, sf, dbg = oracle.silu_pack(x, bf16=bf16, debug=True)
        gate, up = x[:, :256].float(), x[:, 256:].float()
        act = (gate / (1 + torch.exp(-gate))).to(dtype)
        v = (act.float() * up).to(dtype)
        got = torch.from_numpy(dbg.view(np.int16)).view(dtype)
        assert (got.view(torch.int16) != v.view(torch.int16)).float().mean() < 1e-3   # expf implementations differ by <=1ulp
        q2, sf2 = oracle.pack(got, fp4=False, bf16=bf16)
        assert np.array_equal(q, q2) and np.array_equal(sf, sf2)


# ---- offline exponent search (allocation/fp4_quant.py:28-58) -------------------------------------------------

@pytest.mark.parametrize("tag", ["plain", "weighted", "up", "heavy"])
def test_clip_search_matches_reference_composition(golden, tag):
    """Codes and scale bytes equal the reference's pieces composed as its `quantize` composes them."""
    CLIP = golden("clip_search.npz")
    bits, importance = CLIP[tag + "__w"], CLIP[tag + "__importance"]
    offsets = tuple(int(o) for o in CLIP[tag + "__offsets"])
    q4, scales = oracle.clip_pack(bits, importance if importance.size else None, offsets, bf16=False)
    assert (scales == CLIP[tag + "__scales"]).all() and (q4 == CLIP[tag + "__q4"]).all()
    base_q, base_sf = oracle.pack(bits, fp4=True, bf16=False)
    base = base_sf[oracle.scale_indices(*bits.shape)]
    assert (scales != base).any()                                   # the fixture exercises the search
    assert ((scales.astype(int) - base.astype(int)) != 0).sum() == (scales != base).sum()


def test_clip_search_without_offsets_is_pack():
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((40, 256)) * 0.1).astype(np.float16)
    q4, scales = oracle.clip_pack(w.view(np.uint16), None, (), bf16=False)
    base_q, base_sf = oracle.pack(w.view(np.uint16), fp4=True, bf16=False)
    assert (q4 == base_q).all() and (scales == base_sf[oracle.scale_indices(40, 256)]).all()


def test_clip_search_never_increases_the_weighted_error():
    rng = np.random.default_rng(6)
    w = (rng.standard_normal((64, 384)) * 0.05).astype(np.float16)
    w[rng.random((64, 384)) < 0.03] *= 10
    importance = rng.random(384).astype(np.float32) * 2
    q4, scales = oracle.clip_pack(w.view(np.uint16), importance, (0, -1, -2), bf16=False)
    base_q, base_sf = oracle.pack(w.view(np.uint16), fp4=True, bf16=False)

    def error(q, logical):
        sf = np.full(oracle.scale_size(64, 384), 127, np.uint8)
        sf[oracle.scale_indices(64, 384)] = logical
        diff = oracle.decode(q, sf, 384, True).astype(np.float64) - w.astype(np.float64)
        return ((diff ** 2) * importance).reshape(64, 12, 32).sum(-1)

    after, before = error(q4, scales), error(base_q, base_sf[oracle.scale_indices(64, 384)])
    assert (after <= before * (1 + 1e-6) + 1e-25).all() and after.sum() < before.sum()
