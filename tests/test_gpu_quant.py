"""Quantiser and SwiGLU producer through the C ABI vs the CPU oracle (bit-exact)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import bits
from hygemm_vllm import native, producer

pytestmark = pytest.mark.gpu

ROWS = [1, 3, 8, 17, 31, 32, 33, 64, 127, 128, 129, 255, 256, 257]


def _random(rows, k, dtype, scale, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, k, generator=g) * scale
    x[:, ::53] *= 20
    if rows > 2:
        x[1, :64] = 0                      # all-zero K32 blocks
        x[2, 5] = -0.0
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("fp4", [False, True])
def test_pack_is_bit_exact_incl_padding(dtype, fp4):
    """Matrix of optimization/check_pack.py:17-35 of the reference (rows x K x scales), codes AND
    the whole scale buffer, with the buffer pre-filled with 0xff so stale padding would show."""
    for rows in ROWS:
        for k, scale in [(128, 0.125), (896, 2.0), (3584, 1.0)]:
            x = _random(rows, k, dtype, scale, rows * 7 + k)
            xd = x.cuda()
            q, sf = native.pack(xd, fp4)
            sf.fill_(255)
            q2, sf2 = native.pack(xd, fp4)          # second call must rewrite every byte
            want_q, want_sf = oracle.pack(x, fp4=fp4, bf16=dtype == torch.bfloat16)
            assert np.array_equal(q2.cpu().numpy(), want_q), (rows, k)
            assert np.array_equal(sf2.cpu().numpy(), want_sf), (rows, k)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_pack_every_finite_16bit_value(dtype):
    """Every finite bit pattern as an input and as a group maximum
    (performance/check.py:39-44, performance/check_pack_maxima.py:9-22 of the reference)."""
    allbits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(dtype)
    finite = allbits[torch.isfinite(allbits.float())]
    pad = (-finite.numel()) % 128
    x = torch.cat([finite, finite[:pad]]).reshape(-1, 128)
    for fp4 in (False, True):
        q, sf = native.pack(x.cuda(), fp4)
        want_q, want_sf = oracle.pack(x, fp4=fp4, bf16=dtype == torch.bfloat16)
        assert np.array_equal(q.cpu().numpy(), want_q)
        assert np.array_equal(sf.cpu().numpy(), want_sf)
    # each value as the maximum of an otherwise tiny group (scale-boundary ties)
    vals = finite[finite.float().abs() > 0][::3]
    rows = vals.numel()
    x = torch.zeros(rows, 128, dtype=dtype)
    x[:, 0] = vals
    x[:, 1] = (vals.float() * 0.37).to(dtype)
    x[:, 33] = vals
    x[:, 40] = -(vals.float() * 0.5).to(dtype)
    q, sf = native.pack(x.cuda(), False)
    want_q, want_sf = oracle.pack(x, fp4=False, bf16=dtype == torch.bfloat16)
    assert np.array_equal(q.cpu().numpy(), want_q)
    assert np.array_equal(sf.cpu().numpy(), want_sf)


def test_fp4_tie_table():
    """allocation/check_components.py:14 of the reference: exact ties and signed zeros."""
    ties = [0., -0., .25, .75, 1.25, 1.75, 2.5, 3.5, 5., 6., -.25, -.75, -1.25, -1.75, -2.5, -3.5, -5., -6.]
    x = torch.zeros(1, 128, dtype=torch.float16)
    x[0, :len(ties)] = torch.tensor(ties, dtype=torch.float16)
    x[0, 31] = 6.0
    q, sf = native.pack(x.cuda(), True)
    want_q, want_sf = oracle.pack(x, fp4=True, bf16=False)
    assert np.array_equal(q.cpu().numpy(), want_q) and np.array_equal(sf.cpu().numpy(), want_sf)


def test_pack_rejects_bad_arguments():
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        native.pack(x)
    lib = native.library()
    assert lib.hg_pack(None, None, None, 1, 128, 0, None) == -1
    assert b"Invalid MX pack arguments" in lib.hg_last_error()
    assert lib.hg_silu_pack(None, None, None, None, 1, 128, None, 0) == 1     # cudaErrorInvalidValue


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_silu_pack_matches_oracle_and_two_step_path(dtype):
    """performance/check_producer.py:17-28 of the reference: codes, scales and the 16-bit product of the
    fused kernel equal SiluAndMul followed by pack.  expf differs by <= 1 ulp between CPU and GPU libraries,
    so the CPU comparison allows rare 16-bit neighbours; the quantisation of the device's own product
    must be bit-exact."""
    bf16 = dtype == torch.bfloat16
    for rows, k, scale in [(1, 128, 1.0), (3, 896, 4.0), (33, 4864, 0.1), (128, 18944, 2.0), (129, 896, 16.0)]:
        g = torch.Generator().manual_seed(rows + k)
        x = (torch.randn(rows, 2 * k, generator=g) * scale).to(dtype)
        q, sf, dbg = producer.silu_pack(x.cuda(), 0, debug=True)
        oq, osf, odbg = oracle.silu_pack(x, bf16=bf16, debug=True)
        got = bits(dbg)
        differ = got != odbg
        assert differ.mean() < 1e-3, (rows, k, differ.mean())
        # neighbours only
        assert np.all(np.abs(got[differ].astype(np.int32) - odbg[differ].astype(np.int32)) <= 1)
        q2, sf2 = oracle.pack(dbg.cpu(), fp4=False, bf16=bf16)
        assert np.array_equal(q.cpu().numpy(), q2) and np.array_equal(sf.cpu().numpy(), sf2), (rows, k)
        # two-step device path: torch SiLU*up (same expf library) then hg_pack
        xd = x.cuda()
        act = torch.nn.functional.silu(xd[:, :k].float()).to(dtype)
        prod = (act.float() * (xd[:, k:].float() + 0.0)).to(dtype)
        q3, sf3 = native.pack(prod.contiguous())
        same = (bits(prod) == got).mean()
        assert same > 0.999, (rows, k, same)
        if same == 1.0:
            assert torch.equal(q3, q) and torch.equal(sf3, sf)


def test_silu_pack_vs_vllm_op():
    """Bitwise parity with the installed vLLM SiluAndMul op followed by pack, when that op is available."""
    try:
        import vllm._custom_ops  # noqa: F401
        op = torch.ops._C.silu_and_mul
    except Exception:
        pytest.skip("vLLM custom ops not loadable")
    for dtype in (torch.bfloat16, torch.float16):
        for rows, k in [(1, 128), (33, 896), (128, 18944)]:
            g = torch.Generator().manual_seed(rows * 3 + k)
            x = (torch.randn(rows, 2 * k, generator=g) * 2).to(dtype).cuda()
            out = torch.empty(rows, k, dtype=dtype, device="cuda")
            op(out, x)
            q_ref, sf_ref = native.pack(out)
            q, sf, dbg = producer.silu_pack(x, 0, debug=True)
            assert torch.equal(dbg.view(torch.int16), out.view(torch.int16)), (dtype, rows, k)
            assert torch.equal(q, q_ref) and torch.equal(sf, sf_ref)
