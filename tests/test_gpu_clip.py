"""Offline MXFP4 exponent search (hg_clip_pack / fp4_quant.quantize) against the CPU oracle: bit-exact codes
and scale bytes, on the committed golden inputs and on larger seeded matrices of both dtypes."""
import numpy as np
import pytest
import torch

import oracle
from helpers import SEED, dev
from hygemm_vllm import fp4_quant, native, offline_weights

pytestmark = pytest.mark.gpu
GOLDEN = np.load(__import__("pathlib").Path(__file__).parent / "golden" / "clip_search.npz")


@pytest.mark.parametrize("tag", ["plain", "weighted", "up", "heavy"])
def test_golden_cases_bit_exact(tag):
    bits = GOLDEN[tag + "__w"]
    importance = GOLDEN[tag + "__importance"]
    offsets = tuple(int(o) for o in GOLDEN[tag + "__offsets"])
    w = dev(bits).view(torch.float16)
    q4, scales, stats = fp4_quant.quantize(w, dev(importance) if importance.size else None, offsets)
    assert (q4.cpu().numpy() == GOLDEN[tag + "__q4"]).all()
    assert (scales.cpu().numpy() == GOLDEN[tag + "__scales"]).all()
    assert stats["groups"] == scales.numel() and sum(stats["shift_groups"].values()) == scales.numel()
    assert stats["weighted_error_after"] <= stats["weighted_error_before"]
    np.testing.assert_allclose(stats["weighted_error_after"], GOLDEN[tag + "__error"].astype(np.float64).sum(), rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,k", [(1, 128), (129, 384), (1000, 3584)])
def test_random_matrices_match_the_oracle(dtype, rows, k):
    g = torch.Generator().manual_seed(SEED + rows)
    w = torch.randn(rows, k, generator=g) * 0.03
    w[torch.rand(rows, k, generator=g) < 0.01] *= 15
    w[0, :64] = 0
    w = w.to(dtype)
    importance = torch.rand(k, generator=g) * 3
    for weight, offsets in [(None, (0, -1, -2)), (importance, (0, -1, -2)), (importance, (0, 1, -1, -3))]:
        q4, scales, stats = fp4_quant.quantize(w.cuda(), None if weight is None else weight.cuda(), offsets)
        want_q4, want_scales = oracle.clip_pack(w, None if weight is None else weight.numpy(), offsets,
                                                bf16=dtype == torch.bfloat16)
        assert (scales.cpu().numpy() == want_scales).all()
        assert (q4.cpu().numpy() == want_q4).all()
        assert stats["shift_groups"]["0"] < scales.numel() or rows == 1


def test_no_offsets_is_round_to_nearest_and_feeds_a_layer():
    """Without offsets the result is hg_pack's; a searched bank installs into a layer and changes only the low rows."""
    g = torch.Generator().manual_seed(SEED)
    w = (torch.randn(384, 512, generator=g) * 0.02).to(torch.bfloat16).cuda()
    q4, scales, _ = fp4_quant.quantize(w, offsets=())
    base_q, base_sf = native.pack(w, True)
    assert torch.equal(q4, base_q) and torch.equal(offline_weights.physical_scales(scales, 512), base_sf)
    ids = torch.arange(0, 384, 7, device="cuda")
    layer = native.DualLinear(w, ids)
    bank_q, bank_scales, stats = fp4_quant.quantize(w)
    offline_weights.replace_low_weight(layer, bank_q, bank_scales)
    x = torch.randn(8, 512, generator=g).to(torch.bfloat16).cuda()
    y = layer(x)
    dense = x.float() @ w.float().t()
    assert (y.float() - dense).norm() / dense.norm() < 0.12
    assert stats["weight_error_after"] <= stats["weight_error_before"]
