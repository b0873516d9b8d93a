"""Schedule tuner: every candidate validates against the dequantised matmul, the plan file binds to the
library and drives a layer through `PlanTable`."""
import json

import pytest
import torch

from hygemm_vllm import native, plans, tune

pytestmark = pytest.mark.gpu


def test_tune_bind_and_apply(tmp_path):
    device = torch.device("cuda", 0)
    log = []
    rows = tune.tune_shape(640, 512, 64, [2, 16], device, log=log)
    assert [r["tokens"] for r in rows] == [2, 16]
    for row, record in zip(rows, log):
        assert row["policy"] in native.POLICIES and row["validated_full_output"]
        assert len(record["screen"]) == (6 if row["tokens"] <= 4 else 3)
        best = min(record["refined"], key=lambda s: s["us"])
        kept_default = (row["low_id"], row["high_id"]) == (0, 0)
        assert kept_default == (record["base"]["us"] / best["us"] < tune.SWITCH_MARGIN)
    path = tmp_path / "plans.json"
    path.write_text(json.dumps(tune.bind(rows)))
    table = plans.PlanTable(path, "hygemm")
    assert table.binding["layout"] == plans.LAYOUT
    assert table.get(640, 512, 64, 9)["tokens"] == 16
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(640, 512, generator=g) * .04).half().cuda()
    ids = torch.sort(torch.randperm(640, generator=g)[:64]).values.cuda()
    planned, plain = native.DualLinear(w, ids, plans=table), native.DualLinear(w, ids)
    x = torch.randn(16, 512, generator=g).half().cuda()
    torch.testing.assert_close(planned(x), plain(x), atol=.01, rtol=.003)
    assert planned.plans_used[16][0] == 16
    # a plan bound to another binary is refused
    document = tune.bind(rows)
    document["binding"]["library_sha256"] = "0" * 64
    path.write_text(json.dumps(document))
    with pytest.raises(ValueError, match="different binary"):
        plans.PlanTable(path, "hygemm")
