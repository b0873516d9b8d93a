"""`hygemm_offline`: E2M1 helpers against the reference's golden vectors, bank files, plan inheritance
and (GPU) a bank built with the exponent search loaded into a layer, whole and as tensor-parallel shards."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

vllm = pytest.importorskip("vllm")
from hygemm_vllm import fp4_quant, offline, quantization as Q  # noqa: E402

GOLDEN = Path(__file__).parent / "golden"


def test_e2m1_helpers_match_reference_vectors():
    g = np.load(GOLDEN / "codes_rne.npz")
    values = torch.from_numpy(g["values"])
    codes = fp4_quant.codes_rne(values)
    assert (codes.numpy() == g["codes"]).all()
    packed = fp4_quant.pack_codes(codes)
    assert (packed.numpy() == g["packed"]).all()
    assert (fp4_quant.unpack(packed).numpy() == g["codes"]).all()
    decoded = fp4_quant.decode_logical(packed, torch.from_numpy(g["logical"]), 64)
    assert (decoded.numpy() == g["decoded"]).all()


def test_offline_config_is_registered_and_optional_keys_default():
    from vllm.model_executor.layers.quantization import get_quantization_config
    assert get_quantization_config("hygemm_offline") is offline.OfflineConfig
    config = offline.OfflineConfig.from_config({"selection": {}, "tuning_plan": "/nonexistent/ignored.json"})
    assert config.get_name() == "hygemm_offline" and config.kind == "hygemm"
    assert config.bank is None and config.reference_plans is None and config.plans is None
    layer = torch.nn.Module()
    assert config.get_quant_method(layer, "model.layers.0.mlp.down_proj") is None


class _Plans:
    def __init__(self):
        self.calls = []

    def get(self, outputs, k, high, tokens):
        self.calls.append(("get", outputs, k, high, tokens))
        return {"low_id": 1, "high_id": 1, "policy": "serial", "tokens": tokens}

    def get_layer(self, name, outputs, k, high, tokens):
        self.calls.append(("layer", name, outputs, k, high, tokens))
        return {"low_id": 3, "high_id": 3, "policy": "serial", "tokens": tokens}


def test_inherited_plans_use_the_tuned_width_and_the_decode_override():
    base, override = _Plans(), _Plans()
    reference = {"layer": "m.mlp.down_proj", "out": 64, "k": 256, "high": 8}
    plans = offline.InheritedLayerPlans(base, reference, (64, 256, 12))
    assert plans.get(64, 256, 12, 200)["low_id"] == 1 and base.calls == [("get", 64, 256, 8, 200)]
    with pytest.raises(ValueError):
        plans.get(64, 256, 8, 1)
    plans = offline.InheritedLayerPlans(base, reference, (64, 256, 12), override)
    assert plans.get(64, 256, 12, 128)["low_id"] == 3
    assert override.calls == [("layer", "m.mlp.down_proj", 64, 256, 12, 128)]
    assert plans.get(64, 256, 12, 129)["low_id"] == 1


def test_bank_entry_is_checked_against_its_digest(tmp_path):
    entry = {"q4": torch.zeros(4, 64, dtype=torch.uint8), "scales": torch.full((4, 4), 127, dtype=torch.uint8)}
    torch.save(entry, tmp_path / "a.pt")
    manifest = {"layers": {"a": {"file": "a.pt", "sha256": offline.file_sha256(tmp_path / "a.pt")}}}
    q4, scales = offline.read_bank_entry(manifest, tmp_path, "a")
    assert q4.shape == (4, 64) and scales.shape == (4, 4)
    manifest["layers"]["a"]["sha256"] = "0" * 64
    with pytest.raises(ValueError, match="does not match its manifest"):
        offline.read_bank_entry(manifest, tmp_path, "a")


def test_bound_decode_plan_refuses_another_selection(tmp_path):
    plan = {"hygemm": [], "binding": None}
    (tmp_path / "plan.json").write_text(json.dumps(plan))
    config = offline.OfflineConfig.from_config({"selection": {"a": [1]}, "decode_plans": str(tmp_path / "plan.json")})
    with pytest.raises(ValueError, match="different channel selection"):
        config._check_binding({"selection": {"a": [1]}}, {"selection_canonical_sha256": "0" * 64})
    import hashlib
    digest = hashlib.sha256(json.dumps({"a": [1]}, sort_keys=True, separators=(",", ":")).encode()).hexdigest()
    with pytest.raises(ValueError, match="different FP4 bank"):
        config._check_binding({"selection": {"a": [1]}}, {"selection_canonical_sha256": digest, "bank_manifest_sha256": "x"})


# ---- GPU: build a bank, load it ---------------------------------------------------------------------------

class _StubUnquantized:
    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **attrs):
        layer.weight = torch.nn.Parameter(torch.empty(sum(output_partition_sizes), input_size_per_partition,
                                                      dtype=params_dtype), requires_grad=False)


def _load(monkeypatch, config, prefix, weight, parts, full_k=None, tp=None):
    monkeypatch.setattr(Q, "UnquantizedLinearMethod", _StubUnquantized)
    method = offline.OfflineLinearMethod(config, prefix)
    layer = torch.nn.Module()
    method.create_weights(layer, weight.shape[1], parts, full_k or weight.shape[1], sum(parts), weight.dtype,
                          weight_loader=lambda *a: None)
    layer.weight = torch.nn.Parameter(weight.cuda(), requires_grad=False)
    if tp:
        layer.tp_size, layer.tp_rank = tp
        layer.reduce_results = False
    method.process_weights_after_loading(layer)
    return method


@pytest.mark.gpu
def test_bank_round_trip_through_the_offline_method(tmp_path, monkeypatch):
    from hygemm_vllm import native, offline_weights
    g = torch.Generator().manual_seed(20261024)
    gate = (torch.randn(256, 512, generator=g) * 0.03).to(torch.bfloat16)
    up = (torch.randn(256, 512, generator=g) * 0.03).to(torch.bfloat16)
    gate[torch.rand(256, 512, generator=g) < 0.02] *= 10
    names = {"m.mlp.gate_proj": gate, "m.mlp.up_proj": up}
    selection = {"m.mlp.gate_proj": list(range(0, 256, 9)), "m.mlp.up_proj": [3, 200]}
    fused = torch.cat([gate, up])

    native_manifest = offline.build_bank(tmp_path / "native_rtn", names, "native_rtn")
    clip_manifest = offline.build_bank(tmp_path / "mse_clip", names, "mse_clip", chunk_rows=100)
    manifest = json.loads(clip_manifest.read_text())
    assert manifest["completed"] and manifest["offsets"] == [0, -1, -2] and manifest["format"] == offline.BANK_FORMAT
    stats = manifest["layers"]["m.mlp.gate_proj"]["stats"]
    assert stats["groups"] == 256 * 16 and sum(stats["shift_groups"].values()) == stats["groups"]
    assert stats["weight_error_after"] < stats["weight_error_before"]

    # native_rtn: verified bit for bit against the load-time quantiser
    config = offline.OfflineConfig.from_config({"selection": selection, "q4_bank": str(native_manifest)})
    method = _load(monkeypatch, config, "m.mlp.gate_up_proj", fused, [256, 256])
    plain = native.DualLinear(fused.cuda(), method.runtime.hi.long())
    assert torch.equal(method.runtime.w4, plain.w4) and torch.equal(method.runtime.sf4, plain.sf4)

    # mse_clip: low rows come from the bank, high rows and activations untouched
    config = offline.OfflineConfig.from_config({"selection": selection, "q4_bank": str(clip_manifest)})
    method = _load(monkeypatch, config, "m.mlp.gate_up_proj", fused, [256, 256])
    runtime = method.runtime
    q4, scales, _ = fp4_quant.quantize(fused.cuda())
    assert torch.equal(runtime.w4, q4[runtime.lo.long()])
    assert torch.equal(runtime.sf4, offline_weights.physical_scales(scales[runtime.lo.long()], 512))
    assert torch.equal(runtime.w8, plain.w8) and not torch.equal(runtime.w4, plain.w4)
    x = torch.randn(8, 512, generator=g).to(torch.bfloat16).cuda()
    y = method.apply(None, x)
    dense = x.float() @ fused.cuda().float().t()
    assert (y.float() - dense).norm() / dense.norm() < 0.2       # 4-bit weights with x10 outliers in 2 % of gate

    # a damaged bank is refused
    entry = tmp_path / "mse_clip" / "m.mlp.up_proj.pt"
    damaged = bytearray(entry.read_bytes())
    damaged[len(damaged) // 2] ^= 0xFF
    entry.write_bytes(bytes(damaged))
    with pytest.raises(ValueError, match="does not match its manifest"):
        _load(monkeypatch, config, "m.mlp.gate_up_proj", fused, [256, 256])


@pytest.mark.gpu
def test_tensor_parallel_shards_read_their_slice_of_the_bank(tmp_path, monkeypatch):
    g = torch.Generator().manual_seed(7)
    down = (torch.randn(128, 512, generator=g) * 0.03).to(torch.bfloat16)
    gate = (torch.randn(256, 256, generator=g) * 0.03).to(torch.bfloat16)
    up = (torch.randn(256, 256, generator=g) * 0.03).to(torch.bfloat16)
    manifest = offline.build_bank(tmp_path / "bank", {"m.mlp.down_proj": down, "m.mlp.gate_proj": gate,
                                                       "m.mlp.up_proj": up}, "mse_clip")
    selection = {"m.mlp.down_proj": [1, 64], "m.mlp.gate_proj": [0, 130], "m.mlp.up_proj": [255]}
    config = offline.OfflineConfig.from_config({"selection": selection, "q4_bank": str(manifest)})
    # row-parallel rank 1 of 2: second half of K
    method = _load(monkeypatch, config, "m.mlp.down_proj", down[:, 256:].contiguous(), [128], full_k=512, tp=(2, 1))
    q4, _, _ = fp4_quant.quantize(down[:, 256:].contiguous().cuda())
    assert torch.equal(method.runtime.w4, q4[method.runtime.lo.long()])
    # column-parallel rank 1 of 2: rows 128..255 of gate and of up
    shard = torch.cat([gate[128:], up[128:]])
    method = _load(monkeypatch, config, "m.mlp.gate_up_proj", shard, [128, 128], tp=(2, 1))
    q4, _, _ = fp4_quant.quantize(shard.cuda())
    assert method.runtime.hi.tolist() == [2, 255] and torch.equal(method.runtime.w4, q4[method.runtime.lo.long()])
