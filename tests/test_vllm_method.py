"""The vLLM quantization config / linear method surface on CPU (no GPU, no model): names, selection
contract of the reference (quantization.py:104-122) and its tensor-parallel extension."""
import pytest
import torch

vllm = pytest.importorskip("vllm")
from hygemm_vllm import quantization as Q  # noqa: E402


class _StubUnquantized:
    """Stands in for vLLM's UnquantizedLinearMethod, whose create_weights needs an initialised
    tensor-parallel group; records that the delegation carries the reference's argument list."""

    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                       params_dtype, **attrs):
        assert "weight_loader" in attrs
        layer.weight = torch.nn.Parameter(torch.empty(sum(output_partition_sizes), input_size_per_partition,
                                                      dtype=params_dtype), requires_grad=False)


@pytest.fixture(autouse=True)
def _stub(monkeypatch):
    monkeypatch.setattr(Q, "UnquantizedLinearMethod", _StubUnquantized)


def make(prefix, parts, k=256, full_k=None, selection=None):
    config = Q.HyGEMMConfig.from_config({"quant_method": "hygemm", "selection": selection or {}})
    method = Q.MixedLinearMethod(config, prefix)
    layer = torch.nn.Module()
    method.create_weights(layer, k, parts, full_k or k, sum(parts), torch.bfloat16, weight_loader=lambda *a: None)
    return config, method, layer


def test_config_surface():
    config = Q.HyGEMMConfig.from_config({"selection": {}, "low_id": 3, "high_id": 0, "concurrent": False})
    assert Q.HyGEMMConfig.get_name() == "hygemm"
    assert Q.HyGEMMConfig.get_supported_act_dtypes() == [torch.bfloat16, torch.float16]
    assert Q.HyGEMMConfig.get_min_capability() == 100
    assert Q.HyGEMMConfig.get_config_filenames() == ["quant_config.json", "quantize_config.json"]
    assert (config.low_id, config.high_id, config.concurrent, config.format) == (3, 0, False, "fp16_rtn")
    with pytest.raises(ValueError, match="Unsupported checkpoint format"):
        Q.HyGEMMConfig.from_config({"checkpoint_format": "mixllm_v1"})
    from vllm.model_executor.layers.quantization import get_quantization_config
    assert get_quantization_config("hygemm") is Q.HyGEMMConfig


def test_create_weights_delegates_and_validates():
    _, method, layer = make("model.layers.0.mlp.down_proj", [64], k=256, selection={"model.layers.0.mlp.down_proj": [1]})
    assert layer.weight.shape == (64, 256) and layer.weight.dtype == torch.bfloat16
    assert (method.outputs, method.k) == (64, 256)
    with pytest.raises(ValueError, match="K divisible by 128"):
        make("x.down_proj", [64], k=200)
    config = Q.HyGEMMConfig.from_config({})
    with pytest.raises(ValueError):
        Q.MixedLinearMethod(config, "x").create_weights(torch.nn.Module(), 256, [64], 256, 64, torch.float32,
                                                        weight_loader=lambda *a: None)


def test_selected_rows_fused_offsets_and_errors():
    sel = {"m.self_attn.q_proj": [5, 0], "m.self_attn.k_proj": [3], "m.self_attn.v_proj": [7, 1]}
    _, method, layer = make("m.self_attn.qkv_proj", [16, 8, 8], selection=sel)
    assert method.selected_rows("cpu").tolist() == [0, 5, 16 + 3, 24 + 1, 24 + 7]
    _, method, _ = make("m.mlp.gate_up_proj", [8, 8], selection={"m.mlp.gate_proj": [2], "m.mlp.up_proj": [2]})
    assert method.selected_rows("cpu").tolist() == [2, 10]
    _, method, _ = make("m.self_attn.qkv_proj", [16, 8, 8], selection={"m.self_attn.q_proj": [0]})
    with pytest.raises(ValueError, match="Missing channel selection"):
        method.selected_rows("cpu")
    for bad in ([1, 1], [-1], [16]):
        _, method, _ = make("m.self_attn.o_proj", [16], selection={"m.self_attn.o_proj": bad})
        with pytest.raises(ValueError, match="Invalid channel map"):
            method.selected_rows("cpu")
    _, method, _ = make("m.self_attn.qkv_proj", [16, 8], selection=sel)
    with pytest.raises(ValueError, match="Projection partition mismatch"):
        method.selected_rows("cpu")


def test_selected_rows_tensor_parallel_shards():
    sel = {"m.self_attn.q_proj": [1, 9, 17, 30], "m.self_attn.k_proj": [0, 5], "m.self_attn.v_proj": [7]}
    # column-parallel rank 1 of 2: per-rank sizes 16 / 4 / 4 of full 32 / 8 / 8
    _, method, layer = make("m.self_attn.qkv_proj", [16, 4, 4], selection=sel)
    layer.tp_size, layer.tp_rank = 2, 1
    assert method.selected_rows("cpu", layer).tolist() == [1, 14, 16 + 1, 20 + 3]
    # row-parallel: K sharded, every rank keeps the whole selection
    _, method, layer = make("m.self_attn.o_proj", [32], k=128, full_k=256, selection={"m.self_attn.o_proj": [3, 31]})
    layer.tp_size, layer.tp_rank = 2, 1
    assert method.selected_rows("cpu", layer).tolist() == [3, 31]
    # l2norm rule on the loaded weight
    config = Q.HyGEMMConfig.from_config({"selection": {"rule": "l2norm", "fraction": 0.25}})
    method = Q.MixedLinearMethod(config, "m.mlp.gate_up_proj")
    layer = torch.nn.Module()
    method.create_weights(layer, 128, [8, 8], 128, 16, torch.bfloat16, weight_loader=lambda *a: None)
    w = torch.ones(16, 128)
    w[[2, 5, 9, 15]] *= 3
    assert method.selected_rows("cpu", layer, w).tolist() == [2, 5, 9, 15]
