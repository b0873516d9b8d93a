"""vLLM quantization config and linear method of the hybrid MXFP4/MXFP8 layer.

Mirror of the reference's `integrations/vllm/hygemm_vllm/quantization.py`
(`CommonConfig`, `HyGEMMConfig`, `MixedLinearMethod`, `model_audit`, op
`hygemm_vllm::linear`) for the `hygemm` method.  Kept from the reference: the
`quantization_config` keys (`selection`, `checkpoint_format`, `low_id`,
`high_id`, `concurrent`, `tuning_plan`), delegation of `create_weights` to the
unquantised method so vLLM's stock (TP-aware) loader fills `layer.weight`,
load-time packing in `process_weights_after_loading`, and `apply`.

Added: bfloat16 (primary) next to float16; tensor parallelism (column-parallel
layers shard the selection with their rows, row-parallel layers shard K and let
vLLM's RowParallelLinear all-reduce the partial sums); and a selection *rule*
`{"rule": "l2norm", "fraction": f, "multiple": m}` evaluated at load time, for
random-init models whose weights only exist after loading.
"""
from __future__ import annotations

import torch
from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase, UnquantizedLinearMethod
from vllm.model_executor.layers.quantization import register_quantization_config
from vllm.model_executor.layers.quantization.base_config import QuantizationConfig

from . import tp
from .ops import _runtimes, linear, register_runtime  # noqa: F401  (`_runtimes` is read by producer/worker code)

_FUSED = {".qkv_proj": ("q", "k", "v"), ".gate_up_proj": ("gate", "up")}


class CommonConfig(QuantizationConfig):
    kind = ""

    def __init__(self, config):
        super().__init__()
        self.selection = config.get("selection", {})
        self.format = config.get("checkpoint_format", "fp16_rtn")
        self.low_id = int(config.get("low_id", 0))
        self.high_id = int(config.get("high_id", 0))
        self.concurrent = bool(config.get("concurrent", True))
        self.plans = None
        if config.get("tuning_plan"):
            from .plans import PlanTable
            self.plans = PlanTable(config["tuning_plan"], self.kind)
        # `fp16_rtn`: plain 16-bit weights quantised round-to-nearest at load time
        # (bf16 checkpoints use the same name; `bf16_rtn` is accepted as an alias).
        if self.format not in ("fp16_rtn", "bf16_rtn"):
            raise ValueError("Unsupported checkpoint format")

    @classmethod
    def get_name(cls):
        return cls.kind

    @classmethod
    def get_supported_act_dtypes(cls):
        return [torch.bfloat16, torch.float16]

    @classmethod
    def get_min_capability(cls):
        return 100

    @staticmethod
    def get_config_filenames():
        return ["quant_config.json", "quantize_config.json"]

    @classmethod
    def from_config(cls, config):
        return cls(config)

    def get_quant_method(self, layer, prefix):
        if isinstance(layer, LinearBase):
            if prefix.endswith("lm_head"):
                return UnquantizedLinearMethod()
            return MixedLinearMethod(self, prefix)
        return None


@register_quantization_config("hygemm")
class HyGEMMConfig(CommonConfig):
    kind = "hygemm"


class MixedLinearMethod(LinearMethodBase):
    def __init__(self, config, prefix):
        self.config, self.prefix = config, prefix
        self.runtime = None
        self.handle = None

    # -- creation -----------------------------------------------------------------------------
    def create_weights(self, layer, input_size_per_partition, output_partition_sizes,
                       input_size, output_size, params_dtype, **attrs):
        if input_size_per_partition % 128 or params_dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("Requires FP16/BF16 activations and K divisible by 128")
        self.parts = list(output_partition_sizes)
        self.outputs, self.k = sum(self.parts), input_size_per_partition
        self.full_k, self.full_outputs = input_size, output_size
        UnquantizedLinearMethod().create_weights(layer, input_size_per_partition, output_partition_sizes,
                                                 input_size, output_size, params_dtype, **attrs)

    # -- selection ------------------------------------------------------------------------------
    def projection_names(self):
        for suffix, parts in _FUSED.items():
            if self.prefix.endswith(suffix):
                return [self.prefix.replace(suffix, f".{p}_proj") for p in parts]
        return [self.prefix]

    def _tp(self, layer):
        world = int(getattr(layer, "tp_size", 1))
        rank = int(getattr(layer, "tp_rank", 0))
        row_parallel = self.k != self.full_k
        return rank, world, row_parallel

    def selected_rows(self, device, layer=None, weight=None):
        """Sorted fused-row ids of the MXFP8 channels of this rank's shard
        (reference: quantization.py:104-122, extended to TP shards and to selection rules)."""
        names = self.projection_names()
        if len(names) != len(self.parts):
            raise ValueError(f"Projection partition mismatch: {self.prefix}, {self.parts}")
        rank, world, row_parallel = self._tp(layer) if layer is not None else (0, 1, False)
        selection = self.config.selection
        if isinstance(selection, dict) and "rule" in selection:
            if selection["rule"] != "l2norm" or weight is None:
                raise ValueError(f"Unknown channel selection rule {selection.get('rule')}")
            group = None
            if row_parallel and world > 1:
                from vllm.distributed import get_tp_group
                group = get_tp_group().device_group
            rows, offset = [], 0
            for size in self.parts:
                part = weight[offset:offset + size]
                ids = tp.select_by_l2norm(part, float(selection["fraction"]), int(selection.get("multiple", 1)),
                                          group=group, row_parallel=row_parallel)
                rows.extend(i + offset for i in ids)
                offset += size
            return torch.tensor(sorted(rows), dtype=torch.long, device=device)
        if world == 1 or row_parallel:
            # Row-parallel shards keep every output channel, hence the whole selection.
            rows, offset = [], 0
            for name, size in zip(names, self.parts):
                if name not in selection:
                    raise ValueError(f"Missing channel selection for {name}")
                tp.validate_ids(selection[name], size, name)
                rows.extend(i + offset for i in selection[name])
                offset += size
            return torch.tensor(sorted(rows), dtype=torch.long, device=device)
        # Column-parallel: this rank's slice of every projection.
        replicas = int(getattr(layer, "num_kv_head_replicas", 1))
        shard_ranks, full_sizes = [], []
        for p, size in enumerate(self.parts):
            kv = len(names) == 3 and p > 0 and replicas > 1
            parts = world // replicas if kv else world
            shard_ranks.append((rank // replicas if kv else rank, parts))
            full_sizes.append(size * parts)
        rows = tp.column_parallel_rows(selection, names, full_sizes, rank, world, shard_ranks)
        return torch.tensor(rows, dtype=torch.long, device=device)

    # -- load time ------------------------------------------------------------------------------
    def process_weights_after_loading(self, layer):
        from .native import DualLinear
        weight = layer.weight.data.contiguous()
        ids = self.selected_rows(weight.device, layer, weight)
        self.runtime = DualLinear(weight, ids, self.config.low_id, self.config.high_id,
                                  self.config.concurrent, self.config.plans)
        self.runtime.layer_name = self.prefix
        rank, world, row_parallel = self._tp(layer)
        self.reduce_group = row_parallel and world > 1 and bool(getattr(layer, "reduce_results", True))
        del layer.weight
        self.handle = register_runtime(self.runtime)

    # -- forward --------------------------------------------------------------------------------
    def apply(self, layer, x, bias=None):
        lead = x.shape[:-1]
        y = linear(x.reshape(-1, self.k).contiguous(), self.handle, self.outputs)
        if bias is not None:
            y = y + bias
        return y.reshape(*lead, self.outputs)

    def reduce(self, y):
        """All-reduce of row-parallel partial sums for callers that bypass the layer's forward."""
        if getattr(self, "reduce_group", False):
            from vllm.distributed import tensor_model_parallel_all_reduce
            return tensor_model_parallel_all_reduce(y)
        return y


def model_audit(model):
    """Per-layer audit record (reference: quantization.py:161-170)."""
    layers = []
    for name, module in model.named_modules():
        method = getattr(module, "quant_method", None)
        if isinstance(method, MixedLinearMethod) and method.runtime is not None:
            r = method.runtime
            layers.append({"name": name, "kind": method.config.kind, "k": method.k, "outputs": method.outputs,
                           "high": r.hi.numel(), "low": r.lo.numel(), "calls_by_tokens": dict(r.calls),
                           "plans_used": dict(r.plans_used)})
    return layers
