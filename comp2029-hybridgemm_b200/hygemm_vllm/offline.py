"""`hygemm_offline`: the hybrid layer with its MXFP4 rows taken from an offline bank.

Counterpart of the reference's `integrations/vllm/hygemm_vllm/offline.py` (loader) and
`allocation/build_banks.py` (bank writer).  Forward computation is the unchanged `DualLinear`; only the
stored MXFP4 codes and scales of the low partition are replaced at load time.

Bank format (kept from the reference so existing banks load): a folder with `manifest.json`
`{"mode", "format", "offsets", "layers": {unfused layer name: {"file", "sha256", "rows", "k", "stats"}},
"completed"}` and one `torch.save({"q4": [rows, K/2] uint8, "scales": [rows, K/32] uint8})` per layer.
`mode == "native_rtn"` banks must reproduce the load-time quantiser bit for bit and are verified against it.

Config keys next to those of `hygemm`: `q4_bank` (manifest path), `reference_plans` + `reference_cases`
(per-layer plan inheritance; both optional here, since plan files tuned for another GPU do not apply and the
library then chooses its own schedule), `decode_plans` (bound per-layer plans for at most 128 tokens).

Added over the reference: tensor-parallel shards read their slice of a bank entry (rows for column-parallel
layers, whole K128 blocks of codes and scales for row-parallel ones).
"""
from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path
from typing import Mapping

import torch
from vllm.model_executor.layers.linear import LinearBase, UnquantizedLinearMethod
from vllm.model_executor.layers.quantization import register_quantization_config

from .offline_weights import replace_low_weight
from .plans import PlanTable
from .quantization import HyGEMMConfig, MixedLinearMethod

BANK_FORMAT = "E2M1 packed nibbles + logical K32 E8M0 scales"
# Runtime switches a bound decode plan may pin, with their defaults (reference: offline.py:46-50).
_OPTION_DEFAULTS = {"HYGEMM_PACK_MODE": "0", "HYGEMM_FUSE_SILU": "0", "HYGEMM_SILU_MATH": "0",
                    "HYGEMM_ROW_ORDER": "none", "HYGEMM_FUSED_GATEUP": "0", "HYGEMM_FUSE_LLAMA": "0"}


def file_sha256(path) -> str:
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


def build_bank(folder, weights: Mapping[str, torch.Tensor], mode: str = "mse_clip",
               moments: Mapping[str, torch.Tensor] | None = None, offsets=None, chunk_rows: int = 4096) -> Path:
    """Quantise every `[rows, K]` weight of `weights` (unfused layer names) into a bank under `folder`.

    `native_rtn` stores the round-to-nearest result, `mse_clip` searches exponent offsets (0,-1,-2) for the
    plain squared error, `act_mse_clip` weights the error by `moments[name]` (second moment of each input
    channel).  Returns the manifest path.  (reference: allocation/build_banks.py:39-71)
    """
    from .fp4_quant import quantize
    if mode not in ("native_rtn", "mse_clip", "act_mse_clip"):
        raise ValueError(f"Unknown bank mode {mode}")
    if mode == "act_mse_clip" and moments is None:
        raise ValueError("act_mse_clip needs per-layer input moments")
    offsets = tuple(offsets) if offsets is not None else ((0,) if mode == "native_rtn" else (0, -1, -2))
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    manifest = {"mode": mode, "format": BANK_FORMAT, "offsets": list(offsets), "layers": {}, "completed": False,
                "activation_unchanged": True, "fp8_weight_unchanged": True}
    keys = ("groups", "weighted_error_before", "weighted_error_after", "weight_error_before", "weight_error_after")
    for name, weight in weights.items():
        codes, scales, totals, shifts = [], [], dict.fromkeys(keys, 0), {}
        importance = moments[name] if mode == "act_mse_clip" else None
        for start in range(0, weight.shape[0], chunk_rows):
            q, s, stats = quantize(weight[start:start + chunk_rows].cuda(), importance, offsets)
            codes.append(q.cpu())
            scales.append(s.cpu())
            for key in keys:
                totals[key] += stats[key]
            for shift, count in stats["shift_groups"].items():
                shifts[shift] = shifts.get(shift, 0) + count
        path = folder / f"{name}.pt"
        torch.save({"q4": torch.cat(codes), "scales": torch.cat(scales)}, path)
        manifest["layers"][name] = {"file": path.name, "sha256": file_sha256(path), "rows": weight.shape[0],
                                    "k": weight.shape[1], "stats": {**totals, "shift_groups": shifts}}
    manifest["completed"] = True
    target = folder / "manifest.json"
    target.write_text(json.dumps(manifest, indent=1, sort_keys=True))
    return target


def read_bank_entry(manifest: dict, folder: Path, name: str):
    """`(q4, scales)` of one unfused layer, after checking the file against the manifest's digest."""
    spec = manifest["layers"][name]
    path = folder / spec["file"]
    if file_sha256(path) != spec["sha256"]:
        raise ValueError(f"FP4 bank file for {name} does not match its manifest")
    entry = torch.load(path, map_location="cpu", weights_only=True)
    return entry["q4"], entry["scales"]


class InheritedLayerPlans:
    """Plan lookup of one layer whose high-partition width differs from the tuned one: it keeps the tuned
    layer's schedule choice (looked up with the tuned width); a bound per-layer decode plan, if present,
    takes over up to 128 tokens.  No fallback for shapes that were never tuned.  (reference: offline.py:16-27)"""

    def __init__(self, base, reference, actual, override=None):
        self.base, self.reference, self.actual, self.override = base, reference, actual, override

    def get(self, outputs, k, high, tokens):
        if (outputs, k, high) != self.actual:
            raise ValueError(f"Plan lookup for {(outputs, k, high)} on a layer of shape {self.actual}")
        if self.override is not None and tokens <= 128:
            return self.override.get_layer(self.reference["layer"], outputs, k, high, tokens)
        return self.base.get(outputs, k, self.reference["high"], tokens)


@register_quantization_config("hygemm_offline")
class OfflineConfig(HyGEMMConfig):
    kind = "hygemm"

    def __init__(self, config):
        super().__init__({key: value for key, value in config.items() if key != "tuning_plan"})
        self.reference_plans = PlanTable(config["reference_plans"], "hygemm") if config.get("reference_plans") else None
        self.reference_layers = {}
        if config.get("reference_cases"):
            cases = json.loads(Path(config["reference_cases"]).read_text())
            self.reference_layers = {row["layer"]: row for row in cases["layers"]}
        self.bank_path = Path(config["q4_bank"]) if config.get("q4_bank") else None
        self.bank = json.loads(self.bank_path.read_text()) if self.bank_path else None
        self.decode_plans = PlanTable(config["decode_plans"], "hygemm") if config.get("decode_plans") else None
        if self.decode_plans is not None and self.decode_plans.binding:
            self._check_binding(config, self.decode_plans.binding)

    def _check_binding(self, config, binding):
        """A bound decode plan applies only to the selection, bank, runtime switches and libraries it was
        tuned with (reference: offline.py:40-58)."""
        canonical = json.dumps(config["selection"], sort_keys=True, separators=(",", ":")).encode()
        if hashlib.sha256(canonical).hexdigest() != binding["selection_canonical_sha256"]:
            raise ValueError("Tuning plan is bound to a different channel selection")
        if self.bank_path is None or file_sha256(self.bank_path) != binding["bank_manifest_sha256"]:
            raise ValueError("Tuning plan is bound to a different FP4 bank")
        for name, value in binding.get("runtime_options", {}).items():
            if name not in _OPTION_DEFAULTS or os.environ.get(name, _OPTION_DEFAULTS[name]) != str(value):
                raise ValueError(f"Tuning plan runtime option mismatch: {name}")
        for key, variable in (("producer_sha256", "HYGEMM_PRODUCER_LIBRARY"), ("fused_sha256", "HYGEMM_FUSED_LIBRARY")):
            if binding.get(key):
                from .native import library_path
                path = Path(os.environ[variable]) if variable in os.environ else library_path()
                if file_sha256(path) != binding[key]:
                    raise ValueError(f"Tuning plan is bound to a different {key}")

    @classmethod
    def get_name(cls):
        return "hygemm_offline"

    def get_quant_method(self, layer, prefix):
        if isinstance(layer, LinearBase):
            return UnquantizedLinearMethod() if prefix.endswith("lm_head") else OfflineLinearMethod(self, prefix)
        return None


class OfflineLinearMethod(MixedLinearMethod):
    def _bank_rows(self, layer, runtime):
        """Codes and scales of this rank's fused rows, cut from the bank entries of the unfused projections."""
        rank, world, row_parallel = self._tp(layer)
        replicas = int(getattr(layer, "num_kv_head_replicas", 1))
        names = self.projection_names()
        codes, scales = [], []
        for p, (name, rows) in enumerate(zip(names, self.parts)):
            q4, sf = read_bank_entry(self.config.bank, self.config.bank_path.parent, name)
            if row_parallel and world > 1:
                begin = rank * runtime.k                     # K shards are equal whole K128 blocks
                q4, sf = q4[:, begin // 2:(begin + runtime.k) // 2], sf[:, begin // 32:(begin + runtime.k) // 32]
            elif world > 1:
                kv = len(names) == 3 and p > 0 and replicas > 1
                shard = rank // replicas if kv else rank
                q4, sf = q4[shard * rows:(shard + 1) * rows], sf[shard * rows:(shard + 1) * rows]
            if q4.shape != (rows, runtime.k // 2) or sf.shape != (rows, runtime.k // 32):
                raise ValueError(f"FP4 bank entry of {name} does not fit a [{rows}, {runtime.k}] shard")
            codes.append(q4)
            scales.append(sf)
        return torch.cat(codes), torch.cat(scales)

    def process_weights_after_loading(self, layer):
        super().process_weights_after_loading(layer)
        runtime = self.runtime
        if os.environ.get("HYGEMM_ROW_ORDER", "none") != "none":
            raise ValueError("Row reordering of gate_up is not available in this library")
        reference = self.config.reference_layers.get(self.prefix)
        if self.config.reference_plans is not None:
            if reference is None or (reference["out"], reference["k"]) != (runtime.outputs, runtime.k):
                raise ValueError(f"No reference case for {self.prefix} with shape {(runtime.outputs, runtime.k)}")
            runtime.plans = InheritedLayerPlans(self.config.reference_plans, reference,
                                                (runtime.outputs, runtime.k, runtime.hi.numel()), self.config.decode_plans)
        if self.config.bank is None or not runtime.lo.numel():
            return
        q4, scales = self._bank_rows(layer, runtime)
        replace_low_weight(runtime, q4, scales, verify_native=self.config.bank["mode"] == "native_rtn")
