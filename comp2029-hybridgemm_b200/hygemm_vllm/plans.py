"""Offline tuning plans: exact (N, K, H) key, ceiling token bucket.

Mirror of the reference's `integrations/vllm/hygemm_vllm/plans.py`.  A plan
file is JSON `{"hygemm": [{"out","k","high","tokens","low_id","high_id",
"policy"}, ...], "layer_plans": [...], "binding": {...}}`; `low_id`/`high_id`
are schedule ids of this library (include/hygemm.h), `policy` a key of
`native.POLICIES`.
"""
from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path

LAYOUT = "MX K32 E8M0 native physical scales v1"


def _bucketed(rows, what):
    table = {}
    for row in rows:
        table.setdefault(what(row), []).append(row)
    for bucket in table.values():
        bucket.sort(key=lambda r: r["tokens"])
        tokens = [r["tokens"] for r in bucket]
        if len(set(tokens)) != len(tokens):
            raise ValueError("Duplicate tuning bucket")
    return table


class PlanTable:
    def __init__(self, path, kind):
        document = json.loads(Path(path).read_text())
        self.binding = document.get("binding")
        if self.binding:
            # A bound plan only applies to the binary and scale layout it was tuned on
            # (reference: plans.py:9-19).
            variable = "HYGEMM_LIBRARY" if kind == "hygemm" else "MIXLLM_LIBRARY"
            if variable in os.environ:
                library = os.environ[variable]
            elif kind == "hygemm":
                from .native import library_path
                library = library_path()
            else:
                raise KeyError(variable)
            digest = hashlib.sha256(Path(library).read_bytes()).hexdigest()
            if digest != self.binding["library_sha256"]:
                raise ValueError("Tuning plan is bound to a different binary")
            if kind == "hygemm" and self.binding["layout"] != LAYOUT:
                raise ValueError("Unknown tuning-plan quantization layout")
        self.rows = _bucketed(document[kind], lambda r: (r["out"], r["k"], r["high"]))
        self.layer_rows = _bucketed(document.get("layer_plans", []), lambda r: r["layer"])

    def get(self, outputs, k, high, tokens):
        key = (outputs, k, high)
        if key not in self.rows:
            raise ValueError(f"Missing tuned shape {key}")
        for row in self.rows[key]:
            if row["tokens"] >= tokens:
                return row
        raise ValueError(f"Token count {tokens} exceeds tuned buckets for {key}")

    def get_layer(self, name, outputs, k, high, tokens):
        if not self.layer_rows:
            return self.get(outputs, k, high, tokens)
        if name not in self.layer_rows:
            raise ValueError(f"Missing tuned layer {name}")
        for row in self.layer_rows[name]:
            if (row["out"], row["k"], row["high"]) != (outputs, k, high):
                raise ValueError(f"Changed tuned shape for {name}")
            if row["tokens"] >= tokens:
                return row
        raise ValueError(f"Token count exceeds layer buckets for {name}")
