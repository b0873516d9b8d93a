"""Host-side logic and the C ABI surface (no GPU): exported symbols, tile schedules, plan tables,
scale-layout helpers, tensor-parallel shard arithmetic."""
import ctypes as C
import json
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from hygemm_vllm import native, offline_weights, plans, tp

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "hygemm.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hg_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = native.library()
    names = declared_symbols()
    assert {"hg_pack", "hg_pack_mode", "hg_scale_size", "hg_create", "hg_run", "hg_info", "hg_destroy",
            "hg_last_error", "hg_silu_pack", "hg_fused_create", "hg_fused_run", "hg_fused_update",
            "hg_fused_info", "hg_fused_destroy", "hg_fused_error"} <= set(names)      # the reference's ABI
    for name in names:
        assert hasattr(lib, name), name


def test_problem_struct_matches_header_layout():
    assert C.sizeof(native.Problem) == 4 * 4 + 6 * 8
    assert [f[0] for f in native.Problem._fields_] == ["rows", "tokens", "k", "outputs", "weight", "activation",
                                                       "weight_scales", "activation_scales", "ids", "output"]


def test_scale_size_and_argument_errors_without_gpu():
    lib = native.library()
    for rows, k in [(1, 128), (128, 128), (129, 256), (486, 896), (37888, 3584)]:
        assert lib.hg_scale_size(rows, k) == oracle.scale_size(rows, k) == offline_weights.scale_size(rows, k)
    assert lib.hg_scale_size(0, 128) == 0
    assert lib.hg_pack(None, None, None, 4, 128, 0, None) == -1
    assert lib.hg_last_error() == b"Invalid MX pack arguments"
    assert lib.hg_pack_bf16(None, None, None, 4, 100, 0, None) == -1
    assert lib.hg_silu_pack(None, None, None, None, 4, 128, None, 0) == 1
    assert lib.hg_silu_pack_bf16(None, None, None, None, 4, 128, None, 5) == 1
    handle = C.c_void_p()
    empty = native.Problem()
    assert lib.hg_create(0, 0, C.byref(empty), C.byref(empty), None, C.byref(handle)) == -1
    assert b"at least one weight row" in lib.hg_last_error()
    assert lib.hg_run(None, C.byref(empty), C.byref(empty), None, 0) == -1
    count = C.c_int(0)
    assert lib.hg_trace(None, None, (C.c_uint64 * 16)(), 16, C.byref(count)) == -1     # diagnostic entry point
    assert lib.hg_last_error() == b"Invalid hg_trace arguments"


def plan(lo, hi, tokens, k, schedule=0, sms=148):
    lib = native.library()
    header = (C.c_int * 12)()
    native.check(lib.hg_plan(lo, hi, tokens, k, sms, schedule, header, None, 0))
    units = (C.c_int * (9 * header[9]))()
    native.check(lib.hg_plan(lo, hi, tokens, k, sms, schedule, header, units, header[9]))
    return list(header), np.array(units[:], dtype=np.int64).reshape(-1, 9)


SHAPES = [(4096, 512, 3584), (3200, 384, 3584), (34048, 3840, 3584), (3200, 384, 18944), (4378, 486, 896),
          (257, 0, 256), (0, 257, 256), (1, 1, 128), (129, 127, 384)]


def test_data_parallel_ctas_run_their_mxfp8_tiles_first():
    """An MXFP8 tile scatters to channels all over the output row; first in its CTA, that epilogue runs under
    the next unit's main loop instead of ending the CTA."""
    lo, hi, k = 34048, 3840, 3584
    tiles_low = lo // 128
    for tokens in (16, 128, 300):
        header, units = plan(lo, hi, tokens, k, schedule=1)
        per_cta = {}
        for cta, tile, *_ in units:
            per_cta.setdefault(int(cta), []).append(int(tile) >= tiles_low)
        assert any(any(flags) for flags in per_cta.values())
        for flags in per_cta.values():
            assert flags == sorted(flags, reverse=True)     # every MXFP8 unit precedes every MXFP4 unit


@pytest.mark.parametrize("schedule", [0, 1, 2, 3])
@pytest.mark.parametrize("tokens", [1, 16, 17, 128, 130, 300])
def test_every_schedule_covers_each_tile_and_k_block_exactly_once(schedule, tokens):
    for lo, hi, k in SHAPES:
        for sms in (148, 7):
            header, units = plan(lo, hi, tokens, k, schedule, sms)
            sched, grid, n_tile, token_tiles, stages, smem, tmem, slots, counters, n_units, reduce2, issuers = header
            assert reduce2 == int(n_tile >= 64 and slots > 0)
            # up to 64 tokens the issuers own alternate stages (depth a multiple of their count); wider tiles
            # have two issuers that both read every stage, one K128 block each, so any depth works
            assert (issuers == 2 and stages >= 2) if n_tile > 64 else stages % issuers == 0
            assert 1 <= grid <= sms and n_tile % 16 == 0 and 16 <= n_tile <= 128
            # several token tiles only with 128-token tiles, or two 64-token tiles for 65..128 tokens on a
            # layer with few row tiles (the activation scale columns of a tile start on an even TMEM column)
            assert token_tiles == -(-tokens // n_tile) and (token_tiles == 1 or n_tile == 128 or (n_tile == 64 and token_tiles == 2))
            if 64 < tokens <= 128:
                assert n_tile == (64 if 2 * (-(-lo // 128) + -(-hi // 128)) <= sms else 128 if tokens == 128 else -(-tokens // 16) * 16)
            assert stages >= 2 and smem <= 232448 and tmem in (32, 64, 128, 256, 512)
            tiles = -(-lo // 128) + -(-hi // 128)
            kblocks = k // 128
            cover = {}
            for cta, tile, tt, b, e, split, nsplit, slot, counter in units:
                assert 0 <= cta < grid and 0 <= tile < tiles and 0 <= tt < token_tiles and 0 <= b < e <= kblocks
                cover.setdefault((tile, tt), []).append((b, e, split, nsplit, slot, counter))
            assert len(cover) == tiles * token_tiles
            used_slots, used_counters = set(), set()
            for pieces in cover.values():
                pieces.sort()
                assert pieces[0][0] == 0 and pieces[-1][1] == kblocks
                assert all(pieces[i][1] == pieces[i + 1][0] for i in range(len(pieces) - 1))
                assert [p[2] for p in pieces] == list(range(len(pieces)))         # split index follows K order
                assert all(p[3] == len(pieces) for p in pieces)
                if len(pieces) > 1:
                    assert len({(p[4], p[5]) for p in pieces}) == 1
                    slot, counter = pieces[0][4], pieces[0][5]
                    rng = set(range(slot, slot + len(pieces)))
                    assert not (rng & used_slots) and counter not in used_counters and max(rng) < slots
                    used_slots |= rng
                    used_counters.add(counter)
                    assert counter < counters
            assert np.all(np.diff(units[:, 0]) >= 0)                               # units listed CTA by CTA


def test_stream_k_balances_the_7b_decode_shapes():
    for lo, hi, k in SHAPES[:4]:
        header, units = plan(lo, hi, 1, k, 3)
        tiles_low = -(-lo // 128)
        cost = np.where(units[:, 1] < tiles_low, 1, 2) * (units[:, 4] - units[:, 3])
        load = np.bincount(units[:, 0], weights=cost, minlength=header[1])
        assert load.max() <= load.mean() + 4.5


def test_plan_table(tmp_path):
    rows = [{"out": 4608, "k": 3584, "high": 512, "tokens": t, "low_id": i, "high_id": i, "policy": "serial"}
            for i, t in enumerate([1, 16, 128])]
    path = tmp_path / "plan.json"
    path.write_text(json.dumps({"hygemm": rows}))
    table = plans.PlanTable(path, "hygemm")
    assert table.get(4608, 3584, 512, 1)["low_id"] == 0
    assert table.get(4608, 3584, 512, 2)["tokens"] == 16                       # ceiling bucket
    assert table.get(4608, 3584, 512, 128)["low_id"] == 2
    with pytest.raises(ValueError, match="exceeds tuned buckets"):
        table.get(4608, 3584, 512, 129)
    with pytest.raises(ValueError, match="Missing tuned shape"):
        table.get(4608, 3584, 384, 1)
    path.write_text(json.dumps({"hygemm": rows + [rows[0]]}))
    with pytest.raises(ValueError, match="Duplicate"):
        plans.PlanTable(path, "hygemm")
    # binding to another binary / layout is refused (performance/check_binding.py of the reference)
    import hashlib
    digest = hashlib.sha256(native.library_path().read_bytes()).hexdigest()
    path.write_text(json.dumps({"hygemm": rows, "binding": {"library_sha256": digest, "layout": plans.LAYOUT}}))
    plans.PlanTable(path, "hygemm")
    path.write_text(json.dumps({"hygemm": rows, "binding": {"library_sha256": "0" * 64, "layout": plans.LAYOUT}}))
    with pytest.raises(ValueError, match="different binary"):
        plans.PlanTable(path, "hygemm")
    path.write_text(json.dumps({"hygemm": rows, "binding": {"library_sha256": digest, "layout": "other"}}))
    with pytest.raises(ValueError, match="layout"):
        plans.PlanTable(path, "hygemm")
    layer_rows = [dict(r, layer="model.layers.0.self_attn.qkv_proj") for r in rows]
    path.write_text(json.dumps({"hygemm": rows, "layer_plans": layer_rows}))
    table = plans.PlanTable(path, "hygemm")
    assert table.get_layer("model.layers.0.self_attn.qkv_proj", 4608, 3584, 512, 5)["tokens"] == 16
    with pytest.raises(ValueError, match="Missing tuned layer"):
        table.get_layer("other", 4608, 3584, 512, 5)


def test_scale_layout_helpers_round_trip(golden):
    g = golden("scale_indices.npz")
    for key in g.files:
        rows, k = (int(s[1:]) for s in key.split("_"))
        assert np.array_equal(offline_weights.scale_indices(rows, k, "cpu").numpy(), g[key])
        logical = torch.randint(0, 255, (rows, k // 32), dtype=torch.uint8)
        physical = offline_weights.physical_scales(logical, k)
        assert physical.numel() == oracle.scale_size(rows, k)
        assert torch.equal(offline_weights.logical_scales(physical, rows, k), logical)
        valid = torch.zeros(physical.numel(), dtype=torch.bool)
        valid[torch.from_numpy(g[key]).flatten()] = True
        assert torch.all(physical[~valid] == 127)


def test_column_parallel_selection_matches_global_selection():
    rng = np.random.default_rng(3)
    names = ["l.q_proj", "l.k_proj", "l.v_proj"]
    sizes = [3584, 512, 512]
    selection = {n: sorted(rng.choice(s, s // 10, replace=False).tolist()) for n, s in zip(names, sizes)}
    for world in (1, 2, 4, 8):
        seen = {n: [] for n in names}
        for rank in range(world):
            rows = tp.column_parallel_rows(selection, names, sizes, rank, world)
            assert rows == sorted(rows)
            offset = 0
            for n, s in zip(names, sizes):
                step = s // world
                local = [r - offset for r in rows if offset <= r < offset + step]
                seen[n] += [i + rank * step for i in local]
                offset += step
        assert {n: sorted(v) for n, v in seen.items()} == selection
    # replicated KV heads: 4 shards of k/v served to 8 ranks
    rows = tp.column_parallel_rows(selection, names, sizes, 5, 8, [(5, 8), (2, 4), (2, 4)])
    q_local = [r for r in rows if r < 448]
    assert q_local == [i - 5 * 448 for i in selection["l.q_proj"] if 5 * 448 <= i < 6 * 448]
    with pytest.raises(ValueError, match="Missing channel selection"):
        tp.column_parallel_rows({}, names, sizes, 0, 2)
    with pytest.raises(ValueError, match="Invalid channel map"):
        tp.column_parallel_rows({n: [0, 0] for n in names}, names, sizes, 0, 2)


def test_row_parallel_shards_and_l2norm_rule():
    assert tp.row_parallel_k(4096, 3, 8) == (1536, 2048)
    with pytest.raises(ValueError):
        tp.row_parallel_k(3584, 0, 8)                                              # 448 is not a multiple of 128
    w = torch.randn(1280, 256)
    w[[5, 17, 900]] *= 10
    ids = tp.select_by_l2norm(w, 0.1, 128)
    assert len(ids) == 128 and {5, 17, 900} <= set(ids) and ids == sorted(ids)
    assert tp.select_by_l2norm(w, 0.0) == []


def test_exchange_arguments_are_checked():
    """hg_run_partial / hg_tp_allreduce refuse bad arguments before touching a device."""
    lib = native.library()
    ptrs = (C.c_void_p * 2)(16, 16)
    assert lib.hg_tp_allreduce(None, None, 8, 16, 0, 2, 0, ptrs, None, 1, None) == -1
    assert lib.hg_tp_allreduce(ptrs, 16, 12, 32, 0, 2, 0, ptrs, 16, 1, None) == -1
    assert b"multiple of 8" in lib.hg_last_error()
    assert lib.hg_tp_allreduce(ptrs, 16, 8, 16, 1, 2, 0, ptrs, 16, 1, None) == -1      # 8 fp32 values do not fit 16 bytes
    assert lib.hg_tp_allreduce(ptrs, 16, 8, 16, 0, 9, 0, ptrs, 16, 1, None) == -1
    assert lib.hg_run_partial(None, None, None, None, 0, None, 16, 0, None, None) == -1


def test_gemm_arguments_are_checked_on_every_policy():
    """A null or misaligned pointer is an error on the SIMT policies too, never a launch (no GPU needed: the
    check runs before anything is enqueued; the handle itself needs a device, so only hg_run_static is used)."""
    lib = native.library()
    bad = native.Problem(128, 4, 256, 128, None, None, None, None, None, None)
    assert lib.hg_run_static(0, C.byref(bad), C.byref(bad), None, 1) == -1
    assert b"Null pointer" in lib.hg_last_error() or b"share" in lib.hg_last_error()
    odd = native.Problem(128, 4, 256, 128, 64, 24, 64, 64, 64, 64)       # activation codes not 16-byte aligned
    none = native.Problem(0, 4, 256, 128, None, None, None, None, None, None)
    assert lib.hg_run_static(0, C.byref(odd), C.byref(none), None, 1) == -1
    assert b"aligned" in lib.hg_last_error()
    assert lib.hg_static_status(None, None) == -1


def test_tuner_candidates_and_plan_binding(tmp_path):
    """The tuner's search space and the bound plan document (no GPU): schedules 1-3, the SIMT pair policies up
    to four tokens, and a binding that `PlanTable` accepts for this library and refuses for another."""
    from hygemm_vllm import tune
    assert [c["low_id"] for c in tune.candidates(16)] == [1, 2, 3]
    small = tune.candidates(4)
    assert [c["policy"] for c in small[3:]] == ["gemv_pair1", "gemv_pair2", "gemv_pair4"] and all(c["low_id"] == 28 for c in small[3:])
    rows = [{"out": 640, "k": 512, "high": 64, "tokens": t, "low_id": 3, "high_id": 3, "policy": "serial"} for t in (8, 128)]
    document = tune.bind(rows)
    assert document["binding"]["layout"] == plans.LAYOUT and len(document["binding"]["library_sha256"]) == 64
    path = tmp_path / "plan.json"
    path.write_text(json.dumps(document))
    table = plans.PlanTable(path, "hygemm")
    assert table.get(640, 512, 64, 9)["tokens"] == 128 and table.get(640, 512, 64, 1)["tokens"] == 8
    with pytest.raises(ValueError, match="exceeds tuned buckets"):
        table.get(640, 512, 64, 129)
    other = tmp_path / "other.so"
    other.write_bytes(b"not this library")
    path.write_text(json.dumps(tune.bind(rows, other)))
    with pytest.raises(ValueError, match="different binary"):
        plans.PlanTable(path, "hygemm")
