"""Generate the golden fixtures in this directory.

Runs only where the reference checkout and the CUTLASS headers are present
(the build container); the fixtures it writes are committed and are what the
tests read.  Usage::

    python tests/golden/make_golden.py --reference /path/to/reference

Sources of truth, by fixture:

* ``decode_mx.npz``, ``reference_linear.npz`` — the reference's own PyTorch
  oracle (``integrations/vllm/test_components.py``: ``decode_mx`` and the
  dequantise-matmul expression of ``reference``), imported and run on CPU.
* ``codes_rne.npz`` — ``integrations/vllm/allocation/fp4_quant.py``
  (``codes_rne``, ``pack_codes``, ``decode_logical``) and the tie table of
  ``integrations/vllm/allocation/check_components.py:14``.
* ``scale_indices.npz`` — ``integrations/vllm/hygemm_vllm/offline_weights.py``
  (``scale_indices``).
* ``cutlass_codecs.npz`` — host conversions ``cutlass::float_e4m3_t(float)`` and
  ``cutlass::float_e2m1_t(float)`` (the third-party conversions the reference's
  CUDA quantiser calls) for every fp16 and bf16 bit pattern, produced by
  ``cutlass_codecs.cpp`` against the CUTLASS headers found in the container.

* ``clip_search.npz`` — the exponent search of
  ``integrations/vllm/allocation/fp4_quant.py:28-58`` (``quantize``).  That
  function itself asserts a CUDA tensor and calls the CUDA ``pack``, so it cannot
  run here; the fixture composes the reference's own CPU-runnable pieces
  (``unpack``, ``codes_rne``, ``pack_codes``, ``decode_logical``,
  ``offline_weights.logical_scales``) in the order ``quantize`` uses them, with
  the round-to-nearest baseline taken from this repository's oracle (whose
  quantiser is pinned by the codec fixtures).  Error sums are torch CPU
  reductions.

The quantised operands fed to ``reference_linear`` come from the CPU oracle of
this repository; the fixture pins the *decode and matmul* half against the
reference, the quantiser half is pinned by the codec fixtures.
"""
from __future__ import annotations

import argparse
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))


def cutlass_include() -> Path:
    import flashinfer
    return Path(flashinfer.__file__).parent / "data" / "cutlass" / "include"


def run_codec(binary: Path, kind: str, values: np.ndarray) -> np.ndarray:
    out = subprocess.run([str(binary), kind], input=values.astype(np.float32).tobytes(),
                         capture_output=True, check=True).stdout
    return np.frombuffer(out, dtype=np.uint8).copy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference checkout")
    args = ap.parse_args()
    ref = Path(args.reference) / "integrations" / "vllm"
    sys.path.insert(0, str(ref))
    import test_components as tc                      # noqa: E402  (reference code)
    from allocation import fp4_quant                  # noqa: E402
    from hygemm_vllm import offline_weights as ow     # noqa: E402
    import oracle                                     # noqa: E402  (this repository's CPU oracle)

    rng = np.random.default_rng(20261024)

    # ---- decode_mx -----------------------------------------------------------------
    dec = {}
    for rows, k in [(3, 128), (130, 256), (33, 896)]:
        for fp4 in (True, False):
            q = rng.integers(0, 256, size=(rows, k // 2 if fp4 else k), dtype=np.uint8)
            if not fp4:
                q[(q & 0x7f) == 0x7f] = 0x3c          # no NaN codes
            sf = rng.integers(96, 150, size=oracle.scale_size(rows, k), dtype=np.uint8)
            out = tc.decode_mx(torch.from_numpy(q), torch.from_numpy(sf), k, fp4).numpy()
            tag = f"r{rows}_k{k}_{'fp4' if fp4 else 'fp8'}"
            dec[tag + "_q"], dec[tag + "_sf"], dec[tag + "_out"] = q, sf, out.astype(np.float32)
    np.savez_compressed(HERE / "decode_mx.npz", **dec)

    # ---- FP4 RNE codes ---------------------------------------------------------------
    ties = [.25, .75, 1.25, 1.75, 2.5, 3.5, 5., 6.]
    table = np.array([0., -0.] + ties + [-t for t in ties], dtype=np.float32)
    halves = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
    halves = halves[np.isfinite(halves) & (np.abs(halves) <= 8)]
    rand = (rng.standard_normal(4096) * 3).astype(np.float32)
    values = np.concatenate([table, halves, rand]).astype(np.float32)
    values = values[: (values.size // 64) * 64].reshape(-1, 64)
    codes = fp4_quant.codes_rne(torch.from_numpy(values))
    packed = fp4_quant.pack_codes(codes)
    logical = rng.integers(120, 134, size=(values.shape[0], 2), dtype=np.uint8)
    decoded = fp4_quant.decode_logical(packed, torch.from_numpy(logical), 64).numpy()
    np.savez_compressed(HERE / "codes_rne.npz", values=values, codes=codes.numpy(), packed=packed.numpy(),
                        logical=logical, decoded=decoded.astype(np.float32))

    # ---- scale layout ----------------------------------------------------------------
    idx = {}
    for rows, k in [(1, 128), (129, 256), (257, 896), (486, 384)]:
        idx[f"r{rows}_k{k}"] = ow.scale_indices(rows, k, "cpu").numpy().astype(np.int64)
    np.savez_compressed(HERE / "scale_indices.npz", **idx)

    # ---- dequantise + matmul (reference()) ---------------------------------------------
    lin = {}
    torch.manual_seed(20261024)
    for outputs, k, high, tokens in [(257, 256, 26, 3), (257, 256, 0, 17), (257, 128, 257, 5), (300, 384, 40, 17)]:
        w = (torch.randn(outputs, k) * .04).bfloat16()
        x = torch.randn(tokens, k).bfloat16()
        ids = torch.randperm(outputs)[:high].numpy()
        lo, hi = oracle.partition(outputs, ids)
        w4, sf4 = oracle.pack(w[torch.from_numpy(lo).long()], fp4=True)
        w8, sf8 = oracle.pack(w[torch.from_numpy(hi).long()], fp4=False)
        xq, xsf = oracle.pack(x, fp4=False)
        dx = tc.decode_mx(torch.from_numpy(xq), torch.from_numpy(xsf), k, False)
        wd = torch.empty(outputs, k)
        wd[torch.from_numpy(lo).long()] = tc.decode_mx(torch.from_numpy(w4), torch.from_numpy(sf4), k, True)
        wd[torch.from_numpy(hi).long()] = tc.decode_mx(torch.from_numpy(w8), torch.from_numpy(sf8), k, False)
        y = dx @ wd.t()
        tag = f"o{outputs}_k{k}_h{high}_t{tokens}"
        for name, value in dict(w=oracle.as_u16(w), x=oracle.as_u16(x), lo=lo, hi=hi, w4=w4, sf4=sf4, w8=w8,
                                sf8=sf8, xq=xq, xsf=xsf, y=y.numpy().astype(np.float32),
                                y_half=oracle.as_u16(y.half()), y_bf16=oracle.as_u16(y.bfloat16())).items():
            lin[f"{tag}__{name}"] = value
    np.savez_compressed(HERE / "reference_linear.npz", **lin)

    # ---- offline exponent search (fp4_quant.quantize, composed from its CPU-runnable pieces) -----------
    clip = {}
    torch.manual_seed(20261024 + 7)
    for tag, rows, k, weighted, offsets in [("plain", 64, 256, False, (0, -1, -2)), ("weighted", 48, 384, True, (0, -1, -2)),
                                            ("up", 32, 128, False, (0, 1, -1)), ("heavy", 32, 256, True, (0, -1, -2, -3))]:
        w = (torch.randn(rows, k) * .05)
        w[torch.rand(rows, k) < .02] *= 12          # outliers, so that clipping sometimes wins
        w[0, :32] = 0                               # an all-zero group
        w = w.half()
        importance = (torch.rand(k) * 4).float() if weighted else None
        q, sf = oracle.pack(w, fp4=True, bf16=False)
        q, sf = torch.from_numpy(q), torch.from_numpy(sf)
        logical = ow.logical_scales(sf, rows, k)
        source = w.float().reshape(rows, k // 32, 32)
        weight = (torch.ones(k) if importance is None else importance).reshape(1, k // 32, 32)
        best_error = ((fp4_quant.decode_logical(q, logical, k).reshape_as(source) - source).square() * weight).sum(-1)
        best_codes, best_scale = fp4_quant.unpack(q).reshape(rows, k // 32, 32), logical.clone()
        for shift in offsets:
            if shift == 0:
                continue
            exponent = (logical.to(torch.int16) + shift).clamp(0, 254).to(torch.uint8)
            codes = fp4_quant.codes_rne(source / torch.exp2(exponent.float() - 127)[:, :, None])
            values = fp4_quant.decode_logical(fp4_quant.pack_codes(codes.reshape(rows, k)), exponent, k).reshape_as(source)
            error = ((values - source).square() * weight).sum(-1)
            better = error < best_error
            best_error = torch.where(better, error, best_error)
            best_codes = torch.where(better[:, :, None], codes, best_codes)
            best_scale = torch.where(better, exponent, best_scale)
        clip[tag + "__w"] = oracle.as_u16(w)
        clip[tag + "__importance"] = np.zeros(0, np.float32) if importance is None else importance.numpy()
        clip[tag + "__offsets"] = np.array(offsets, dtype=np.int32)
        clip[tag + "__q4"] = fp4_quant.pack_codes(best_codes.reshape(rows, k)).numpy()
        clip[tag + "__scales"] = best_scale.numpy()
        clip[tag + "__error"] = best_error.numpy().astype(np.float32)
    np.savez_compressed(HERE / "clip_search.npz", **clip)

    # ---- CUTLASS element conversions -----------------------------------------------------
    with tempfile.TemporaryDirectory() as tmp:
        binary = Path(tmp) / "cutlass_codecs"
        subprocess.run(["g++", "-O1", "-std=c++17", f"-I{cutlass_include()}", "-I/usr/local/cuda/include",
                        str(HERE / "cutlass_codecs.cpp"), "-o", str(binary)], check=True)
        all16 = np.arange(65536, dtype=np.uint16)
        half = all16.view(np.float16).astype(np.float32)
        bf = (all16.astype(np.uint32) << 16).view(np.float32)
        finite_h, finite_b = np.isfinite(half), np.isfinite(bf)
        out = dict(
            e4m3_from_half=run_codec(binary, "e4m3", np.where(finite_h, half, 0)),
            e4m3_from_bf16=run_codec(binary, "e4m3", np.where(finite_b, bf, 0)),
            e2m1_from_half=run_codec(binary, "e2m1", np.where(finite_h, half, 0)),
            e2m1_from_bf16=run_codec(binary, "e2m1", np.where(finite_b, bf, 0)),
        )
    np.savez_compressed(HERE / "cutlass_codecs.npz", **out)
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
