"""ctypes binding of the CUDA library and the per-layer runtime (`DualLinear`).

Host-side mirror of the reference's `integrations/vllm/hygemm_vllm/native.py`:
same names (`Problem`, `library`, `check`, `pack`, `DualLinear`, `POLICIES`),
same argument meaning and the same errors, so code and tests written against
the reference read the same here.  PyTorch owns every tensor and supplies the
current stream; the native side borrows pointers.  There is no CPU path: if
the shared library is missing this module raises.

Differences, all additive: bfloat16 is accepted wherever the reference takes
IEEE half (the output of a layer has the dtype of the weights it was built
from), and both precision partitions run in ONE persistent tcgen05 launch.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch


class Problem(C.Structure):
    """`hg_problem` of include/hygemm.h (reference: native.py:7-9)."""
    _fields_ = [("rows", C.c_int), ("tokens", C.c_int), ("k", C.c_int), ("outputs", C.c_int),
                ("weight", C.c_void_p), ("activation", C.c_void_p), ("weight_scales", C.c_void_p),
                ("activation_scales", C.c_void_p), ("ids", C.c_void_p), ("output", C.c_void_p)]


PACK_MODE = int(os.environ.get("HYGEMM_PACK_MODE", "0"))
# Decode sizes (at most FUSED_QUANT_TOKENS tokens) quantise the activations inside the GEMM kernel
# (`hg_run_x`: one launch instead of two, identical bytes); HYGEMM_FUSED_QUANT=0 turns it off.
FUSED_QUANT_TOKENS = 16 if os.environ.get("HYGEMM_FUSED_QUANT", "1") != "0" else 0
# Every CTA quantises the K slice it multiplies, so the work repeats once per row tile; layers wider than this
# many output channels keep the separate quantiser launch (gate_up, 37888 wide, measured 30.8 us with its own
# quantiser launch against 36.3 us fused at 16 tokens; the narrow layers gain from the missing launch).
FUSED_QUANT_MAX_OUTPUTS = int(os.environ.get("HYGEMM_FUSED_QUANT_MAX_OUTPUTS", "8192"))
# Row-parallel exchange: up to this many tokens the partial sums cross NVLink as fp32 (rounded once after the sum).
FUSED_QUANT_TOKENS_F32 = 16
# Launch policies of hg_run (reference: native.py:14-15).
POLICIES = {"serial": 0, "concurrent": 1, "high_first": 2, "high_main": 3,
            "gemv_pair1": 4, "gemv_pair2": 5, "gemv_pair4": 6}
DTYPES = {torch.float16: 0, torch.bfloat16: 1}

_DEFAULT_LIBRARY = Path(__file__).resolve().parent.parent / "lib" / "libhygemm_b200.so"
_lib = None


def library_path() -> Path:
    return Path(os.environ.get("HYGEMM_LIBRARY", _DEFAULT_LIBRARY))


def library():
    """Load the shared library once and declare its prototypes (reference: native.py:19-32)."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise FileNotFoundError(f"HyGEMM CUDA library not found at {path}; build it with "
                                f"`python {_DEFAULT_LIBRARY.parent.parent / 'build.py'}` or set HYGEMM_LIBRARY")
    lib = C.CDLL(str(path))
    vp, ci = C.c_void_p, C.c_int
    pp = C.POINTER(Problem)
    lib.hg_last_error.restype = C.c_char_p
    lib.hg_scale_size.argtypes, lib.hg_scale_size.restype = [ci, ci], C.c_int64
    for name in ("hg_pack", "hg_pack_bf16"):
        getattr(lib, name).argtypes = [vp, vp, vp, ci, ci, ci, vp]
    for name in ("hg_pack_mode", "hg_pack_mode_bf16"):
        getattr(lib, name).argtypes = [vp, vp, vp, ci, ci, ci, vp, ci]
    for name in ("hg_silu_pack", "hg_silu_pack_bf16"):
        getattr(lib, name).argtypes = [vp, vp, vp, vp, ci, ci, vp, ci]
    lib.hg_create.argtypes = [ci, ci, pp, pp, vp, C.POINTER(vp)]
    lib.hg_create_dtype.argtypes = [ci, ci, pp, pp, vp, ci, C.POINTER(vp)]
    lib.hg_run.argtypes = [vp, pp, pp, vp, ci]
    lib.hg_run_x.argtypes = [vp, pp, pp, vp, ci, vp]
    lib.hg_info.argtypes = [vp, C.POINTER(ci)]
    lib.hg_status.argtypes = [vp, vp, C.POINTER(ci)]
    lib.hg_destroy.argtypes, lib.hg_destroy.restype = [vp], None
    lib.hg_plan.argtypes = [ci] * 6 + [C.POINTER(ci), C.POINTER(ci), ci]
    lib.hg_trace.argtypes = [vp, vp, C.POINTER(C.c_uint64), ci, C.POINTER(ci)]
    lib.hg_run_static.argtypes = [ci, pp, pp, vp, ci]
    lib.hg_static_status.argtypes = [vp, C.POINTER(ci)]
    lib.hg_run_partial.argtypes = [vp, pp, pp, vp, ci, vp, C.c_int64, ci, vp, vp]
    lib.hg_tp_allreduce.argtypes = [C.POINTER(vp), vp, C.c_int64, C.c_int64, ci, ci, ci, C.POINTER(vp), vp, ci, vp]
    lib.hg_tp_status.argtypes = [vp, vp, C.POINTER(ci)]
    lib.hg_fused_error.restype = C.c_char_p
    lib.hg_fused_create.argtypes = [ci, pp, pp, vp, C.POINTER(vp)]
    lib.hg_fused_create_dtype.argtypes = [ci, pp, pp, vp, ci, C.POINTER(vp)]
    lib.hg_fused_update.argtypes = [vp, pp, pp]
    lib.hg_fused_run.argtypes = [vp, vp]
    lib.hg_fused_info.argtypes = [vp, C.POINTER(ci)]
    lib.hg_fused_destroy.argtypes, lib.hg_fused_destroy.restype = [vp], None
    _lib = lib
    return lib


def check(status: int) -> None:
    """Raise the library's thread-local message on a non-zero status (reference: native.py:35-37)."""
    if status:
        raise RuntimeError(library().hg_last_error().decode())


def scale_size(rows: int, k: int) -> int:
    """Bytes of the padded scale buffer; the closed form of `hg_scale_size` (no foreign call on the hot path)."""
    return ((rows + 127) // 128) * (k // 128) * 512 if rows > 0 and k > 0 else 0


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def pack(x: torch.Tensor, fp4: bool = False):
    """Quantise `[rows,K]` fp16/bf16 to MX codes + padded E8M0 scales (reference: native.py:40-50).

    Returns `(q, sf)`: `q` is uint8 `[rows,K]` (E4M3) or `[rows,K/2]` (packed
    E2M1, even k in the low nibble); `sf` has `hg_scale_size(rows,K)` bytes with
    every padding byte 0x7f.  Zero rows give zero-length tensors and no launch.
    """
    if not (x.is_cuda and x.dtype in DTYPES and x.ndim == 2 and x.is_contiguous() and x.shape[1] % 128 == 0):
        raise ValueError("MX pack requires contiguous CUDA FP16/BF16 [rows,K], K divisible by 128")
    rows, k = x.shape
    q = torch.empty((rows, k // 2 if fp4 else k), dtype=torch.uint8, device=x.device)
    sf = torch.empty(scale_size(rows, k) if rows else 0, dtype=torch.uint8, device=x.device)
    if rows:
        lib = library()
        bf16 = x.dtype == torch.bfloat16
        args = (x.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, k, int(fp4), _stream(x.device))
        # HYGEMM_PACK_MODE keeps its reference meaning (3 = vector kernel from 16 rows);
        # every mode produces the same bytes.
        mode = (2 if rows >= 16 else 0) if PACK_MODE == 3 else PACK_MODE
        if mode:
            check((lib.hg_pack_mode_bf16 if bf16 else lib.hg_pack_mode)(*args, mode))
        else:
            check((lib.hg_pack_bf16 if bf16 else lib.hg_pack)(*args))
    return q, sf


class DualLinear:
    """One hybrid linear layer: FP4 rows + FP8 rows, packed once, run per call.

    Mirrors the reference class (native.py:53-116): `weight` is `[N,K]`,
    `high_ids` the output channels kept in MXFP8; the rest are MXFP4.
    Attributes read elsewhere: outputs, k, hi, lo, w4, sf4, w8, sf8, handles,
    fused_handles, calls, plans, plans_used, low_id, high_id, concurrent.
    """

    def __init__(self, weight, high_ids, low_id=0, high_id=0, concurrent=True, plans=None):
        if weight.ndim != 2 or weight.dtype not in DTYPES:
            raise ValueError("HyGEMM weights must be a CUDA FP16/BF16 [N,K] matrix")
        self.outputs, self.k = weight.shape
        self.dtype = weight.dtype
        selected = torch.zeros(self.outputs, dtype=torch.bool, device=weight.device)
        selected[high_ids] = True
        rows = torch.arange(self.outputs, device=weight.device)
        self.hi = rows[selected].to(torch.int32)
        self.lo = rows[~selected].to(torch.int32)
        self.w4, self.sf4 = pack(weight.index_select(0, self.lo.long()).contiguous(), True)
        self.w8, self.sf8 = pack(weight.index_select(0, self.hi.long()).contiguous(), False)
        # The GEMM starts reading weights before it waits for the kernel in front of it (programmatic
        # dependent launch), so the packed weights must be complete before the first call: load time only.
        torch.cuda.current_stream(weight.device).synchronize()
        self.low_id, self.high_id, self.concurrent = low_id, high_id, concurrent
        self.handles = {}
        self.fused_handles = {}
        self.calls = {}
        self.plans = plans
        self.plans_used = {}
        self._problems = {}

    def __call__(self, x):
        if x.ndim != 2 or x.shape[1] != self.k or x.device != self.w4.device:
            raise ValueError("HyGEMM input shape/device does not match its weights")
        if 0 < x.shape[0] <= FUSED_QUANT_TOKENS and x.dtype in DTYPES and x.is_contiguous() and not self.plans \
                and not 28 <= self.low_id <= 34 and self.outputs <= FUSED_QUANT_MAX_OUTPUTS:
            return self._run_fused(x)
        q, sf = pack(x)
        return self.run_packed(q, sf)

    def _run_fused(self, x):
        """Decode path: activation quantisation inside the GEMM launch (`hg_run_x`)."""
        tokens = x.shape[0]
        y = torch.empty((tokens, self.outputs), dtype=self.dtype, device=x.device)
        low, high, _, low_ref, high_ref = self._rebound(tokens, x, x, y)
        stream = _stream(x.device)
        handle = self._handle(tokens, self.low_id, self.high_id, low_ref, high_ref, stream)
        status = _lib.hg_run_x(handle, low_ref, high_ref, x.data_ptr(), DTYPES[x.dtype], stream)
        if status:
            check(status)
        self.calls[tokens] = self.calls.get(tokens, 0) + 1
        return y

    def _handle(self, tokens, low_id, high_id, low_ref, high_ref, stream):
        """GEMM handle of one (token count, schedule ids) pair, created on first use: never during stream
        capture, where an unseen shape is an error (reference: native.py:95-104)."""
        key = (tokens, low_id, high_id, self.lo.numel(), self.hi.numel())
        handle = self.handles.get(key)
        if handle is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"HyGEMM shape T={key} must be warmed before graph capture")
            handle = C.c_void_p()
            check(library().hg_create_dtype(low_id, high_id, low_ref, high_ref, stream, DTYPES[self.dtype], C.byref(handle)))
            self.handles[key] = handle
        return handle

    def problems(self, q, sf, y):
        """The two `Problem` structs of a call (shared activation, scales and output pointers)."""
        tokens = q.shape[0]
        low = Problem(self.lo.numel(), tokens, self.k, self.outputs, self.w4.data_ptr(), q.data_ptr(),
                      self.sf4.data_ptr(), sf.data_ptr(), self.lo.data_ptr(), y.data_ptr())
        high = Problem(self.hi.numel(), tokens, self.k, self.outputs, self.w8.data_ptr(), q.data_ptr(),
                       self.sf8.data_ptr(), sf.data_ptr(), self.hi.data_ptr(), y.data_ptr())
        return low, high

    def _rebound(self, tokens, q, sf, y):
        """Per-token-count `Problem` pair kept between calls; only the three per-call pointers change."""
        pair = self._problems.get(tokens)
        if pair is None or pair[2] != (self.w4.data_ptr(), self.sf4.data_ptr()):
            low, high = self.problems(q, sf, y)
            pair = self._problems[tokens] = (low, high, (self.w4.data_ptr(), self.sf4.data_ptr()),
                                             C.byref(low), C.byref(high))
            return pair
        qp, sp, yp = q.data_ptr(), sf.data_ptr(), y.data_ptr()
        for prob in pair[:2]:
            prob.activation, prob.activation_scales, prob.output = qp, sp, yp
        return pair

    def run_packed(self, q, sf):
        """GEMM on already-quantised activations (reference: native.py:75-107)."""
        if q.dtype != torch.uint8 or q.ndim != 2 or q.shape[1] != self.k or q.device != self.w4.device \
                or not q.is_contiguous():
            raise ValueError("Invalid prepacked MXFP8 activation")
        tokens = q.shape[0]
        if sf.dtype != torch.uint8 or sf.device != q.device or not sf.is_contiguous() \
                or sf.numel() != scale_size(tokens, self.k):
            raise ValueError("Invalid prepacked MXFP8 scale buffer")
        # Fresh output per call: under CUDA-graph capture the graph's pool owns it.
        y = torch.empty((tokens, self.outputs), dtype=self.dtype, device=q.device)
        if tokens == 0:
            return y
        low, high, _, low_ref, high_ref = self._rebound(tokens, q, sf, y)
        stream = _stream(q.device)
        low_id, high_id, policy = self.low_id, self.high_id, int(self.concurrent)
        if self.plans:
            plan = self.plans.get(self.outputs, self.k, self.hi.numel(), tokens)
            low_id, high_id, policy = plan["low_id"], plan["high_id"], POLICIES[plan["policy"]]
            self.plans_used[tokens] = [plan["tokens"], low_id, high_id, policy]
        handle = self._handle(tokens, low_id, high_id, low_ref, high_ref, stream)
        status = _lib.hg_run(handle, low_ref, high_ref, stream, policy)
        if status:
            check(status)
        self.calls[tokens] = self.calls.get(tokens, 0) + 1
        return y

    def run_exchange(self, exchange, x=None, q=None, sf=None):
        """Row-parallel shard: the GEMM writes its partial sums into this rank's peer-mapped exchange buffer and
        a second, small launch tells the peers, waits for them, pulls their partials over NVLink and adds them in
        rank order (`hg_run_partial` + `hg_tp_allreduce`).  Two launches on purpose: the GEMM's CTAs leave their
        SMs as soon as their tiles are stored, so the next GEMM in the stream starts streaming its weights while
        the exchange is still waiting for the peers (doing the exchange in the tail of the GEMM launch measured
        slower: 0.70 against 0.63 ms per step of the layer sweep on two GPUs).

        `exchange` is a `tp.PeerExchange`.  Pass 16-bit `x` (at most FUSED_QUANT_TOKENS tokens, quantised in the
        GEMM launch) or prepacked `(q, sf)`.  Returns the summed `[tokens, outputs]`, identical on every rank;
        a peer that never arrives turns it into NaN and leaves a status behind (`exchange.status()`).
        """
        fused = x is not None
        src = x if fused else q
        tokens = src.shape[0]
        if src.ndim != 2 or src.shape[1] != self.k or not src.is_contiguous() or tokens == 0:
            raise ValueError("HyGEMM input shape does not match its weights")
        if fused and not (tokens <= FUSED_QUANT_TOKENS and x.dtype in DTYPES):
            raise ValueError("Fused quantisation serves at most 16 tokens of FP16/BF16")
        if not fused and (sf is None or sf.numel() != scale_size(tokens, self.k)):
            raise ValueError("Invalid prepacked MXFP8 scale buffer")
        elems = tokens * self.outputs
        if elems * 2 > exchange.half_bytes or self.dtype != exchange.dtype or elems % 8:
            raise ValueError("Exchange buffers are too small or of another dtype")
        # Decode sizes exchange fp32 partial sums, so the result is rounded once instead of once per rank.
        f32 = int(tokens <= FUSED_QUANT_TOKENS_F32 and elems * 4 <= exchange.half_bytes)
        y = torch.empty((tokens, self.outputs), dtype=self.dtype, device=src.device)
        low, high, _, low_ref, high_ref = self._rebound(tokens, src, src if fused else sf, y)
        stream = _stream(src.device)
        handle = self._handle(tokens, self.low_id, self.high_id, low_ref, high_ref, stream)
        lib = library()
        check(lib.hg_run_partial(handle, low_ref, high_ref, x.data_ptr() if fused else None,
                                 DTYPES[x.dtype] if fused else 0, exchange.buffer.data_ptr(), exchange.half_bytes, f32,
                                 exchange.state.data_ptr(), stream))
        check(lib.hg_tp_allreduce(exchange.buffer_ptrs, y.data_ptr(), elems, exchange.half_bytes, f32, exchange.world,
                                  exchange.rank, exchange.flag_ptrs, exchange.state.data_ptr(), DTYPES[self.dtype], stream))
        self.calls[tokens] = self.calls.get(tokens, 0) + 1
        return y

    def info(self, tokens):
        """`hg_info` of the handle warmed for `tokens` (20 ints, 10 per partition)."""
        out = (C.c_int * 20)()
        for key, handle in self.handles.items():
            if key[0] == tokens:
                check(library().hg_info(handle, out))
                return list(out)
        raise KeyError(f"no handle warmed for {tokens} tokens")

    def status(self):
        """Sum of the device status words of every handle: (error, K128 blocks, units)."""
        total = [0, 0, 0]
        stream = _stream(self.w4.device)
        for handle in self.handles.values():
            out = (C.c_int * 3)()
            check(library().hg_status(handle, stream, out))
            total = [total[0] or out[0], total[1] + out[1], total[2] + out[2]]
        return tuple(total)

    def close(self):
        for handle in self.handles.values():
            library().hg_destroy(handle)
        self.handles.clear()
        for handle in self.fused_handles.values():
            library().hg_fused_destroy(handle)
        self.fused_handles.clear()
