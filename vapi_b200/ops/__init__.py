"""The kernels of the package as Python functions over torch tensors.

Every function here launches hand-written CUDA for sm_100a from ``vapi_b200/csrc`` on the
current torch stream (``linear`` alone is a library matrix product, as in the reference,
which calls cuBLAS through candle for every projection).  There is no CPU path: a tensor
that is not on a CUDA device is refused, and a missing or unbuildable extension raises.

Activation tensors are float32 (the true 32-bit path) or bfloat16 (the serving path); the
residual stream is always float32; small parameter vectors (norm weights, biases, conv
taps) are always float32.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Dict, Optional, Tuple

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_libs: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
loaded_libraries: Dict[str, str] = {}


class KernelError(RuntimeError):
    pass


def _lib(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _libs.get(name)
        if lib is None:
            path = _build.build(name)
            lib = ctypes.CDLL(path)
            lib.vapi_last_error.restype = ctypes.c_char_p
            _libs[name] = lib
            loaded_libraries[name] = path
            if _trace is not None:
                _trace_attach(name, lib)
    return lib


# ---- time stamps from inside captured graphs (a build with VAPI_NVCC_FLAGS=-DVAPI_TRACE) ----------
_trace: Optional[Tuple[torch.Tensor, torch.Tensor, Dict[str, int]]] = None


def _trace_attach(name: str, lib: ctypes.CDLL) -> None:
    buf, count, ids = _trace
    if not hasattr(lib, "vapi_trace_set"):
        raise KernelError(f"lib{name} was built without -DVAPI_TRACE (set VAPI_NVCC_FLAGS before the first import)")
    ids.setdefault(name, len(ids))
    rc = lib.vapi_trace_set(ctypes.c_void_p(buf.data_ptr()), ctypes.c_void_p(count.data_ptr()), buf.numel() // 2, ids[name])
    if rc != 0:
        raise KernelError(lib.vapi_last_error().decode(errors="replace"))


def trace_start(capacity: int = 1 << 16, device: str = "cuda") -> None:
    """Start collecting the kernels' own time stamps (first block's start, return of its dependency
    wait): every library loaded from now on, and those loaded already, writes into one buffer."""
    global _trace
    buf = torch.zeros(2 * capacity, dtype=torch.int64, device=device)
    count = torch.zeros(1, dtype=torch.int32, device=device)
    _trace = (buf, count, {})
    for name, lib in list(_libs.items()):
        if name != "host":
            _trace_attach(name, lib)


def trace_read() -> list:
    """The stamps so far, in time order: dicts with ``ns``, ``kind`` ("start" | "released"), ``library``,
    ``threads`` and ``blocks`` of the kernel that wrote them."""
    if _trace is None:
        raise KernelError("trace_start() was not called")
    buf, count, ids = _trace
    torch.cuda.synchronize()
    n = min(int(count.item()), buf.numel() // 2)
    raw = buf[:2 * n].cpu().tolist()
    names = {v: k for k, v in ids.items()}
    out = []
    for i in range(n):
        t, meta = raw[2 * i], raw[2 * i + 1]
        out.append({"ns": t, "kind": "start" if (meta & 15) == 0 else "released", "library": names.get((meta >> 4) & 15, "?"),
                    "threads": (meta >> 8) & 0xffff, "blocks": meta >> 24})
    out.sort(key=lambda e: e["ns"])
    return out


#: how many of this package's own kernels have been launched (library products not counted)
launch_count = 0


def _check(lib: ctypes.CDLL, rc: int, launches: int = 1) -> None:
    global launch_count
    if rc != 0:
        raise KernelError(lib.vapi_last_error().decode(errors="replace") + f" (code {rc})")
    launch_count += launches


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32, bfloat16)")


def _cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("vapi_b200 kernels run on CUDA tensors only; there is no CPU fallback")


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_held_stream = threading.local()


def _stream() -> ctypes.c_void_p:
    h = getattr(_held_stream, "handle", None)
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream if h is None else h)


class one_stream:
    """Within the block every kernel of this module launches on the stream that is current at its
    entry, looked up once instead of once per kernel (a step launches a few hundred).  The caller
    must not switch streams inside the block."""

    def __enter__(self):
        self.before = getattr(_held_stream, "handle", None)
        _held_stream.handle = torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else None
        return self

    def __exit__(self, *exc):
        _held_stream.handle = self.before
        return False


def _contig(t: torch.Tensor, what: str) -> None:
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32")


def _f32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
        raise KernelError(f"{what} must be contiguous float32")


_sm_counts: Dict[int, int] = {}


def sm_count() -> int:
    """Multiprocessors of the current CUDA device, asked of the device (once per device)."""
    if not torch.cuda.is_available():
        raise KernelError("vapi_b200 kernels need a CUDA device; there is no CPU fallback")
    dev = torch.cuda.current_device()
    n = _sm_counts.get(dev)
    if n is None:
        n = _sm_counts[dev] = int(torch.cuda.get_device_properties(dev).multi_processor_count)
    return n


# ---------------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, status: Optional[torch.Tensor] = None,
          next_weight: Optional[torch.Tensor] = None, scale: float = 1.0):
    """Rows of ``table`` [V, H] for ``tokens`` [n], times ``scale`` (a float32 product), as the float32 residual
    stream [n, H].

    With ``next_weight`` (the weight of the norm that will read the stream) the call also
    returns what a deferred norm needs: the sums of squares of the rows, [1, n], and
    bfloat16(row * next_weight), [n, H]: ``(x, ss, xw)``."""
    _cuda(table, tokens, next_weight)
    _contig(table, "embedding table")
    _i32(tokens, "tokens")
    _f32(next_weight, "norm weight")
    n, (vocab, hidden) = tokens.numel(), table.shape
    out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    ss = xw = None
    if next_weight is not None:
        ss = torch.empty((1, n), dtype=torch.float32, device=table.device)
        xw = torch.empty((n, hidden), dtype=torch.bfloat16, device=table.device)
    lib = _lib("elementwise")
    _check(lib, lib.vapi_embed(_p(table), _dt(table), _p(tokens), _p(out), _p(ss), _p(next_weight), _p(xw), n,
                               hidden, vocab, _p(status), _stream(), ctypes.c_float(scale)))
    return (out, ss, xw) if next_weight is not None else out


def add_residual_ss(x: torch.Tensor, delta: torch.Tensor, next_weight: torch.Tensor):
    """``x += delta`` on the float32 stream; returns ``(ss, xw)`` for the norm that follows:
    the sums of squares of the new rows, [1, n], and bfloat16(new row * next_weight)."""
    _cuda(x, delta, next_weight)
    _f32(x, "residual stream")
    _f32(next_weight, "norm weight")
    _contig(delta, "delta")
    n, hidden = x.shape
    ss = torch.empty((1, n), dtype=torch.float32, device=x.device)
    xw = torch.empty((n, hidden), dtype=torch.bfloat16, device=x.device)
    lib = _lib("elementwise")
    _check(lib, lib.vapi_add_residual_ss(_p(x), _p(delta), _dt(delta), _p(ss), _p(next_weight), _p(xw), n, hidden,
                                         _stream()))
    return ss, xw


def resolve_tokens(tokens: torch.Tensor, src: torch.Tensor, prev: torch.Tensor,
                   status: Optional[torch.Tensor] = None) -> None:
    """In place: ``tokens[i] = prev[src[i]]`` wherever ``src[i] >= 0`` (tokens that the step before
    sampled and the host has not read yet)."""
    _cuda(tokens, src, prev)
    for t, w in ((tokens, "tokens"), (src, "token sources"), (prev, "sampled tokens")):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"{w} must be contiguous int32")
    lib = _lib("elementwise")
    _check(lib, lib.vapi_resolve_tokens(_p(tokens), _p(src), _p(prev), tokens.numel(), prev.numel(), _p(status),
                                        _stream()))


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x += delta`` (when given) and ``out = rmsnorm(x) * weight``; x is the float32 stream.

    With ``rows`` the output has one row per entry of ``rows`` and ``x`` is left untouched
    (the sum is formed on the fly): that is the form the final norm uses for the rows whose
    logits are wanted.
    """
    _cuda(x, delta, weight, rows)
    _f32(x, "residual stream")
    _f32(weight, "norm weight")
    _i32(rows, "rows")
    hidden = x.shape[-1]
    if weight.numel() != hidden:
        raise KernelError(f"norm weight has {weight.numel()} elements for rows of {hidden}")
    if delta is not None:
        _contig(delta, "delta")
        if delta.shape != x.shape or delta.dtype != out_dtype:
            raise KernelError("delta must have the stream's shape and the activation dtype")
    n_out = rows.numel() if rows is not None else x.shape[0]
    out = torch.empty((n_out, hidden), dtype=out_dtype, device=x.device)
    lib = _lib("elementwise")
    _check(lib, lib.vapi_add_rmsnorm(_p(x), _p(delta), _p(weight), ctypes.c_float(eps), _p(rows), _p(out),
                                     _dt(out), n_out, hidden, _stream()))
    return out


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    """``x += delta`` on the float32 stream."""
    _cuda(x, delta)
    _f32(x, "residual stream")
    _contig(delta, "delta")
    lib = _lib("elementwise")
    _check(lib, lib.vapi_add_residual(_p(x), _p(delta), _dt(delta), ctypes.c_longlong(x.numel()), _stream()))


def swiglu(g: torch.Tensor) -> torch.Tensor:
    """``silu(g[:, :F]) * g[:, F:]`` for a stacked gate/up product [n, 2F]."""
    _cuda(g)
    _contig(g, "gate/up product")
    rows, two_f = g.shape
    if two_f % 2:
        raise KernelError("swiglu needs an even number of columns")
    out = torch.empty((rows, two_f // 2), dtype=g.dtype, device=g.device)
    lib = _lib("elementwise")
    _check(lib, lib.vapi_swiglu(_p(g), _p(out), _dt(g), rows, two_f // 2, _stream()))
    return out


SKINNY_MAX_ROWS = int(os.environ.get("VAPI_SKINNY_MAX_ROWS", "16"))
#: set False to send every product to the library (for comparisons)
use_skinny = os.environ.get("VAPI_SKINNY", "1") != "0"

_PRO = {"act": 0, "norm": 1}
_EPI = {"bf16": 0, "swiglu": 1, "resid": 2, "f32": 3}


def skinny_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether the weight-streaming kernel takes this product: bfloat16 weight, at most 16
    rows, inner size a multiple of 32."""
    return (use_skinny and weight.is_cuda and weight.dtype == torch.bfloat16 and 0 < rows <= SKINNY_MAX_ROWS
            and weight.dim() == 2 and weight.shape[1] % 32 == 0 and weight.is_contiguous())


def skinny_use_tma(on: bool) -> bool:
    """Choose the form of the decode product whose weight stream is moved by TMA into mbarrier
    rings (steps of at most 8 tokens, inner size up to 2048) instead of per-lane asynchronous
    copies; returns what was chosen before.  ``VAPI_GV_TMA=1`` chooses it from the start."""
    return bool(_lib("gemv").vapi_skinny_linear_use_tma(1 if on else 0))


def skinny_blocks(n_out: int, epilogue: str, rows_per_block: int = 16) -> int:
    if epilogue == "swiglu":
        return (n_out // 2 + 7) // 8
    return -(-n_out // rows_per_block)


def skinny_linear(weight: torch.Tensor, *, act: Optional[torch.Tensor] = None,
                  xw: Optional[torch.Tensor] = None, ss_in: Optional[torch.Tensor] = None, eps: float = 0.0,
                  epilogue: str = "bf16", bias: Optional[torch.Tensor] = None,
                  resid: Optional[torch.Tensor] = None, next_weight: Optional[torch.Tensor] = None,
                  rows_per_block: Optional[int] = None):
    """The weight-streaming product for decode steps (at most 16 rows), with its fusions.

    Token operand: ``act`` [M, K] bfloat16; or the residual stream seen through an RMSNorm not
    applied yet: ``xw`` [M, K] = bfloat16(stream * norm weight) with the partial sums of squares
    ``ss_in`` [parts, M] of the stream's rows (both left by whoever wrote the stream last) and the
    norm's ``eps``.  ``epilogue``: "bf16" -> [M, N] bfloat16; "f32" -> [M, N] float32; "swiglu" ->
    [M, N/2] bfloat16 = silu(first half) * second half; "resid" -> adds into ``resid`` [M, N]
    float32 in place and returns ``(ss, xw)`` of the new stream for the norm whose weight is
    ``next_weight`` (``(None, None)`` without it).
    """
    _cuda(weight, act, xw, ss_in, bias, resid, next_weight)
    N, K = weight.shape
    pro = "act" if act is not None else "norm"
    src = act if act is not None else xw
    if src is None:
        raise KernelError("skinny_linear needs a token operand (act or xw)")
    M = src.shape[0]
    if weight.dtype != torch.bfloat16 or not weight.is_contiguous():
        raise KernelError("skinny_linear needs a contiguous bfloat16 weight")
    if src.shape[1] != K or not src.is_contiguous() or src.dtype != torch.bfloat16:
        raise KernelError(f"skinny_linear: token operand {tuple(src.shape)} / {src.dtype} does not fit a weight of {N}x{K}")
    if pro == "norm":
        _f32(ss_in, "partial sums")
        if ss_in is None or ss_in.dim() != 2 or ss_in.shape[1] != M:
            raise KernelError("partial sums must be [parts, M]")
    _f32(bias, "bias")
    _f32(next_weight, "norm weight")
    rpb = rows_per_block or 16
    out_bf16 = out_f32 = sso = xwo = None
    out_stride = N
    if epilogue == "bf16":
        out_bf16 = torch.empty((M, N), dtype=torch.bfloat16, device=weight.device)
    elif epilogue == "f32":
        out_f32 = torch.empty((M, N), dtype=torch.float32, device=weight.device)
    elif epilogue == "swiglu":
        out_stride = N // 2
        out_bf16 = torch.empty((M, N // 2), dtype=torch.bfloat16, device=weight.device)
    elif epilogue == "resid":
        _f32(resid, "residual stream")
        if resid is None or tuple(resid.shape) != (M, N):
            raise KernelError("the residual stream must be [M, N]")
        if next_weight is not None:
            sso = torch.empty((skinny_blocks(N, epilogue, rpb), M), dtype=torch.float32, device=weight.device)
            xwo = torch.empty((M, N), dtype=torch.bfloat16, device=weight.device)
    else:
        raise KernelError(f"unknown epilogue {epilogue}")
    lib = _lib("gemv")
    _check(lib, lib.vapi_skinny_linear(
        _p(weight), N, K, M, _PRO[pro], _p(act), _p(xw), _p(ss_in), 0 if ss_in is None else ss_in.shape[0],
        ctypes.c_float(eps), _EPI[epilogue], _p(out_bf16), _p(out_f32), ctypes.c_longlong(out_stride), _p(bias),
        _p(resid), _p(sso), _p(next_weight), _p(xwo), rpb, _stream()))
    if epilogue == "resid":
        return sso, xwo
    return out_bf16 if out_bf16 is not None else out_f32


#: Steps of up to this many rows go to the tcgen05 product with its fused epilogues.  The kernel
#: itself takes up to 256 rows, but it has one tile per block and pays its fixed costs (cluster
#: reduction, epilogue) per launch: measured in the captured decode step of LFM2-1.2B sizes it
#: beats the library's product plus separate norm / SwiGLU / add kernels at 32 rows (1.26 vs 1.33
#: ms), loses narrowly at 64 (1.71 vs 1.68 ms) and clearly beyond (2-7x slower at 256 rows).
TC_MAX_ROWS = int(os.environ.get("VAPI_TC_MAX_ROWS", "32"))
#: set False to keep products of 17..TC_MAX_ROWS rows on the library
use_tc = os.environ.get("VAPI_TC", "1") != "0"


def skinny_shortconv_applies(rows: int, w_in: torch.Tensor, kernel: int, state_layer: Optional[torch.Tensor]) -> bool:
    """Whether :func:`skinny_shortconv` takes a decode step of ``rows`` single-token sequences."""
    return (skinny_applies(rows, w_in) and 1 <= kernel <= 8 and w_in.shape[0] % 3 == 0
            and (kernel == 1 or (state_layer is not None and state_layer.dtype == torch.bfloat16)))


def skinny_shortconv(w_in: torch.Tensor, *, xw: torch.Tensor, ss_in: torch.Tensor, eps: float,
                     in_bias: Optional[torch.Tensor], taps: torch.Tensor, conv_bias: Optional[torch.Tensor],
                     state_layer: Optional[torch.Tensor], state_slots: torch.Tensor, positions: torch.Tensor,
                     status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The short-conv mixer up to its out_proj for a decode step, in one launch: in_proj on the
    stream seen through a deferred norm (``xw``, ``ss_in``, ``eps`` as for :func:`skinny_linear`),
    gate, taps over each request's state, ``C * conv``, state update.  Every one of the M <= 16
    tokens must be a sequence of its own: token m uses ``state_slots[m]`` and ``positions[m]``.
    Returns y [M, H] bfloat16."""
    _cuda(w_in, xw, ss_in, in_bias, taps, conv_bias, state_layer, state_slots, positions)
    H3, K = w_in.shape
    H, M, L = H3 // 3, xw.shape[0], taps.shape[0]
    if w_in.dtype != torch.bfloat16 or not w_in.is_contiguous() or H3 != 3 * H:
        raise KernelError("skinny_shortconv needs a contiguous bfloat16 in_proj weight of 3H rows")
    if xw.dtype != torch.bfloat16 or tuple(xw.shape) != (M, K) or not xw.is_contiguous():
        raise KernelError("skinny_shortconv: the weighted stream must be [M, K] bfloat16")
    _f32(ss_in, "partial sums")
    if ss_in.dim() != 2 or ss_in.shape[1] != M:
        raise KernelError("partial sums must be [parts, M]")
    for t, w in ((in_bias, "in_proj bias"), (taps, "conv taps"), (conv_bias, "conv bias")):
        _f32(t, w)
    if tuple(taps.shape) != (L, H):
        raise KernelError("taps must be [L, H]")
    _i32(state_slots, "state slots")
    _i32(positions, "positions")
    if state_slots.numel() < M or positions.numel() < M:
        raise KernelError("skinny_shortconv: one state slot and one position per token are needed")
    slot_stride = num_slots = 0
    if L > 1:
        if state_layer is None or state_layer.dtype != torch.bfloat16 or tuple(state_layer.shape[1:]) != (L - 1, H):
            raise KernelError(f"state must be [slots, {L - 1}, {H}] bfloat16")
        if state_layer.stride(2) != 1 or state_layer.stride(1) != H:
            raise KernelError("state rows must be contiguous")
        slot_stride, num_slots = state_layer.stride(0), state_layer.shape[0]
    out = torch.empty((M, H), dtype=torch.bfloat16, device=w_in.device)
    lib = _lib("gemv")
    _check(lib, lib.vapi_skinny_linear_conv(
        _p(w_in), H, K, M, _p(xw), _p(ss_in), ss_in.shape[0], ctypes.c_float(eps), _p(in_bias), _p(taps), _p(conv_bias),
        L, _p(state_layer if L > 1 else None), ctypes.c_longlong(slot_stride), num_slots, _p(state_slots),
        _p(positions), _p(out), _p(status), _stream()))
    return out


def tc_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes this product: bfloat16 weight, 17..TC_MAX_ROWS rows, inner size
    a multiple of 8 (16-byte rows for TMA)."""
    return (use_tc and weight.is_cuda and weight.dtype == torch.bfloat16 and SKINNY_MAX_ROWS < rows <= TC_MAX_ROWS
            and weight.dim() == 2 and weight.shape[1] % 8 == 0 and weight.is_contiguous())


def _tc_plan(N: int, K: int, M: int, epi: int):
    lib = _lib("linear_tc")
    t, s, b = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib.vapi_linear_tc_plan(N, K, M, epi, ctypes.byref(t), ctypes.byref(s), ctypes.byref(b))
    return t.value, s.value, b.value


def _fused_product(which: str, weight: torch.Tensor, act, xw, ss_in, eps: float, epilogue: str, bias, resid,
                   next_weight, status):
    """Operand checks, outputs and the call shared by :func:`linear_tc` and :func:`prompt_linear`."""
    _cuda(weight, act, xw, ss_in, bias, resid, next_weight)
    N, K = weight.shape
    pro = "act" if act is not None else "norm"
    src = act if act is not None else xw
    if src is None:
        raise KernelError(f"{which} needs a token operand (act or xw)")
    M = src.shape[0]
    if weight.dtype != torch.bfloat16 or not weight.is_contiguous():
        raise KernelError(f"{which} needs a contiguous bfloat16 weight")
    if src.shape[1] != K or not src.is_contiguous() or src.dtype != torch.bfloat16:
        raise KernelError(f"{which}: token operand {tuple(src.shape)} / {src.dtype} does not fit a weight of {N}x{K}")
    if pro == "norm":
        _f32(ss_in, "partial sums")
        if ss_in is None or ss_in.dim() != 2 or ss_in.shape[1] != M:
            raise KernelError("partial sums must be [parts, M]")
    _f32(bias, "bias")
    _f32(next_weight, "norm weight")
    if epilogue not in _EPI:
        raise KernelError(f"unknown epilogue {epilogue}")
    lib = _lib(which)
    if which == "linear_tc":
        parts = _tc_plan(N, K, M, _EPI[epilogue])[0]
        fn = lib.vapi_linear_tc
    else:
        parts = _prompt_plan(N, K, M, _EPI[epilogue])[2]
        fn = lib.vapi_prompt_linear
    out_bf16 = out_f32 = sso = xwo = None
    out_stride = N
    if epilogue == "bf16":
        out_bf16 = torch.empty((M, N), dtype=torch.bfloat16, device=weight.device)
    elif epilogue == "f32":
        out_f32 = torch.empty((M, N), dtype=torch.float32, device=weight.device)
    elif epilogue == "swiglu":
        out_stride = N // 2
        out_bf16 = torch.empty((M, N // 2), dtype=torch.bfloat16, device=weight.device)
    else:
        _f32(resid, "residual stream")
        if resid is None or tuple(resid.shape) != (M, N) or not resid.is_contiguous():
            raise KernelError("the residual stream must be a contiguous [M, N]")
        if next_weight is not None:
            sso = torch.empty((parts, M), dtype=torch.float32, device=weight.device)
            xwo = torch.empty((M, N), dtype=torch.bfloat16, device=weight.device)
    _check(lib, fn(
        _p(weight), N, K, M, _PRO[pro], _p(src), _p(ss_in), 0 if ss_in is None else ss_in.shape[0], ctypes.c_float(eps),
        _EPI[epilogue], _p(out_bf16), _p(out_f32), ctypes.c_longlong(out_stride), _p(bias), _p(resid), _p(sso),
        _p(next_weight), _p(xwo), _p(status), _stream()))
    if epilogue == "resid":
        return sso, xwo
    return out_bf16 if out_bf16 is not None else out_f32


def linear_tc(weight: torch.Tensor, *, act: Optional[torch.Tensor] = None, xw: Optional[torch.Tensor] = None,
              ss_in: Optional[torch.Tensor] = None, eps: float = 0.0, epilogue: str = "bf16",
              bias: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
              next_weight: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
    """The tcgen05 / TMA product for 17..256 rows; same operands, epilogues and results as
    :func:`skinny_linear`."""
    return _fused_product("linear_tc", weight, act, xw, ss_in, eps, epilogue, bias, resid, next_weight, status)


#: steps of more rows than TC_MAX_ROWS go to the persistent tcgen05 product of csrc/linear_prompt.cu
#: (with its fused prologue and epilogues) from this many rows on; 0 keeps them on the library's
#: product with separate norm / SwiGLU / add kernels
PROMPT_MIN_ROWS = int(os.environ.get("VAPI_PROMPT_MIN_ROWS", "0"))


def prompt_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether the persistent tcgen05 product takes this product: bfloat16 weight, at least
    PROMPT_MIN_ROWS rows, inner size a multiple of 8 (16-byte rows for TMA)."""
    return (PROMPT_MIN_ROWS > 0 and rows >= PROMPT_MIN_ROWS and rows > TC_MAX_ROWS and weight.is_cuda
            and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0
            and weight.shape[0] % 8 == 0 and weight.is_contiguous())


def _prompt_plan(N: int, K: int, M: int, epi: int):
    lib = _lib("linear_prompt")
    b, pr, parts = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib.vapi_prompt_linear_plan(N, K, M, epi, ctypes.byref(b), ctypes.byref(pr), ctypes.byref(parts))
    return b.value, pr.value, parts.value


#: a feed-forward's gate|up product with SwiGLU as its epilogue goes to the persistent tcgen05 product
#: from this many rows on, also where the other products stay on the library (0: never)
PROMPT_SWIGLU_MIN_ROWS = int(os.environ.get("VAPI_PROMPT_SWIGLU_MIN_ROWS", "256"))


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` for ``weight = [Wg; Wu]``: one kernel with SwiGLU as the
    product's epilogue for prompt-sized bfloat16 steps, else the product followed by :func:`swiglu`."""
    rows = x.shape[0]
    if (x.dtype == torch.bfloat16 and 0 < PROMPT_SWIGLU_MIN_ROWS <= rows and rows > TC_MAX_ROWS and weight.is_cuda
            and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0 and weight.shape[0] % 16 == 0
            and weight.is_contiguous() and x.is_contiguous()):
        return prompt_linear(weight, act=x, epilogue="swiglu")
    if (x.dtype == torch.bfloat16 and x.is_contiguous() and weight.shape[0] % 16 == 0 and rows <= TC_MAX_ROWS
            and few_rows_applies(rows, weight)):
        return few_rows_linear(weight, act=x, epilogue="swiglu")      # a decode step: SwiGLU rides on the product
    return swiglu(linear(x, weight))


def prompt_force(bn: int = 0, pair: int = 0) -> None:
    """Fix the tile (128 | 256 features) and the blocks working on a tile (1 | 2) of
    :func:`prompt_linear` for the calls that follow; 0 gives the choice back to the kernel's plan."""
    lib = _lib("linear_prompt")
    _check(lib, lib.vapi_prompt_linear_force(bn, pair), launches=0)


def prompt_linear(weight: torch.Tensor, *, act: Optional[torch.Tensor] = None, xw: Optional[torch.Tensor] = None,
                  ss_in: Optional[torch.Tensor] = None, eps: float = 0.0, epilogue: str = "bf16",
                  bias: Optional[torch.Tensor] = None, resid: Optional[torch.Tensor] = None,
                  next_weight: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
    """The persistent tcgen05 / TMA product for prompt-sized steps; same operands, epilogues and
    results as :func:`skinny_linear`."""
    return _fused_product("linear_prompt", weight, act, xw, ss_in, eps, epilogue, bias, resid, next_weight, status)


def few_rows_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether one of this package's own products (with their fused prologues and epilogues)
    takes a step of ``rows`` rows against ``weight``."""
    return skinny_applies(rows, weight) or tc_applies(rows, weight) or prompt_applies(rows, weight)


def few_rows_linear(weight: torch.Tensor, **kw):
    """:func:`skinny_linear` up to 16 rows, :func:`linear_tc` up to TC_MAX_ROWS, :func:`prompt_linear` above."""
    src = kw.get("act") if kw.get("act") is not None else kw.get("xw")
    if src.shape[0] <= SKINNY_MAX_ROWS:
        return skinny_linear(weight, **kw)
    if src.shape[0] <= TC_MAX_ROWS:
        return linear_tc(weight, **kw)
    return prompt_linear(weight, **kw)


def skinny_f32_applies(rows: int, weight: torch.Tensor) -> bool:
    """Whether the float32 weight-streaming kernel takes this product: float32 weight, at most 16
    rows, inner size a multiple of 4."""
    return (use_skinny and weight.is_cuda and weight.dtype == torch.float32 and 0 < rows <= SKINNY_MAX_ROWS
            and weight.dim() == 2 and weight.shape[1] % 4 == 0 and weight.is_contiguous() and weight.data_ptr() % 16 == 0)


def skinny_linear_f32(weight: torch.Tensor, act: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act @ weight.T (+ bias)`` for at most 16 rows in true float32 (FMA only): the decode
    product of the 32-bit path, bound by reading the weight once."""
    _cuda(weight, act, bias)
    N, K = weight.shape
    M = act.shape[0]
    if weight.dtype != torch.float32 or not weight.is_contiguous():
        raise KernelError("skinny_linear_f32 needs a contiguous float32 weight")
    if act.dtype != torch.float32 or tuple(act.shape) != (M, K) or not act.is_contiguous():
        raise KernelError(f"skinny_linear_f32: token operand {tuple(act.shape)} / {act.dtype} does not fit a weight of {N}x{K}")
    _f32(bias, "bias")
    out = torch.empty((M, N), dtype=torch.float32, device=weight.device)
    lib = _lib("gemv")
    _check(lib, lib.vapi_skinny_linear_f32(_p(weight), N, K, M, _p(act), _p(bias), _p(out), ctypes.c_longlong(N), _stream()))
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)``.  The library matrix product, except for decode-sized
    bfloat16 products (at most 16 rows), which go to the weight-streaming kernel.

    float32 runs without any reduced-precision mode (see :func:`strict_fp32`).  A weight kept
    in float32 beside bfloat16 activations is multiplied in float32.
    """
    _cuda(x, weight)
    if x.dtype == torch.bfloat16 and skinny_applies(x.shape[0], weight) and x.is_contiguous():
        if out_dtype in (None, torch.bfloat16):
            return skinny_linear(weight, act=x, epilogue="bf16", bias=bias)
        if out_dtype == torch.float32:
            return skinny_linear(weight, act=x, epilogue="f32", bias=bias)
    if x.dtype == torch.bfloat16 and tc_applies(x.shape[0], weight) and x.is_contiguous():
        if out_dtype in (None, torch.bfloat16):
            return linear_tc(weight, act=x, epilogue="bf16", bias=bias)
        if out_dtype == torch.float32:
            return linear_tc(weight, act=x, epilogue="f32", bias=bias)
    if (x.dtype == torch.float32 and out_dtype in (None, torch.float32) and skinny_f32_applies(x.shape[0], weight)
            and x.is_contiguous() and x.data_ptr() % 16 == 0):
        return skinny_linear_f32(weight, x, bias)
    if weight.dtype != x.dtype:
        y = torch.mm(x.to(torch.float32), weight.to(torch.float32).t())
        if bias is not None:
            y = y + bias
        return y.to(out_dtype or x.dtype)
    if out_dtype is not None and out_dtype != x.dtype:
        if bias is not None:
            return (torch.mm(x, weight.t(), out_dtype=out_dtype) + bias.to(out_dtype))
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if bias is not None:
        return torch.addmm(bias.to(x.dtype), x, weight.t())
    return torch.mm(x, weight.t())


def strict_fp32() -> None:
    """Switch off every reduced-precision matrix mode of the library products."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    try:
        torch.set_float32_matmul_precision("highest")
    except Exception:  # pragma: no cover
        pass


def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of ``position * inv_freq`` in float32: two [n, len(inv_freq)] tensors."""
    _cuda(positions, inv_freq)
    _i32(positions, "positions")
    _f32(inv_freq, "inv_freq")
    n, half = positions.numel(), inv_freq.numel()
    cos = torch.empty((n, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    lib = _lib("rope")
    _check(lib, lib.vapi_rope_cos_sin(_p(positions), _p(inv_freq), _p(cos), _p(sin), n, half, _stream()))
    return cos, sin


def qk_norm_rope_write(qkv: torch.Tensor, nh: int, nkv: int, d: int,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot: int,
                       cache_layer: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                       status: Optional[torch.Tensor] = None) -> None:
    """Per-head RMSNorm and rotate-half RoPE of q and k in a fused ``qkv`` [n, (nh+2nkv)*d];
    q is rewritten in place, k (normed, roped) and v go to ``cache_layer``
    [pages, 2, nkv, page_size, d] at ``slot_mapping``.  ``cache_layer=None`` leaves the
    cache alone (a layer that reads another layer's cache)."""
    _cuda(qkv, q_weight, k_weight, cos, sin, cache_layer, slot_mapping)
    _contig(qkv, "qkv")
    _f32(q_weight, "q norm weight")
    _f32(k_weight, "k norm weight")
    _f32(cos, "cos")
    _f32(sin, "sin")
    _i32(slot_mapping, "slot mapping")
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected {(nh + 2 * nkv) * d}")
    page_size = num_pages = 0
    if cache_layer is not None:
        _contig(cache_layer, "cache layer")
        if cache_layer.dtype != qkv.dtype or tuple(cache_layer.shape[1:3]) != (2, nkv) or cache_layer.shape[4] != d:
            raise KernelError(f"cache layer {tuple(cache_layer.shape)} / {cache_layer.dtype} does not fit "
                              f"nkv={nkv} d={d} {qkv.dtype}")
        num_pages, page_size = cache_layer.shape[0], cache_layer.shape[3]
    if cos is not None and (cos.shape != (n, rot // 2) or sin is None or sin.shape != cos.shape):
        raise KernelError("cos/sin must be [n, rot/2]")
    lib = _lib("rope")
    _check(lib, lib.vapi_qk_norm_rope_write(
        _p(qkv), _dt(qkv), _p(q_weight), _p(k_weight), ctypes.c_float(eps), _p(cos), _p(sin), rot,
        _p(cache_layer), _p(slot_mapping), n, nh, nkv, d, page_size, num_pages, _p(status), _stream()))


# "tma": decode steps at head size 64 on the TMA-fed decode kernel; "mma": on the one-warp flash kernel
DECODE_ATTENTION = os.environ.get("VAPI_DECODE_ATTENTION", "tma")
_decode_limits: Optional[Tuple[int, int]] = None


def decode_attention_limits() -> Tuple[int, int]:
    """(blocks of the decode kernel that the device holds at once, the most slices of the keys that
    it combines inside the kernel), as the library reports them."""
    global _decode_limits
    if _decode_limits is None:
        lib = _lib("attention")
        lib.vapi_attention_use_decode_kernel(1 if DECODE_ATTENTION == "tma" else 0)
        _decode_limits = (int(lib.vapi_decode_attention_slots()) or sm_count() * 3, int(lib.vapi_decode_attention_cluster()))
    return _decode_limits


def decode_attention_applies(dtype: torch.dtype, d: int, page_size: int, rows: int) -> bool:
    """Whether a step whose sequences bring at most ``rows`` rows (tokens x q heads per kv head)
    runs on the decode kernel (the library's own rule, restated)."""
    return (DECODE_ATTENTION == "tma" and dtype == torch.bfloat16 and d == 64 and page_size % 64 == 0
            and rows <= 16)


def decode_attention_combines(num_seqs: int, nkv: int, splits: int) -> bool:
    """Whether the decode kernel combines its slices itself (at most a cluster's worth of slices,
    the whole grid resident at once, and a cluster of that size fits the device): the library's answer."""
    if splits <= 1:
        return False
    decode_attention_limits()
    return bool(_lib("attention").vapi_decode_attention_combines(num_seqs, nkv, splits))


def attention_splits(num_seqs: int, max_q: int, max_k: int, nh: int, nkv: int, decode_kernel: bool = False) -> int:
    """How many blocks share the keys of one row tile: 1 unless the step is so small that
    the device would sit idle (decode of few sequences over long contexts).  A block of the
    one-warp flash kernel has 48 KB of shared memory, so 4 fit on a multiprocessor: aim at one
    full wave of 4 blocks on each, every block with at least 128 keys.

    The decode kernel (measured at head size 64, 8 kv heads, context 4096 and 32768): while the
    (sequence, kv head) pairs are fewer than two blocks per SM, slices up to that many blocks, and
    no more than the kernel combines itself unless a slice would then be longer than 32 tiles and
    there would be fewer blocks than SMs;
    a step with more pairs than the device holds blocks is cut for about four rounds of blocks, so
    that the last ones do not run alone."""
    n_rep = nh // nkv
    rows = max_q * n_rep
    tiles = -(-rows // (16 if rows <= 16 else 64))
    blocks = max(1, num_seqs * nkv * tiles)
    if decode_kernel:
        key_tiles = max(1, -(-max_k // 64))
        slots, cluster = decode_attention_limits()
        by_len = max(1, key_tiles // 2)
        if blocks > slots:
            return max(1, min(-(-4 * slots // blocks), by_len, 32))
        want = max(1, int(round(2 * slots / 3 / blocks)))
        if want > cluster and (key_tiles <= 32 * cluster or 3 * blocks * cluster >= slots):
            want = cluster
        return max(1, min(want, by_len, 32))
    sms = sm_count()
    if rows > 16 and blocks >= sms:
        return 1
    want = max(1, 4 * sms // blocks)
    by_len = max(1, max_k // 128)
    return max(1, min(want, by_len, 32))


def paged_attention(q: torch.Tensor, q_row_stride: int, cache_layer: torch.Tensor,
                    block_table: torch.Tensor, cu_q: torch.Tensor, seqlens_k: torch.Tensor,
                    n: int, num_seqs: int, max_q: int, max_k: int, nh: int, nkv: int, d: int,
                    scale: float, window: int = 0, splits: Optional[int] = None,
                    status: Optional[torch.Tensor] = None, impl: str = "auto") -> torch.Tensor:
    """Causal GQA attention of a mixed batch over the paged cache; returns [n, nh*d].

    ``q`` may be a view into a fused qkv tensor: head h of token t is at
    ``t*q_row_stride + h*d``.  ``window`` > 0 limits each query to the last ``window`` keys.
    ``impl``: "tcgen05" forces the kernel on the fifth-generation tensor cores (bfloat16, head_dim 64,
    pages of 64n, no split), which "auto" uses for steps with prompt portions of 64 tokens or more;
    "auto" otherwise picks the tensor-core kernel where it applies (bfloat16, head_dim 64 or
    128, page size a multiple of 64) and the general kernel elsewhere; "general" and
    "tensor_core" force one (the latter raises where it does not apply); "decode" forces the
    TMA-fed decode kernel (bfloat16, head_dim 64, at most 16 rows per sequence and kv head).
    """
    _cuda(q, cache_layer, block_table, cu_q, seqlens_k)
    _i32(block_table, "block table")
    _i32(cu_q, "cu_q")
    _i32(seqlens_k, "seqlens_k")
    _contig(cache_layer, "cache layer")
    if cache_layer.dtype != q.dtype:
        raise KernelError("q and the cache must have one dtype")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block table must be [S, width] with unit inner stride")
    num_pages, page_size = cache_layer.shape[0], cache_layer.shape[3]
    if splits is None:
        splits = 1 if impl == "tcgen05" else attention_splits(
            num_seqs, max_q, max_k, nh, nkv,
            impl == "decode" or (impl == "auto" and decode_attention_applies(q.dtype, d, page_size, max_q * (nh // nkv))))
    out = torch.empty((n, nh * d), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((n * nh * splits * d,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * nh * splits * 2,), dtype=torch.float32, device=q.device)
    lib = _lib("attention")
    decode_attention_limits()             # (also tells the library whether the decode kernel is in use)
    # how many kernels the library launches (its own rule, restated for the launch count): the
    # tcgen05 kernel takes steps with prompt portions, beside the flash kernel and the decode kernel in a mixed step
    tc = impl == "tcgen05" or (impl == "auto" and q.dtype == torch.bfloat16 and d == 64 and page_size % 64 == 0
                               and splits == 1 and max_q >= 64 and q_row_stride % 8 == 0 and scale > 0)
    launches = (1 if impl == "tcgen05" or num_seqs == 1 else (3 if nh // nkv <= 16 and DECODE_ATTENTION == "tma" else 2)) \
        if tc else (2 if splits > 1 else 1)
    if (impl == "decode" or (impl == "auto" and decode_attention_applies(q.dtype, d, page_size, max_q * (nh // nkv)))) \
            and decode_attention_combines(num_seqs, nkv, splits):
        launches = 1                      # the decode kernel's slices combine among themselves
    elif (not tc and impl == "auto" and DECODE_ATTENTION == "tma" and max_q * (nh // nkv) > 16
            and decode_attention_applies(q.dtype, d, page_size, nh // nkv)):
        launches += 1                     # short portions on the flash kernel, decode tokens on the decode kernel
    code = {"auto": 0, "general": 1, "tensor_core": 2, "tcgen05": 3, "decode": 4}[impl]
    _check(lib, lib.vapi_paged_attention(
        _p(q), ctypes.c_longlong(q_row_stride), _p(cache_layer), _dt(q), _p(block_table),
        block_table.stride(0), _p(cu_q), _p(seqlens_k), _p(out), _p(part_o), _p(part_ml), n, num_seqs,
        max_q, nh, nkv, d, page_size, num_pages, ctypes.c_float(scale), window, splits,
        code, _p(status), _stream()), launches)
    return out


#: whether decode steps run q/k norm, RoPE and the cache write inside the decode attention kernel.  Off
#: unless asked for: it gives the same bits with one launch fewer per attention layer, but measured no
#: faster (batch 8) to 1 % slower (batch 1 and 64) than the two kernels, whose first one hides behind
#: the product before it.
FUSED_DECODE_ROPE = os.environ.get("VAPI_FUSED_DECODE_ROPE", "0") == "1"


def decode_attention_fused_applies(dtype: torch.dtype, d: int, page_size: int, rows: int, rot: Optional[int]) -> bool:
    """Whether :func:`decode_attention_fused` takes a step of this shape (``rot``: the rotated width, or
    None without a position encoding)."""
    return decode_attention_applies(dtype, d, page_size, rows) and (rot is None or rot == d)


def decode_attention_fused(qkv: torch.Tensor, nh: int, nkv: int, d: int,
                           q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                           cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                           cache_layer: torch.Tensor, write_kv: bool, block_table: torch.Tensor,
                           cu_q: torch.Tensor, seqlens_k: torch.Tensor, n: int, num_seqs: int, max_q: int,
                           max_k: int, scale: float, window: int = 0, splits: Optional[int] = None,
                           status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`qk_norm_rope_write` and :func:`paged_attention` of a decode step in one kernel: per-head
    RMSNorm and rotate-half RoPE of q and of the new keys, the new keys and values written to
    ``cache_layer`` (``write_kv``) at the places the block table gives for the sequences' last
    ``q`` positions, and attention over the cache.  ``qkv`` [n, (nh+2nkv)*d] is left as it was.
    bfloat16, head_dim 64, pages of 64n, at most 16 rows per sequence and kv head.  Gives exactly
    what the two calls give."""
    _cuda(qkv, q_weight, k_weight, cos, sin, cache_layer, block_table, cu_q, seqlens_k)
    _contig(qkv, "qkv")
    _contig(cache_layer, "cache layer")
    _f32(q_weight, "q norm weight")
    _f32(k_weight, "k norm weight")
    _f32(cos, "cos")
    _f32(sin, "sin")
    _i32(block_table, "block table")
    _i32(cu_q, "cu_q")
    _i32(seqlens_k, "seqlens_k")
    if qkv.dtype != torch.bfloat16 or cache_layer.dtype != torch.bfloat16:
        raise KernelError("the fused decode attention is for bfloat16")
    if qkv.shape[0] != n or qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError(f"qkv is {tuple(qkv.shape)}, expected ({n}, {(nh + 2 * nkv) * d})")
    if tuple(cache_layer.shape[1:3]) != (2, nkv) or cache_layer.shape[4] != d:
        raise KernelError(f"cache layer {tuple(cache_layer.shape)} does not fit nkv={nkv} d={d}")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block table must be [S, width] with unit inner stride")
    if cos is not None and (cos.shape != (n, d // 2) or sin is None or sin.shape != cos.shape or not cos.is_contiguous()
                            or not sin.is_contiguous()):
        raise KernelError("cos/sin must be contiguous [n, head_dim/2]")
    for w, name in ((q_weight, "q"), (k_weight, "k")):
        if w is not None and (w.numel() != d or not w.is_contiguous()):
            raise KernelError(f"the {name} norm weight must be [head_dim]")
    num_pages, page_size = cache_layer.shape[0], cache_layer.shape[3]
    if splits is None:
        splits = attention_splits(num_seqs, max_q, max_k, nh, nkv, True)
    out = torch.empty((n, nh * d), dtype=qkv.dtype, device=qkv.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((n * nh * splits * d,), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n * nh * splits * 2,), dtype=torch.float32, device=qkv.device)
    lib = _lib("attention")
    decode_attention_limits()
    launches = 1 if splits == 1 or decode_attention_combines(num_seqs, nkv, splits) else 2
    _check(lib, lib.vapi_decode_attention_fused(
        _p(qkv), _p(q_weight), _p(k_weight), ctypes.c_float(eps), _p(cos), _p(sin), _p(cache_layer),
        1 if write_kv else 0, _p(block_table), block_table.stride(0), _p(cu_q), _p(seqlens_k), _p(out),
        _p(part_o), _p(part_ml), n, num_seqs, max_q, nh, nkv, d, page_size, num_pages, ctypes.c_float(scale),
        window, splits, _p(status), _stream()), launches)
    return out


def shortconv(h3: torch.Tensor, in_bias: Optional[torch.Tensor], taps: torch.Tensor,
              conv_bias: Optional[torch.Tensor], state_layer: Optional[torch.Tensor],
              state_slots: torch.Tensor, tok_seq: torch.Tensor, cu_q: torch.Tensor,
              positions: torch.Tensor, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gating, causal depthwise convolution and state update of the short-conv mixer.

    ``h3`` [n, 3H] = B | C | x; ``taps`` [L, H] oldest first; ``state_layer`` is a view
    [slots, L-1, H] of the per-request state (any slot stride).  Returns y [n, H].
    """
    _cuda(h3, in_bias, taps, conv_bias, state_layer, state_slots, tok_seq, cu_q, positions)
    _contig(h3, "h3")
    _f32(in_bias, "in_proj bias")
    _f32(taps, "conv taps")
    _f32(conv_bias, "conv bias")
    for t, w in ((state_slots, "state slots"), (tok_seq, "tok_seq"), (cu_q, "cu_q"), (positions, "positions")):
        _i32(t, w)
    n, three_h = h3.shape
    hidden = three_h // 3
    L = taps.shape[0]
    if three_h != 3 * hidden or taps.shape[1] != hidden:
        raise KernelError("h3 must be [n, 3H] and taps [L, H]")
    slot_stride = num_slots = 0
    if L > 1:
        if state_layer is None or state_layer.dtype != h3.dtype or tuple(state_layer.shape[1:]) != (L - 1, hidden):
            raise KernelError(f"state must be [slots, {L - 1}, {hidden}] of {h3.dtype}")
        if state_layer.stride(2) != 1 or state_layer.stride(1) != hidden:
            raise KernelError("state rows must be contiguous")
        slot_stride, num_slots = state_layer.stride(0), state_layer.shape[0]
    out = torch.empty((n, hidden), dtype=h3.dtype, device=h3.device)
    num_seqs = cu_q.numel() - 1
    lib = _lib("shortconv")
    _check(lib, lib.vapi_shortconv(
        _p(h3), _dt(h3), _p(in_bias), _p(taps), _p(conv_bias), _p(state_layer if L > 1 else None),
        ctypes.c_longlong(slot_stride), _p(state_slots), _p(tok_seq), _p(cu_q), _p(positions), _p(out),
        n, num_seqs, hidden, L, num_slots, _p(status), _stream()))
    return out


_sample_bufs: Dict[str, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}


def _sample_scratch(device, rows: int, slices: int):
    """Persistent scratch of the sliced argmax (the counters start at zero and every launch
    leaves them zero, so the buffer must not be handed out fresh each call)."""
    key = str(device)
    buf = _sample_bufs.get(key)
    need = rows * slices
    if buf is None or buf[0].numel() < need or buf[2].numel() < rows:
        cap_r, cap = max(rows, 256), max(need, 256 * 32)
        buf = (torch.empty(cap, dtype=torch.float32, device=device), torch.empty(cap, dtype=torch.int32, device=device),
               torch.zeros(cap_r, dtype=torch.int32, device=device))
        _sample_bufs[key] = buf
    return buf


def sample_rows(logits: torch.Tensor, mode: Optional[torch.Tensor] = None,
                inv_t: Optional[torch.Tensor] = None, seeds: Optional[torch.Tensor] = None,
                draws: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 ``logits`` [R, V]: greedy argmax (lowest id wins ties),
    or, where ``mode`` is 2, Gumbel-max temperature sampling keyed by (seed, draw)."""
    _cuda(logits, mode, inv_t, seeds, draws)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 with unit inner stride")
    _i32(mode, "mode")
    _f32(inv_t, "inverse temperatures")
    for t in (seeds, draws):
        if t is not None and t.dtype != torch.int64:
            raise KernelError("seeds and draw counters must be int64")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    # few rows over a large vocabulary: cut each row into slices so that more than `rows` blocks work
    slices = 1
    wave = 4 * sm_count()
    if rows < wave and vocab >= 8192:
        slices = max(1, min(32, wave // rows, vocab // 2048))
    part_v = part_i = counters = None
    if slices > 1:
        part_v, part_i, counters = _sample_scratch(logits.device, rows, slices)
    lib = _lib("sampling")
    _check(lib, lib.vapi_sample_rows(_p(logits), rows, vocab, ctypes.c_longlong(logits.stride(0)), _p(mode),
                                     _p(inv_t), _p(seeds), _p(draws), _p(out), slices, _p(part_v), _p(part_i),
                                     _p(counters), _stream()))
    return out


def sample_truncated(logits: torch.Tensor, inv_t: torch.Tensor, top_k: Optional[torch.Tensor],
                     top_p: Optional[torch.Tensor], min_p: Optional[torch.Tensor], seeds: torch.Tensor,
                     draws: torch.Tensor, out: Optional[torch.Tensor] = None, check: bool = False):
    """One token per row from the temperature distribution cut by top-k (0: none; negative: leave
    the row alone), min-p (0: none) and top-p (1: none), drawn by Gumbel-max over the survivors
    with noise keyed by (seed, draw).  With ``check`` also returns the threshold on the scaled
    logits and the number of survivors per row."""
    _cuda(logits, inv_t, top_k, top_p, min_p, seeds, draws, out)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 with unit inner stride")
    _f32(inv_t, "inverse temperatures")
    _f32(top_p, "top_p")
    _f32(min_p, "min_p")
    _i32(top_k, "top_k")
    for t in (seeds, draws):
        if t.dtype != torch.int64:
            raise KernelError("seeds and draw counters must be int64")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    tau = cnt = None
    if check:
        tau = torch.zeros((rows,), dtype=torch.float32, device=logits.device)
        cnt = torch.zeros((rows,), dtype=torch.int32, device=logits.device)
    lib = _lib("sampling")
    _check(lib, lib.vapi_sample_truncated(_p(logits), rows, vocab, ctypes.c_longlong(logits.stride(0)), _p(inv_t), _p(top_k),
                                          _p(top_p), _p(min_p), _p(seeds), _p(draws), _p(out), _p(tau), _p(cnt), _stream()))
    return (out, tau, cnt) if check else out


def apply_penalties(logits: torch.Tensor, rows: torch.Tensor, toks: torch.Tensor, counts: torch.Tensor,
                    rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    """Repetition / frequency / presence penalties on (row, token) pairs, in place."""
    _cuda(logits, rows, toks, counts, rep, freq, pres)
    _i32(rows, "rows")
    _i32(toks, "tokens")
    for t, w in ((counts, "counts"), (rep, "repetition"), (freq, "frequency"), (pres, "presence")):
        _f32(t, w)
    lib = _lib("sampling")
    _check(lib, lib.vapi_apply_penalties(_p(logits), logits.shape[1], ctypes.c_longlong(logits.stride(0)),
                                         _p(rows), _p(toks), _p(counts), _p(rep), _p(freq), _p(pres),
                                         rows.numel(), _stream()))


# ---------------------------------------------------------------------------------------
# blocks that norm a sublayer on both sides; rotary tables with scaled frequencies; attention
# with unlike key and value widths, chunked masks, sinks and head gates; recurrent mixers
def postnorm_add_rmsnorm(x: torch.Tensor, y: Optional[torch.Tensor], post_weight: Optional[torch.Tensor], post_eps: float,
                         mult: float, weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                         rows: Optional[torch.Tensor] = None, copy: bool = False, branches=None) -> Optional[torch.Tensor]:
    """``x += mult * rmsnorm(y) * post_weight`` on the float32 stream and, with ``weight``,
    ``out = rmsnorm(x) * weight`` in one pass.  With ``rows`` only those rows are produced and
    ``x`` is left untouched.  ``y`` None: nothing is pending.  ``weight`` None: no norm follows; with ``copy`` the
    rows of the stream themselves are returned in ``out_dtype`` (for a sublayer that reads the stream as it is),
    else only the stream is updated (returns None).  ``branches`` = (y2, weight_a, weight_b, eps, scale): the
    sublayer was two mixers side by side whose raw outputs are ``y`` and ``y2``, and
    ``scale * (rmsnorm(y) * weight_a + rmsnorm(y2) * weight_b)`` (float32) stands where ``y`` stands above."""
    _cuda(x, y, post_weight, weight, rows)
    y2 = wa = wb = None
    eps_b = scale_b = 0.0
    if branches is not None:
        y2, wa, wb, eps_b, scale_b = branches
        _cuda(y2, wa, wb)
        _f32(wa, "norm weight")
        _f32(wb, "norm weight")
        _contig(y2, "sublayer output")
        if y is None or y2.shape != y.shape or y2.dtype != y.dtype or wa.numel() != x.shape[-1] or wb.numel() != x.shape[-1]:
            raise KernelError("two branches come with outputs of one shape and dtype and a weight per column each")
    _f32(x, "residual stream")
    _f32(post_weight, "norm weight")
    _f32(weight, "norm weight")
    _i32(rows, "rows")
    hidden = x.shape[-1]
    if y is not None:
        _contig(y, "sublayer output")
        if y.shape != x.shape or y.dtype != out_dtype:
            raise KernelError("the sublayer's output must have the stream's shape and the activation dtype")
        if post_weight is None or post_weight.numel() != hidden:
            raise KernelError(f"norm weights must have {hidden} elements")
    if weight is not None and weight.numel() != hidden:
        raise KernelError(f"norm weights must have {hidden} elements")
    n_out = rows.numel() if rows is not None else x.shape[0]
    wants = weight is not None or copy
    if y is None and not wants:
        return None
    out = torch.empty((n_out, hidden), dtype=out_dtype, device=x.device) if wants else None
    lib = _lib("elementwise")
    _check(lib, lib.vapi_postnorm_add_rmsnorm(_p(x), _p(y), _DT[out_dtype], _p(post_weight), ctypes.c_float(post_eps),
                                              ctypes.c_float(mult), _p(weight), ctypes.c_float(eps), _p(rows), _p(out),
                                              n_out, hidden, _p(y2), _p(wa), _p(wb), ctypes.c_float(eps_b),
                                              ctypes.c_float(scale_b), _stream()))
    return out


def scaled_add_rmsnorm(x: torch.Tensor, y1: Optional[torch.Tensor], s1: Optional[torch.Tensor], y2: Optional[torch.Tensor],
                       s2: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                       rows: Optional[torch.Tensor] = None, copy: bool = False,
                       out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``x += s1 * y1 + s2 * y2`` on the float32 stream (two sublayers side by side, each with a scale per column; a
    missing scale counts as one, ``y2`` or both may be missing) and, with ``weight``, ``out = rmsnorm(x) * weight`` in
    the same pass.  ``weight`` None with ``copy``: the rows of the stream themselves in ``out_dtype``; without
    ``copy`` only the stream is updated (returns None).  With ``rows`` only those rows are produced and ``x`` is left
    untouched.  ``out`` may be given: [rows, >= hidden] with unit inner stride, e.g. the left part of a wider buffer."""
    _cuda(x, y1, s1, y2, s2, weight, rows, out)
    _f32(x, "residual stream")
    _f32(s1, "layer scale")
    _f32(s2, "layer scale")
    _f32(weight, "norm weight")
    _i32(rows, "rows")
    hidden = x.shape[-1]
    for y in (y1, y2):
        if y is not None:
            _contig(y, "sublayer output")
            if y.shape != x.shape or y.dtype != out_dtype:
                raise KernelError("a sublayer's output must have the stream's shape and the activation dtype")
    for v in (s1, s2, weight):
        if v is not None and v.numel() != hidden:
            raise KernelError(f"scales and norm weights must have {hidden} elements")
    n_out = rows.numel() if rows is not None else x.shape[0]
    wants = weight is not None or copy
    if y1 is None and y2 is None and not wants:
        return None
    if y1 is None and y2 is not None:
        y1, s1, y2, s2 = y2, s2, None, None
    if wants:
        if out is None:
            out = torch.empty((n_out, hidden), dtype=out_dtype, device=x.device)
        elif out.dtype != out_dtype or out.dim() != 2 or out.shape[0] != n_out or out.shape[1] != hidden or out.stride(1) != 1:
            raise KernelError("the given output must be [rows, hidden] of the activation dtype with unit inner stride")
    else:
        out = None
    lib = _lib("elementwise")
    _check(lib, lib.vapi_scaled_add_rmsnorm(_p(x), _p(y1), _p(s1), _p(y2), _p(s2), _p(weight), ctypes.c_float(eps), _p(rows),
                                            _p(out), ctypes.c_longlong(out.stride(0) if out is not None else 0),
                                            _DT[out_dtype], n_out, hidden, _stream()))
    return out


def latent_prepare(down: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, q_weight: Optional[torch.Tensor],
                   kv_weight: torch.Tensor, eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot: int,
                   cache_layer: Optional[torch.Tensor], page_size: int, slot_mapping: Optional[torch.Tensor],
                   out_dtype: torch.dtype, status: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Latent attention's cache write.  ``down`` [n, >= q_rank + kv_rank + rot_dim] float32 holds a token's three
    down-projections.  Returns the query latent ``rmsnorm(down[:, :q_rank]) * q_weight`` [n, q_rank] in ``out_dtype``
    (None for ``q_rank`` 0) and writes ``rmsnorm(latent) * kv_weight | rotate(key part)`` as the token's row of
    ``cache_layer``, flat pages [pages, page_size * (kv_rank + rot_dim)].  The rotation pairs element i with
    i + rot/2 over the first ``rot`` elements of the key part; ``cos``/``sin`` [n, rot/2] float32."""
    _cuda(down, q_weight, kv_weight, cos, sin, cache_layer, slot_mapping)
    _f32(q_weight, "query latent norm weight")
    _f32(kv_weight, "latent norm weight")
    _f32(cos, "cos")
    _f32(sin, "sin")
    _i32(slot_mapping, "slot mapping")
    if down.dtype != torch.float32 or down.dim() != 2 or down.stride(1) != 1:
        raise KernelError("the down-projections must be float32 [n, columns] with unit inner stride")
    n = down.shape[0]
    if (q_rank > 0 and (q_weight is None or q_weight.numel() != q_rank)) or kv_weight.numel() != kv_rank:
        raise KernelError("norm weights must be as wide as their latents")
    if rot > 0 and (cos is None or sin is None or cos.shape != (n, rot // 2) or sin.shape != cos.shape):
        raise KernelError("cos/sin must be [n, rot/2]")
    num_pages = 0
    if cache_layer is not None:
        _contig(cache_layer, "cache layer")
        if cache_layer.dtype != out_dtype or cache_layer.dim() != 2 or cache_layer.shape[1] != page_size * (kv_rank + rot_dim):
            raise KernelError(f"cache layer {tuple(cache_layer.shape)} / {cache_layer.dtype} does not fit pages of "
                              f"{page_size} x ({kv_rank} + {rot_dim}) {out_dtype}")
        num_pages = cache_layer.shape[0]
    cq = torch.empty((n, q_rank), dtype=out_dtype, device=down.device) if q_rank > 0 else None
    lib = _lib("latent")
    _check(lib, lib.vapi_latent_prepare(_p(down), ctypes.c_longlong(down.stride(0)), _p(q_weight), _p(kv_weight),
                                        ctypes.c_float(eps), _p(cos), _p(sin), int(rot), _p(cq), _p(cache_layer),
                                        _DT[out_dtype], _p(slot_mapping), n, int(q_rank), int(kv_rank), int(rot_dim),
                                        int(page_size), num_pages, _p(status), _stream()))
    return cq


def latent_rotate_q(q: torch.Tensor, qfull: torch.Tensor, heads: int, dim: int, rot_dim: int, kv_rank: int,
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot: int) -> None:
    """The rotated part of every head's query, ``q`` [n, heads * (dim + rot_dim)], rotated by the token's position
    into the last ``rot_dim`` columns of ``qfull`` [n, heads, kv_rank + rot_dim] (contiguous)."""
    _cuda(q, qfull, cos, sin)
    _f32(cos, "cos")
    _f32(sin, "sin")
    _contig(qfull, "attention queries")
    n = q.shape[0]
    if q.dtype != qfull.dtype or q.stride(1) != 1 or qfull.numel() != n * heads * (kv_rank + rot_dim):
        raise KernelError("queries of one dtype, [n, heads * (dim + rot_dim)] and [n, heads, kv_rank + rot_dim]")
    if rot > 0 and (cos is None or sin is None or cos.shape != (n, rot // 2) or sin.shape != cos.shape):
        raise KernelError("cos/sin must be [n, rot/2]")
    lib = _lib("latent")
    _check(lib, lib.vapi_latent_rotate_q(_p(q), ctypes.c_longlong(q.stride(0)), _p(cos), _p(sin), int(rot), _p(qfull), _dt(q),
                                         n, int(heads), int(dim), int(rot_dim), int(kv_rank), _stream()))


def head_products(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One matrix product per head: ``out[t, h, :] = x[t, h, :] @ w[h]`` for ``x`` [n, heads, k] (any row and head
    strides, unit inner stride), ``w`` [heads, k, m] contiguous and ``out`` [n, heads, m] (likewise strided; made when
    None).  The library's batched product, as :func:`linear` is the library's product."""
    _cuda(x, w, out)
    if x.dim() != 3 or w.dim() != 3 or x.shape[1] != w.shape[0] or x.shape[2] != w.shape[1] or x.dtype != w.dtype or x.stride(2) != 1:
        raise KernelError(f"head products of {tuple(x.shape)} {x.dtype} with {tuple(w.shape)} {w.dtype}")
    if out is None:
        out = torch.empty((x.shape[0], x.shape[1], w.shape[2]), dtype=x.dtype, device=x.device)
    elif out.shape != (x.shape[0], x.shape[1], w.shape[2]) or out.dtype != x.dtype or out.stride(2) != 1:
        raise KernelError("the given output must be [n, heads, m] of the inputs' dtype with unit inner stride")
    torch.bmm(x.transpose(0, 1), w, out=out.transpose(0, 1))
    return out


def latent_attention(q: torch.Tensor, cache_layer: torch.Tensor, page_size: int, block_table: torch.Tensor, cu_q: torch.Tensor,
                     seqlens_k: torch.Tensor, n: int, num_seqs: int, max_q: int, max_k: int, heads: int, kv_rank: int,
                     rot_dim: int, scale: float, *, splits: Optional[int] = None,
                     status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of ``heads`` query heads over one cached row per token, ``[latent (kv_rank) | rotated key part
    (rot_dim)]``: a score is ``scale * q . row`` over the whole row and a head's output is the softmax-weighted sum of
    the rows' latents, so keys and values are the same memory.  ``q`` [n, heads * (kv_rank + rot_dim)] contiguous;
    ``cache_layer`` flat pages [pages, page_size * (kv_rank + rot_dim)]; returns [n, heads * kv_rank]."""
    width = kv_rank + rot_dim
    _contig(q, "queries")
    return masked_attention(q, heads * width, cache_layer, page_size, block_table, cu_q, seqlens_k, n, num_seqs, max_q, max_k,
                            heads, 1, width, kv_rank, scale, splits=splits, status=status, shared_kv=True)


def gated_group_rmsnorm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, group: int,
                        gate_first: bool, out_dtype: torch.dtype, gate: str = "silu") -> torch.Tensor:
    """RMS norm over equal groups of ``group`` columns of the float32 rows ``y`` [n, width] with a
    SiLU gate ``z`` [n, width] (any row stride): ``norm(y) * weight * silu(z)``, or with
    ``gate_first`` ``norm(y * silu(z)) * weight``.  ``weight`` is indexed by column modulo its
    length (one weight per group member, or one per column).  ``gate`` "sigmoid" puts ``sigmoid(z)`` where
    ``silu(z)`` stands."""
    if gate not in ("silu", "sigmoid"):
        raise KernelError(f"gate `{gate}` is not one of silu, sigmoid")
    _cuda(y, z, weight)
    _f32(y, "recurrence output")
    _f32(weight, "norm weight")
    n, width = y.shape
    if z.shape != y.shape or z.stride(1) != 1 or z.dtype != out_dtype:
        raise KernelError("the gate must be [n, width] of the activation dtype with unit inner stride")
    out = torch.empty((n, width), dtype=out_dtype, device=y.device)
    lib = _lib("elementwise")
    _check(lib, lib.vapi_gated_group_rmsnorm(_p(y), _p(z), ctypes.c_longlong(z.stride(0)), _dt(z), _p(weight),
                                             weight.numel(), ctypes.c_float(eps),
                                             (1 if gate_first else 0) | (2 if gate == "sigmoid" else 0), _p(out), n, width,
                                             int(group), _stream()))
    return out


def scale_rows(x: torch.Tensor, factor: float) -> torch.Tensor:
    """``x *= factor`` in place on a contiguous float32 tensor."""
    _cuda(x)
    _f32(x, "rows")
    lib = _lib("elementwise")
    _check(lib, lib.vapi_scale(_p(x), ctypes.c_float(factor), ctypes.c_longlong(x.numel()), _stream()))
    return x


def rope_cos_sin_scaled(positions: torch.Tensor, freq: torch.Tensor, mult: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``mult * cos`` and ``mult * sin`` of ``position * freq`` in float32: two [n, len(freq)] tensors
    (frequencies that an interpolation rule has already changed, and its multiplier)."""
    _cuda(positions, freq)
    _i32(positions, "positions")
    _f32(freq, "frequencies")
    n, half = positions.numel(), freq.numel()
    cos = torch.empty((n, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    lib = _lib("rope")
    _check(lib, lib.vapi_rope_cos_sin_scaled(_p(positions), _p(freq), ctypes.c_float(mult), _p(cos), _p(sin), n, half,
                                             _stream()))
    return cos, sin


def qk_norm_rope_write_split(qkv: torch.Tensor, nh: int, nkv: int, dk: int, dv: int,
                             q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                             cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot: int, interleaved: bool,
                             cache_layer: Optional[torch.Tensor], page_size: int, slot_mapping: Optional[torch.Tensor],
                             status: Optional[torch.Tensor] = None, whole: bool = False,
                             positions: Optional[torch.Tensor] = None, q_temp: Optional[Tuple[float, int]] = None) -> None:
    """:func:`qk_norm_rope_write` for keys of width ``dk`` and values of width ``dv``: ``qkv`` [n, >=
    (nh+nkv)*dk + nkv*dv] holds q heads, k heads, v heads (columns beyond them are left alone);
    the rotation pairs (2i, 2i+1) when ``interleaved``, else (i, i + rot/2); ``cache_layer`` is the
    call site's pages, flat [pages, page_size * nkv * (dk + dv)]: keys [nkv, page_size, dk], then
    values [nkv, page_size, dv].  ``whole``: the RMS norms run over a token's whole q (and whole k), all heads at
    once, with weights of ``nh * dk`` and ``nkv * dk`` elements, instead of per head with weights of ``dk``.
    ``q_temp`` = (coef, every) with ``positions`` [n]: the query at position p is multiplied by
    ``1 + coef * ln(floor((p + 1) / every) + 1)`` (float32) before it is stored."""
    qt_coef, qt_every = (float(q_temp[0]), int(q_temp[1])) if q_temp is not None else (0.0, 0)
    if q_temp is not None and (qt_every < 1 or positions is None or positions.numel() != qkv.shape[0]):
        raise KernelError("a query temperature needs `every` >= 1 and one position per token")
    _cuda(positions)
    _i32(positions, "positions")
    for wt, heads, what in ((q_weight, nh, "q"), (k_weight, nkv, "k")):
        if wt is not None and wt.numel() != (heads * dk if whole else dk):
            raise KernelError(f"the {what} norm's weight has {wt.numel()} elements")
    _cuda(qkv, q_weight, k_weight, cos, sin, cache_layer, slot_mapping)
    _contig(qkv, "qkv")
    _f32(q_weight, "q norm weight")
    _f32(k_weight, "k norm weight")
    _f32(cos, "cos")
    _f32(sin, "sin")
    _i32(slot_mapping, "slot mapping")
    n = qkv.shape[0]
    num_pages = 0
    if cache_layer is not None:
        _contig(cache_layer, "cache layer")
        if cache_layer.dtype != qkv.dtype or cache_layer.dim() != 2 or cache_layer.shape[1] != page_size * nkv * (dk + dv):
            raise KernelError(f"cache layer {tuple(cache_layer.shape)} / {cache_layer.dtype} does not fit pages of "
                              f"{page_size} x {nkv} x ({dk} + {dv}) {qkv.dtype}")
        num_pages = cache_layer.shape[0]
    if cos is not None and (cos.shape != (n, rot // 2) or sin is None or sin.shape != cos.shape):
        raise KernelError("cos/sin must be [n, rot/2]")
    lib = _lib("rope")
    _check(lib, lib.vapi_qk_norm_rope_write_split(
        _p(qkv), ctypes.c_longlong(qkv.stride(0)), _dt(qkv), _p(q_weight), _p(k_weight), ctypes.c_float(eps), _p(cos),
        _p(sin), int(rot), 1 if interleaved else 0, _p(cache_layer), _p(slot_mapping), n, nh, nkv, dk, dv, int(page_size),
        num_pages, 1 if whole else 0, _p(status), _stream(), _p(positions), ctypes.c_float(qt_coef), qt_every))


def masked_attention_splits(num_seqs: int, max_q: int, max_k: int, nh: int, nkv: int) -> int:
    """How many blocks share the keys of one row tile of :func:`masked_attention`: 1 unless the step
    leaves the device idle (few sequences decoding over long contexts)."""
    rows = max_q * (nh // nkv)
    blocks = max(1, num_seqs * nkv * -(-rows // 16))
    sms = sm_count()
    if blocks >= 2 * sms:
        return 1
    return max(1, min(4 * sms // blocks, max_k // 128, 32))


def masked_attention(q: torch.Tensor, q_row_stride: int, cache_layer: torch.Tensor, page_size: int,
                     block_table: torch.Tensor, cu_q: torch.Tensor, seqlens_k: torch.Tensor, n: int, num_seqs: int,
                     max_q: int, max_k: int, nh: int, nkv: int, dk: int, dv: int, scale: float, *, window: int = 0,
                     chunk: int = 0, sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                     splits: Optional[int] = None, status: Optional[torch.Tensor] = None, keep: int = 0,
                     shared_kv: bool = False) -> torch.Tensor:
    """Causal GQA attention of a mixed batch over the paged cache for keys of width ``dk`` and values
    of width ``dv``; returns [n, nh*dv].  A query at position p sees key i iff i <= p, (i > p - window or
    i < keep) (``window`` > 0; ``keep``: the first tokens of a sequence, which a window never leaves behind)
    and i // chunk == p // chunk (``chunk`` > 0).  ``sinks`` [nh] float32 adds
    exp(sink_h) to head h's softmax denominator; ``gate`` [n, nh] (any row stride) multiplies head
    h's output by sigmoid(gate).  ``cache_layer``: flat pages as for :func:`qk_norm_rope_write_split`.
    ``shared_kv``: a page holds key rows alone, [nkv, page_size, dk], and a key's value is the first ``dv`` elements
    of its own row (latent attention)."""
    _cuda(q, cache_layer, block_table, cu_q, seqlens_k, sinks, gate)
    _i32(block_table, "block table")
    _i32(cu_q, "cu_q")
    _i32(seqlens_k, "seqlens_k")
    _f32(sinks, "sinks")
    _contig(cache_layer, "cache layer")
    if cache_layer.dtype != q.dtype:
        raise KernelError("q and the cache must have one dtype")
    if cache_layer.dim() != 2 or cache_layer.shape[1] != page_size * nkv * (dk if shared_kv else dk + dv):
        raise KernelError(f"cache layer {tuple(cache_layer.shape)} does not fit pages of {page_size} x {nkv} x "
                          f"({dk}{'' if shared_kv else f' + {dv}'})")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("block table must be [S, width] with unit inner stride")
    if sinks is not None and sinks.numel() != nh:
        raise KernelError("one sink per head is needed")
    gate_stride = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.shape != (n, nh) or gate.stride(1) != 1:
            raise KernelError("the gate must be [n, heads] of the activation dtype with unit inner stride")
        gate_stride = gate.stride(0)
    if splits is None:
        keys = max_k
        if window > 0:
            keys = min(keys, window + max_q - 1 + max(int(keep), 0))
        if chunk > 0:
            keys = min(keys, chunk + max_q - 1)
        splits = masked_attention_splits(num_seqs, max_q, keys, nh, nkv)
    out = torch.empty((n, nh * dv), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((n * nh * splits * dv,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * nh * splits * 2,), dtype=torch.float32, device=q.device)
    lib = _lib("attention_masked")
    _check(lib, lib.vapi_masked_attention(
        _p(q), ctypes.c_longlong(q_row_stride), _p(cache_layer), _dt(q), _p(block_table), block_table.stride(0), _p(cu_q),
        _p(seqlens_k), _p(sinks), _p(gate), ctypes.c_longlong(gate_stride), _p(out), _p(part_o), _p(part_ml), n, num_seqs,
        max_q, nh, nkv, dk, dv, int(page_size), cache_layer.shape[0], ctypes.c_float(scale), int(window), int(chunk),
        int(splits), _p(status), _stream(), int(keep), 1 if shared_kv else 0),
        2 if splits > 1 or (not shared_kv and q.dtype == torch.bfloat16 and dk == dv == 64 and max_q >= 64 and num_seqs > 1) else 1)
    return out


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor],
                     state_slots: torch.Tensor, tok_seq: torch.Tensor, cu_q: torch.Tensor, positions: torch.Tensor,
                     max_q: int, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`causal_conv` with SiLU behind it."""
    return causal_conv(x, taps, bias, state, state_slots, tok_seq, cu_q, positions, max_q, status, act="silu")


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor],
                state_slots: torch.Tensor, tok_seq: torch.Tensor, cu_q: torch.Tensor, positions: torch.Tensor,
                max_q: int, status: Optional[torch.Tensor] = None, act: str = "none") -> torch.Tensor:
    """``act(bias + causal depthwise convolution)`` (``act``: "none" or "silu") of ``x`` [n, C] (a column range of a wider tensor
    is fine: unit inner stride, any row stride) with ``taps`` [L, C] float32, oldest first.  ``state``
    [slots, >= (L-1)*C] float32 holds each request's last L-1 inputs at its front and is moved on.
    Returns [n, C] in x's dtype."""
    _cuda(x, taps, bias, state, state_slots, tok_seq, cu_q, positions)
    _f32(taps, "conv taps")
    _f32(bias, "conv bias")
    for t, w in ((state_slots, "state slots"), (tok_seq, "tok_seq"), (cu_q, "cu_q"), (positions, "positions")):
        _i32(t, w)
    n, C = x.shape
    L = taps.shape[0]
    if x.stride(1) != 1 or taps.shape[1] != C:
        raise KernelError("x must be [n, C] with unit inner stride and taps [L, C]")
    slot_stride = num_slots = 0
    if L > 1:
        if state is None or state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < (L - 1) * C:
            raise KernelError(f"the state must be float32 [slots, >= {(L - 1) * C}] with unit inner stride")
        slot_stride, num_slots = state.stride(0), state.shape[0]
    out = torch.empty((n, C), dtype=x.dtype, device=x.device)
    lib = _lib("recurrent")
    if act not in ("none", "silu"):
        raise KernelError(f"activation `{act}` is not one of none, silu")
    _check(lib, lib.vapi_causal_conv(
        _p(x), ctypes.c_longlong(x.stride(0)), _dt(x), _p(taps), _p(bias), _p(state if L > 1 else None),
        ctypes.c_longlong(slot_stride), _p(state_slots), _p(tok_seq), _p(cu_q), _p(positions), _p(out), n,
        cu_q.numel() - 1, C, L, num_slots, int(max_q), 1 if act == "silu" else 0, _p(status), _stream()))
    return out


def gated_delta(qkv: torch.Tensor, ab: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, state: torch.Tensor,
                state_offset: int, state_slots: torch.Tensor, cu_q: torch.Tensor, positions: torch.Tensor, nh: int,
                nkv: int, dk: int, dv: int, norm_eps: float = 1e-6, status: Optional[torch.Tensor] = None,
                max_q: int = 1 << 30) -> torch.Tensor:
    """The gated delta rule over every sequence of the step.  ``qkv`` [n, 2*nkv*dk + nh*dv] holds q
    heads, k heads (``nkv`` of ``dk``) and v heads (``nh`` of ``dv``); ``ab`` [n, 2*nh] (unit inner
    stride, any row stride) holds the decay's pre-activation a and the write strength's
    pre-activation b.  Per head: q, k made unit vectors (``norm_eps`` inside the root; q also times
    dk^-1/2); ``S <- g S; u = sigmoid(b) (v - S^T k); S <- S + k u^T; o = S^T q`` with
    ``g = exp(-exp(A_log) softplus(a + dt_bias))``.  ``state`` [slots, >= state_offset + nh*dk*dv]
    float32 carries S [nh, dk, dv] at ``state_offset``.  ``max_q``: the step's longest portion, when known (a
    decode step's kernel may start beside the tail of the kernel before it; a long walk starts on an empty
    device, where its few blocks spread evenly).  Returns o [n, nh*dv] float32."""
    _cuda(qkv, ab, A_log, dt_bias, state, state_slots, cu_q, positions)
    _contig(qkv, "qkv")
    _f32(A_log, "A_log")
    _f32(dt_bias, "dt_bias")
    for t, w in ((state_slots, "state slots"), (cu_q, "cu_q"), (positions, "positions")):
        _i32(t, w)
    n = qkv.shape[0]
    if qkv.shape[1] != 2 * nkv * dk + nh * dv:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected {2 * nkv * dk + nh * dv}")
    if ab.dtype != qkv.dtype or ab.shape != (n, 2 * nh) or ab.stride(1) != 1:
        raise KernelError("a|b must be [n, 2*heads] of qkv's dtype with unit inner stride")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < state_offset + nh * dk * dv:
        raise KernelError("the state must be float32 [slots, >= offset + heads*dk*dv] with unit inner stride")
    out = torch.empty((n, nh * dv), dtype=torch.float32, device=qkv.device)
    lib = _lib("recurrent")
    _check(lib, lib.vapi_gated_delta(
        _p(qkv), ctypes.c_longlong(qkv.stride(0)), 0, nkv * dk, 2 * nkv * dk, _p(ab), ctypes.c_longlong(ab.stride(0)),
        _dt(qkv), _p(A_log), _p(dt_bias), ctypes.c_void_p(state.data_ptr() + 4 * int(state_offset)),
        ctypes.c_longlong(state.stride(0)), _p(state_slots), _p(cu_q), _p(positions), _p(out), cu_q.numel() - 1, nh, nkv,
        dk, dv, state.shape[0], ctypes.c_float(norm_eps), int(min(max_q, 1 << 30)), _p(status), _stream()))
    return out


def state_space(xbc: torch.Tensor, dt: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, D: torch.Tensor,
                state: torch.Tensor, state_offset: int, state_slots: torch.Tensor, cu_q: torch.Tensor,
                positions: torch.Tensor, nh: int, groups: int, n_state: int, head: int,
                status: Optional[torch.Tensor] = None, max_q: int = 1 << 30) -> torch.Tensor:
    """The selective state-space recurrence of Mamba-2 over every sequence of the step.  ``xbc``
    [n, nh*head + 2*groups*n_state] holds x heads, then B and C per group; ``dt`` [n, nh] (unit inner
    stride, any row stride) the step sizes' pre-activations.  Per head, with
    ``step = softplus(dt + dt_bias)``: ``S <- exp(-exp(A_log) step) S + step B x^T; y = S^T C + D x``.
    ``state`` carries S [nh, n_state, head] float32 at ``state_offset``.  ``max_q`` as for :func:`gated_delta`.
    Returns y [n, nh*head] float32."""
    _cuda(xbc, dt, A_log, dt_bias, D, state, state_slots, cu_q, positions)
    _contig(xbc, "x|B|C")
    _f32(A_log, "A_log")
    _f32(dt_bias, "dt_bias")
    _f32(D, "D")
    for t, w in ((state_slots, "state slots"), (cu_q, "cu_q"), (positions, "positions")):
        _i32(t, w)
    n = xbc.shape[0]
    if xbc.shape[1] != nh * head + 2 * groups * n_state:
        raise KernelError(f"x|B|C has {xbc.shape[1]} columns, expected {nh * head + 2 * groups * n_state}")
    if dt.dtype != xbc.dtype or dt.shape != (n, nh) or dt.stride(1) != 1:
        raise KernelError("dt must be [n, heads] of x's dtype with unit inner stride")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < state_offset + nh * n_state * head:
        raise KernelError("the state must be float32 [slots, >= offset + heads*state*head] with unit inner stride")
    out = torch.empty((n, nh * head), dtype=torch.float32, device=xbc.device)
    lib = _lib("recurrent")
    _check(lib, lib.vapi_state_space(
        _p(xbc), ctypes.c_longlong(xbc.stride(0)), _p(dt), ctypes.c_longlong(dt.stride(0)), _dt(xbc), _p(A_log),
        _p(dt_bias), _p(D), ctypes.c_void_p(state.data_ptr() + 4 * int(state_offset)), ctypes.c_longlong(state.stride(0)),
        _p(state_slots), _p(cu_q), _p(positions), _p(out), cu_q.numel() - 1, nh, groups, n_state, head, state.shape[0],
        int(min(max_q, 1 << 30)), _p(status), _stream()))
    return out


# ---------------------------------------------------------------------------------------
# several residual streams, mixers side by side, the gated linear recurrence, a mixture of experts
def embed_sinusoid(table: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor, freq: Optional[torch.Tensor],
                   streams: int = 1, status: Optional[torch.Tensor] = None,
                   pos_table: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows of ``table`` [V, H] for ``tokens`` [n] plus a sinusoidal position vector (entry 2i the sine, entry
    2i+1 the cosine of ``position * freq[i]``; ``freq`` None: nothing is added), as ``streams`` equal copies of
    the float32 residual stream: [n, streams, H].  ``pos_table`` [P, H] of the table's dtype: row ``position`` of it
    is added too, as it is (a learned position vector)."""
    _cuda(table, tokens, positions, freq, pos_table)
    if pos_table is not None:
        _contig(pos_table, "position table")
        if pos_table.dtype != table.dtype or pos_table.dim() != 2 or pos_table.shape[1] != table.shape[1]:
            raise KernelError("the position table must be [positions, H] of the embedding table's dtype")
    _contig(table, "embedding table")
    _i32(tokens, "tokens")
    _i32(positions, "positions")
    _f32(freq, "frequencies")
    n, (vocab, hidden) = tokens.numel(), table.shape
    if freq is not None and freq.numel() != (hidden + 1) // 2:
        raise KernelError(f"{freq.numel()} frequencies for rows of {hidden}")
    out = torch.empty((n, int(streams), hidden), dtype=torch.float32, device=table.device)
    lib = _lib("hyper")
    _check(lib, lib.vapi_embed_sinusoid(_p(table), _dt(table), _p(tokens), _p(positions), _p(freq), _p(pos_table),
                                        0 if pos_table is None else pos_table.shape[0], _p(out), n, hidden,
                                        vocab, int(streams), _p(status), _stream()))
    return out


_NORM_KINDS = {"layer": 0, "rms": 1}


def hyper_read_norm(x: torch.Tensor, y: Optional[torch.Tensor], mix: Optional[torch.Tensor], write: Optional[torch.Tensor],
                    read: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None, kind: str = "layer", branch=None) -> Optional[torch.Tensor]:
    """On the float32 streams ``x`` [n, S, H]: first the pending write of a sublayer's output ``y`` [n, H]
    (``x_t <- sum_s mix[s, t] x_s + write[t] y`` for all t at once; ``y`` None: nothing pending; with
    ``branch`` = ``(y2 | None, w_y, w_y2 | None, eps, scale)`` what is written is
    ``scale * (rmsnorm(y) * w_y + rmsnorm(y2) * w_y2)``, the mean of two mixers' normed outputs), then
    ``u = sum_s read[s] x_s`` (``read`` None: every copy counts once) and its norm with ``weight`` (``kind``
    "layer": ``(u - mean) / sqrt(var + eps) * w``; "rms": ``u / sqrt(mean u^2 + eps) * w``) in ``out_dtype``.
    With ``rows`` only those rows are produced and ``x`` is left untouched; ``weight`` None: only the streams
    are updated (returns None)."""
    _cuda(x, y, mix, write, read, weight, rows)
    _f32(x, "residual streams")
    for t, w in ((mix, "mix matrix"), (write, "write vector"), (read, "read vector"), (weight, "norm weight")):
        _f32(t, w)
    _i32(rows, "rows")
    if x.dim() != 3:
        raise KernelError("the residual streams must be [n, streams, hidden]")
    n, S, hidden = x.shape
    if y is not None:
        _contig(y, "sublayer output")
        if y.shape != (n, hidden) or y.dtype != out_dtype:
            raise KernelError("the sublayer's output must be [n, hidden] of the activation dtype")
        if mix is None or write is None or mix.numel() != S * S or write.numel() != S:
            raise KernelError(f"a pending output needs a mix matrix [{S}, {S}] and a write vector [{S}]")
    if read is not None and read.numel() != S:
        raise KernelError(f"the read vector must have {S} elements")
    if weight is not None and weight.numel() != hidden:
        raise KernelError(f"norm weight has {weight.numel()} elements for rows of {hidden}")
    y2 = wy = wy2 = None
    eps_y, y_scale = 0.0, 1.0
    if branch is not None:
        if y is None:
            raise KernelError("branch norms come with a pending output")
        y2, wy, wy2, eps_y, y_scale = branch
        _cuda(y2, wy, wy2)
        _f32(wy, "branch norm weight")
        _f32(wy2, "branch norm weight")
        if wy is None or wy.numel() != hidden or (y2 is not None and (wy2 is None or wy2.numel() != hidden)):
            raise KernelError(f"branch norm weights must have {hidden} elements")
        if y2 is not None and (not y2.is_contiguous() or y2.shape != y.shape or y2.dtype != y.dtype):
            raise KernelError("the second branch must have the first one's shape and dtype")
    n_out = rows.numel() if rows is not None else n
    out = torch.empty((n_out, hidden), dtype=out_dtype, device=x.device) if weight is not None else None
    lib = _lib("hyper")
    _check(lib, lib.vapi_hyper_read_norm(_p(x), _p(y), _p(y2), _DT[out_dtype], _p(wy), _p(wy2), ctypes.c_float(eps_y),
                                         ctypes.c_float(y_scale), _p(mix), _p(write), _p(read), _p(weight),
                                         ctypes.c_float(eps), _NORM_KINDS[kind], _p(rows), _p(out), n_out, hidden, S,
                                         _stream()))
    return out


def branch_rmsnorm_mean(branches, weights, eps: float, scale: float) -> torch.Tensor:
    """``scale * sum_b rmsnorm(branches[b]) * weights[b]`` over up to four [n, H] tensors of one dtype."""
    _cuda(*branches, *weights)
    if not 1 <= len(branches) <= 4 or len(weights) != len(branches):
        raise KernelError("one to four branches, each with its weight")
    a0 = branches[0]
    for a, w in zip(branches, weights):
        _contig(a, "branch output")
        _f32(w, "norm weight")
        if a.shape != a0.shape or a.dtype != a0.dtype or w.numel() != a0.shape[1]:
            raise KernelError("branches must agree in shape and dtype, weights in length")
    n, hidden = a0.shape
    out = torch.empty_like(a0)
    ptrs = (ctypes.c_void_p * len(branches))(*[a.data_ptr() for a in branches])
    wptrs = (ctypes.c_void_p * len(branches))(*[w.data_ptr() for w in weights])
    lib = _lib("hyper")
    _check(lib, lib.vapi_branch_rmsnorm_mean(ptrs, wptrs, len(branches), _dt(a0), ctypes.c_float(eps), ctypes.c_float(scale),
                                             _p(out), n, hidden, _stream()))
    return out


def sigmoid_gate(y: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``y * sigmoid(gate)`` for ``y`` [n, width] contiguous and ``gate`` [n, width] of the same dtype (unit inner
    stride, any row stride: a column range of a wider product)."""
    _cuda(y, gate)
    _contig(y, "gated tensor")
    if gate.shape != y.shape or gate.dtype != y.dtype or gate.stride(1) != 1:
        raise KernelError("the gate must have the tensor's shape and dtype and unit inner stride")
    out = torch.empty_like(y)
    lib = _lib("hyper")
    _check(lib, lib.vapi_sigmoid_gate(_p(y), _p(gate), ctypes.c_longlong(gate.stride(0)), _dt(y), _p(out), y.shape[0],
                                      y.shape[1], _stream()))
    return out


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """``x <- cap * tanh(x / cap)`` in place on a contiguous float32 tensor."""
    _cuda(x)
    _f32(x, "logits")
    lib = _lib("hyper")
    _check(lib, lib.vapi_softcap(_p(x), ctypes.c_float(cap), ctypes.c_longlong(x.numel()), _stream()))
    return x


def rglru(u: torch.Tensor, y: torch.Tensor, w_a: torch.Tensor, b_a: torch.Tensor, w_i: torch.Tensor, b_i: torch.Tensor,
          lam: torch.Tensor, decay_c: float, state: torch.Tensor, state_offset: int, state_slots: torch.Tensor,
          cu_q: torch.Tensor, positions: torch.Tensor, status: Optional[torch.Tensor] = None,
          max_q: int = 1 << 30) -> torch.Tensor:
    """The real-gated linear recurrent unit over every sequence of the step.  ``u`` [n, C] (contiguous) is the
    recurrence's input, ``y`` [n, C] (unit inner stride, any row stride) the other branch before its GELU;
    ``w_a``, ``w_i`` [blocks, C/blocks, C/blocks] (stored [out, in], u's dtype) and ``b_a``, ``b_i`` [C] float32 give
    ``r = sigmoid(W_a u + b_a)`` and ``i = sigmoid(W_i u + b_i)`` block by block; ``a = exp(-decay_c r softplus(lam))``;
    ``S <- a S + sqrt(1 - a^2) i u``; returns ``S * gelu_tanh(y)`` [n, C] in u's dtype.  ``state`` [slots, >=
    state_offset + C] float32 carries S at ``state_offset``."""
    _cuda(u, y, w_a, b_a, w_i, b_i, lam, state, state_slots, cu_q, positions)
    _contig(u, "recurrence input")
    _contig(w_a, "recurrence gate matrix")
    _contig(w_i, "input gate matrix")
    for t, w in ((b_a, "gate bias"), (b_i, "gate bias"), (lam, "decay parameter")):
        _f32(t, w)
    for t, w in ((state_slots, "state slots"), (cu_q, "cu_q"), (positions, "positions")):
        _i32(t, w)
    n, C = u.shape
    blocks = w_a.shape[0]
    if w_a.shape != (blocks, C // blocks, C // blocks) or w_i.shape != w_a.shape or C % blocks:
        raise KernelError(f"gate matrices {tuple(w_a.shape)} do not fit {C} channels")
    if w_a.dtype != u.dtype or w_i.dtype != u.dtype or y.dtype != u.dtype:
        raise KernelError("the gate matrices and the other branch must have the input's dtype")
    if y.shape != (n, C) or y.stride(1) != 1:
        raise KernelError("the other branch must be [n, C] with unit inner stride")
    if b_a.numel() != C or b_i.numel() != C or lam.numel() != C:
        raise KernelError(f"gate biases and the decay parameter must have {C} elements")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < state_offset + C:
        raise KernelError("the state must be float32 [slots, >= offset + C] with unit inner stride")
    a_buf = torch.empty((n, C), dtype=torch.float32, device=u.device)
    g_buf = torch.empty((n, C), dtype=torch.float32, device=u.device)
    out = torch.empty((n, C), dtype=u.dtype, device=u.device)
    lib = _lib("rglru")
    _check(lib, lib.vapi_rglru(
        _p(u), ctypes.c_longlong(u.stride(0)), _p(y), ctypes.c_longlong(y.stride(0)), _dt(u), _p(w_a), _p(b_a), _p(w_i),
        _p(b_i), _p(lam), ctypes.c_float(decay_c), _p(a_buf), _p(g_buf),
        ctypes.c_void_p(state.data_ptr() + 4 * int(state_offset)), ctypes.c_longlong(state.stride(0)), _p(state_slots),
        _p(cu_q), _p(positions), _p(out), n, cu_q.numel() - 1, C, blocks, state.shape[0], int(min(max_q, 1 << 30)),
        _p(status), _stream()), 2)
    return out


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    """``relu(x)^2`` elementwise."""
    _cuda(x)
    _contig(x, "activations")
    out = torch.empty_like(x)
    lib = _lib("moe")
    _check(lib, lib.vapi_relu_squared(_p(x), _p(out), _dt(x), ctypes.c_longlong(x.numel()), _stream()))
    return out


def moe_route(h: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], experts: int, top: int, groups: int,
              keep: int, bias: Optional[torch.Tensor] = None, score: str = "softmax"):
    """The router of a mixture of experts for ``h`` [n, W]: ``router`` [outputs, W] and ``correction`` [outputs]
    float32, ``outputs`` = ``experts`` + identity experts.  Scores are the softmax of the float32 logits over all
    outputs; the ``top`` largest of score + correction win, among the outputs of the ``keep`` best of ``groups``
    equal groups of neighbours (a group's score is its largest score + correction); the weights are the chosen
    scores divided by their sum (+ 1e-20).  Returns ``(ids [n, top] int32, weights [n, top] float32, plan)``;
    ``plan`` lists the step's (token, choice) pairs expert by expert for :func:`moe_experts`.  ``bias`` [outputs] is
    added to the logits.  ``score`` "chosen": the ``top`` largest logits win and the weights are the softmax over
    the chosen logits only (no correction)."""
    _cuda(h, router, correction, bias)
    _f32(bias, "router bias")
    if score not in ("softmax", "chosen"):
        raise KernelError(f"score `{score}` is not one of softmax, chosen")
    _contig(h, "router input")
    _f32(router, "router matrix")
    _f32(correction, "router correction")
    n, W = h.shape
    outputs = router.shape[0]
    if router.shape != (outputs, W) or (correction is not None and correction.numel() != outputs) or \
            (bias is not None and bias.numel() != outputs):
        raise KernelError("the router must be [outputs, W], the correction and the bias [outputs]")
    dev = h.device
    pairs = n * top
    ids = torch.empty((n, top), dtype=torch.int32, device=dev)
    wts = torch.empty((n, top), dtype=torch.float32, device=dev)
    # ranks | offsets | pair_of | number of tiles | tile_expert | tile_row0, one allocation
    max_tiles = pairs // 64 + max(experts, 1)
    sizes = [pairs, experts + 1, pairs, 1, max_tiles, max_tiles]
    book = torch.empty((sum(sizes),), dtype=torch.int32, device=dev)
    parts, at = [], 0
    for z in sizes:
        parts.append(book[at:at + z])
        at += z
    ranks, offsets, pair_of, ntiles, tile_expert, tile_row0 = parts
    lib = _lib("moe")
    _check(lib, lib.vapi_moe_route(_p(h), _dt(h), _p(router), _p(correction), _p(bias), 1 if score == "chosen" else 0,
                                   _p(ids), _p(wts), _p(ranks),
                                   _p(offsets), _p(pair_of), _p(ntiles), _p(tile_expert), _p(tile_row0), n, W, outputs,
                                   int(experts), int(top), int(groups), int(keep), _stream()), 2 if experts > 0 else 1)
    return ids, wts, (offsets, pair_of, ntiles, tile_expert, tile_row0)


def moe_table_route(tokens: torch.Tensor, table: torch.Tensor, experts: int, status: Optional[torch.Tensor] = None):
    """A mixture of experts without a router: row ``tokens[t]`` of ``table`` [vocab, top] int32 names token t's
    experts, each with weight ``1 / top``.  Returns what :func:`moe_route` returns."""
    _cuda(tokens, table)
    _i32(tokens, "tokens")
    _i32(table, "expert table")
    _contig(table, "expert table")
    if table.dim() != 2:
        raise KernelError("the expert table must be [vocab, top]")
    n, (vocab, top) = tokens.numel(), table.shape
    dev = tokens.device
    pairs = n * top
    ids = torch.empty((n, top), dtype=torch.int32, device=dev)
    wts = torch.empty((n, top), dtype=torch.float32, device=dev)
    max_tiles = pairs // 64 + max(experts, 1)
    sizes = [pairs, experts + 1, pairs, 1, max_tiles, max_tiles]
    book = torch.empty((sum(sizes),), dtype=torch.int32, device=dev)
    parts, at = [], 0
    for z in sizes:
        parts.append(book[at:at + z])
        at += z
    ranks, offsets, pair_of, ntiles, tile_expert, tile_row0 = parts
    lib = _lib("moe")
    _check(lib, lib.vapi_moe_table_route(_p(tokens), _p(table), int(vocab), _p(ids), _p(wts), _p(ranks), _p(offsets),
                                         _p(pair_of), _p(ntiles), _p(tile_expert), _p(tile_row0), n, int(experts), int(top),
                                         _p(status), _stream()), 2)
    return ids, wts, (offsets, pair_of, ntiles, tile_expert, tile_row0)


def moe_experts(h: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, plan, w_up: Optional[torch.Tensor],
                w_down: Optional[torch.Tensor], shared: Optional[torch.Tensor] = None, gated: bool = False,
                act: Tuple[float, float, float] = (0.0, 1.0, 0.0)) -> torch.Tensor:
    """The weighted sum of the chosen experts' outputs for ``h`` [n, W]: expert e is ``W_down[e] relu(W_up[e] h)^2``
    with ``w_up`` [experts, ff, W] and ``w_down`` [experts, W, ff] of h's dtype; a choice >= experts is an identity
    expert (its output is h); ``shared`` [n, W] is added when given.  ``ids``, ``wts``, ``plan``: from
    :func:`moe_route`.  ``gated``: expert e is ``W_down[e] (silu(W_gate[e] h) * (W_up[e] h))`` and ``w_up`` is
    [experts, 2 * ff, W] with rows alternating gate_0, up_0, gate_1, up_1, ...  ``act`` = (limit, alpha, shift)
    generalises the gated form to ``g' * sigmoid(alpha g') * (u' + shift)`` with ``g' = min(g, limit)`` and
    ``u' = clamp(u, -limit, limit)`` when ``limit`` > 0 (the default is SiLU gating)."""
    _cuda(h, ids, wts, w_up, w_down, shared)
    limit, alpha, shift = (ctypes.c_float(float(v)) for v in act)
    _contig(h, "expert input")
    n, W = h.shape
    top = ids.shape[1]
    experts = 0 if w_up is None else w_up.shape[0]
    pairs = n * top
    y = None
    lib = _lib("moe")
    if experts > 0:
        rows_up = w_up.shape[1]
        ff = rows_up // 2 if gated else rows_up
        _contig(w_up, "expert up matrices")
        _contig(w_down, "expert down matrices")
        if w_up.shape != (experts, rows_up, W) or (gated and rows_up % 2) or w_down.shape != (experts, W, ff) or w_up.dtype != h.dtype or w_down.dtype != h.dtype:
            raise KernelError("expert matrices must be [experts, ff, W] and [experts, W, ff] of the input's dtype")
        offsets, pair_of, ntiles, tile_expert, tile_row0 = plan
        hid = torch.empty((pairs, ff), dtype=h.dtype, device=h.device)
        y = torch.empty((pairs, W), dtype=torch.float32, device=h.device)
        _check(lib, lib.vapi_moe_grouped(_p(h), ctypes.c_longlong(h.stride(0)), _p(w_up), _dt(h), _p(ntiles), _p(tile_expert),
                                         _p(tile_row0), _p(offsets), _p(pair_of), _p(wts), _p(hid), pairs, experts, rows_up, W,
                                         top, 2 if gated else 0, _stream(), limit, alpha, shift))
        _check(lib, lib.vapi_moe_grouped(_p(hid), ctypes.c_longlong(ff), _p(w_down), _dt(h), _p(ntiles), _p(tile_expert),
                                         _p(tile_row0), _p(offsets), _p(pair_of), _p(wts), _p(y), pairs, experts, W, ff,
                                         top, 1, _stream(), limit, alpha, shift))
    if shared is not None:
        _contig(shared, "shared expert output")
        if shared.shape != h.shape or shared.dtype != h.dtype:
            raise KernelError("the shared expert's output must have the input's shape and dtype")
    out = torch.empty_like(h)
    _check(lib, lib.vapi_moe_combine(_p(y), _p(ids), _p(wts), _p(h), _p(shared), _p(out), _dt(h), n, W, top, experts,
                                     _stream()))
    return out


# ---------------------------------------------------------------------------------------
# mixers whose state is a decayed sum of outer products: the matrix memory (mLSTM) and gated linear attention
def _linear_memory_args(qkv, nh, dk, dv, state, need, state_slots, cu_q, positions):
    _cuda(qkv, state, state_slots, cu_q, positions)
    for t, w in ((state_slots, "state slots"), (cu_q, "cu_q"), (positions, "positions")):
        _i32(t, w)
    if qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[1] < 2 * nh * dk + nh * dv:
        raise KernelError(f"q|k|v needs {2 * nh * dk + nh * dv} columns with unit inner stride")
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < need:
        raise KernelError(f"the state must be float32 [slots, >= {need}] with unit inner stride")


def matrix_memory(qkv: torch.Tensor, gates: torch.Tensor, gate_bias: Optional[torch.Tensor], cap: float, state: torch.Tensor,
                  state_slots: torch.Tensor, cu_q: torch.Tensor, positions: torch.Tensor, nh: int, dk: int, dv: int,
                  q_scale: float, floor_eps: float = 1e-6, status: Optional[torch.Tensor] = None,
                  max_q: int = 1 << 30) -> torch.Tensor:
    """The matrix memory of the mLSTM over every sequence of the step.  ``qkv`` [n, >= 2*nh*dk + nh*dv] (unit inner
    stride, any row stride) holds q heads, k heads (``nh`` of ``dk``) and v heads (``nh`` of ``dv``); ``gates``
    [n, 2*nh] float32 (unit inner stride) the pre-activations of the input gates, then of the forget gates, and
    ``gate_bias`` [2*nh] what is added to them.  Per head, with ``li = cap tanh(a_i / cap)``,
    ``lf = logsigmoid(cap tanh(a_f / cap))`` and a running maximum m that starts at 0:
    ``m' = max(lf + m, li); S <- exp(lf + m - m') S + exp(li - m') k v^T``, n likewise with k alone, and
    ``o = S^T (q_scale q) / (max(|n . q_scale q|, exp(-m')) + floor_eps)``.  ``state`` [slots, >= nh*dk*dv + nh*dk + nh]
    float32 carries S [nh, dv, dk] (column by column: a value column's key rows side by side), n [nh, dk] and m [nh].
    Returns o [n, nh*dv] float32."""
    need = nh * dk * dv + nh * dk + nh
    _linear_memory_args(qkv, nh, dk, dv, state, need, state_slots, cu_q, positions)
    _cuda(gates, gate_bias)
    _f32(gate_bias, "gate bias")
    n = qkv.shape[0]
    if gates.dtype != torch.float32 or gates.shape != (n, 2 * nh) or gates.stride(1) != 1:
        raise KernelError("the gates must be float32 [n, 2*heads] with unit inner stride")
    if gate_bias is not None and gate_bias.numel() != 2 * nh:
        raise KernelError("the gates' bias must have 2*heads elements")
    out = torch.empty((n, nh * dv), dtype=torch.float32, device=qkv.device)
    lib = _lib("linear_memory")
    _check(lib, lib.vapi_matrix_memory(
        _p(qkv), ctypes.c_longlong(qkv.stride(0)), 0, nh * dk, 2 * nh * dk, _dt(qkv), _p(gates),
        ctypes.c_longlong(gates.stride(0)), _p(gate_bias), ctypes.c_float(cap), ctypes.c_float(q_scale),
        ctypes.c_float(floor_eps), _p(state), ctypes.c_longlong(state.stride(0)), _p(state_slots), _p(cu_q), _p(positions),
        _p(out), cu_q.numel() - 1, nh, dk, dv, state.shape[0], int(min(max_q, 1 << 30)), _p(status), _stream()))
    return out


def gated_linear_attention(qkv: torch.Tensor, decay_logits: torch.Tensor, tau: float, state: torch.Tensor,
                           state_slots: torch.Tensor, cu_q: torch.Tensor, positions: torch.Tensor, nh: int, dk: int, dv: int,
                           q_scale: float, status: Optional[torch.Tensor] = None, max_q: int = 1 << 30) -> torch.Tensor:
    """Gated linear attention over every sequence of the step.  ``qkv`` as for :func:`matrix_memory`;
    ``decay_logits`` [n, nh*dk] float32 (unit inner stride) holds z, and key channel r of a head decays by
    ``alpha = sigmoid(z)^(1/tau)``: ``S <- diag(alpha) S + k v^T; o = S^T (q_scale q)``.  ``state``
    [slots, >= nh*dk*dv] float32 carries S [nh, dv, dk] (column by column).  Returns o [n, nh*dv] float32.  ``decay_logits`` is scratch:
    a step with portions of 16 tokens or more (``max_q``) leaves the decays in it, worked out once per element by a
    kernel of their own instead of by every block of a head."""
    _linear_memory_args(qkv, nh, dk, dv, state, nh * dk * dv, state_slots, cu_q, positions)
    _cuda(decay_logits)
    n = qkv.shape[0]
    if decay_logits.dtype != torch.float32 or decay_logits.shape != (n, nh * dk) or decay_logits.stride(1) != 1:
        raise KernelError("the decay's logits must be float32 [n, heads*dk] with unit inner stride")
    if not tau > 0:
        raise KernelError("tau must be positive")
    out = torch.empty((n, nh * dv), dtype=torch.float32, device=qkv.device)
    lib = _lib("linear_memory")
    _check(lib, lib.vapi_gated_linear_attention(
        _p(qkv), ctypes.c_longlong(qkv.stride(0)), 0, nh * dk, 2 * nh * dk, _dt(qkv), _p(decay_logits),
        ctypes.c_longlong(decay_logits.stride(0)), ctypes.c_float(1.0 / tau), ctypes.c_float(q_scale), _p(state),
        ctypes.c_longlong(state.stride(0)), _p(state_slots), _p(cu_q), _p(positions), _p(out), n, cu_q.numel() - 1, nh, dk, dv,
        state.shape[0], int(min(max_q, 1 << 30)), _p(status), _stream()), 2 if max_q >= 16 else 1)
    return out
