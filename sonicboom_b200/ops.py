"""Python face of the kernel library: each function checks its tensors, then calls one
`extern "C"` entry point on torch's current CUDA stream.

Nothing here computes with torch; a tensor that is not on a CUDA device, or a missing
library, is an error (there is no CPU path).  Shapes a kernel does not take are refused by
the kernel's own host-side checks, whose message is raised here.
"""
from __future__ import annotations

import ctypes

import torch

from . import abi as _abi
from .csrc import build as _build

F32, BF16 = 0, 1
EPI_NONE, EPI_BIAS, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
SWIGLU_BLOCK = 8                 # rows of gate and up alternate in blocks of this many
SKINNY_MAX_ROWS = 64             # bfloat16 products of at most this many rows stream the weights
DECODE_ATTENTION_ROWS = 16       # query rows (new tokens x heads) of one key/value head that the split decode attention takes


class KernelError(RuntimeError):
    pass


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = _abi.apply(_build.load(), _abi.CORE)
    return _lib


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 and bfloat16 tensors, not {dtype}")


def _ptr(t):
    """The device address of a tensor as the typed entry points take it (an int; None is a null
    pointer).  A step makes a few thousand of these, so no ctypes object is made here."""
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors only; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError("kernels take contiguous tensors")
    return t.data_ptr()


# torch.cuda.current_stream() resolves the device, builds a Stream object and costs several
# microseconds; a prompt step asks for the stream some four hundred times.  The raw handle of
# the current device's current stream is one call where torch has it.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = 0          # kernels launched through this module so far (a running count)


# Opt-in NVTX ranges around steps and schedule entries, in the manner of the reference's
# SONICBOOM_NVTX switch (core/src/model/gemma4_plan.cpp:50, 87-91): SB_TRACE=1 in the
# environment or `set_trace(True)`.  Off, `trace_range` hands out one shared no-op object.
import contextlib as _contextlib
import os as _os

TRACE = _os.environ.get("SB_TRACE", "0") not in ("", "0")
_NO_RANGE = _contextlib.nullcontext()


def set_trace(on: bool) -> None:
    global TRACE
    TRACE = bool(on)


class _Range:
    def __init__(self, name):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()


def trace_range(name: str):
    """A context manager that is an NVTX range when tracing is on, else nothing."""
    return _Range(name) if TRACE else _NO_RANGE


def _check(rc: int, what: str, launches: int = 1) -> None:
    global LAUNCHES
    if rc != 0:
        raise KernelError(f"{what}: {lib().sb_last_error().decode()}")
    LAUNCHES += launches


def _i32(t, what):
    if t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")
    return _ptr(t)


def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
          scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[tokens[t]] * scale as float32; an id outside the table gives a row of NaN."""
    n, width = tokens.numel(), table.shape[1]
    assert out.dtype == torch.float32 and out.shape == (n, width)
    _check(lib().sb_embed(_i32(tokens, "tokens"), n, _ptr(table), _code(table.dtype),
                          table.shape[0], width, ctypes.c_float(scale), _ptr(out), _stream()), "embed")
    return out


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[m, n] += bias[n] in place (x float32 [rows, width])."""
    assert x.dtype == torch.float32 and x.dim() == 2 and bias.numel() == x.shape[1]
    _check(lib().sb_add_bias(_ptr(x), _ptr(bias), _code(bias.dtype), x.shape[0], x.shape[1], _stream()),
           "add_bias")
    return x


def softcap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap) in place (float32)."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(lib().sb_softcap(_ptr(x), ctypes.c_size_t(x.numel()), ctypes.c_float(cap), _stream()),
           "softcap")
    return x


def scale(x: torch.Tensor, c: float) -> torch.Tensor:
    """x *= c in place (float32)."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(lib().sb_scale(_ptr(x), ctypes.c_size_t(x.numel()), ctypes.c_float(c), _stream()), "scale")
    return x


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: torch.Tensor | None = None, width: int | None = None) -> torch.Tensor:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x is the float32 residual stream.  With
    `width`, only the first `width` values of every row of x are normed (and written)."""
    assert x.dtype == torch.float32 and x.dim() == 2
    n = out.shape[0]
    ld = x.shape[1]
    width = ld if width is None else width
    assert out.shape[1] == width and weight.numel() == width and width <= ld
    if rows is None:
        assert x.shape[0] == n
    _check(lib().sb_rmsnorm_ld(_ptr(x), ld, _i32(rows, "rows") if rows is not None else _ptr(None), n,
                               width, _ptr(weight), _code(weight.dtype), ctypes.c_float(eps),
                               _ptr(out), _code(out.dtype), _stream()), "rmsnorm")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    out = torch.empty_like(x, dtype=dtype)
    _check(lib().sb_cast(_ptr(x), _code(x.dtype), _ptr(out), _code(dtype),
                         ctypes.c_size_t(x.numel()), _stream()), "cast")
    return out


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
           bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
           kernel: str = "auto", norm: tuple | None = None,
           warm: torch.Tensor | None = None, gate: tuple | None = None,
           gate_kind: int = 0) -> torch.Tensor:
    """out = a @ w.T with a fused epilogue; a [M,K], w [N,K]; float32 accumulation.

    `gate` = (limit, slope) with EPI_SWIGLU makes the gated epilogue the clamped form
    a * sigmoid(slope a) * (b + 1), a = min(gate, limit), b = clamp(up, -limit, limit): inside the
    tcgen05 and the weight-streaming kernels where they run, else as the plain product followed
    by `glu_clamped`.

    `gate_kind` = GATE_GELU_TANH with EPI_SWIGLU: gelu(gate) * up in gelu's tanh form, in the same
    places (inside the tcgen05 and the weight-streaming kernels, else the plain product followed by
    `gated_act`).

    `norm` = (weight, eps, norm_out) also writes norm_out = rmsnorm(out, weight, eps) [M,N]
    (out must be float32): in the kernel that finishes the product where one does (the split-K
    decode form of the tcgen05 kernel), else with the norm kernel after it.
    `warm`: weights that a later kernel streams; the blocks of the tcgen05 kernel ask for them
    into L2 as they end (other kernels ignore it).  A hint: it changes no result.  It pays only
    for a consumer that cannot request its own weights early (see `requests_weights_late`).

    bfloat16 operands run on tensor cores: `kernel` "tc5" (TMA + tcgen05), "skinny" (weights
    streamed into mma.sync fragments, at most SKINNY_MAX_ROWS rows), "tiled" (mma.sync tiles),
    or "auto", which picks between the first two (see `_pick_kernel`).  float32 operands, inner
    sizes that are not multiples of 8, and `kernel="plain"` run the plain FFMA kernel.  A
    bfloat16 activation with a float32 weight is cast to float32 first.  The split-K decode
    form keeps one workspace per device, so products on one device must be ordered in a stream.
    """
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K, f"linear: a is [{M},{K}], w is {tuple(w.shape)}"
    n_out = N // 2 if epilogue == EPI_SWIGLU else N
    assert tuple(out.shape) == (M, n_out), f"linear: out is {tuple(out.shape)}, want {(M, n_out)}"
    if a.dtype != w.dtype:
        a = cast(a, torch.float32)
        if w.dtype != torch.float32:
            raise KernelError("linear: a float32 activation needs float32 weights")
    if gate_kind == GATE_GELU_TANH:
        assert epilogue == EPI_SWIGLU and gate is None
    if gate is not None or gate_kind == GATE_GELU_TANH:
        assert epilogue == EPI_SWIGLU and N % (2 * SWIGLU_BLOCK) == 0
        limit, slope = gate if gate is not None else (0.0, 1.0)
        kind = GATE_CLAMPED if gate is not None else GATE_GELU_TANH
        picked = kernel if kernel != "auto" else _pick_kernel(M, N, K, a.device)
        fused = a.dtype == torch.bfloat16 and K % 8 == 0 and picked == "tc5"
        if a.dtype == torch.bfloat16 and K % 8 == 0 and picked == "skinny" and M <= SKINNY_MAX_ROWS:
            _check(lib().sb_gemm_skinny_gated(_ptr(a), BF16, _ptr(w), BF16, M, N, K, _ptr(out), _code(out.dtype),
                                              ctypes.c_float(limit), ctypes.c_float(slope), kind, _stream()),
                   "linear (weight-streaming kernel, gated)")
            return out
        if not fused:
            gu = torch.empty((M, N), dtype=torch.float32, device=a.device)
            linear(a, w, gu, EPI_NONE, kernel=kernel)
            return gated_act(gu, kind, out, interleaved=True, limit=limit, slope=slope)
        kernel = "tc5"
    args = (_ptr(a), _code(a.dtype), _ptr(w), _code(w.dtype), M, N, K, epilogue, _ptr(bias),
            _code(bias.dtype) if bias is not None else 0, _ptr(residual), _ptr(out),
            _code(out.dtype), _stream())
    if residual is not None:
        assert residual.dtype == torch.float32 and tuple(residual.shape) == (M, N)
    if bias is not None:
        assert bias.numel() == N
    fast = a.dtype == torch.bfloat16 and kernel != "plain" and K % 8 == 0
    l = lib()
    if norm is not None:
        norm_w, norm_eps, norm_out = norm
        assert out.dtype == torch.float32 and epilogue != EPI_SWIGLU
        assert norm_w.numel() == N and tuple(norm_out.shape) == (M, N)
        fuses = fast and kernel in ("auto", "tc5") and bool(l.sb_gemm_tc5_fuses_norm(
            M, N, K, _sm_count(a.device), epilogue, _code(out.dtype), 0))
        if fuses and (kernel == "tc5" or FORCE_DECODE_KERNEL != "skinny"):
            kernel = "tc5"
        else:
            linear(a, w, out, epilogue, bias, residual, kernel, warm=warm)
            rmsnorm(out, norm_w, norm_eps, norm_out)
            return out
    if kernel == "auto" and fast:
        kernel = _pick_kernel(M, N, K, a.device)
    if fast and kernel in ("tc5", "tc5_normal"):
        form = 1 if kernel == "tc5_normal" else 0
        ws = _tc5_workspace(M, N, K, a.device) if form == 0 else None
        extras = None
        if norm is not None or (warm is not None and WARM) or gate is not None or gate_kind == GATE_GELU_TANH:
            extras = LinearExtras()
            extras.gate_kind = gate_kind if gate_kind == GATE_GELU_TANH else 0
            if gate is not None:
                extras.gate_limit, extras.gate_slope = float(gate[0]), float(gate[1])
            if norm is not None:
                extras.norm_weight, extras.norm_weight_dtype = norm_w.data_ptr(), _code(norm_w.dtype)
                extras.norm_eps, extras.norm_out = norm_eps, norm_out.data_ptr()
                extras.norm_out_dtype = _code(norm_out.dtype)
            if warm is not None and WARM:
                extras.warm, extras.warm_bytes = warm.data_ptr(), warm.numel() * warm.element_size()
        _check(l.sb_gemm_tc5_ex(*args[:-1], _ptr(ws), ctypes.c_size_t(ws.numel() if ws is not None else 0),
                                _sm_count(a.device), form,
                                ctypes.byref(extras) if extras is not None else None, _stream()),
               "linear (tcgen05 kernel)",
               launches=2 if ws is not None else 1)        # a split product adds its reduce kernel
    elif fast and kernel == "skinny":
        _check(l.sb_gemm_skinny(*args), "linear (weight-streaming kernel)")
    elif fast and kernel == "tiled":
        _check(l.sb_gemm_tiled(*args), "linear (tiled kernel)")
    elif kernel in ("plain", "auto") or not fast:
        _check(l.sb_gemm_plain(*args), "linear (plain kernel)")
    else:
        raise KernelError(f"linear: unknown kernel {kernel!r}")
    return out


class RopeStore(ctypes.Structure):
    """SbRopeStore of the kernel library: the rotation + cache write that finishes a q|k|v product."""
    _fields_ = [("n_q_heads", ctypes.c_int), ("n_kv_heads", ctypes.c_int), ("hd", ctypes.c_int),
                ("rot", ctypes.c_int), ("inv_freq", ctypes.c_void_p), ("row_seq", ctypes.c_void_p),
                ("row_pos", ctypes.c_void_p), ("page_off", ctypes.c_void_p), ("page_ids", ctypes.c_void_p),
                ("page_size", ctypes.c_int), ("cache", ctypes.c_void_p), ("q_out", ctypes.c_void_p)]


class LinearExtras(ctypes.Structure):
    """SbLinearExtras of the kernel library: what may accompany a product."""
    _fields_ = [("norm_weight", ctypes.c_void_p), ("norm_weight_dtype", ctypes.c_int),
                ("norm_eps", ctypes.c_float), ("norm_out", ctypes.c_void_p),
                ("norm_out_dtype", ctypes.c_int), ("warm", ctypes.c_void_p),
                ("warm_bytes", ctypes.c_size_t), ("rope", ctypes.POINTER(RopeStore)),
                ("gate_limit", ctypes.c_float), ("gate_slope", ctypes.c_float), ("gate_kind", ctypes.c_int)]


def qkv_rope_store(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, n_q_heads: int,
                   n_kv_heads: int, head_dim: int, rotary_dim: int, inv_freq: torch.Tensor, row_seq,
                   row_pos, page_off, page_ids, page_size: int, cache: torch.Tensor | None,
                   q_out: torch.Tensor) -> torch.Tensor:
    """The fused [q | k | v] projection of the rows `h` (+ bias), the rotation of q and k, q into
    `q_out` [rows, heads, hd] and k, v into the cache pages (`cache=None`: the weight holds the
    query rows only).  Where the split-K decode form of the tcgen05 product runs (9 to 64 rows of
    bfloat16), its reduce kernel does the rotation and the cache write too and the float32 row
    is never written; else the product and `rope_store` run one after the other."""
    M, K = h.shape
    N = w.shape[0]
    has_kv = cache is not None
    l = lib()
    fused = (h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16
             and (not has_kv or cache.dtype == torch.bfloat16) and K % 8 == 0
             and (bias is None or bias.numel() == N)
             and _pick_kernel(M, N, K, h.device) == "tc5"
             and bool(l.sb_gemm_tc5_fuses_rope(M, N, K, _sm_count(h.device), n_q_heads, n_kv_heads, head_dim,
                                              rotary_dim, 1 if has_kv else 0)))
    if not fused:
        qkv = torch.empty((M, N), dtype=torch.float32, device=h.device)
        linear(h, w, qkv, EPI_BIAS if bias is not None else EPI_NONE, bias=bias)
        return rope_store(qkv, n_q_heads, n_kv_heads, head_dim, rotary_dim, inv_freq, row_seq, row_pos,
                          page_off, page_ids, page_size, cache, q_out)
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2
    rope = RopeStore(n_q_heads, n_kv_heads, head_dim, rotary_dim, inv_freq.data_ptr(),
                     _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos"),
                     _i32(page_off, "page_off") if has_kv else None,
                     _i32(page_ids, "page_ids") if has_kv else None, page_size,
                     cache.data_ptr() if has_kv else None, _ptr(q_out))
    extras = LinearExtras()
    extras.rope = ctypes.pointer(rope)
    ws = _tc5_workspace(M, N, K, h.device)
    _check(l.sb_gemm_tc5_ex(_ptr(h), BF16, _ptr(w), BF16, M, N, K, EPI_BIAS if bias is not None else EPI_NONE,
                            _ptr(bias), _code(bias.dtype) if bias is not None else 0, _ptr(None), _ptr(None), F32,
                            _ptr(ws), ctypes.c_size_t(ws.numel()), _sm_count(h.device), 0,
                            ctypes.byref(extras), _stream()),
           "q|k|v product with rotation (tcgen05 kernel)", launches=2)
    return q_out


def _warm_args(warm):
    """(pointer, bytes) of an L2 hint as the kernels take it."""
    if warm is None or not WARM:
        return _ptr(None), ctypes.c_size_t(0)
    return _ptr(warm), ctypes.c_size_t(warm.numel() * warm.element_size())


WARM = _os.environ.get("SB_WARM", "1") != "0"       # L2 hints on (SB_WARM=0: off, for measurements)
# "skinny" or "tc5": overrides the choice below (for measurements; SB_DECODE_KERNEL in the environment)
FORCE_DECODE_KERNEL = _os.environ.get("SB_DECODE_KERNEL") or None


def _pick_kernel(M: int, N: int, K: int, device) -> str:
    """Which bfloat16 product kernel "auto" means.  The tcgen05 kernel, except for small
    matrices at up to 8 rows: there the kernel that streams W into mma.sync fragments has lower
    fixed costs (measured on B200 at the 7B layer sizes, alone inside CUDA graphs: 9 us against
    12 us for the 4608 x 3584 product at 8 rows, while at 64 rows the tcgen05 kernel takes 12 us
    and the streaming kernel 19 us; inside the decode step, where the tcgen05 kernel requests its
    weights while the kernel before it ends, the streaming kernel wins by 0.5 % of the step at
    8 rows and loses by 1.3 % at 16)."""
    if M > 8:
        return "tc5"
    if FORCE_DECODE_KERNEL:
        return FORCE_DECODE_KERNEL
    tiles = (N + 127) // 128
    if tiles >= _sm_count(device) or K >= 8192:
        return "tc5"
    return "skinny"


def requests_weights_late(M: int, N: int, K: int, device) -> bool:
    """Whether the bfloat16 product kernel that "auto" picks for these sizes starts only when
    the kernel before it has ended (it is launched without programmatic dependent launch), so
    that its weights are worth an L2 hint from an earlier kernel."""
    kernel = _pick_kernel(M, N, K, device)
    cls = PDL_TC5 if kernel == "tc5" else PDL_SKINNY
    return not (int(lib().sb_pdl_enabled()) & cls)


_sm_counts: dict = {}
_tc5_buffers: dict = {}          # device -> list of workspaces (never freed:
                                 # captured graphs may hold their addresses)


def _sm_count(device) -> int:
    n = _sm_counts.get(device)
    if n is None:
        key = torch.device(device).index or 0
        n = _sm_counts[device] = torch.cuda.get_device_properties(key).multi_processor_count
    return n


def _tc5_workspace(M: int, N: int, K: int, device):
    """Workspace of a tcgen05 product that splits K (the decode form, and the many-rows form when
    it has few row tiles): the partial sums.  One buffer per device serves every call on the
    stream; it only grows."""
    l = lib()
    need = int(l.sb_gemm_tc5_scratch_bytes(M, N, K, _sm_count(device)))
    if need == 0:
        return None
    key = torch.device(device).index or 0
    bufs = _tc5_buffers.setdefault(key, [])
    if not bufs or bufs[-1].numel() < need:
        bufs.append(torch.empty(max(need, 16 << 20), dtype=torch.uint8, device=device))
    return bufs[-1]


PDL_TC5, PDL_SKINNY, PDL_ATTENTION, PDL_ELEMENTWISE, PDL_REDUCE, PDL_OTHER, PDL_ALL = 1, 2, 4, 8, 16, 32, 63


def set_pdl(level) -> None:
    """Which kernels are launched with programmatic dependent launch: a mask of the PDL_* bits
    (0 none, PDL_ALL every kernel; the default is every class but PDL_SKINNY).  The
    environment variable SB_PDL sets it at start."""
    level = int(level)
    lib().sb_set_pdl(level)
    for l in _attn_libs.values():
        if l is not None:
            l.sb_set_pdl(level)


def tc5_status() -> int:
    """0 unless a tcgen05 kernel gave up on a bounded wait since the last call (synchronizes)."""
    return int(lib().sb_tc5_status())


def tc5_tile_width(M: int, N: int) -> int:
    """The tile width the tcgen05 product of M rows and N features runs with in its many-rows
    form (0: that form does not run): for tests that want every width covered."""
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return int(lib().sb_gemm_tc5_tile_width(int(M), int(N), sms))


def force_tc5_tile_width(width: int) -> None:
    """256, 240, 224, 208 or 192: every many-rows tcgen05 product uses that tile width (for
    measurements and tests); 0: chosen by the sizes again."""
    lib().sb_gemm_tc5_force_width(int(width))


def set_tc5_pairs(mode: int) -> None:
    """Whether the tcgen05 product of more than 128 rows runs on pairs of SMs (a cluster of two
    blocks on one 256-row tile): 1 yes, 0 no (one block per 128-row tile), -1 by SB_TC5_PAIR
    (default yes).  The result is the same to the bit either way."""
    lib().sb_gemm_tc5_pairs(int(mode))


def rope_store(qkv: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
               inv_freq: torch.Tensor, row_seq, row_pos, page_off, page_ids, page_size: int,
               cache: torch.Tensor | None, q_out: torch.Tensor) -> torch.Tensor:
    """Rotates q and k, writes q to q_out [rows, heads, hd] and k, v into the cache pages.
    With cache=None the input row holds queries only (a layer that reads another's cache)."""
    n = qkv.shape[0]
    has_kv = cache is not None
    assert qkv.dtype == torch.float32
    assert qkv.shape[1] == (n_q_heads + (2 * n_kv_heads if has_kv else 0)) * head_dim
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2
    _check(lib().sb_rope_store(
        _ptr(qkv), n, n_q_heads, n_kv_heads, head_dim, rotary_dim, _ptr(inv_freq),
        _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos"),
        _i32(page_off, "page_off") if has_kv else _ptr(None),
        _i32(page_ids, "page_ids") if has_kv else _ptr(None), page_size,
        _ptr(cache), _code(cache.dtype) if has_kv else _code(q_out.dtype), _ptr(q_out),
        _code(q_out.dtype), 1 if has_kv else 0, _stream()), "rope_store")
    return q_out


_attn_libs: dict = {}
_attn_counter_bufs: dict = {}    # device -> zeroed int32 buffers (kernels leave them zero; never freed)


def _attn_counters(n: int, device) -> torch.Tensor:
    """Arrival counters of the split attention's merge: zero between launches."""
    key = torch.device(device).index or 0
    bufs = _attn_counter_bufs.setdefault(key, [])
    if not bufs or bufs[-1].numel() < n:
        bufs.append(torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device))
    return bufs[-1]



def attention_lib(head_dim: int):
    """The tensor-core attention library of one head size, or None when the head size is
    outside what those kernels are written for (multiples of 16 up to 256)."""
    if head_dim not in _attn_libs:
        if head_dim in _build.HEAD_DIMS:
            al = _abi.apply(_build.load_attention(head_dim), _abi.ATTENTION)
            # SB_ATTN=mma|tma in the environment: one kernel family for every step (for measurements)
            al.sb_attention_force_mma({"mma": 1, "tma": 2}.get(_os.environ.get("SB_ATTN", ""), 0))
            _attn_libs[head_dim] = al
        else:
            _attn_libs[head_dim] = None
    return _attn_libs[head_dim]


def attention(q: torch.Tensor, out: torch.Tensor, plan, group_index: int, cache: torch.Tensor,
              n_q_heads: int, n_kv_heads: int, head_dim: int, window: int, scale: float,
              kernel: str = "auto", warm: torch.Tensor | None = None,
              sink: torch.Tensor | None = None, softcap: float = 0.0) -> torch.Tensor:
    """Causal grouped-query attention of the step's rows over one cache entry's pages.
    `sink` (float32, one per query head): exp(sink) joins that head's softmax denominator.
    `softcap` c > 0: a score s becomes c tanh(s / c) before the softmax.

    bfloat16 runs the tensor-core kernels (built for the head size at first use); float32, a
    head size those kernels do not take, or `kernel="plain"` run the plain kernel.  `"mma"` keeps
    to the mma.sync kernels where the tensor-memory prefill kernel or the persistent TMA decode
    kernel would run (head sizes 64, 128); `"tma"` runs that decode kernel whatever the number of
    key splits (by itself it runs from about a wave of splits on).
    `warm`: a tensor the kernel after this one will stream (weights); the decode kernel asks for
    it into L2 while it merges its partial results.  A hint: it changes no result."""
    n = q.shape[0]
    g = plan.groups[group_index]
    if sink is not None:
        assert sink.dtype == torch.float32 and sink.numel() == n_q_heads
    al = attention_lib(head_dim) if (q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
                                     and kernel != "plain") else None
    if al is not None:
        need = int(al.sb_attention_scratch_bytes(n, n_q_heads, n_kv_heads, plan.max_new, plan.max_len))
        scratch = plan.scratch(need, q.device)
        counters = _attn_counters(plan.n_seqs * n_kv_heads, q.device)
        if kernel in ("mma", "tma"):
            al.sb_attention_force_mma(1 if kernel == "mma" else 2)
        rc = al.sb_attention(
            _ptr(q), _ptr(out), n, plan.n_seqs, plan.max_new, _i32(plan.seq_row0, "seq_row0"),
            _i32(plan.seq_pos0, "seq_pos0"), _i32(g.page_off, "page_off"),
            _i32(g.page_ids, "page_ids"), g.page_size, _ptr(cache), n_q_heads, n_kv_heads,
            head_dim, window, ctypes.c_float(scale), _ptr(scratch),
            ctypes.c_size_t(scratch.numel() if scratch is not None else 0),
            _ptr(counters), counters.numel(), plan.max_len, cache.shape[0], _sm_count(q.device),
            *_warm_args(warm), _ptr(sink), ctypes.c_float(softcap), _stream())
        if kernel in ("mma", "tma"):
            al.sb_attention_force_mma({"mma": 1, "tma": 2}.get(_os.environ.get("SB_ATTN", ""), 0))
        if rc != 0:
            raise KernelError(f"attention: {al.sb_last_error().decode()}")
        global LAUNCHES
        LAUNCHES += int(al.sb_attention_last_launches())
    else:
        _check(lib().sb_attention_plain(
            _ptr(q), _ptr(out), _code(q.dtype), n, _i32(plan.row_seq, "row_seq"),
            _i32(plan.row_pos, "row_pos"), _i32(g.page_off, "page_off"),
            _i32(g.page_ids, "page_ids"), g.page_size, _ptr(cache), _code(cache.dtype),
            n_q_heads, n_kv_heads, head_dim, window, ctypes.c_float(scale), _ptr(sink),
            ctypes.c_float(softcap), _stream()), "attention (plain kernel)")
    return out


def attention_status(head_dim: int) -> int:
    """0 when no tensor-memory attention kernel of this head size has given up on a wait since the
    last call (else the code of that wait); -1 when the head size has no such kernel."""
    al = attention_lib(head_dim)
    return int(al.sb_attention_status()) if al is not None else -1


def sample_params_size() -> int:
    return lib().sb_sample_params_size()


def sample(logits: torch.Tensor, params: torch.Tensor, history: torch.Tensor | None,
           out_tokens: torch.Tensor, fed_pos: torch.Tensor | None = None) -> torch.Tensor:
    """One token per logits row; `params` is a uint8 tensor of packed per-row records.  With
    `fed_pos` (int32 per row) the draw's position is fed_pos + 1 instead of the record's.
    A row whose logits are not finite may get -1: `check_tokens` turns that into an error."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and params.dtype == torch.uint8
    assert params.numel() == n * sample_params_size()
    stride = history.shape[1] if history is not None else 0
    _check(lib().sb_sample(_ptr(logits), n, vocab, _ptr(params),
                           _i32(history, "history") if history is not None else _ptr(None),
                           stride, _i32(fed_pos, "fed_pos") if fed_pos is not None else _ptr(None),
                           _i32(out_tokens, "out_tokens"), _stream()), "sample")
    return out_tokens


def check_tokens(ids: list, live: list | None = None) -> list:
    """Sampled ids as read on the host: raises where the sampler chose no token (rows whose
    `live` entry is false are not looked at)."""
    bad = [i for i, t in enumerate(ids) if t < 0 and (live is None or live[i])]
    if bad:
        raise KernelError(f"the sampler chose no token for row {bad[0]}: its logits are not finite")
    return ids


def check_status() -> None:
    """Raises KernelError if a kernel of any loaded library gave up on one of its bounded waits
    since the last look (its output is then incomplete).  Reading synchronizes with the device,
    so this is called where the host waits anyway."""
    if _lib is None:
        return
    code = tc5_status()
    if code:
        raise KernelError(f"a tcgen05 product kernel gave up on a bounded wait (code {code}): "
                          "results since the last check are incomplete")
    for hd, l in _attn_libs.items():
        if l is not None:
            code = int(l.sb_attention_status())
            if code > 0:
                raise KernelError(f"the tensor-memory attention kernel of head size {hd} gave up "
                                  f"on a bounded wait (code {code}): results since the last check "
                                  "are incomplete")


def add_i32(x: torch.Tensor, delta: int) -> torch.Tensor:
    """x += delta on the device (int32)."""
    _check(lib().sb_add_i32(_i32(x, "x"), x.numel(), int(delta), _stream()), "add_i32")
    return x


def advance_rows(pos: torch.Tensor, last: torch.Tensor) -> torch.Tensor:
    """pos[i] = min(pos[i] + 1, last[i]) on the device (int32): the positions of a captured
    decode batch move on, each row at most to the last position it holds pages for."""
    assert pos.numel() == last.numel()
    _check(lib().sb_advance_rows(_i32(pos, "pos"), _i32(last, "last"), pos.numel(), _stream()),
           "advance_rows")
    return pos


def random_normal(out: torch.Tensor, key0: int, key1: int, mean: float, std: float) -> torch.Tensor:
    """Fills `out` (float32 or bfloat16, contiguous) with mean + std * z, z standard normal drawn
    from the counter-based generator keyed by (key0, key1) and the element index."""
    _check(lib().sb_random_normal(_ptr(out), _code(out.dtype), ctypes.c_size_t(out.numel()),
                                  ctypes.c_uint32(key0 & 0xffffffff), ctypes.c_uint32(key1 & 0xffffffff),
                                  ctypes.c_float(mean), ctypes.c_float(std), _stream()),
           "random_normal")
    return out


# ---------------------------------------------------------------------- residual-stream rows
def _next_norm_args(next_norm, width, rows):
    """(weight, dtype, eps, out, dtype) of the optional norm of a finished row."""
    if next_norm is None:
        return _ptr(None), 0, ctypes.c_float(0.0), _ptr(None), 0
    w, eps, normed = next_norm
    assert tuple(normed.shape) == (rows, width)
    if w is None:                      # no norm: the finished rows as they are, in `normed`'s dtype
        return _ptr(None), 0, ctypes.c_float(0.0), _ptr(normed), _code(normed.dtype)
    assert w.numel() == width
    return _ptr(w), _code(w.dtype), ctypes.c_float(eps), _ptr(normed), _code(normed.dtype)


def _join_args(join, coef, rows, width):
    if join is None:
        return _ptr(None), _ptr(None), _ptr(None), 0, ctypes.c_float(0.0)
    y, x, w, eps = join
    assert y.dtype == x.dtype == torch.float32 and tuple(y.shape) == tuple(x.shape) == (rows, width)
    assert w.numel() == width
    if w.dtype != coef.dtype:
        raise KernelError("depth_mix: the joined norm's weight and the coefficients differ in dtype")
    return _ptr(y), _ptr(x), _ptr(w), _code(w.dtype), ctypes.c_float(eps)


def norm_add(y: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             next_norm: tuple | None = None) -> torch.Tensor:
    """out = x + y / sqrt(mean(y^2) + eps) * weight, row by row in float32 (out may be x).
    `next_norm` = (weight, eps, normed) also writes the RMS norm of the finished rows; with a
    weight of None, `normed` receives the finished rows themselves in its own dtype."""
    rows, width = y.shape
    assert y.dtype == x.dtype == out.dtype == torch.float32 and x.shape == y.shape == out.shape
    assert weight.numel() == width
    _check(lib().sb_norm_add(_ptr(y), _ptr(x), rows, width, _ptr(weight), _code(weight.dtype),
                             ctypes.c_float(eps), _ptr(out), *_next_norm_args(next_norm, width, rows),
                             _stream()), "norm_add")
    return out


def depth_mix(planes: torch.Tensor, n_inputs: int, coef: torch.Tensor, out: torch.Tensor,
              next_norm: tuple | None = None, join: tuple | None = None) -> torch.Tensor:
    """out = sum_j coef[j] * planes[j] over the first n_inputs planes of float32 [n, rows, width].
    `join` = (y, x, weight, eps) makes the last of those planes first, as `norm_add` would:
    planes[n_inputs - 1] = x + y / sqrt(mean(y^2) + eps) * weight (x may be that plane)."""
    rows, width = out.shape
    assert planes.dtype == out.dtype == torch.float32 and planes.dim() == 3
    assert tuple(planes.shape[1:]) == (rows, width) and 1 <= n_inputs <= planes.shape[0]
    assert coef.numel() == n_inputs
    _check(lib().sb_depth_mix(_ptr(planes), ctypes.c_size_t(rows * width), n_inputs, _ptr(coef),
                              _code(coef.dtype), rows, width, _ptr(out),
                              *_next_norm_args(next_norm, width, rows), *_join_args(join, coef, rows, width),
                              _stream()), "depth_mix")
    return out


def glu_clamped(gate_up: torch.Tensor, limit: float, slope: float, out: torch.Tensor,
                interleaved: bool = False) -> torch.Tensor:
    """out = a * sigmoid(slope a) * (b + 1) with a = min(gate, limit), b = clamp(up, -limit, limit);
    gate_up is float32 [rows, 2 ff] = [gate | up], or with `interleaved` blocks of SWIGLU_BLOCK
    gates followed by the up values of the same outputs."""
    rows, ff = out.shape
    assert gate_up.dtype == torch.float32 and tuple(gate_up.shape) == (rows, 2 * ff)
    _check(lib().sb_glu_clamped(_ptr(gate_up), rows, ff, ctypes.c_float(limit), ctypes.c_float(slope),
                                1 if interleaved else 0, _ptr(out), _code(out.dtype), _stream()), "glu_clamped")
    return out


GATE_SILU, GATE_CLAMPED, GATE_GELU_TANH = 0, 1, 2
GATE_KINDS = {"silu": GATE_SILU, "glu_clamped": GATE_CLAMPED, "gelu_tanh": GATE_GELU_TANH}


def gated_act(gate_up: torch.Tensor, kind: int, out: torch.Tensor, interleaved: bool = False,
              limit: float = 0.0, slope: float = 1.0) -> torch.Tensor:
    """out = act(gate) * up over float32 rows [gate | up] (or, `interleaved`, blocks of SWIGLU_BLOCK
    gates followed by the up values of the same outputs); `kind` is GATE_SILU, GATE_CLAMPED (the form
    of `glu_clamped`, with `limit` and `slope`) or GATE_GELU_TANH (gelu in its tanh form)."""
    rows, ff = out.shape
    assert gate_up.dtype == torch.float32 and tuple(gate_up.shape) == (rows, 2 * ff)
    _check(lib().sb_gated_act(_ptr(gate_up), rows, ff, int(kind), ctypes.c_float(limit), ctypes.c_float(slope),
                              1 if interleaved else 0, _ptr(out), _code(out.dtype), _stream()), "gated_act")
    return out


# ---------------------------------------------------------------------- attention over a latent
def latent_prep(proj: torch.Tensor, n_heads: int, dim: int, rot_dim: int, rank: int, rotary_dim: int,
                inv_freq: torch.Tensor, row_seq, row_pos, page_off, page_ids, page_size: int,
                cnorm: torch.Tensor | None, eps: float, cache: torch.Tensor | None,
                q_wide: torch.Tensor, q_group: int = 0, kv: tuple | None = None,
                interleaved: bool = True, rot_scale: float = 1.0) -> torch.Tensor:
    """Finishes the fused projection rows [heads x (dim | rot_dim) | rank | rot_dim] (the last two
    only when `cache` is given): rotation in interleaved pairs, the latent's RMS norm, the cache
    write (key plane [latent | key part], value plane [latent | 0]), and every head's rotated
    part into q_wide[:, :, rank:].  With `q_group` (a divisor of the heads) q_wide lies
    [head group, row, head in group, rank + rot_dim].  `kv` = (float32 rows, offset): the latent and
    the key part [rank | rot_dim] start at `offset` of rows of their own (`proj` then holds the heads only).  Not `interleaved`: the pairs are (i, i + rotary_dim/2).
    `rot_scale` multiplies every cosine and sine."""
    n = proj.shape[0]
    q_group = q_group or n_heads
    has_kv = cache is not None
    assert proj.dtype == torch.float32
    assert proj.shape[1] == n_heads * (dim + rot_dim) + ((rank + rot_dim) if has_kv and kv is None else 0)
    kv_ptr, kv_ld = None, 0
    if kv is not None:
        rows_kv, off = kv
        assert has_kv and rows_kv.dtype == torch.float32 and rows_kv.is_contiguous() and rows_kv.shape[0] == n
        assert off + rank + rot_dim <= rows_kv.shape[1]
        kv_ptr, kv_ld = rows_kv.data_ptr() + 4 * off, rows_kv.shape[1]
    assert n_heads % q_group == 0 and q_wide.numel() == n * n_heads * (rank + rot_dim)
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= max(1, rotary_dim // 2)
    _check(lib().sb_latent_prep(
        _ptr(proj), n, n_heads, dim, rot_dim, rank, rotary_dim, _ptr(inv_freq),
        _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos"),
        _i32(page_off, "page_off") if has_kv else _ptr(None),
        _i32(page_ids, "page_ids") if has_kv else _ptr(None), page_size,
        _ptr(cnorm) if has_kv else _ptr(None), _code(cnorm.dtype) if has_kv else 0, ctypes.c_float(eps),
        _ptr(cache), _code(cache.dtype) if has_kv else 0, _ptr(q_wide), _code(q_wide.dtype),
        q_group, 1 if has_kv else 0, kv_ptr, kv_ld, 1 if interleaved else 0,
        ctypes.c_float(rot_scale), _stream()), "latent_prep")
    return q_wide


def head_linear(x: torch.Tensor, x_offset: int, x_row: int, x_head: int, w: torch.Tensor, out: torch.Tensor,
                out_offset: int, out_row: int, out_head: int, n_rows: int) -> torch.Tensor:
    """out[r, h, :N] = w[h] @ x[r, h, :K] for w [heads, N, K]; x and out are addressed by element
    offsets: row r, head h starts at offset + r * row + h * head."""
    heads, N, K = w.shape
    assert x.is_contiguous() and out.is_contiguous() and w.is_contiguous()
    assert x_offset + (n_rows - 1) * x_row + (heads - 1) * x_head + K <= x.numel()
    assert out_offset + (n_rows - 1) * out_row + (heads - 1) * out_head + N <= out.numel()
    _check(lib().sb_head_linear(x.data_ptr() + x_offset * x.element_size(), _code(x.dtype),
                                ctypes.c_size_t(x_row), ctypes.c_size_t(x_head), _ptr(w), _code(w.dtype),
                                n_rows, heads, N, K, out.data_ptr() + out_offset * out.element_size(),
                                _code(out.dtype), ctypes.c_size_t(out_row), ctypes.c_size_t(out_head),
                                _stream()), "head_linear")
    return out


# ---------------------------------------------------------------------- matrix-memory recurrence
def mlstm_scan(proj: torch.Tensor, plan, n_heads: int, dim: int, vdim: int, i_bias: torch.Tensor,
               f_bias: torch.Tensor, cap: float, q_scale: float, state: torch.Tensor,
               num: torch.Tensor, m_row: torch.Tensor) -> torch.Tensor:
    """Walks every sequence's rows of the step through the recurrence, from and to the state
    rows of the sequences' slots (float32 [slots, heads, vdim + 1, dim + 1 or more])."""
    rows = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.shape[1] == 2 * n_heads * (dim + vdim + 1)
    assert state.dtype == torch.float32 and tuple(state.shape[1:3]) == (n_heads, vdim + 1) and state.shape[3] > dim
    assert num.dtype == torch.float32 and tuple(num.shape) == (rows, n_heads, vdim + 1)
    assert m_row.dtype == torch.float32 and tuple(m_row.shape) == (rows, n_heads)
    assert i_bias.dtype == f_bias.dtype and i_bias.numel() == f_bias.numel() == n_heads
    _check(lib().sb_mlstm_scan(_ptr(proj), plan.n_seqs, _i32(plan.seq_row0, "seq_row0"),
                               _i32(plan.seq_slot, "seq_slot"), n_heads, dim, vdim, _ptr(i_bias),
                               _ptr(f_bias), _code(i_bias.dtype), ctypes.c_float(cap),
                               ctypes.c_float(q_scale), int(plan.max_new), _ptr(state), int(state.shape[3]), _ptr(num), _ptr(m_row),
                               _stream()),
           "mlstm_scan")
    return num


def mlstm_out(num: torch.Tensor, m_row: torch.Tensor, proj: torch.Tensor, n_heads: int, dim: int,
              vdim: int, norm_w: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """The recurrence's outputs: division by the normalizer, RMS norm per head, the norm's weight
    and the gate sigmoid(g) of the projection row; out [rows, heads * vdim]."""
    rows = proj.shape[0]
    assert tuple(out.shape) == (rows, n_heads * vdim) and norm_w.numel() == n_heads * vdim
    _check(lib().sb_mlstm_out(_ptr(num), _ptr(m_row), _ptr(proj), rows, n_heads, dim, vdim, _ptr(norm_w),
                              _code(norm_w.dtype), ctypes.c_float(eps), _ptr(out), _code(out.dtype),
                              _stream()), "mlstm_out")
    return out


# ---------------------------------------------------------------------- a vector joins the stream
def stream_add(x: torch.Tensor, add: torch.Tensor | None, vec: torch.Tensor | None, out: torch.Tensor,
               next_norm: tuple | None = None) -> torch.Tensor:
    """out = x + add + vec row by row in float32 (`add` [rows, width] and `vec` [width] are optional;
    out may be x).  `next_norm` = (weight, eps, normed) also writes the RMS norm of the finished rows."""
    rows, width = x.shape
    assert x.dtype == out.dtype == torch.float32 and out.shape == x.shape
    assert add is None or (add.dtype == torch.float32 and add.shape == x.shape)
    assert vec is None or vec.numel() == width
    _check(lib().sb_stream_add(_ptr(x), _ptr(add), _ptr(vec), _code(vec.dtype) if vec is not None else 0, rows,
                               width, _ptr(out), *_next_norm_args(next_norm, width, rows), _stream()),
           "stream_add")
    return out


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 row by row, N(u) = u / sqrt(mean(u^2) + eps);
    z float32 [rows, ff], coef four numbers."""
    rows, ff = z.shape
    assert z.dtype == torch.float32 and tuple(out.shape) == (rows, ff) and coef.numel() == 4
    _check(lib().sb_polynorm(_ptr(z), rows, ff, _ptr(coef), _code(coef.dtype), ctypes.c_float(eps), _ptr(out),
                             _code(out.dtype), _stream()), "polynorm")
    return out


# ---------------------------------------------------------------------- attention: rows in and out
def attn_prep(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, n_q_heads: int, n_kv_heads: int,
              dim: int, vdim: int, head_size: int, rotary_dim: int, interleaved: bool,
              inv_freq: torch.Tensor | None, v_inv_freq: torch.Tensor | None, q_norm: torch.Tensor | None,
              k_norm: torch.Tensor | None, eps: float, row_seq, row_pos, page_off, page_ids, page_size: int,
              cache: torch.Tensor | None, q_out: torch.Tensor, head_norm: str | None = None,
              rot_scale: float = 1.0) -> torch.Tensor:
    """Projection rows to queries and cache rows (see sb_attn_prep in the kernel library's header):
    optional RMS norm over the whole q and k projection, rotation in either layout of pairs,
    values that are the raw keys (`v_off` < 0), values rotated over their whole size (`v_inv_freq`),
    heads padded with zeros to `head_size`.  `cache=None`: queries only.
    `head_norm` "before": every q and k head is RMS-normed by itself before the rotation, `q_norm` and
    `k_norm` being one weight [dim] for all heads; "after": every head is divided by its root mean
    square after the rotation (no weights).  `rot_scale` multiplies every cosine and sine."""
    n, ld = proj.shape
    assert head_norm in (None, "before", "after")
    has_kv = cache is not None
    assert proj.dtype == torch.float32 and tuple(q_out.shape) == (n, n_q_heads, head_size)
    assert q_off + n_q_heads * dim <= ld and (not has_kv or k_off + n_kv_heads * dim <= ld)
    assert not has_kv or v_off < 0 or v_off + n_kv_heads * vdim <= ld
    assert rotary_dim == 0 or (inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2)
    assert v_inv_freq is None or (v_inv_freq.dtype == torch.float32 and v_inv_freq.numel() >= vdim // 2)
    if q_norm is not None and head_norm == "before":
        assert q_norm.dtype == k_norm.dtype and q_norm.numel() == k_norm.numel() == dim
    elif q_norm is not None:
        assert q_norm.dtype == k_norm.dtype and q_norm.numel() == n_q_heads * dim and k_norm.numel() == n_kv_heads * dim
    _check(lib().sb_attn_prep(
        _ptr(proj), n, ld, q_off, k_off, v_off, n_q_heads, n_kv_heads, dim, vdim, head_size, rotary_dim,
        1 if interleaved else 0, _ptr(inv_freq), _ptr(v_inv_freq), _ptr(q_norm), _ptr(k_norm),
        _code(q_norm.dtype) if q_norm is not None else 0, {None: 0, "before": 1, "after": 2}[head_norm],
        ctypes.c_float(rot_scale), ctypes.c_float(eps),
        _i32(row_seq, "row_seq"), _i32(row_pos, "row_pos"),
        _i32(page_off, "page_off") if has_kv else _ptr(None),
        _i32(page_ids, "page_ids") if has_kv else _ptr(None), page_size, _ptr(cache),
        _code(cache.dtype) if has_kv else 0, _ptr(q_out), _code(q_out.dtype), 1 if has_kv else 0, _stream()),
        "attn_prep")
    return q_out


def attn_unrotate(x: torch.Tensor, out: torch.Tensor, n_heads: int, head_size: int, vdim: int,
                  interleaved: bool, v_inv_freq: torch.Tensor | None, row_pos,
                  gate: tuple | None = None) -> torch.Tensor:
    """out [rows, heads * vdim] = the first vdim values of every head of x [rows, heads * head_size],
    turned back by the row's position when a table is given.  `gate` = (rows float32 [rows, ld],
    offset): head h of a row is multiplied by sigmoid(rows[r, offset + h])."""
    n = out.shape[0]
    g_ptr, g_ld = None, 0
    if gate is not None:
        g, off = gate
        assert g.dtype == torch.float32 and g.is_contiguous() and g.shape[0] == n and off + n_heads <= g.shape[1]
        g_ptr, g_ld = g.data_ptr() + 4 * off, g.shape[1]
    assert x.dtype == out.dtype and x.numel() == n * n_heads * head_size and out.shape[1] == n_heads * vdim
    _check(lib().sb_attn_unrotate(_ptr(x), _ptr(out), _code(x.dtype), n, n_heads, head_size, vdim,
                                  1 if interleaved else 0, _ptr(v_inv_freq), _i32(row_pos, "row_pos"), g_ptr, g_ld,
                                  _stream()), "attn_unrotate")
    return out


# ---------------------------------------------------------------------- linear recurrence
def linrec_prep(proj: torch.Tensor, q_off: int, k_off: int, n_heads: int, dim: int, q_scale: float,
                k_scale: float, rotary_dim: int, interleaved: bool, inv_freq: torch.Tensor | None, row_pos,
                z: torch.Tensor | None = None, inv_tau: float = 1.0, low_rank: tuple | None = None) -> torch.Tensor:
    """In place: rotates and scales the q and k of the projection rows; turns decay logits `z`
    [rows, heads * dim] into decays exp(logsigmoid(z) * inv_tau).  `low_rank` = (a2 [heads * dim, rank],
    bias, a1_off): the logits are made here first, a2 times the rank values at `a1_off` of every
    projection row plus the bias, and `z` only receives the decays."""
    n, ld = proj.shape
    a2 = bias = None
    rank = a1_off = 0
    if low_rank is not None:
        a2, bias, a1_off = low_rank
        rank = a2.shape[1]
        assert z is not None and a2.dtype == bias.dtype and a2.shape[0] == bias.numel() == n_heads * dim
        assert 0 <= a1_off and a1_off + rank <= ld
    assert proj.dtype == torch.float32 and max(q_off, k_off) + n_heads * dim <= ld
    assert z is None or (z.dtype == torch.float32 and tuple(z.shape) == (n, n_heads * dim))
    _check(lib().sb_linrec_prep(_ptr(proj), n, ld, q_off, k_off, n_heads, dim, ctypes.c_float(q_scale),
                                ctypes.c_float(k_scale), rotary_dim, 1 if interleaved else 0, _ptr(inv_freq),
                                _i32(row_pos, "row_pos"), _ptr(z), ctypes.c_float(inv_tau), _ptr(a2), _ptr(bias),
                                _code(a2.dtype) if a2 is not None else 0, rank, a1_off, _stream()),
           "linrec_prep")
    return proj


def linrec_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, plan, n_heads: int, dim: int,
                vdim: int, decay: torch.Tensor | None, head_decay: torch.Tensor | None,
                state: torch.Tensor, out: torch.Tensor, token_decay: torch.Tensor | None = None,
                heads_per_qk: int = 1) -> torch.Tensor:
    """Walks every sequence's rows of the step through S = diag(a) S + k v^T, o = S^T q, from and
    to the state rows of the sequences' slots (float32 [slots, heads, vdim, dim]).  The decay is
    `decay` [rows, heads * dim], `head_decay` [heads] or `token_decay` [rows, heads]; `heads_per_qk`
    neighbouring heads read the same q and k."""
    n, ld = proj.shape
    assert proj.dtype == torch.float32 and state.dtype == torch.float32 and out.dtype == torch.float32
    assert tuple(state.shape[1:]) == (n_heads, vdim, dim) and tuple(out.shape) == (n, n_heads, vdim)
    assert decay is None or (decay.dtype == torch.float32 and tuple(decay.shape) == (n, n_heads * dim))
    assert head_decay is None or (head_decay.dtype == torch.float32 and head_decay.numel() == n_heads)
    assert token_decay is None or (token_decay.dtype == torch.float32 and tuple(token_decay.shape) == (n, n_heads))
    _check(lib().sb_linrec_scan(_ptr(proj), ld, q_off, k_off, v_off, _ptr(decay), _ptr(head_decay),
                                _ptr(token_decay), heads_per_qk, plan.n_seqs,
                                _i32(plan.seq_row0, "seq_row0"), _i32(plan.seq_slot, "seq_slot"), n_heads, dim,
                                vdim, _ptr(state), _ptr(out), _stream()), "linrec_scan")
    return out


def force_linrec_columns(cpt: int) -> None:
    """1 or 2: every `linrec_scan` keeps that many columns of the state per thread (for measurements
    and tests; the results are the same bits); 0: chosen by the sizes again."""
    lib().sb_linrec_force_columns(int(cpt))


def linrec_out(o: torch.Tensor, proj: torch.Tensor, g_off: int, n_heads: int, vdim: int,
               norm_w: torch.Tensor | None, eps: float, out: torch.Tensor, gate: str = "silu") -> torch.Tensor:
    """out [rows, heads * vdim] = rms(o) per head * weight (optional: [vdim] for all heads, or
    [heads * vdim]) * gate(g of the row); the gate is "silu" or "sigmoid"."""
    n, ld = proj.shape
    assert tuple(o.shape) == (n, n_heads, vdim) and tuple(out.shape) == (n, n_heads * vdim)
    assert g_off + n_heads * vdim <= ld and (norm_w is None or norm_w.numel() in (vdim, n_heads * vdim))
    assert gate in ("silu", "sigmoid")
    per_head = norm_w is not None and n_heads > 1 and norm_w.numel() == n_heads * vdim
    _check(lib().sb_linrec_out(_ptr(o), _ptr(proj), n, ld, g_off, n_heads, vdim, _ptr(norm_w),
                               _code(norm_w.dtype) if norm_w is not None else 0, 1 if per_head else 0,
                               1 if gate == "sigmoid" else 0, ctypes.c_float(eps), _ptr(out),
                               _code(out.dtype), _stream()), "linrec_out")
    return out


# ---------------------------------------------------------------------- rows and their neighbours
def embed_pair(plan, prev_token: torch.Tensor, table: torch.Tensor, pair: torch.Tensor, buckets: int,
               mul_prev: int, mul_cur: int, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[r] = table[token] * scale + pair[(previous token * mul_prev + token * mul_cur) mod buckets],
    row `buckets` of `pair` for a sequence's first token.  The token before a step's first row of a
    sequence is `prev_token[slot]` (int32, one per slot); `keep_last_token` stores it."""
    n, width = plan.n_rows, table.shape[1]
    assert out.dtype == torch.float32 and tuple(out.shape) == (n, width) and table.dtype == pair.dtype
    assert tuple(pair.shape) == (buckets + 1, width) and prev_token.dtype == torch.int32
    _check(lib().sb_embed_pair(_i32(plan.tokens, "tokens"), n, _i32(plan.row_seq, "row_seq"),
                               _i32(plan.row_pos, "row_pos"), _i32(plan.seq_row0, "seq_row0"),
                               _i32(plan.seq_slot, "seq_slot"), _ptr(prev_token), _ptr(table), _code(table.dtype),
                               table.shape[0], _ptr(pair), buckets, mul_prev, mul_cur, width,
                               ctypes.c_float(scale), _ptr(out), _stream()), "embed_pair")
    return out


def keep_last_token(plan, prev_token: torch.Tensor) -> None:
    """prev_token[slot] = the last token the step brings for the sequence in that slot."""
    _check(lib().sb_keep_last_token(_i32(plan.tokens, "tokens"), _i32(plan.seq_row0, "seq_row0"),
                                    _i32(plan.seq_slot, "seq_slot"), plan.n_seqs, _i32(prev_token, "prev_token"),
                                    _stream()), "keep_last_token")


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
              rows: torch.Tensor | None = None) -> torch.Tensor:
    """out[r] = (x - mean) / sqrt(var + eps) * weight over the row x[rows[r]] or x[r] (no bias)."""
    assert x.dtype == torch.float32 and x.dim() == 2
    n, width = out.shape[0], x.shape[1]
    assert out.shape[1] == width and weight.numel() == width and (rows is not None or x.shape[0] == n)
    _check(lib().sb_layernorm(_ptr(x), _i32(rows, "rows") if rows is not None else _ptr(None), n, width,
                              _ptr(weight), _code(weight.dtype), ctypes.c_float(eps), _ptr(out), _code(out.dtype),
                              _stream()), "layernorm")
    return out


def causal_conv(x: torch.Tensor, x_off: int, channels: int, w: torch.Tensor, bias: torch.Tensor | None,
                plan, state: torch.Tensor | None, out: torch.Tensor, out_off: int = 0, act: str = "none",
                add_input: bool = False) -> torch.Tensor:
    """out[r, out_off + c] = act([x +] [bias +] sum_j w[c, j] x_(t - taps + 1 + j)) on `channels`
    columns of the float32 rows x from x_off; the taps before a step's first row of a sequence are
    read from `state` [slot, taps - 1, channels] float32, which then takes the step's last inputs."""
    n, ld = x.shape
    taps = w.shape[1]
    assert x.dtype == torch.float32 and tuple(w.shape) == (channels, taps) and out.shape[0] == n
    assert bias is None or (bias.dtype == w.dtype and bias.numel() == channels)
    assert act in ("none", "silu")
    if taps > 1:
        assert state.dtype == torch.float32 and tuple(state.shape[1:]) == (taps - 1, channels)
    own = plan.n_rows == plan.n_seqs
    _check(lib().sb_causal_conv(_ptr(x), n, ld, x_off, channels, taps, _ptr(w), _ptr(bias), _code(w.dtype),
                                1 if act == "silu" else 0, 1 if add_input else 0, plan.n_seqs,
                                _i32(plan.row_seq, "row_seq"), _i32(plan.row_pos, "row_pos"),
                                _i32(plan.seq_row0, "seq_row0"), _i32(plan.seq_pos0, "seq_pos0"),
                                _i32(plan.seq_slot, "seq_slot"), _ptr(state), _ptr(out), _code(out.dtype),
                                out.shape[1], out_off, _stream()), "causal_conv",
           launches=1 if own or taps == 1 else 2)
    return out


# ---------------------------------------------------------------------- the generalized delta rule
def delta_prep(proj: torch.Tensor, k_off: int, a_off: int, z_off: int, n_heads: int, dim: int,
               w2: torch.Tensor, w0: torch.Tensor, a_bias: torch.Tensor, decay_scale: float, key_eps: float,
               aux: torch.Tensor) -> torch.Tensor:
    """aux [rows, 3, heads * dim] = decays exp(-decay_scale * sigmoid(w2 tanh(z1) + w0)) | removal
    rates sigmoid(a + a_bias) times the unit key | the unit key k / sqrt(sum k^2 + key_eps)."""
    n, ld = proj.shape
    hk, rank = n_heads * dim, w2.shape[1]
    assert proj.dtype == torch.float32 and aux.dtype == torch.float32 and tuple(aux.shape) == (n, 3, hk)
    assert w2.shape[0] == hk and w0.numel() == hk and a_bias.numel() == hk and w2.dtype == w0.dtype == a_bias.dtype
    _check(lib().sb_delta_prep(_ptr(proj), n, ld, k_off, a_off, z_off, n_heads, dim, rank, _ptr(w2), _ptr(w0),
                               _ptr(a_bias), _code(w2.dtype), ctypes.c_float(decay_scale), ctypes.c_float(key_eps),
                               _ptr(aux), _stream()), "delta_prep")
    return aux


def delta_scan(proj: torch.Tensor, r_off: int, k_off: int, v_off: int, aux: torch.Tensor, plan, n_heads: int,
               dim: int, state: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """S = diag(w) S - (a u)(u^T S) + k v^T, o = S^T r per head, token by token, from and to the
    state rows of the sequences' slots (float32 [slots, heads, dim, dim], value channel first)."""
    n, ld = proj.shape
    assert proj.dtype == torch.float32 and state.dtype == torch.float32 and out.dtype == torch.float32
    assert tuple(state.shape[1:]) == (n_heads, dim, dim) and tuple(out.shape) == (n, n_heads, dim)
    assert tuple(aux.shape) == (n, 3, n_heads * dim) and max(r_off, k_off, v_off) + n_heads * dim <= ld
    _check(lib().sb_delta_scan(_ptr(proj), ld, r_off, k_off, v_off, _ptr(aux), plan.n_seqs,
                               _i32(plan.seq_row0, "seq_row0"), _i32(plan.seq_slot, "seq_slot"), n_heads, dim,
                               _ptr(state), _ptr(out), _stream()), "delta_scan")
    return out


# ---------------------------------------------------------------------- the state-space mixer's rows
def ssd_prep(proj: torch.Tensor, dt_off: int, xbc: torch.Tensor, x_off: int, xdt_off: int, n_heads: int,
             vdim: int, dt_bias: torch.Tensor, a_log: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
    """decay [rows, heads] = exp(-exp(a_log) dt), dt = softplus(proj[dt_off + h] + dt_bias[h]); the
    columns of `xbc` at xdt_off receive dt * (its columns at x_off)."""
    n = proj.shape[0]
    assert proj.dtype == xbc.dtype == decay.dtype == torch.float32 and tuple(decay.shape) == (n, n_heads)
    assert dt_bias.dtype == a_log.dtype and dt_bias.numel() == a_log.numel() == n_heads and xbc.shape[0] == n
    _check(lib().sb_ssd_prep(_ptr(proj), n, proj.shape[1], dt_off, _ptr(xbc), xbc.shape[1], x_off, xdt_off,
                             n_heads, vdim, _ptr(dt_bias), _ptr(a_log), _code(a_log.dtype), _ptr(decay), _stream()),
           "ssd_prep")
    return decay


def ssd_out(o: torch.Tensor, xbc: torch.Tensor, x_off: int, proj: torch.Tensor, z_off: int, n_heads: int,
            vdim: int, norm_groups: int, d_skip: torch.Tensor, norm_w: torch.Tensor, eps: float,
            out: torch.Tensor) -> torch.Tensor:
    """out [rows, heads * vdim] = ((o + d_skip[h] x) silu(z)) / its root mean square over each of
    `norm_groups` equal parts of the row, times norm_w."""
    n, inner = o.shape[0], n_heads * vdim
    assert o.dtype == xbc.dtype == proj.dtype == torch.float32 and o.numel() == n * inner
    assert tuple(out.shape) == (n, inner) and d_skip.dtype == norm_w.dtype
    assert d_skip.numel() == n_heads and norm_w.numel() == inner
    _check(lib().sb_ssd_out(_ptr(o), _ptr(xbc), n, xbc.shape[1], x_off, _ptr(proj), proj.shape[1], z_off, n_heads,
                            vdim, norm_groups, _ptr(d_skip), _ptr(norm_w), _code(norm_w.dtype), ctypes.c_float(eps),
                            _ptr(out), _code(out.dtype), _stream()), "ssd_out")
    return out


# ---------------------------------------------------------------------- attention with logistic weights
def attention_sigmoid(q: torch.Tensor, out: torch.Tensor, plan, group_index: int, cache: torch.Tensor,
                      n_q_heads: int, n_kv_heads: int, head_dim: int, window: int, keep_first: int,
                      scale: float, softcap: float, head_bias: torch.Tensor | None) -> torch.Tensor:
    """Causal grouped-query attention whose weights are sigmoid(cap(q . k * scale) + head_bias[h]),
    not normalised over the keys, over one cache entry's pages.  Key j is visible to the query at
    position i when j <= i and (i - j < window or j < keep_first); window 0: every earlier key.
    bfloat16 at head sizes 64 and 128 runs on tensor cores, everything else the plain kernel."""
    n = q.shape[0]
    g = plan.groups[group_index]
    assert q.dtype == out.dtype and tuple(q.shape) == (n, n_q_heads, head_dim) and out.numel() == q.numel()
    assert head_bias is None or (head_bias.dtype == torch.float32 and head_bias.numel() == n_q_heads)
    _check(lib().sb_attention_sigmoid(
        _ptr(q), _ptr(out), _code(q.dtype), n, _i32(plan.row_seq, "row_seq"), _i32(plan.row_pos, "row_pos"),
        plan.n_seqs, plan.max_new, _i32(plan.seq_row0, "seq_row0"), _i32(plan.seq_pos0, "seq_pos0"),
        _i32(g.page_off, "page_off"), _i32(g.page_ids, "page_ids"), g.page_size, _ptr(cache), _code(cache.dtype),
        n_q_heads, n_kv_heads, head_dim, window, keep_first, ctypes.c_float(scale), ctypes.c_float(softcap),
        _ptr(head_bias), _stream()), "attention_sigmoid")
    return out


# ---------------------------------------------------------------------- mixture of experts
def moe_route(logits: torch.Tensor, top: int, ids: torch.Tensor, weights: torch.Tensor) -> None:
    """Per row of float32 logits [rows, experts]: the `top` largest (the lower index wins a tie) into
    ids [rows, top] int32, and their softmax over the chosen ones into weights [rows, top]."""
    n, e = logits.shape
    assert logits.dtype == weights.dtype == torch.float32 and ids.dtype == torch.int32
    assert tuple(ids.shape) == tuple(weights.shape) == (n, top)
    _check(lib().sb_moe_route(_ptr(logits), n, e, top, _ptr(ids), _ptr(weights), _stream()), "moe_route")


def moe_route_scored(logits: torch.Tensor, correction: torch.Tensor | None, top: int, ids: torch.Tensor,
                     weights: torch.Tensor, groups: tuple = (1, 1), group_top: int = 2, scale: float = 1.0,
                     renormalize: bool = False) -> None:
    """Per row of float32 logits: scores s = sigmoid(logits); the `top` experts with the largest
    choice scores s + correction (float32 [experts] or None; the lower index wins a tie) into ids, their
    s * scale (over the chosen ones' sum of s first when `renormalize`) into weights.  `groups` =
    (count, keep): the experts lie in `count` equal groups of neighbours, a group's score is the sum of
    its `group_top` largest choice scores, and only experts of the `keep` best groups can be chosen."""
    n, e = logits.shape
    assert logits.dtype == weights.dtype == torch.float32 and ids.dtype == torch.int32
    assert tuple(ids.shape) == tuple(weights.shape) == (n, top)
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == e)
    _check(lib().sb_moe_route_scored(_ptr(logits), _ptr(correction), n, e, top, int(groups[0]), int(groups[1]),
                                     int(group_top), ctypes.c_float(scale), 1 if renormalize else 0, _ptr(ids),
                                     _ptr(weights), _stream()), "moe_route_scored")


def moe_experts(h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_up: torch.Tensor,
                w_down: torch.Tensor, limit: float, slope: float, x: torch.Tensor) -> torch.Tensor:
    """x[r] += sum over the row's choices k of weights[r, k] * expert ids[r, k] applied to h[r]; an
    expert is down (g * sigmoid(slope g) * (u + 1)), g = min(gate h, limit), u = clamp(up h, +-limit).
    w_up [experts, 2 (gate, up), ff, width], w_down [experts, width, ff], both in h's dtype."""
    n, width = h.shape
    top = ids.shape[1]
    n_experts, _, ff, _ = w_up.shape
    assert tuple(w_up.shape) == (n_experts, 2, ff, width) and tuple(w_down.shape) == (n_experts, width, ff)
    assert h.dtype == w_up.dtype == w_down.dtype and x.dtype == torch.float32 and tuple(x.shape) == (n, width)
    pairs = n * top
    l = lib()
    order = torch.empty(pairs, dtype=torch.int32, device=h.device)
    tile = int(l.sb_moe_tile_rows(_code(h.dtype), pairs, n_experts, ff, width))
    meta = torch.empty(1 + 3 * int(l.sb_moe_max_tiles(pairs, n_experts, tile)), dtype=torch.int32, device=h.device)
    act = torch.empty((pairs, ff), dtype=h.dtype, device=h.device)
    pair_out = torch.empty((pairs, width), dtype=torch.float32, device=h.device)
    _check(l.sb_moe_group(_ptr(ids), pairs, n_experts, tile, _ptr(order), _ptr(meta), _stream()), "moe_group")
    _check(l.sb_moe_up(_ptr(h), _code(h.dtype), _ptr(w_up), _code(w_up.dtype), _ptr(order), _ptr(meta), pairs,
                       n_experts, tile, top, ff, width, ctypes.c_float(limit), ctypes.c_float(slope), _ptr(act),
                       _stream()), "moe_up")
    _check(l.sb_moe_down(_ptr(act), _code(act.dtype), _ptr(w_down), _code(w_down.dtype), _ptr(order), _ptr(meta),
                         pairs, n_experts, tile, top, width, ff, _ptr(pair_out), _stream()), "moe_down")
    _check(l.sb_moe_combine(_ptr(x), _ptr(pair_out), _ptr(weights), n, top, width, _stream()), "moe_combine")
    return x
