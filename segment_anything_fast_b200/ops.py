"""Tensor-level wrappers over the C ABI: torch owns memory and streams, the
library owns every kernel.  Each wrapper validates dtype/device/contiguity,
passes raw pointers plus the current CUDA stream, and raises on any error code.
"""
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import EPI_BIAS, EPI_GELU, EPI_RAW, EPI_RESIDUAL  # noqa: F401  (re-exported)

_status_words = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _same_device(index: Optional[int], name: str) -> None:
    """Every launch goes to the *current* device and its current stream (the C side reads the current
    device for its architecture check and SM count), so a tensor living on another GPU would hand that
    GPU's pointers to a kernel running here.  Reject it before anything is enqueued."""
    cur = torch.cuda.current_device()
    if index is not None and index != cur:
        raise RuntimeError(f"{name} is on cuda:{index} but the current device is cuda:{cur}; "
                           f"call torch.cuda.set_device({index}) (or use `with torch.cuda.device({index})`) first")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels write when a bounded wait expires."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel on ``device`` reported a device-side timeout."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    w = status_word(device)
    v = int(w.item())
    if v != 0:
        w.zero_()
        code = _lib.load().samb_decode_status(v)
        raise RuntimeError(f"device status 0x{v & 0xffffffff:08x}: {_lib.error_string(code)}")


def _need(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name}: expected a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected {dtype}, got {t.dtype}")
    _same_device(t.device.index, name)


def _rows2d(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dim() != 2 or t.stride(1) != 1:
        raise RuntimeError(f"{name}: expected a 2-D tensor with unit inner stride")
    return t


def window_rows(rows: int, grid: int, window: int) -> int:
    """Number of rows of the zero-padded window-partitioned layout."""
    if window == 0:
        return rows
    nw = -(-grid // window)
    return rows // (grid * grid) * nw * nw * window * window


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-6, grid: int = 0,
              window: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row LayerNorm of ``x [rows, C]`` (bf16); with ``window > 0`` the result is in the
    zero-padded window order (see ``samb_layernorm_bf16``)."""
    _need(x, torch.bfloat16, "x"); _need(gamma, torch.float32, "gamma"); _need(beta, torch.float32, "beta")
    x = _rows2d(x, "x")
    if not x.is_contiguous():
        raise RuntimeError("x must be contiguous")
    rows, C = x.shape
    orow = window_rows(rows, grid, window)
    if out is None:
        out = torch.empty(orow, C, dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.load().samb_layernorm_bf16(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(), rows, C,
                                               eps, grid, window, _stream()), "samb_layernorm_bf16")
    return out


def layernorm_quant_i8(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float = 1e-6, grid: int = 0,
                       window: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    _need(x, torch.bfloat16, "x"); _need(gamma, torch.float32, "gamma"); _need(beta, torch.float32, "beta")
    x = _rows2d(x, "x")
    if not x.is_contiguous():
        raise RuntimeError("x must be contiguous")
    rows, C = x.shape
    orow = window_rows(rows, grid, window)
    yq = torch.empty(orow, C, dtype=torch.int8, device=x.device)
    scale = torch.empty(orow, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().samb_layernorm_quant_i8(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), yq.data_ptr(),
                                                   scale.data_ptr(), rows, C, eps, grid, window, _stream()),
               "samb_layernorm_quant_i8")
    return yq, scale


def quant_rows_i8(x: torch.Tensor, gelu: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric int8 quantisation of bf16 rows; ``gelu`` applies the exact GELU (rounded to bf16) first."""
    _need(x, torch.bfloat16, "x")
    x = _rows2d(x, "x")
    if not x.is_contiguous():
        raise RuntimeError("x must be contiguous")
    rows, C = x.shape
    yq = torch.empty(rows, C, dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    fn = _lib.load().samb_gelu_quant_rows_i8 if gelu else _lib.load().samb_quant_rows_i8
    _lib.check(fn(x.data_ptr(), yq.data_ptr(), scale.data_ptr(), rows, C, _stream()),
               "samb_gelu_quant_rows_i8" if gelu else "samb_quant_rows_i8")
    return yq, scale


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
              residual: Optional[torch.Tensor] = None, gelu: bool = False, raw: bool = False,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``epilogue(a [M,K] @ w [N,K]^T)``; residual ``[R, N]`` with ``M % R == 0`` is broadcast over
    row blocks.  ``raw`` returns the fp32 accumulator."""
    _need(a, torch.bfloat16, "a"); _need(w, torch.bfloat16, "w")
    a, w = _rows2d(a, "a"), _rows2d(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise RuntimeError("gemm_bf16: inner dimensions differ")
    epi = 0
    if raw:
        epi = EPI_RAW
    else:
        if bias is not None:
            _need(bias, torch.float32, "bias"); epi |= EPI_BIAS
        if gelu:
            epi |= EPI_GELU
        if residual is not None:
            _need(residual, torch.bfloat16, "residual"); residual = _rows2d(residual, "residual"); epi |= EPI_RESIDUAL
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if raw else torch.bfloat16, device=a.device)
    out = _rows2d(out, "out")
    st = status_word(a.device)
    _lib.check(_lib.load().samb_gemm_bf16(
        a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), _ptr(bias), _ptr(residual),
        residual.stride(0) if residual is not None else 0, residual.shape[0] if residual is not None else 0,
        out.data_ptr(), out.stride(0), M, N, K, epi, st.data_ptr(), _stream()), "samb_gemm_bf16")
    return out


def gemm_i8(aq: torch.Tensor, a_scale: Optional[torch.Tensor], wq: torch.Tensor, w_scale: Optional[torch.Tensor],
            bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None, gelu: bool = False,
            raw: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """int8 x int8 -> int32 GEMM with the dequantising epilogue; ``raw`` returns the int32 accumulator."""
    _need(aq, torch.int8, "aq"); _need(wq, torch.int8, "wq")
    aq, wq = _rows2d(aq, "aq"), _rows2d(wq, "wq")
    M, K = aq.shape
    N = wq.shape[0]
    if wq.shape[1] != K:
        raise RuntimeError("gemm_i8: inner dimensions differ")
    epi = 0
    if raw:
        epi = EPI_RAW
    else:
        _need(a_scale, torch.float32, "a_scale"); _need(w_scale, torch.float32, "w_scale")
        if bias is not None:
            _need(bias, torch.float32, "bias"); epi |= EPI_BIAS
        if gelu:
            epi |= EPI_GELU
        if residual is not None:
            _need(residual, torch.bfloat16, "residual"); residual = _rows2d(residual, "residual"); epi |= EPI_RESIDUAL
    if out is None:
        out = torch.empty(M, N, dtype=torch.int32 if raw else torch.bfloat16, device=aq.device)
    st = status_word(aq.device)
    _lib.check(_lib.load().samb_gemm_i8(
        aq.data_ptr(), aq.stride(0), _ptr(a_scale), wq.data_ptr(), wq.stride(0), _ptr(w_scale), _ptr(bias),
        _ptr(residual), residual.stride(0) if residual is not None else 0,
        residual.shape[0] if residual is not None else 0, out.data_ptr(), out.stride(0), M, N, K, epi,
        st.data_ptr(), _stream()), "samb_gemm_i8")
    return out


def gemm_i8_requant(aq: torch.Tensor, a_scale: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor,
                    bias: Optional[torch.Tensor] = None, gelu: bool = False, out: Optional[torch.Tensor] = None,
                    meta: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """int8 Linear (+ bias, + GELU) whose output is also quantised per row for the next int8 Linear: returns
    ``(yq int8 [M, N], y_scale [M], out bf16 [M, N])``.  The row maxima come out of the GEMM epilogue (atomic
    maxima into a scratch array of M floats), so no pass over ``out`` reduces anything.  With ``meta`` the weight
    is the 2:4-compressed pair ``(wq = wc [N, K/2], meta)`` of ``pack_sp24``."""
    _need(aq, torch.int8, "aq"); _need(wq, torch.int8, "wq")
    _need(a_scale, torch.float32, "a_scale"); _need(w_scale, torch.float32, "w_scale")
    aq, wq = _rows2d(aq, "aq"), _rows2d(wq, "wq")
    M, K = aq.shape
    N = wq.shape[0]
    if wq.shape[1] * (2 if meta is not None else 1) != K:
        raise RuntimeError("gemm_i8_requant: inner dimensions differ")
    epi = 0
    if bias is not None:
        _need(bias, torch.float32, "bias"); epi |= EPI_BIAS
    if gelu:
        epi |= EPI_GELU
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
    yq = torch.empty(M, N, dtype=torch.int8, device=aq.device)
    y_scale = torch.empty(M, dtype=torch.float32, device=aq.device)
    scratch = torch.empty(M, dtype=torch.float32, device=aq.device)
    st = status_word(aq.device)
    if meta is not None:
        _need(meta, torch.uint8, "meta")
        _lib.check(_lib.load().samb_gemm_i8_sp24_requant(
            aq.data_ptr(), aq.stride(0), a_scale.data_ptr(), wq.data_ptr(), wq.stride(0), meta.data_ptr(),
            w_scale.data_ptr(), _ptr(bias), out.data_ptr(), out.stride(0), yq.data_ptr(), y_scale.data_ptr(),
            scratch.data_ptr(), M, N, K, epi, st.data_ptr(), _stream()), "samb_gemm_i8_sp24_requant")
        return yq, y_scale, out
    _lib.check(_lib.load().samb_gemm_i8_requant(
        aq.data_ptr(), aq.stride(0), a_scale.data_ptr(), wq.data_ptr(), wq.stride(0), w_scale.data_ptr(), _ptr(bias),
        out.data_ptr(), out.stride(0), yq.data_ptr(), y_scale.data_ptr(), scratch.data_ptr(), M, N, K, epi,
        st.data_ptr(), _stream()), "samb_gemm_i8_requant")
    return yq, y_scale, out


def pack_sp24(wq: torch.Tensor):
    """Compress a 2:4-sparse int8 weight ``wq [N, K]`` for ``gemm_i8_sp24``: returns ``(wc [N, K/2] int8,
    meta uint8)``.  A group of four with more than two non-zeros is reported by ``check_status``."""
    _need(wq, torch.int8, "wq")
    wq = _rows2d(wq, "wq")
    N, K = wq.shape
    lib = _lib.load()
    wc = torch.zeros(N, K // 2, dtype=torch.int8, device=wq.device)
    meta = torch.empty(max(int(lib.samb_sp24_meta_bytes(N, K)), 16), dtype=torch.uint8, device=wq.device)
    st = status_word(wq.device)
    _lib.check(lib.samb_pack_sp24(wq.data_ptr(), wq.stride(0), N, K, wc.data_ptr(), wc.stride(0), meta.data_ptr(),
                                  st.data_ptr(), _stream()), "samb_pack_sp24")
    return wc, meta


def gemm_i8_sp24(xq: torch.Tensor, x_scale: Optional[torch.Tensor], wc: torch.Tensor, meta: torch.Tensor,
                 w_scale: Optional[torch.Tensor], bias: Optional[torch.Tensor] = None,
                 residual: Optional[torch.Tensor] = None, gelu: bool = False, raw: bool = False,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``gemm_i8`` with the weight given as ``pack_sp24`` output (sparse tensor-core path)."""
    _need(xq, torch.int8, "xq"); _need(wc, torch.int8, "wc"); _need(meta, torch.uint8, "meta")
    xq, wc = _rows2d(xq, "xq"), _rows2d(wc, "wc")
    T, K = xq.shape
    N = wc.shape[0]
    if wc.shape[1] * 2 != K:
        raise RuntimeError("gemm_i8_sp24: inner dimensions differ")
    epi = 0
    if raw:
        epi = EPI_RAW
    else:
        _need(x_scale, torch.float32, "x_scale"); _need(w_scale, torch.float32, "w_scale")
        if bias is not None:
            _need(bias, torch.float32, "bias"); epi |= EPI_BIAS
        if gelu:
            epi |= EPI_GELU
        if residual is not None:
            _need(residual, torch.bfloat16, "residual"); residual = _rows2d(residual, "residual"); epi |= EPI_RESIDUAL
    if out is None:
        out = torch.empty(T, N, dtype=torch.int32 if raw else torch.bfloat16, device=xq.device)
    st = status_word(xq.device)
    _lib.check(_lib.load().samb_gemm_i8_sp24(
        xq.data_ptr(), xq.stride(0), _ptr(x_scale), wc.data_ptr(), wc.stride(0), meta.data_ptr(), _ptr(w_scale),
        _ptr(bias), _ptr(residual), residual.stride(0) if residual is not None else 0,
        residual.shape[0] if residual is not None else 0, out.data_ptr(), out.stride(0), T, N, K, epi,
        st.data_ptr(), _stream()), "samb_gemm_i8_sp24")
    return out


def layernorm2d(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, hw: int, eps: float = 1e-6,
                to_nchw: bool = False) -> torch.Tensor:
    """Channel LayerNorm of token rows ``x [tokens, C]``; ``to_nchw`` stores ``[tokens/hw, C, hw]``."""
    _need(x, torch.bfloat16, "x"); _need(gamma, torch.float32, "gamma"); _need(beta, torch.float32, "beta")
    x = _rows2d(x, "x")
    if not x.is_contiguous():
        raise RuntimeError("x must be contiguous")
    tokens, C = x.shape
    out = torch.empty((tokens // hw, C, hw) if to_nchw else (tokens, C), dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.load().samb_layernorm2d_nchw(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(),
                                                 tokens, C, hw, eps, int(to_nchw), _stream()), "samb_layernorm2d_nchw")
    return out


def selftest_bounded_wait(limit_polls: int = 20000) -> int:
    """Run the give-up path of the bounded barrier wait; returns the raw status word."""
    w = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(_lib.load().samb_selftest_bounded_wait(w.data_ptr(), limit_polls, _stream()),
               "samb_selftest_bounded_wait")
    return int(w.item())


def attn_relpos_global(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rel_h: torch.Tensor,
                       rel_w: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Global-block attention with rel-pos bias: q, k, v ``[B,H,N,d]``, rel_h ``[B,H,N,N/64]``,
    rel_w ``[B,H,N,64]`` (all contiguous, all bfloat16 or all float16) -> ``[B,H,N,d]`` of the same type."""
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"q must be bfloat16 or float16, got {q.dtype}")
    for name, t in (("q", q), ("k", k), ("v", v), ("rel_h", rel_h), ("rel_w", rel_w)):
        _need(t, q.dtype, name)
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    B, H, N, d = q.shape
    if rel_h.shape != (B, H, N, N // 64) or rel_w.shape != (B, H, N, 64):
        raise RuntimeError("rel_h / rel_w shapes do not match q")
    o = torch.empty_like(q)
    st = status_word(q.device)
    lib = _lib.load()
    fn = lib.samb_attn_relpos_global_f16 if q.dtype == torch.float16 else lib.samb_attn_relpos_global
    _lib.check(fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), rel_h.data_ptr(), rel_w.data_ptr(), o.data_ptr(), B, H, N, d,
                  float(scale if scale is not None else d ** -0.5), st.data_ptr(), _stream()), "samb_attn_relpos_global")
    return o


def attn_relpos_global_qkv(qkv: torch.Tensor, tab: torch.Tensor, t_head_stride: int, t_w_off: int, B: int, H: int,
                           N: int, d: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Global-block attention over the head-major ``qkv [3H, B*N, d]`` buffer with the bias taken from
    the table products ``tab [B*N, ldt]``; returns ``[B*N, H*d]``."""
    _need(qkv, torch.bfloat16, "qkv"); _need(tab, torch.bfloat16, "tab")
    if not qkv.is_contiguous() or qkv.shape != (3 * H, B * N, d):
        raise RuntimeError("qkv must be contiguous [3H, B*N, d]")
    tab = _rows2d(tab, "tab")
    if out is None:
        out = torch.empty(B * N, H * d, dtype=torch.bfloat16, device=qkv.device)
    st = status_word(qkv.device)
    _lib.check(_lib.load().samb_attn_relpos_global_qkv(
        qkv.data_ptr(), tab.data_ptr(), tab.stride(0), t_head_stride, t_w_off, out.data_ptr(), out.stride(0), B, H, N,
        d, float(d ** -0.5), st.data_ptr(), _stream()), "samb_attn_relpos_global_qkv")
    return out


def attn_relpos_global_tables(qkv: torch.Tensor, tables: torch.Tensor, B: int, H: int, N: int, d: int,
                              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Global-block attention over the head-major ``qkv [3H, B*N, d]`` buffer with the rel-pos bias computed inside
    the kernel from ``tables [256, d]`` (rel_pos_h from row 0, rel_pos_w from row 128); returns ``[B*N, H*d]``."""
    _need(qkv, torch.bfloat16, "qkv"); _need(tables, torch.bfloat16, "tables")
    if not qkv.is_contiguous() or qkv.shape != (3 * H, B * N, d):
        raise RuntimeError("qkv must be contiguous [3H, B*N, d]")
    if not tables.is_contiguous() or tables.shape != (256, d):
        raise RuntimeError("tables must be contiguous [256, d]")
    if out is None:
        out = torch.empty(B * N, H * d, dtype=torch.bfloat16, device=qkv.device)
    st = status_word(qkv.device)
    _lib.check(_lib.load().samb_attn_relpos_global_tables(
        qkv.data_ptr(), tables.data_ptr(), out.data_ptr(), out.stride(0), B, H, N, d, float(d ** -0.5), st.data_ptr(),
        _stream()), "samb_attn_relpos_global_tables")
    return out


def attn_relpos_window(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rel_h: torch.Tensor,
                       rel_w: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Windowed attention with rel-pos bias: q, k, v ``[B,H,196,d]``, rel_h / rel_w ``[B,H,196,14]`` (all bfloat16 or
    all float16) -> ``[B,H,196,d]`` of the same type."""
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"q must be bfloat16 or float16, got {q.dtype}")
    for name, t in (("q", q), ("k", k), ("v", v), ("rel_h", rel_h), ("rel_w", rel_w)):
        _need(t, q.dtype, name)
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    B, H, N, d = q.shape
    ws = int(round(N ** 0.5))
    if ws * ws != N or rel_h.shape != (B, H, N, ws) or rel_w.shape != (B, H, N, ws):
        raise RuntimeError("rel_h / rel_w shapes do not match q")
    o = torch.empty_like(q)
    st = status_word(q.device)
    lib = _lib.load()
    fn = lib.samb_attn_relpos_window_f16 if q.dtype == torch.float16 else lib.samb_attn_relpos_window
    _lib.check(fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), rel_h.data_ptr(), rel_w.data_ptr(), o.data_ptr(), B, H, ws, d,
                  float(scale if scale is not None else d ** -0.5), st.data_ptr(), _stream()), "samb_attn_relpos_window")
    return o


def attn_relpos_window_qkv(qkv: torch.Tensor, tab: torch.Tensor, t_head_stride: int, t_w_off: int, B: int, H: int,
                           grid: int, window: int, d: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Windowed attention over the window-ordered head-major ``qkv [3H, B*nw*nw*window^2, d]``; returns
    raster-order ``[B*grid*grid, H*d]`` (pad tokens dropped)."""
    _need(qkv, torch.bfloat16, "qkv"); _need(tab, torch.bfloat16, "tab")
    rows = window_rows(B * grid * grid, grid, window)
    if not qkv.is_contiguous() or qkv.shape != (3 * H, rows, d):
        raise RuntimeError("qkv must be contiguous [3H, B*nw*nw*window^2, d]")
    tab = _rows2d(tab, "tab")
    if out is None:
        out = torch.empty(B * grid * grid, H * d, dtype=torch.bfloat16, device=qkv.device)
    st = status_word(qkv.device)
    _lib.check(_lib.load().samb_attn_relpos_window_qkv(
        qkv.data_ptr(), tab.data_ptr(), tab.stride(0), t_head_stride, t_w_off, out.data_ptr(), out.stride(0), B, H,
        grid, window, d, float(d ** -0.5), st.data_ptr(), _stream()), "samb_attn_relpos_window_qkv")
    return out


def attn_relpos_window_raster(qkv: torch.Tensor, qkv_bias: torch.Tensor, tab: torch.Tensor, t_head_stride: int,
                              t_w_off: int, B: int, H: int, grid: int, window: int, d: int,
                              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Windowed attention over raster-order head-major ``qkv [3H, B*grid*grid, d]`` (no padded copy of the
    tokens); ``qkv_bias`` is the projection bias as bf16 ``[3H*d]`` (the keys / values of the zero-padded
    tokens of border windows).  Returns raster-order ``[B*grid*grid, H*d]``."""
    _need(qkv, torch.bfloat16, "qkv"); _need(tab, torch.bfloat16, "tab"); _need(qkv_bias, torch.bfloat16, "qkv_bias")
    if not qkv.is_contiguous() or qkv.shape != (3 * H, B * grid * grid, d):
        raise RuntimeError("qkv must be contiguous [3H, B*grid*grid, d]")
    if not qkv_bias.is_contiguous() or qkv_bias.numel() != 3 * H * d:
        raise RuntimeError("qkv_bias must be contiguous [3H*d]")
    tab = _rows2d(tab, "tab")
    if out is None:
        out = torch.empty(B * grid * grid, H * d, dtype=torch.bfloat16, device=qkv.device)
    st = status_word(qkv.device)
    _lib.check(_lib.load().samb_attn_relpos_window_raster(
        qkv.data_ptr(), qkv_bias.data_ptr(), tab.data_ptr(), tab.stride(0), t_head_stride, t_w_off, out.data_ptr(),
        out.stride(0), B, H, grid, window, d, float(d ** -0.5), st.data_ptr(), _stream()),
        "samb_attn_relpos_window_raster")
    return out


def attn_relpos_window_tables(qkv: torch.Tensor, qkv_bias: torch.Tensor, tables: torch.Tensor, B: int, H: int,
                              grid: int, window: int, d: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``attn_relpos_window_raster`` with the rel-pos bias computed inside the kernel from ``tables [64, d]``
    (rel_pos_h from row 0, rel_pos_w from row 32).  Returns raster-order ``[B*grid*grid, H*d]``."""
    _need(qkv, torch.bfloat16, "qkv"); _need(tables, torch.bfloat16, "tables"); _need(qkv_bias, torch.bfloat16, "qkv_bias")
    if not qkv.is_contiguous() or qkv.shape != (3 * H, B * grid * grid, d):
        raise RuntimeError("qkv must be contiguous [3H, B*grid*grid, d]")
    if not qkv_bias.is_contiguous() or qkv_bias.numel() != 3 * H * d:
        raise RuntimeError("qkv_bias must be contiguous [3H*d]")
    if not tables.is_contiguous() or tables.shape != (64, d):
        raise RuntimeError("tables must be contiguous [64, d]")
    if out is None:
        out = torch.empty(B * grid * grid, H * d, dtype=torch.bfloat16, device=qkv.device)
    st = status_word(qkv.device)
    _lib.check(_lib.load().samb_attn_relpos_window_tables(
        qkv.data_ptr(), qkv_bias.data_ptr(), tables.data_ptr(), out.data_ptr(), out.stride(0), B, H, grid, window, d,
        float(d ** -0.5), st.data_ptr(), _stream()), "samb_attn_relpos_window_tables")
    return out


def gemm_heads(a: torch.Tensor, a_scale: Optional[torch.Tensor], w: torch.Tensor, w_scale: Optional[torch.Tensor],
               bias: Optional[torch.Tensor], head_dim: int) -> torch.Tensor:
    """qkv projection with a head-major result ``[N/head_dim, M, head_dim]`` (bf16).  ``a``/``w`` are bf16,
    or int8 with their row scales."""
    a, w = _rows2d(a, "a"), _rows2d(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if bias is not None:
        _need(bias, torch.float32, "bias")
    out = torch.empty(N // head_dim, M, head_dim, dtype=torch.bfloat16, device=a.device)
    st = status_word(a.device)
    if a.dtype == torch.int8:
        _need(w, torch.int8, "w"); _need(a_scale, torch.float32, "a_scale"); _need(w_scale, torch.float32, "w_scale")
        _lib.check(_lib.load().samb_gemm_i8_heads(a.data_ptr(), a.stride(0), a_scale.data_ptr(), w.data_ptr(), w.stride(0),
                                                  w_scale.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, head_dim,
                                                  st.data_ptr(), _stream()), "samb_gemm_i8_heads")
    else:
        _need(a, torch.bfloat16, "a"); _need(w, torch.bfloat16, "w")
        _lib.check(_lib.load().samb_gemm_bf16_heads(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), _ptr(bias),
                                                    out.data_ptr(), M, N, K, head_dim, st.data_ptr(), _stream()),
                   "samb_gemm_bf16_heads")
    return out


def relpos_table_products(qkv_hm: torch.Tensor, tables: torch.Tensor, col_scale: torch.Tensor, H: int,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``tab[t, h*T + m] = (q_h[t] . tables[m]) * col_scale[m]`` for the H query planes of the head-major
    ``qkv_hm [3H, rows, d]``; ``T = tables.shape[0]``."""
    _need(qkv_hm, torch.bfloat16, "qkv_hm"); _need(tables, torch.bfloat16, "tables"); _need(col_scale, torch.float32, "col_scale")
    if qkv_hm.dim() != 3 or not qkv_hm.is_contiguous() or qkv_hm.shape[0] != 3 * H:
        raise RuntimeError("qkv_hm must be a contiguous [3H, rows, d] tensor")
    _, rows, d = qkv_hm.shape
    T = tables.shape[0]
    if not tables.is_contiguous() or tables.shape != (T, d) or col_scale.shape != (T,):
        raise RuntimeError("tables must be contiguous [T, d] with a [T] scale")
    if out is None:
        out = torch.empty(rows, H * T, dtype=torch.bfloat16, device=qkv_hm.device)
    st = status_word(qkv_hm.device)
    _lib.check(_lib.load().samb_relpos_table_products(
        qkv_hm.data_ptr(), tables.data_ptr(), col_scale.data_ptr(), out.data_ptr(), out.stride(0), rows, H, d, T,
        st.data_ptr(), _stream()), "samb_relpos_table_products")
    return out


def patch_rows(x: torch.Tensor, patch: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """NCHW image batch ``[B,Cin,S,S]`` (bf16) -> patch rows ``[B*(S/patch)^2, Cin*patch*patch]``."""
    _need(x, torch.bfloat16, "x")
    if x.dim() != 4 or not x.is_contiguous() or x.shape[2] != x.shape[3] or x.shape[2] % patch:
        raise RuntimeError("x must be a contiguous square NCHW batch whose side is a multiple of the patch size")
    B, Cin, S, _ = x.shape
    grid = S // patch
    if out is None:
        out = torch.empty(B * grid * grid, Cin * patch * patch, dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.load().samb_patch_rows(x.data_ptr(), out.data_ptr(), B, Cin, grid, patch, _stream()), "samb_patch_rows")
    return out


def patch_rows_u8(x: torch.Tensor, patch: int, mean, std, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """uint8 NCHW image batch ``[B,3,S,S]`` -> normalised bf16 patch rows ``[B*(S/patch)^2, 3*patch*patch]``
    (``(x - mean[c]) / std[c]``, then the gather of ``patch_rows``) in one pass."""
    import ctypes
    _need(x, torch.uint8, "x")
    if x.dim() != 4 or not x.is_contiguous() or x.shape[1] != 3 or x.shape[2] != x.shape[3] or x.shape[2] % patch:
        raise RuntimeError("x must be a contiguous square [B,3,S,S] uint8 batch whose side is a multiple of the patch size")
    B, Cin, S, _ = x.shape
    grid = S // patch
    if out is None:
        out = torch.empty(B * grid * grid, Cin * patch * patch, dtype=torch.bfloat16, device=x.device)
    m = (ctypes.c_float * 3)(*[float(v) for v in mean])
    s = (ctypes.c_float * 3)(*[float(v) for v in std])
    _lib.check(_lib.load().samb_patch_rows_u8(x.data_ptr(), out.data_ptr(), B, Cin, grid, patch, m, s, _stream()),
               "samb_patch_rows_u8")
    return out


def conv3x3_rows(x: torch.Tensor, grid: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token rows ``[tokens, C]`` -> 3x3 neighbourhood rows ``[tokens, 9*C]`` (zero padding 1)."""
    _need(x, torch.bfloat16, "x")
    x = _rows2d(x, "x")
    if not x.is_contiguous():
        raise RuntimeError("x must be contiguous")
    tokens, C = x.shape
    if out is None:
        out = torch.empty(tokens, 9 * C, dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.load().samb_conv3x3_rows(x.data_ptr(), out.data_ptr(), tokens, grid, C, _stream()), "samb_conv3x3_rows")
    return out


def normalize_u8(x: torch.Tensor, mean, std, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """uint8 ``[B,3,H,W]`` -> bf16 ``(x - mean[c]) / std[c]``."""
    import ctypes
    _need(x, torch.uint8, "x")
    if x.dim() != 4 or not x.is_contiguous():
        raise RuntimeError("x must be a contiguous [B,3,H,W] uint8 tensor")
    B, C, H, W = x.shape
    if out is None:
        out = torch.empty(B, C, H, W, dtype=torch.bfloat16, device=x.device)
    m = (ctypes.c_float * 3)(*[float(v) for v in mean])
    s = (ctypes.c_float * 3)(*[float(v) for v in std])
    _lib.check(_lib.load().samb_normalize_u8(x.data_ptr(), out.data_ptr(), B, C, H, W, m, s, _stream()), "samb_normalize_u8")
    return out
