"""CPU restatement of the int8 dynamic-quant and 2:4 pruning arithmetic (checker only).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the
benchmark's CPU-baseline leg.  The shipped package never imports it.

PARITY UNPINNED for the int8 part: the reference gets it from ``torchao``
(``apply_dynamic_quant``, call site experiments/eval_combo.py:357-360; declared
without a version pin at setup.py:16), which is neither vendored in the
reference tree nor installed here, and the reference has no test or golden
vector for it.  The arithmetic below is therefore the published per-token /
per-channel symmetric absmax scheme as the benchmark configuration states it:

    s_tok = max(absmax_row(X), 1e-5) / 127 ;  Xq = clamp(rint(X / s_tok), -127, 127)
    s_ch  = max(absmax_row(W), 1e-5) / 127 ;  Wq = clamp(rint(W / s_ch),  -127, 127)
    acc   = int32(Xq) @ int32(Wq)^T                      (exact integer arithmetic)
    Y     = bf16(float(acc) * s_tok * s_ch + bias)       (optionally GELU before rounding)

The 1e-5 floor is the all-zero-row guard (zero-padded window tokens after
LayerNorm are exactly zero).  ``rint`` is round-half-to-even, the rounding of
``torch.round``.  The 2:4 mask IS pinned: the CPU tests compare
:func:`prune_2_4_mask` with the mask ``apply_fake_sparsity`` (sparse.py:6-25)
produced here on seeded weights (stored under tests/golden/).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

ABSMAX_FLOOR = 1e-5


def quantize_rows_absmax(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric per-row int8 quantisation of a 2-D float tensor.
    Returns (int8 ``[R, K]``, float32 scale ``[R]``)."""
    xf = x.to(torch.float32)
    scale = xf.abs().amax(dim=-1).clamp(min=ABSMAX_FLOOR) / 127.0
    q = torch.round(xf / scale[:, None]).clamp(-127, 127).to(torch.int8)
    return q, scale


def int8_matmul_i32(xq: torch.Tensor, wq: torch.Tensor) -> torch.Tensor:
    """Exact ``int32(Xq) @ int32(Wq)^T`` → int32 ``[M, N]``.  Evaluated as a float64 matmul: every product and
    every partial sum is an integer of magnitude at most 127²·K < 2^53, which float64 holds exactly, so the result
    is the integer product whatever order a BLAS kernel sums in (and it runs a hundred times faster than
    torch's int64 matmul, which matters at ViT-H size).  |acc| fits int32 for K < 133 000."""
    return (xq.to(torch.float64) @ wq.to(torch.float64).t()).to(torch.int32)


def int8_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                gelu: bool = False, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dynamic-quant Linear on a bf16-valued activation ``x [M, K]`` and float
    weight ``w [N, K]``; returns bf16-rounded float32 ``[M, N]``."""
    xq, s_tok = quantize_rows_absmax(x)
    wq, s_ch = quantize_rows_absmax(w)
    acc = int8_matmul_i32(xq, wq)
    y = acc.to(torch.float32) * s_tok[:, None] * s_ch[None, :]
    if bias is not None:
        y = y + bias.to(torch.float32)[None, :]
    if gelu:
        y = F.gelu(y)
    if residual is not None:
        y = y + residual.to(torch.float32)
    return y.to(torch.bfloat16).to(torch.float32)


def prune_2_4_mask(w: torch.Tensor) -> torch.Tensor:
    """Boolean keep-mask: in every group of 4 consecutive in-features keep the 2
    entries of largest magnitude — what ``WeightNormSparsifier(sparsity_level=1.0,
    sparse_block_shape=(1,4), zeros_per_block=2)`` leaves after ``squash_mask``
    (sparse.py:18-25).  Ties keep the lower index (immaterial for continuous
    random weights)."""
    N, K = w.shape
    if K % 4:
        raise ValueError("in-features must be a multiple of 4")
    mag = w.to(torch.float32).abs().reshape(N, K // 4, 4)
    order = torch.argsort(mag, dim=-1, descending=True, stable=True)
    keep = torch.zeros_like(mag, dtype=torch.bool)
    keep.scatter_(-1, order[..., :2], True)
    return keep.reshape(N, K)


def compress_2_4(wq: torch.Tensor, keep: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Pack a 2:4 int8 weight: values ``[N, K/2]`` (kept entries in order) and the
    2-bit in-group positions ``[N, K/2]`` (uint8 in 0..3) of each kept entry."""
    N, K = wq.shape
    pos = torch.arange(4).expand(N, K // 4, 4)[keep.reshape(N, K // 4, 4)].reshape(N, K // 2)
    vals = wq[keep].reshape(N, K // 2)
    return vals, pos.to(torch.uint8)
