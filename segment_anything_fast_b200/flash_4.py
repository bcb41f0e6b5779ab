"""Drop-in for ``segment_anything_fast.flash_4``'s two plug points on the attention path:

* ``_attention_rel_h_rel_w(q_, k_, v_, rel_h_, rel_w_)`` (flash_4.py:335-370), the function
  ``modeling/image_encoder.py:15,245`` imports and calls.  Same argument layout, B200 kernels underneath, and
  no SDPA fallback: shapes or dtypes the kernels do not cover raise.
* the dispatcher op ``customflash::custom_flash_aligned(q, k, v, rel_h_w, sm_scale)`` (flash_4.py:268-279),
  registered here as ``samb200::custom_flash_aligned`` with the same schema and ``CUDA`` + ``Meta``
  implementations.  The namespace differs on purpose: the reference defines ``customflash`` when it is
  imported, and both packages may live in one process.

Both kernels exist for bfloat16 and for float16 tensors, the two types the reference's own test of the operator
sweeps (test/test_flash_4.py:41-43).  Any other type is rejected rather than converted, and so are mixed types: a
silent conversion would change the precision the caller asked for.
"""
import torch

from . import ops

_lib = torch.library.Library("samb200", "FRAGMENT")
_lib.define("custom_flash_aligned(Tensor q, Tensor k, Tensor v, Tensor rel_h_w, float sm_scale) -> Tensor")


def _check_dtype(*tensors: torch.Tensor) -> None:
    want = tensors[0].dtype
    if want not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"the B200 attention kernels take bfloat16 or float16 tensors, got {want}; "
                           "convert explicitly with .to(torch.bfloat16) if that precision is acceptable")
    for t in tensors:
        if t.dtype != want:
            raise RuntimeError(f"q, k, v and the bias tensors must share one dtype, got {want} and {t.dtype}")


@torch.library.impl(_lib, "custom_flash_aligned", "Meta")
def _custom_flash_aligned_meta(q, k, v, rel_h_w, sm_scale):
    return torch.empty_like(q, memory_format=torch.contiguous_format)


@torch.library.impl(_lib, "custom_flash_aligned", "CUDA")
def _custom_flash_aligned_cuda(q, k, v, rel_h_w, sm_scale):
    """q, k, v ``[B, H, N, d]``; ``rel_h_w [B, H, N, N/64 + 64]`` = ``cat(rel_h, rel_w)`` along the last axis, the
    layout flash_4.py:352,363 builds.  Head dim 64 or 80 (un-padded: the reference pads 80 to 128 for its Triton
    kernel, flash_4.py:359-361; this kernel runs 80 natively, so a 128-wide zero-padded tensor is refused)."""
    _check_dtype(q, k, v, rel_h_w)
    B, H, N, d = q.shape
    Sh = N // 64
    if d not in (64, 80):
        raise RuntimeError(f"custom_flash_aligned: head dim {d} is not supported (64 or 80; pass ViT-H heads un-padded)")
    if rel_h_w.shape != (B, H, N, Sh + 64) or N % 256 or N > 4096:
        raise RuntimeError("custom_flash_aligned: expected N a multiple of 256 up to 4096 and rel_h_w [B, H, N, N/64 + 64]")
    rel_h = rel_h_w[..., :Sh].contiguous()
    rel_w = rel_h_w[..., Sh:].contiguous()
    return ops.attn_relpos_global(q.contiguous(), k.contiguous(), v.contiguous(), rel_h, rel_w, scale=float(sm_scale))


def _attention_rel_h_rel_w(q_: torch.Tensor, k_: torch.Tensor, v_: torch.Tensor, rel_h_: torch.Tensor,
                           rel_w_: torch.Tensor) -> torch.Tensor:
    """q_, k_, v_: ``[B, H, N, d]``; rel_h_: ``[B, H, N, Sh, 1]``; rel_w_: ``[B, H, N, 1, Sw]``; all bfloat16 or all
    float16."""
    B, H, N, d = q_.shape
    _check_dtype(q_, k_, v_, rel_h_, rel_w_)
    rel_h = rel_h_.squeeze(-1).contiguous()
    rel_w = rel_w_.squeeze(-2).contiguous()
    q, k, v = (t.contiguous() for t in (q_, k_, v_))
    if rel_w.shape[-1] == 64 and N % 256 == 0 and N <= 4096 and d in (64, 80):
        return ops.attn_relpos_global(q, k, v, rel_h, rel_w)
    if N == 196 and rel_w.shape[-1] == 14 and d in (64, 80):
        return ops.attn_relpos_window(q, k, v, rel_h, rel_w)
    raise RuntimeError(f"attention shape N={N}, d={d}, bias widths {rel_h.shape[-1]}x{rel_w.shape[-1]} is not covered "
                       "by the B200 kernels (64-wide rasters of up to 4096 tokens in multiples of 256, or 14x14 windows)")
