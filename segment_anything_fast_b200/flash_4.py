"""Drop-in for ``segment_anything_fast.flash_4._attention_rel_h_rel_w`` (flash_4.py:335-370): the function
``modeling/image_encoder.py:15,245`` imports and calls.  Same argument layout, B200 kernels underneath,
and no SDPA fallback: shapes the kernels do not cover raise."""
import torch

from . import ops


def _attention_rel_h_rel_w(q_: torch.Tensor, k_: torch.Tensor, v_: torch.Tensor, rel_h_: torch.Tensor,
                           rel_w_: torch.Tensor) -> torch.Tensor:
    """q_, k_, v_: ``[B, H, N, d]``; rel_h_: ``[B, H, N, Sh, 1]``; rel_w_: ``[B, H, N, 1, Sw]``."""
    B, H, N, d = q_.shape
    dt = q_.dtype
    rel_h = rel_h_.squeeze(-1).to(torch.bfloat16).contiguous()
    rel_w = rel_w_.squeeze(-2).to(torch.bfloat16).contiguous()
    q, k, v = (t.to(torch.bfloat16).contiguous() for t in (q_, k_, v_))
    if rel_w.shape[-1] == 64 and N % 128 == 0 and N <= 4096 and d in (64, 80):
        return ops.attn_relpos_global(q, k, v, rel_h, rel_w).to(dt)
    if N == 196 and rel_w.shape[-1] == 14 and d in (64, 80):
        return ops.attn_relpos_window(q, k, v, rel_h, rel_w).to(dt)
    raise RuntimeError(f"attention shape N={N}, d={d}, bias widths {rel_h.shape[-1]}x{rel_w.shape[-1]} is not covered "
                       "by the B200 kernels (64-wide rasters up to 4096 tokens, or 14x14 windows)")
