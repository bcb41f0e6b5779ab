"""The fused mask-filter kernel against the CPU oracle and the reference's own outputs (integer exact)."""
import os

import numpy as np
import pytest
import torch

from oracle import amg_oracle as ao

pytestmark = pytest.mark.gpu


def _check(logits: torch.Tensor, thr: float, off: float):
    from segment_anything_fast_b200 import amg, ops
    score, boxes, binary = amg.mask_stats(logits.cuda(), thr, off)
    ops.check_status()
    x = logits.float().numpy()
    inter, uni = ao.stability_counts(x, thr, off)
    ref_score = torch.from_numpy(inter) / torch.from_numpy(uni)
    assert torch.equal(torch.nan_to_num(score.cpu(), nan=-1.0), torch.nan_to_num(ref_score, nan=-1.0))
    assert np.array_equal(boxes.cpu().numpy(), ao.batched_mask_to_box(x > np.float32(thr)))
    assert np.array_equal(binary.cpu().numpy(), x > np.float32(thr))
    return score, boxes


def test_mask_stats_matches_reference_outputs(golden_dir):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    g = np.load(os.path.join(golden_dir, "amg_fp32.npz"))
    score, boxes = _check(torch.from_numpy(g["logits"]), 0.0, 1.0)
    assert np.array_equal(np.nan_to_num(score.cpu().numpy(), nan=-1), np.nan_to_num(g["score"], nan=-1))
    assert np.array_equal(boxes.cpu().numpy(), g["boxes"])
    from segment_anything_fast_b200 import amg
    b2 = amg.batched_mask_to_box(torch.from_numpy(g["logits"] > 0).cuda())
    assert np.array_equal(b2.cpu().numpy(), g["boxes"])


@pytest.mark.parametrize("N,H,W,dtype", [(5, 1024, 1024, torch.float32), (3, 683, 1023, torch.float32),
                                         (4, 480, 640, torch.bfloat16), (2, 97, 131, torch.bfloat16), (1, 1, 1, torch.float32)])
def test_mask_stats_shapes_and_alignment(N, H, W, dtype):
    """Full-size masks, odd sizes (masks that start off a 16-byte boundary take the scalar path), bf16 logits."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    g = torch.Generator().manual_seed(N * 1000 + W)
    logits = (torch.randn(N, H, W, generator=g) * 2.0 - 1.0).to(dtype)
    if N > 2:
        logits[1] = -9.0
        logits[2, : H // 2] = -9.0
    _check(logits, 0.0, 1.0)
    _check(logits, 0.5, 0.25)
