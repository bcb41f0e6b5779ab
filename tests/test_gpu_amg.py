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


def _rle_check(masks: torch.Tensor, cap: int = 4096):
    from segment_anything_fast_b200 import amg, ops
    got = amg.mask_to_rle_pytorch(masks.cuda()) if cap == 4096 else None
    counts, n = amg.mask_rle_counts(masks.cuda(), cap=cap)
    ops.check_status()
    want = ao.mask_to_rle(masks.numpy())
    assert n.cpu().tolist() == [len(r["counts"]) for r in want]
    rows = counts.cpu().tolist()
    for r, k, w in zip(rows, n.cpu().tolist(), want):
        assert r[:k] == w["counts"]
    if got is not None:
        assert got == want
    return want


def test_mask_rle_matches_reference_outputs(golden_dir):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    g = np.load(os.path.join(golden_dir, "amg_fp32.npz"))
    masks = torch.from_numpy(g["logits"] > 0)            # includes an empty and a full mask, W % 4 != 0
    want = _rle_check(masks)
    assert [len(r["counts"]) for r in want] == g["rle_len"].tolist()
    assert np.array_equal(np.concatenate([np.asarray(r["counts"]) for r in want]), g["rle_counts"])


@pytest.mark.parametrize("N,H,W", [(6, 1024, 1024), (3, 683, 1023), (4, 480, 640), (2, 97, 131), (1, 1, 1), (2, 5, 4096),
                                   (2, 300, 2050), (3, 1, 37), (3, 257, 1), (1, 4200, 4096)])
def test_mask_rle_shapes(N, H, W):
    """Blob-like masks (a smooth field thresholded), noise masks, empty / full / single-pixel masks at aligned and odd
    sizes (the tall one exceeds what a thread's change list can index and takes the second walk); every encoding is
    bit-exact and decodes back to its mask."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    g = torch.Generator().manual_seed(N * 7919 + W)
    ys = torch.linspace(0, 6.0, H)[:, None]
    xs = torch.linspace(0, 6.0, W)[None, :]
    masks = torch.zeros(N, H, W, dtype=torch.bool)
    for i in range(N):
        ph = torch.rand(4, generator=g) * 6.28
        field = torch.sin(ys * 1.7 + ph[0]) * torch.cos(xs * 2.3 + ph[1]) + 0.5 * torch.sin((ys + xs) * 3.1 + ph[2])
        masks[i] = field > 0.2
    if N > 1:
        masks[1] = torch.rand(H, W, generator=g) > 0.5                   # noise: about H*W/2 runs (cap grows)
    if N > 2:
        masks[2] = False
        masks[2, H - 1, W - 1] = True                                    # one pixel, the very last in column-major order
    want = _rle_check(masks)
    for r, m in zip(want[:2], masks[:2]):
        assert np.array_equal(ao.rle_to_mask(r), m.numpy())
    full = torch.ones(1, H, W, dtype=torch.bool)
    assert _rle_check(full)[0]["counts"] == [0, H * W]
    _rle_check(masks[:1], cap=3)                                         # far too small a first guess


def test_mask_rle_after_mask_stats_pipeline():
    """The generator's sequence: logits -> thresholded masks (mask_stats) -> run lengths; areas agree with the
    stability counts' threshold and the encoding equals the reference restatement's."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from segment_anything_fast_b200 import amg
    g = torch.Generator().manual_seed(77)
    logits = torch.nn.functional.interpolate(torch.randn(5, 1, 32, 40, generator=g), size=(512, 640), mode="bilinear")[:, 0]
    _, _, binary = amg.mask_stats(logits.cuda(), 0.0, 1.0)
    rles = amg.mask_to_rle_pytorch(binary)
    assert amg.mask_to_rle_pytorch(binary.cpu()[:1]) == rles[:1]          # host masks are uploaded, not encoded on the CPU
    assert rles == ao.mask_to_rle((logits > 0).numpy())
    for r, m in zip(rles, logits > 0):
        assert sum(r["counts"][1::2]) == int(m.sum())                    # area_from_rle, utils/amg.py:188-189
