"""The automatic mask generator's per-mask filters and run-length encoding on the GPU, under the reference's
function names (segment_anything_fast/utils/amg.py:106-170, 193-213, 340-383), so that
``automatic_mask_generator.py`` can import them from here instead.  ``mask_stats`` is the fused form: one pass over the logits gives the stability
score, the boxes and the thresholded masks that ``_process_batch`` computes with four passes
(automatic_mask_generator.py:335-345).
"""
from typing import Any, Dict, List, Optional, Tuple

import torch

from . import _lib
from .ops import _need, _stream


def mask_stats(logits: torch.Tensor, mask_threshold: float, threshold_offset: float,
               want_binary: bool = True) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """``logits [..., H, W]`` (fp32 / bf16, CUDA) -> stability score ``[...]`` (float32), XYXY boxes ``[..., 4]``
    (int32) of ``logits > mask_threshold``, and that boolean mask (or None)."""
    if logits.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("mask_stats: logits must be float32 or bfloat16")
    _need(logits, logits.dtype, "logits")
    lead, (H, W) = logits.shape[:-2], logits.shape[-2:]
    x = logits.reshape(-1, H, W).contiguous()
    N = x.shape[0]
    inter = torch.empty(N, dtype=torch.int32, device=x.device)
    uni = torch.empty(N, dtype=torch.int32, device=x.device)
    boxes = torch.empty(N, 4, dtype=torch.int32, device=x.device)
    binary = torch.empty(N, H, W, dtype=torch.uint8, device=x.device) if want_binary else None
    _lib.check(_lib.load().samb_mask_stats(
        x.data_ptr(), int(x.dtype == torch.bfloat16), N, H, W, float(mask_threshold), float(threshold_offset),
        inter.data_ptr(), uni.data_ptr(), boxes.data_ptr(), binary.data_ptr() if want_binary else None, _stream()),
        "samb_mask_stats")
    score = inter / uni                                   # int32 / int32 -> float32, as the reference divides
    return (score.reshape(lead), boxes.reshape(*lead, 4),
            binary.view(torch.bool).reshape(*lead, H, W) if want_binary else None)


def calculate_stability_score(masks: torch.Tensor, mask_threshold: float, threshold_offset: float) -> torch.Tensor:
    return mask_stats(masks, mask_threshold, threshold_offset, want_binary=False)[0]


def batched_mask_to_box(masks: torch.Tensor) -> torch.Tensor:
    """Boolean masks ``[..., H, W]`` -> XYXY boxes, zeros for empty masks."""
    if masks.numel() == 0:
        return torch.zeros(*masks.shape[:-2], 4, device=masks.device)
    return mask_stats(masks.to(torch.float32), 0.5, 0.0, want_binary=False)[1].to(torch.int64)


def mask_rle_counts(masks: torch.Tensor, cap: int = 4096) -> Tuple[torch.Tensor, torch.Tensor]:
    """Boolean masks ``[N, H, W]`` (CUDA) -> run lengths ``[N, cap']`` (int32, column-major pixel order, leading run
    of zeros) and the number of runs ``[N]`` of each mask; ``cap'`` grows to the longest encoding when ``cap`` is
    too small (one more launch).  Reads ``n_counts`` back, so it synchronises the stream."""
    _need(masks, torch.bool, "masks")
    if masks.dim() != 3:
        raise RuntimeError("mask_rle_counts: masks must be [N, H, W]")
    x = masks.contiguous().view(torch.uint8)
    N, H, W = x.shape
    n_counts = torch.empty(N, dtype=torch.int32, device=x.device)
    while True:
        counts = torch.empty(N, cap, dtype=torch.int32, device=x.device)
        _lib.check(_lib.load().samb_mask_rle(x.data_ptr(), N, H, W, counts.data_ptr(), n_counts.data_ptr(), cap, _stream()),
                   "samb_mask_rle")
        need = int(n_counts.max().item()) if N else 0
        if need <= cap:
            return counts[:, :max(need, 1)], n_counts
        cap = need


def mask_to_rle_pytorch(tensor: torch.Tensor) -> List[Dict[str, Any]]:
    """Masks ``[N, H, W]`` -> ``[{"size": [H, W], "counts": [...]}, ...]``, the uncompressed RLE pycocotools reads."""
    if tensor.shape[0] == 0:
        return []
    _, h, w = tensor.shape
    if not tensor.is_cuda:                                # the small-region post-processing hands over host masks
        tensor = tensor.cuda()
    counts, n = mask_rle_counts(tensor.to(torch.bool))
    rows, n = counts.cpu().tolist(), n.cpu().tolist()
    return [{"size": [h, w], "counts": r[:k]} for r, k in zip(rows, n)]


mask_to_rle_pytorch_2 = mask_to_rle_pytorch


def is_box_near_crop_edge(boxes: torch.Tensor, crop_box, orig_box, atol: float = 20.0) -> torch.Tensor:
    """True for boxes that touch an edge of the crop which is not an edge of the image (utils/amg.py:78-88)."""
    crop = torch.as_tensor(crop_box, dtype=torch.float, device=boxes.device)
    orig = torch.as_tensor(orig_box, dtype=torch.float, device=boxes.device)
    x0, y0 = float(crop_box[0]), float(crop_box[1])
    b = boxes.float() + torch.tensor([x0, y0, x0, y0], device=boxes.device)         # uncrop_boxes_xyxy
    near_crop = (b - crop[None]).abs() <= atol
    near_image = (b - orig[None]).abs() <= atol
    return (near_crop & ~near_image).any(dim=1)


def process_batch_filters(mask_logits: torch.Tensor, iou_preds: torch.Tensor, points: torch.Tensor, crop_box,
                          orig_size: Tuple[int, int], pred_iou_thresh: float = 0.88, mask_threshold: float = 0.0,
                          stability_score_offset: float = 1.0, stability_score_thresh: float = 0.95) -> Dict[str, Any]:
    """The filter stage the mask generator runs on one batch of point prompts
    (``_process_batch_2``, automatic_mask_generator.py:312-359) with one fused pass over the logits.

    ``mask_logits [P, C, H, W]`` (the decoder's masks upsampled to the crop, un-thresholded), ``iou_preds [P, C]``,
    ``points [P, 2]``.  Keeps the masks whose predicted IoU exceeds ``pred_iou_thresh``, whose stability score
    reaches ``stability_score_thresh`` and whose box does not touch a crop edge inside the image.  The reference
    filters after each step, so later steps see fewer masks; the order of the survivors is the same because every
    filter is a per-mask predicate.  Returns ``masks`` (boolean ``[K, H, W]``), ``iou_preds``, ``points``,
    ``stability_score``, ``boxes`` (int64 XYXY in crop coordinates) and ``keep`` (indices into the flattened
    ``P*C`` masks)."""
    P, C = mask_logits.shape[:2]
    orig_h, orig_w = orig_size
    flat = mask_logits.flatten(0, 1)
    iou = iou_preds.flatten(0, 1)
    pts = points.to(mask_logits.device).repeat_interleave(C, dim=0)
    keep = torch.ones(P * C, dtype=torch.bool, device=flat.device)
    if pred_iou_thresh > 0.0:
        keep &= iou > pred_iou_thresh
    score, boxes, binary = mask_stats(flat, mask_threshold, stability_score_offset)
    if stability_score_thresh > 0.0:
        keep &= score >= stability_score_thresh
    boxes = boxes.to(torch.int64)
    keep &= ~is_box_near_crop_edge(boxes, crop_box, [0, 0, orig_w, orig_h])
    idx = keep.nonzero().squeeze(1)
    return {"masks": binary[idx], "iou_preds": iou[idx], "points": pts[idx], "stability_score": score[idx],
            "boxes": boxes[idx], "keep": idx}
