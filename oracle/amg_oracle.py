"""CPU restatement of the mask filters the automatic mask generator applies to predicted mask logits.

TEST INFRASTRUCTURE ONLY (checker for ``samb_mask_stats`` and ``samb_mask_rle``).  numpy, integer-exact.  Pinned by
``tests/golden/amg_fp32.npz``, outputs of the reference's own functions on seeded logits and masks.

Reference code followed (segment_anything_fast/utils/amg.py):
  calculate_stability_score :193-213 — IoU of the masks thresholded at ``thr + offset`` and ``thr - offset``
  (one contains the other, so the IoU is a ratio of two pixel counts);
  batched_mask_to_box :340-383 — XYXY bounds of a boolean mask, [0,0,0,0] when it is empty;
  mask_to_rle_pytorch :144-170 (and its batched twin :106-141) — run lengths of the mask read column by column,
  starting with a run of zeros; rle_to_mask :173-185 is the inverse.
"""
import numpy as np


def stability_counts(logits: np.ndarray, thr: float, offset: float):
    """``logits [N, H, W]`` -> pixel counts above ``thr + offset`` and above ``thr - offset`` (int32 each)."""
    hi = np.float32(thr) + np.float32(offset)
    lo = np.float32(thr) - np.float32(offset)
    x = logits.astype(np.float32)
    return (x > hi).reshape(x.shape[0], -1).sum(1).astype(np.int32), (x > lo).reshape(x.shape[0], -1).sum(1).astype(np.int32)


def calculate_stability_score(logits: np.ndarray, thr: float, offset: float) -> np.ndarray:
    inter, uni = stability_counts(logits, thr, offset)
    with np.errstate(divide="ignore", invalid="ignore"):
        return inter.astype(np.float32) / uni.astype(np.float32)


def batched_mask_to_box(masks: np.ndarray) -> np.ndarray:
    """Boolean ``[N, H, W]`` -> int ``[N, 4]`` (x0, y0, x1, y1), zeros for an empty mask."""
    out = np.zeros((masks.shape[0], 4), dtype=np.int64)
    for i, m in enumerate(masks):
        ys, xs = np.nonzero(m)
        if ys.size:
            out[i] = (xs.min(), ys.min(), xs.max(), ys.max())
    return out


def mask_to_rle(masks: np.ndarray):
    """Boolean ``[N, H, W]`` -> list of ``{"size": [H, W], "counts": [...]}``."""
    out = []
    n, h, w = masks.shape
    for m in masks:
        flat = np.ascontiguousarray(m.T).reshape(-1).astype(bool)           # column-major pixel order
        edges = np.flatnonzero(flat[1:] != flat[:-1]) + 1
        bounds = np.concatenate(([0], edges, [h * w]))
        counts = ([0] if flat[0] else []) + np.diff(bounds).tolist()
        out.append({"size": [h, w], "counts": counts})
    return out


def rle_to_mask(rle) -> np.ndarray:
    h, w = rle["size"]
    flat = np.zeros(h * w, dtype=bool)
    pos, val = 0, False
    for c in rle["counts"]:
        flat[pos:pos + c] = val
        pos += c
        val = not val
    return flat.reshape(w, h).T


def is_box_near_crop_edge(boxes: np.ndarray, crop_box, orig_box, atol: float = 20.0) -> np.ndarray:
    """utils/amg.py:78-88: a box edge within ``atol`` of a crop edge that is not also within ``atol`` of the
    image edge."""
    x0, y0 = crop_box[0], crop_box[1]
    b = boxes.astype(np.float32) + np.array([x0, y0, x0, y0], dtype=np.float32)
    near_crop = np.abs(b - np.asarray(crop_box, dtype=np.float32)[None]) <= atol
    near_image = np.abs(b - np.asarray(orig_box, dtype=np.float32)[None]) <= atol
    return np.any(near_crop & ~near_image, axis=1)


def process_batch_filters(mask_logits: np.ndarray, iou_preds: np.ndarray, crop_box, orig_size, pred_iou_thresh=0.88,
                          mask_threshold=0.0, stability_score_offset=1.0, stability_score_thresh=0.95):
    """``_process_batch_2`` (automatic_mask_generator.py:312-359) step by step, filtering after every step as the
    reference does: predicted IoU, stability score, threshold + boxes, crop-edge boxes.  ``mask_logits
    [P, C, H, W]``, ``iou_preds [P, C]`` -> (indices of the kept masks in the flattened ``P*C`` order, their
    stability scores, boxes, boolean masks)."""
    flat = mask_logits.reshape((-1,) + mask_logits.shape[2:]).astype(np.float32)
    iou = iou_preds.reshape(-1)
    idx = np.arange(flat.shape[0])
    if pred_iou_thresh > 0.0:
        idx = idx[iou[idx] > np.float32(pred_iou_thresh)]
    score = calculate_stability_score(flat[idx], mask_threshold, stability_score_offset)
    if stability_score_thresh > 0.0:
        sel = score >= np.float32(stability_score_thresh)
        idx, score = idx[sel], score[sel]
    masks = flat[idx] > np.float32(mask_threshold)
    boxes = batched_mask_to_box(masks)
    orig_h, orig_w = orig_size
    sel = ~is_box_near_crop_edge(boxes, crop_box, [0, 0, orig_w, orig_h]) if len(idx) else np.zeros(0, dtype=bool)
    return idx[sel], score[sel], boxes[sel], masks[sel]
