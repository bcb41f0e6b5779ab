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


# ---------------------------------------------------------------------------------------------------------------
# The generator around the filters (segment_anything_fast/automatic_mask_generator.py:204-274 and
# utils/amg.py:216-274).  The point grids and crop boxes are pinned by ``tests/golden/amg_fp32.npz``; the reference's
# generator itself cannot run without a GPU (it pins a jagged tensor, automatic_mask_generator.py:292), so
# ``generate`` is a restatement composed of pinned parts.
# ---------------------------------------------------------------------------------------------------------------
def build_point_grid(n_per_side: int) -> np.ndarray:
    """utils/amg.py:216-224: cell centres of an n x n grid over the unit square, x fastest."""
    offset = 1 / (2 * n_per_side)
    side = np.linspace(offset, 1 - offset, n_per_side)
    pts = np.empty((n_per_side, n_per_side, 2), dtype=np.float64)
    pts[..., 0] = side[None, :]
    pts[..., 1] = side[:, None]
    return pts.reshape(-1, 2)


def generate_crop_boxes(im_size, n_layers: int, overlap_ratio: float):
    """utils/amg.py:238-274: XYXY boxes, layer 0 = the image, layer i = (2**i)**2 overlapping crops."""
    import math
    im_h, im_w = im_size
    boxes, layers = [[0, 0, im_w, im_h]], [0]
    for i in range(n_layers):
        n = 2 ** (i + 1)
        overlap = int(overlap_ratio * min(im_h, im_w) * (2 / n))
        cw = int(math.ceil((overlap * (n - 1) + im_w) / n))
        ch = int(math.ceil((overlap * (n - 1) + im_h) / n))
        for ix in range(n):
            for iy in range(n):
                x0, y0 = int((cw - overlap) * ix), int((ch - overlap) * iy)
                boxes.append([x0, y0, min(x0 + cw, im_w), min(y0 + ch, im_h)])
                layers.append(i + 1)
    return boxes, layers


def nms(boxes: np.ndarray, scores: np.ndarray, thr: float) -> np.ndarray:
    """Greedy box NMS as ``torchvision.ops.nms`` defines it: visit boxes by decreasing score, drop a box whose IoU
    with a kept box exceeds ``thr``; returns the kept indices in that order."""
    b = boxes.astype(np.float64)
    area = (b[:, 2] - b[:, 0]) * (b[:, 3] - b[:, 1])
    order = np.argsort(-scores, kind="stable")
    kept = []
    for i in order:
        ok = True
        for j in kept:
            iw = max(0.0, min(b[i, 2], b[j, 2]) - max(b[i, 0], b[j, 0]))
            ih = max(0.0, min(b[i, 3], b[j, 3]) - max(b[i, 1], b[j, 1]))
            inter = iw * ih
            union = area[i] + area[j] - inter
            if union > 0 and inter / union > thr:
                ok = False
                break
        if ok:
            kept.append(int(i))
    return np.asarray(kept, dtype=np.int64)


def generate(image: np.ndarray, predict_fn, points_per_side=32, points_per_batch=64, pred_iou_thresh=0.88,
             stability_score_thresh=0.95, stability_score_offset=1.0, box_nms_thresh=0.7, crop_n_layers=0,
             crop_nms_thresh=0.7, crop_overlap_ratio=512 / 1500, crop_n_points_downscale_factor=1, mask_threshold=0.0):
    """``SamAutomaticMaskGenerator.generate`` with ``output_mode="uncompressed_rle"`` and no small-region pass.
    ``predict_fn(crop_image, points)`` stands for ``set_image`` + ``predict_torch(multimask_output=True,
    return_logits=True)``: crop ``h x w x 3`` uint8 and ``[P, 2]`` points in crop pixels -> (logits ``[P, 3, h, w]``,
    predicted IoUs ``[P, 3]``) as numpy arrays."""
    orig_h, orig_w = image.shape[:2]
    grids = [build_point_grid(int(points_per_side / (crop_n_points_downscale_factor ** i))) for i in range(crop_n_layers + 1)]
    crop_boxes, layers = generate_crop_boxes((orig_h, orig_w), crop_n_layers, crop_overlap_ratio)
    recs = []
    for crop_box, layer in zip(crop_boxes, layers):
        x0, y0, x1, y1 = crop_box
        crop = image[y0:y1, x0:x1]
        ch, cw = crop.shape[:2]
        points = grids[layer] * np.array([cw, ch], dtype=np.float64)[None]
        rows = []
        for s in range(0, len(points), points_per_batch):
            pts = points[s:s + points_per_batch]
            logits, iou = predict_fn(crop, pts)
            idx, score, boxes, masks = process_batch_filters(logits, iou, crop_box, (orig_h, orig_w), pred_iou_thresh,
                                                             mask_threshold, stability_score_offset, stability_score_thresh)
            flat_iou = iou.reshape(-1)
            for k, i in enumerate(idx):
                rows.append({"mask": masks[k], "iou": float(flat_iou[i]), "point": pts[i // logits.shape[1]],
                             "score": float(score[k]), "box": boxes[k]})
        if rows:
            keep = nms(np.stack([r["box"] for r in rows]), np.array([r["iou"] for r in rows], dtype=np.float32), box_nms_thresh)
            rows = [rows[i] for i in keep]
        for r in rows:
            full = np.zeros((orig_h, orig_w), dtype=bool)
            full[y0:y1, x0:x1] = r["mask"]
            recs.append({"rle": mask_to_rle(full[None])[0], "predicted_iou": r["iou"], "stability_score": r["score"],
                         "box": r["box"] + np.array([x0, y0, x0, y0]), "point": r["point"] + np.array([x0, y0]),
                         "crop_box": list(crop_box)})
    if len(crop_boxes) > 1 and recs:
        cb = np.array([r["crop_box"] for r in recs], dtype=np.float64)
        keep = nms(np.stack([r["box"] for r in recs]), (1.0 / ((cb[:, 2] - cb[:, 0]) * (cb[:, 3] - cb[:, 1]))).astype(np.float32),
                   crop_nms_thresh)
        recs = [recs[i] for i in keep]
    out = []
    for r in recs:
        b, c = r["box"], r["crop_box"]
        out.append({"segmentation": r["rle"], "area": int(sum(r["rle"]["counts"][1::2])),
                    "bbox": [int(b[0]), int(b[1]), int(b[2] - b[0]), int(b[3] - b[1])],
                    "predicted_iou": r["predicted_iou"], "point_coords": [[float(r["point"][0]), float(r["point"][1])]],
                    "stability_score": r["stability_score"], "crop_box": [c[0], c[1], c[2] - c[0], c[3] - c[1]]})
    return out
