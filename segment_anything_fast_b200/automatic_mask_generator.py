"""``SamAutomaticMaskGenerator`` under the reference's name and arguments
(segment_anything_fast/automatic_mask_generator.py:36-410): a grid of point prompts over the image (and over
crops of it), the decoder's three masks per point, the quality filters, box NMS inside a crop and between crops,
and one record per surviving mask.

What differs from the reference is where the per-mask work runs.  The filter stage of a batch of prompts is
``amg.process_batch_filters`` (stability score, threshold, mask -> box in one fused pass over the logits,
``samb_mask_stats``) and the run-length encoding is ``samb_mask_rle``; both are CUDA kernels, so the model has to
sit on a CUDA device.  Prompts go to the decoder as one dense ``[P, 1, 2]`` tensor per batch: every prompt of
the generator is a single point, so the reference's jagged NestedTensor (``_process_batch`` :276-310) has nothing
ragged to carry.  Removing small regions (``min_mask_region_area > 0``) needs OpenCV, as in the reference, and
``coco_rle`` output needs pycocotools.
"""
import math
from itertools import product
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from . import amg
from .predictor import SamPredictor


# ----------------------------------------------------------------------------------------------- geometry helpers
def build_point_grid(n_per_side: int) -> np.ndarray:
    """``n x n`` points at the cell centres of the unit square, x fastest (utils/amg.py:216-224)."""
    offset = 1 / (2 * n_per_side)
    centres = np.linspace(offset, 1 - offset, n_per_side)
    xs, ys = np.meshgrid(centres, centres)               # xs varies along a row
    return np.stack([xs, ys], axis=-1).reshape(-1, 2)


def build_all_layer_point_grids(n_per_side: int, n_layers: int, scale_per_layer: int) -> List[np.ndarray]:
    """One grid per crop layer, ``n_per_side / scale_per_layer**layer`` points a side (utils/amg.py:227-235)."""
    return [build_point_grid(int(n_per_side / (scale_per_layer ** layer))) for layer in range(n_layers + 1)]


def generate_crop_boxes(im_size: Tuple[int, ...], n_layers: int, overlap_ratio: float) -> Tuple[List[List[int]], List[int]]:
    """XYXY crop boxes and the layer of each: the whole image, then ``(2**i)**2`` overlapping crops for layer ``i``
    (utils/amg.py:238-274; the x offsets are the outer loop)."""
    im_h, im_w = im_size
    boxes, layers = [[0, 0, im_w, im_h]], [0]
    for layer in range(1, n_layers + 1):
        n = 2 ** layer
        overlap = int(overlap_ratio * min(im_h, im_w) * (2 / n))
        crop_w = int(math.ceil((overlap * (n - 1) + im_w) / n))
        crop_h = int(math.ceil((overlap * (n - 1) + im_h) / n))
        xs = [int((crop_w - overlap) * i) for i in range(n)]
        ys = [int((crop_h - overlap) * i) for i in range(n)]
        for x0, y0 in product(xs, ys):
            boxes.append([x0, y0, min(x0 + crop_w, im_w), min(y0 + crop_h, im_h)])
            layers.append(layer)
    return boxes, layers


def rle_to_mask(rle: Dict[str, Any]) -> np.ndarray:
    """Uncompressed RLE (column-major runs, zeros first) -> boolean ``H x W`` (utils/amg.py:173-185)."""
    h, w = rle["size"]
    counts = np.asarray(rle["counts"], dtype=np.int64)
    values = (np.arange(counts.size) & 1).astype(bool)
    return np.repeat(values, counts).reshape(w, h).T


def area_from_rle(rle: Dict[str, Any]) -> int:
    return int(sum(rle["counts"][1::2]))


def box_xyxy_to_xywh(box: torch.Tensor) -> torch.Tensor:
    out = box.clone()
    out[..., 2] = out[..., 2] - out[..., 0]
    out[..., 3] = out[..., 3] - out[..., 1]
    return out


def coco_encode_rle(uncompressed_rle: Dict[str, Any]) -> Dict[str, Any]:
    from pycocotools import mask as mask_utils
    h, w = uncompressed_rle["size"]
    rle = mask_utils.frPyObjects(uncompressed_rle, h, w)
    rle["counts"] = rle["counts"].decode("utf-8")
    return rle


def remove_small_regions(mask: np.ndarray, area_thresh: float, mode: str) -> Tuple[np.ndarray, bool]:
    """Drops holes or islands smaller than ``area_thresh`` pixels; says whether the mask changed
    (utils/amg.py:293-318)."""
    import cv2
    if mode not in ("holes", "islands"):
        raise ValueError("mode must be 'holes' or 'islands'")
    holes = mode == "holes"
    work = (holes ^ mask).astype(np.uint8)
    n, regions, stats, _ = cv2.connectedComponentsWithStats(work, 8)
    sizes = stats[:, -1][1:]
    small = [i + 1 for i, s in enumerate(sizes) if s < area_thresh]
    if not small:
        return mask, False
    fill = [0] + small
    if not holes:
        fill = [i for i in range(n) if i not in fill]
        if not fill:                                     # every island is small: keep the largest
            fill = [int(np.argmax(sizes)) + 1]
    return np.isin(regions, fill), True


def _nms(boxes: torch.Tensor, scores: torch.Tensor, iou_threshold: float) -> torch.Tensor:
    """Single-category ``torchvision.ops.batched_nms``, which the reference calls with all-zero categories."""
    from torchvision.ops import nms
    if boxes.numel() == 0:
        return torch.empty(0, dtype=torch.int64, device=boxes.device)
    return nms(boxes.float(), scores.float(), iou_threshold)


# ----------------------------------------------------------------------------------------------- the generator
class SamAutomaticMaskGenerator:
    def __init__(self, model, points_per_side: Optional[int] = 32, points_per_batch: int = 64,
                 pred_iou_thresh: float = 0.88, stability_score_thresh: float = 0.95,
                 stability_score_offset: float = 1.0, box_nms_thresh: float = 0.7, crop_n_layers: int = 0,
                 crop_nms_thresh: float = 0.7, crop_overlap_ratio: float = 512 / 1500,
                 crop_n_points_downscale_factor: int = 1, point_grids: Optional[List[np.ndarray]] = None,
                 min_mask_region_area: int = 0, output_mode: str = "binary_mask",
                 process_batch_size: Optional[int] = None) -> None:
        """Arguments as in the reference (automatic_mask_generator.py:37-142).  ``process_batch_size`` is accepted
        and has no effect: it sizes the reference's jagged decoder batches, which do not exist here."""
        if (points_per_side is None) == (point_grids is None):
            raise ValueError("Exactly one of points_per_side or point_grids must be provided.")
        if output_mode not in ("binary_mask", "uncompressed_rle", "coco_rle"):
            raise ValueError(f"Unknown output_mode {output_mode}.")
        if output_mode == "coco_rle":
            from pycocotools import mask as _mask_utils  # noqa: F401
        if min_mask_region_area > 0:
            import cv2  # noqa: F401
        self.point_grids = (build_all_layer_point_grids(points_per_side, crop_n_layers, crop_n_points_downscale_factor)
                            if points_per_side is not None else point_grids)
        self.predictor = SamPredictor(model)
        self.points_per_batch = points_per_batch
        self.pred_iou_thresh = pred_iou_thresh
        self.stability_score_thresh = stability_score_thresh
        self.stability_score_offset = stability_score_offset
        self.box_nms_thresh = box_nms_thresh
        self.crop_n_layers = crop_n_layers
        self.crop_nms_thresh = crop_nms_thresh
        self.crop_overlap_ratio = crop_overlap_ratio
        self.crop_n_points_downscale_factor = crop_n_points_downscale_factor
        self.min_mask_region_area = min_mask_region_area
        self.output_mode = output_mode
        self.process_batch_size = process_batch_size

    # -- one batch of point prompts on the image the predictor holds
    def _process_batch(self, points: np.ndarray, im_size: Tuple[int, ...], crop_box: List[int],
                       orig_size: Tuple[int, ...]) -> Dict[str, Any]:
        dev = self.predictor.device
        in_points = torch.as_tensor(self.predictor.transform.apply_coords(points, im_size), dtype=torch.float, device=dev)
        labels = torch.ones(in_points.shape[0], 1, dtype=torch.int, device=dev)
        logits, iou_preds, _ = self.predictor.predict_torch(in_points[:, None, :], labels, multimask_output=True,
                                                            return_logits=True)
        kept = amg.process_batch_filters(
            logits.float(), iou_preds.float(), torch.as_tensor(points, device=dev), crop_box, orig_size,
            pred_iou_thresh=self.pred_iou_thresh, mask_threshold=self.predictor.model.mask_threshold,
            stability_score_offset=self.stability_score_offset, stability_score_thresh=self.stability_score_thresh)
        kept.pop("keep")
        return kept

    def _process_crop(self, image: np.ndarray, crop_box: List[int], layer: int, orig_size: Tuple[int, ...]) -> Dict[str, Any]:
        x0, y0, x1, y1 = crop_box
        crop = image[y0:y1, x0:x1, :]
        crop_size = crop.shape[:2]
        self.predictor.set_image(crop)
        points = self.point_grids[layer] * np.array(crop_size)[None, ::-1]
        parts = [self._process_batch(points[i:i + self.points_per_batch], crop_size, crop_box, orig_size)
                 for i in range(0, len(points), self.points_per_batch)]
        self.predictor.reset_image()
        data = {k: torch.cat([p[k] for p in parts], dim=0) for k in parts[0]}
        # duplicates inside the crop, best predicted IoU first
        keep = _nms(data["boxes"], data["iou_preds"], self.box_nms_thresh)
        data = {k: v[keep] for k, v in data.items()}
        # back to the frame of the whole image; the masks are encoded at full size
        orig_h, orig_w = orig_size
        masks = torch.nn.functional.pad(data.pop("masks"), (x0, orig_w - x1, y0, orig_h - y1), value=False)
        data["rles"] = amg.mask_to_rle_pytorch(masks)
        data["boxes"] = data["boxes"] + torch.tensor([x0, y0, x0, y0], device=data["boxes"].device)
        data["points"] = data["points"] + torch.tensor([x0, y0], device=data["points"].device)
        data["crop_boxes"] = torch.tensor([crop_box] * len(data["rles"]), dtype=torch.int64).reshape(-1, 4)
        return data

    @staticmethod
    def _filter(data: Dict[str, Any], keep: torch.Tensor) -> Dict[str, Any]:
        idx = keep.cpu().tolist()
        return {k: ([v[i] for i in idx] if isinstance(v, list) else v[keep.to(v.device)]) for k, v in data.items()}

    def _generate_masks(self, image: np.ndarray) -> Dict[str, Any]:
        orig_size = image.shape[:2]
        crop_boxes, layers = generate_crop_boxes(orig_size, self.crop_n_layers, self.crop_overlap_ratio)
        crops = [self._process_crop(image, box, layer, orig_size) for box, layer in zip(crop_boxes, layers)]
        data = {k: (sum((c[k] for c in crops), []) if isinstance(crops[0][k], list)
                    else torch.cat([c[k] for c in crops], dim=0)) for k in crops[0]}
        if len(crop_boxes) > 1:                          # duplicates between crops: the smaller crop wins
            cb = data["crop_boxes"].float()
            scores = 1.0 / ((cb[:, 2] - cb[:, 0]) * (cb[:, 3] - cb[:, 1]))
            keep = _nms(data["boxes"], scores.to(data["boxes"].device), self.crop_nms_thresh)
            data = self._filter(data, keep)
        return {k: (v if isinstance(v, list) else v.cpu()) for k, v in data.items()}

    def postprocess_small_regions(self, data: Dict[str, Any], min_area: int, nms_thresh: float) -> Dict[str, Any]:
        """Holes and islands below ``min_area`` pixels go; boxes are recomputed and NMS runs again with the untouched
        masks preferred (automatic_mask_generator.py:361-410)."""
        if not data["rles"]:
            return data
        new_masks, scores = [], []
        for rle in data["rles"]:
            mask = rle_to_mask(rle)
            mask, changed_h = remove_small_regions(mask, min_area, "holes")
            mask, changed_i = remove_small_regions(mask, min_area, "islands")
            new_masks.append(torch.as_tensor(mask)[None])
            scores.append(float(not (changed_h or changed_i)))
        masks = torch.cat(new_masks, dim=0).to(self.predictor.device)
        boxes = amg.batched_mask_to_box(masks).cpu()
        keep = _nms(boxes, torch.as_tensor(scores), nms_thresh)
        for i in keep.tolist():
            if scores[i] == 0.0:
                data["rles"][i] = amg.mask_to_rle_pytorch(masks[i][None])[0]
                data["boxes"][i] = boxes[i]
        return self._filter(data, keep)

    @torch.no_grad()
    def generate(self, image: np.ndarray) -> List[Dict[str, Any]]:
        """``H x W x 3`` uint8 image -> one dict per mask with the reference's keys: ``segmentation``, ``area``,
        ``bbox`` (XYWH), ``predicted_iou``, ``point_coords``, ``stability_score``, ``crop_box`` (XYWH)
        (automatic_mask_generator.py:144-202)."""
        data = self._generate_masks(image)
        if self.min_mask_region_area > 0:
            data = self.postprocess_small_regions(data, self.min_mask_region_area,
                                                  max(self.box_nms_thresh, self.crop_nms_thresh))
        if self.output_mode == "coco_rle":
            segmentations = [coco_encode_rle(r) for r in data["rles"]]
        elif self.output_mode == "binary_mask":
            segmentations = [rle_to_mask(r) for r in data["rles"]]
        else:
            segmentations = data["rles"]
        return [{
            "segmentation": segmentations[i],
            "area": area_from_rle(data["rles"][i]),
            "bbox": box_xyxy_to_xywh(data["boxes"][i]).tolist(),
            "predicted_iou": data["iou_preds"][i].item(),
            "point_coords": [data["points"][i].tolist()],
            "stability_score": data["stability_score"][i].item(),
            "crop_box": box_xyxy_to_xywh(data["crop_boxes"][i]).tolist(),
        } for i in range(len(segmentations))]
