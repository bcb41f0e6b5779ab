"""``SamPredictor`` with the reference's methods (segment_anything_fast/predictor.py:17-278) over a ``Sam`` whose
image encoder is the B200 encoder: ``set_image`` / ``set_torch_image`` run the encoder once, ``predict`` /
``predict_torch`` run the prompt encoder and mask decoder on the stored embedding.

``ResizeLongestSide`` (segment_anything_fast/utils/transforms.py:16-102) is the image / coordinate transform
the predictor applies: scale so that the long side equals the encoder's input size.

Host code only; the image goes to the encoder as the model's dtype (predictor.py:88-90) and everything
downstream of the embedding is torch.
"""
from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F


class ResizeLongestSide:
    def __init__(self, target_length: int) -> None:
        self.target_length = target_length

    @staticmethod
    def get_preprocess_shape(oldh: int, oldw: int, long_side_length: int) -> Tuple[int, int]:
        scale = long_side_length * 1.0 / max(oldh, oldw)
        return int(oldh * scale + 0.5), int(oldw * scale + 0.5)

    def apply_image(self, image: np.ndarray) -> np.ndarray:
        """``H x W x C`` uint8 -> resized uint8 (PIL bilinear, what torchvision's ``resize`` of a PIL image does)."""
        from PIL import Image
        h, w = self.get_preprocess_shape(image.shape[0], image.shape[1], self.target_length)
        return np.array(Image.fromarray(image).resize((w, h), Image.BILINEAR))

    def apply_coords(self, coords: np.ndarray, original_size: Tuple[int, ...]) -> np.ndarray:
        old_h, old_w = original_size
        new_h, new_w = self.get_preprocess_shape(old_h, old_w, self.target_length)
        out = np.array(coords, dtype=float, copy=True)
        out[..., 0] *= new_w / old_w
        out[..., 1] *= new_h / old_h
        return out

    def apply_boxes(self, boxes: np.ndarray, original_size: Tuple[int, ...]) -> np.ndarray:
        return self.apply_coords(np.asarray(boxes).reshape(-1, 2, 2), original_size).reshape(-1, 4)

    def apply_image_torch(self, image: torch.Tensor) -> torch.Tensor:
        """``[B, C, H, W]`` float -> resized (bilinear, antialiased)."""
        size = self.get_preprocess_shape(image.shape[2], image.shape[3], self.target_length)
        return F.interpolate(image, size, mode="bilinear", align_corners=False, antialias=True)

    def apply_coords_torch(self, coords: torch.Tensor, original_size: Tuple[int, ...]) -> torch.Tensor:
        old_h, old_w = original_size
        new_h, new_w = self.get_preprocess_shape(old_h, old_w, self.target_length)
        out = coords.clone().to(torch.float)
        out[..., 0] *= new_w / old_w
        out[..., 1] *= new_h / old_h
        return out

    def apply_boxes_torch(self, boxes: torch.Tensor, original_size: Tuple[int, ...]) -> torch.Tensor:
        return self.apply_coords_torch(boxes.reshape(-1, 2, 2), original_size).reshape(-1, 4)


class SamPredictor:
    def __init__(self, sam_model) -> None:
        self.model = sam_model
        self.transform = ResizeLongestSide(sam_model.image_encoder.img_size)
        self.reset_image()

    @property
    def device(self) -> torch.device:
        return self.model.device

    def reset_image(self) -> None:
        self.is_image_set = False
        self.features = None
        self.original_size = None
        self.input_size = None

    def set_image(self, image: np.ndarray, image_format: str = "RGB") -> None:
        """``H x W x 3`` uint8 image -> embedding (predictor.py:34-59)."""
        if image_format not in ("RGB", "BGR"):
            raise ValueError(f"image_format must be 'RGB' or 'BGR', is {image_format!r}")
        if image_format != self.model.image_format:
            image = image[..., ::-1]
        x = torch.as_tensor(np.ascontiguousarray(self.transform.apply_image(image)), device=self.device)
        self.set_torch_image(x.permute(2, 0, 1).contiguous()[None], image.shape[:2])

    @torch.no_grad()
    def set_torch_image(self, transformed_image: torch.Tensor, original_image_size: Tuple[int, ...]) -> None:
        """``[B, 3, H, W]`` pixels with long side ``img_size`` -> embeddings (predictor.py:61-91).  The reference
        takes one image here; with a batch, ``predict_torch(..., image_index=i)`` prompts image ``i``."""
        S = self.model.image_encoder.img_size
        if transformed_image.dim() != 4 or transformed_image.shape[1] != 3 or max(transformed_image.shape[2:]) != S:
            raise ValueError(f"set_torch_image input must be BCHW with long side {S}")
        self.reset_image()
        self.original_size = tuple(original_image_size)
        self.input_size = tuple(transformed_image.shape[-2:])
        x = self.model.preprocess(transformed_image)
        model_dtype = self.model.mask_decoder.iou_prediction_head.layers[0].weight.dtype
        self.features = self.model.image_encoder(x.to(model_dtype))
        self.is_image_set = True

    def predict(self, point_coords: Optional[np.ndarray] = None, point_labels: Optional[np.ndarray] = None,
                box: Optional[np.ndarray] = None, mask_input: Optional[np.ndarray] = None,
                multimask_output: bool = True, return_logits: bool = False):
        """numpy prompts in original-image pixels -> (masks ``C x H x W``, IoU predictions ``C``, low-resolution
        logits ``C x 256 x 256``) as numpy arrays (predictor.py:93-168)."""
        if not self.is_image_set:
            raise RuntimeError("An image must be set with .set_image(...) before mask prediction.")
        coords_t = labels_t = box_t = mask_t = None
        if point_coords is not None:
            if point_labels is None:
                raise ValueError("point_labels must be supplied if point_coords is supplied.")
            pc = self.transform.apply_coords(point_coords, self.original_size)
            coords_t = torch.as_tensor(pc, dtype=torch.float, device=self.device)[None]
            labels_t = torch.as_tensor(point_labels, dtype=torch.int, device=self.device)[None]
        if box is not None:
            b = self.transform.apply_boxes(box, self.original_size)
            box_t = torch.as_tensor(b, dtype=torch.float, device=self.device)[None].reshape(1, 4)
        if mask_input is not None:
            mask_t = torch.as_tensor(mask_input, dtype=torch.float, device=self.device)[None]
        masks, iou, low = self.predict_torch(coords_t, labels_t, box_t, mask_t, multimask_output, return_logits)
        return (masks[0].detach().cpu().numpy(), iou[0].detach().cpu().float().numpy(),
                low[0].detach().cpu().float().numpy())

    @torch.no_grad()
    def predict_torch(self, point_coords: Optional[torch.Tensor], point_labels: Optional[torch.Tensor],
                      boxes: Optional[torch.Tensor] = None, mask_input: Optional[torch.Tensor] = None,
                      multimask_output: bool = True, return_logits: bool = False,
                      image_index: Optional[int] = None):
        """Batched torch prompts in the input frame (predictor.py:170-252): masks ``B x C x H x W`` at the original
        size (boolean unless ``return_logits``), IoU predictions ``B x C``, low-resolution logits.
        ``image_index`` selects one embedding when ``set_torch_image`` was given a batch of images."""
        if not self.is_image_set:
            raise RuntimeError("An image must be set with .set_image(...) before mask prediction.")
        points = (point_coords, point_labels) if point_coords is not None else None
        sparse, dense = self.model.prompt_encoder(points, boxes, mask_input)
        feats = self.features if image_index is None else self.features[image_index:image_index + 1]
        low, iou = self.model.mask_decoder(feats, self.model.prompt_encoder.get_dense_pe(), sparse, dense,
                                           multimask_output)
        masks = self.model.postprocess_masks(low, self.input_size, self.original_size)
        if not return_logits:
            masks = masks > self.model.mask_threshold
        return masks, iou, low

    def get_image_embedding(self) -> torch.Tensor:
        if not self.is_image_set or self.features is None:
            raise RuntimeError("An image must be set with .set_image(...) to generate an embedding.")
        return self.features
