"""B200-native SAM image-encoder hot path behind the segment_anything_fast API.

Public names mirror segment_anything_fast/__init__.py:7-20 for the part this package implements.
"""
from .build_sam import (build_image_encoder_vit_b, build_image_encoder_vit_h, build_image_encoder_vit_l,  # noqa: F401
                        build_sam, build_sam_fast, build_sam_fast_vit_b, build_sam_fast_vit_h, build_sam_fast_vit_l,
                        build_sam_vit_b, build_sam_vit_h, build_sam_vit_l, install, sam_model_fast_registry,
                        sam_model_registry)
from . import flash_4  # noqa: F401  (registers the samb200::custom_flash_aligned dispatcher op)
from .image_encoder import ImageEncoderViT  # noqa: F401
from .predictor import ResizeLongestSide, SamPredictor  # noqa: F401
from .automatic_mask_generator import SamAutomaticMaskGenerator  # noqa: F401
from .runtime import EncoderSession  # noqa: F401
from .sparse import apply_fake_sparsity, apply_sparse  # noqa: F401
from .sam_heads import MaskDecoder, PromptEncoder, Sam, TwoWayTransformer  # noqa: F401
