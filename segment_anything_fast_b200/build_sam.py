"""Registries with the reference's names and signatures (build_sam.py:14-92).

``build_image_encoder_vit_{h,l,b}`` build only the B200 image encoder.  ``sam_model_registry`` /
``sam_model_fast_registry`` build a full ``Sam`` from this package's encoder and its torch prompt encoder /
mask decoder (``sam_heads.py``; reference checkpoints load unchanged).  ``install(sam)`` instead takes a
``Sam`` built by the reference package and puts the B200 encoder in its ``image_encoder`` slot with the same
weights: the substitution the reference's own fast registry performs when it reassigns ``sam.image_encoder``
(build_sam.py:70,78,84).  ``compile_mode`` is accepted and ignored: nothing here is traced or compiled.
"""
from functools import partial
from typing import Optional

import torch

from .image_encoder import ImageEncoderViT

_VIT = {
    "vit_h": dict(embed_dim=1280, depth=32, num_heads=16, global_attn_indexes=(7, 15, 23, 31)),   # build_sam.py:14-21
    "vit_l": dict(embed_dim=1024, depth=24, num_heads=16, global_attn_indexes=(5, 11, 17, 23)),   # :27-34
    "vit_b": dict(embed_dim=768, depth=12, num_heads=12, global_attn_indexes=(2, 5, 8, 11)),      # :37-44
}


def _build_image_encoder(name: str) -> ImageEncoderViT:
    cfg = _VIT[name]
    return ImageEncoderViT(                         # arguments of build_sam.py:107-120
        depth=cfg["depth"], embed_dim=cfg["embed_dim"], img_size=1024, mlp_ratio=4,
        norm_layer=partial(torch.nn.LayerNorm, eps=1e-6), num_heads=cfg["num_heads"], patch_size=16,
        qkv_bias=True, use_rel_pos=True, global_attn_indexes=cfg["global_attn_indexes"], window_size=14,
        out_chans=256).eval()


def build_image_encoder_vit_h() -> ImageEncoderViT:
    return _build_image_encoder("vit_h")


def build_image_encoder_vit_l() -> ImageEncoderViT:
    return _build_image_encoder("vit_l")


def build_image_encoder_vit_b() -> ImageEncoderViT:
    return _build_image_encoder("vit_b")


def install(sam, quant: Optional[str] = None):
    """Replace ``sam.image_encoder`` (a reference ``ImageEncoderViT``) by the B200 encoder carrying the
    same weights, dtype and device.  Returns ``sam``."""
    old = sam.image_encoder
    old = getattr(old, "_orig_mod", old)           # unwrap a torch.compile wrapper
    first = old.blocks[0]
    depth = len(old.blocks)
    new = ImageEncoderViT(
        depth=depth, embed_dim=first.norm1.normalized_shape[0], img_size=old.img_size, mlp_ratio=
        first.mlp.lin1.out_features / first.mlp.lin1.in_features, norm_layer=partial(torch.nn.LayerNorm, eps=first.norm1.eps),
        num_heads=first.attn.num_heads, patch_size=old.patch_embed.proj.kernel_size[0], qkv_bias=first.attn.qkv.bias is not None,
        use_rel_pos=first.attn.use_rel_pos, window_size=max(b.window_size for b in old.blocks),
        global_attn_indexes=tuple(i for i, b in enumerate(old.blocks) if b.window_size == 0),
        out_chans=old.neck[0].out_channels).eval()
    new.load_state_dict(old.state_dict())
    p = next(old.parameters())
    sam.image_encoder = new.to(device=p.device, dtype=p.dtype).set_quant(quant)
    return sam


def _build_sam(name: str, checkpoint=None):
    """Full ``Sam`` (this package's encoder, prompt encoder and mask decoder; build_sam.py:95-149).  ``checkpoint``
    is a path to a reference ``state_dict`` file."""
    from .sam_heads import Sam, build_heads
    prompt_encoder, mask_decoder = build_heads()
    sam = Sam(_build_image_encoder(name), prompt_encoder, mask_decoder).eval()
    if checkpoint is not None:
        with open(checkpoint, "rb") as f:
            sam.load_state_dict(torch.load(f, map_location="cpu"))
    return sam


def build_sam_vit_h(checkpoint=None):
    return _build_sam("vit_h", checkpoint)


def build_sam_vit_l(checkpoint=None):
    return _build_sam("vit_l", checkpoint)


def build_sam_vit_b(checkpoint=None):
    return _build_sam("vit_b", checkpoint)


build_sam = build_sam_vit_h
sam_model_registry = {"default": build_sam_vit_h, "vit_h": build_sam_vit_h, "vit_l": build_sam_vit_l,
                      "vit_b": build_sam_vit_b}


def _fast(name: str, checkpoint=None, compile_mode="max-autotune", dtype=torch.bfloat16, quant: Optional[str] = None):
    sam = _build_sam(name, checkpoint)
    for part in ("image_encoder", "prompt_encoder", "mask_decoder"):      # _apply_eval_dtype_sam, build_sam.py:54-65
        m = getattr(sam, part).eval()
        setattr(sam, part, m.to(dtype) if dtype is not None else m)
    sam.image_encoder.set_quant(quant)
    return sam


def build_sam_fast_vit_h(checkpoint=None, compile_mode="max-autotune", dtype=torch.bfloat16, quant=None):
    return _fast("vit_h", checkpoint, compile_mode, dtype, quant)


def build_sam_fast_vit_l(checkpoint=None, compile_mode="max-autotune", dtype=torch.bfloat16, quant=None):
    return _fast("vit_l", checkpoint, compile_mode, dtype, quant)


def build_sam_fast_vit_b(checkpoint=None, compile_mode="max-autotune", dtype=torch.bfloat16, quant=None):
    return _fast("vit_b", checkpoint, compile_mode, dtype, quant)


build_sam_fast = build_sam_fast_vit_h
sam_model_fast_registry = {"default": build_sam_fast_vit_h, "vit_h": build_sam_fast_vit_h,
                           "vit_l": build_sam_fast_vit_l, "vit_b": build_sam_fast_vit_b}
