"""Host-facing session around the encoder: pinned staging buffers, one H2D copy of the uint8 image
batch, normalisation + encoder on the device, one D2H copy of the embeddings.

This is the call a data-parallel worker makes per batch (one process per GPU).  It replaces the
upload + ``Sam.preprocess`` + ``image_encoder`` sequence of ``SamPredictor.set_torch_image``
(predictor.py:57-58,88-90; sam.py:164-174) for a batch of already-resized 1024x1024 images.
"""
from typing import Optional, Sequence

import torch

from . import ops

PIXEL_MEAN = (123.675, 116.28, 103.53)   # build_sam.py:139
PIXEL_STD = (58.395, 57.12, 57.375)      # build_sam.py:140


class EncoderSession:
    def __init__(self, encoder, batch: int, device: Optional[torch.device] = None,
                 pixel_mean: Sequence[float] = PIXEL_MEAN, pixel_std: Sequence[float] = PIXEL_STD) -> None:
        self.encoder = encoder
        self.device = device or next(encoder.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("EncoderSession needs the encoder on a CUDA device")
        S, g, oc = encoder.img_size, encoder.img_size // encoder.patch_size, encoder.out_chans
        self.batch = batch
        self.mean, self.std = tuple(pixel_mean), tuple(pixel_std)
        self.host_in = torch.empty(batch, 3, S, S, dtype=torch.uint8).pin_memory()
        self.host_out = torch.empty(batch, oc, g, g, dtype=torch.bfloat16).pin_memory()
        self.dev_in = torch.empty(batch, 3, S, S, dtype=torch.uint8, device=self.device)
        self.dev_norm = torch.empty(batch, 3, S, S, dtype=torch.bfloat16, device=self.device)

    @property
    def h2d_bytes(self) -> int:
        return self.host_in.numel()

    @property
    def d2h_bytes(self) -> int:
        return self.host_out.numel() * 2

    def encode_device(self, images_u8: torch.Tensor) -> torch.Tensor:
        """uint8 ``[B,3,S,S]`` on the device -> embeddings ``[B,out_chans,S/16,S/16]`` (bf16, device)."""
        x = ops.normalize_u8(images_u8, self.mean, self.std, out=self.dev_norm[: images_u8.shape[0]])
        return self.encoder(x)

    def encode(self, images_u8_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Host uint8 batch (or what is already in ``self.host_in``) -> host bf16 embeddings.
        Blocking: returns when the embeddings are in ``self.host_out``."""
        if images_u8_host is not None:
            self.host_in.copy_(images_u8_host)
        self.dev_in.copy_(self.host_in, non_blocking=True)
        emb = self.encode_device(self.dev_in)
        self.host_out.copy_(emb, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self.host_out
