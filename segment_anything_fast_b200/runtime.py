"""Host-facing session around the encoder: pinned staging buffers, one H2D copy of the uint8 image
batch, normalisation + encoder on the device, one D2H copy of the embeddings.

``encode`` is the blocking form; ``submit`` / ``result`` is the pipelined form (two slots, copies on their own
streams): the upload of batch i+1 and the download of batch i-1 overlap the encoder pass of batch i.
With ``graph=True`` the normalise + encoder launch sequence (about 230 kernels for ViT-H) is recorded once per
staging buffer as a CUDA graph and replayed, which takes the per-launch host cost out of small-batch latency.

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
                 pixel_mean: Sequence[float] = PIXEL_MEAN, pixel_std: Sequence[float] = PIXEL_STD,
                 graph: bool = False) -> None:
        self.encoder = encoder
        self.graph = graph
        self._graphs = {}          # device input buffer address -> (CUDAGraph, embeddings written by a replay, weights key)
        self._pool = None
        self.device = device or next(encoder.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("EncoderSession needs the encoder on a CUDA device")
        S, g, oc = encoder.img_size, encoder.img_size // encoder.patch_size, encoder.out_chans
        self.batch = batch
        self.mean, self.std = tuple(pixel_mean), tuple(pixel_std)
        self.host_in = torch.empty(batch, 3, S, S, dtype=torch.uint8).pin_memory()
        self.host_out = torch.empty(batch, oc, g, g, dtype=torch.bfloat16).pin_memory()
        self.dev_in = torch.empty(batch, 3, S, S, dtype=torch.uint8, device=self.device)
        self.dev_norm = None       # normalised bf16 copy of a batch: only for patch sizes the fused gather does not cover
        # host copy of the device status word, refreshed with every download: a bounded wait that ran out
        # inside a kernel must surface as an exception, not as silently wrong embeddings
        self._host_status = torch.zeros(1, dtype=torch.int32).pin_memory()
        # second slot and the copy streams of the pipelined form are created on first use
        self._slots = None
        self._next = 0

    @property
    def h2d_bytes(self) -> int:
        return self.host_in.numel()

    @property
    def d2h_bytes(self) -> int:
        return self.host_out.numel() * 2

    def encode_device(self, images_u8: torch.Tensor) -> torch.Tensor:
        """uint8 ``[B,3,S,S]`` on the device -> embeddings ``[B,out_chans,S/16,S/16]`` (bf16, device)."""
        if self.graph and images_u8.shape[0] == self.batch:
            return self._replay(images_u8)
        return self._run(images_u8)

    def _run(self, images_u8: torch.Tensor) -> torch.Tensor:
        """Normalisation + encoder.  With 16-pixel-aligned patches the normalisation rides on the patch-embedding
        gather (``forward_u8``); otherwise a normalised bf16 copy of the batch goes through ``forward``."""
        if self.encoder.patch_size % 16 == 0:
            return self.encoder.forward_u8(images_u8, self.mean, self.std)
        x = ops.normalize_u8(images_u8, self.mean, self.std, out=self._norm_buffer()[: images_u8.shape[0]])
        return self.encoder(x)

    def _norm_buffer(self) -> torch.Tensor:
        if self.dev_norm is None:
            S = self.host_in.shape[-1]
            self.dev_norm = torch.empty(self.batch, 3, S, S, dtype=torch.bfloat16, device=self.device)
        return self.dev_norm

    def _replay(self, dev_in: torch.Tensor) -> torch.Tensor:
        """Replay (recording it on first use) the graph that reads ``dev_in``; its output tensor is reused by
        every replay, so a caller that keeps embeddings across calls must copy them."""
        ent = self._graphs.get(dev_in.data_ptr())
        key = self.encoder._params_key()
        if ent is not None and ent[2] != key:
            # weights, dtype, quantisation or pruning changed since the recording: the graph still points at
            # the old packed buffers, so it is recorded again
            ent = None
        if ent is None:
            run = lambda: self._run(dev_in)
            main = torch.cuda.current_stream(self.device)
            side = torch.cuda.Stream(self.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):          # weight packing and allocator warm-up stay outside the recording
                run()
                run()
            main.wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self._pool):
                emb = run()
            self._pool = g.pool()                  # the graphs never run concurrently: one pool for their scratch
            ent = self._graphs[dev_in.data_ptr()] = (g, emb, key)
        ent[0].replay()
        return ent[1]

    def encode(self, images_u8_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Host uint8 batch (or what is already in ``self.host_in``) -> host bf16 embeddings.
        Blocking: returns when the embeddings are in ``self.host_out``."""
        if images_u8_host is not None:
            self.host_in.copy_(images_u8_host)
        self.dev_in.copy_(self.host_in, non_blocking=True)
        emb = self.encode_device(self.dev_in)
        self.host_out.copy_(emb, non_blocking=True)
        self._host_status.copy_(ops.status_word(self.device), non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        self._raise_on_status(self._host_status)
        return self.host_out

    def _raise_on_status(self, host_word: torch.Tensor) -> None:
        v = int(host_word.item())
        if v != 0:
            ops.status_word(self.device).zero_()
            raise RuntimeError(f"EncoderSession: a kernel reported device status 0x{v & 0xffffffff:08x} "
                               "(a bounded hardware-barrier wait ran out); the embeddings of this batch are not valid")

    # ------------------------------------------------------------------ pipelined form
    def _init_slots(self) -> None:
        S = self.host_in.shape[-1]
        mk = lambda: torch.cuda.Event()
        self._slots = []
        for i in range(2):
            self._slots.append({
                "host_in": self.host_in if i == 0 else torch.empty_like(self.host_in).pin_memory(),
                "host_out": self.host_out if i == 0 else torch.empty_like(self.host_out).pin_memory(),
                "dev_in": self.dev_in if i == 0 else torch.empty_like(self.dev_in),
                "host_status": torch.zeros(1, dtype=torch.int32).pin_memory(),
                "uploaded": mk(), "computed": mk(), "downloaded": mk(), "emb": None, "busy": False})
        self._s_in = torch.cuda.Stream(self.device)
        self._s_out = torch.cuda.Stream(self.device)

    def slot_input(self, slot: int) -> torch.Tensor:
        """Pinned uint8 staging buffer of a slot (fill it, then ``submit(slot=...)``)."""
        if self._slots is None:
            self._init_slots()
        return self._slots[slot]["host_in"]

    def submit(self, images_u8_host: Optional[torch.Tensor] = None, slot: Optional[int] = None) -> int:
        """Queue one batch: upload (copy stream) -> normalise + encoder (current stream) -> download (copy
        stream).  Returns the slot to pass to ``result``.  At most two batches are in flight; a slot must have
        been collected with ``result`` before it is submitted again."""
        if self._slots is None:
            self._init_slots()
        if slot is None:
            slot, self._next = self._next, self._next ^ 1
        sl = self._slots[slot]
        if sl["busy"]:
            raise RuntimeError("EncoderSession.submit: slot still in flight; call result(slot) first")
        if images_u8_host is not None:
            sl["host_in"].copy_(images_u8_host)
        main = torch.cuda.current_stream(self.device)
        self._s_in.wait_event(sl["computed"])             # the previous pass that read this slot's device input
        with torch.cuda.stream(self._s_in):
            sl["dev_in"].copy_(sl["host_in"], non_blocking=True)
            sl["uploaded"].record(self._s_in)
        main.wait_event(sl["uploaded"])
        if self.graph:
            main.wait_event(sl["downloaded"])             # a replay overwrites the embeddings of this slot's last pass
        emb = self.encode_device(sl["dev_in"])
        sl["computed"].record(main)
        self._s_out.wait_event(sl["computed"])
        with torch.cuda.stream(self._s_out):
            sl["host_out"].copy_(emb, non_blocking=True)
            sl["host_status"].copy_(ops.status_word(self.device), non_blocking=True)
            sl["downloaded"].record(self._s_out)
        if not self.graph:
            emb.record_stream(self._s_out)
        sl["emb"], sl["busy"] = emb, True
        return slot

    def result(self, slot: int) -> torch.Tensor:
        """Block until the batch submitted in ``slot`` is in host memory; returns the pinned bf16 embeddings."""
        sl = self._slots[slot]
        if not sl["busy"]:
            raise RuntimeError("EncoderSession.result: nothing was submitted in this slot")
        sl["downloaded"].synchronize()
        sl["emb"], sl["busy"] = None, False
        self._raise_on_status(sl["host_status"])
        return sl["host_out"]
