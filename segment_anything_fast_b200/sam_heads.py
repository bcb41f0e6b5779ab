"""What sits downstream of the image encoder, as plain torch modules on the model's device: prompt
encoder (points / boxes), two-way transformer mask decoder, mask post-processing, and a ``Sam``
container holding them next to the B200 image encoder.

Parameter names and shapes are the reference's (segment_anything_fast/modeling/prompt_encoder.py,
mask_decoder.py, transformer.py, sam.py), so a reference checkpoint loads with ``load_state_dict``.
The modules are thin: the arithmetic is a handful of small matmuls per prompt, run by torch's own GPU
operators; none of it is on the encoder's hot path.
"""
import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class _Norm2d(nn.Module):
    """Channel LayerNorm over NCHW (modeling/common.py:31-43), eps 1e-6."""

    def __init__(self, c: int):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(c))
        self.bias = nn.Parameter(torch.zeros(c))

    def forward(self, x):
        u = x.mean(1, keepdim=True)
        s = (x - u).pow(2).mean(1, keepdim=True)
        return self.weight[:, None, None] * ((x - u) / torch.sqrt(s + 1e-6)) + self.bias[:, None, None]


class PositionEmbeddingRandom(nn.Module):
    """Random-Fourier positional encoding (prompt_encoder.py:183-212)."""

    def __init__(self, num_pos_feats: int = 64):
        super().__init__()
        self.register_buffer("positional_encoding_gaussian_matrix", torch.randn(2, num_pos_feats))

    def encode(self, coords01: torch.Tensor) -> torch.Tensor:
        g = self.positional_encoding_gaussian_matrix
        c = (2.0 * coords01.to(g.dtype) - 1.0) @ g
        c = 2.0 * math.pi * c
        return torch.cat([torch.sin(c), torch.cos(c)], dim=-1)

    def forward(self, size: Tuple[int, int]) -> torch.Tensor:
        h, w = size
        g = self.positional_encoding_gaussian_matrix
        ys = (torch.arange(h, device=g.device, dtype=g.dtype) + 0.5) / h
        xs = (torch.arange(w, device=g.device, dtype=g.dtype) + 0.5) / w
        grid = torch.stack([xs[None, :].expand(h, w), ys[:, None].expand(h, w)], dim=-1)
        return self.encode(grid).permute(2, 0, 1)


class PromptEncoder(nn.Module):
    def __init__(self, embed_dim: int = 256, image_embedding_size: Tuple[int, int] = (64, 64),
                 input_image_size: Tuple[int, int] = (1024, 1024), mask_in_chans: int = 16):
        super().__init__()
        self.embed_dim = embed_dim
        self.image_embedding_size = image_embedding_size
        self.input_image_size = input_image_size
        self.pe_layer = PositionEmbeddingRandom(embed_dim // 2)
        self.point_embeddings = nn.ModuleList([nn.Embedding(1, embed_dim) for _ in range(4)])
        self.not_a_point_embed = nn.Embedding(1, embed_dim)
        self.no_mask_embed = nn.Embedding(1, embed_dim)
        # the mask-prompt branch (prompt_encoder.py:50-58, 111-114)
        self.mask_downscaling = nn.Sequential(
            nn.Conv2d(1, mask_in_chans // 4, kernel_size=2, stride=2), _Norm2d(mask_in_chans // 4), nn.GELU(),
            nn.Conv2d(mask_in_chans // 4, mask_in_chans, kernel_size=2, stride=2), _Norm2d(mask_in_chans), nn.GELU(),
            nn.Conv2d(mask_in_chans, embed_dim, kernel_size=1))

    def get_dense_pe(self) -> torch.Tensor:
        return self.pe_layer(self.image_embedding_size).unsqueeze(0)

    def forward(self, points: Optional[Tuple[torch.Tensor, torch.Tensor]], boxes: Optional[torch.Tensor],
                masks: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        S = float(self.input_image_size[1])
        w = [e.weight for e in self.point_embeddings]
        sparse = None
        if points is not None:
            coords, labels = points
            coords = coords.to(torch.float32) + 0.5
            labels = labels.to(torch.float32)
            if boxes is None:                                    # pad with a "not a point" entry
                coords = torch.cat([coords, coords.new_zeros(coords.shape[0], 1, 2)], dim=1)
                labels = torch.cat([labels, -labels.new_ones(labels.shape[0], 1)], dim=1)
            e = self.pe_layer.encode(coords / S)
            lab = labels.unsqueeze(-1)
            e = torch.where(lab == -1, self.not_a_point_embed.weight.expand_as(e), e)
            e = torch.where(lab == 0, e + w[0], e)
            e = torch.where(lab == 1, e + w[1], e)
            sparse = e
        if boxes is not None:
            c = (boxes.to(torch.float32) + 0.5).reshape(-1, 2, 2)
            e = self.pe_layer.encode(c / S)
            sparse = torch.stack([e[:, 0] + w[2], e[:, 1] + w[3]], dim=1)
        if sparse is None:
            if masks is None:
                raise ValueError("at least one of points / boxes / masks is required")
            sparse = w[0].new_zeros(masks.shape[0], 0, self.embed_dim)       # a mask prompt alone: no sparse tokens
        if masks is not None:                                                # _embed_masks, prompt_encoder.py:111-114
            dense = self.mask_downscaling(masks.to(w[0].dtype))
        else:
            h, wd = self.image_embedding_size
            dense = self.no_mask_embed.weight.reshape(1, -1, 1, 1).expand(sparse.shape[0], -1, h, wd)
        return sparse.to(dense.dtype), dense


class _Attention(nn.Module):
    """q / k / v projections to ``embedding_dim // downsample_rate``, softmax attention, output projection
    (transformer.py:185-233)."""

    def __init__(self, dim: int, heads: int, downsample_rate: int = 1):
        super().__init__()
        self.num_heads = heads
        inner = dim // downsample_rate
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(dim, inner), nn.Linear(dim, inner), nn.Linear(dim, inner)
        self.out_proj = nn.Linear(inner, dim)

    def forward(self, q, k, v):
        def split(t):
            b, n, c = t.shape
            return t.reshape(b, n, self.num_heads, c // self.num_heads).transpose(1, 2)

        o = F.scaled_dot_product_attention(split(self.q_proj(q)), split(self.k_proj(k)), split(self.v_proj(v)))
        o = o.transpose(1, 2)
        return self.out_proj(o.reshape(o.shape[0], o.shape[1], -1))


class _Mlp(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.lin1, self.lin2 = nn.Linear(dim, hidden), nn.Linear(hidden, dim)

    def forward(self, x):
        return self.lin2(F.relu(self.lin1(x)))


class _TwoWayBlock(nn.Module):
    """transformer.py:99-164."""

    def __init__(self, dim: int, heads: int, mlp_dim: int, rate: int, skip_first_layer_pe: bool):
        super().__init__()
        self.self_attn = _Attention(dim, heads)
        self.norm1 = nn.LayerNorm(dim)
        self.cross_attn_token_to_image = _Attention(dim, heads, rate)
        self.norm2 = nn.LayerNorm(dim)
        self.mlp = _Mlp(dim, mlp_dim)
        self.norm3 = nn.LayerNorm(dim)
        self.norm4 = nn.LayerNorm(dim)
        self.cross_attn_image_to_token = _Attention(dim, heads, rate)
        self.skip_first_layer_pe = skip_first_layer_pe

    def forward(self, queries, keys, query_pe, key_pe):
        if self.skip_first_layer_pe:
            queries = self.self_attn(queries, queries, queries)
        else:
            q = queries + query_pe
            queries = queries + self.self_attn(q, q, queries)
        queries = self.norm1(queries)
        queries = self.norm2(queries + self.cross_attn_token_to_image(queries + query_pe, keys + key_pe, keys))
        queries = self.norm3(queries + self.mlp(queries))
        keys = self.norm4(keys + self.cross_attn_image_to_token(keys + key_pe, queries + query_pe, queries))
        return queries, keys


class TwoWayTransformer(nn.Module):
    def __init__(self, depth: int = 2, embedding_dim: int = 256, num_heads: int = 8, mlp_dim: int = 2048,
                 attention_downsample_rate: int = 2):
        super().__init__()
        self.layers = nn.ModuleList([
            _TwoWayBlock(embedding_dim, num_heads, mlp_dim, attention_downsample_rate, skip_first_layer_pe=(i == 0))
            for i in range(depth)])
        self.final_attn_token_to_image = _Attention(embedding_dim, num_heads, attention_downsample_rate)
        self.norm_final_attn = nn.LayerNorm(embedding_dim)

    def forward(self, image_embedding, image_pe, point_embedding):
        keys = image_embedding.flatten(2).transpose(1, 2)
        key_pe = image_pe.flatten(2).transpose(1, 2)
        queries = point_embedding
        for layer in self.layers:
            queries, keys = layer(queries, keys, point_embedding, key_pe)
        attn = self.final_attn_token_to_image(queries + point_embedding, keys + key_pe, keys)
        return self.norm_final_attn(queries + attn), keys


class _HeadMlp(nn.Module):
    """ReLU MLP with ``layers`` (mask_decoder.py:216-232)."""

    def __init__(self, dims):
        super().__init__()
        self.layers = nn.ModuleList(nn.Linear(a, b) for a, b in zip(dims[:-1], dims[1:]))

    def forward(self, x):
        for i, l in enumerate(self.layers):
            x = l(x) if i == len(self.layers) - 1 else F.relu(l(x))
        return x


class MaskDecoder(nn.Module):
    def __init__(self, transformer_dim: int = 256, transformer: Optional[nn.Module] = None,
                 num_multimask_outputs: int = 3, iou_head_depth: int = 3, iou_head_hidden_dim: int = 256):
        super().__init__()
        C = transformer_dim
        self.transformer_dim = C
        self.transformer = transformer if transformer is not None else TwoWayTransformer(embedding_dim=C)
        self.num_mask_tokens = num_multimask_outputs + 1
        self.iou_token = nn.Embedding(1, C)
        self.mask_tokens = nn.Embedding(self.num_mask_tokens, C)
        self.output_upscaling = nn.Sequential(
            nn.ConvTranspose2d(C, C // 4, kernel_size=2, stride=2), _Norm2d(C // 4), nn.GELU(),
            nn.ConvTranspose2d(C // 4, C // 8, kernel_size=2, stride=2), nn.GELU())
        self.output_hypernetworks_mlps = nn.ModuleList(
            [_HeadMlp([C, C, C, C // 8]) for _ in range(self.num_mask_tokens)])
        self.iou_prediction_head = _HeadMlp([C] + [iou_head_hidden_dim] * (iou_head_depth - 1) + [self.num_mask_tokens])

    def forward(self, image_embeddings, image_pe, sparse_prompt_embeddings, dense_prompt_embeddings,
                multimask_output: bool = True):
        """One image embedding ``[1, C, h, w]`` against ``B`` prompts: mask logits ``[B, 3 or 1, 4h, 4w]``, IoU
        predictions (mask_decoder.py:73-160)."""
        dt = self.iou_token.weight.dtype
        sparse, dense = sparse_prompt_embeddings.to(dt), dense_prompt_embeddings.to(dt)
        tokens = torch.cat([self.iou_token.weight, self.mask_tokens.weight], dim=0)
        tokens = torch.cat([tokens.unsqueeze(0).expand(sparse.shape[0], -1, -1), sparse], dim=1)
        src = torch.repeat_interleave(image_embeddings.to(dt), tokens.shape[0], dim=0) + dense
        pos = torch.repeat_interleave(image_pe.to(dt), tokens.shape[0], dim=0)
        b, c, h, w = src.shape
        hs, src = self.transformer(src, pos, tokens)
        up = self.output_upscaling(src.transpose(1, 2).reshape(b, c, h, w))
        hyper = torch.stack([m(hs[:, 1 + i, :]) for i, m in enumerate(self.output_hypernetworks_mlps)], dim=1)
        masks = (hyper @ up.flatten(2)).reshape(b, -1, up.shape[2], up.shape[3])
        iou = self.iou_prediction_head(hs[:, 0, :])
        sl = slice(1, None) if multimask_output else slice(0, 1)
        return masks[:, sl], iou[:, sl]


class Sam(nn.Module):
    """Image encoder + prompt encoder + mask decoder with the reference's attribute names (sam.py:18-51)."""
    mask_threshold: float = 0.0
    image_format: str = "RGB"

    def __init__(self, image_encoder: nn.Module, prompt_encoder: PromptEncoder, mask_decoder: MaskDecoder,
                 pixel_mean=(123.675, 116.28, 103.53), pixel_std=(58.395, 57.12, 57.375)):
        super().__init__()
        self.image_encoder = image_encoder
        self.prompt_encoder = prompt_encoder
        self.mask_decoder = mask_decoder
        self.register_buffer("pixel_mean", torch.tensor(pixel_mean).view(-1, 1, 1), False)
        self.register_buffer("pixel_std", torch.tensor(pixel_std).view(-1, 1, 1), False)

    @property
    def device(self):
        return self.pixel_mean.device

    def preprocess(self, x: torch.Tensor) -> torch.Tensor:
        """Normalise and zero-pad to the encoder's square input (sam.py:164-174)."""
        x = (x - self.pixel_mean) / self.pixel_std
        S = self.image_encoder.img_size
        return F.pad(x, (0, S - x.shape[-1], 0, S - x.shape[-2]))

    def postprocess_masks(self, masks: torch.Tensor, input_size: Tuple[int, int], original_size: Tuple[int, int]):
        """sam.py:133-162."""
        S = self.image_encoder.img_size
        masks = F.interpolate(masks, (S, S), mode="bilinear", align_corners=False)
        masks = masks[..., :input_size[0], :input_size[1]]
        return F.interpolate(masks, original_size, mode="bilinear", align_corners=False)

    @torch.no_grad()
    def forward(self, batched_input, multimask_output: bool):
        """``Sam.forward`` (sam.py:54-131).  ``batched_input`` is a list of per-image dictionaries: ``image``
        (``[3, H, W]`` float pixels, already resized so that the long side is ``img_size``), ``original_size``
        ``(H, W)``, and optionally ``point_coords [B, N, 2]`` + ``point_labels [B, N]``, ``boxes [B, 4]``,
        ``mask_inputs [B, 1, 256, 256]``.  All images go through the encoder in one batch; returns one dictionary
        per image with ``masks`` (boolean, at the original size), ``iou_predictions`` and ``low_res_logits``."""
        x = torch.stack([self.preprocess(r["image"]) for r in batched_input], dim=0)
        model_dtype = self.mask_decoder.iou_prediction_head.layers[0].weight.dtype
        emb = self.image_encoder(x.to(model_dtype))
        pe = self.prompt_encoder.get_dense_pe()
        outputs = []
        for rec, e in zip(batched_input, emb):
            points = (rec["point_coords"], rec["point_labels"]) if "point_coords" in rec else None
            sparse, dense = self.prompt_encoder(points, rec.get("boxes"), rec.get("mask_inputs"))
            low, iou = self.mask_decoder(e.unsqueeze(0), pe, sparse, dense, multimask_output)
            masks = self.postprocess_masks(low, tuple(rec["image"].shape[-2:]), tuple(rec["original_size"]))
            outputs.append({"masks": masks > self.mask_threshold, "iou_predictions": iou, "low_res_logits": low})
        return outputs

    @torch.no_grad()
    def predict_boxes(self, images: torch.Tensor, boxes: torch.Tensor, multimask_output: bool = True):
        """Batched box prompting, one box per image: ``images [B, 3, S, S]`` already normalised, ``boxes [B, 4]`` in
        input pixels.  Returns binary masks ``[B, 3 or 1, S, S]``, predicted IoUs and low-resolution logits: the
        ``SamPredictor.set_torch_image`` + ``predict_torch`` sequence (predictor.py:69-90, 221-239) per image."""
        emb = self.image_encoder(images)
        pe = self.prompt_encoder.get_dense_pe()
        S = self.image_encoder.img_size
        masks, ious, lows = [], [], []
        for i in range(emb.shape[0]):
            sparse, dense = self.prompt_encoder(None, boxes[i:i + 1])
            low, iou = self.mask_decoder(emb[i:i + 1], pe, sparse, dense, multimask_output)
            full = self.postprocess_masks(low.float(), (S, S), (S, S))
            masks.append(full > self.mask_threshold); ious.append(iou); lows.append(low)
        return torch.cat(masks), torch.cat(ious), torch.cat(lows)


def build_heads(prompt_embed_dim: int = 256, image_size: int = 1024, patch: int = 16):
    """Prompt encoder and mask decoder with the sizes of build_sam.py:102-138."""
    g = image_size // patch
    pe = PromptEncoder(prompt_embed_dim, (g, g), (image_size, image_size), mask_in_chans=16)
    md = MaskDecoder(prompt_embed_dim, TwoWayTransformer(2, prompt_embed_dim, 8, 2048), 3, 3, 256)
    return pe, md
