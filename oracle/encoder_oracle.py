"""CPU restatement of the SAM ViT image encoder (the checker, never the product).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the
benchmark's CPU-baseline leg.  The shipped package never imports it.

Every function is a functional restatement (plain torch CPU ops on a
``state_dict`` with the reference's key names) of one piece of
``segment_anything_fast/modeling/image_encoder.py`` and cites the lines it
follows.  Parity is pinned: ``tests/golden/make_golden.py`` runs the real
reference modules on seeded weights/inputs and stores their outputs; the
CPU test-suite checks this file against those stored vectors.

Three arithmetic modes:
  * ``precision="fp32"``: everything in float32 (the mathematical definition).
  * ``precision="bf16"``: values are rounded to bfloat16 at exactly the points
    where the reference's bf16 eager path materialises a bf16 tensor (each
    module / torch op output); arithmetic inside an op stays float32, as the
    GPU library kernels do.  This is the noise model for the bf16 tolerance.
  * ``precision="int8"``: the bf16 mode with qkv / proj / lin1 / lin2 evaluated by the
    dynamic-quantisation restatement in ``oracle/quant_oracle.py`` (parity unpinned, see there).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class EncoderConfig:
    """Hyper-parameters of ``ImageEncoderViT`` (image_encoder.py:19-37) as set by
    ``_build_sam`` (build_sam.py:95-120)."""

    embed_dim: int = 1280
    depth: int = 32
    num_heads: int = 16
    global_attn_indexes: Tuple[int, ...] = (7, 15, 23, 31)
    img_size: int = 1024
    patch_size: int = 16
    window_size: int = 14
    mlp_ratio: float = 4.0
    out_chans: int = 256
    ln_eps: float = 1e-6
    use_rel_pos: bool = True

    @property
    def grid(self) -> int:
        return self.img_size // self.patch_size

    @property
    def head_dim(self) -> int:
        return self.embed_dim // self.num_heads


VIT_H = EncoderConfig(1280, 32, 16, (7, 15, 23, 31))   # build_sam.py:14-21
VIT_L = EncoderConfig(1024, 24, 16, (5, 11, 17, 23))   # build_sam.py:27-34
VIT_B = EncoderConfig(768, 12, 12, (2, 5, 8, 11))      # build_sam.py:37-44

# False: attention written out as matmul / softmax / matmul (the definition the tests check against).
# True: torch's fused scaled_dot_product_attention with the bias as attn_mask, which is what the
# reference's CPU path executes; the CPU-baseline timing switches this on.
USE_SDPA = False

PIXEL_MEAN = (123.675, 116.28, 103.53)                 # build_sam.py:139
PIXEL_STD = (58.395, 57.12, 57.375)                    # build_sam.py:140


def _rounder(precision: str):
    if precision == "fp32":
        return lambda t: t
    if precision in ("bf16", "int8"):
        return lambda t: t.to(torch.bfloat16).to(torch.float32)
    raise ValueError(f"unknown precision {precision!r}")


# --------------------------------------------------------------------------
# weights and inputs
# --------------------------------------------------------------------------
def state_dict_keys(cfg: EncoderConfig) -> Dict[str, Tuple[int, ...]]:
    """Key → shape of ``ImageEncoderViT.state_dict()`` for ``cfg``
    (image_encoder.py:57-105,152-165,213-223; common.py:21-22,34-35)."""
    C, g, hd = cfg.embed_dim, cfg.grid, cfg.head_dim
    hidden = int(C * cfg.mlp_ratio)
    keys: Dict[str, Tuple[int, ...]] = {
        "pos_embed": (1, g, g, C),
        "patch_embed.proj.weight": (C, 3, cfg.patch_size, cfg.patch_size),
        "patch_embed.proj.bias": (C,),
    }
    for i in range(cfg.depth):
        s = g if i in cfg.global_attn_indexes else cfg.window_size
        p = f"blocks.{i}."
        keys[p + "norm1.weight"] = (C,)
        keys[p + "norm1.bias"] = (C,)
        if cfg.use_rel_pos:
            keys[p + "attn.rel_pos_h"] = (2 * s - 1, hd)
            keys[p + "attn.rel_pos_w"] = (2 * s - 1, hd)
        keys[p + "attn.qkv.weight"] = (3 * C, C)
        keys[p + "attn.qkv.bias"] = (3 * C,)
        keys[p + "attn.proj.weight"] = (C, C)
        keys[p + "attn.proj.bias"] = (C,)
        keys[p + "norm2.weight"] = (C,)
        keys[p + "norm2.bias"] = (C,)
        keys[p + "mlp.lin1.weight"] = (hidden, C)
        keys[p + "mlp.lin1.bias"] = (hidden,)
        keys[p + "mlp.lin2.weight"] = (C, hidden)
        keys[p + "mlp.lin2.bias"] = (C,)
    keys["neck.0.weight"] = (cfg.out_chans, C, 1, 1)
    keys["neck.1.weight"] = (cfg.out_chans,)
    keys["neck.1.bias"] = (cfg.out_chans,)
    keys["neck.2.weight"] = (cfg.out_chans, cfg.out_chans, 3, 3)
    keys["neck.3.weight"] = (cfg.out_chans,)
    keys["neck.3.bias"] = (cfg.out_chans,)
    return keys


def seeded_state_dict(cfg: EncoderConfig, seed: int = 0, std: float = 0.02,
                      nonzero_rel_pos: bool = True) -> Dict[str, torch.Tensor]:
    """Random weights that need no reference import: every matrix ~ N(0, std),
    LayerNorm gains ~ 1 + N(0, 0.1), biases ~ N(0, std).  The reference
    zero-initialises ``pos_embed`` and ``rel_pos_{h,w}`` (image_encoder.py:69-71,
    222-223), which would leave the relative-position path untested, so they are
    drawn from N(0, std) too unless ``nonzero_rel_pos`` is False."""
    g = torch.Generator().manual_seed(seed)
    sd: Dict[str, torch.Tensor] = {}
    for k, shape in state_dict_keys(cfg).items():
        t = torch.empty(shape, dtype=torch.float32).normal_(0.0, std, generator=g)
        if k.endswith("weight") and len(shape) == 1:          # LayerNorm gains
            t = 1.0 + 5.0 * t
        if ("rel_pos" in k or k == "pos_embed") and not nonzero_rel_pos:
            t.zero_()
        sd[k] = t
    return sd


def seeded_images_u8(batch: int, seed: int = 0, img_size: int = 1024) -> torch.Tensor:
    """The raw pixels of ``seeded_images``: uint8 U{0..255}, ``[B,3,S,S]`` contiguous."""
    g = torch.Generator().manual_seed(seed)
    u8 = torch.randint(0, 256, (batch, img_size, img_size, 3), generator=g, dtype=torch.uint8)
    return u8.permute(0, 3, 1, 2).contiguous()


def seeded_images(batch: int, seed: int = 0, img_size: int = 1024) -> torch.Tensor:
    """uint8-valued images U{0..255}, normalised with SAM's pixel mean/std the way
    ``Sam.preprocess`` does (sam.py:164-174) → float32 ``[B,3,S,S]``."""
    x = seeded_images_u8(batch, seed, img_size).to(torch.float32)
    mean = torch.tensor(PIXEL_MEAN).view(1, 3, 1, 1)
    std = torch.tensor(PIXEL_STD).view(1, 3, 1, 1)
    return (x - mean) / std


# --------------------------------------------------------------------------
# pieces of the forward pass
# --------------------------------------------------------------------------
def patch_embed(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, patch: int) -> torch.Tensor:
    """Non-overlapping conv, NCHW → NHWC (image_encoder.py:398-406)."""
    return F.conv2d(x, w, b, stride=patch).permute(0, 2, 3, 1)


def window_partition(x: torch.Tensor, ws: int) -> Tuple[torch.Tensor, Tuple[int, int]]:
    """Zero-pad H, W up to a multiple of ``ws`` and cut into ws×ws windows,
    window index major (image_encoder.py:256-277)."""
    B, H, W, C = x.shape
    ph, pw = (-H) % ws, (-W) % ws
    xp = F.pad(x, (0, 0, 0, pw, 0, ph))
    Hp, Wp = H + ph, W + pw
    xp = xp.reshape(B, Hp // ws, ws, Wp // ws, ws, C).permute(0, 1, 3, 2, 4, 5)
    return xp.reshape(-1, ws, ws, C), (Hp, Wp)


def window_unpartition(win: torch.Tensor, ws: int, pad_hw: Tuple[int, int],
                       hw: Tuple[int, int]) -> torch.Tensor:
    """Inverse of :func:`window_partition`, cropping the pad (image_encoder.py:280-302)."""
    Hp, Wp = pad_hw
    H, W = hw
    B = win.shape[0] // ((Hp // ws) * (Wp // ws))
    x = win.reshape(B, Hp // ws, Wp // ws, ws, ws, -1).permute(0, 1, 3, 2, 4, 5)
    return x.reshape(B, Hp, Wp, -1)[:, :H, :W, :]


def rel_pos_table(q_size: int, k_size: int, rel_pos: torch.Tensor) -> torch.Tensor:
    """``R[q, k, :] = rel_pos[q - k + (k_size - 1), :]`` (image_encoder.py:305-335).
    SAM always has ``rel_pos.shape[0] == 2*size-1`` and q_size == k_size, so the
    interpolation branch (:318-326) is never taken; it is rejected here."""
    if q_size != k_size or rel_pos.shape[0] != 2 * q_size - 1:
        raise ValueError("oracle covers only the q_size == k_size, un-interpolated case")
    idx = torch.arange(q_size)[:, None] - torch.arange(k_size)[None, :] + (k_size - 1)
    return rel_pos[idx]


def decomposed_rel_pos(q: torch.Tensor, rel_pos_h: torch.Tensor, rel_pos_w: torch.Tensor,
                       size: Tuple[int, int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """``rel_h[b,(h,w),kh] = q[b,(h,w),:]·Rh[h,kh,:]``, ``rel_w[b,(h,w),kw] = q·Rw[w,kw,:]``
    with the *unscaled* q (image_encoder.py:338-372).  q: ``[B', N, d]`` →
    ``([B', N, S], [B', N, S])``."""
    S_h, S_w = size
    Bq, N, d = q.shape
    Rh = rel_pos_table(S_h, S_h, rel_pos_h)
    Rw = rel_pos_table(S_w, S_w, rel_pos_w)
    rq = q.reshape(Bq, S_h, S_w, d)
    rel_h = torch.einsum("bhwc,hkc->bhwk", rq, Rh).reshape(Bq, N, S_h)
    rel_w = torch.einsum("bhwc,wkc->bhwk", rq, Rw).reshape(Bq, N, S_w)
    return rel_h, rel_w


def attention_rel_h_rel_w(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                          rel_h: torch.Tensor, rel_w: torch.Tensor,
                          precision: str = "fp32") -> torch.Tensor:
    """``softmax(q kᵀ / sqrt(d) + rel_h[..., :, None] + rel_w[..., None, :]) v``: the
    composite that ``_attention_rel_h_rel_w`` reduces to (flash_4.py:343,368-370).
    q, k, v ``[..., N, d]``; rel_h ``[..., N, Sh]``; rel_w ``[..., N, Sw]`` with
    ``N == Sh*Sw`` and key ``j = kh*Sw + kw``.  In bf16 mode the summed bias is
    rounded once (flash_4.py:368 adds two bf16 tensors) and the output once."""
    r = _rounder(precision)
    d = q.shape[-1]
    bias = r(rel_h.unsqueeze(-1) + rel_w.unsqueeze(-2)).flatten(-2)
    if USE_SDPA:   # the same composite through torch's fused CPU kernel, as the reference calls it (flash_4.py:370)
        return r(F.scaled_dot_product_attention(q, k, v, attn_mask=bias))
    logits = torch.matmul(q, k.transpose(-1, -2)) * (1.0 / math.sqrt(d)) + bias
    return r(torch.matmul(torch.softmax(logits, dim=-1), v))


def _linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], precision: str) -> torch.Tensor:
    """``nn.Linear``; with ``precision="int8"`` the dynamic-quantisation arithmetic of
    :func:`oracle.quant_oracle.int8_linear` (per-token activations, per-channel weights, int32
    accumulation) that the benchmark's int8 configuration swaps in for qkv / proj / lin1 / lin2."""
    if precision == "int8":
        from . import quant_oracle as qo
        return qo.int8_linear(x.reshape(-1, x.shape[-1]), w, b).reshape(*x.shape[:-1], w.shape[0])
    return F.linear(x, w, b)


def attention_module(x: torch.Tensor, sd: Dict[str, torch.Tensor], prefix: str, num_heads: int,
                     use_rel_pos: bool, precision: str) -> torch.Tensor:
    """``Attention.forward`` (image_encoder.py:225-253) on ``x [B', S, S, C]``."""
    r = _rounder(precision)
    Bp, H, W, C = x.shape
    N, hd = H * W, C // num_heads
    qkv = r(_linear(x, sd[prefix + "qkv.weight"], sd[prefix + "qkv.bias"], precision))
    qkv = qkv.reshape(Bp, N, 3, num_heads, hd).permute(2, 0, 3, 1, 4)       # :228
    q, k, v = qkv.reshape(3, Bp * num_heads, N, hd).unbind(0)               # :230
    if use_rel_pos:
        rel_h, rel_w = decomposed_rel_pos(q, sd[prefix + "rel_pos_h"], sd[prefix + "rel_pos_w"], (H, W))
        rel_h, rel_w = r(rel_h), r(rel_w)
    else:
        rel_h = q.new_zeros(Bp * num_heads, N, H)
        rel_w = q.new_zeros(Bp * num_heads, N, W)
    o = attention_rel_h_rel_w(q, k, v, rel_h, rel_w, precision)             # :245
    o = o.reshape(Bp, num_heads, H, W, hd).permute(0, 2, 3, 1, 4).reshape(Bp, H, W, C)  # :249
    return r(_linear(o, sd[prefix + "proj.weight"], sd[prefix + "proj.bias"], precision))          # :251


def mlp_block(x: torch.Tensor, sd: Dict[str, torch.Tensor], prefix: str, precision: str) -> torch.Tensor:
    """``lin2(GELU_erf(lin1(x)))`` (common.py:25-26)."""
    r = _rounder(precision)
    h = r(_linear(x, sd[prefix + "lin1.weight"], sd[prefix + "lin1.bias"], precision))
    h = r(F.gelu(h))
    return r(_linear(h, sd[prefix + "lin2.weight"], sd[prefix + "lin2.bias"], precision))


def block_forward(x: torch.Tensor, sd: Dict[str, torch.Tensor], i: int, cfg: EncoderConfig,
                  precision: str) -> torch.Tensor:
    """``Block.forward`` (image_encoder.py:167-183).  Note the zero padding of
    :func:`window_partition` happens *after* norm1, so pad tokens go through the
    biased qkv projection and are attended to as keys."""
    r = _rounder(precision)
    p = f"blocks.{i}."
    C = cfg.embed_dim
    ws = 0 if i in cfg.global_attn_indexes else cfg.window_size
    shortcut = x
    y = r(F.layer_norm(x, (C,), sd[p + "norm1.weight"], sd[p + "norm1.bias"], cfg.ln_eps))
    if ws > 0:
        H, W = y.shape[1], y.shape[2]
        y, pad_hw = window_partition(y, ws)
    y = attention_module(y, sd, p + "attn.", cfg.num_heads, cfg.use_rel_pos, precision)
    if ws > 0:
        y = window_unpartition(y, ws, pad_hw, (H, W))
    x = r(shortcut + y)
    z = r(F.layer_norm(x, (C,), sd[p + "norm2.weight"], sd[p + "norm2.bias"], cfg.ln_eps))
    return r(x + mlp_block(z, sd, p + "mlp.", precision))


def layer_norm_2d(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float,
                  precision: str) -> torch.Tensor:
    """Channel LayerNorm on NCHW written as elementwise tensor ops (common.py:37-43);
    in the reference's bf16 path each of those ops rounds to bf16."""
    r = _rounder(precision)
    u = r(x.mean(1, keepdim=True))
    dlt = r(x - u)
    s = r(r(dlt * dlt).mean(1, keepdim=True))
    y = r(dlt / r(torch.sqrt(r(s + eps))))
    return r(r(w[None, :, None, None] * y) + b[None, :, None, None])


def neck_forward(x_nhwc: torch.Tensor, sd: Dict[str, torch.Tensor], cfg: EncoderConfig,
                 precision: str) -> torch.Tensor:
    """conv1×1 → LayerNorm2d → conv3×3(pad 1) → LayerNorm2d, no conv biases
    (image_encoder.py:89-105,115)."""
    r = _rounder(precision)
    x = x_nhwc.permute(0, 3, 1, 2)
    x = r(F.conv2d(x, sd["neck.0.weight"]))
    x = layer_norm_2d(x, sd["neck.1.weight"], sd["neck.1.bias"], 1e-6, precision)
    x = r(F.conv2d(x, sd["neck.2.weight"], padding=1))
    return layer_norm_2d(x, sd["neck.3.weight"], sd["neck.3.bias"], 1e-6, precision)


def image_encoder_forward(x: torch.Tensor, sd: Dict[str, torch.Tensor], cfg: EncoderConfig,
                          precision: str = "fp32", blocks: Optional[Sequence[int]] = None,
                          taps: Optional[dict] = None) -> torch.Tensor:
    """``ImageEncoderViT.forward`` (image_encoder.py:107-117): ``[B,3,S,S]`` →
    ``[B,out_chans,S/16,S/16]``.  ``blocks`` restricts the depth loop to a subset
    (used by the bounded CPU-baseline sample); ``taps`` collects intermediate
    activations ("patch", "block{i}") for stage-wise comparisons."""
    r = _rounder(precision)
    sd = {k: r(v.to(torch.float32)) for k, v in sd.items()}
    x = r(x.to(torch.float32))
    x = r(patch_embed(x, sd["patch_embed.proj.weight"], sd["patch_embed.proj.bias"], cfg.patch_size))
    x = r(x + sd["pos_embed"])
    if taps is not None:
        taps["patch"] = x
    for i in (range(cfg.depth) if blocks is None else blocks):
        x = block_forward(x, sd, i, cfg, precision)
        if taps is not None:
            taps[f"block{i}"] = x
    return neck_forward(x, sd, cfg, precision)
