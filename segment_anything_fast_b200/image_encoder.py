"""``ImageEncoderViT`` with the reference's constructor, parameters and ``state_dict`` keys
(segment_anything_fast/modeling/image_encoder.py:18-117) whose forward pass runs entirely on the
sm_100a kernels of ``libsamb200.so``.

The sub-modules (``patch_embed.proj``, ``blocks[i].norm1/attn.qkv/attn.proj/norm2/mlp.lin1/mlp.lin2``,
``neck``) are plain torch parameter containers created in the reference's order, so
``torch.manual_seed(s)`` + construction reproduces the reference's default initialisation and
``load_state_dict`` accepts a reference checkpoint unchanged.  They are never *called*: ``forward``
drives the C ABI directly.  There is no eager or CPU path; a missing library or a CPU tensor raises.
"""
from typing import Dict, List, Optional, Tuple, Type

import torch
import torch.nn as nn

from . import ops


class LayerNorm2d(nn.Module):
    """Parameter container for the neck's channel LayerNorm (modeling/common.py:31-43)."""

    def __init__(self, num_channels: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(num_channels))
        self.bias = nn.Parameter(torch.zeros(num_channels))
        self.eps = eps


class MLPBlock(nn.Module):
    """lin1 -> GELU -> lin2 parameters (modeling/common.py:13-26)."""

    def __init__(self, embedding_dim: int, mlp_dim: int, act: Type[nn.Module] = nn.GELU) -> None:
        super().__init__()
        self.lin1 = nn.Linear(embedding_dim, mlp_dim)
        self.lin2 = nn.Linear(mlp_dim, embedding_dim)
        self.act = act()


class Attention(nn.Module):
    """qkv / proj / rel_pos parameters (modeling/image_encoder.py:189-223)."""

    def __init__(self, dim: int, num_heads: int = 8, qkv_bias: bool = True, use_rel_pos: bool = False,
                 rel_pos_zero_init: bool = True, input_size: Optional[Tuple[int, int]] = None) -> None:
        super().__init__()
        self.num_heads = num_heads
        head_dim = dim // num_heads
        self.scale = head_dim ** -0.5
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        self.proj = nn.Linear(dim, dim)
        self.use_rel_pos = use_rel_pos
        if self.use_rel_pos:
            assert input_size is not None, "Input size must be provided if using relative positional encoding."
            self.rel_pos_h = nn.Parameter(torch.zeros(2 * input_size[0] - 1, head_dim))
            self.rel_pos_w = nn.Parameter(torch.zeros(2 * input_size[1] - 1, head_dim))


class Block(nn.Module):
    """One transformer block's parameters (modeling/image_encoder.py:120-165)."""

    def __init__(self, dim: int, num_heads: int, mlp_ratio: float = 4.0, qkv_bias: bool = True,
                 norm_layer: Type[nn.Module] = nn.LayerNorm, act_layer: Type[nn.Module] = nn.GELU,
                 use_rel_pos: bool = False, rel_pos_zero_init: bool = True, window_size: int = 0,
                 input_size: Optional[Tuple[int, int]] = None) -> None:
        super().__init__()
        self.norm1 = norm_layer(dim)
        self.attn = Attention(dim, num_heads=num_heads, qkv_bias=qkv_bias, use_rel_pos=use_rel_pos,
                              rel_pos_zero_init=rel_pos_zero_init,
                              input_size=input_size if window_size == 0 else (window_size, window_size))
        self.norm2 = norm_layer(dim)
        self.mlp = MLPBlock(embedding_dim=dim, mlp_dim=int(dim * mlp_ratio), act=act_layer)
        self.window_size = window_size


class PatchEmbed(nn.Module):
    """Patch-embedding convolution parameters (modeling/image_encoder.py:375-406)."""

    def __init__(self, kernel_size=(16, 16), stride=(16, 16), padding=(0, 0), in_chans: int = 3,
                 embed_dim: int = 768) -> None:
        super().__init__()
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=kernel_size, stride=stride, padding=padding)


def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.detach().to(torch.float32).contiguous()


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to(torch.bfloat16).contiguous()


def quantize_rows_absmax(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric int8: scale = max(absmax, 1e-5) / 127, q = clamp(rint(w / scale), -127, 127).
    Tensor-by-tensor divisions so that the GPU result is the IEEE quotient, bit for bit what a CPU
    evaluation of the same formula gives."""
    wf = w.detach().to(torch.float32)
    scale = wf.abs().amax(dim=1).clamp(min=1e-5) / torch.full((wf.shape[0],), 127.0, device=wf.device)
    q = torch.round(wf / scale[:, None]).clamp(-127, 127).to(torch.int8)
    return q.contiguous(), scale.contiguous()


class ImageEncoderViT(nn.Module):
    """Drop-in for the reference ``ImageEncoderViT``; see the module docstring.

    ``quant``: ``None`` (bf16 tcgen05 GEMMs) or ``"int8"`` (per-token dynamic activation quantisation,
    per-channel weights, int32 accumulation, for qkv / proj / lin1 / lin2 — the arithmetic torchao's
    ``apply_dynamic_quant`` installs at experiments/eval_combo.py:357-360)."""

    def __init__(self, img_size: int = 1024, patch_size: int = 16, in_chans: int = 3, embed_dim: int = 768,
                 depth: int = 12, num_heads: int = 12, mlp_ratio: float = 4.0, out_chans: int = 256,
                 qkv_bias: bool = True, norm_layer: Type[nn.Module] = nn.LayerNorm,
                 act_layer: Type[nn.Module] = nn.GELU, use_abs_pos: bool = True, use_rel_pos: bool = False,
                 rel_pos_zero_init: bool = True, window_size: int = 0,
                 global_attn_indexes: Tuple[int, ...] = ()) -> None:
        super().__init__()
        self.img_size = img_size
        self.patch_size = patch_size
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.out_chans = out_chans
        self.patch_embed = PatchEmbed(kernel_size=(patch_size, patch_size), stride=(patch_size, patch_size),
                                      in_chans=in_chans, embed_dim=embed_dim)
        self.pos_embed: Optional[nn.Parameter] = None
        if use_abs_pos:
            self.pos_embed = nn.Parameter(torch.zeros(1, img_size // patch_size, img_size // patch_size, embed_dim))
        self.blocks = nn.ModuleList()
        for i in range(depth):
            self.blocks.append(Block(
                dim=embed_dim, num_heads=num_heads, mlp_ratio=mlp_ratio, qkv_bias=qkv_bias, norm_layer=norm_layer,
                act_layer=act_layer, use_rel_pos=use_rel_pos, rel_pos_zero_init=rel_pos_zero_init,
                window_size=window_size if i not in global_attn_indexes else 0,
                input_size=(img_size // patch_size, img_size // patch_size)))
        self.neck = nn.Sequential(
            nn.Conv2d(embed_dim, out_chans, kernel_size=1, bias=False), LayerNorm2d(out_chans),
            nn.Conv2d(out_chans, out_chans, kernel_size=3, padding=1, bias=False), LayerNorm2d(out_chans))
        self.quant: Optional[str] = None
        self._packed: Optional[dict] = None
        self._packed_key = None
        self._buffers_cache: Dict[tuple, dict] = {}

    # ------------------------------------------------------------------ weight packing
    def set_quant(self, quant: Optional[str]) -> "ImageEncoderViT":
        if quant not in (None, "int8"):
            raise ValueError(f"unknown quant mode {quant!r}")
        self.quant = quant
        self._packed = None
        return self

    def _params_key(self):
        return (self.quant,) + tuple((p.data_ptr(), p._version, p.dtype) for p in self.parameters()) + tuple(
            bool(b.attn.use_rel_pos) for b in self.blocks)

    def _rel_tables(self, attn: Attention, size: int, dev) -> Tuple[torch.Tensor, torch.Tensor, int, int]:
        """[T, d] table = rel_pos_h rows, zero rows, rel_pos_w rows at t_w_off; column scale 1 | 1/scale."""
        t_w_off = 128 if size > 16 else 32
        T = 2 * t_w_off
        d = self.embed_dim // self.num_heads
        tab = torch.zeros(T, d, dtype=torch.bfloat16, device=dev)
        cs = torch.ones(T, dtype=torch.float32, device=dev)
        if attn.use_rel_pos:
            L = 2 * size - 1
            if attn.rel_pos_h.shape[0] != L or attn.rel_pos_w.shape[0] != L:
                raise RuntimeError("relative-position tables must have 2*size-1 rows (no interpolation path)")
            tab[:L] = _bf16(attn.rel_pos_h)
            tab[t_w_off:t_w_off + L] = _bf16(attn.rel_pos_w)
        cs[t_w_off:] = 1.0 / attn.scale
        return tab, cs, T, t_w_off

    def _pack(self) -> dict:
        C = self.embed_dim
        g = self.img_size // self.patch_size
        # the attention kernels know two geometries: a 64 x 64 token raster attended globally (keys indexed
        # kh*64 + kw) and 14 x 14 windows; anything else would index the bias tables wrongly without an error
        for i, blk in enumerate(self.blocks):
            if blk.window_size == 0 and g != 64:
                raise RuntimeError(f"block {i}: global attention is built for a 64x64 token grid "
                                   f"(img_size / patch_size = {g})")
            if blk.window_size not in (0, 14):
                raise RuntimeError(f"block {i}: window_size {blk.window_size} is not supported (0 or 14)")
        dev = self.patch_embed.proj.weight.device
        if dev.type != "cuda":
            raise RuntimeError("ImageEncoderViT (B200) needs its parameters on a CUDA device; there is no CPU path")
        pk: dict = {"blocks": []}
        pe = self.patch_embed.proj
        pk["pe_w"] = _bf16(pe.weight.reshape(C, -1))
        pk["pe_b"] = _f32(pe.bias)
        pk["pos"] = _bf16(self.pos_embed.reshape(g * g, C)) if self.pos_embed is not None else None

        def lin(m: nn.Linear, sparse_ok: bool = True):
            if self.quant == "int8":
                q, s = quantize_rows_absmax(m.weight)
                # a layer pruned by apply_sparse (2 of every 4 in-features zero) runs on the sparse
                # tensor-core path; the check guards against weights edited after the pruning
                if (sparse_ok and getattr(m, "_samb_sparse24", False) and q.shape[1] % 32 == 0
                        and bool(((q != 0).reshape(q.shape[0], -1, 4).sum(-1) <= 2).all())):
                    wc, meta = ops.pack_sp24(q)
                    return {"wc": wc, "meta": meta, "ws": s, "b": _f32(m.bias)}
                return {"wq": q, "ws": s, "b": _f32(m.bias)}
            return {"w": _bf16(m.weight), "b": _f32(m.bias)}

        for blk in self.blocks:
            size = g if blk.window_size == 0 else blk.window_size
            tab, cs, T, t_w_off = self._rel_tables(blk.attn, size, dev)
            pk["blocks"].append({
                "window": blk.window_size,
                "n1": (_f32(blk.norm1.weight), _f32(blk.norm1.bias), float(blk.norm1.eps)),
                "n2": (_f32(blk.norm2.weight), _f32(blk.norm2.bias), float(blk.norm2.eps)),
                "qkv": lin(blk.attn.qkv, sparse_ok=False), "proj": lin(blk.attn.proj),
                # keys / values of the zero-padded tokens of border windows: the projection of a zero row
                "qkv_b16": (_bf16(blk.attn.qkv.bias) if blk.attn.qkv.bias is not None
                            else torch.zeros(3 * C, dtype=torch.bfloat16, device=dev)),
                "lin1": lin(blk.mlp.lin1), "lin2": lin(blk.mlp.lin2),
                "tab": tab, "tab_scale": cs, "T": T, "t_w_off": t_w_off,
            })
        oc = self.out_chans
        pk["neck0_w"] = _bf16(self.neck[0].weight.reshape(oc, C))
        pk["neck1"] = (_f32(self.neck[1].weight), _f32(self.neck[1].bias), float(self.neck[1].eps))
        # [o, c, ky, kx] -> [o, (ky, kx, c)]: the column order samb_conv3x3_rows produces
        pk["neck2_w"] = _bf16(self.neck[2].weight.permute(0, 2, 3, 1).reshape(oc, 9 * oc))
        pk["neck3"] = (_f32(self.neck[3].weight), _f32(self.neck[3].bias), float(self.neck[3].eps))
        return pk

    def prepare(self) -> "ImageEncoderViT":
        """(Re)build the kernel-side weight views: fp32 vectors, bf16 / int8 matrices, bias tables."""
        key = self._params_key()
        if self._packed is None or key != self._packed_key:
            self._packed = self._pack()
            self._packed_key = key
        return self

    # ------------------------------------------------------------------ forward
    def _linear(self, a, a_scale, w, residual=None, gelu=False, out=None):
        if self.quant == "int8":
            if "wc" in w:
                return ops.gemm_i8_sp24(a, a_scale, w["wc"], w["meta"], w["ws"], w["b"], residual, gelu=gelu, out=out)
            return ops.gemm_i8(a, a_scale, w["wq"], w["ws"], w["b"], residual, gelu=gelu, out=out)
        return ops.gemm_bf16(a, w["w"], w["b"], residual, gelu=gelu, out=out)

    def _norm(self, x, n, grid=0, window=0):
        """LayerNorm (+ window partition) feeding a Linear: bf16 rows, or int8 rows + scales."""
        if self.quant == "int8":
            return ops.layernorm_quant_i8(x, n[0], n[1], n[2], grid=grid, window=window)
        return ops.layernorm(x, n[0], n[1], n[2], grid=grid, window=window), None

    def _act(self, x):
        """Input of proj / lin2: the bf16 activation itself, or its per-row int8 quantisation."""
        if self.quant == "int8":
            return ops.quant_rows_i8(x)
        return x, None

    @torch.no_grad()
    def forward(self, x: torch.Tensor, taps: Optional[dict] = None) -> torch.Tensor:
        """``x [B, C, S, S]`` normalised pixels in the model's dtype (the reference's call).  A device-side timeout
        of a kernel's bounded wait is recorded in the per-device status word; callers that want to know call
        ``ops.check_status()`` after their own synchronisation."""
        self._check_input(x)
        self.prepare()
        rows = ops.patch_rows(x.to(torch.bfloat16).contiguous(), self.patch_size)
        return self._encode_rows(rows, x.shape[0], taps).to(x.dtype)

    @torch.no_grad()
    def forward_u8(self, images_u8: torch.Tensor, pixel_mean, pixel_std, taps: Optional[dict] = None) -> torch.Tensor:
        """Raw ``uint8 [B, 3, S, S]`` pixels in, bf16 embeddings out: ``Sam.preprocess``' normalisation
        (sam.py:164-168) and the cast to the model dtype (predictor.py:88-90) happen inside the patch-embedding
        gather, bit for bit what ``forward((x - mean) / std)`` computes, without a normalised copy of the image."""
        self._check_input(images_u8)
        if images_u8.dtype != torch.uint8:
            raise RuntimeError("forward_u8 expects uint8 pixels")
        self.prepare()
        rows = ops.patch_rows_u8(images_u8.contiguous(), self.patch_size, pixel_mean, pixel_std)
        return self._encode_rows(rows, images_u8.shape[0], taps)

    def _check_input(self, x: torch.Tensor) -> None:
        if not x.is_cuda:
            raise RuntimeError("ImageEncoderViT (B200): input must be a CUDA tensor; there is no CPU path")
        if x.dim() != 4 or x.shape[2] != self.img_size or x.shape[3] != self.img_size:
            raise RuntimeError(f"expected [B, C, {self.img_size}, {self.img_size}] input")

    def _encode_rows(self, rows: torch.Tensor, B: int, taps: Optional[dict] = None) -> torch.Tensor:
        """Patch rows ``[B*g*g, 3*P*P]`` (bf16) -> embeddings ``[B, out_chans, g, g]`` (bf16)."""
        pk = self._packed
        g = self.img_size // self.patch_size
        C, H = self.embed_dim, self.num_heads
        d = C // H
        M = B * g * g
        cur = ops.gemm_bf16(rows, pk["pe_w"], pk["pe_b"], pk["pos"])
        del rows
        if taps is not None:
            taps["patch"] = cur.view(B, g, g, C)
        for i, bw in enumerate(pk["blocks"]):
            ws = bw["window"]
            xn, xs = self._norm(cur, bw["n1"])          # raster order for both block kinds
            wq = bw["qkv"]
            qkv = (ops.gemm_heads(xn, xs, wq["wq"], wq["ws"], wq["b"], d) if self.quant == "int8"
                   else ops.gemm_heads(xn, None, wq["w"], None, wq["b"], d))          # [3H, rows, d]
            # the rel-pos bias comes out of the attention kernels' own products of q with the tables (bw["tab"])
            if ws:
                o = ops.attn_relpos_window_tables(qkv, bw["qkv_b16"], bw["tab"], B, H, g, ws, d)
            else:
                o = ops.attn_relpos_global_tables(qkv, bw["tab"], B, H, g * g, d)
            del qkv, xn
            oa, os_ = self._act(o)
            x1 = self._linear(oa, os_, bw["proj"], residual=cur)
            del o, oa
            xn2, xs2 = self._norm(x1, bw["n2"])
            if self.quant == "int8":
                # int8 lin1 (dense or 2:4): the row maxima of GELU(lin1) come out of the GEMM epilogue, the
                # quantisation for lin2 is a streaming pass (no reduction over the 5120-wide hidden rows)
                w1 = bw["lin1"]
                if "wc" in w1:
                    ha, hs, hid = ops.gemm_i8_requant(xn2, xs2, w1["wc"], w1["ws"], w1["b"], gelu=True, meta=w1["meta"])
                else:
                    ha, hs, hid = ops.gemm_i8_requant(xn2, xs2, w1["wq"], w1["ws"], w1["b"], gelu=True)
            else:
                hid = self._linear(xn2, xs2, bw["lin1"], gelu=True)
                ha, hs = self._act(hid)
            cur = self._linear(ha, hs, bw["lin2"], residual=x1)
            del hid, ha, x1, xn2
            if taps is not None:
                taps[f"block{i}"] = cur.view(B, g, g, C)
        y = ops.gemm_bf16(cur, pk["neck0_w"])
        y = ops.layernorm2d(y, pk["neck1"][0], pk["neck1"][1], g * g, pk["neck1"][2], to_nchw=False)
        y = ops.gemm_bf16(ops.conv3x3_rows(y, g), pk["neck2_w"])
        y = ops.layernorm2d(y, pk["neck3"][0], pk["neck3"][1], g * g, pk["neck3"][2], to_nchw=True)
        return y.view(B, self.out_chans, g, g)
