"""CPU checks of the Python boundary around the encoder: registries, ``install``, ``Sam.forward`` with the
mask-prompt branch, ``SamPredictor``, the dispatcher-op registration and the device-mismatch guard.  The image
encoder itself has no CPU path, so tests that need embeddings use the oracle's stand-in encoder; the expected
values were produced by the reference's own ``Sam`` / ``SamPredictor`` holding the same stand-in
(tests/golden/make_golden.py, part (h))."""
import os
import types
from functools import partial

import numpy as np
import pytest
import torch

from oracle import decoder_oracle as do
from oracle import encoder_oracle as eo


def _heads_state_dict():
    cfg = do.DecoderConfig()
    sd = dict(do.seeded_state_dict(cfg, seed=3))
    sd.update(do.seeded_mask_downscaling(cfg, seed=3))
    return cfg, sd


def _sam_with_stub():
    from segment_anything_fast_b200.sam_heads import Sam, build_heads
    cfg, sd = _heads_state_dict()
    pe, md = build_heads()
    pe.load_state_dict({k[len("prompt_encoder."):]: v for k, v in sd.items() if k.startswith("prompt_encoder.")})   # strict
    md.load_state_dict({k[len("mask_decoder."):]: v for k, v in sd.items() if k.startswith("mask_decoder.")})
    return Sam(do.StubImageEncoder(seed=7), pe, md).eval(), cfg, sd


def _unpack(bits, shape):
    n = int(np.prod(shape))
    return np.unpackbits(bits)[:n].reshape(shape).astype(bool)


# ----------------------------------------------------------------------------- Sam.forward + mask prompts
@pytest.mark.parametrize("multimask", [True, False])
def test_sam_forward_matches_reference(golden_dir, multimask):
    """``Sam.forward`` (sam.py:54-131): non-square image with boxes, square image with points + mask input.
    The package's modules and the oracle restatement both reproduce the reference's outputs."""
    g = np.load(os.path.join(golden_dir, "sam_forward_fp32.npz"))
    sam, cfg, sd = _sam_with_stub()
    recs = do.sam_forward_inputs(seed=9)
    got = sam(recs, multimask_output=multimask)
    ora = do.sam_forward(sd, cfg, do.StubImageEncoder(seed=7), recs, multimask)
    for i, (r, o) in enumerate(zip(got, ora)):
        t = f"mm{int(multimask)}_img{i}"
        low_ref = g[t + "_low"]
        tol = 1e-3 * np.abs(low_ref).max()
        assert tuple(r["masks"].shape) == tuple(g[t + "_shape"]) == tuple(o["masks"].shape)
        for name, res in (("package", r), ("oracle", o)):
            assert np.abs(res["low_res_logits"][:, :, ::4, ::4].numpy() - low_ref).max() < tol, (name, t)
            assert np.allclose(res["iou_predictions"].numpy(), g[t + "_iou"], atol=1e-4), (name, t)
            sub = res["masks"][:, :, ::8, ::8].numpy()
            ref = _unpack(g[t + "_masks"], sub.shape)
            assert (sub != ref).mean() < 1e-3, (name, t)          # pixels whose logit is within rounding of zero
            assert np.allclose(res["masks"].float().mean((2, 3)).numpy(), g[t + "_area"], atol=1e-3), (name, t)


def test_mask_prompt_branch_matches_reference(golden_dir):
    """``PromptEncoder._embed_masks`` (prompt_encoder.py:111-114) replaces the "no mask" embedding."""
    g = np.load(os.path.join(golden_dir, "sam_forward_fp32.npz"))
    sam, cfg, sd = _sam_with_stub()
    rec = do.sam_forward_inputs(seed=9)[1]
    with torch.no_grad():
        _, dense = sam.prompt_encoder((rec["point_coords"], rec["point_labels"]), None, rec["mask_inputs"])
        sparse_only_mask, dense2 = sam.prompt_encoder(None, None, rec["mask_inputs"])
    assert np.allclose(dense[:, :, ::4, ::4].numpy(), g["dense_from_mask"], atol=1e-4)
    assert np.allclose(do.embed_masks(sd, rec["mask_inputs"])[:, :, ::4, ::4].numpy(), g["dense_from_mask"], atol=1e-4)
    assert sparse_only_mask.shape == (1, 0, 256) and torch.equal(dense, dense2)


# ----------------------------------------------------------------------------- SamPredictor
def test_sam_predictor_matches_reference(golden_dir):
    """``SamPredictor.set_image`` / ``predict`` (predictor.py:34-168): resize, preprocess, box prompt, then points
    with the previous low-resolution logits as mask input."""
    from segment_anything_fast_b200 import SamPredictor
    g = np.load(os.path.join(golden_dir, "sam_forward_fp32.npz"))
    sam, _, _ = _sam_with_stub()
    pred = SamPredictor(sam)
    img, box, pts, labels = do.predictor_inputs(seed=11)
    with pytest.raises(RuntimeError):
        pred.predict(box=box)
    pred.set_image(img)
    assert pred.input_size == (768, 1024) and pred.original_size == (480, 640)
    assert np.array_equal(pred.transform.apply_image(img)[::8, ::8], g["pred_resized"])
    assert np.allclose(pred.get_image_embedding()[:, ::8, ::4, ::4].numpy(), g["pred_features"], atol=1e-4)
    m, q, low = pred.predict(box=box, multimask_output=True)
    assert m.shape == (3, 480, 640) and m.dtype == bool and low.shape == (3, 256, 256)
    assert np.allclose(q, g["pred_box_iou"], atol=1e-4)
    assert np.abs(low[:, ::4, ::4] - g["pred_box_low"]).max() < 1e-3 * np.abs(g["pred_box_low"]).max()
    assert (m[:, ::4, ::4] != _unpack(g["pred_box_masks"], (3, 120, 160))).mean() < 1e-3
    best = int(q.argmax())
    m2, q2, low2 = pred.predict(point_coords=pts, point_labels=labels, mask_input=low[best:best + 1],
                                multimask_output=False, return_logits=True)
    assert np.allclose(q2, g["pred_pts_iou"], atol=1e-4)
    assert np.abs(low2[:, ::4, ::4] - g["pred_pts_low"]).max() < 1e-3 * np.abs(g["pred_pts_low"]).max()
    assert np.abs(m2[:, ::8, ::8] - g["pred_pts_logits"]).max() < 1e-3 * np.abs(g["pred_pts_logits"]).max()
    pred.reset_image()
    with pytest.raises(RuntimeError):
        pred.get_image_embedding()


def test_resize_longest_side_coordinates():
    from segment_anything_fast_b200 import ResizeLongestSide
    t = ResizeLongestSide(1024)
    assert t.get_preprocess_shape(480, 640, 1024) == (768, 1024)
    assert t.get_preprocess_shape(1500, 999, 1024) == (1024, 682)
    c = t.apply_coords(np.array([[320.0, 240.0]]), (480, 640))
    assert np.allclose(c, [[512.0, 384.0]])
    b = t.apply_boxes(np.array([10.0, 20.0, 30.0, 40.0]), (480, 640))
    assert np.allclose(b, [[16.0, 32.0, 48.0, 64.0]])
    assert torch.allclose(t.apply_boxes_torch(torch.tensor([[10.0, 20.0, 30.0, 40.0]]), (480, 640)), torch.tensor(b).float())


# ----------------------------------------------------------------------------- registries and install
_SIZES = {"vit_h": eo.VIT_H, "vit_b": eo.VIT_B, "default": eo.VIT_H,
          "vit_l": eo.EncoderConfig(embed_dim=1024, depth=24, num_heads=16, global_attn_indexes=(5, 11, 17, 23), out_chans=256)}


@pytest.mark.parametrize("name", ["default", "vit_h", "vit_l", "vit_b"])
@pytest.mark.parametrize("fast", [False, True])
def test_registry_entries(name, fast):
    """Every registry entry (build_sam.py:46-52,88-92) builds a ``Sam`` with the reference's key set and shapes
    (meta device: nothing is allocated); the fast registry casts to bf16 and forwards ``quant``."""
    from segment_anything_fast_b200 import sam_model_fast_registry, sam_model_registry
    with torch.device("meta"):
        sam = (sam_model_fast_registry[name](quant="int8") if fast else sam_model_registry[name]())
    cfg = _SIZES[name]
    want = {"image_encoder." + k: v for k, v in eo.state_dict_keys(cfg).items()}
    dcfg = do.DecoderConfig()
    want.update(do.state_dict_shapes(dcfg))
    want.update(do.mask_downscaling_shapes(dcfg))
    sd = sam.state_dict()
    assert set(sd) == set(want)
    for k, shp in want.items():
        assert tuple(sd[k].shape) == tuple(shp), k
    assert sam.image_encoder.img_size == 1024 and not sam.training
    enc_dtypes = {p.dtype for p in sam.image_encoder.parameters()}
    assert enc_dtypes == ({torch.bfloat16} if fast else {torch.float32})
    assert sam.image_encoder.quant == ("int8" if fast else None)
    assert {p.dtype for p in sam.mask_decoder.parameters()} == ({torch.bfloat16} if fast else {torch.float32})


def test_fast_registry_signature_and_dtype_none():
    from segment_anything_fast_b200 import build_sam_fast_vit_b
    with torch.device("meta"):
        sam = build_sam_fast_vit_b(checkpoint=None, compile_mode="max-autotune", dtype=None)
    assert {p.dtype for p in sam.parameters()} == {torch.float32}


def test_checkpoint_round_trip(tmp_path):
    """``checkpoint=`` takes a reference-format ``state_dict`` file (build_sam.py:144-147)."""
    from segment_anything_fast_b200 import build_sam_vit_b
    torch.manual_seed(1)
    a = build_sam_vit_b()
    path = os.path.join(tmp_path, "sam_vit_b.pth")
    torch.save(a.state_dict(), path)
    b = build_sam_vit_b(checkpoint=path)
    for (ka, va), (kb, vb) in zip(a.state_dict().items(), b.state_dict().items()):
        assert ka == kb and torch.equal(va, vb)


class _RefShapedAttention(torch.nn.Module):
    def __init__(self, dim, heads, size):
        super().__init__()
        self.num_heads, self.use_rel_pos = heads, True
        self.qkv, self.proj = torch.nn.Linear(dim, 3 * dim), torch.nn.Linear(dim, dim)
        self.rel_pos_h = torch.nn.Parameter(torch.randn(2 * size - 1, dim // heads))
        self.rel_pos_w = torch.nn.Parameter(torch.randn(2 * size - 1, dim // heads))


class _RefShapedBlock(torch.nn.Module):
    def __init__(self, dim, heads, window):
        super().__init__()
        self.norm1, self.norm2 = torch.nn.LayerNorm(dim, eps=1e-6), torch.nn.LayerNorm(dim, eps=1e-6)
        self.attn = _RefShapedAttention(dim, heads, window if window else 64)
        self.mlp = torch.nn.Module()
        self.mlp.lin1, self.mlp.lin2, self.mlp.act = torch.nn.Linear(dim, 4 * dim), torch.nn.Linear(4 * dim, dim), torch.nn.GELU()
        self.window_size = window


class _RefShapedEncoder(torch.nn.Module):
    """A module tree with the attributes ``install`` reads from the reference's ``ImageEncoderViT``
    (modeling/image_encoder.py:18-105), built from plain torch modules."""

    def __init__(self, dim=32, heads=2, out=16):
        super().__init__()
        self.img_size = 1024
        self.patch_embed = torch.nn.Module()
        self.patch_embed.proj = torch.nn.Conv2d(3, dim, 16, 16)
        self.pos_embed = torch.nn.Parameter(torch.randn(1, 64, 64, dim))
        self.blocks = torch.nn.ModuleList([_RefShapedBlock(dim, heads, w) for w in (14, 0, 14)])
        ln2d = lambda: torch.nn.LayerNorm(out)               # weight / bias of shape [out], like LayerNorm2d
        self.neck = torch.nn.Sequential(torch.nn.Conv2d(dim, out, 1, bias=False), ln2d(),
                                        torch.nn.Conv2d(out, out, 3, padding=1, bias=False), ln2d())


@pytest.mark.parametrize("wrapped", [False, True])
def test_install_replaces_the_encoder_slot(wrapped):
    """``install(sam)`` is the substitution of build_sam.py:70,78,84: same weights, dtype and geometry, also
    through a ``torch.compile``-style wrapper (``_orig_mod``)."""
    from segment_anything_fast_b200 import ImageEncoderViT, install
    torch.manual_seed(2)
    old = _RefShapedEncoder().to(torch.bfloat16)
    sam = types.SimpleNamespace(image_encoder=types.SimpleNamespace(_orig_mod=old) if wrapped else old)
    out = install(sam, quant="int8")
    new = out.image_encoder
    assert out is sam and isinstance(new, ImageEncoderViT)
    assert [b.window_size for b in new.blocks] == [14, 0, 14]
    assert new.quant == "int8" and new.img_size == 1024 and new.num_heads == 2 and new.out_chans == 16
    assert not new.training
    osd, nsd = old.state_dict(), new.state_dict()
    assert set(osd) == set(nsd)
    for k in osd:
        assert nsd[k].dtype == torch.bfloat16 and torch.equal(osd[k], nsd[k]), k
    with pytest.raises(RuntimeError):                      # the B200 encoder has no CPU path
        new(torch.zeros(1, 3, 1024, 1024, dtype=torch.bfloat16))


def test_unsupported_geometry_is_rejected_when_packing():
    """Global attention is built for the 64 x 64 raster and windows for 14 x 14; other geometries must not
    reach the kernels (they would index the bias tables wrongly without any error)."""
    from segment_anything_fast_b200 import ImageEncoderViT
    enc = ImageEncoderViT(img_size=512, depth=1, embed_dim=160, num_heads=2, use_rel_pos=True, window_size=0, out_chans=32)
    with pytest.raises(RuntimeError, match="64x64 token grid"):
        enc._pack()
    enc7 = ImageEncoderViT(depth=1, embed_dim=160, num_heads=2, use_rel_pos=True, window_size=7, out_chans=32)
    with pytest.raises(RuntimeError, match="window_size 7"):
        enc7._pack()


# ----------------------------------------------------------------------------- ops guards and the dispatcher op
def test_device_mismatch_is_rejected_before_any_launch(monkeypatch):
    """A tensor on another GPU than the current one would hand foreign pointers to a kernel launched here."""
    from segment_anything_fast_b200 import ops
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    fake = types.SimpleNamespace(is_cuda=True, dtype=torch.bfloat16, device=torch.device("cuda", 1))
    with pytest.raises(RuntimeError, match="cuda:1"):
        ops._need(fake, torch.bfloat16, "x")
    ops._need(types.SimpleNamespace(is_cuda=True, dtype=torch.bfloat16, device=torch.device("cuda", 0)), torch.bfloat16, "x")
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops._need(torch.zeros(1, dtype=torch.bfloat16), torch.bfloat16, "x")


def test_dispatcher_op_is_registered_with_the_reference_schema():
    """``samb200::custom_flash_aligned`` carries the schema of ``customflash::custom_flash_aligned``
    (flash_4.py:268-279) and has a Meta implementation (shape inference without a device)."""
    import segment_anything_fast_b200  # noqa: F401
    op = torch.ops.samb200.custom_flash_aligned
    schema = str(op.default._schema)
    assert "Tensor q, Tensor k, Tensor v, Tensor rel_h_w, float sm_scale" in schema and schema.endswith("-> Tensor")
    q = torch.empty(2, 3, 512, 80, device="meta", dtype=torch.bfloat16)
    rel = torch.empty(2, 3, 512, 8 + 64, device="meta", dtype=torch.bfloat16)
    out = op(q, q, q, rel, 80 ** -0.5)
    assert out.shape == q.shape and out.dtype == torch.bfloat16 and out.device.type == "meta"


def test_attention_wrapper_rejects_what_the_kernels_do_not_cover():
    from segment_anything_fast_b200.flash_4 import _attention_rel_h_rel_w
    q = torch.zeros(1, 1, 196, 80, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="bfloat16"):
        _attention_rel_h_rel_w(q, q, q, torch.zeros(1, 1, 196, 14, 1, dtype=torch.float32),
                               torch.zeros(1, 1, 196, 1, 14, dtype=torch.float32))
    q = torch.zeros(1, 1, 100, 80, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="not covered"):
        _attention_rel_h_rel_w(q, q, q, torch.zeros(1, 1, 100, 10, 1, dtype=torch.bfloat16),
                               torch.zeros(1, 1, 100, 1, 10, dtype=torch.bfloat16))


# ----------------------------------------------------------------------------- automatic mask generator (host side)
def test_mask_generator_geometry_matches_reference(golden_dir):
    """Point grids and crop boxes (utils/amg.py:216-274) of the package and of the oracle restatement against the
    reference's own outputs; run-length decoding, areas and box formats against the oracle."""
    from oracle import amg_oracle as ao
    from segment_anything_fast_b200 import automatic_mask_generator as mg
    gold = np.load(os.path.join(golden_dir, "amg_fp32.npz"))
    grids = mg.build_all_layer_point_grids(12, 2, 2)
    for i, g in enumerate(grids):
        assert np.array_equal(g, gold[f"grid{i}"])
        assert np.array_equal(ao.build_point_grid(int(12 / 2 ** i)), gold[f"grid{i}"])
    for tag in "abc":
        h, w, layers, ratio = gold[f"crop_{tag}_args"]
        for fn in (mg.generate_crop_boxes, ao.generate_crop_boxes):
            boxes, idx = fn((int(h), int(w)), int(layers), float(ratio))
            assert np.array_equal(np.array(boxes), gold[f"crop_{tag}_boxes"])
            assert np.array_equal(np.array(idx), gold[f"crop_{tag}_layers"])
    rng = np.random.default_rng(3)
    m = rng.random((4, 37, 53)) > 0.6
    m[1], m[2] = False, True
    for rle, mask in zip(ao.mask_to_rle(m), m):
        assert np.array_equal(mg.rle_to_mask(rle), mask)
        assert mg.area_from_rle(rle) == int(mask.sum())
    assert mg.box_xyxy_to_xywh(torch.tensor([3, 4, 10, 20])).tolist() == [3, 4, 7, 16]


def test_oracle_nms_is_torchvision_nms():
    """The greedy NMS of the oracle's generator against ``torchvision.ops.nms``, which the reference calls through
    ``batched_nms`` with a single category (automatic_mask_generator.py:216-221,259-264)."""
    from oracle import amg_oracle as ao
    from torchvision.ops import nms
    g = torch.Generator().manual_seed(17)
    lo = torch.randint(0, 300, (200, 2), generator=g).float()
    boxes = torch.cat([lo, lo + torch.randint(5, 150, (200, 2), generator=g).float()], dim=1)
    scores = torch.rand(200, generator=g)
    for thr in (0.3, 0.7):
        assert ao.nms(boxes.numpy(), scores.numpy(), thr).tolist() == nms(boxes, scores, thr).tolist()


def test_mask_generator_arguments():
    from segment_anything_fast_b200 import SamAutomaticMaskGenerator
    model = types.SimpleNamespace(image_encoder=types.SimpleNamespace(img_size=1024), device=torch.device("cpu"))
    with pytest.raises(ValueError, match="Exactly one"):
        SamAutomaticMaskGenerator(model, points_per_side=None, point_grids=None)
    with pytest.raises(ValueError, match="Exactly one"):
        SamAutomaticMaskGenerator(model, points_per_side=8, point_grids=[np.zeros((1, 2))])
    with pytest.raises(ValueError, match="output_mode"):
        SamAutomaticMaskGenerator(model, output_mode="png")
    gen = SamAutomaticMaskGenerator(model, points_per_side=4, crop_n_layers=1, crop_n_points_downscale_factor=2)
    assert [g.shape for g in gen.point_grids] == [(16, 2), (4, 2)]
