"""GPU checks of what sits either side of the encoder kernels on the timed path and at the Python boundary:
the uint8 normalisation kernel and ``EncoderSession`` against the oracle, the attention drop-in with the
reference's argument shapes, the dispatcher op, ``Sam.forward`` / ``SamPredictor`` with the CUDA encoder, the
mask-generator filter stage, and the re-recording of a CUDA graph after the weights change."""
import numpy as np
import pytest
import torch

from oracle import amg_oracle as ao
from oracle import decoder_oracle as do
from oracle import encoder_oracle as eo

pytestmark = pytest.mark.gpu

TINY = eo.EncoderConfig(embed_dim=160, depth=4, num_heads=2, global_attn_indexes=(1, 3), out_chans=32)
TINY256 = eo.EncoderConfig(embed_dim=160, depth=4, num_heads=2, global_attn_indexes=(1, 3), out_chans=256)


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0).item()


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from segment_anything_fast_b200 import ops as _ops
    return _ops


# ----------------------------------------------------------------------------- preprocess + session
@pytest.mark.parametrize("B,S", [(2, 1024), (1, 64), (3, 256)])
def test_normalize_u8_is_bit_exact(ops, B, S):
    """``samb_normalize_u8`` against ``(u8 - mean) / std`` in fp32 (Sam.preprocess, sam.py:164-168) rounded to
    bf16 (the cast at predictor.py:88-90): the same bits, every pixel."""
    u8 = eo.seeded_images_u8(B, seed=51, img_size=S)
    want = eo.seeded_images(B, seed=51, img_size=S).to(torch.bfloat16)
    got = ops.normalize_u8(u8.cuda(), eo.PIXEL_MEAN, eo.PIXEL_STD).cpu()
    assert got.dtype == torch.bfloat16 and got.shape == want.shape
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("B,S,P", [(2, 1024, 16), (1, 256, 32), (3, 64, 16)])
def test_patch_rows_from_uint8_is_bit_exact(ops, B, S, P):
    """``samb_patch_rows_u8`` (normalisation inside the patch-embedding gather) against the two-step path
    normalise -> gather, and against the oracle's normalisation: the same bits."""
    u8 = eo.seeded_images_u8(B, seed=54, img_size=S)
    fused = ops.patch_rows_u8(u8.cuda(), P, eo.PIXEL_MEAN, eo.PIXEL_STD)
    two_step = ops.patch_rows(ops.normalize_u8(u8.cuda(), eo.PIXEL_MEAN, eo.PIXEL_STD), P)
    assert torch.equal(fused, two_step)
    want = eo.seeded_images(B, seed=54, img_size=S).to(torch.bfloat16)            # [B, 3, S, S]
    g = S // P
    rows = want.reshape(B, 3, g, P, g, P).permute(0, 2, 4, 1, 3, 5).reshape(B * g * g, 3 * P * P)
    assert torch.equal(fused.cpu().view(torch.int16), rows.contiguous().view(torch.int16))


def test_forward_u8_equals_forward_on_normalised_pixels(ops):
    from test_gpu_encoder import build_encoder
    sd = eo.seeded_state_dict(TINY, seed=1)
    enc = build_encoder(TINY, sd)
    u8 = eo.seeded_images_u8(2, seed=55)
    a = enc.forward_u8(u8.cuda(), eo.PIXEL_MEAN, eo.PIXEL_STD)
    b = enc(eo.seeded_images(2, seed=55).to(torch.bfloat16).cuda())
    ops.check_status()
    assert a.dtype == torch.bfloat16 and torch.equal(a, b)
    with pytest.raises(RuntimeError):
        enc.forward_u8(u8.cuda().float(), eo.PIXEL_MEAN, eo.PIXEL_STD)


@pytest.mark.parametrize("graph", [False, True])
def test_encoder_session_uint8_against_oracle(ops, graph):
    """The benchmark's timed path, host uint8 pixels -> ``EncoderSession.encode`` -> host embeddings, against the
    oracle's normalise -> encoder on the same pixels and weights."""
    from test_gpu_encoder import build_encoder
    from segment_anything_fast_b200 import EncoderSession
    sd = eo.seeded_state_dict(TINY, seed=1)
    enc = build_encoder(TINY, sd)
    sess = EncoderSession(enc, batch=2, graph=graph)
    u8 = eo.seeded_images_u8(2, seed=52)
    got = sess.encode(u8).float().clone()
    ref = eo.image_encoder_forward(eo.seeded_images(2, seed=52), sd, TINY, "fp32")
    err = (got - ref).abs().max().item()
    print(f"EncoderSession(graph={graph}) vs fp32 oracle: cosine {_cos(got, ref):.6f}, max-abs {err:.4f}")
    assert _cos(got, ref) > 0.999
    assert err < 0.1
    direct = enc(eo.seeded_images(2, seed=52).to(torch.bfloat16).cuda()).float().cpu()
    assert torch.equal(direct, got)                     # the session adds nothing but the normalisation


def test_graph_is_recorded_again_after_the_weights_change(ops):
    """A recorded graph points at the packed weights of its recording; new weights must not be ignored."""
    from test_gpu_encoder import build_encoder
    from segment_anything_fast_b200 import EncoderSession
    sd1 = eo.seeded_state_dict(TINY, seed=1)
    sd2 = eo.seeded_state_dict(TINY, seed=2)
    enc = build_encoder(TINY, sd1)
    sess = EncoderSession(enc, batch=1, graph=True)
    u8 = eo.seeded_images_u8(1, seed=53)
    a = sess.encode(u8).clone()
    enc.load_state_dict({k: v.to(torch.bfloat16) for k, v in sd2.items()})
    b = sess.encode(u8).clone()
    want = build_encoder(TINY, sd2)(eo.seeded_images(1, seed=53).to(torch.bfloat16).cuda()).cpu()
    assert not torch.equal(a, b)
    assert torch.equal(b, want)
    enc.set_quant("int8")
    c = sess.encode(u8).clone()
    want8 = build_encoder(TINY, sd2, quant="int8")(eo.seeded_images(1, seed=53).to(torch.bfloat16).cuda()).cpu()
    assert torch.equal(c, want8)


# ----------------------------------------------------------------------------- attention drop-in
def _flash4_inputs(B, H, N, d, dtype, seed=20):
    """The tensors of the reference's own op test (test/test_flash_4.py:10-31): N(0, 0.5), seed 20."""
    torch.manual_seed(seed)
    q, k, v = (torch.empty(B, H, N, d, dtype=dtype, device="cuda").normal_(0.0, 0.5) for _ in range(3))
    w = int(N ** 0.5)
    rel_h = torch.empty(B, H, N, w, 1, dtype=dtype, device="cuda").normal_(0.0, 0.5)
    rel_w = torch.empty(B, H, N, 1, w, dtype=dtype, device="cuda").normal_(0.0, 0.5)
    return q, k, v, rel_h, rel_w


@pytest.mark.parametrize("B,H,N,d", [(1, 16, 4096, 80), (2, 12, 4096, 64), (8, 2, 4096, 80), (3, 2, 196, 80)])
def test_attention_wrapper_reference_procedure(ops, B, H, N, d):
    """``_attention_rel_h_rel_w`` with the reference's 5-D bias tensors, compared the way test/test_flash_4.py:33-39
    compares: SDPA with the materialised bias, rtol = atol = 1e-3 (here the comparison arm is fp32 SDPA on the
    bf16-rounded inputs)."""
    from segment_anything_fast_b200.flash_4 import _attention_rel_h_rel_w
    q, k, v, rel_h, rel_w = _flash4_inputs(B, H, N, d, torch.bfloat16)
    out = _attention_rel_h_rel_w(q, k, v, rel_h, rel_w)
    ops.check_status()
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    for b in {0, B - 1}:
        f = lambda t: t[b:b + 1].float()
        bias = (f(rel_h) + f(rel_w)).view(1, H, N, N)
        ref = torch.nn.functional.scaled_dot_product_attention(f(q), f(k), f(v), attn_mask=bias)
        torch.testing.assert_close(out[b:b + 1].float(), ref, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("B,H,N,d", [(1, 16, 4096, 80), (8, 12, 4096, 64), (2, 3, 1024, 80), (5, 4, 196, 80), (3, 2, 196, 64)])
def test_attention_wrapper_float16(ops, B, H, N, d):
    """The float16 half of the reference's op test (test/test_flash_4.py:41-43: both dtypes, both head shapes,
    batch 1 and 8), same procedure and tolerance as above; also through the dispatcher op."""
    from segment_anything_fast_b200.flash_4 import _attention_rel_h_rel_w
    q, k, v, rel_h, rel_w = _flash4_inputs(B, H, N, d, torch.float16)
    if N == 1024:                                          # 1024 tokens: a 16 x 64 raster
        rel_h = rel_h[:, :, :, :N // 64].contiguous()
        rel_w = torch.empty(B, H, N, 1, 64, dtype=torch.float16, device="cuda").normal_(0.0, 0.5)
    out = _attention_rel_h_rel_w(q, k, v, rel_h, rel_w)
    ops.check_status()
    assert out.shape == q.shape and out.dtype == torch.float16
    worst = 0.0
    for b in {0, B - 1}:
        f = lambda t: t[b:b + 1].float()
        bias = (f(rel_h) + f(rel_w)).view(1, H, N, N)
        ref = torch.nn.functional.scaled_dot_product_attention(f(q), f(k), f(v), attn_mask=bias)
        worst = max(worst, (out[b:b + 1].float() - ref).abs().max().item())
        torch.testing.assert_close(out[b:b + 1].float(), ref, rtol=1e-3, atol=1e-3)
    print(f"float16 attention B={B} H={H} N={N} d={d}: max-abs {worst:.2e}")
    if N != 196:                                           # the dispatcher op is the global kernel's slot
        rel_h_w = torch.cat([rel_h.squeeze(-1), rel_w.squeeze(-2)], dim=-1)
        assert torch.equal(torch.ops.samb200.custom_flash_aligned(q, k, v, rel_h_w, d ** -0.5), out)


def test_attention_wrapper_refuses_what_it_does_not_convert(ops):
    """float32 and mixed types are refused, not converted."""
    from segment_anything_fast_b200.flash_4 import _attention_rel_h_rel_w
    q, k, v, rel_h, rel_w = _flash4_inputs(1, 2, 256, 80, torch.float32)
    with pytest.raises(RuntimeError, match="bfloat16"):
        _attention_rel_h_rel_w(q, k, v, rel_h, rel_w)
    q, k, v, rel_h, rel_w = _flash4_inputs(1, 2, 4096, 80, torch.float16)
    with pytest.raises(RuntimeError, match="share one dtype"):
        _attention_rel_h_rel_w(q, k.to(torch.bfloat16), v, rel_h, rel_w)


def test_dispatcher_op_on_cuda(ops):
    """``torch.ops.samb200.custom_flash_aligned(q, k, v, cat(rel_h, rel_w), sm_scale)``: the call flash_4.py:352-355
    makes, answered by the global-attention kernel; a non-default ``sm_scale`` is honoured."""
    from segment_anything_fast_b200.flash_4 import _attention_rel_h_rel_w
    q, k, v, rel_h, rel_w = _flash4_inputs(2, 3, 1024, 64, torch.bfloat16)       # 1024 tokens: rel_h is 16 wide
    rel_h = rel_h[:, :, :, :16].contiguous()
    rel_w = torch.empty(2, 3, 1024, 1, 64, dtype=torch.bfloat16, device="cuda").normal_(0.0, 0.5)
    rel_h_w = torch.cat([rel_h.squeeze(-1), rel_w.squeeze(-2)], dim=-1)
    out = torch.ops.samb200.custom_flash_aligned(q, k, v, rel_h_w, 64 ** -0.5)
    assert torch.equal(out, _attention_rel_h_rel_w(q, k, v, rel_h, rel_w))
    out2 = torch.ops.samb200.custom_flash_aligned(q, k, v, rel_h_w, 0.05)
    ops.check_status()
    bias = (rel_h.float() + rel_w.float()).view(2, 3, 1024, 1024)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=bias, scale=0.05)
    torch.testing.assert_close(out2.float(), ref, rtol=1e-3, atol=1e-3)
    with pytest.raises(RuntimeError, match="head dim"):
        p = torch.nn.functional.pad(q, (0, 64))
        torch.ops.samb200.custom_flash_aligned(p, p, p, rel_h_w, 0.1)


# ----------------------------------------------------------------------------- Sam.forward / SamPredictor
def _sam_on_gpu(enc_cfg, enc_sd, quant=None, sparse_mlp=False):
    from test_gpu_encoder import build_encoder
    from segment_anything_fast_b200 import apply_sparse
    from segment_anything_fast_b200.sam_heads import Sam, build_heads
    dcfg = do.DecoderConfig()
    dsd = dict(do.seeded_state_dict(dcfg, seed=3))
    dsd.update(do.seeded_mask_downscaling(dcfg, seed=3))
    pe, md = build_heads()
    pe.load_state_dict({k[len("prompt_encoder."):]: v for k, v in dsd.items() if k.startswith("prompt_encoder.")})
    md.load_state_dict({k[len("mask_decoder."):]: v for k, v in dsd.items() if k.startswith("mask_decoder.")})
    enc = build_encoder(enc_cfg, enc_sd, quant=quant)
    if sparse_mlp:
        apply_sparse(enc, mlp_only=True)
    return Sam(enc, pe, md).cuda().eval(), dcfg, dsd


def _iou(a, b):
    inter = (a & b).flatten(2).sum(-1).double()
    union = (a | b).flatten(2).sum(-1).double()
    return torch.where(union > 0, inter / union.clamp(min=1), torch.ones_like(union))


def test_sam_forward_on_gpu_against_oracle(ops):
    """``Sam.forward`` with the CUDA encoder: non-square image + boxes, square image + points + mask input, against
    the oracle's ``sam_forward`` over the fp32 encoder oracle on the same (bf16-rounded) weights."""
    from test_gpu_masks import scene_images  # noqa: F401  (same scene generator family)
    sd = eo.seeded_state_dict(TINY256, seed=11)
    sam, dcfg, dsd = _sam_on_gpu(TINY256, sd)
    recs = do.sam_forward_inputs(seed=9)
    # piecewise-flat pixels instead of noise, so that the masks have object-like regions
    g = torch.Generator().manual_seed(4)
    for r in recs:
        r["image"] = torch.nn.functional.interpolate(
            torch.randint(0, 256, (1, 3, 6, 8), generator=g).float(), r["image"].shape[-2:], mode="nearest")[0]
        if "mask_inputs" in r:                                    # a smooth blob, like a previous prediction's logits
            r["mask_inputs"] = torch.nn.functional.interpolate(
                torch.randn(1, 1, 4, 4, generator=g) * 6.0, (256, 256), mode="bilinear", align_corners=False)
    dev = [{k: (v.cuda() if torch.is_tensor(v) else v) for k, v in r.items()} for r in recs]
    got = sam(dev, multimask_output=True)
    ops.check_status()
    ref_sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    want = do.sam_forward(dsd, dcfg, lambda x: eo.image_encoder_forward(x, ref_sd, TINY256, "fp32"), recs, True)
    same = do.sam_forward(dsd, dcfg, lambda x: eo.image_encoder_forward(x, ref_sd, TINY256, "bf16"), recs, True)
    for i, (a, b, c) in enumerate(zip(got, want, same)):
        assert a["masks"].shape == b["masks"].shape
        iou = _iou(a["masks"].cpu(), b["masks"]).flatten()
        floor = _iou(c["masks"], b["masks"]).flatten()            # the oracle's own bf16 arithmetic against fp32
        area = b["masks"].float().mean((2, 3)).flatten()
        print(f"Sam.forward image {i}: IoU vs fp32 pipeline {[round(v, 4) for v in iou.tolist()]} "
              f"(oracle bf16 vs fp32 {[round(v, 4) for v in floor.tolist()]})")
        for j in range(iou.numel()):
            if area[j] >= 1e-3:
                assert iou[j].item() >= min(0.99, floor[j].item() - 0.01), (i, j)
        assert (a["iou_predictions"].float().cpu() - b["iou_predictions"]).abs().max().item() < 5e-2


def test_sam_predictor_call_sequence_on_gpu(ops):
    """``SamPredictor.set_torch_image`` + ``predict_torch`` (predictor.py:61-91,170-252) with the CUDA encoder, one
    box per image, against the oracle pipeline."""
    from test_gpu_masks import _boxes, scene_images
    from segment_anything_fast_b200 import SamPredictor
    sd = eo.seeded_state_dict(TINY256, seed=11)
    sam, dcfg, dsd = _sam_on_gpu(TINY256, sd)
    pred = SamPredictor(sam)
    x = scene_images(2, seed=12)                                  # normalised scenes; undo the normalisation to get pixels
    mean, std = torch.tensor(eo.PIXEL_MEAN).view(1, 3, 1, 1), torch.tensor(eo.PIXEL_STD).view(1, 3, 1, 1)
    pixels = (x * std + mean).round()
    boxes = _boxes(2, seed=13)
    ref_sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    for i in range(2):
        pred.set_torch_image(pixels[i:i + 1].cuda(), (1024, 1024))
        masks, iou_p, low = pred.predict_torch(None, None, boxes=boxes[i:i + 1].cuda(), multimask_output=True)
        ops.check_status()
        assert masks.shape == (1, 3, 1024, 1024) and masks.dtype == torch.bool and low.shape == (1, 3, 256, 256)
        emb = eo.image_encoder_forward((pixels[i:i + 1] - mean) / std, ref_sd, TINY256, "fp32")
        m_ref, iou_ref, _ = do.predict_masks_from_embedding(dsd, dcfg, emb, boxes[i:i + 1])
        iou = _iou(masks.cpu(), m_ref)[0]
        area = m_ref.float().mean((2, 3))[0]
        print(f"SamPredictor image {i}: IoU {[round(v, 4) for v in iou.tolist()]}")
        assert ((iou >= 0.99) | (area < 1e-3)).all()
        assert (iou_p[0].float().cpu() - iou_ref[0]).abs().max().item() < 5e-2


# ----------------------------------------------------------------------------- mask generator filter stage
def test_process_batch_filters_against_oracle(ops):
    """The filter stage of ``_process_batch_2`` (automatic_mask_generator.py:312-359) on a batch of 16 point prompts
    x 3 masks of disc-shaped logits inside a crop: same survivors, scores, boxes and masks as the step-by-step
    restatement."""
    from segment_anything_fast_b200 import amg
    g = torch.Generator().manual_seed(61)
    P, C, H, W = 16, 3, 300, 300
    # cone-shaped logits over discs of random centre, radius and steepness: steep ones are stable, some touch the
    # crop's inner edges, so that every filter keeps some masks and drops others
    cy, cx = torch.rand(P, C, 1, 1, generator=g) * H, torch.rand(P, C, 1, 1, generator=g) * W
    rad = torch.rand(P, C, 1, 1, generator=g) * 50 + 15
    amp = torch.rand(P, C, 1, 1, generator=g) * 100 + 20
    yy, xx = torch.arange(H).view(1, 1, H, 1).float(), torch.arange(W).view(1, 1, 1, W).float()
    logits = amp * (1.0 - ((yy - cy) ** 2 + (xx - cx) ** 2).sqrt() / rad)
    logits[0] = -8.0                                             # empty masks
    logits[1, 0] = 8.0                                           # a full mask: touches every crop edge
    iou_preds = torch.rand(P, C, generator=g) * 0.3 + 0.75
    points = torch.rand(P, 2, generator=g) * 300
    crop_box, orig_size = [100, 50, 400, 350], (350, 420)
    kw = dict(pred_iou_thresh=0.88, mask_threshold=0.0, stability_score_offset=1.0, stability_score_thresh=0.9)
    out = amg.process_batch_filters(logits.cuda(), iou_preds.cuda(), points, crop_box, orig_size, **kw)
    ops.check_status()
    idx, score, boxes, masks = ao.process_batch_filters(logits.numpy(), iou_preds.numpy(), crop_box, orig_size, **kw)
    assert 4 <= len(idx) < P * C // 2
    assert np.array_equal(out["keep"].cpu().numpy(), idx)
    assert np.array_equal(out["stability_score"].cpu().numpy(), score)
    assert np.array_equal(out["boxes"].cpu().numpy(), boxes)
    assert np.array_equal(out["masks"].cpu().numpy(), masks)
    assert np.array_equal(out["iou_preds"].cpu().numpy(), iou_preds.reshape(-1).numpy()[idx])
    assert np.array_equal(out["points"].cpu().numpy(), points.repeat_interleave(C, dim=0).numpy()[idx])
    rles = amg.mask_to_rle_pytorch(out["masks"])
    assert rles == ao.mask_to_rle(masks)


# ----------------------------------------------------------------------------- automatic mask generator
def _cone_logits(size, points, image_tone):
    """Deterministic stand-in for the decoder: three cone-shaped logit maps per point prompt (radius and steepness
    depend on the channel, the point and the crop's mean colour) and predicted IoUs, as float32 numpy arrays."""
    h, w = size
    yy, xx = np.mgrid[0:h, 0:w].astype(np.float64)
    P = points.shape[0]
    logits = np.empty((P, 3, h, w), dtype=np.float32)
    iou = np.empty((P, 3), dtype=np.float32)
    for p, (px, py) in enumerate(np.round(np.asarray(points, dtype=np.float64) * 64.0) / 64.0):   # the generator hands
        for c in range(3):                                    # the points over in float32: snap both sides to 1/64 pixel
            key = (int(px) * 7 + int(py) * 13 + c * 29 + int(image_tone)) % 97
            rad = 12.0 + 9.0 * c + 0.6 * key
            amp = 4.0 + (key % 11) * 3.0
            logits[p, c] = amp * (1.0 - np.sqrt((xx - px) ** 2 + (yy - py) ** 2) / rad)
            iou[p, c] = 0.55 + 0.004 * key + 0.001 * c
    return logits, iou


class _ConePredictor:
    """What the generator needs from ``SamPredictor``, answered by ``_cone_logits`` (computed on the host, so that
    the generator under test and the oracle see the same bits)."""

    def __init__(self):
        import types
        self.model = types.SimpleNamespace(mask_threshold=0.0)
        self.transform = types.SimpleNamespace(apply_coords=lambda pts, size: pts)
        self.device = torch.device("cuda")
        self.calls = []

    def set_image(self, crop):
        self.size, self.tone = crop.shape[:2], float(crop.mean())

    def reset_image(self):
        self.size = None

    def predict_torch(self, point_coords, point_labels, multimask_output=True, return_logits=False):
        assert multimask_output and return_logits and point_coords.shape[1:] == (1, 2) and point_labels.shape[1] == 1
        self.calls.append(point_coords.shape[0])
        logits, iou = _cone_logits(self.size, point_coords[:, 0].cpu().numpy().astype(np.float64), self.tone)
        return torch.as_tensor(logits).cuda(), torch.as_tensor(iou).cuda(), None


@pytest.mark.parametrize("layers,mode", [(0, "uncompressed_rle"), (1, "uncompressed_rle"), (1, "binary_mask")])
def test_mask_generator_against_oracle(ops, layers, mode):
    """``SamAutomaticMaskGenerator.generate`` (automatic_mask_generator.py:144-274): crops, point batches, the fused
    filter stage, NMS inside and between crops, the uncropping, the run-length encoding on the GPU and the records,
    against the oracle's restatement fed with the same decoder stand-in.  Everything downstream of the logits is
    integer-exact, so the records are equal."""
    from segment_anything_fast_b200 import SamAutomaticMaskGenerator
    from segment_anything_fast_b200.automatic_mask_generator import rle_to_mask
    g = torch.Generator().manual_seed(23)
    image = torch.randint(0, 256, (250, 330, 3), generator=g, dtype=torch.uint8).numpy()
    kw = dict(points_per_side=7, points_per_batch=16, pred_iou_thresh=0.6, stability_score_thresh=0.8,
              stability_score_offset=1.0, box_nms_thresh=0.5, crop_n_layers=layers, crop_nms_thresh=0.5,
              crop_n_points_downscale_factor=1)
    model = type("M", (), {"image_encoder": type("E", (), {"img_size": 1024})(), "device": torch.device("cuda")})()
    gen = SamAutomaticMaskGenerator(model, output_mode=mode, **kw)
    gen.predictor = _ConePredictor()
    got = gen.generate(image)
    ops.check_status()

    def predict_fn(crop, pts):
        return _cone_logits(crop.shape[:2], pts, float(crop.mean()))

    want = ao.generate(image, predict_fn, **kw)
    assert len(want) >= 8                                             # the filters and the NMS keep a real population
    assert len(got) == len(want)
    assert gen.predictor.calls[:4] == [16, 16, 16, 1]                 # 49 points in batches of 16
    for a, b in zip(got, want):
        assert a["bbox"] == b["bbox"] and a["area"] == b["area"] and a["crop_box"] == b["crop_box"]
        assert a["point_coords"] == b["point_coords"]
        assert abs(a["predicted_iou"] - b["predicted_iou"]) < 1e-6 and abs(a["stability_score"] - b["stability_score"]) < 1e-6
        if mode == "binary_mask":
            assert a["segmentation"].dtype == bool and np.array_equal(a["segmentation"], ao.rle_to_mask(b["segmentation"]))
        else:
            assert a["segmentation"] == b["segmentation"]
            assert int(rle_to_mask(a["segmentation"]).sum()) == a["area"]
    if layers:
        assert len({tuple(r["crop_box"]) for r in got}) > 1               # masks from crops survive the cross-crop NMS


def test_mask_generator_runs_on_the_cuda_encoder(ops):
    """The generator on a ``Sam`` with the CUDA encoder (random weights): the records are consistent with their own
    masks (area, box, point inside the crop) whatever the masks are."""
    from segment_anything_fast_b200 import SamAutomaticMaskGenerator
    sam, _, _ = _sam_on_gpu(TINY256, eo.seeded_state_dict(TINY256, seed=11))
    gen = SamAutomaticMaskGenerator(sam, points_per_side=4, points_per_batch=8, pred_iou_thresh=0.0,
                                    stability_score_thresh=0.0, crop_n_layers=0, output_mode="binary_mask")
    g = torch.Generator().manual_seed(29)
    image = torch.randint(0, 256, (3,), generator=g, dtype=torch.uint8).repeat(300, 400, 1)
    image[60:200, 80:300] = torch.randint(0, 256, (3,), generator=g, dtype=torch.uint8)
    recs = gen.generate(image.numpy())
    ops.check_status()
    assert len(recs) >= 1
    for r in recs:
        m = r["segmentation"]
        assert m.shape == (300, 400) and int(m.sum()) == r["area"]
        if r["area"]:
            ys, xs = np.nonzero(m)
            assert r["bbox"] == [int(xs.min()), int(ys.min()), int(xs.max() - xs.min()), int(ys.max() - ys.min())]
        assert r["crop_box"] == [0, 0, 400, 300] and 0.0 <= r["stability_score"] <= 1.0


def test_mask_generator_with_no_survivors(ops):
    """Thresholds nothing passes: every crop contributes empty tensors and the generator returns an empty list."""
    from segment_anything_fast_b200 import SamAutomaticMaskGenerator
    model = type("M", (), {"image_encoder": type("E", (), {"img_size": 1024})(), "device": torch.device("cuda")})()
    gen = SamAutomaticMaskGenerator(model, points_per_side=3, points_per_batch=4, pred_iou_thresh=2.0, crop_n_layers=1,
                                    output_mode="uncompressed_rle")
    gen.predictor = _ConePredictor()
    image = np.zeros((120, 160, 3), dtype=np.uint8)
    assert gen.generate(image) == []
    ops.check_status()
