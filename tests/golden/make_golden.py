"""Generate the golden vectors under tests/golden/ by running the REAL reference.

Run once, in a container that has the reference checkout (it is not needed,
and not read, by any test):

    python tests/golden/make_golden.py --reference /path/to/segment-anything-fast

It imports ``segment_anything_fast`` from that checkout with
``SEGMENT_ANYTHING_FAST_USE_FLASH_4=0`` (CPU, SDPA composite), feeds it the
seeded weights / inputs that ``oracle.encoder_oracle`` can regenerate anywhere,
and stores (sub-sampled, float32) outputs as small ``.npz`` files.  The tests
then check the oracle restatement against these files on CPU and the CUDA
path against the oracle on the GPU.
"""
import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

TINY = dict(embed_dim=160, depth=4, num_heads=2, global_attn_indexes=(1, 3), out_chans=32)


def sd_digest(sd):
    h = hashlib.sha256()
    for k in sorted(sd):
        h.update(k.encode())
        h.update(sd[k].detach().to(torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


def golden_decoder():
    """(f) prompt encoder + mask decoder + post-processing of the reference's ``Sam`` on seeded decoder
    weights, a seeded embedding and two box prompts (+ one point prompt through the prompt encoder)."""
    from segment_anything_fast.build_sam import sam_model_registry

    from oracle import decoder_oracle as do

    torch.manual_seed(0)
    sam = sam_model_registry["vit_b"]().eval()
    cfg = do.DecoderConfig()
    sd = do.seeded_state_dict(cfg, seed=3)
    pe_sd = {k[len("prompt_encoder."):]: v for k, v in sd.items() if k.startswith("prompt_encoder.")}
    md_sd = {k[len("mask_decoder."):]: v for k, v in sd.items() if k.startswith("mask_decoder.")}
    missing = sam.prompt_encoder.load_state_dict(pe_sd, strict=False).missing_keys
    assert all(k.startswith("mask_downscaling.") for k in missing), missing       # unused without mask prompts
    sam.mask_decoder.load_state_dict(md_sd)                                        # strict: key set agrees
    emb = torch.randn(1, 256, 64, 64, generator=torch.Generator().manual_seed(5))
    boxes = torch.tensor([[100.0, 200.0, 600.0, 800.0], [10.0, 20.0, 300.0, 400.0]])
    sp, de = sam.prompt_encoder(points=None, boxes=boxes, masks=None)
    low, iou = sam.mask_decoder(image_embeddings=emb, image_pe=sam.prompt_encoder.get_dense_pe(),
                                sparse_prompt_embeddings=sp, dense_prompt_embeddings=de, multimask_output=True)
    full = sam.postprocess_masks(low, (1024, 1024), (1024, 1024))
    pts = (torch.tensor([[[500.0, 300.0], [100.0, 100.0]]]), torch.tensor([[1, 0]]))
    sp_pts, _ = sam.prompt_encoder(points=pts, boxes=None, masks=None)
    np.savez_compressed(
        os.path.join(HERE, "decoder_fp32.npz"), boxes=boxes.numpy(), sparse=sp.numpy(), low=low[:, :, ::4, ::4].numpy(),
        iou=iou.numpy(), full_logits=full[:, :, ::16, ::16].numpy(), area=(full > 0).float().mean((2, 3)).numpy(),
        dense_pe=sam.prompt_encoder.get_dense_pe()[:, :, ::8, ::8].numpy(), sparse_points=sp_pts.numpy())


def golden_sam_forward():
    """(h) the reference's ``Sam.forward`` (sam.py:54-131) with the mask-prompt branch of its prompt encoder
    (prompt_encoder.py:111-114), on seeded decoder weights, with a stand-in image encoder (the encoder itself is
    covered by (a)/(b)): one non-square image with two boxes, one square image with points + a mask input."""
    from segment_anything_fast.build_sam import sam_model_registry

    from oracle import decoder_oracle as do

    torch.manual_seed(0)
    sam = sam_model_registry["vit_b"]().eval()
    cfg = do.DecoderConfig()
    sd = dict(do.seeded_state_dict(cfg, seed=3))
    sd.update(do.seeded_mask_downscaling(cfg, seed=3))
    sam.prompt_encoder.load_state_dict({k[len("prompt_encoder."):]: v for k, v in sd.items() if k.startswith("prompt_encoder.")})
    sam.mask_decoder.load_state_dict({k[len("mask_decoder."):]: v for k, v in sd.items() if k.startswith("mask_decoder.")})
    sam.image_encoder = do.StubImageEncoder(seed=7)
    recs = do.sam_forward_inputs(seed=9)
    out = {}
    for mm in (True, False):
        res = sam(recs, multimask_output=mm)
        for i, r in enumerate(res):
            t = f"mm{int(mm)}_img{i}"
            out[t + "_low"] = r["low_res_logits"][:, :, ::4, ::4].numpy()
            out[t + "_iou"] = r["iou_predictions"].numpy()
            out[t + "_area"] = r["masks"].float().mean((2, 3)).numpy()
            out[t + "_masks"] = np.packbits(r["masks"][:, :, ::8, ::8].numpy())
            out[t + "_shape"] = np.array(r["masks"].shape)
    dense = sam.prompt_encoder(points=(recs[1]["point_coords"], recs[1]["point_labels"]), boxes=None,
                               masks=recs[1]["mask_inputs"])[1]
    out["dense_from_mask"] = dense[:, :, ::4, ::4].detach().numpy()
    # the reference's SamPredictor on the same model: set_image on a 480 x 640 uint8 image, a box prompt, then
    # points + the first answer's best low-resolution logits fed back as mask_input (predictor.py:34-168)
    from segment_anything_fast.predictor import SamPredictor
    pred = SamPredictor(sam)
    img, box, pts, labels = do.predictor_inputs(seed=11)
    pred.set_image(img)
    out["pred_resized"] = pred.transform.apply_image(img)[::8, ::8]
    out["pred_features"] = pred.get_image_embedding()[:, ::8, ::4, ::4].numpy()
    m, q, low = pred.predict(box=box, multimask_output=True)
    out["pred_box_masks"] = np.packbits(m[:, ::4, ::4])
    out["pred_box_area"] = m.reshape(3, -1).mean(1)
    out["pred_box_iou"], out["pred_box_low"] = q, low[:, ::4, ::4]
    best = int(q.argmax())
    m2, q2, low2 = pred.predict(point_coords=pts, point_labels=labels, mask_input=low[best:best + 1],
                                multimask_output=False, return_logits=True)
    out["pred_pts_logits"] = m2[:, ::8, ::8]
    out["pred_pts_iou"], out["pred_pts_low"] = q2, low2[:, ::4, ::4]
    np.savez_compressed(os.path.join(HERE, "sam_forward_fp32.npz"), **out)


def golden_amg():
    """(g) the automatic mask generator's logit filters on seeded logits (an empty and a full mask included)."""
    from segment_anything_fast.utils.amg import batched_mask_to_box, calculate_stability_score
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(6, 37, 50, generator=g) * 2.0
    logits[1] = -5.0                      # empty at every threshold
    logits[2] = 5.0                       # full
    logits[3, :, :] = -3.0
    logits[3, 5:9, 40:50] = 4.0           # one rectangle touching the right border
    score = calculate_stability_score(logits, 0.0, 1.0)
    boxes = batched_mask_to_box(logits > 0.0)
    # run-length encodings of the thresholded masks (both reference encoders agree; checked here)
    from segment_anything_fast.utils.amg import mask_to_rle_pytorch, mask_to_rle_pytorch_2
    masks = logits > 0.0
    rles = mask_to_rle_pytorch(masks)
    assert rles == mask_to_rle_pytorch_2(masks)
    rle_len = np.array([len(r["counts"]) for r in rles], dtype=np.int64)
    rle_counts = np.concatenate([np.asarray(r["counts"], dtype=np.int64) for r in rles])
    # crop-edge filter of _process_batch_2 on seeded boxes inside a crop of a larger image
    from segment_anything_fast.utils.amg import is_box_near_crop_edge
    ge = torch.Generator().manual_seed(9)
    lo = torch.randint(0, 200, (64, 2), generator=ge)
    eb = torch.cat([lo, lo + torch.randint(1, 120, (64, 2), generator=ge)], dim=1).clamp(max=299)
    crop, orig = [100, 50, 400, 350], [0, 0, 420, 350]
    edge = is_box_near_crop_edge(eb, crop, orig)
    # the generator's point grids and crop boxes (utils/amg.py:216-274)
    from segment_anything_fast.utils.amg import build_all_layer_point_grids, generate_crop_boxes
    grids = build_all_layer_point_grids(12, 2, 2)
    geo = {f"grid{i}": g for i, g in enumerate(grids)}
    for tag, size, layers, ratio in (("a", (480, 640), 2, 512 / 1500), ("b", (1024, 1024), 1, 512 / 1500),
                                     ("c", (333, 517), 3, 0.2)):
        cb, li = generate_crop_boxes(size, layers, ratio)
        geo[f"crop_{tag}_args"] = np.array([size[0], size[1], layers, ratio], dtype=np.float64)
        geo[f"crop_{tag}_boxes"] = np.array(cb, dtype=np.int64)
        geo[f"crop_{tag}_layers"] = np.array(li, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "amg_fp32.npz"), logits=logits.numpy(), score=score.numpy(), boxes=boxes.numpy(),
                        rle_len=rle_len, rle_counts=rle_counts, edge_boxes=eb.numpy(), edge_crop=np.array(crop),
                        edge_orig=np.array(orig), edge_out=edge.numpy(), **geo)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of segment-anything-fast to import")
    ap.add_argument("--only", choices=["decoder", "amg", "sam_forward"], default=None, help="regenerate just this file")
    args = ap.parse_args()
    os.environ["SEGMENT_ANYTHING_FAST_USE_FLASH_4"] = "0"
    sys.path.insert(0, args.reference)
    torch.set_grad_enabled(False)
    if args.only == "decoder":
        golden_decoder()
        return
    if args.only == "sam_forward":
        golden_sam_forward()
        return
    if args.only == "amg":
        golden_amg()
        return
    from functools import partial

    import segment_anything_fast as saf
    from segment_anything_fast.flash_4 import _attention_rel_h_rel_w
    from segment_anything_fast.modeling.image_encoder import ImageEncoderViT, add_decomposed_rel_pos
    from segment_anything_fast.sparse import apply_fake_sparsity

    from oracle import encoder_oracle as eo

    torch.set_grad_enabled(False)

    # (a) tiny encoder, seeded non-zero rel-pos / pos-embed, fp32 -------------------------
    cfg = eo.EncoderConfig(**TINY)
    ref = ImageEncoderViT(
        depth=cfg.depth, embed_dim=cfg.embed_dim, img_size=1024, mlp_ratio=4,
        norm_layer=partial(torch.nn.LayerNorm, eps=1e-6), num_heads=cfg.num_heads, patch_size=16,
        qkv_bias=True, use_rel_pos=True, global_attn_indexes=list(cfg.global_attn_indexes),
        window_size=14, out_chans=cfg.out_chans).eval()
    sd = eo.seeded_state_dict(cfg, seed=1)
    ref.load_state_dict(sd)                      # also proves the key set / shapes agree
    x = eo.seeded_images(1, seed=2)
    taps = {}
    hooks = [blk.register_forward_hook(lambda m, i, o, n=n: taps.__setitem__(n, o))
             for n, blk in enumerate(ref.blocks)]
    out = ref(x)
    for h in hooks:
        h.remove()
    np.savez_compressed(
        os.path.join(HERE, "enc_tiny_fp32.npz"),
        out=out[:, :, ::2, ::2].numpy(),
        **{f"block{n}": t[0, ::8, ::8, :].numpy() for n, t in taps.items()})
    # the same model through the reference's bf16 module path on CPU (noise-floor record)
    ref_bf = ref.to(torch.bfloat16)
    out_bf = ref_bf(x.to(torch.bfloat16)).float()
    np.savez_compressed(os.path.join(HERE, "enc_tiny_bf16.npz"), out=out_bf[:, :, ::2, ::2].numpy())

    # (b) ViT-B, torch.manual_seed(0) default init through the reference registry ---------
    torch.manual_seed(0)
    sam = saf.sam_model_registry["vit_b"]()
    enc = sam.image_encoder
    xb = eo.seeded_images(1, seed=0)
    outb = enc(xb)
    np.savez_compressed(
        os.path.join(HERE, "enc_vit_b_default_init_fp32.npz"),
        out=outb[:, :, ::4, ::4].numpy(),
        weights_sha256=np.array(sd_digest(enc.state_dict())),
        qkv0_head=enc.state_dict()["blocks.0.attn.qkv.weight"][:4, :8].numpy())

    # (c) the attention op: the procedure of test/test_flash_4.py, on CPU --------------------
    att = {}
    for name, (B, H, N, d, S) in {"global_d80": (1, 2, 4096, 80, 64), "global_d64": (1, 2, 4096, 64, 64),
                                  "window_d80": (3, 2, 196, 80, 14)}.items():
        torch.manual_seed(20)
        q, k, v = (torch.empty(B, H, N, d).normal_(0.0, 0.5) for _ in range(3))
        rel_h = torch.empty(B, H, N, S, 1).normal_(0.0, 0.5)
        rel_w = torch.empty(B, H, N, 1, S).normal_(0.0, 0.5)
        o = _attention_rel_h_rel_w(q, k, v, rel_h, rel_w)
        att[name] = o[:, :, ::(16 if N > 256 else 1), :].numpy()
    np.savez_compressed(os.path.join(HERE, "attention_op_fp32.npz"), **att)

    # (d) decomposed rel-pos --------------------------------------------------------------
    torch.manual_seed(3)
    q = torch.randn(4, 14 * 14, 80)
    rph, rpw = torch.randn(27, 80), torch.randn(27, 80)
    rh, rw = add_decomposed_rel_pos(q, rph, rpw, (14, 14), (14, 14))
    np.savez_compressed(os.path.join(HERE, "rel_pos_fp32.npz"), rel_h=rh.squeeze(-1).numpy(),
                        rel_w=rw.squeeze(-2).numpy())

    # (e) 2:4 mask from the reference's sparsifier flow ------------------------------------
    torch.manual_seed(4)
    lin = torch.nn.Sequential(torch.nn.Linear(64, 48), torch.nn.Linear(48, 32))
    w_before = [m.weight.detach().clone() for m in lin]
    apply_fake_sparsity(lin)
    np.savez_compressed(
        os.path.join(HERE, "sparse24_mask.npz"),
        w0=w_before[0].numpy(), w1=w_before[1].numpy(),
        keep0=(lin[0].weight != 0).numpy(), keep1=(lin[1].weight != 0).numpy())
    golden_decoder()
    golden_amg()
    golden_sam_forward()
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
