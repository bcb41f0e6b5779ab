"""The CPU oracle restatement against vectors produced by the real reference
(tests/golden/make_golden.py).  Runs without a GPU."""
import os

import numpy as np
import torch

from oracle import encoder_oracle as eo
from oracle import quant_oracle as qo

TINY = eo.EncoderConfig(embed_dim=160, depth=4, num_heads=2, global_attn_indexes=(1, 3), out_chans=32)


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_tiny_encoder_fp32_matches_reference(golden_dir):
    g = _load(golden_dir, "enc_tiny_fp32.npz")
    sd = eo.seeded_state_dict(TINY, seed=1)
    x = eo.seeded_images(1, seed=2)
    taps = {}
    out = eo.image_encoder_forward(x, sd, TINY, "fp32", taps=taps)
    for n in range(TINY.depth):
        ref = torch.from_numpy(g[f"block{n}"])
        torch.testing.assert_close(taps[f"block{n}"][0, ::8, ::8, :], ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(out[:, :, ::2, ::2], torch.from_numpy(g["out"]), rtol=1e-3, atol=1e-3)


def test_tiny_encoder_bf16_model_tracks_reference_bf16(golden_dir):
    """The bf16 rounding model is a noise model, not bit parity: it has to sit as
    close to the reference's bf16 module path as that path sits to fp32."""
    g32 = torch.from_numpy(_load(golden_dir, "enc_tiny_fp32.npz")["out"])
    g16 = torch.from_numpy(_load(golden_dir, "enc_tiny_bf16.npz")["out"])
    sd = eo.seeded_state_dict(TINY, seed=1)
    x = eo.seeded_images(1, seed=2)
    out = eo.image_encoder_forward(x, sd, TINY, "bf16")[:, :, ::2, ::2]
    floor = (g16 - g32).abs().max().item()
    assert (out - g16).abs().max().item() <= 2.0 * floor + 1e-3
    cos = torch.nn.functional.cosine_similarity(out.flatten(), g16.flatten(), dim=0).item()
    assert cos > 0.999


def test_attention_op_matches_reference(golden_dir):
    g = _load(golden_dir, "attention_op_fp32.npz")
    for name, (B, H, N, d, S) in {"global_d80": (1, 2, 4096, 80, 64), "global_d64": (1, 2, 4096, 64, 64),
                                  "window_d80": (3, 2, 196, 80, 14)}.items():
        torch.manual_seed(20)
        q, k, v = (torch.empty(B, H, N, d).normal_(0.0, 0.5) for _ in range(3))
        rel_h = torch.empty(B, H, N, S, 1).normal_(0.0, 0.5)
        rel_w = torch.empty(B, H, N, 1, S).normal_(0.0, 0.5)
        o = eo.attention_rel_h_rel_w(q, k, v, rel_h.squeeze(-1), rel_w.squeeze(-2))
        o = o[:, :, ::(16 if N > 256 else 1), :]
        torch.testing.assert_close(o, torch.from_numpy(g[name]), rtol=1e-4, atol=1e-5)


def test_decomposed_rel_pos_matches_reference(golden_dir):
    g = _load(golden_dir, "rel_pos_fp32.npz")
    torch.manual_seed(3)
    q = torch.randn(4, 14 * 14, 80)
    rph, rpw = torch.randn(27, 80), torch.randn(27, 80)
    rh, rw = eo.decomposed_rel_pos(q, rph, rpw, (14, 14))
    torch.testing.assert_close(rh, torch.from_numpy(g["rel_h"]), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(rw, torch.from_numpy(g["rel_w"]), rtol=1e-5, atol=1e-5)


def test_window_partition_roundtrip_and_padding():
    x = torch.arange(2 * 64 * 64 * 3, dtype=torch.float32).reshape(2, 64, 64, 3) + 1.0
    win, pad_hw = eo.window_partition(x, 14)
    assert win.shape == (2 * 25, 14, 14, 3) and pad_hw == (70, 70)
    # last window of each image: only its top-left 8x8 corner is real
    assert (win[24, 8:, :, :] == 0).all() and (win[24, :, 8:, :] == 0).all()
    assert (win[24, :8, :8, :] == x[0, 56:, 56:, :]).all()
    back = eo.window_unpartition(win, 14, pad_hw, (64, 64))
    assert torch.equal(back, x)


def test_sparse24_mask_matches_reference_sparsifier(golden_dir):
    g = _load(golden_dir, "sparse24_mask.npz")
    for i in (0, 1):
        keep = qo.prune_2_4_mask(torch.from_numpy(g[f"w{i}"]))
        assert torch.equal(keep, torch.from_numpy(g[f"keep{i}"]))
        assert (keep.reshape(keep.shape[0], -1, 4).sum(-1) == 2).all()


def test_int8_accumulator_is_exact_and_matches_int_mm():
    torch.manual_seed(0)
    x = torch.randn(64, 256).to(torch.bfloat16).float()
    w = torch.randn(48, 256) * 0.02
    xq, sx = qo.quantize_rows_absmax(x)
    wq, sw = qo.quantize_rows_absmax(w)
    acc = qo.int8_matmul_i32(xq, wq)
    ref = torch._int_mm(xq, wq.t().contiguous())
    assert torch.equal(acc, ref)
    assert xq.abs().max() <= 127 and (xq.abs().amax(dim=1) == 127).all()
    # all-zero rows (zero-padded window tokens) must not divide by zero
    z, sz = qo.quantize_rows_absmax(torch.zeros(2, 16))
    assert torch.equal(z, torch.zeros(2, 16, dtype=torch.int8)) and torch.isfinite(sz).all()
    y = qo.int8_linear(x, w, torch.zeros(48))
    full = x @ w.t()
    assert (y - full).abs().max() < 0.05 * full.abs().max()


def test_decoder_oracle_matches_reference_modules(golden_dir):
    """Prompt encoder, two-way transformer mask decoder and post-processing restatement against the
    outputs of the reference's own modules on the same seeded weights."""
    from oracle import decoder_oracle as do
    g = _load(golden_dir, "decoder_fp32.npz")
    cfg = do.DecoderConfig()
    sd = do.seeded_state_dict(cfg, seed=3)
    emb = torch.randn(1, 256, 64, 64, generator=torch.Generator().manual_seed(5))
    boxes = torch.from_numpy(g["boxes"])
    sparse, _ = do.prompt_encoder_forward(sd, cfg, boxes=boxes)
    assert torch.allclose(sparse, torch.from_numpy(g["sparse"]), atol=1e-5)
    assert torch.allclose(do.dense_pe(sd, cfg)[:, :, ::8, ::8], torch.from_numpy(g["dense_pe"]), atol=1e-5)
    pts = (torch.tensor([[[500.0, 300.0], [100.0, 100.0]]]), torch.tensor([[1, 0]]))
    sp_pts, _ = do.prompt_encoder_forward(sd, cfg, points=pts)
    assert torch.allclose(sp_pts, torch.from_numpy(g["sparse_points"]), atol=1e-5)
    masks, iou, low = do.predict_masks_from_embedding(sd, cfg, emb, boxes)
    low_ref = torch.from_numpy(g["low"])
    assert (low[:, :, ::4, ::4] - low_ref).abs().max().item() < 1e-3 * low_ref.abs().max().item()
    assert torch.allclose(iou, torch.from_numpy(g["iou"]), atol=1e-4)
    area = masks.float().mean((2, 3))
    assert torch.allclose(area, torch.from_numpy(g["area"]), atol=1e-4)


def test_amg_oracle_matches_reference_functions(golden_dir):
    """Stability score, mask boxes and run-length encoding restatements against the outputs of the reference's
    own functions on the same seeded logits (integer exact); the encoding decodes back to the mask."""
    from oracle import amg_oracle as ao
    g = _load(golden_dir, "amg_fp32.npz")
    logits = g["logits"]
    score = ao.calculate_stability_score(logits, 0.0, 1.0)
    assert np.array_equal(np.nan_to_num(score, nan=-1), np.nan_to_num(g["score"], nan=-1))
    masks = logits > 0
    assert np.array_equal(ao.batched_mask_to_box(masks), g["boxes"])
    rles = ao.mask_to_rle(masks)
    assert [len(r["counts"]) for r in rles] == g["rle_len"].tolist()
    assert np.array_equal(np.concatenate([np.asarray(r["counts"]) for r in rles]), g["rle_counts"])
    for r, m in zip(rles, masks):
        assert r["size"] == list(m.shape) and sum(r["counts"]) == m.size
        assert np.array_equal(ao.rle_to_mask(r), m)


def test_amg_crop_edge_filter_and_batch_filters(golden_dir):
    """``is_box_near_crop_edge`` against the reference's output on seeded boxes, and the step-by-step
    ``process_batch_filters`` restatement against a direct evaluation of its three predicates."""
    import numpy as np
    from oracle import amg_oracle as ao
    g = _load(golden_dir, "amg_fp32.npz")
    got = ao.is_box_near_crop_edge(g["edge_boxes"], g["edge_crop"].tolist(), g["edge_orig"].tolist())
    assert np.array_equal(got, g["edge_out"]) and 0 < got.sum() < len(got)
    rng = np.random.default_rng(3)
    logits = np.repeat(np.repeat(rng.normal(0, 4, (5, 3, 6, 6)), 10, axis=2), 10, axis=3).astype(np.float32)
    iou = rng.uniform(0.7, 1.0, (5, 3)).astype(np.float32)
    crop, orig = [20, 10, 80, 70], (70, 100)
    idx, score, boxes, masks = ao.process_batch_filters(logits, iou, crop, orig, 0.8, 0.0, 1.0, 0.5)
    flat = logits.reshape(15, 60, 60)
    s_all = ao.calculate_stability_score(flat, 0.0, 1.0)
    b_all = ao.batched_mask_to_box(flat > 0)
    keep = (iou.reshape(-1) > 0.8) & (s_all >= 0.5) & ~ao.is_box_near_crop_edge(b_all, crop, [0, 0, 100, 70])
    assert np.array_equal(idx, np.flatnonzero(keep))
    assert np.array_equal(score, s_all[keep]) and np.array_equal(boxes, b_all[keep]) and np.array_equal(masks, (flat > 0)[keep])
