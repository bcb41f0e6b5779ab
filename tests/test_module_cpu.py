"""CPU checks of the host-side mirror of the reference interface: parameter names/shapes, default
initialisation stream, and the loud failure on CPU tensors."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import encoder_oracle as eo


def _digest(sd):
    h = hashlib.sha256()
    for k in sorted(sd):
        h.update(k.encode())
        h.update(sd[k].detach().to(torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


def test_state_dict_keys_and_shapes_match_the_reference_layout():
    from segment_anything_fast_b200 import build_image_encoder_vit_b
    enc = build_image_encoder_vit_b()
    sd = enc.state_dict()
    want = eo.state_dict_keys(eo.VIT_B)
    assert set(sd) == set(want)
    for k, shape in want.items():
        assert tuple(sd[k].shape) == shape, k
    assert enc.img_size == 1024


def test_default_init_reproduces_the_reference_weights(golden_dir):
    """torch.manual_seed(0) + construction draws the same parameters as the reference registry did
    when the golden file was made (same modules, same creation order)."""
    from segment_anything_fast_b200 import build_image_encoder_vit_b
    g = np.load(os.path.join(golden_dir, "enc_vit_b_default_init_fp32.npz"))
    torch.manual_seed(0)
    enc = build_image_encoder_vit_b()
    sd = enc.state_dict()
    np.testing.assert_array_equal(sd["blocks.0.attn.qkv.weight"][:4, :8].numpy(), g["qkv0_head"])
    assert _digest(sd) == str(g["weights_sha256"])


def test_oracle_vit_b_default_init_matches_reference_output(golden_dir):
    """BASELINE configuration 1 (ViT-B, fp32, CPU, batch 1, default init, seeded image): the oracle
    on these weights reproduces the reference's stored output."""
    from segment_anything_fast_b200 import build_image_encoder_vit_b
    g = np.load(os.path.join(golden_dir, "enc_vit_b_default_init_fp32.npz"))
    torch.manual_seed(0)
    sd = build_image_encoder_vit_b().state_dict()
    out = eo.image_encoder_forward(eo.seeded_images(1, seed=0), sd, eo.VIT_B, "fp32")
    torch.testing.assert_close(out[:, :, ::4, ::4], torch.from_numpy(g["out"]), rtol=2e-3, atol=2e-3)


def test_cpu_tensors_fail_loudly():
    from segment_anything_fast_b200 import ImageEncoderViT
    enc = ImageEncoderViT(depth=1, embed_dim=160, num_heads=2, use_rel_pos=True, window_size=14, out_chans=32)
    with pytest.raises(RuntimeError):
        enc(torch.zeros(1, 3, 1024, 1024))


def test_quant_mode_validation():
    from segment_anything_fast_b200 import ImageEncoderViT
    enc = ImageEncoderViT(depth=1, embed_dim=160, num_heads=2, use_rel_pos=True, window_size=14, out_chans=32)
    with pytest.raises(ValueError):
        enc.set_quant("fp4")
    assert enc.set_quant("int8").quant == "int8"


def test_sparse_prune_matches_reference_sparsifier(golden_dir):
    """The package's 2:4 pruning keeps exactly what the reference's sparsifier flow kept (golden masks
    made by running the reference's apply_fake_sparsity)."""
    import numpy as np
    import os
    from segment_anything_fast_b200.sparse import apply_sparse, prune_2_4_
    g = np.load(os.path.join(golden_dir, "sparse24_mask.npz"))
    for i in (0, 1):
        w = torch.from_numpy(g[f"w{i}"]).clone()
        keep = prune_2_4_(w)
        assert torch.equal(keep, torch.from_numpy(g[f"keep{i}"]))
        assert torch.equal(w != 0, keep)
    m = torch.nn.Sequential(torch.nn.Linear(16, 8), torch.nn.ReLU(), torch.nn.Linear(8, 4))
    apply_sparse(m)
    for lin in (m[0], m[2]):
        assert ((lin.weight != 0).reshape(lin.weight.shape[0], -1, 4).sum(-1) <= 2).all()


def test_sam_heads_match_decoder_oracle_and_reference_keys(golden_dir):
    """The package's prompt encoder / mask decoder modules: reference key set, and the same numbers as the
    decoder oracle (itself pinned to the reference modules) on seeded weights."""
    import numpy as np
    import os
    from oracle import decoder_oracle as do
    from segment_anything_fast_b200.sam_heads import build_heads
    cfg = do.DecoderConfig()
    sd = do.seeded_state_dict(cfg, seed=3)
    pe, md = build_heads()
    keys = {"prompt_encoder." + k for k in pe.state_dict()} | {"mask_decoder." + k for k in md.state_dict()}
    extra = {k for k in keys - set(sd) if "mask_downscaling" not in k}
    assert not extra and not (set(sd) - keys)
    pe.load_state_dict({k[len("prompt_encoder."):]: v for k, v in sd.items() if k.startswith("prompt_encoder.")}, strict=False)
    md.load_state_dict({k[len("mask_decoder."):]: v for k, v in sd.items() if k.startswith("mask_decoder.")})
    g = np.load(os.path.join(golden_dir, "decoder_fp32.npz"))
    emb = torch.randn(1, 256, 64, 64, generator=torch.Generator().manual_seed(5))
    boxes = torch.from_numpy(g["boxes"])
    with torch.no_grad():
        sparse, dense = pe(None, boxes)
        low, iou = md(emb, pe.get_dense_pe(), sparse, dense, True)
        pts = (torch.tensor([[[500.0, 300.0], [100.0, 100.0]]]), torch.tensor([[1, 0]]))
        sp_pts, _ = pe(pts, None)
    assert torch.allclose(sparse, torch.from_numpy(g["sparse"]), atol=1e-5)
    assert torch.allclose(sp_pts, torch.from_numpy(g["sparse_points"]), atol=1e-5)
    low_ref = torch.from_numpy(g["low"])
    assert (low[:, :, ::4, ::4] - low_ref).abs().max().item() < 1e-3 * low_ref.abs().max().item()
    assert torch.allclose(iou, torch.from_numpy(g["iou"]), atol=1e-4)
    _, _, low_o = do.predict_masks_from_embedding(sd, cfg, emb, boxes)
    assert (low - low_o).abs().max().item() < 1e-3 * low_o.abs().max().item()
