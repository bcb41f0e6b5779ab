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
