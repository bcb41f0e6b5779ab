"""End-to-end parity of the B200 image encoder against the CPU oracle on identical seeded weights
and inputs (the oracle itself is pinned to the reference by tests/test_oracle_golden.py)."""
import os
from functools import partial

import numpy as np
import pytest
import torch

from oracle import encoder_oracle as eo

pytestmark = pytest.mark.gpu

TINY = eo.EncoderConfig(embed_dim=160, depth=4, num_heads=2, global_attn_indexes=(1, 3), out_chans=32)


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0).item()


def build_encoder(cfg, sd, quant=None):
    from segment_anything_fast_b200.image_encoder import ImageEncoderViT
    enc = ImageEncoderViT(
        depth=cfg.depth, embed_dim=cfg.embed_dim, img_size=cfg.img_size, mlp_ratio=cfg.mlp_ratio,
        norm_layer=partial(torch.nn.LayerNorm, eps=cfg.ln_eps), num_heads=cfg.num_heads,
        patch_size=cfg.patch_size, qkv_bias=True, use_rel_pos=True,
        global_attn_indexes=cfg.global_attn_indexes, window_size=cfg.window_size, out_chans=cfg.out_chans)
    enc.load_state_dict(sd)
    return enc.eval().to(torch.bfloat16).cuda().set_quant(quant)


@pytest.fixture(scope="module")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from segment_anything_fast_b200 import ops
    return ops


def test_tiny_encoder_stagewise_and_output(cuda, golden_dir):
    sd = eo.seeded_state_dict(TINY, seed=1)
    x = eo.seeded_images(1, seed=2)
    enc = build_encoder(TINY, sd)
    taps = {}
    out = enc(x.to(torch.bfloat16).cuda(), taps=taps).float().cpu()
    cuda.check_status()
    ref_taps = {}
    ref = eo.image_encoder_forward(x, sd, TINY, "fp32", taps=ref_taps)
    for name in ["patch"] + [f"block{i}" for i in range(TINY.depth)]:
        a, b = taps[name].float().cpu(), ref_taps[name]
        err = (a - b).abs().max().item()
        print(f"{name}: max-abs {err:.4f}  ref abs-max {b.abs().max().item():.3f}  cos {_cos(a, b):.6f}")
        assert _cos(a, b) > 0.9995, name
    g32 = torch.from_numpy(np.load(os.path.join(golden_dir, "enc_tiny_fp32.npz"))["out"])
    g16 = torch.from_numpy(np.load(os.path.join(golden_dir, "enc_tiny_bf16.npz"))["out"])
    floor = (g16 - g32).abs().max().item()          # what the reference's own bf16 path loses vs fp32
    err = (out - ref).abs().max().item()
    print(f"output: max-abs {err:.4f} (reference bf16 floor {floor:.4f}), cos {_cos(out, ref):.6f}")
    assert _cos(out, ref) > 0.999
    assert err <= 1.5 * floor
    # and directly against what the real reference produced
    e16 = (out[:, :, ::2, ::2] - g16).abs().max().item()
    e32 = (out[:, :, ::2, ::2] - g32).abs().max().item()
    print(f"vs the reference's stored outputs: bf16 path max-abs {e16:.4f} cos {_cos(out[:, :, ::2, ::2], g16):.6f}; "
          f"fp32 path max-abs {e32:.4f} cos {_cos(out[:, :, ::2, ::2], g32):.6f}")
    assert _cos(out[:, :, ::2, ::2], g32) > 0.999 and _cos(out[:, :, ::2, ::2], g16) > 0.999
    # two independently rounded bf16 evaluations, each `floor` from fp32, can be up to 2 x floor apart
    assert e16 <= 2.0 * floor and e32 <= 1.5 * floor


def test_tiny_encoder_batch_and_determinism(cuda):
    sd = eo.seeded_state_dict(TINY, seed=1)
    enc = build_encoder(TINY, sd)
    x = eo.seeded_images(3, seed=5).to(torch.bfloat16).cuda()
    a = enc(x)
    b = enc(x)
    assert torch.equal(a, b)
    single = enc(x[1:2])
    assert torch.equal(single, a[1:2])            # images are independent units
    cuda.check_status()


def test_tiny_encoder_int8(cuda):
    """int8 dynamic-quant Linears: end-to-end output stays within bf16-level distance of fp32."""
    sd = eo.seeded_state_dict(TINY, seed=1)
    x = eo.seeded_images(1, seed=2)
    enc = build_encoder(TINY, sd, quant="int8")
    out = enc(x.to(torch.bfloat16).cuda()).float().cpu()
    cuda.check_status()
    ref = eo.image_encoder_forward(x, sd, TINY, "fp32")
    sd16 = {k: v.to(torch.bfloat16).float() if v.is_floating_point() else v for k, v in sd.items()}
    ref8 = eo.image_encoder_forward(x, sd16, TINY, "int8")
    floor = (ref8 - ref).abs().max().item()
    print(f"int8 output: vs fp32 max-abs {(out - ref).abs().max().item():.4f} cos {_cos(out, ref):.6f}; vs int8 oracle "
          f"max-abs {(out - ref8).abs().max().item():.4f} cos {_cos(out, ref8):.6f}; int8 oracle vs fp32 max-abs {floor:.4f}")
    assert _cos(out, ref) > 0.995 and _cos(out, ref8) > 0.999
    assert (out - ref8).abs().max().item() <= 2.0 * floor


def test_cpu_input_is_rejected(cuda):
    sd = eo.seeded_state_dict(TINY, seed=1)
    enc = build_encoder(TINY, sd)
    with pytest.raises(RuntimeError):
        enc(torch.zeros(1, 3, 1024, 1024))


def _pruned_state_dict(sd, mlp_only):
    from oracle import quant_oracle as qo
    out = {}
    for k, v in sd.items():
        is_lin = v.dim() == 2 and k.endswith(".weight") and (".attn.qkv" in k or ".attn.proj" in k or ".mlp.lin" in k)
        if is_lin and (not mlp_only or ".mlp.lin" in k):
            v = v * qo.prune_2_4_mask(v).to(v.dtype)
        out[k] = v
    return out


@pytest.mark.parametrize("mlp_only,quant", [(False, None), (True, "int8")])
def test_tiny_encoder_sparse24(cuda, mlp_only, quant):
    """apply_sparse prunes the same entries as the oracle's 2:4 mask; the pruned encoder matches the
    oracle run on the pruned weights (bf16 tolerance; int8 adds its quantisation error)."""
    from segment_anything_fast_b200.sparse import apply_sparse
    sd = eo.seeded_state_dict(TINY, seed=1)
    x = eo.seeded_images(1, seed=2)
    enc = build_encoder(TINY, sd, quant=quant)
    dense = enc(x.to(torch.bfloat16).cuda()).float().cpu()
    apply_sparse(enc, mlp_only=mlp_only)
    sd_bf16 = {k: v.to(torch.bfloat16).float() if v.is_floating_point() else v for k, v in sd.items()}
    ref_sd = _pruned_state_dict(sd_bf16, mlp_only)
    for k, v in enc.state_dict().items():
        if k.endswith("lin1.weight") or (not mlp_only and k.endswith("qkv.weight")):
            assert torch.equal(v.float().cpu() != 0, ref_sd[k] != 0), k
            assert ((v != 0).reshape(v.shape[0], -1, 4).sum(-1) <= 2).all()
    out = enc(x.to(torch.bfloat16).cuda()).float().cpu()       # weights changed in place: repacked
    cuda.check_status()
    ref = eo.image_encoder_forward(x, ref_sd, TINY, "fp32")
    print(f"sparse mlp_only={mlp_only} quant={quant}: cos vs pruned oracle {_cos(out, ref):.6f}, "
          f"cos vs dense output {_cos(out, dense):.6f}")
    assert _cos(out, ref) > (0.995 if quant else 0.999)
    assert _cos(out, dense) < _cos(out, ref)                    # the pruning really took effect


def test_encoder_session_blocking_and_pipelined_agree(cuda):
    """EncoderSession: host uint8 in, host bf16 embeddings out.  The pipelined form (two batches in flight, copies
    on their own streams) returns bit for bit what the blocking form returns, batch after batch."""
    from segment_anything_fast_b200 import EncoderSession
    sd = eo.seeded_state_dict(TINY, seed=1)
    enc = build_encoder(TINY, sd)
    sess = EncoderSession(enc, batch=2)
    g = torch.Generator().manual_seed(31)
    batches = [torch.randint(0, 256, (2, 3, 1024, 1024), generator=g, dtype=torch.uint8) for _ in range(4)]
    want = [sess.encode(b).clone() for b in batches]
    got, pending = [], None
    for b in batches:
        slot = sess.submit(b)
        if pending is not None:
            got.append(sess.result(pending).clone())
        pending = slot
    got.append(sess.result(pending).clone())
    cuda.check_status()
    for a, b in zip(want, got):
        assert torch.equal(a, b)
    with pytest.raises(RuntimeError):
        sess.result(0)                                   # nothing in flight any more


def test_encoder_session_graph_replay_matches_eager(cuda):
    """EncoderSession(graph=True) records the normalise + encoder launches once per staging buffer and replays
    them: blocking and pipelined results are bit for bit those of the eager session."""
    from segment_anything_fast_b200 import EncoderSession
    sd = eo.seeded_state_dict(TINY, seed=1)
    enc = build_encoder(TINY, sd)
    eager = EncoderSession(enc, batch=2)
    graph = EncoderSession(enc, batch=2, graph=True)
    g = torch.Generator().manual_seed(32)
    batches = [torch.randint(0, 256, (2, 3, 1024, 1024), generator=g, dtype=torch.uint8) for _ in range(5)]
    want = [eager.encode(b).clone() for b in batches]
    for b, w in zip(batches[:2], want[:2]):
        assert torch.equal(graph.encode(b), w)
    got, pending = [], None
    for b in batches:
        slot = graph.submit(b)
        if pending is not None:
            got.append(graph.result(pending).clone())
        pending = slot
    got.append(graph.result(pending).clone())
    cuda.check_status()
    assert len(graph._graphs) == 2                       # one recording per device staging buffer
    for a, b in zip(want, got):
        assert torch.equal(a, b)
