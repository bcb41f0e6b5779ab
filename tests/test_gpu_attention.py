"""GPU parity of the relative-position attention kernels (through the C ABI) against the CPU oracle."""
import math

import pytest
import torch

from oracle import encoder_oracle as eo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from segment_anything_fast_b200 import ops as _ops
    return _ops


def _inputs(B, H, N, d, S_h, S_w, std_qkv, std_rel, seed):
    torch.manual_seed(seed)
    q, k, v = (torch.empty(B, H, N, d).normal_(0.0, std_qkv).bfloat16() for _ in range(3))
    rel_h = torch.empty(B, H, N, S_h).normal_(0.0, std_rel).bfloat16()
    rel_w = torch.empty(B, H, N, S_w).normal_(0.0, std_rel).bfloat16()
    return q, k, v, rel_h, rel_w


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0).item()


@pytest.mark.parametrize("B,H,N,d", [(1, 2, 4096, 80), (2, 3, 4096, 64), (1, 1, 256, 80), (3, 2, 1024, 80)])
def test_global_attention_reference_procedure(ops, B, H, N, d):
    """The procedure of the reference's own op test: seed 20, N(0, 0.5) inputs, atol = rtol = 1e-3."""
    q, k, v, rel_h, rel_w = _inputs(B, H, N, d, N // 64, 64, 0.5, 0.5, 20)
    ref = eo.attention_rel_h_rel_w(q.float(), k.float(), v.float(), rel_h.float(), rel_w.float())
    out = ops.attn_relpos_global(q.cuda(), k.cuda(), v.cuda(), rel_h.cuda(), rel_w.cuda())
    ops.check_status()
    torch.testing.assert_close(out.float().cpu(), ref, rtol=1e-3, atol=1e-3)


def test_global_attention_unit_variance_inputs(ops):
    """Benchmark-configuration distributions: q, k, v ~ N(0,1), rel ~ N(0,0.5); bf16 tolerance
    max-abs 2e-2 and cosine >= 0.999."""
    q, k, v, rel_h, rel_w = _inputs(2, 4, 4096, 80, 64, 64, 1.0, 0.5, 0)
    ref = eo.attention_rel_h_rel_w(q.float(), k.float(), v.float(), rel_h.float(), rel_w.float())
    out = ops.attn_relpos_global(q.cuda(), k.cuda(), v.cuda(), rel_h.cuda(), rel_w.cuda()).float().cpu()
    ops.check_status()
    assert (out - ref).abs().max().item() < 2e-2
    assert _cos(out, ref) > 0.999


def test_global_attention_is_deterministic(ops):
    q, k, v, rel_h, rel_w = (t.cuda() for t in _inputs(1, 2, 2048, 80, 32, 64, 1.0, 0.5, 3))
    a = ops.attn_relpos_global(q, k, v, rel_h, rel_w)
    b = ops.attn_relpos_global(q, k, v, rel_h, rel_w)
    assert torch.equal(a, b)


@pytest.mark.parametrize("B,H,d", [(2, 2, 80), (1, 3, 64)])
def test_global_attention_fused_qkv_layout(ops, B, H, d):
    """q/k/v read from the head-major qkv projection buffer, bias from the q . rel_pos table products."""
    N, S = 4096, 64
    torch.manual_seed(7)
    qkv = torch.empty(B * N, 3 * H * d).normal_(0.0, 1.0).bfloat16()
    rph = torch.empty(2 * S - 1, d).normal_(0.0, 0.1).bfloat16()
    rpw = torch.empty(2 * S - 1, d).normal_(0.0, 0.1).bfloat16()
    t = qkv.float().reshape(B, N, 3, H, d).permute(2, 0, 3, 1, 4)
    q, k, v = (t[i].reshape(B * H, N, d) for i in range(3))
    rel_h, rel_w = eo.decomposed_rel_pos(q, rph.float(), rpw.float(), (S, S))
    rel_h, rel_w = rel_h.bfloat16().float(), rel_w.bfloat16().float()
    ref = eo.attention_rel_h_rel_w(q, k, v, rel_h, rel_w)                       # [B*H, N, d]
    ref = ref.reshape(B, H, N, d).permute(0, 2, 1, 3).reshape(B * N, H * d)
    # table products: per head [127 rel_pos_h | pad | 127 rel_pos_w (pre-divided by scale) | pad] = 256 columns
    tables = torch.zeros(256, d, dtype=torch.bfloat16)
    tables[:127], tables[128:255] = rph, rpw
    col_scale = torch.ones(256)
    col_scale[128:] = math.sqrt(d)
    qkv_hm = qkv.reshape(B * N, 3 * H, d).permute(1, 0, 2).contiguous().cuda()         # [3H, B*N, d] planes
    tab = ops.relpos_table_products(qkv_hm, tables.cuda(), col_scale.cuda(), H)
    qh = qkv.float().reshape(B * N, 3, H, d)[:, 0]                                # [B*N, H, d]
    tab_ref = torch.einsum("nhc,mc->nhm", qh, tables.float()) * col_scale
    torch.testing.assert_close(tab.float().cpu().view(B * N, H, 256), tab_ref, rtol=1e-2, atol=1e-2)
    out = ops.attn_relpos_global_qkv(qkv_hm, tab, 256, 128, B, H, N, d).float().cpu()
    ops.check_status()
    assert (out - ref).abs().max().item() < 2e-2
    assert _cos(out, ref) > 0.999
    # the same with the products computed inside the attention kernel from the tables (no product tensor at all)
    fused = ops.attn_relpos_global_tables(qkv_hm, tables.cuda(), B, H, N, d).float().cpu()
    ops.check_status()
    print(f"in-kernel table products: max-abs vs oracle {(fused - ref).abs().max().item():.4f}, "
          f"vs the stored-product path {(fused - out).abs().max().item():.5f}")
    assert (fused - ref).abs().max().item() < 2e-2
    assert _cos(fused, ref) > 0.999
    assert (fused - out).abs().max().item() < 4e-3        # same roundings; only the accumulation order may differ


@pytest.mark.parametrize("B,H,d,N", [(1, 2, 80, 1024), (2, 1, 64, 256)])
def test_global_attention_in_kernel_tables_small_rasters(ops, B, H, d, N):
    """Shorter rasters (16 and 4 rows of 64 tokens): the table block holds 2*N/64 - 1 rel_pos_h rows."""
    S_h = N // 64
    torch.manual_seed(N)
    qkv = torch.empty(B * N, 3 * H * d).normal_(0.0, 1.0).bfloat16()
    rph = torch.empty(2 * S_h - 1, d).normal_(0.0, 0.1).bfloat16()
    rpw = torch.empty(127, d).normal_(0.0, 0.1).bfloat16()
    t = qkv.float().reshape(B, N, 3, H, d).permute(2, 0, 3, 1, 4)
    q, k, v = (t[i].reshape(B * H, N, d) for i in range(3))
    rel_h, rel_w = eo.decomposed_rel_pos(q, rph.float(), rpw.float(), (S_h, 64))
    ref = eo.attention_rel_h_rel_w(q, k, v, rel_h.bfloat16().float(), rel_w.bfloat16().float())
    ref = ref.reshape(B, H, N, d).permute(0, 2, 1, 3).reshape(B * N, H * d)
    tables = torch.zeros(256, d, dtype=torch.bfloat16)
    tables[:2 * S_h - 1], tables[128:255] = rph, rpw
    qkv_hm = qkv.reshape(B * N, 3 * H, d).permute(1, 0, 2).contiguous().cuda()
    out = ops.attn_relpos_global_tables(qkv_hm, tables.cuda(), B, H, N, d).float().cpu()
    ops.check_status()
    assert (out - ref).abs().max().item() < 2e-2
    assert _cos(out, ref) > 0.999


@pytest.mark.parametrize("B,H,d,std", [(3, 2, 80, 0.5), (25, 4, 80, 1.0), (2, 3, 64, 1.0)])
def test_window_attention_op(ops, B, H, d, std):
    """14x14 windows (N = 196): the composite the reference falls back to for the windowed blocks."""
    q, k, v, rel_h, rel_w = _inputs(B, H, 196, d, 14, 14, std, 0.5, 20)
    ref = eo.attention_rel_h_rel_w(q.float(), k.float(), v.float(), rel_h.float(), rel_w.float())
    out = ops.attn_relpos_window(q.cuda(), k.cuda(), v.cuda(), rel_h.cuda(), rel_w.cuda()).float().cpu()
    ops.check_status()
    assert (out - ref).abs().max().item() < 2e-2
    assert _cos(out, ref) > 0.999
    if std == 0.5:
        torch.testing.assert_close(out, ref, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("B,H,d,grid", [(2, 2, 80, 64), (1, 3, 64, 32)])
def test_window_attention_fused_layout_with_padding(ops, B, H, d, grid):
    """Window-ordered, zero-padded qkv rows in; raster-order tokens out (pad queries dropped, pad keys live)."""
    ws, C = 14, H * d
    nw = -(-grid // ws)
    torch.manual_seed(11)
    # what the qkv projection of zero-padded LayerNorm rows looks like: pad rows carry the bias only
    x = torch.empty(B, grid, grid, 3 * C).normal_(0.0, 1.0).bfloat16().float()
    bias = torch.empty(3 * C).normal_(0.0, 0.5).bfloat16().float()
    win, _ = eo.window_partition(x, ws)                                   # zeros at pads
    pad = (win.abs().sum(-1, keepdim=True) == 0).float()
    qkv = (win + pad * bias).reshape(-1, 3 * C)                           # [B*nw*nw*196, 3C]
    rph = torch.empty(2 * ws - 1, d).normal_(0.0, 0.1).bfloat16().float()
    rpw = torch.empty(2 * ws - 1, d).normal_(0.0, 0.1).bfloat16().float()
    W, N = B * nw * nw, ws * ws
    t = qkv.reshape(W, N, 3, H, d).permute(2, 0, 3, 1, 4)
    q, k, v = (t[i].reshape(W * H, N, d) for i in range(3))
    rel_h, rel_w = eo.decomposed_rel_pos(q, rph, rpw, (ws, ws))
    rel_h, rel_w = rel_h.bfloat16().float(), rel_w.bfloat16().float()
    o = eo.attention_rel_h_rel_w(q, k, v, rel_h, rel_w).reshape(W, H, ws, ws, d).permute(0, 2, 3, 1, 4)
    ref = eo.window_unpartition(o.reshape(W, ws, ws, C), ws, (nw * ws, nw * ws), (grid, grid)).reshape(-1, C)
    tables = torch.zeros(64, d, dtype=torch.bfloat16)
    tables[:27], tables[32:59] = rph.bfloat16(), rpw.bfloat16()
    col_scale = torch.ones(64)
    col_scale[32:] = math.sqrt(d)
    qkv_hm = qkv.bfloat16().reshape(W * N, 3 * H, d).permute(1, 0, 2).contiguous().cuda()   # [3H, W*N, d] planes
    tab = ops.relpos_table_products(qkv_hm, tables.cuda(), col_scale.cuda(), H)
    out = ops.attn_relpos_window_qkv(qkv_hm, tab, 64, 32, B, H, grid, ws, d)
    ops.check_status()
    out = out.float().cpu()
    assert (out - ref).abs().max().item() < 2e-2
    assert _cos(out, ref) > 0.999


@pytest.mark.parametrize("B,H,d,grid", [(2, 2, 80, 64), (1, 3, 64, 32), (1, 2, 80, 28), (3, 1, 80, 64)])
def test_window_attention_raster_layout(ops, B, H, d, grid):
    """Raster-order qkv in (no padded copy of the tokens): border windows take the projection bias as the
    key / value of their pad tokens, exactly as the zero-padded, window-partitioned reference does."""
    ws, C = 14, H * d
    nw = -(-grid // ws)
    torch.manual_seed(11)
    x = torch.empty(B, grid, grid, 3 * C).normal_(0.0, 1.0).bfloat16().float()      # qkv of the real tokens
    bias = torch.empty(3 * C).normal_(0.0, 0.5).bfloat16().float()
    # reference: partition, pad rows carry the bias only (the projection of a zero row)
    xp = torch.nn.functional.pad(x, (0, 0, 0, nw * ws - grid, 0, nw * ws - grid), value=float("nan"))
    win, _ = eo.window_partition(xp, ws)
    qkv = torch.where(torch.isnan(win), bias.expand_as(win), win).reshape(-1, 3 * C)
    rph = torch.empty(2 * ws - 1, d).normal_(0.0, 0.1).bfloat16().float()
    rpw = torch.empty(2 * ws - 1, d).normal_(0.0, 0.1).bfloat16().float()
    W, N = B * nw * nw, ws * ws
    t = qkv.reshape(W, N, 3, H, d).permute(2, 0, 3, 1, 4)
    q, k, v = (t[i].reshape(W * H, N, d) for i in range(3))
    rel_h, rel_w = eo.decomposed_rel_pos(q, rph, rpw, (ws, ws))
    rel_h, rel_w = rel_h.bfloat16().float(), rel_w.bfloat16().float()
    o = eo.attention_rel_h_rel_w(q, k, v, rel_h, rel_w).reshape(W, H, ws, ws, d).permute(0, 2, 3, 1, 4)
    ref = eo.window_unpartition(o.reshape(W, ws, ws, C), ws, (nw * ws, nw * ws), (grid, grid)).reshape(-1, C)
    tables = torch.zeros(64, d, dtype=torch.bfloat16)
    tables[:27], tables[32:59] = rph.bfloat16(), rpw.bfloat16()
    col_scale = torch.ones(64)
    col_scale[32:] = math.sqrt(d)
    qkv_hm = x.bfloat16().reshape(B * grid * grid, 3 * H, d).permute(1, 0, 2).contiguous().cuda()   # raster planes
    tab = ops.relpos_table_products(qkv_hm, tables.cuda(), col_scale.cuda(), H)
    out = ops.attn_relpos_window_raster(qkv_hm, bias.bfloat16().cuda(), tab, 64, 32, B, H, grid, ws, d)
    ops.check_status()
    out = out.float().cpu()
    print(f"raster window attention grid {grid}: max-abs {(out - ref).abs().max().item():.4f} cos {_cos(out, ref):.6f}")
    assert (out - ref).abs().max().item() < 2e-2
    assert _cos(out, ref) > 0.999
    # the same with the products computed inside the attention kernel from the tables (no product tensor at all)
    fused = ops.attn_relpos_window_tables(qkv_hm, bias.bfloat16().cuda(), tables.cuda(), B, H, grid, ws, d).float().cpu()
    ops.check_status()
    print(f"in-kernel table products: max-abs vs oracle {(fused - ref).abs().max().item():.4f}, "
          f"vs the stored-product path {(fused - out).abs().max().item():.5f}")
    assert (fused - ref).abs().max().item() < 2e-2
    assert _cos(fused, ref) > 0.999
    assert (fused - out).abs().max().item() < 4e-3        # same roundings; only the accumulation order may differ
