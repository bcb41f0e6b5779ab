"""GPU parity of the individual kernels, called through the C ABI, against the CPU oracle /
a float32 restatement of the same op on identical seeded inputs."""
import pytest
import torch

from oracle import quant_oracle as qo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from segment_anything_fast_b200 import ops as _ops
    return _ops


def _bf16(t):
    return t.to(torch.bfloat16)


def test_bounded_wait_gives_up_cleanly(ops):
    word = ops.selftest_bounded_wait(20000)
    assert (word >> 24) & 0xff == 0x7E and (word >> 16) & 0xff == 0x55
    # the context is still usable afterwards
    assert torch.ones(4, device="cuda").sum().item() == 4.0


@pytest.mark.parametrize("M,N,K", [(128, 256, 16), (128, 256, 64), (128, 256, 256), (256, 512, 1280),
                                   (300, 480, 160), (4096, 3840, 1280), (1000, 1280, 5120), (77, 8, 8)])
def test_gemm_bf16_raw_accumulator(ops, M, N, K):
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    a = _bf16(torch.randn(M, K, generator=g))
    w = _bf16(torch.randn(N, K, generator=g) * 0.05)
    ref = a.float() @ w.float().t()
    out = ops.gemm_bf16(a.cuda(), w.cuda(), raw=True)
    ops.check_status()
    torch.testing.assert_close(out.cpu(), ref, rtol=2e-4, atol=2e-4 * ref.abs().max().item())


def test_gemm_bf16_identity_layout(ops):
    """W = I: the output must reproduce A column for column (catches any tile/swizzle permutation)."""
    M, K = 256, 256
    a = _bf16(torch.arange(M * K, dtype=torch.float32).reshape(M, K) % 251 - 125)
    w = _bf16(torch.eye(K))
    out = ops.gemm_bf16(a.cuda(), w.cuda(), raw=True)
    ops.check_status()
    assert torch.equal(out.cpu(), a.float())


@pytest.mark.parametrize("bias,gelu,res", [(True, False, False), (True, True, False), (True, False, True),
                                           (False, False, True)])
def test_gemm_bf16_epilogues(ops, bias, gelu, res):
    M, N, K = 520, 640, 320
    g = torch.Generator().manual_seed(5)
    a = _bf16(torch.randn(M, K, generator=g))
    w = _bf16(torch.randn(N, K, generator=g) * 0.05)
    b = torch.randn(N, generator=g)
    r = _bf16(torch.randn(M, N, generator=g))
    ref = a.float() @ w.float().t()
    if bias:
        ref = ref + b
    if gelu:
        ref = torch.nn.functional.gelu(ref)
    if res:
        ref = ref + r.float()
    out = ops.gemm_bf16(a.cuda(), w.cuda(), b.cuda() if bias else None, r.cuda() if res else None, gelu=gelu)
    ops.check_status()
    torch.testing.assert_close(out.float().cpu(), ref, rtol=1e-2, atol=1e-2)


def test_gemm_bf16_broadcast_residual(ops):
    M, N, K, R = 512, 256, 64, 128
    g = torch.Generator().manual_seed(6)
    a = _bf16(torch.randn(M, K, generator=g))
    w = _bf16(torch.randn(N, K, generator=g) * 0.1)
    r = _bf16(torch.randn(R, N, generator=g))
    ref = a.float() @ w.float().t() + r.float().repeat(M // R, 1)
    out = ops.gemm_bf16(a.cuda(), w.cuda(), None, r.cuda())
    ops.check_status()
    torch.testing.assert_close(out.float().cpu(), ref, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 32), (128, 256, 128), (300, 480, 160), (4096, 1280, 1280),
                                   (777, 5120, 1280), (512, 1280, 5120)])
def test_gemm_i8_accumulator_bit_exact(ops, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    aq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    wq = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    ref = qo.int8_matmul_i32(aq, wq)
    out = ops.gemm_i8(aq.cuda(), None, wq.cuda(), None, raw=True)
    ops.check_status()
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("gelu,res", [(False, False), (True, False), (False, True)])
def test_gemm_i8_dequant_epilogue_matches_oracle(ops, gelu, res):
    M, N, K = 392, 640, 320
    g = torch.Generator().manual_seed(9)
    x = _bf16(torch.randn(M, K, generator=g))
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.02
    r = _bf16(torch.randn(M, N, generator=g))
    ref = qo.int8_linear(x.float(), w, b, gelu=gelu, residual=r.float() if res else None)
    xq, sx = ops.quant_rows_i8(x.cuda())
    wq, sw = qo.quantize_rows_absmax(w)
    xq_ref, sx_ref = qo.quantize_rows_absmax(x.float())
    assert torch.equal(xq.cpu(), xq_ref) and torch.equal(sx.cpu(), sx_ref)
    out = ops.gemm_i8(xq, sx, wq.cuda(), sw.cuda(), b.cuda(), r.cuda() if res else None, gelu=gelu)
    ops.check_status()
    # same int32 accumulators and scales; only fma contraction / erf differences remain
    torch.testing.assert_close(out.float().cpu(), ref, rtol=8e-3, atol=2e-3)


@pytest.mark.parametrize("rows,C", [(64 * 64, 1280), (2 * 64 * 64, 768), (1000, 160), (3, 2048)])
def test_layernorm_rows(ops, rows, C):
    g = torch.Generator().manual_seed(rows + C)
    x = _bf16(torch.randn(rows, C, generator=g) * 3 + 0.5)
    gamma = 1 + 0.1 * torch.randn(C, generator=g)
    beta = 0.1 * torch.randn(C, generator=g)
    ref = torch.nn.functional.layer_norm(x.float(), (C,), gamma, beta, 1e-6)
    out = ops.layernorm(x.cuda(), gamma.cuda(), beta.cuda(), 1e-6)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=8e-3, atol=8e-3)


@pytest.mark.parametrize("grid,window,C,B", [(64, 14, 160, 2), (32, 14, 768, 1), (28, 14, 64, 1)])
def test_layernorm_window_partition_order(ops, grid, window, C, B):
    from oracle import encoder_oracle as eo
    g = torch.Generator().manual_seed(grid)
    x = _bf16(torch.randn(B * grid * grid, C, generator=g))
    gamma = 1 + 0.1 * torch.randn(C, generator=g)
    beta = 0.1 * torch.randn(C, generator=g)
    y = torch.nn.functional.layer_norm(x.float(), (C,), gamma, beta, 1e-6).to(torch.bfloat16).float()
    ref, _ = eo.window_partition(y.reshape(B, grid, grid, C), window)
    ref = ref.reshape(-1, C)
    out = ops.layernorm(x.cuda(), gamma.cuda(), beta.cuda(), 1e-6, grid=grid, window=window).float().cpu()
    assert out.shape == ref.shape
    pad = ref.abs().sum(dim=1) == 0
    assert (out[pad] == 0).all()          # pad rows are exactly zero
    torch.testing.assert_close(out, ref, rtol=8e-3, atol=8e-3)


def test_layernorm_quant_matches_oracle_bitwise_given_same_ln(ops):
    rows, C, grid, window = 2 * 64 * 64, 160, 64, 14
    g = torch.Generator().manual_seed(11)
    x = _bf16(torch.randn(rows, C, generator=g))
    gamma = 1 + 0.1 * torch.randn(C, generator=g)
    beta = 0.1 * torch.randn(C, generator=g)
    y = ops.layernorm(x.cuda(), gamma.cuda(), beta.cuda(), 1e-6, grid=grid, window=window)
    yq, sc = ops.layernorm_quant_i8(x.cuda(), gamma.cuda(), beta.cuda(), 1e-6, grid=grid, window=window)
    q_ref, s_ref = qo.quantize_rows_absmax(y.float().cpu())
    assert torch.equal(yq.cpu(), q_ref) and torch.equal(sc.cpu(), s_ref)


@pytest.mark.parametrize("rows,C", [(1000, 1280), (8 * 148 * 4 * 3 + 5, 160), (777, 768), (515, 1024), (300, 2048), (7, 1280)])
def test_layernorm_quant_raster_rows_bitwise(ops, rows, C):
    """Raster-order rows (the persistent prefetching kernels): row counts that are not multiples of the warps in
    flight, every vector-count variant.  The int8 rows and scales equal the oracle's quantisation of the bf16
    LayerNorm kernel's own output bit for bit; values include exact ties (x / scale = k + 1/2)."""
    g = torch.Generator().manual_seed(rows + C)
    x = _bf16(torch.randn(rows, C, generator=g) * 2 + 0.25)
    gamma = 1 + 0.1 * torch.randn(C, generator=g)
    beta = 0.1 * torch.randn(C, generator=g)
    y = ops.layernorm(x.cuda(), gamma.cuda(), beta.cuda(), 1e-6)
    ref = torch.nn.functional.layer_norm(x.float(), (C,), gamma, beta, 1e-6)
    torch.testing.assert_close(y.float().cpu(), ref, rtol=8e-3, atol=8e-3)
    yq, sc = ops.layernorm_quant_i8(x.cuda(), gamma.cuda(), beta.cuda(), 1e-6)
    q_ref, s_ref = qo.quantize_rows_absmax(y.float().cpu())
    assert torch.equal(yq.cpu(), q_ref) and torch.equal(sc.cpu(), s_ref)
    # rows holding ties: absmax 127 makes the scale exactly 1, and k + 0.5 is a bf16 value for small k
    t = torch.zeros(64, C)
    t[:, 0] = 127.0
    t[:, 1:41] = torch.arange(-20, 20).float() + 0.5
    t[:, 41] = -127.0
    tq, ts = ops.quant_rows_i8(_bf16(t).cuda())
    q_ref, s_ref = qo.quantize_rows_absmax(_bf16(t))
    assert torch.equal(tq.cpu(), q_ref) and torch.equal(ts.cpu(), s_ref)


def test_layernorm2d_nchw(ops):
    B, hw, C = 2, 64 * 64, 256
    g = torch.Generator().manual_seed(12)
    x = _bf16(torch.randn(B * hw, C, generator=g) * 2)
    gamma = 1 + 0.1 * torch.randn(C, generator=g)
    beta = 0.1 * torch.randn(C, generator=g)
    ref = torch.nn.functional.layer_norm(x.float(), (C,), gamma, beta, 1e-6)
    out = ops.layernorm2d(x.cuda(), gamma.cuda(), beta.cuda(), hw, 1e-6, to_nchw=True).float().cpu()
    torch.testing.assert_close(out, ref.reshape(B, hw, C).permute(0, 2, 1), rtol=8e-3, atol=8e-3)
    out2 = ops.layernorm2d(x.cuda(), gamma.cuda(), beta.cuda(), hw, 1e-6, to_nchw=False).float().cpu()
    torch.testing.assert_close(out2, ref, rtol=8e-3, atol=8e-3)


@pytest.mark.parametrize("int8", [False, True])
def test_gemm_head_major_output(ops, int8):
    """The qkv projection variant that writes one contiguous [M, head_dim] plane per (q|k|v, head)."""
    M, H, d, K = 392, 2, 80, 160
    N = 3 * H * d
    g = torch.Generator().manual_seed(21)
    x = _bf16(torch.randn(M, K, generator=g))
    w = torch.randn(N, K, generator=g) * 0.05
    b = torch.randn(N, generator=g) * 0.1
    if int8:
        xq, sx = ops.quant_rows_i8(x.cuda())
        wq, sw = qo.quantize_rows_absmax(w)
        out = ops.gemm_heads(xq, sx, wq.cuda(), sw.cuda(), b.cuda(), d)
        plain = ops.gemm_i8(xq, sx, wq.cuda(), sw.cuda(), b.cuda())
    else:
        out = ops.gemm_heads(x.cuda(), None, _bf16(w).cuda(), None, b.cuda(), d)
        plain = ops.gemm_bf16(x.cuda(), _bf16(w).cuda(), b.cuda())
    ops.check_status()
    assert out.shape == (3 * H, M, d)
    assert torch.equal(out.permute(1, 0, 2).reshape(M, N), plain)        # same numbers, different layout


@pytest.mark.parametrize("rows,C", [(300, 5120), (65, 4096), (17, 3072), (1000, 1280)])
def test_quant_rows_wide_and_narrow_bit_exact(ops, rows, C):
    g = torch.Generator().manual_seed(rows + C)
    x = _bf16(torch.randn(rows, C, generator=g) * 2.0)
    x[0].zero_()                                     # an all-zero row must take the floor scale
    q, s = ops.quant_rows_i8(x.cuda())
    q_ref, s_ref = qo.quantize_rows_absmax(x.float())
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)


# ------------------------------------------------------------------ 2:4 sparse int8 GEMM
def _sparse_weight(N, K, seed):
    from oracle import quant_oracle as qo
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g)
    keep = qo.prune_2_4_mask(w)
    wq = (torch.randint(-127, 128, (N, K), generator=g) * keep).to(torch.int8)
    return wq


@pytest.mark.parametrize("T,N,K", [(300, 256, 256), (1000, 160, 160), (4096 + 17, 640, 1280), (224, 128, 32),
                                   (3000, 512, 640), (4096 + 17, 1280, 5120)])       # the last two run on CTA pairs
def test_gemm_i8_sp24_accumulators_bit_exact(ops, T, N, K):
    """Sparse tensor-core path: int32 accumulators equal the dense integer product with the uncompressed
    weight, bit for bit (token / channel / K tails included)."""
    wq = _sparse_weight(N, K, 3)
    g = torch.Generator().manual_seed(4)
    xq = torch.randint(-127, 128, (T, K), generator=g, dtype=torch.int8)
    wc, meta = ops.pack_sp24(wq.cuda())
    acc = ops.gemm_i8_sp24(xq.cuda(), None, wc, meta, None, raw=True)
    ops.check_status()
    ref = (xq.double() @ wq.double().t()).to(torch.int32)          # exact: |sum| < 2^53
    assert torch.equal(acc.cpu(), ref)


def test_pack_sp24_round_trip_and_rejects_dense(ops):
    """Decompressing (values, positions read back through an identity activation) restores the weight;
    a weight that is not 2:4 sets the status word."""
    N, K = 256, 384
    wq = _sparse_weight(N, K, 5)
    wc, meta = ops.pack_sp24(wq.cuda())
    eye = torch.eye(K, dtype=torch.int8, device="cuda")
    back = ops.gemm_i8_sp24(eye, None, wc, meta, None, raw=True).t()
    ops.check_status()
    assert torch.equal(back.cpu(), wq.int())
    dense = torch.ones(128, 64, dtype=torch.int8, device="cuda")
    ops.pack_sp24(dense)
    with pytest.raises(RuntimeError, match="2:4"):
        ops.check_status()


@pytest.mark.parametrize("epi,T,N", [("bias", 1500, 320), ("gelu", 1500, 320), ("residual", 1500, 320),
                                     ("bias", 3000, 512), ("residual", 5000, 1280)])   # the last two run on CTA pairs
def test_gemm_i8_sp24_epilogues_match_dense_kernel(ops, epi, T, N):
    """Same dequantising epilogue as the dense int8 kernel on the same (pruned) weight: bitwise equal."""
    K = 640
    wq = _sparse_weight(N, K, 6).cuda()
    g = torch.Generator().manual_seed(7)
    xq = torch.randint(-127, 128, (T, K), generator=g, dtype=torch.int8).cuda()
    sx = (torch.rand(T, generator=g) * 0.02 + 0.001).cuda()
    sw = (torch.rand(N, generator=g) * 0.002 + 0.0001).cuda()
    bias = torch.randn(N, generator=g).cuda()
    res = torch.randn(T, N, generator=g).bfloat16().cuda() if epi == "residual" else None
    wc, meta = ops.pack_sp24(wq)
    a = ops.gemm_i8_sp24(xq, sx, wc, meta, sw, bias, res, gelu=epi == "gelu")
    b = ops.gemm_i8(xq, sx, wq, sw, bias, res, gelu=epi == "gelu")
    ops.check_status()
    assert torch.equal(a, b)


@pytest.mark.parametrize("rows,C", [(500, 5120), (300, 640), (64, 1280)])
def test_gelu_quant_rows_matches_oracle(ops, rows, C):
    """GELU + bf16 rounding + per-row quantisation in one pass over the hidden activation: scales equal the
    oracle's to float rounding, int8 values differ by at most one step on at most 0.1 % of the entries (the
    erf approximation can move a value across a bf16 rounding boundary)."""
    from oracle import quant_oracle as qo
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(rows, C, generator=g) * 2.0).bfloat16()
    ref_act = torch.nn.functional.gelu(x.float()).bfloat16().float()
    rq, rs = qo.quantize_rows_absmax(ref_act)
    yq, ys = ops.quant_rows_i8(x.cuda(), gelu=True)
    ops.check_status()
    torch.testing.assert_close(ys.cpu(), rs, rtol=1e-2, atol=0)
    d = (yq.cpu().int() - rq.int()).abs()
    assert d.max().item() <= 1
    assert (d != 0).float().mean().item() < 1e-3


@pytest.mark.parametrize("M,N,K,gelu", [(4096 + 100, 512, 1280, True), (300, 160, 160, True), (2048, 5120, 1280, True),
                                        (1000, 640, 320, False)])
def test_gemm_i8_requant_equals_gemm_then_row_quantisation(ops, M, N, K, gelu):
    """The re-quantising Linear (row maxima from the GEMM epilogue's atomics, streaming quantisation): its bf16
    output is the plain int8 GEMM's, and its int8 rows / scales are what the row quantiser gives on that output,
    bit for bit; on CTA pairs (first and third shape) and on the single-CTA kernel, and twice in a row (the scratch
    is cleared inside the call)."""
    g = torch.Generator().manual_seed(M + N)
    x = _bf16(torch.randn(M, K, generator=g))
    w = torch.randn(N, K, generator=g) * 0.05
    b = torch.randn(N, generator=g) * 0.1
    xq, sx = ops.quant_rows_i8(x.cuda())
    wq, sw = qo.quantize_rows_absmax(w)
    plain = ops.gemm_i8(xq, sx, wq.cuda(), sw.cuda(), b.cuda(), gelu=gelu)
    q_ref, s_ref = ops.quant_rows_i8(plain)
    for _ in range(2):
        yq, ys, out = ops.gemm_i8_requant(xq, sx, wq.cuda(), sw.cuda(), b.cuda(), gelu=gelu)
        ops.check_status()
        assert torch.equal(out, plain)
        assert torch.equal(ys, s_ref) and torch.equal(yq, q_ref)
    oq, os_ = qo.quantize_rows_absmax(plain.float().cpu())              # and the oracle's quantiser on the same rows
    assert torch.equal(yq.cpu(), oq) and torch.equal(ys.cpu(), os_)


@pytest.mark.parametrize("T,N,K,gelu", [(4096 + 100, 512, 1280, True), (300, 160, 160, True), (3000, 512, 640, False)])
def test_gemm_i8_sp24_requant_equals_gemm_then_row_quantisation(ops, T, N, K, gelu):
    """The same for a 2:4-compressed weight: the sparse kernel's epilogue supplies the row maxima (single-CTA with
    the GELU, CTA pairs without)."""
    g = torch.Generator().manual_seed(T + N)
    x = _bf16(torch.randn(T, K, generator=g))
    b = torch.randn(N, generator=g) * 0.1
    xq, sx = ops.quant_rows_i8(x.cuda())
    wq = _sparse_weight(N, K, seed=T)
    sw = torch.rand(N, generator=g) * 0.002 + 0.0005
    wc, meta = ops.pack_sp24(wq.cuda())
    plain = ops.gemm_i8_sp24(xq, sx, wc, meta, sw.cuda(), b.cuda(), gelu=gelu)
    q_ref, s_ref = ops.quant_rows_i8(plain)
    for _ in range(2):
        yq, ys, out = ops.gemm_i8_requant(xq, sx, wc, sw.cuda(), b.cuda(), gelu=gelu, meta=meta)
        ops.check_status()
        assert torch.equal(out, plain)
        assert torch.equal(ys, s_ref) and torch.equal(yq, q_ref)


# ------------------------------------------------------------------ CTA-pair GEMM
@pytest.mark.parametrize("M,N,K", [(4096 + 100, 512, 1280), (8192, 1280, 5120), (2048, 256, 64)])
def test_gemm_pair_kernel_equals_single_cta_kernel(ops, M, N, K, monkeypatch):
    """Large products run on CTA pairs (cta_group::2); the same call with SAMB_GEMM_SINGLE_CTA=1 runs the
    single-CTA kernel.  Same accumulation order per output element, same epilogue: bitwise equal, for every
    epilogue, int8, and the head-major output; and both agree with a float64 reference."""
    g = torch.Generator().manual_seed(13)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().cuda()
    b = torch.randn(N, generator=g).cuda()
    r = torch.randn(M, N, generator=g).bfloat16().cuda()
    xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).cuda()
    wq = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).cuda()
    sx, sw = torch.rand(M, generator=g).cuda(), torch.rand(N, generator=g).cuda()
    calls = {
        "bias": lambda: ops.gemm_bf16(x, w, b),
        "gelu": lambda: ops.gemm_bf16(x, w, b, gelu=True),
        "residual": lambda: ops.gemm_bf16(x, w, b, r),
        "int8": lambda: ops.gemm_i8(xq, sx, wq, sw, b),
        "int8 residual": lambda: ops.gemm_i8(xq, sx, wq, sw, b, r),
    }
    if N % 80 == 0:
        calls["head-major"] = lambda: ops.gemm_heads(x, None, w, None, b, 80)
    pair = {k: f() for k, f in calls.items()}
    monkeypatch.setenv("SAMB_GEMM_SINGLE_CTA", "1")
    single = {k: f() for k, f in calls.items()}
    ops.check_status()
    for k in calls:
        assert torch.equal(pair[k], single[k]), k
    ref = (x.double() @ w.double().t() + b.double()).float()
    torch.testing.assert_close(pair["bias"].float(), ref, rtol=2e-2, atol=2e-2)
