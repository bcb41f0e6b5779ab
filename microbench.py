"""Single-kernel timings through the C ABI (CUDA events, L2 flushed by inputs larger than L2 where
the shape allows it).  One JSON line per run:

    python microbench.py gemm --m 131072 --n 3840 --k 1280 --epilogue bias [--int8 | --sp24]
    python microbench.py attn-global --batch 8 --heads 16 --tokens 4096 --dim 80
    python microbench.py attn-window --batch 200 --heads 16 --dim 80
    python microbench.py layernorm --rows 131072 --cols 1280 [--quant]
    python microbench.py mask-stats --n 192 --h 1024 --w 1024 [--bf16]
    python microbench.py mask-rle --n 192 --h 1024 --w 1024
    python microbench.py tab-products --rows 131072 --heads 16 --dim 80 --t 64
    python microbench.py quant-rows --rows 131072 --cols 5120
    python microbench.py attn-global --arm sdpa | --arm ref-triton        (the reference's GPU paths, for comparison)

The two attention commands at their defaults are the standalone relative-position attention
benchmark (q, k, v ~ N(0,1), rel_h / rel_w ~ N(0,0.5), bf16).
"""
import argparse
import json

import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from segment_anything_fast_b200 import ops  # noqa: E402


def _time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    ops.check_status()
    return a.elapsed_time(b) / iters


def _attention_arm(arm, q, k, v, rh, rw):
    """The callable an attention subcommand times: this library's kernel, or one of the reference's two GPU paths
    (measurement only; neither is part of the product)."""
    if arm == "sdpa":
        B, H, N, _ = q.shape
        def run():
            bias = (rh.unsqueeze(-1) + rw.unsqueeze(-2)).view(B, H, N, N)          # materialised as the reference does
            return torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=bias)
        return run
    if arm == "ref-triton":
        os.environ["SEGMENT_ANYTHING_FAST_USE_FLASH_4"] = "1"
        from oracle.make_ref import REF_DIR
        sys.path.insert(0, REF_DIR)
        os.chdir(os.environ.get("TMPDIR", "/tmp"))                               # the autotuner writes its cache to the cwd
        from segment_anything_fast.flash_4 import _attention_rel_h_rel_w
        return lambda: _attention_rel_h_rel_w(q, k, v, rh.unsqueeze(-1), rw.unsqueeze(-2))
    N = q.shape[2]
    return (lambda: ops.attn_relpos_global(q, k, v, rh, rw)) if N != 196 else (lambda: ops.attn_relpos_window(q, k, v, rh, rw))


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=131072); g.add_argument("--n", type=int, default=3840)
    g.add_argument("--k", type=int, default=1280)
    g.add_argument("--epilogue", choices=["none", "bias", "gelu", "residual"], default="bias")
    g.add_argument("--int8", action="store_true")
    g.add_argument("--sp24", action="store_true", help="int8 with a 2:4-sparse weight on the sparse tensor-core path")
    g.add_argument("--requant", action="store_true",
                   help="int8 product + per-row re-quantisation of its output (row maxima from the GEMM epilogue)")
    ag = sub.add_parser("attn-global")
    ag.add_argument("--batch", type=int, default=8); ag.add_argument("--heads", type=int, default=16)
    ag.add_argument("--tokens", type=int, default=4096); ag.add_argument("--dim", type=int, default=80)
    aw = sub.add_parser("attn-window")
    aw.add_argument("--batch", type=int, default=200); aw.add_argument("--heads", type=int, default=16)
    aw.add_argument("--dim", type=int, default=80)
    ln = sub.add_parser("layernorm")
    ln.add_argument("--rows", type=int, default=131072); ln.add_argument("--cols", type=int, default=1280)
    ln.add_argument("--quant", action="store_true")
    ms_ = sub.add_parser("mask-stats")
    ms_.add_argument("--n", type=int, default=192); ms_.add_argument("--h", type=int, default=1024)
    ms_.add_argument("--w", type=int, default=1024); ms_.add_argument("--bf16", action="store_true")
    mr = sub.add_parser("mask-rle")
    mr.add_argument("--n", type=int, default=192); mr.add_argument("--h", type=int, default=1024)
    mr.add_argument("--w", type=int, default=1024)
    tp = sub.add_parser("tab-products")
    tp.add_argument("--rows", type=int, default=131072); tp.add_argument("--heads", type=int, default=16)
    tp.add_argument("--dim", type=int, default=80); tp.add_argument("--t", type=int, default=64)
    for p in (ag, aw):
        p.add_argument("--tables", action="store_true",
                       help="the encoder's form: head-major raster-order qkv of --batch images (64 x 64 tokens), rel-pos "
                            "products computed in the kernel from the tables")
        p.add_argument("--arm", choices=["b200", "sdpa", "ref-triton"], default="b200",
                       help="b200: this library's kernel; sdpa: torch SDPA with the materialised [B,H,N,N] bias, the "
                            "reference's fallback (flash_4.py:368-370); ref-triton: the reference's own Triton kernel "
                            "from a copy of its package under oracle/_ref (flash_4.py:30-145; autotunes on first use)")
    qr = sub.add_parser("quant-rows")
    qr.add_argument("--rows", type=int, default=131072); qr.add_argument("--cols", type=int, default=1280)
    cp = sub.add_parser("copy", help="torch's own b.copy_(a) at a row-kernel size: what a plain copy reaches on this working set")
    cp.add_argument("--rows", type=int, default=131072); cp.add_argument("--cols", type=int, default=1280)
    for p in (g, ag, aw, ln, ms_, mr, tp, qr, cp):
        p.add_argument("--iters", type=int, default=10); p.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    torch.manual_seed(0)
    dev = "cuda"
    out = {"kernel": a.cmd}
    if a.cmd == "gemm":
        M, N, K = a.m, a.n, a.k
        bias = torch.randn(N, device=dev) if a.epilogue != "none" else None
        res = torch.randn(M, N, device=dev).bfloat16() if a.epilogue == "residual" else None
        y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        if a.int8 or a.sp24:
            x = torch.randint(-127, 128, (M, K), device=dev, dtype=torch.int8)
            w = torch.randint(-127, 128, (N, K), device=dev, dtype=torch.int8)
            sx, sw = torch.rand(M, device=dev), torch.rand(N, device=dev)
            if a.sp24:
                w.view(N, K // 4, 4)[:, :, 2:] = 0               # any 2:4 pattern times the same
                wc, meta = ops.pack_sp24(w)
                fn = lambda: ops.gemm_i8_sp24(x, sx, wc, meta, sw, bias, res, gelu=a.epilogue == "gelu", out=y)
            elif a.requant:
                fn = lambda: ops.gemm_i8_requant(x, sx, w, sw, bias, gelu=a.epilogue == "gelu", out=y)
            else:
                fn = lambda: ops.gemm_i8(x, sx, w, sw, bias, res, gelu=a.epilogue == "gelu", out=y)
        else:
            x = torch.randn(M, K, device=dev).bfloat16()
            w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
            fn = lambda: ops.gemm_bf16(x, w, bias, res, gelu=a.epilogue == "gelu", out=y)
        ms = _time(fn, a.iters, a.warmup)
        out.update(shape=[M, N, K], epilogue=a.epilogue, dtype="int8-sp24" if a.sp24 else ("int8" if a.int8 else "bf16"),
                   ms=round(ms, 4),
                   tflops=round(2.0 * M * N * K / ms / 1e9, 1))
    elif a.cmd == "attn-global":
        B, H, N, d = a.batch, a.heads, a.tokens, a.dim
        if a.tables:
            qkv = torch.randn(3 * H, B * N, d, device=dev).bfloat16()
            tables = (torch.randn(256, d, device=dev) * 0.1).bfloat16()
            y = torch.empty(B * N, H * d, device=dev, dtype=torch.bfloat16)
            ms = _time(lambda: ops.attn_relpos_global_tables(qkv, tables, B, H, N, d, out=y), a.iters, a.warmup)
            out.update(arm="b200-tables", shape=[B, H, N, d], ms=round(ms, 4), tflops=round(4.0 * B * H * N * N * d / ms / 1e9, 1))
            print(json.dumps(out))
            return
        q, k, v = (torch.randn(B, H, N, d, device=dev).bfloat16() for _ in range(3))
        rh = (torch.randn(B, H, N, N // 64, device=dev) * 0.5).bfloat16()
        rw = (torch.randn(B, H, N, 64, device=dev) * 0.5).bfloat16()
        ms = _time(_attention_arm(a.arm, q, k, v, rh, rw), a.iters, a.warmup)
        out.update(arm=a.arm, shape=[B, H, N, d], ms=round(ms, 4), tflops=round(4.0 * B * H * N * N * d / ms / 1e9, 1))
    elif a.cmd == "attn-window":
        B, H, d = a.batch, a.heads, a.dim
        if a.tables:                                       # B images: 25 windows each, gathered from raster order
            qkv = torch.randn(3 * H, B * 4096, d, device=dev).bfloat16()
            tables = (torch.randn(64, d, device=dev) * 0.1).bfloat16()
            bias = torch.randn(3 * H * d, device=dev).bfloat16()
            y = torch.empty(B * 4096, H * d, device=dev, dtype=torch.bfloat16)
            ms = _time(lambda: ops.attn_relpos_window_tables(qkv, bias, tables, B, H, 64, 14, d, out=y), a.iters, a.warmup)
            nbytes = 4 * B * 4096 * H * d * 2                                  # q, k, v in, o out (real tokens)
            out.update(arm="b200-tables", shape=[B * 25, H, 196, d], ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1))
            print(json.dumps(out))
            return
        q, k, v = (torch.randn(B, H, 196, d, device=dev).bfloat16() for _ in range(3))
        rh = (torch.randn(B, H, 196, 14, device=dev) * 0.5).bfloat16()
        rw = (torch.randn(B, H, 196, 14, device=dev) * 0.5).bfloat16()
        ms = _time(_attention_arm(a.arm, q, k, v, rh, rw), a.iters, a.warmup)
        nbytes = 4 * B * H * 196 * d * 2 + 2 * B * H * 196 * 14 * 2          # q, k, v, o + rel_h, rel_w
        out.update(arm=a.arm, shape=[B, H, 196, d], ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1),
                   tflops=round(4.0 * B * H * 196 * 196 * d / ms / 1e9, 1))
    elif a.cmd == "copy":
        x = torch.randn(a.rows, a.cols, device=dev).bfloat16()
        y = torch.empty_like(x)
        ms = _time(lambda: y.copy_(x), a.iters, a.warmup)
        out.update(shape=[a.rows, a.cols], ms=round(ms, 4), gbs=round(a.rows * a.cols * 4 / ms / 1e6, 1))
    elif a.cmd == "quant-rows":
        x = torch.randn(a.rows, a.cols, device=dev).bfloat16()
        ms = _time(lambda: ops.quant_rows_i8(x), a.iters, a.warmup)
        out.update(shape=[a.rows, a.cols], ms=round(ms, 4), gbs=round((a.rows * a.cols * 3 + a.rows * 4) / ms / 1e6, 1))
    elif a.cmd == "mask-stats":
        from segment_anything_fast_b200 import amg
        x = (torch.randn(a.n, a.h, a.w, device=dev) * 2.0).to(torch.bfloat16 if a.bf16 else torch.float32)
        ms = _time(lambda: amg.mask_stats(x, 0.0, 1.0), a.iters, a.warmup)
        nbytes = x.numel() * (x.element_size() + 1)                            # logits in, binary masks out
        out.update(shape=[a.n, a.h, a.w], dtype="bf16" if a.bf16 else "f32", ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1))
    elif a.cmd == "tab-products":
        # rel-pos table products of one block: q planes [3H, rows, d] x tables [T, d] -> [rows, H*T]
        # (T = 64 for the 14x14 windows, 256 for the 64x64 global grid)
        qkv = torch.randn(3 * a.heads, a.rows, a.dim, device=dev).bfloat16()
        tab = torch.randn(a.t, a.dim, device=dev).bfloat16()
        cs = torch.ones(a.t, device=dev)
        y = torch.empty(a.rows, a.heads * a.t, device=dev, dtype=torch.bfloat16)
        ms = _time(lambda: ops.relpos_table_products(qkv, tab, cs, a.heads, out=y), a.iters, a.warmup)
        nbytes = a.heads * a.rows * a.dim * 2 + y.numel() * 2                  # q planes in, products out
        out.update(shape=[a.heads, a.rows, a.dim, a.t], ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1))
    elif a.cmd == "mask-rle":
        from segment_anything_fast_b200 import _lib
        # blob-like masks: a coarse random field upsampled and thresholded (a few hundred runs per mask)
        coarse = torch.randn(a.n, 1, 16, 16, device=dev)
        m = (torch.nn.functional.interpolate(coarse, size=(a.h, a.w), mode="bilinear")[:, 0] > 0.3).contiguous()
        cap = 8192
        counts = torch.empty(a.n, cap, dtype=torch.int32, device=dev)
        n_counts = torch.empty(a.n, dtype=torch.int32, device=dev)
        mv = m.view(torch.uint8)
        fn = lambda: _lib.check(_lib.load().samb_mask_rle(mv.data_ptr(), a.n, a.h, a.w, counts.data_ptr(), n_counts.data_ptr(),
                                                          cap, ops._stream()), "samb_mask_rle")
        ms = _time(fn, a.iters, a.warmup)
        runs = int(n_counts.sum().item())
        nbytes = m.numel() + runs * 4                                          # masks in once, run lengths out
        out.update(shape=[a.n, a.h, a.w], runs_per_mask=round(runs / a.n, 1), ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1))
    else:
        R, C = a.rows, a.cols
        x = torch.randn(R, C, device=dev).bfloat16()
        gm, bt = torch.ones(C, device=dev), torch.zeros(C, device=dev)
        if a.quant:
            ms = _time(lambda: ops.layernorm_quant_i8(x, gm, bt), a.iters, a.warmup)
            nbytes = R * C * 3 + R * 4
        else:
            y = torch.empty(R, C, device=dev, dtype=torch.bfloat16)
            ms = _time(lambda: ops.layernorm(x, gm, bt, out=y), a.iters, a.warmup)
            nbytes = R * C * 4
        out.update(shape=[R, C], quant=bool(a.quant), ms=round(ms, 4), gbs=round(nbytes / ms / 1e6, 1))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
