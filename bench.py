#!/usr/bin/env python
"""Benchmark of the SAM ViT-H image-encoder hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--quant none|int8|int8-sp24] [--impl reference]

One step = one pass of the encoder over a batch of 32 synthetic 1024x1024 images per GPU (images
shard by rank, weak scaling; the only collective is the all-gather of the embeddings at the end of a
step, issued on a side stream).  Prints ONE JSON line (rank 0).  `value` is device-resident throughput
(CUDA events, max over ranks); `e2e` goes through the host-facing session (pinned uint8 images in, H2D,
normalise, encoder, D2H of the embeddings).  Without `--quant` the headline is the bf16 encoder and the
same measurement is repeated for the int8 and the int8 + 2:4-sparse-MLP encoders, reported under
`configs`; with `--quant X` only that configuration runs and is the headline.  `--impl reference` times
the reference's own CPU encoder (a copy of its package under oracle/_ref; the CPU restatement when that
copy is absent) on the host cores (rank 0 only) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from functools import partial

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH = 32
METRIC = "ViT-H encoder images/sec at batch 32"
# Algorithmic FLOPs per ViT-H image (2*M*N*K, real tokens only, no credit for zero-padded window
# tokens): patch 8.05e9 + linear 5.154e12 + global attention 3.49e11 + window attention 1.475e11 +
# neck 7.52e9.
FLOPS_PER_IMAGE = 5.666e12
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes (read + write) per launch of the Linear GEMM kernel: ncu captures of the 32768-row qkv /
# lin1 / lin2 launches (292 / 380 / 525 MB), scaled x4 to the 131072-row launches of this workload
# (traffic grows with the rows; the weights stay in L2), proj taken at its algorithmic 1.0 GB; mean
# over the four Linear shapes of a block.
GEMM_TRAFFIC_BYTES_PER_LAUNCH = 1.45e9


def env_int(name, default):
    return int(os.environ.get(name, default))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi samples of the SM clock and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.idx)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 8:
                    continue
                try:
                    clocks.append(float(f[1])); mx = float(f[2])
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if clocks:
            busy = sorted(clocks)[len(clocks) // 4:]          # drop the idle head/tail samples
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(clocks))
        return out


class LaunchProfiler:
    """Counts every samb_* launch and brackets the Linear GEMMs with CUDA events on the launch stream."""
    # positions of M, N, K in the call; the 2:4 kernel is credited with the multiply-adds it executes (half)
    GEMMS = {"samb_gemm_bf16": (10, 11, 12, 2.0), "samb_gemm_i8": (12, 13, 14, 2.0),
             "samb_gemm_bf16_heads": (6, 7, 8, 2.0), "samb_gemm_i8_heads": (8, 9, 10, 2.0),
             "samb_gemm_i8_sp24": (13, 14, 15, 1.0)}

    def __init__(self):
        self.launches = 0
        self.records = []          # (flops, start_event, end_event, (name, N, K))

    def begin(self, name, args):
        if name in ("samb_abi_version", "samb_error_string", "samb_decode_status", "samb_sp24_meta_bytes"):
            return None                                        # host-only helpers: nothing is launched
        self.launches += 3 if "requant" in name else 1                    # clear + GEMM + streaming quantisation
        pos = self.GEMMS.get(name)
        if pos is None:
            return None
        M, N, K = (int(args[i]) for i in pos[:3])
        M = min(M, BATCH * 4096)   # algorithmic rows: the window-padding tokens of the qkv projection earn nothing
        if K < 1024:               # patch-embed / neck GEMMs are not "the Linear layers"
            return None
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        return (pos[3] * M * N * K, s, e, (name, N, K))

    def end(self, tok):
        if tok is not None:
            tok[2].record()
            self.records.append(tok)


def build_vit_h(quant, device, sparse_mlp=False):
    from segment_anything_fast_b200 import apply_sparse, build_image_encoder_vit_h
    torch.manual_seed(0)
    enc = build_image_encoder_vit_h()
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for name, p in enc.named_parameters():                 # random-init weights of the ViT-H architecture
            if p.dim() >= 2 or "rel_pos" in name:
                p.normal_(0.0, 0.02, generator=g)
    if sparse_mlp:                                             # 2:4-pruned mlp.lin1 / mlp.lin2
        apply_sparse(enc, mlp_only=True)
    return enc.to(torch.bfloat16).to(device).set_quant(quant)


def measure_tensor_peaks(device, seconds=2.0):
    """Rate of back-to-back tcgen05.mma on operands resident in shared memory (``samb_selftest_mma_rate``, one CTA
    per SM): the best of a few short launches (burst) and a seconds-long train of launches under the power cap
    (sustained), for kind::i8 and for kind::f16 on bf16.  The int8 figures are the peak the int8 GEMMs are quoted
    against; the bf16 figures cross-check the probe against the library-GEMM peak in MEASURED_PEAKS.json."""
    import ctypes
    from segment_anything_fast_b200 import _lib, ops
    lib = _lib.load()
    st = ops.status_word(device)
    n_sm = torch.cuda.get_device_properties(device).multi_processor_count
    stream = torch.cuda.current_stream().cuda_stream
    out = {}
    for name, int8 in (("int8", 1), ("bf16", 0)):
        def launch(rounds):
            n = ctypes.c_double(0.0)
            _lib.check(lib.samb_selftest_mma_rate(int8, rounds, n_sm, st.data_ptr(), None, ctypes.byref(n), stream),
                       "samb_selftest_mma_rate")
            return n.value
        launch(200)
        torch.cuda.synchronize()
        best = 0.0
        short = 4000 if int8 else 2000                       # a few milliseconds per launch
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); n_ops = launch(short); b.record()
            torch.cuda.synchronize()
            best = max(best, n_ops / (a.elapsed_time(b) * 1e-3) / 1e12)
        sampler = ClockSampler(device.index or 0)
        sampler.start()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        total, t0 = 0.0, time.perf_counter()
        a.record()
        while time.perf_counter() - t0 < seconds:
            for _ in range(4):
                total += launch(8 * short)
            torch.cuda.synchronize()
        b.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        out[name] = {"burst": round(best, 1), "sustained": round(total / (a.elapsed_time(b) * 1e-3) / 1e12, 1),
                     "sm_mhz_sustained": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}
    ops.check_status(device)
    return out


def measure_config(args, quant_name, device, dist, world, rank, local, tensor_peaks):
    """Build the ViT-H encoder in one arithmetic (none | int8 | int8-sp24), time ``steps`` device-resident passes and
    ``steps`` end-to-end passes; returns the fields of the JSON line that depend on the configuration."""
    from segment_anything_fast_b200 import EncoderSession, _lib, ops
    from segment_anything_fast_b200.dist import gather_embeddings
    sparse_mlp = quant_name == "int8-sp24"
    quant = None if quant_name == "none" else "int8"
    torch.cuda.reset_peak_memory_stats(device)
    enc = build_vit_h(quant, device, sparse_mlp)
    sess = EncoderSession(enc, BATCH, device)
    g = torch.Generator().manual_seed(1000 + rank)
    sess.host_in.copy_(torch.randint(0, 256, sess.host_in.shape, generator=g, dtype=torch.uint8))
    images_dev = sess.host_in.to(device)
    gathered = torch.empty(world * BATCH, enc.out_chans, 64, 64, dtype=torch.bfloat16, device=device) if world > 1 else None
    main = torch.cuda.current_stream(device)
    side = torch.cuda.Stream(device) if dist is not None else None     # the all-gather overlaps the next step's encoder
    done = torch.cuda.Event()

    def step_device():
        emb = sess.encode_device(images_dev)
        if dist is not None:
            done.record(main)
            side.wait_event(done)
            with torch.cuda.stream(side):
                gather_embeddings(emb, out=gathered)
            emb.record_stream(side)
        return emb

    def barrier():
        if dist is not None:
            main.wait_stream(side)
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step_device()
    barrier()
    ops.check_status(device)

    # ---- timed region: device-resident inputs
    prof = LaunchProfiler()
    _lib.set_profiler(prof)
    sampler = ClockSampler(local)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step_device()
    if side is not None:
        main.wait_stream(side)             # the last gather is inside the timed region
    ev1.record()
    barrier()
    clocks = sampler.stop()
    _lib.set_profiler(None)
    ms = ev0.elapsed_time(ev1)
    gemm_flops = sum(r[0] for r in prof.records)
    gemm_ms = sum(r[1].elapsed_time(r[2]) for r in prof.records)
    if args.gemm_breakdown and rank == 0:                      # average time per Linear shape, to stderr
        by_shape = {}
        for r in prof.records:
            by_shape.setdefault(r[3], []).append(r[1].elapsed_time(r[2]))
        for key, ts in sorted(by_shape.items()):
            print(f"[{quant_name}] {key[0]} N={key[1]} K={key[2]}: {len(ts)} launches, mean {sum(ts) / len(ts):.4f} ms",
                  file=sys.stderr)
    launches = prof.launches

    # ---- end to end: pinned host uint8 in, host embeddings out, every step (two batches in flight: the upload
    # of step i+1 and the download of step i-1 overlap the encoder pass of step i)
    sess.slot_input(1).copy_(sess.host_in)
    for _ in range(2):
        sess.result(sess.submit())
    barrier()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    pending = None
    for _ in range(args.steps):
        slot = sess.submit()               # H2D (pinned uint8) -> normalise -> encoder -> D2H, all queued
        if pending is not None:
            sess.result(pending)           # blocks until the previous step's embeddings are in host memory
        pending = slot
    sess.result(pending)
    t1.record()
    barrier()
    e2e_ms = t0.elapsed_time(t1)
    ops.check_status(device)
    peak_mem = torch.cuda.max_memory_allocated(device)

    if dist is not None:
        t = torch.tensor([ms, e2e_ms, float(peak_mem)], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, peak_mem = t.tolist()
    h2d, d2h = sess.h2d_bytes, sess.d2h_bytes
    del sess, enc, images_dev, gathered
    torch.cuda.empty_cache()

    pk, pk_kind = peaks()
    bf16_peak = float(pk.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    if quant == "int8":
        if tensor_peaks is not None:       # measured here: back-to-back kind::i8 MMAs, seconds long, power-capped
            peak_tf = float(tensor_peaks["int8"]["sustained"])
            peak_note = ("measured in this run: samb_selftest_mma_rate kind::i8, one CTA per SM, sustained "
                         f"(burst {tensor_peaks['int8']['burst']}); the same probe on bf16 gives "
                         f"{tensor_peaks['bf16']['sustained']} sustained / {tensor_peaks['bf16']['burst']} burst against "
                         f"{bf16_peak} / {pk.get('bf16_tflops')} for the {pk_kind} cuBLAS GEMM")
        else:
            peak_tf, peak_note = 2.0 * bf16_peak, f"2 x {pk_kind} bf16 cuBLAS sustained (probe skipped)"
    else:
        peak_tf, peak_note = bf16_peak, f"{pk_kind} bf16 cuBLAS sustained"
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    value = world * BATCH * args.steps / (ms * 1e-3)
    # whole-step roofline time: the Linear FLOPs at the Linear peak of this arithmetic (2:4 layers at their
    # executed half), everything else at the bf16 peak
    f_lin = 5.154e12 * (0.5 + 0.5 * (1280 * 1280 * 4) / (1280 * 1280 * 12)) if sparse_mlp else 5.154e12
    t_roof = f_lin / (peak_tf * 1e12) + (FLOPS_PER_IMAGE - 5.154e12) / (bf16_peak * 1e12)
    return {
        "value": round(value, 2), "ms_per_step": round(ms / args.steps, 3),
        "dtype": "int8" if quant == "int8" else "bf16",
        "config": {"workload": "SAM ViT-H image encoder, batch 32 per GPU, 1024x1024 seeded uint8 images, "
                               "random-init weights" + (", int8 dynamic-quant linears" if quant else ", bf16 linears")
                               + (", 2:4-sparse mlp.lin1/lin2 on the sparse tensor-core path" if sparse_mlp else ""),
                   "batch_per_gpu": BATCH, "parallelism": f"dp{world} (images sharded by rank, all-gather of embeddings "
                                                           "on a side stream)",
                   "l2": "inputs_larger_than_l2", "quant": quant_name},
        "clocks": clocks,
        "e2e": {"value": round(world * BATCH * args.steps / (e2e_ms * 1e-3), 2), "unit": "img/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "peak_mem_bytes": int(peak_mem),
        "roofline": {"bound": "tensor", "kernel": ("gemm_pair_kernel" if quant is None else "gemm_pair_kernel / gemm_tc_kernel")
                               + (" + gemm_sp24_kernel" if sparse_mlp else "") + " (qkv/proj/lin1/lin2 launches)",
                     "achieved": None if achieved is None else round(achieved, 1), "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": None if achieved is None else round(achieved / peak_tf, 4),
                     "traffic": GEMM_TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peak_note,
                     "whole_step_frac": round((value / world) * t_roof, 4)},
    }


def run_b200(args):
    world = env_int("WORLD_SIZE", 1)
    rank = env_int("RANK", 0)
    local = env_int("LOCAL_RANK", 0)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    names = [args.quant] if args.quant else ["none", "int8", "int8-sp24"]
    tensor_peaks = None
    if any(n != "none" for n in names) and not args.no_peak_probe:
        if rank == 0:
            tensor_peaks = measure_tensor_peaks(device)
        if dist is not None:
            dist.barrier()
    results = {n: measure_config(args, n, device, dist, world, rank, local, tensor_peaks) for n in names}
    if rank == 0:
        head = results[names[0]]
        line = {"metric": METRIC, "value": head["value"], "unit": "img/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic"}
        line.update({k: head[k] for k in ("config", "clocks", "e2e", "gpu_launches", "peak_mem_bytes", "roofline")})
        if len(names) > 1:
            line["configs"] = {n.replace("-", "_"): {k: v for k, v in results[n].items() if k != "config"} for n in names[1:]}
            line["gpu_launches"] = sum(results[n]["gpu_launches"] for n in names)
        if tensor_peaks is not None:
            line["tensor_peaks"] = tensor_peaks
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_reference(steps=1, warmup=0)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def _cpu_reference_own_code(steps, warmup, cores):
    """The reference's own encoder on the host: ``sam_model_registry['vit_h']().image_encoder`` in fp32 with its CPU
    attention path (SDPA composite), one whole image per step."""
    from oracle.make_ref import import_ref
    from oracle import encoder_oracle as eo
    import_ref()
    from segment_anything_fast.build_sam import sam_model_registry
    torch.manual_seed(0)
    enc = sam_model_registry["vit_h"]().image_encoder.eval()
    x = eo.seeded_images(1, seed=1000)
    times = []
    with torch.no_grad():
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            enc(x)
            if it >= warmup:
                times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return {"value": round(1.0 / sec, 5), "unit": "img/s", "cores": cores, "kind": "reference",
            "sample": f"{steps} x 1 whole ViT-H image (of the 32 of a step), fp32, the reference's own CPU encoder "
                      f"(SDPA attention path), median of {steps}", "seconds_per_image": round(sec, 2)}


def _cpu_reference_port(steps, warmup, cores):
    """CPU restatement of the reference encoder (oracle port), fp32, one whole image per step."""
    from oracle import encoder_oracle as eo
    eo.USE_SDPA = True                      # the fused CPU attention the reference itself runs
    cfg = eo.VIT_H
    sd = eo.seeded_state_dict(cfg, seed=0)
    x = eo.seeded_images(1, seed=1000)
    times = []
    with torch.no_grad():
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            eo.image_encoder_forward(x, sd, cfg, "fp32")
            if it >= warmup:
                times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return {"value": round(1.0 / sec, 5), "unit": "img/s", "cores": cores, "kind": "port",
            "sample": f"{steps} x 1 whole ViT-H image (of the 32 of a step), fp32, CPU restatement of the reference "
                      f"encoder (oracle/_ref absent), median of {steps}", "seconds_per_image": round(sec, 2)}


def cpu_reference(steps=1, warmup=0):
    """The reference's CPU path on all host threads, on a bounded sample of the workload: whole images, one at a
    time (a step of the GPU arm is 32 of them)."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    try:
        return _cpu_reference_own_code(steps, warmup, cores)
    except ImportError:
        return _cpu_reference_port(steps, warmup, cores)


def run_reference(args):
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))      # whole images; a few seconds each
    warmup = 1 if args.warmup > 0 else 0
    base = cpu_reference(steps=steps, warmup=warmup)
    world = env_int("WORLD_SIZE", 1)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "img/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(BATCH * base["seconds_per_image"] * 1e3, 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "SAM ViT-H image encoder, batch 32 per GPU, 1024x1024 seeded uint8 images, random-init weights "
                                   f"(CPU, {base['kind']}; timed on {steps} whole image(s), ms_per_step = 32 x the per-image time)"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "img/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--quant", choices=["none", "int8", "int8-sp24"], default=None,
                    help="run only this configuration (default: bf16 headline + int8 + int8-sp24 under `configs`)")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gemm-breakdown", action="store_true", help="print the mean time per Linear shape to stderr")
    ap.add_argument("--no-peak-probe", action="store_true", help="skip the tensor-pipe rate probe (int8 peak)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
