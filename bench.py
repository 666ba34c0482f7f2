#!/usr/bin/env python
"""Benchmark of the dot / dotMPI hot path: the README two-layer skinny product
(128 x 100000) . (100000 x 40000) . (40000 x 20000), fp32, W column-sharded over the ranks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--mode 3xtf32|tf32] [--exchange fp32|8bit]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE for N > 1).  Rank 0 prints one JSON line.

  value     whole-job TFLOP/s of the two dotMPI calls with the batch and the weights resident in HBM
            (2*M*N*K flops, the three TF32 products of the 3xTF32 mode counted once), CUDA events, max over ranks
  e2e       the same two calls through the C ABI starting from a pinned HOST batch (row-major) and ending with the
            row-major result in pinned host memory: upload + transpose, broadcast, two dotMPI, transpose + download;
            the upload of the next batch and the download of the previous result run on side streams
  roofline  the tensor-core kernel of layer 1 alone, timed by events around its launches inside the timed region
  codec     8-bit compress / decompress / absmax GB/s on config 2 (4096 x 4096, rotating buffers) and on 1 GiB
  cpu_baseline  multithreaded fp32 sgemm (numpy / OpenBLAS) of a column sample of the same product on the host cores

--impl reference times the CPU stand-in of the reference path (clusterNet itself is CUDA + MPI only and cannot be
built here): the same sgemm on a bounded column sample per step.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, K1, N1, N2 = 128, 100000, 40000, 20000


def set_sizes(k1, n1, n2):
    """The headline workload is fixed; smaller N1 / N2 exist only so that a profiler capture stays small."""
    global K1, N1, N2, FLOPS_L1, FLOPS_L2, FLOPS_STEP
    K1, N1, N2 = k1, n1, n2
    FLOPS_L1 = 2.0 * M * K1 * N1
    FLOPS_L2 = 2.0 * M * N1 * N2
    FLOPS_STEP = FLOPS_L1 + FLOPS_L2          # 1.2288e12 at the headline sizes


set_sizes(K1, N1, N2)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [l.split(", ") for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l.split(", ") for (_, l) in self.lines[-3:]]
        sm, reasons, smax = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax = float(r[2])
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sgemm_sample(seconds_target=12.0, threads=None):
    """Multithreaded fp32 sgemm of column samples of both layers; returns TFLOP/s and a description."""
    cores = len(os.sched_getaffinity(0))
    rng = np.random.default_rng(0)
    batch = rng.random((M, K1), dtype=np.float32)
    lim1 = 4.0 * np.sqrt(6.0 / (K1 + N1))
    probe_cols = 256
    W = rng.uniform(-lim1, lim1, (K1, probe_cols)).astype(np.float32)
    t = time.perf_counter(); batch @ W; dt = time.perf_counter() - t
    t = time.perf_counter(); batch @ W; dt = min(dt, time.perf_counter() - t)
    rate = 2.0 * M * K1 * probe_cols / dt
    cols1 = int(min(N1, max(probe_cols, seconds_target * 0.8 * rate / (2.0 * M * K1) / 3)))
    cols1 = max(256, cols1 // 256 * 256)
    W1 = rng.uniform(-lim1, lim1, (K1, cols1)).astype(np.float32)
    lim2 = 4.0 * np.sqrt(6.0 / (N1 + N2))
    cols2 = max(128, cols1 // 2)
    W2 = rng.uniform(-lim2, lim2, (N1, cols2)).astype(np.float32)
    act = rng.random((M, N1), dtype=np.float32)
    best = None
    for _ in range(3):
        t = time.perf_counter()
        batch @ W1
        act @ W2
        d = time.perf_counter() - t
        best = d if best is None else min(best, d)
    flops = 2.0 * M * K1 * cols1 + 2.0 * M * N1 * cols2
    return flops / best / 1e12, cores, f"numpy float32 @ (OpenBLAS): 128x{K1} . {K1}x{cols1} + 128x{N1} . {N1}x{cols2} column sample, best of 3"


def run_reference(args, rank):
    """CPU stand-in of the reference path: rank 0 alone, bounded column sample per step."""
    if rank != 0:
        return
    cores = len(os.sched_getaffinity(0))
    rng = np.random.default_rng(0)
    batch = rng.random((M, K1), dtype=np.float32)
    lim1, lim2 = 4.0 * np.sqrt(6.0 / (K1 + N1)), 4.0 * np.sqrt(6.0 / (N1 + N2))
    cols1, cols2 = 1024, 512
    W1 = rng.uniform(-lim1, lim1, (K1, cols1)).astype(np.float32)
    W2 = rng.uniform(-lim2, lim2, (N1, cols2)).astype(np.float32)
    act = rng.random((M, N1), dtype=np.float32)
    for _ in range(args.warmup):
        batch @ W1; act @ W2
    t0 = time.perf_counter()
    for _ in range(args.steps):
        batch @ W1; act @ W2
    dt = time.perf_counter() - t0
    flops = (2.0 * M * K1 * cols1 + 2.0 * M * N1 * cols2) * args.steps
    v = flops / dt / 1e12
    sample = f"per step 128x{K1} . {K1}x{cols1} and 128x{N1} . {N1}x{cols2} (column sample of both layers), numpy float32 @ on the host"
    print(json.dumps({
        "impl": "reference", "metric": "dotMPI TFLOP/s", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": "README dotMPI two-layer skinny GEMM: 128x100000 . 100000x40000 . 40000x20000, W column-sharded",
                   "note": "host CPU stand-in: clusterNet has no CPU path and cannot be built here (MPI, HDF5 absent)"},
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)


def codec_bench(ctx, torch, peaks):
    """compress / decompress / absmax GB/s: config 2 (4096^2, five rotating buffer sets so that no launch finds its
    input in L2) and a 1 GiB tensor."""
    out = {}
    for label, n, sets, iters in (("config2_4096x4096", 4096 * 4096, 6, 30), ("1GiB", 1 << 28, 2, 6)):
        xs = [torch.randn(n, device="cuda") * 0.1 for _ in range(sets)]
        codes = [torch.empty(n, dtype=torch.uint8, device="cuda") for _ in range(sets)]
        outs = [torch.empty(n, device="cuda") for _ in range(sets)]
        pm = ctx.absmax(xs[0])
        p = float(pm.item())
        res = {}
        for name, fn, bytes_per in (("compress", lambda i: ctx.compress(xs[i], p, out=codes[i]), 5),
                                    ("decompress", lambda i: ctx.decompress(codes[i], p, out=outs[i]), 5),
                                    ("absmax", lambda i: ctx.absmax(xs[i], out=pm), 4)):
            for i in range(sets):
                fn(i)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for it in range(iters):
                fn(it % sets)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            gbs = n * bytes_per / ms / 1e6
            res[name] = {"GB/s": round(gbs, 1), "us": round(ms * 1e3, 2), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4)}
        # the pipeline a caller runs when the scale is not known beforehand: absmax, then the compressor with the scale
        # taken from device memory (no host synchronisation); 9 algorithmic bytes per element (4 + 4 read, 1 written)
        scale = torch.zeros(1, device="cuda")

        def pipeline(i):
            ctx.absmax(xs[i], out=scale)
            ctx.compress(xs[i], scale, out=codes[i])
        for i in range(sets):
            pipeline(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for it in range(iters):
            pipeline(it % sets)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        res["absmax_then_compress"] = {"GB/s": round(n * 9 / ms / 1e6, 1), "us": round(ms * 1e3, 2),
                                       "frac_of_hbm_peak": round(n * 9 / ms / 1e6 / peaks["hbm_gbs"], 4)}
        # yardstick at the same size: a plain device copy (read + write bytes) through torch, same rotation of buffers.
        # At 64 MiB a launch lasts ~20 us, so launch ramp and tail weigh on every kernel, the copy included.
        for i in range(sets):
            outs[i].copy_(xs[i])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for it in range(iters):
            outs[it % sets].copy_(xs[it % sets])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        res["torch_copy_same_size"] = {"GB/s": round(n * 8 / ms / 1e6, 1), "us": round(ms * 1e3, 2)}
        out[label] = res
        del xs, codes, outs
        torch.cuda.empty_cache()
    return out


def train_step_bench(ctx, cn, _lib, torch, dist, world, rank, steps=30):
    """Config 4: data-parallel MLP 784-1200-1200-10, ReLU, dropout (0.2 input, 0.5 hidden), softmax, batch 128 per GPU,
    8-bit compressed gradient exchange (per-rank absmax scales gathered with the codes), RMSprop — the call sequence of the
    reference's Layer class (source/Layer.cpp:250-261,314-339,341-471) through the C ABI.  Returns ms per step."""
    lib, h, sp = ctx.lib, ctx.h, ctx.stream_ptr()
    B, sizes, drops = 128, [784, 1200, 1200, 10], [0.2, 0.5, 0.5]
    X = ctx.randn(B, sizes[0], seed=100 + rank)
    y = torch.randint(0, 10, (B,), device="cuda").float()
    W = [ctx.uniform_sqrt_weight(sizes[i], sizes[i + 1], seed=7 + i) for i in range(3)]     # same weights on every rank
    bias = [torch.zeros(sizes[i + 1], device="cuda") for i in range(3)]
    rms = [torch.zeros_like(w) for w in W]
    grad = [torch.zeros_like(w) for w in W]
    act = [X] + [ctx.empty(B, sizes[i + 1]) for i in range(3)]
    out = [ctx.empty(B, s) for s in sizes]
    err = [None] + [ctx.empty(B, sizes[i + 1]) for i in range(3)]
    tmat = ctx.empty(B, 10)
    d_seed = torch.tensor([1000 + rank], dtype=torch.int64, device="cuda")     # dropout seed in device memory

    def one_step():
        sp = ctx.stream_ptr()                                                    # the capture stream while recording
        # forward: (wait for the previous exchange + update), fused dot+bias+activation, dropout
        cn.check(lib.cn_dropout_dp(h, act[0].data_ptr(), out[0].data_ptr(), act[0].numel(), drops[0], d_seed.data_ptr(), 0, sp))
        for l in range(3):
            if True:   # first step: the gradients are zero, the exchange and the update are no-ops on the weights
                cn.check(lib.cn_grad_sync_8bit(h, grad[l].data_ptr(), grad[l].numel(), 0.0, sp))
                cn.check(lib.cn_rmsprop_update(h, rms[l].data_ptr(), grad[l].data_ptr(), W[l].data_ptr(), 0.9, 0.006, W[l].numel(), sp))
            last = l == 2
            ctx.gemm(out[l], W[l], out=(out[l + 1] if last else act[l + 1]), bias=bias[l],
                     activation=_lib.ACT_LINEAR if last else _lib.ACT_RELU)
            if last:
                cn.check(lib.cn_softmax(h, out[3].data_ptr(), out[3].data_ptr(), B, 10, sp))
            else:
                cn.check(lib.cn_dropout_dp(h, act[l + 1].data_ptr(), out[l + 1].data_ptr(), act[l + 1].numel(), drops[l + 1], d_seed.data_ptr(),
                                           1 << (20 + l), sp))
        # backward errors
        cn.check(lib.cn_create_t_matrix(h, y.data_ptr(), tmat.data_ptr(), B, 10, sp))
        cn.check(lib.cn_sub(h, out[3].data_ptr(), tmat.data_ptr(), err[3].data_ptr(), err[3].numel(), sp))
        for l in (2, 1):
            cn.check(lib.cn_activation_gradient(h, act[l].data_ptr(), _lib.ACT_RELU, out[l].data_ptr(), out[l].numel(), sp))
            ctx.gemm(err[l + 1], W[l], out=err[l], transB=True)
            cn.check(lib.cn_mul(h, err[l].data_ptr(), out[l].data_ptr(), err[l].data_ptr(), err[l].numel(), sp))
        # gradients
        for l in range(3):
            ctx.gemm(act[l], err[l + 1], out=grad[l], transA=True)
        cn.check(lib.cn_seed_advance(h, d_seed.data_ptr(), sp))

    def timed(fn):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    for _ in range(5):
        one_step()
    n0 = lib.cn_kernel_launches()
    ms_eager = timed(one_step)
    launches = (lib.cn_kernel_launches() - n0) / steps
    # the same step recorded once in a CUDA graph and replayed (the dropout seed advances on the device)
    ms = ms_eager
    graph_ms = None
    try:
        if world > 1:
            raise RuntimeError("not attempted with more than one rank (collectives inside a capture)")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            one_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            one_step()
        for _ in range(3):
            g.replay()
        graph_ms = timed(g.replay)
        ms = min(ms, graph_ms)
    except Exception as exc:   # capture is an optimisation of the harness, not of the library
        graph_ms = f"no graph: {exc}"[:120]
    if world > 1:
        t = torch.tensor([ms_eager], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = ms_eager = float(t.item())
    ctx.gemm_check()
    return {"workload": "config 4: MLP 784-1200-1200-10, batch 128 per GPU, 8-bit gradient exchange, RMSprop", "ms_per_step": ms,
            "ms_per_step_eager": ms_eager, "ms_per_step_cuda_graph": graph_ms,
            "samples_per_s": 128 * world / (ms * 1e-3), "launches_per_step": launches,
            "flops_per_step_per_gpu": 6.0 * 128 * (784 * 1200 + 1200 * 1200 + 1200 * 10)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="3xtf32", choices=["3xtf32", "tf32"])
    ap.add_argument("--exchange", default="fp32", choices=["fp32", "8bit", "8bit-fused"],
                    help="fp32: gather C in fp32; 8bit: gather codes, decode to fp32; 8bit-fused: layer-1 output stays coded and is\n"
                         "decoded inside layer 2's GEMM pre-pass")
    ap.add_argument("--nccl-gather", action="store_true", help="gather C with ncclAllGather instead of the fused peer stores")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-codec", action="store_true")
    ap.add_argument("--no-train-step", action="store_true", help="skip the config-4 training-step measurement")
    ap.add_argument("--only-codec", action="store_true", help="run the codec measurements alone (small profiler captures)")
    ap.add_argument("--k1", type=int, default=K1, help="profiling aid: inner dimension of layer 1")
    ap.add_argument("--n1", type=int, default=N1, help="profiling aid: columns of W1 (headline: 40000)")
    ap.add_argument("--n2", type=int, default=N2, help="profiling aid: columns of W2 (headline: 20000)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    headline = (args.k1, args.n1, args.n2) == (K1, N1, N2)
    set_sizes(args.k1, args.n1, args.n2)
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    import clusternet_b200 as cn
    from clusternet_b200 import _lib

    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torchrun (--nproc-per-node N) for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    ctx = cn.Context(local_rank)
    lib = ctx.lib
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        ids = [ctx.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        ctx.comm_init(ids[0], rank, world)
    peaks = measured_peaks()
    if args.only_codec:
        if rank == 0:
            print(json.dumps({"codec": codec_bench(ctx, torch, peaks)}), flush=True)
        return
    mode = _lib.GEMM_3XTF32 if args.mode == "3xtf32" else _lib.GEMM_TF32
    exchange = 1 if args.exchange == "8bit" else 0

    # ---- workload: weights sharded by columns, created on the owning rank (distributed_uniformSqrtWeight)
    s1, c1 = ctx.shard_cols(N1, rank, world)
    s2, c2 = ctx.shard_cols(N2, rank, world)
    seed = 0 + 10000 * rank + 12345
    W1 = ctx.empty(K1, c1)
    cn.check(lib.cn_uniform_sqrt_weight(ctx.h, W1.data_ptr(), W1.numel(), K1, N1, seed, 0, ctx.stream_ptr()))
    W2 = ctx.empty(N1, c2)
    cn.check(lib.cn_uniform_sqrt_weight(ctx.h, W2.data_ptr(), W2.numel(), N1, N2, seed + 1, 0, ctx.stream_ptr()))
    # batch: uniform [0,1) seed 0 on the host (row-major, pinned), as a user of the reference would hold it
    h_batch = torch.from_numpy(np.random.default_rng(0).random((M, K1), dtype=np.float32)).pin_memory()
    h_out = torch.empty((M, N2), dtype=torch.float32).pin_memory()
    d_stage_in = torch.empty((M, K1), dtype=torch.float32, device="cuda")
    d_stage_out = torch.empty((M, N2), dtype=torch.float32, device="cuda")
    batch = ctx.empty(M, K1)
    # outputs in symmetric buffers: the all-gather of each layer is fused into the GEMM epilogue (stores to peer memory)
    fused = world > 1 and args.exchange != "8bit" and not args.nccl_gather
    out1 = ctx.sym_empty(M, N1) if fused else ctx.empty(M, N1)
    out2 = ctx.sym_empty(M, N2) if fused else ctx.empty(M, N2)
    sp = ctx.stream_ptr()

    def upload():
        if rank == 0:
            cn.check(lib.cn_upload_row_major(ctx.h, h_batch.data_ptr(), d_stage_in.data_ptr(), batch.data_ptr(), M, K1, sp))
        if world > 1:
            ctx.bcast(batch, 0)

    coded = None
    if args.exchange == "8bit-fused":
        c_codes = torch.empty((N1, M), dtype=torch.uint8, device="cuda")
        c_scales = torch.zeros(world, dtype=torch.float32, device="cuda")
        c_own = torch.empty((c1, M), dtype=torch.float32, device="cuda")
        coded = _lib.Coded(c_codes.data_ptr(), c_scales.data_ptr(), c_own.data_ptr(), M, N1)
        no_epi = cn.Epilogue(None, 0, 0, None)

    def two_layers(a_ptr=None):
        """The two sharded products; a_ptr: device address of the column-major batch (default: the resident copy)."""
        a_ptr = ctypes.c_void_p(a_ptr if a_ptr is not None else batch.data_ptr())
        if coded is not None:
            cn.check(lib.cn_dotmpi_to_coded_f32(ctx.h, M, K1, N1, a_ptr, W1.data_ptr(), ctypes.byref(coded), ctypes.byref(no_epi), mode, sp))
            cn.check(lib.cn_dotmpi_from_coded_f32(ctx.h, ctypes.byref(coded), N2, W2.data_ptr(), out2.data_ptr(), ctypes.byref(no_epi), mode, 0, sp))
            return
        plain = cn.Epilogue(None, 0, 0, None)
        cn.check(lib.cn_dotmpi_f32(ctx.h, M, K1, N1, a_ptr, W1.data_ptr(), out1.data_ptr(), ctypes.byref(plain), mode, exchange, sp))
        ctx.dotmpi(out1, W2, N2, out=out2, mode=mode, exchange=exchange)

    def download():
        if rank == 0:
            cn.check(lib.cn_download_row_major(ctx.h, out2.data_ptr(), d_stage_out.data_ptr(), h_out.data_ptr(), M, N2, sp))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    upload()
    for _ in range(args.warmup):
        two_layers()
    ctx.gemm_check()

    # ---- timed region 1: resident inputs
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    cn.check(lib.cn_gemm_profile_enable(ctx.h, 1))
    launches0 = lib.cn_kernel_launches()
    barrier()
    t_wall0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        two_layers()
    e1.record()
    barrier()
    t_wall1 = time.time()
    launches = lib.cn_kernel_launches() - launches0
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    buf = (ctypes.c_float * (4 * args.steps + 8))()
    cnt = ctypes.c_int()
    cn.check(lib.cn_gemm_profile_read(ctx.h, buf, len(buf), ctypes.byref(cnt)))
    cn.check(lib.cn_gemm_profile_enable(ctx.h, 0))
    kern_ms = [buf[i] for i in range(min(cnt.value, len(buf)))]
    l1_ms = max_over_ranks(float(np.mean(kern_ms[0::2]))) if kern_ms else None
    l2_ms = max_over_ranks(float(np.mean(kern_ms[1::2]))) if kern_ms else None
    ctx.gemm_check()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None

    # ---- timed region 2: end to end from host memory through the C ABI.  The host holds a (pinned, row-major) data set
    # of two batches; every step one batch is copied host->device by the asynchronous batch allocator on its side
    # stream (the copy of step i+1 runs while step i computes, as allocate_next_batch_async is meant to be used),
    # transposed into the current batch, broadcast, multiplied twice, and the result is transposed and copied back.
    h_set = torch.cat([h_batch, h_batch.flip(0)], 0).pin_memory() if rank == 0 else None
    h_lab = torch.zeros((2 * M, 1), dtype=torch.float32).pin_memory() if rank == 0 else None
    bh = ctypes.c_void_p()
    if rank == 0:
        cn.check(lib.cn_batch_create(ctx.h, h_set.data_ptr(), h_lab.data_ptr(), 2 * M, K1, 1, M, 0, ctypes.byref(bh)))
    px, py, pn = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int64()

    # The result leaves the same way the batch arrives: on a side stream.  The step's output is transposed into a staging
    # buffer on the compute stream; the device->host copy of that buffer runs on the copy stream while the next step
    # computes, and the staging buffer is not rewritten before that copy has finished (two events).
    copy_stream = torch.cuda.Stream() if rank == 0 else None
    ev_staged, ev_drained = torch.cuda.Event(), torch.cuda.Event()
    if rank == 0:
        ev_drained.record(torch.cuda.current_stream())

    def download_overlapped():
        if rank != 0:
            return
        main = torch.cuda.current_stream()
        main.wait_event(ev_drained)
        cn.check(lib.cn_to_row_major(ctx.h, out2.data_ptr(), d_stage_out.data_ptr(), M, N2, sp))
        ev_staged.record(main)
        copy_stream.wait_event(ev_staged)
        err = cudart.cudaMemcpyAsync(ctypes.c_void_p(h_out.data_ptr()), ctypes.c_void_p(d_stage_out.data_ptr()),
                                     ctypes.c_size_t(M * N2 * 4), 2, ctypes.c_void_p(copy_stream.cuda_stream))
        assert err == 0, f"cudaMemcpyAsync (device to host) failed: {err}"
        ev_drained.record(copy_stream)

    def e2e_step():
        # rank 0 multiplies the allocator's current batch where it lies and broadcasts it from there; the other ranks
        # receive into their resident buffer
        a_ptr = batch.data_ptr()
        if rank == 0:
            cn.check(lib.cn_batch_copy_next_async(bh))                     # prefetch of the NEXT batch (side stream)
            cn.check(lib.cn_batch_current(bh, ctypes.byref(px), ctypes.byref(py), ctypes.byref(pn)))
            a_ptr = px.value
        if world > 1:
            cn.check(lib.cn_bcast_f32(ctx.h, ctypes.c_void_p(a_ptr), M * K1, 0, sp))
        two_layers(a_ptr)
        download_overlapped()
        if rank == 0:
            cn.check(lib.cn_batch_swap(bh, sp, ctypes.byref(px), ctypes.byref(py), ctypes.byref(pn)))

    cudart = ctypes.CDLL("libcudart.so.12")
    for _ in range(2):
        e2e_step()
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(args.steps):
        e2e_step()
    if rank == 0:
        torch.cuda.current_stream().wait_event(ev_drained)   # the last step's result must be on the host inside the timed region
    e3.record()
    barrier()
    ms_e2e = max_over_ranks(e2.elapsed_time(e3))
    checksum = float(h_out.double().abs().mean())
    if rank == 0:
        lib.cn_batch_destroy(bh)

    # ---- accuracy on sampled columns against an fp64 host product (rank 0's shard edges + random columns)
    def sampled_error(act_dev, W_dev, out_dev, col0, ncols_local, kdim):
        rng_s = np.random.default_rng(7)
        cols = np.unique(np.concatenate([[0, 1, 127, 128, 129, ncols_local - 1], rng_s.integers(0, ncols_local, 58)]))
        cols = cols[(cols >= 0) & (cols < ncols_local)]
        a64 = act_dev.T.double().cpu().numpy()                      # (M, kdim)
        w64 = W_dev[torch.from_numpy(cols).cuda()].double().cpu().numpy().T   # (kdim, ncols)
        ref = a64 @ w64
        got = out_dev[torch.from_numpy(cols + col0).cuda()].double().cpu().numpy().T
        scale = float(out_dev.abs().max().item())
        return float(np.abs(got - ref).max() / scale)

    if coded is not None:   # out1 was never materialised: rebuild this rank's view of it for the check
        out1[s1:s1 + c1] = c_own
        for r in range(world):
            if r != rank:
                sr, cr = ctx.shard_cols(N1, r, world)
                ctx.decompress(c_codes[sr:sr + cr], c_scales[r:r + 1], out=out1[sr:sr + cr])
    err1 = sampled_error(batch, W1, out1, s1, c1, K1)
    err2 = sampled_error(out1, W2, out2, s2, c2, N1)

    train = None if (args.no_train_step or not headline) else train_step_bench(ctx, cn, _lib, torch, dist if world > 1 else None, world, rank)

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    value = FLOPS_STEP * args.steps / (ms_total * 1e-3) / 1e12
    e2e_value = FLOPS_STEP * args.steps / (ms_e2e * 1e-3) / 1e12
    tf32_peak = peaks["bf16_tflops"] / 2.0
    peak = tf32_peak / 3.0 if args.mode == "3xtf32" else tf32_peak
    l1_flops_rank = 2.0 * M * K1 * (N1 // world if world > 1 else N1)
    achieved = l1_flops_rank / (l1_ms * 1e-3) / 1e12 if l1_ms else None
    line = {
        "metric": "dotMPI TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": ("README dotMPI two-layer skinny GEMM: " if headline else "REDUCED (profiling) two-layer skinny GEMM: ") +
                               f"128x{K1} . {K1}x{N1} . {N1}x{N2}, W column-sharded",
                   "gemm_mode": args.mode, "exchange": args.exchange, "gather": ("fused peer stores" if fused else ("nccl" if world > 1 else "none")), "parallelism": f"tp{world} (columns of W)",
                   "l2": f"inputs larger than L2 ({4e-9 * (K1 * N1 + N1 * N2):.1f} GB of weights stream once per step)", "flops_per_step": FLOPS_STEP},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": M * K1 * 4,
                "d2h_bytes_per_step": M * N2 * 4, "result_checksum": checksum},
        "accuracy": {"metric": "max |C - C64| / max |C| over 64 sampled columns of rank 0's shard, fp64 host product of the same inputs",
                     "layer1": err1, "layer2": err2},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"kernel": "cn_gemm_tc_kernel (layer 1, per rank)", "bound": "tensor", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": (achieved / peak) if achieved else None,
                     # DRAM bytes per launch: ncu capture of 128x100000x4096 (profiles/gemm_tc_kernel_128x100000x4096.md:
                     # 1.772 GB for 1.6384 GB of W), scaled by the W bytes of this rank's layer-1 launch
                     "traffic": 1.772e9 / 1.6384e9 * 4.0 * K1 * (N1 // world if world > 1 else N1),
                     "traffic_source": "ncu dram__bytes_read+write of a 4096-column case, scaled by W bytes",
                     "ms_per_launch": l1_ms, "layer2_ms_per_launch": l2_ms,
                     "peak_source": f"{peaks['source']}: bf16_tflops {peaks['bf16_tflops']} / 2 (TF32 rate)" + (" / 3 (three TF32 products per tile)" if args.mode == "3xtf32" else ""),
                     # the same against the power-capped (seconds-long) cuBLAS figure, for runs whose clocks show sw_power_cap
                     "peak_sustained": peaks["bf16_tflops_sustained"] / 2.0 / (3.0 if args.mode == "3xtf32" else 1.0),
                     "frac_sustained": (achieved / (peaks["bf16_tflops_sustained"] / 2.0 / (3.0 if args.mode == "3xtf32" else 1.0))) if achieved else None,
                     "hbm_frac_layer1": (4.0 * K1 * (N1 / world) / (l1_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]) if l1_ms else None},
    }
    if train:
        line["train_step"] = train
    if not args.no_codec and world == 1:
        line["codec"] = codec_bench(ctx, torch, peaks)
    if not args.no_cpu_baseline and world == 1:
        v, cores, sample = cpu_sgemm_sample()
        line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
