#!/usr/bin/env python
"""Benchmark of the dot / dotMPI hot path: the README two-layer skinny product
(128 x 100000) . (100000 x 40000) . (40000 x 20000), fp32, W column-sharded over the ranks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--mode 3xtf32|tf32] [--exchange fp32|8bit|8bit-fused]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE for N > 1).  Rank 0 prints one JSON line and the
process exits non-zero when an accuracy or multi-rank check of that line fails.

  value     whole-job TFLOP/s of the two dotMPI calls with the batch and the weights resident in HBM
            (2*M*N*K flops, the three TF32 products of the 3xTF32 mode counted once), CUDA events, max over ranks
  e2e       the same two products through the C ABI starting from a pinned, row-major HOST data set and ending with the
            row-major result in pinned host memory.  Every rank holds the data set (as every process of the reference
            does with the Matrix* form of BatchAllocator::init), uploads 1/N of the rows of each batch over its own PCIe
            link on the allocator's side stream and exchanges the blocks over NVLink; the product reads the row-major
            batch as a transposed operand (TdotMPI form), the result is transposed and copied back on a copy stream
  accuracy  max |C - C64| / max |C| on columns sampled from EVERY rank's shard of both layers: each rank computes the fp64
            product of its own weight columns on the host, rank 0 compares them with its gathered copy (so columns that
            crossed NVLink are checked), and all ranks' gathered copies are compared bit for bit through checksums
  tf32      the same step in the single-pass TF32 mode, with its own (looser) bound and its HBM roofline
  roofline  the tensor-core kernel of layer 1 alone, timed by events around its launches inside the timed region
  codec     8-bit compress / decompress / absmax GB/s on config 2 (4096 x 4096, rotating buffers) and on 1 GiB
  cpu_baseline  multithreaded fp32 sgemm (numpy / OpenBLAS) with the flops of the whole step on the host cores

--impl reference times the CPU stand-in of the reference path (clusterNet itself is CUDA + MPI only and cannot be
built here): the same sgemm routine, all host threads, one whole step's flops per step.
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
TOL = {"3xtf32": 1e-5, "tf32": 2e-3}     # max |C - C64| / max |C|: the fp32-level bound, and the stated TF32 bound


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


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_sgemm_steps(steps, warmup):
    """The ONE CPU routine, used by both `--impl reference` and the cpu_baseline leg: multithreaded fp32 sgemm
    (numpy / OpenBLAS) with the flops of one whole step per step.  The weights are a block of 10000 columns per
    layer that is multiplied 4 (layer 1) and 2 (layer 2) times per step: 40000 and 20000 columns of work without 19 GB of
    host memory; each block (4 GB, 1.6 GB) is far larger than the CPU caches, so it streams from DRAM like distinct
    columns would.  The thread count is set explicitly (a launcher such as torchrun exports OMP_NUM_THREADS=1)."""
    from threadpoolctl import threadpool_info, threadpool_limits
    cores = len(os.sched_getaffinity(0))
    blk = 10000
    reps1, reps2 = max(1, N1 // blk), max(1, N2 // blk)
    blk1, blk2 = N1 // reps1, N2 // reps2
    rng = np.random.default_rng(0)
    lim1, lim2 = 4.0 * np.sqrt(6.0 / (K1 + N1)), 4.0 * np.sqrt(6.0 / (N1 + N2))
    batch = rng.random((M, K1), dtype=np.float32)
    act = rng.random((M, N1), dtype=np.float32)
    W1 = rng.random((K1, blk1), dtype=np.float32)
    W1 *= np.float32(2 * lim1); W1 -= np.float32(lim1)
    W2 = rng.random((N1, blk2), dtype=np.float32)
    W2 *= np.float32(2 * lim2); W2 -= np.float32(lim2)
    o1, o2 = np.empty((M, blk1), np.float32), np.empty((M, blk2), np.float32)

    def step():
        for _ in range(reps1):
            np.matmul(batch, W1, out=o1)
        for _ in range(reps2):
            np.matmul(act, W2, out=o2)

    with threadpool_limits(limits=cores):
        used = max([d.get("num_threads", 1) for d in threadpool_info() if d.get("user_api") == "blas"] or [1])
        for _ in range(warmup):
            step()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        dt = time.perf_counter() - t0
    flops = 2.0 * M * (K1 * blk1 * reps1 + N1 * blk2 * reps2)
    sample = (f"per step {reps1} x (128x{K1} . {K1}x{blk1}) + {reps2} x (128x{N1} . {N1}x{blk2}) = {flops / FLOPS_STEP:.3f} of the step's flops; "
              f"numpy float32 matmul (OpenBLAS), {used} threads, mean of {steps} steps after {warmup} warm-up")
    return {"value": flops * steps / dt / 1e12, "ms_per_step": dt / steps * 1e3, "cores": used, "sample": sample,
            "fraction_of_config": flops / FLOPS_STEP, "host_cores_available": cores}


def run_reference(args, rank):
    """CPU stand-in of the reference path: rank 0 alone."""
    if rank != 0:
        return
    r = cpu_sgemm_steps(args.steps, max(args.warmup, 1))
    print(json.dumps({
        "impl": "reference", "metric": "dotMPI TFLOP/s", "value": r["value"], "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"README dotMPI two-layer skinny GEMM: 128x{K1} . {K1}x{N1} . {N1}x{N2}, W column-sharded",
                   "note": "host CPU stand-in: clusterNet has no CPU path and cannot be built here (MPI, HDF5 absent)",
                   "fraction_of_config_per_step": r["fraction_of_config"]},
        "cpu_baseline": {"value": r["value"], "unit": "TFLOP/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)


# ------------------------------------------------------------------------------------------------ helpers
def cuda_time(torch, fn, iters, warm=1):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def codec_bench(ctx, torch, peaks):
    """compress / decompress / absmax GB/s: config 2 (4096^2, six rotating buffer sets so that no launch finds its
    input in L2) and a 1 GiB tensor."""
    out = {}
    for label, n, sets, iters in (("config2_4096x4096", 4096 * 4096, 6, 30), ("1GiB", 1 << 28, 2, 6),
                                  ("config4_gradients_2392800", 2392800, 8, 40)):
        xs = [torch.randn(n, device="cuda") * 0.1 for _ in range(sets)]
        codes = [torch.empty(n, dtype=torch.uint8, device="cuda") for _ in range(sets)]
        outs = [torch.empty(n, device="cuda") for _ in range(sets)]
        pm = ctx.absmax(xs[0])
        p = float(pm.item())
        res = {}
        scale = torch.zeros(1, device="cuda")

        def pipeline(i):
            # what a caller runs when the scale is not known beforehand: absmax, then the compressor with the scale taken
            # from device memory (no host synchronisation); 9 algorithmic bytes per element (4 + 4 read, 1 written)
            ctx.absmax(xs[i], out=scale)
            ctx.compress(xs[i], scale, out=codes[i])

        def fused(i):
            # the same through cn_absmax_compress_8bit: one cooperative launch up to 4 Mi elements, above that absmax and a
            # compressor that loads its first tiles while absmax drains
            ctx.absmax_compress(xs[i], scale=scale, out=codes[i])
        for name, fn, bytes_per in (("compress", lambda i: ctx.compress(xs[i], p, out=codes[i]), 5),
                                    ("decompress", lambda i: ctx.decompress(codes[i], p, out=outs[i]), 5),
                                    ("absmax", lambda i: ctx.absmax(xs[i], out=pm), 4),
                                    ("absmax_then_compress", pipeline, 9),
                                    ("absmax_compress_entry_point", fused, 9)):
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
    pushed = world > 1 and os.environ.get("CN_BENCH_PUSH_EXCHANGE", "1") == "1"
    if world > 1:
        cn.check(lib.cn_comm_set_push_exchange(h, 1 if pushed else 0))
    B, sizes, drops = 128, [784, 1200, 1200, 10], [0.2, 0.5, 0.5]
    X = ctx.randn(B, sizes[0], seed=100 + rank)
    y = torch.randint(0, 10, (B,), device="cuda").float()
    W = [ctx.uniform_sqrt_weight(sizes[i], sizes[i + 1], seed=7 + i) for i in range(3)]     # same weights on every rank
    bias = [torch.zeros(sizes[i + 1], device="cuda") for i in range(3)]
    # gradients, RMS state and weights of the three layers each live in ONE packed buffer, so that the exchange and the
    # update are one call each per step (cn_grad_sync_8bit_multi: a scale per layer, one gather, one decode-sum pass)
    numel = [w.numel() for w in W]
    offs = [0, numel[0], numel[0] + numel[1]]
    total = sum(numel)
    Wp = torch.empty(total, device="cuda")
    for i in range(3):
        Wp[offs[i]:offs[i] + numel[i]] = W[i].reshape(-1)
    W = [Wp[offs[i]:offs[i] + numel[i]].view(sizes[i + 1], sizes[i]) for i in range(3)]
    rms_p = torch.zeros(total, device="cuda")
    grad_p = torch.zeros(total, device="cuda")
    grad = [grad_p[offs[i]:offs[i] + numel[i]].view(sizes[i + 1], sizes[i]) for i in range(3)]
    seg = (ctypes.c_int64 * 3)(*numel)
    act = [X] + [ctx.empty(B, sizes[i + 1]) for i in range(3)]
    out = [ctx.empty(B, s) for s in sizes]
    err = [None] + [ctx.empty(B, sizes[i + 1]) for i in range(3)]
    d_seed = torch.tensor([1000 + rank], dtype=torch.int64, device="cuda")     # dropout seed in device memory

    comm_stream = torch.cuda.Stream()            # the gradient exchange and the weight update run beside the backward pass
    ev_grad = [torch.cuda.Event() for _ in range(3)]
    ev_err = [torch.cuda.Event() for _ in range(3)]
    ev_updated = torch.cuda.Event()
    seg1 = [(ctypes.c_int64 * 1)(numel[l]) for l in range(3)]

    def exchange_and_update(l):
        """Layer l's gradient: 8-bit exchange, then RMSprop on its weights - on the side stream, as soon as the gradient GEMM
        has finished (the reference starts its sends right after backward_grads, source/Layer.cpp:332-390).  The update
        waits for the backward product that still reads the old weights of this layer."""
        main_s = torch.cuda.current_stream()
        ev_grad[l].record(main_s)
        comm_stream.wait_event(ev_grad[l])
        if l > 0:
            comm_stream.wait_event(ev_err[l])
        cs = ctypes.c_void_p(comm_stream.cuda_stream)
        cn.check(lib.cn_grad_sync_8bit_rmsprop(h, grad[l].data_ptr(), seg1[l], 1, 0.0, rms_p[offs[l]:].data_ptr(), W[l].data_ptr(), 0.9, 0.006, cs))

    def one_step():
        sp = ctx.stream_ptr()                                                    # the capture stream while recording
        main_s = torch.cuda.current_stream()
        # forward: fused dot+bias+activation, dropout
        cn.check(lib.cn_dropout_dp(h, act[0].data_ptr(), out[0].data_ptr(), act[0].numel(), drops[0], d_seed.data_ptr(), 0, sp))
        for l in range(3):
            last = l == 2
            ctx.gemm(out[l], W[l], out=(out[l + 1] if last else act[l + 1]), bias=bias[l],
                     activation=_lib.ACT_LINEAR if last else _lib.ACT_RELU)
            if not last:
                cn.check(lib.cn_dropout_dp(h, act[l + 1].data_ptr(), out[l + 1].data_ptr(), act[l + 1].numel(), drops[l + 1], d_seed.data_ptr(),
                                           1 << (20 + l), sp))
        # output layer: softmax and error softmax - onehot(y) in one pass
        cn.check(lib.cn_softmax_error(h, out[3].data_ptr(), y.data_ptr(), out[3].data_ptr(), err[3].data_ptr(), B, 10, sp))
        # backward, last layer first; each layer's gradient goes to the exchange as soon as it exists
        for l in (2, 1, 0):
            ctx.gemm(act[l], err[l + 1], out=grad[l], transA=True)
            if l > 0:
                ctx.gemm(err[l + 1], W[l], out=err[l], transB=True)              # reads the old W[l]
                ev_err[l].record(main_s)
                cn.check(lib.cn_mul_activation_gradient(h, err[l].data_ptr(), act[l].data_ptr(), _lib.ACT_RELU, None, err[l].data_ptr(), err[l].numel(), sp))
            exchange_and_update(l)
        cn.check(lib.cn_seed_advance(h, d_seed.data_ptr(), sp))
        ev_updated.record(comm_stream)
        main_s.wait_event(ev_updated)                                            # the next forward pass needs the new weights

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
    # the same step recorded once in a CUDA graph and replayed (the dropout seed advances on the device; with several
    # ranks the all-gather of the gradient exchange is part of the recording)
    graph_ms, g = None, None
    try:
        if world > 1 and os.environ.get("CN_BENCH_GRAPH_MULTI", "1") != "1":
            raise RuntimeError("switched off for more than one rank (CN_BENCH_GRAPH_MULTI=0)")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            one_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            one_step()
    except Exception as exc:   # capture is an optimisation of the harness, not of the library
        graph_ms, g = f"no graph: {exc}"[:120], None
    captured = g is not None
    if world > 1:
        # every rank replays, or none does (a rank that replays alone would wait in the all-gather)
        t = torch.tensor([1 if captured else 0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if captured and not bool(t.item()):
            graph_ms = "no graph: another rank could not capture"
        captured = bool(t.item())
    if captured:
        for _ in range(3):
            g.replay()
        graph_ms = timed(g.replay)
    if world > 1:
        t = torch.tensor([ms_eager, graph_ms if captured else 0.0], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_eager = float(t[0].item())
        if captured:
            graph_ms = float(t[1].item())
    ms = min(ms_eager, graph_ms) if captured else ms_eager
    ctx.gemm_check()
    return {"workload": "config 4: MLP 784-1200-1200-10, batch 128 per GPU, 8-bit gradient exchange, RMSprop", "ms_per_step": ms,
            "ms_per_step_eager": ms_eager, "ms_per_step_cuda_graph": graph_ms,
            "samples_per_s": 128 * world / (ms * 1e-3), "launches_per_step": launches,
            "gradient_exchange": ("codes stored into the peers' memory by one kernel" if pushed else "ncclAllGather") if world > 1 else "none (one rank)",
            "flops_per_step_per_gpu": 6.0 * 128 * (784 * 1200 + 1200 * 1200 + 1200 * 10)}


def sample_cols(ncols, n_random, seed):
    """Columns of a shard to check: both ends, the neighbours of the first tile edges, and random ones."""
    rng_s = np.random.default_rng(seed)
    fixed = [0, 1, 127, 128, 129, 255, 256, 257, ncols - 2, ncols - 1]
    cols = np.unique(np.concatenate([fixed, rng_s.integers(0, max(ncols, 1), n_random)]))
    return cols[(cols >= 0) & (cols < ncols)]


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
    ap.add_argument("--no-extras", action="store_true", help="skip the TF32 leg, config 1, the config-5 sweep and the GPU comparators")
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
    cudart = ctypes.CDLL("libcudart.so.12")

    # ---- workload: weights sharded by columns, created on the owning rank (distributed_uniformSqrtWeight)
    s1, c1 = ctx.shard_cols(N1, rank, world)
    s2, c2 = ctx.shard_cols(N2, rank, world)
    seed = 0 + 10000 * rank + 12345
    W1 = ctx.empty(K1, c1)
    cn.check(lib.cn_uniform_sqrt_weight(ctx.h, W1.data_ptr(), W1.numel(), K1, N1, seed, 0, ctx.stream_ptr()))
    W2 = ctx.empty(N1, c2)
    cn.check(lib.cn_uniform_sqrt_weight(ctx.h, W2.data_ptr(), W2.numel(), N1, N2, seed + 1, 0, ctx.stream_ptr()))
    # data set of two batches, uniform [0,1) seed 0, on the host (row-major, pinned) of EVERY rank
    h_batch = torch.from_numpy(np.random.default_rng(0).random((M, K1), dtype=np.float32))
    h_set = torch.cat([h_batch, h_batch.flip(0)], 0).pin_memory()
    h_lab = torch.zeros((2 * M, 1), dtype=torch.float32).pin_memory()
    h_out = torch.empty((M, N2), dtype=torch.float32).pin_memory()
    d_stage_in = torch.empty((M, K1), dtype=torch.float32, device="cuda")
    d_stage_out = torch.empty((M, N2), dtype=torch.float32, device="cuda")
    batch = ctx.empty(M, K1)
    # outputs in symmetric buffers: the all-gather of each layer is fused into the GEMM epilogue (stores to peer memory)
    fused = world > 1 and args.exchange != "8bit" and not args.nccl_gather
    out1 = ctx.sym_empty(M, N1) if fused else ctx.empty(M, N1)
    out2 = ctx.sym_empty(M, N2) if fused else ctx.empty(M, N2)
    sp = ctx.stream_ptr()

    def upload(which=0):
        """Plain (untimed) upload of batch `which` of the data set into the resident column-major copy, on every rank."""
        cn.check(lib.cn_upload_row_major(ctx.h, h_set[which * M:(which + 1) * M].data_ptr(), d_stage_in.data_ptr(), batch.data_ptr(), M, K1, sp))

    coded = None
    if args.exchange == "8bit-fused":
        c_codes = torch.empty((N1, M), dtype=torch.uint8, device="cuda")
        c_scales = torch.zeros(world, dtype=torch.float32, device="cuda")
        c_own = torch.empty((c1, M), dtype=torch.float32, device="cuda")
        coded = _lib.Coded(c_codes.data_ptr(), c_scales.data_ptr(), c_own.data_ptr(), M, N1)
    no_epi = cn.Epilogue(None, 0, 0, None)

    def two_layers(a_ptr=None, gemm_mode=None, row_major=False):
        """The two sharded products.  a_ptr: device address of the batch (default: the resident column-major copy);
        row_major: a_ptr is the row-major batch, read as a transposed operand."""
        gm = mode if gemm_mode is None else gemm_mode
        a_ptr = ctypes.c_void_p(a_ptr if a_ptr is not None else batch.data_ptr())
        if coded is not None:
            cn.check(lib.cn_dotmpi_to_coded_f32(ctx.h, M, K1, N1, a_ptr, W1.data_ptr(), ctypes.byref(coded), ctypes.byref(no_epi), gm, sp))
            cn.check(lib.cn_dotmpi_from_coded_f32(ctx.h, ctypes.byref(coded), N2, W2.data_ptr(), out2.data_ptr(), ctypes.byref(no_epi), gm, 0, sp))
            return
        if row_major:
            cn.check(lib.cn_tdotmpi_f32(ctx.h, M, K1, N1, a_ptr, K1, W1.data_ptr(), out1.data_ptr(), ctypes.byref(no_epi), gm, exchange, sp))
        else:
            cn.check(lib.cn_dotmpi_f32(ctx.h, M, K1, N1, a_ptr, W1.data_ptr(), out1.data_ptr(), ctypes.byref(no_epi), gm, exchange, sp))
        ctx.dotmpi(out1, W2, N2, out=out2, mode=gm, exchange=exchange)

    # Layer 1's activation planes are made one step ahead on a second stream (cn_gemm_prepare), so that the pass over the
    # batch overlaps the previous step's products instead of preceding its own: two handles alternate; a handle is refilled
    # only after the product that read it has finished (ev_read), and a product starts only after its handle is filled
    # (ev_filled).  Every step still makes one set of planes - for its successor.
    use_prep = coded is None and os.environ.get("CN_BENCH_PREPARE", "1") == "1"
    prep, prep_stream, ev_filled, ev_read = [], None, [], []
    if use_prep:
        prep_stream = torch.cuda.Stream()              # default priority: below the stream of the timed loops (see there)
        for _ in range(2):
            hnd = ctypes.c_void_p()
            cn.check(lib.cn_gemm_prepare_create(ctx.h, M, K1, mode, ctypes.byref(hnd)))
            prep.append(hnd)
            ev_filled.append(torch.cuda.Event())
            ev_read.append(torch.cuda.Event())

    def prepare_planes(k, a_ptr=None, row_major=False, after=None):
        """Fill handle k from the batch at a_ptr on the second stream (after: an event the batch itself depends on)."""
        prep_stream.wait_event(ev_read[k])
        if after is not None:
            prep_stream.wait_event(after)
        a = ctypes.c_void_p(a_ptr if a_ptr is not None else batch.data_ptr())
        cn.check(lib.cn_gemm_prepare(ctx.h, prep[k], 1 if row_major else 0, a, K1 if row_major else M, ctypes.c_void_p(prep_stream.cuda_stream)))
        ev_filled[k].record(prep_stream)

    def two_layers_prepared(k):
        main_s = torch.cuda.current_stream()
        main_s.wait_event(ev_filled[k])
        cn.check(lib.cn_dotmpi_prepared_f32(ctx.h, prep[k], N1, W1.data_ptr(), out1.data_ptr(), ctypes.byref(no_epi), exchange, sp))
        ev_read[k].record(main_s)
        ctx.dotmpi(out1, W2, N2, out=out2, mode=mode, exchange=exchange)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def rest(seconds=1.5):
        """Every timed region starts from the same state: the GPUs idle for a moment first.  The products are bound by the
        1 kW power limit, so a region that follows seconds of load would otherwise be measured at lower clocks than the
        first one and the regions could not be compared with each other."""
        barrier()
        time.sleep(seconds)
        barrier()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def decoded_out1():
        """With the coded exchange out1 is never materialised: rebuild this rank's view of it for the checks."""
        if coded is None:
            return
        out1[s1:s1 + c1] = c_own
        for r in range(world):
            if r != rank:
                sr, cr = ctx.shard_cols(N1, r, world)
                ctx.decompress(c_codes[sr:sr + cr], c_scales[r:r + 1], out=out1[sr:sr + cr])

    # ---- accuracy over every rank's shard.  Rank r computes, in fp64 on the host, the product of the layer's input with a
    # sample of ITS OWN weight columns; rank 0 compares all ranks' references with the values in its own gathered copy of
    # the output, so that columns which arrived from a peer are checked; the gathered copies of all ranks are compared
    # with each other through a checksum of their bit patterns.
    def layer_check(act_dev, W_dev, out_dev, col0, ncols_local, seed_):
        cols = sample_cols(ncols_local, max(6, 54 // world), seed_ + rank)
        a64 = act_dev.T.double().cpu().numpy()                                # (M, K)
        w64 = W_dev[torch.from_numpy(cols).cuda()].double().cpu().numpy().T   # (K, ncols)
        mine = (cols + col0, a64 @ w64)
        allrefs = [mine]
        if world > 1:
            allrefs = [None] * world if rank == 0 else None
            dist.gather_object(mine, allrefs, dst=0)
        bits = out_dev.view(torch.int32).to(torch.int64)
        digest = torch.stack([bits.sum(), (bits * torch.arange(1, bits.shape[1] + 1, device="cuda")).sum()])
        same = True
        if world > 1:
            digests = [torch.zeros_like(digest) for _ in range(world)]
            dist.all_gather(digests, digest)
            same = all(bool(torch.equal(d, digests[0])) for d in digests)
        if rank != 0:
            return None
        scale = float(out_dev.abs().max().item())
        worst, nchecked = 0.0, 0
        for gcols, ref in allrefs:
            got = out_dev[torch.from_numpy(gcols).cuda()].double().cpu().numpy().T
            worst = max(worst, float(np.abs(got - ref).max() / scale))
            nchecked += len(gcols)
        return {"err": worst, "columns": nchecked, "replicas_identical": same}

    def accuracy(bound, label):
        decoded_out1()
        r1 = layer_check(batch, W1, out1, s1, c1, 7)
        r2 = layer_check(out1, W2, out2, s2, c2, 11)
        if rank != 0:
            return None
        # with an 8-bit exchange the peers' blocks of out1 are quantised: layer 1 is then checked on rank 0's own shard only
        lossy = args.exchange != "fp32" and world > 1
        ok = (r1["err"] <= bound or lossy) and r2["err"] <= bound and r1["replicas_identical"] and r2["replicas_identical"]
        return {"metric": "max |C - C64| / max |C| over sampled columns of every rank's shard (fp64 host product of the same inputs), "
                          "compared in rank 0's gathered copy; layer 2 takes the layer-1 output as its input",
                "mode": label, "layer1": r1["err"], "layer2": r2["err"], "bound": bound, "ok": bool(ok),
                "shards_checked": world, "columns_checked": [r1["columns"], r2["columns"]],
                "gathered_copies_identical_on_all_ranks": bool(r1["replicas_identical"] and r2["replicas_identical"]),
                **({"note": "8-bit exchange: the peers' blocks of layer 1 carry the codec's quantisation error by design"} if lossy else {})}

    upload(0)
    two_layers()          # first call: scratch buffers are allocated here, not inside a timed region
    ctx.gemm_check()
    # The products of the two timed loops run on a stream of raised priority and the plane-making stream keeps the default
    # one: where both have thread blocks waiting for an SM, the product goes first, and the planes take what it leaves
    # free (a few SMs during the products, all of them in between).  Everything after the loops is back on the default stream.
    torch.cuda.synchronize()
    torch.cuda.set_stream(torch.cuda.Stream(priority=-1))
    sp = ctx.stream_ptr()
    rest()
    step_no = 0

    def resident_step():
        nonlocal step_no
        if not use_prep:
            two_layers()
            return
        prepare_planes((step_no + 1) % 2)          # for the next step; overlaps this step's products
        two_layers_prepared(step_no % 2)
        step_no += 1

    if use_prep:
        prepare_planes(0)
    for _ in range(args.warmup):
        resident_step()

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
        resident_step()
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
    # the outputs of the last timed step were computed from the resident batch: check them now, before anything else runs
    acc_main = accuracy(TOL[args.mode], args.mode)

    # ---- the same step in the other precision mode (3xTF32 <-> TF32), reported separately with its own bound
    other = None
    if not args.no_extras and coded is None:
        oname = "tf32" if args.mode == "3xtf32" else "3xtf32"
        omode = _lib.GEMM_TF32 if oname == "tf32" else _lib.GEMM_3XTF32
        rest()
        for _ in range(2):
            two_layers(gemm_mode=omode)
        cn.check(lib.cn_gemm_profile_enable(ctx.h, 1))
        barrier()
        o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        osteps = max(5, args.steps // 2)
        o0.record()
        for _ in range(osteps):
            two_layers(gemm_mode=omode)
        o1.record()
        barrier()
        oms = max_over_ranks(o0.elapsed_time(o1)) / osteps
        obuf = (ctypes.c_float * (4 * osteps + 8))()
        cn.check(lib.cn_gemm_profile_read(ctx.h, obuf, len(obuf), ctypes.byref(cnt)))
        cn.check(lib.cn_gemm_profile_enable(ctx.h, 0))
        ok_ms = [obuf[i] for i in range(min(cnt.value, len(obuf)))]
        ol1 = max_over_ranks(float(np.mean(ok_ms[0::2]))) if ok_ms else None
        ctx.gemm_check()
        oacc = accuracy(TOL[oname], oname)
        if rank == 0:
            w_bytes_rank = 4.0 * K1 * (N1 / world)
            tensor_peak = peaks["bf16_tflops"] / 2.0 / (3.0 if oname == "3xtf32" else 1.0)
            hbm_bound = 2.0 * M / 4.0 * peaks["hbm_gbs"] / 1e3          # 64 flop per W byte x HBM GB/s -> TFLOP/s
            l1_tf = 2.0 * M * K1 * (N1 / world) / (ol1 * 1e-3) / 1e12 if ol1 else None
            other = {"mode": oname, "value": FLOPS_STEP / (oms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": oms, "steps": osteps,
                     "accuracy": oacc,
                     "roofline": {"kernel": "cn_gemm_tc_kernel (layer 1, per rank)", "bound": "hbm" if hbm_bound < tensor_peak else "tensor",
                                  "tensor_peak_tflops": tensor_peak, "hbm_bound_tflops": hbm_bound,
                                  "achieved_tflops": l1_tf, "ms_per_launch": ol1,
                                  "achieved": (w_bytes_rank / (ol1 * 1e-3) / 1e9) if ol1 else None, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                  "frac": (w_bytes_rank / (ol1 * 1e-3) / 1e9 / peaks["hbm_gbs"]) if ol1 else None,
                                  "note": "64 flop per weight byte: the single-pass TF32 mode streams W at the HBM roofline before it reaches the tensor peak; "
                                          "achieved = W bytes of the launch / its duration"}}
        two_layers()   # leave out1 / out2 in the main mode again

    # ---- timed region 2: end to end from host memory through the C ABI (see the module docstring)
    use_rm = coded is None
    bflags = _lib.BATCH_SHARDED_UPLOAD | (_lib.BATCH_NO_COL_MAJOR if use_rm else 0)
    if os.environ.get("CN_BENCH_PUSH_BY_KERNEL") == "1":
        bflags |= _lib.BATCH_PUSH_BY_KERNEL
    if world > 1 and os.environ.get("CN_BENCH_LOOKAHEAD", "1") == "1":
        bflags |= _lib.BATCH_LOOKAHEAD       # two uploads in flight: one upload's chain of waits may outlast a short step
    bh = ctypes.c_void_p()
    cn.check(lib.cn_batch_create_ex(ctx.h, h_set.data_ptr(), h_lab.data_ptr(), 2 * M, K1, 1, M, 0, bflags, ctypes.byref(bh)))
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
        main_s = torch.cuda.current_stream()
        main_s.wait_event(ev_drained)
        cn.check(lib.cn_to_row_major(ctx.h, out2.data_ptr(), d_stage_out.data_ptr(), M, N2, sp))
        ev_staged.record(main_s)
        copy_stream.wait_event(ev_staged)
        err = cudart.cudaMemcpyAsync(ctypes.c_void_p(h_out.data_ptr()), ctypes.c_void_p(d_stage_out.data_ptr()),
                                     ctypes.c_size_t(M * N2 * 4), 2, ctypes.c_void_p(copy_stream.cuda_stream))
        assert err == 0, f"cudaMemcpyAsync (device to host) failed: {err}"
        ev_drained.record(copy_stream)

    e2e_batches = []

    e2e_prep = use_prep and use_rm
    e2e_no = 0
    pnx, pnn = ctypes.c_void_p(), ctypes.c_int64()

    def e2e_step(upload_next=True, download_result=True):
        nonlocal e2e_no
        if upload_next:
            cn.check(lib.cn_batch_copy_next_async(bh))                 # upload of the NEXT batch (side stream, all ranks)
        if use_rm:
            cn.check(lib.cn_batch_current_row_major(bh, ctypes.byref(px), ctypes.byref(pn)))
        else:
            cn.check(lib.cn_batch_current(bh, ctypes.byref(px), ctypes.byref(py), ctypes.byref(pn)))
        if e2e_prep and upload_next:
            # the planes of the NEXT batch are made on the second stream as soon as its upload has arrived, beside this
            # step's products; this step's own planes were made during the step before
            cn.check(lib.cn_batch_next_row_major(bh, ctypes.c_void_p(prep_stream.cuda_stream), ctypes.byref(pnx), ctypes.byref(pnn)))
            prepare_planes((e2e_no + 1) % 2, pnx.value, row_major=True)
            two_layers_prepared(e2e_no % 2)
            e2e_no += 1
        else:
            two_layers(px.value, row_major=use_rm)
        if download_result:
            download_overlapped()
        if upload_next:
            cn.check(lib.cn_batch_swap(bh, sp, ctypes.byref(px), ctypes.byref(py), ctypes.byref(pn)))
            e2e_batches.append(len(e2e_batches) % 2)                   # the allocator walks batch 0, 1, 0, 1, ...

    def e2e_prime():
        """Planes of the batch that is current now (the steps make them for their successor only)."""
        if e2e_prep:
            cn.check(lib.cn_batch_current_row_major(bh, ctypes.byref(px), ctypes.byref(pn)))
            ev_now = torch.cuda.Event()
            ev_now.record(torch.cuda.current_stream())
            prepare_planes(e2e_no % 2, px.value, row_major=True, after=ev_now)

    e2e_prime()
    rest()
    for _ in range(args.warmup):
        e2e_step()
    sampler2 = ClockSampler(local_rank)
    if rank == 0:
        sampler2.start()
        time.sleep(0.25)
    barrier()
    t_wall2 = time.time()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(args.steps):
        e2e_step()
    if rank == 0:
        torch.cuda.current_stream().wait_event(ev_drained)   # the last step's result must be on the host inside the timed region
    e3.record()
    barrier()
    t_wall3 = time.time()
    ms_e2e = max_over_ranks(e2.elapsed_time(e3))
    clocks_e2e = sampler2.stop(t_wall2, t_wall3) if rank == 0 else None
    ctx.gemm_check()
    e2e_diag = None
    if os.environ.get("CN_BENCH_E2E_DIAG") == "1":
        # where the end-to-end step spends its time beyond the two products: the same loop without the download, without
        # the upload of the next batch, and without either (analysis aid; not part of any reported figure)
        e2e_diag = {}
        for name, up, down in (("full", True, True), ("no_download", True, False), ("no_upload", False, True), ("products_only", False, False)):
            rest()
            for _ in range(3):
                e2e_step(up, down)
            barrier()
            d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            d0.record()
            h0 = time.perf_counter()
            for _ in range(10):
                e2e_step(up, down)
            host_ms = (time.perf_counter() - h0) * 100.0          # time the host needs to ISSUE one step (no synchronisation)
            if rank == 0:
                torch.cuda.current_stream().wait_event(ev_drained)
            d1.record()
            barrier()
            e2e_diag[name] = max_over_ranks(d0.elapsed_time(d1)) / 10
            e2e_diag[name + "_host_issue"] = max_over_ranks(host_ms)
        # phases of the sharded upload on the copy stream (max over ranks, mean of 6 steps)
        if world > 1:
            ph = (ctypes.c_float * 4)()
            cn.check(lib.cn_batch_profile(bh, 1, ph))
            acc4 = np.zeros(4)
            for _ in range(7):
                e2e_step(True, True)
                cn.check(lib.cn_batch_profile(bh, 1, ph))
                acc4 += np.array(list(ph))
            cn.check(lib.cn_batch_profile(bh, 0, ph))
            t4 = torch.tensor(acc4 / 7, dtype=torch.float64, device="cuda")
            dist.all_reduce(t4, op=dist.ReduceOp.MAX)
            e2e_diag["upload_phases_ms(wait_free,h2d,push,wait_arrived)"] = [round(float(v), 4) for v in t4.tolist()]
        e2e_step(True, True)          # a last full step, so that the host result and the record of its batch agree again
        if rank == 0:
            torch.cuda.current_stream().wait_event(ev_drained)
        barrier()
        if rank == 0:
            print(f"bench.py: e2e diagnosis (ms per step): {e2e_diag}", file=sys.stderr, flush=True)
    lib.cn_batch_destroy(bh)
    torch.cuda.synchronize()
    for hnd in prep:
        lib.cn_gemm_prepare_destroy(hnd)
    barrier()
    # the end-to-end result, as it arrived on the host, against the resident path on the batch that step used: the two
    # paths differ only in how the batch reaches the product, so they must agree bit for bit; the resident recomputation
    # is then checked against fp64 like the main result
    last = e2e_batches[-1]
    upload(last)
    two_layers()
    ctx.gemm_check()
    acc_e2e = accuracy(TOL[args.mode], args.mode)
    e2e_match = None
    if rank == 0:
        cn.check(lib.cn_to_row_major(ctx.h, out2.data_ptr(), d_stage_out.data_ptr(), M, N2, sp))
        torch.cuda.synchronize()
        e2e_match = bool(torch.equal(d_stage_out.cpu(), h_out))
    checksum = float(h_out.double().abs().mean())
    upload(0)
    torch.cuda.synchronize()
    torch.cuda.set_stream(torch.cuda.default_stream())
    sp = ctx.stream_ptr()

    multi = multi_rank_checks(ctx, cn, _lib, torch, dist, world, rank) if world > 1 else None
    train = None if (args.no_train_step or not headline) else train_step_bench(ctx, cn, _lib, torch, dist if world > 1 else None, world, rank)
    extras = None
    if not args.no_extras and headline:
        extras = extra_measurements(ctx, cn, _lib, torch, dist, world, rank, peaks)

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
    e2e_ok = bool(e2e_match and acc_e2e["ok"])
    line = {
        "metric": "dotMPI TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": ("README dotMPI two-layer skinny GEMM: " if headline else "REDUCED (profiling) two-layer skinny GEMM: ") +
                               f"128x{K1} . {K1}x{N1} . {N1}x{N2}, W column-sharded",
                   "gemm_mode": args.mode, "exchange": args.exchange, "gather": ("fused peer stores" if fused else ("nccl" if world > 1 else "none")), "parallelism": f"tp{world} (columns of W)",
                   "activation_planes": ("layer 1's TF32 hi/lo planes are made one step ahead on a second stream (cn_gemm_prepare): every step makes "
                                         "the planes of its successor beside its own products" if use_prep else "made inside each product call"),
                   "timed_regions": "each starts after 1.5 s of idle GPUs and its own warm-up steps (the products are power-limited)",
                   "l2": f"inputs larger than L2 ({4e-9 * (K1 * N1 + N1 * N2):.1f} GB of weights stream once per step)", "flops_per_step": FLOPS_STEP},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": M * K1 * 4,
                "h2d_bytes_per_step_per_rank": M * K1 * 4 // world, "d2h_bytes_per_step": M * N2 * 4, "result_checksum": checksum,
                "upload": (f"each of the {world} ranks uploads 1/{world} of the batch rows over its own PCIe link, blocks exchanged over NVLink" if world > 1
                           else "one rank, whole batch") + ("; row-major batch read as a transposed operand" if use_rm else ""),
                "host_result_equals_resident_path_bitwise": e2e_match, "accuracy_of_that_batch": acc_e2e, "ok": e2e_ok, "clocks": clocks_e2e},
        "accuracy": acc_main,
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"kernel": "cn_gemm_tc_kernel (layer 1, per rank; with its split-K reduction)", "bound": "tensor", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": (achieved / peak) if achieved else None,
                     # DRAM bytes per launch: one ncu capture of a 128 x 100000 x 4096 launch read 1.772 GB for 1.6384 GB of
                     # W; scaled here by the W bytes of this rank's layer-1 launch
                     "traffic": 1.772e9 / 1.6384e9 * 4.0 * K1 * (N1 // world if world > 1 else N1),
                     "traffic_source": "ncu dram__bytes_read+write of a 4096-column case, scaled by W bytes",
                     "ms_per_launch": l1_ms, "layer2_ms_per_launch": l2_ms,
                     "peak_source": f"{peaks['source']} burst: bf16_tflops {peaks['bf16_tflops']} / 2 (TF32 rate)" + (" / 3 (three TF32 products per tile)" if args.mode == "3xtf32" else ""),
                     # side note: the same against the power-capped (seconds-long) cuBLAS figure
                     "frac_sustained": (achieved / (peaks["bf16_tflops_sustained"] / 2.0 / (3.0 if args.mode == "3xtf32" else 1.0))) if achieved else None,
                     "hbm_frac_layer1": (4.0 * K1 * (N1 / world) / (l1_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]) if l1_ms else None},
    }
    if other:
        line[other["mode"]] = other
    if multi:
        line["multi_rank_checks"] = multi
    if train:
        line["train_step"] = train
    if extras:
        line.update(extras)
    if not args.no_codec and world == 1:
        line["codec"] = codec_bench(ctx, torch, peaks)
    if not args.no_cpu_baseline and world == 1:
        torch.cuda.synchronize()
        r = cpu_sgemm_steps(steps=5, warmup=1)
        line["cpu_baseline"] = {"value": r["value"], "unit": "TFLOP/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]}
    failed = []
    if not acc_main["ok"]:
        failed.append("accuracy")
    if not e2e_ok:
        failed.append("e2e")
    if other and not other["accuracy"]["ok"]:
        failed.append(other["mode"] + ".accuracy")
    if multi and not multi["ok"]:
        failed.append("multi_rank_checks")
    line["checks_failed"] = failed
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        print(f"bench.py: FAILED checks: {failed}", file=sys.stderr, flush=True)
        sys.exit(3)


def multi_rank_checks(ctx, cn, _lib, torch, dist, world, rank):
    """Correctness of everything that crosses GPUs, small and exact, on every bench run with more than one rank:
    the reference's own multi-rank pins (tests/clusterNet_test.cu:257-276: dotMPI == dot elementwise on constant
    matrices; :338-394: all-ones sharded weight, dot -> 8783, dotTMPI -> 317, dot into the sharded matrix -> 17) and the
    8-bit paths, each checked against the same computation composed from single-GPU kernels."""
    res = {"ranks": world}
    dev = "cuda"

    def all_true(flag):
        t = torch.tensor([1 if flag else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())
    # dotMPI == dot, elementwise exact, 200x400 . 400x800 constants; plain NCCL gather and the fused peer-store gather
    A = torch.full((400, 200), 0.3, device=dev)
    B = torch.full((800, 400), 1.1748345, device=dev)
    s0, c0 = ctx.shard_cols(800, rank, world)
    full = ctx.gemm(A, B)
    C = ctx.dotmpi(A, B[s0:s0 + c0].contiguous(), 800)
    Cs = ctx.sym_empty(200, 800)
    Cs.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    ctx.dotmpi(A, B[s0:s0 + c0].contiguous(), 800, out=Cs)
    ctx.gemm_check()
    res["dotmpi_equals_dot_exact"] = all_true(torch.equal(C, full))
    res["fused_gather_equals_nccl_gather_exact"] = all_true(torch.equal(Cs, C))
    # random data, uneven shards (N % G != 0), bias + ReLU through the fused gather and through NCCL: identical, and
    # equal to the unsharded product up to the split-K schedule
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    Mx, Kx, Nx = 128, 4096, 2048 + 256 * world + 4
    A = torch.rand((Kx, Mx), device=dev, generator=g) * 2 - 1
    W = torch.rand((Nx, Kx), device=dev, generator=g) * 2 - 1
    bias = torch.rand(Nx, device=dev, generator=g)
    s0, c0 = ctx.shard_cols(Nx, rank, world)
    Wsh = W[s0:s0 + c0].contiguous()
    full = ctx.gemm(A, W, bias=bias, activation=_lib.ACT_RELU)
    Cn = ctx.dotmpi(A, Wsh, Nx, bias=bias, activation=_lib.ACT_RELU)
    Cf = ctx.sym_empty(Mx, Nx)
    ok_f = True
    for rep in range(2):
        Cf.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        ctx.dotmpi(A, Wsh, Nx, out=Cf, bias=bias, activation=_lib.ACT_RELU)
        ctx.gemm_check()
        ok_f = ok_f and bool(torch.equal(Cf, Cn))
    res["uneven_shards_fused_equals_nccl_exact"] = all_true(ok_f)
    ref = torch.relu(A.double().T @ W.double().T + bias.double())            # (M, N) fp64 on the GPU (library, checker only)
    err = float(((Cn.T.double() - ref).abs().max() / ref.abs().max()).item())
    res["uneven_shards_vs_fp64"] = err
    res["uneven_shards_vs_unsharded"] = float(((Cn - full).abs().max() / ref.abs().max()).item())
    # TdotMPI (transposed first operand, sharded B) == dotMPI
    At = A.T.contiguous()                                                     # stored K x M column-major = (M, K) tensor
    Ct = ctx.empty(Mx, Nx)
    epi = cn.Epilogue(bias.data_ptr(), _lib.ACT_RELU, 0, None)
    cn.check(ctx.lib.cn_tdotmpi_f32(ctx.h, Mx, Kx, Nx, At.data_ptr(), Kx, Wsh.data_ptr(), Ct.data_ptr(), ctypes.byref(epi), _lib.GEMM_3XTF32, 0,
                                    ctx.stream_ptr()))
    res["tdotmpi_equals_dotmpi_exact"] = all_true(torch.equal(Ct, Cn))
    # all-ones 8783 x 317 sharded weight
    s0, c0 = ctx.shard_cols(317, rank, world)
    m1 = torch.ones((c0, 8783), device=dev)
    m2, m3, m4 = torch.ones((8783, 111), device=dev), torch.ones((317, 17), device=dev), torch.ones((17, 8783), device=dev)
    ok = True
    for _ in range(2):
        d = ctx.dotmpi(m2, m1, 317)
        ok = ok and bool((d == 8783.0).all())
        t = ctx.dottmpi(m3, m1)
        ok = ok and bool((t == 317.0).all())
        ctx.dot_sharded_out(m4, m3, m1)
        ok = ok and bool((m1 == 17.0).all())
        m1.fill_(1.0)
    res["ones_8783_317_17_exact"] = all_true(ok)
    # dotTMPI on random data against fp64
    Ar = torch.rand((400, 64), device=dev, generator=g) * 2 - 1               # A 64 x 400
    Bf = torch.rand((400, 96), device=dev, generator=g) * 2 - 1               # B 96 x 400 (full), sharded by columns
    s0, c0 = ctx.shard_cols(400, rank, world)
    got = ctx.dottmpi(Ar, Bf[s0:s0 + c0].contiguous())
    ref = Ar.double().T @ Bf.double()                                         # (64 x 400) . (400 x 96)
    res["dottmpi_vs_fp64"] = float(((got.T.double() - ref).abs().max() / ref.abs().max()).item())
    # 8-bit exchange of C: own block exact, peers' blocks = decompress(compress(block, absmax(block))) with the single-GPU kernels
    C8 = ctx.dotmpi(A, Wsh, Nx, bias=bias, activation=_lib.ACT_RELU, exchange=1)
    ok = True
    for r in range(world):
        sr, cr = ctx.shard_cols(Nx, r, world)
        blk = Cn[sr:sr + cr].contiguous()
        if r == rank:
            ok = ok and bool(torch.equal(C8[sr:sr + cr], blk))
        else:
            pm = ctx.absmax(blk)
            ok = ok and bool(torch.equal(C8[sr:sr + cr], ctx.decompress(ctx.compress(blk, pm), pm)))
    res["exchange_8bit_equals_single_gpu_codec_exact"] = all_true(ok)
    # 8-bit exchange decoded in the consumer's prologue == decoding first
    W2 = torch.rand((512, Nx), device=dev, generator=g) * 2 - 1
    s2, c2 = ctx.shard_cols(512, rank, world)
    W2sh = W2[s2:s2 + c2].contiguous()
    ref2 = ctx.dotmpi(C8, W2sh, 512)
    coded, keep = ctx.dotmpi_to_coded(A, Wsh, Nx, bias=bias, activation=_lib.ACT_RELU, rank=rank, nranks=world)
    got2 = ctx.dotmpi_from_coded(coded, W2sh, 512)
    ctx.gemm_check()
    res["coded_chain_equals_decode_first_exact"] = all_true(torch.equal(got2, ref2))
    # 8-bit gradient exchange: own gradient + decode(encode(peer gradient)) in rank order, single call and packed call
    n = 70001
    grads = []
    for r in range(world):
        gg = torch.Generator(device=dev)
        gg.manual_seed(100 + r)
        grads.append(torch.randn(n, device=dev, generator=gg) * (0.01 * (r + 1)))
    want = grads[rank].clone()
    for r in range(world):
        if r != rank:
            pm = ctx.absmax(grads[r])
            want = want + ctx.decompress(ctx.compress(grads[r], pm), pm)
    gmine = grads[rank].clone()
    cn.check(ctx.lib.cn_grad_sync_8bit(ctx.h, gmine.data_ptr(), n, 0.0, ctx.stream_ptr()))
    res["grad_sync_8bit_equals_single_gpu_codec_exact"] = all_true(torch.equal(gmine, want))
    segs = [30001, 40000]
    gpk = grads[rank].clone()
    seg = (ctypes.c_int64 * 2)(*segs)
    cn.check(ctx.lib.cn_grad_sync_8bit_multi(ctx.h, gpk.data_ptr(), seg, 2, 0.0, ctx.stream_ptr()))
    want2 = grads[rank].clone()
    o = 0
    for sz in segs:
        for r in range(world):
            if r != rank:
                piece = grads[r][o:o + sz].contiguous()
                pm = ctx.absmax(piece)
                want2[o:o + sz] += ctx.decompress(ctx.compress(piece, pm), pm)
        o += sz
    res["grad_sync_packed_equals_single_gpu_codec_exact"] = all_true(torch.equal(gpk, want2))
    ctx.gemm_check()
    torch.cuda.synchronize()
    dist.barrier()
    exact = [k for k in res if k.endswith("_exact")]
    res["ok"] = bool(all(res[k] for k in exact) and res["uneven_shards_vs_fp64"] <= 1e-5 and res["dottmpi_vs_fp64"] <= 1e-5
                     and res["uneven_shards_vs_unsharded"] <= 5e-6)   # sharded and unsharded launches split K differently
    return res


def extra_measurements(ctx, cn, _lib, torch, dist, world, rank, peaks):
    """Config 1 latency, config-5 sweep points and, on one GPU, the same-box comparators (library kernels and the
    reference's own codec kernels) - all outside the product's timed regions; a few seconds in total."""
    out = {}
    dev = "cuda"
    g = torch.Generator(device=dev)
    g.manual_seed(0)

    def rnd(rows, cols):
        return torch.rand((cols, rows), device=dev, generator=g) * 2 - 1       # column-major rows x cols

    def sampled_err(A, W, C, nrow=64, ncol=32):
        """max |C - C64| / max |C| on a sample of rows and columns, fp64 product on the GPU (checker only)."""
        Mx, Nx = A.shape[1], W.shape[0]
        ri = torch.randint(0, Mx, (min(nrow, Mx),), device=dev, generator=g)
        ci = torch.randint(0, Nx, (min(ncol, Nx),), device=dev, generator=g)
        ref = A[:, ri].double().T @ W[ci].double().T
        got = C[ci][:, ri].double().T
        return float(((got - ref).abs().max() / C.abs().max().double()).item())
    if rank == 0:
        # config 1: 128x784 . 784x1024 + bias + ReLU, uniform(-1, 1)
        A, W, b = rnd(128, 784), rnd(784, 1024), torch.rand(1024, device=dev, generator=g) * 2 - 1
        C = ctx.empty(128, 1024)
        c1res = {"workload": "config 1: 128x784 . 784x1024 + bias + ReLU"}
        for name, md in (("3xtf32", _lib.GEMM_3XTF32), ("tf32", _lib.GEMM_TF32), ("fp32_simt", _lib.GEMM_FP32_SIMT)):
            ms = cuda_time(torch, lambda: ctx.gemm(A, W, out=C, bias=b, activation=_lib.ACT_RELU, mode=md), 50, 3)
            ref = torch.relu(A.double().T @ W.double().T + b.double())
            c1res[name] = {"us": round(ms * 1e3, 2), "err": float(((C.T.double() - ref).abs().max() / ref.abs().max()).item())}
        ms = cuda_time(torch, lambda: torch.relu(torch.addmm(b, A.T, W.T)), 50, 3)
        c1res["torch_addmm_relu_fp32"] = {"us": round(ms * 1e3, 2), "note": "library comparator (cuBLAS sgemm + elementwise), not on the product path"}
        out["config1"] = c1res
    # config 5 sweep (the points that fit a few seconds): square n^3 and skinny 128 x n x n, both modes, on rank 0's GPU;
    # with more than one rank the skinny 40000 point also runs sharded, with and without the 8-bit gather
    sweep = []
    if rank == 0:
        free = torch.cuda.mem_get_info()[0]
        pts = [("square", 4096, 4096, 4096), ("square", 8192, 8192, 8192), ("skinny", 128, 10000, 10000), ("skinny", 128, 40000, 40000)]
        if world == 1 and free > 60e9:
            pts.append(("skinny", 128, 100000, 100000))
        for kind, Mx, Kx, Nx in pts:
            A, W = rnd(Mx, Kx), ctx.empty(Kx, Nx)
            cn.check(ctx.lib.cn_rand_uniform(ctx.h, W.data_ptr(), W.numel(), 77, 0, ctx.stream_ptr()))
            W.mul_(2).sub_(1)
            C = ctx.empty(Mx, Nx)
            entry = {"shape": f"{Mx}x{Kx} . {Kx}x{Nx}", "kind": kind}
            for name, md in (("3xtf32", _lib.GEMM_3XTF32), ("tf32", _lib.GEMM_TF32)):
                iters = 3 if Kx * Nx > 2e9 else 8
                ms = cuda_time(torch, lambda: ctx.gemm(A, W, out=C, mode=md), iters, 2)
                entry[name] = {"TFLOP/s": round(2.0 * Mx * Kx * Nx / (ms * 1e-3) / 1e12, 1), "ms": round(ms, 4), "err": sampled_err(A, W, C)}
            ctx.gemm_check()
            sweep.append(entry)
            del A, W, C
            torch.cuda.empty_cache()
    if world > 1:
        Mx, Kx, Nx = 128, 40000, 40000
        s0, c0 = ctx.shard_cols(Nx, rank, world)
        A = ctx.empty(Mx, Kx)
        cn.check(ctx.lib.cn_rand_uniform(ctx.h, A.data_ptr(), A.numel(), 5, 0, ctx.stream_ptr()))   # same seed: same A on every rank
        Wsh = ctx.empty(Kx, c0)
        cn.check(ctx.lib.cn_rand_uniform(ctx.h, Wsh.data_ptr(), Wsh.numel(), 1000 + rank, 0, ctx.stream_ptr()))
        Cs = ctx.sym_empty(Mx, Nx)
        Cp = ctx.empty(Mx, Nx)
        entry = {"shape": f"{Mx}x{Kx} . {Kx}x{Nx} sharded over {world} ranks", "kind": "skinny, dotMPI"}
        for name, fn in (("fp32_fused_gather", lambda: ctx.dotmpi(A, Wsh, Nx, out=Cs)),
                         ("fp32_nccl_gather", lambda: ctx.dotmpi(A, Wsh, Nx, out=Cp)),
                         ("8bit_gather", lambda: ctx.dotmpi(A, Wsh, Nx, out=Cp, exchange=1))):
            torch.cuda.synchronize()
            dist.barrier()
            ms = cuda_time(torch, fn, 8, 2)
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            entry[name] = {"TFLOP/s": round(2.0 * Mx * Kx * Nx / (float(t.item()) * 1e-3) / 1e12, 1), "ms": round(float(t.item()), 4)}
        ctx.gemm_check()
        if rank == 0:
            sweep.append(entry)
    if rank == 0:
        out["sweep"] = sweep
    if world == 1:
        out["gpu_comparators"] = gpu_comparators(ctx, cn, _lib, torch, peaks)
    return out


def gpu_comparators(ctx, cn, _lib, torch, peaks):
    """Same-box comparators, bench-only and labelled: (1) the library call the reference makes for its product,
    cublasSgemm (source/clusterNet.cpp:459-461), reached through torch.matmul with TF32 off, on the per-rank shapes of
    both layers; (2) the reference's own codec kernels compiled for sm_100a (oracle/_ref, test infrastructure) timed on
    config 2 and on the reference's compression_test shape (source/test.cu:2037-2057: 5120 x 5120, N(0,1)/10, precision
    0.1), beside the product's kernels on the same data.  Nothing here is on the product path."""
    res = {"note": "library / reference kernels timed for comparison only; never linked into or called by the product"}
    dev = "cuda"
    prev = torch.backends.cuda.matmul.allow_tf32
    try:
        sg = {}
        for label, Mx, Kx, Nx in (("layer1_128x100000x40000", M, K1, N1), ("layer2_128x40000x20000", M, N1, N2)):
            A = torch.rand((Mx, Kx), device=dev)
            W = torch.rand((Nx, Kx), device=dev)
            entry = {}
            for name, tf in (("cublas_sgemm_fp32", False), ("cublas_tf32", True)):
                torch.backends.cuda.matmul.allow_tf32 = tf
                ms = cuda_time(torch, lambda: torch.matmul(A, W.T), 3, 1)
                entry[name] = {"TFLOP/s": round(2.0 * Mx * Kx * Nx / (ms * 1e-3) / 1e12, 1), "ms": round(ms, 3)}
            Ac, Wc, C = A.T.contiguous(), W, ctx.empty(Mx, Nx)     # column-major views of the same data
            for name, md in (("ours_3xtf32", _lib.GEMM_3XTF32), ("ours_tf32", _lib.GEMM_TF32)):
                ms = cuda_time(torch, lambda: ctx.gemm(Ac, Wc, out=C, mode=md), 3, 1)
                entry[name] = {"TFLOP/s": round(2.0 * Mx * Kx * Nx / (ms * 1e-3) / 1e12, 1), "ms": round(ms, 3)}
            sg[label] = entry
            del A, W, Ac, C
            torch.cuda.empty_cache()
        res["sgemm"] = sg
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libcnref.so")
    if not os.path.exists(ref_path):
        res["reference_codec_kernels"] = "oracle/_ref/libcnref.so is not built on this box"
        return res
    ref = ctypes.CDLL(ref_path)
    if not hasattr(ref, "ref_compression_8bit_async"):
        res["reference_codec_kernels"] = "oracle/_ref/libcnref.so predates the asynchronous launchers: rebuild it (make -C oracle ref)"
        return res
    ref.ref_compression_8bit_async.restype = None
    ref.ref_decompression_8bit_async.restype = None
    tbl = torch.from_numpy(ctx.codebook.copy()).cuda()
    codec = {}
    for label, n, p, sigma in (("config2_4096x4096", 4096 * 4096, None, 0.1), ("compression_test_5120x5120_precision_0.1", 5120 * 5120, 0.1, 0.1)):
        sets = 5
        xs = [torch.randn(n, device=dev) * sigma for _ in range(sets)]
        codes = [torch.empty(n, dtype=torch.uint8, device=dev) for _ in range(sets)]
        outs = [torch.empty(n, device=dev) for _ in range(sets)]
        prec = p if p is not None else float(ctx.absmax(xs[0]).item())
        entry = {"precision": prec}
        k = [0]

        def rot(fn):
            def run():
                fn(k[0] % sets)
                k[0] += 1
            return run
        pairs = (("compress", 5, lambda i: ctx.compress(xs[i], prec, out=codes[i]),
                  lambda i: ref.ref_compression_8bit_async(ctypes.c_void_p(tbl.data_ptr()), ctypes.c_void_p(xs[i].data_ptr()), ctypes.c_float(prec), n,
                                                     ctypes.c_void_p(codes[i].data_ptr()))),
                 ("decompress", 5, lambda i: ctx.decompress(codes[i], prec, out=outs[i]),
                  lambda i: ref.ref_decompression_8bit_async(ctypes.c_void_p(tbl.data_ptr()), ctypes.c_void_p(codes[i].data_ptr()), ctypes.c_float(prec), n,
                                                       ctypes.c_void_p(outs[i].data_ptr()))))
        for name, bpe, ours, theirs in pairs:
            ms_o = cuda_time(torch, rot(ours), 20, sets)
            ms_r = cuda_time(torch, rot(theirs), 10, sets)     # the reference launches on the NULL stream, which orders with torch's
            entry[name] = {"ours_us": round(ms_o * 1e3, 2), "ours_GB/s": round(n * bpe / ms_o / 1e6, 1),
                           "reference_kernel_us": round(ms_r * 1e3, 2), "reference_kernel_GB/s": round(n * bpe / ms_r / 1e6, 1),
                           "speedup": round(ms_r / ms_o, 2)}
        codec[label] = entry
        del xs, codes, outs
        torch.cuda.empty_cache()
    res["reference_codec_kernels"] = codec
    return res


if __name__ == "__main__":
    main()
