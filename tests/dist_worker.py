"""Worker of the multi-rank tests (launched by torchrun from tests/test_dist*.py).

    backend nccl: one rank per GPU, sharded product through cn_dotmpi_f32, checked against the single-GPU product
    backend gloo: CPU ranks; the same sharding arithmetic (cn_shard_cols) and gather order with numpy products
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import ctypes  # noqa: E402

import clusternet_b200 as cn  # noqa: E402
from clusternet_b200 import _lib  # noqa: E402
from oracle import oracle  # noqa: E402


def shard(lib, n, r, g):
    a, b = ctypes.c_int64(), ctypes.c_int64()
    cn.check(lib.cn_shard_cols(n, r, g, ctypes.byref(a), ctypes.byref(b)))
    return a.value, b.value


def run_gloo():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    lib = cn.load()
    rng = np.random.default_rng(0)
    for (M, K, N) in [(8, 16, 10), (4, 7, 2 * world), (3, 5, world + 1), (16, 32, 101)]:
        A = rng.standard_normal((M, K))
        W = rng.standard_normal((K, N))
        s0, c0 = shard(lib, N, rank, world)
        local = A @ W[:, s0:s0 + c0]
        # column-major full C: shard r is the contiguous block [M*start_r, M*(start_r+count_r))
        full = np.zeros(M * N)
        full[M * s0:M * (s0 + c0)] = local.T.ravel()
        t = torch.from_numpy(full)
        for r in range(world):                      # grouped broadcasts, the uneven-shard form of the gather
            sr, cr = shard(lib, N, r, world)
            blk = t[M * sr:M * (sr + cr)]
            if cr:
                dist.broadcast(blk, src=r)
        got = t.numpy().reshape(N, M).T
        assert np.allclose(got, A @ W), (M, K, N)
        assert sum(shard(lib, N, r, world)[1] for r in range(world)) == N
    dist.barrier()
    if rank == 0:
        print("GLOO-OK")


def run_nccl():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = cn.Context(local)
    ids = [ctx.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    ctx.comm_init(ids[0], rank, world)
    assert ctx.lib.cn_comm_rank(ctx.h) == rank and ctx.lib.cn_comm_size(ctx.h) == world
    rng = np.random.default_rng(5)
    for (M, K, N) in [(128, 512, 1024), (128, 256, 1000 + world + 1), (64, 384, 272)]:
        A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        W = rng.uniform(-1, 1, (K, N)).astype(np.float32)
        bias = rng.uniform(-1, 1, N).astype(np.float32)
        dA = ctx.colmajor(A if rank == 0 else np.zeros_like(A))
        ctx.bcast(dA, 0)                                        # "A is broadcast"
        s0, c0 = ctx.shard_cols(N, rank, world)
        dW = ctx.colmajor(np.ascontiguousarray(W[:, s0:s0 + c0]))
        db = torch.from_numpy(bias).cuda()
        full = ctx.gemm(dA, ctx.colmajor(W), bias=db, activation=_lib.ACT_RELU)
        C = ctx.dotmpi(dA, dW, N, bias=db, activation=_lib.ACT_RELU)
        ctx.gemm_check()
        ref = np.maximum(oracle.gemm_f64(A, W) + bias, 0)
        got = ctx.to_numpy(C)
        assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-5, (M, K, N)
        # sharded == unsharded up to the different split-K schedules of the two launches
        assert np.abs(got - ctx.to_numpy(full)).max() / np.abs(ref).max() < 2e-6
        # fused GEMM -> all-gather through symmetric buffers: identical to the NCCL gather, twice in a row (epochs)
        Cs = ctx.sym_empty(M, N)
        for rep in range(2):
            Cs.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            ctx.dotmpi(dA, dW, N, out=Cs, bias=db, activation=_lib.ACT_RELU)
            ctx.gemm_check()
            assert torch.equal(Cs, C), (M, K, N, rep, float((Cs - C).abs().max()))
        # 8-bit exchange: own slice exact, peers' slices = decode(encode(slice, absmax of that slice))
        C8 = ctx.dotmpi(dA, dW, N, bias=db, activation=_lib.ACT_RELU, exchange=1)
        ctx.gemm_check()
        got8 = ctx.to_numpy(C8)
        for r in range(world):
            sr, cr = ctx.shard_cols(N, r, world)
            sl = np.ascontiguousarray(got[:, sr:sr + cr].T)       # column-major element order of the slice
            if r == rank:
                assert np.array_equal(got8[:, sr:sr + cr], got[:, sr:sr + cr])
            else:
                p = oracle.absmax(sl)
                want = oracle.decompress(ctx.codebook, oracle.compress(ctx.codebook, sl, p), p)
                assert np.array_equal(got8[:, sr:sr + cr], want.reshape(cr, M).T), (M, K, N, r)
    # tests/clusterNet_test.cu:338-394: sharded all-ones weight 8783 x 317; dot -> 8783, dotTMPI -> 317, dot into the
    # sharded matrix -> 17, exactly, over several epochs
    s0, c0 = ctx.shard_cols(317, rank, world)
    m1 = torch.ones((c0, 8783), device="cuda")                   # local shard 8783 x c0 (column-major)
    m2, m3, m4 = torch.ones((8783, 111), device="cuda"), torch.ones((317, 17), device="cuda"), torch.ones((17, 8783), device="cuda")
    for epoch in range(2):
        d = ctx.dotmpi(m2, m1, 317)
        assert d.shape == (317, 111) and bool((d == 8783.0).all())
        t = ctx.dottmpi(m3, m1)
        assert t.shape == (8783, 17) and bool((t == 317.0).all())
        ctx.dot_sharded_out(m4, m3, m1)
        assert bool((m1 == 17.0).all())
        m1.fill_(1.0)
    # random data: dotTMPI and TdotMPI against fp64
    A = rng.uniform(-1, 1, (64, 400)).astype(np.float32)
    Bf = rng.uniform(-1, 1, (96, 400)).astype(np.float32)       # full B: R x n_total
    s0, c0 = ctx.shard_cols(400, rank, world)
    got = ctx.to_numpy(ctx.dottmpi(ctx.colmajor(A), ctx.colmajor(np.ascontiguousarray(Bf[:, s0:s0 + c0]))))
    ref = oracle.gemm_f64(A, Bf, transB=True)
    assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-5
    At = rng.uniform(-1, 1, (128, 200)).astype(np.float32)      # stored K x M
    Bn = rng.uniform(-1, 1, (128, 300)).astype(np.float32)
    s0, c0 = ctx.shard_cols(300, rank, world)
    osh = ctx.empty(200, c0)
    ctx.dot_sharded_out(ctx.colmajor(At), ctx.colmajor(Bn), osh, transA=True)
    ref = oracle.gemm_f64(At, Bn, transA=True)[:, s0:s0 + c0]
    assert np.abs(ctx.to_numpy(osh) - ref).max() / np.abs(ref).max() < 1e-5
    ctx.gemm_check()
    # two chained layers with the 8-bit exchange decoded inside the second GEMM's pre-pass == the same chain with the
    # codes decoded to fp32 first (exchange = 1); the coded form never writes the peers' fp32 blocks
    M, K, N1c, N2c = 128, 640, 1024 + 8 * world, 512
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    Wa = rng.uniform(-1, 1, (K, N1c)).astype(np.float32)
    Wb = rng.uniform(-1, 1, (N1c, N2c)).astype(np.float32)
    dA = ctx.colmajor(A)
    s1, c1 = ctx.shard_cols(N1c, rank, world)
    s2, c2 = ctx.shard_cols(N2c, rank, world)
    dWa, dWb = ctx.colmajor(np.ascontiguousarray(Wa[:, s1:s1 + c1])), ctx.colmajor(np.ascontiguousarray(Wb[:, s2:s2 + c2]))
    h1 = ctx.dotmpi(dA, dWa, N1c, activation=_lib.ACT_RELU, exchange=1)
    ref2 = ctx.dotmpi(h1, dWb, N2c)
    coded, keep = ctx.dotmpi_to_coded(dA, dWa, N1c, activation=_lib.ACT_RELU, rank=rank, nranks=world)
    got2 = ctx.dotmpi_from_coded(coded, dWb, N2c)
    ctx.gemm_check()
    assert torch.equal(got2, ref2), float((got2 - ref2).abs().max())
    # 8-bit gradient exchange: own gradient + decode(encode(peer gradient)) in rank order, fixed and gathered scales
    n = 70001
    grads = [np.random.default_rng(100 + r).standard_normal(n).astype(np.float32) * np.float32(0.01 * (r + 1)) for r in range(world)]
    for fixed in (1.0, 0.0):
        g = torch.from_numpy(grads[rank].copy()).cuda()
        cn.check(ctx.lib.cn_grad_sync_8bit(ctx.h, g.data_ptr(), n, fixed, ctx.stream_ptr()))
        want = grads[rank].copy()
        for r in range(world):
            if r == rank:
                continue
            p = fixed if fixed > 0 else oracle.absmax(grads[r])
            want = (want + oracle.decompress(ctx.codebook, oracle.compress(ctx.codebook, grads[r], p), p)).astype(np.float32)
        torch.cuda.synchronize()
        assert np.array_equal(g.cpu().numpy(), want), fixed
    # the packed exchange (several tensors, one gather, one decode-and-sum pass) == one exchange per tensor
    segs = [30001, 0, 40000]
    gp = torch.from_numpy(grads[rank].copy()).cuda()
    cn.check(ctx.lib.cn_grad_sync_8bit_multi(ctx.h, gp.data_ptr(), (ctypes.c_int64 * 3)(*segs), 3, 0.0, ctx.stream_ptr()))
    gs = torch.from_numpy(grads[rank].copy()).cuda()
    o = 0
    for sz in segs:
        cn.check(ctx.lib.cn_grad_sync_8bit(ctx.h, gs[o:].data_ptr(), sz, 0.0, ctx.stream_ptr()))
        o += sz
    torch.cuda.synchronize()
    assert torch.equal(gp, gs)
    # ... and the blocks pushed into the peers' memory == the blocks gathered by NCCL, call after call with changing sizes
    # (the area grows, the flags' epochs advance on the device), also when the launches are replayed from a CUDA graph
    for segs2 in ([30001, 0, 40000], [7], [70001], [1000, 2000]):
        tot = sum(segs2)
        res = []
        for on in (1, 0):
            cn.check(ctx.lib.cn_comm_set_push_exchange(ctx.h, on))
            g2 = torch.from_numpy(grads[rank][:tot].copy()).cuda()
            n0 = ctx.lib.cn_kernel_launches()
            cn.check(ctx.lib.cn_grad_sync_8bit_multi(ctx.h, g2.data_ptr(), (ctypes.c_int64 * len(segs2))(*segs2), len(segs2), 0.0, ctx.stream_ptr()))
            torch.cuda.synchronize()
            res.append((g2, ctx.lib.cn_kernel_launches() - n0))
        assert torch.equal(res[0][0], res[1][0]), segs2
        # several tensors: the push is one more kernel of this library (the gather is none); one tensor: coded and pushed in ONE launch
        assert res[0][1] == res[1][1] + (0 if len(segs2) == 1 else 1), segs2
    cn.check(ctx.lib.cn_comm_set_push_exchange(ctx.h, 1))
    ctx.gemm_check()
    # the exchange with the RMSprop step inside its summing pass == the exchange, then cn_rmsprop_update (bit for bit),
    # with segment ends that are no multiples of four and with buffers that are not 16-byte aligned
    for segs3, shift in (([30001, 0, 40000], 0), ([70001], 0), ([1001, 2003], 1)):
        tot = sum(segs3)
        arr = (ctypes.c_int64 * len(segs3))(*segs3)
        rms0 = np.abs(np.random.default_rng(5).standard_normal(tot + 1)).astype(np.float32)
        w0 = np.random.default_rng(6).standard_normal(tot + 1).astype(np.float32)
        outs = []
        for fused in (True, False):
            g3 = torch.from_numpy(grads[rank][:tot + 1].copy()).cuda()[shift:shift + tot]
            r3 = torch.from_numpy(rms0.copy()).cuda()[shift:shift + tot]
            w3 = torch.from_numpy(w0.copy()).cuda()[shift:shift + tot]
            if fused:
                cn.check(ctx.lib.cn_grad_sync_8bit_rmsprop(ctx.h, g3.data_ptr(), arr, len(segs3), 0.0, r3.data_ptr(), w3.data_ptr(), 0.9, 0.006,
                                                           ctx.stream_ptr()))
            else:
                cn.check(ctx.lib.cn_grad_sync_8bit_multi(ctx.h, g3.data_ptr(), arr, len(segs3), 0.0, ctx.stream_ptr()))
                cn.check(ctx.lib.cn_rmsprop_update(ctx.h, r3.data_ptr(), g3.data_ptr(), w3.data_ptr(), 0.9, 0.006, tot, ctx.stream_ptr()))
            torch.cuda.synchronize()
            outs.append((g3.clone(), r3.clone(), w3.clone()))
        for a, b in zip(outs[0], outs[1]):
            assert torch.equal(a, b), (segs3, shift)
    # one tensor with its own absmax goes through ONE launch that codes and pushes; recorded in a CUDA graph and replayed
    # on data that change from replay to replay (the exchange's epochs and the kernel's grid barrier live on the device)
    nrep = 300007
    src = torch.from_numpy(np.random.default_rng(200 + rank).standard_normal(nrep).astype(np.float32)).cuda()
    gg = src.clone()
    seg1 = (ctypes.c_int64 * 1)(nrep)
    n0 = ctx.lib.cn_kernel_launches()
    cn.check(ctx.lib.cn_grad_sync_8bit_multi(ctx.h, gg.data_ptr(), seg1, 1, 0.0, ctx.stream_ptr()))
    assert ctx.lib.cn_kernel_launches() - n0 == 2          # code + push, decode + sum
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        cn.check(ctx.lib.cn_grad_sync_8bit_multi(ctx.h, gg.data_ptr(), seg1, 1, 0.0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    for rep, f in enumerate((1.0, 0.25, 3.0, 0.01)):
        want_g = src * f
        cn.check(ctx.lib.cn_comm_set_push_exchange(ctx.h, 0))
        cn.check(ctx.lib.cn_grad_sync_8bit_multi(ctx.h, want_g.data_ptr(), seg1, 1, 0.0, ctx.stream_ptr()))      # NCCL gather, call by call
        cn.check(ctx.lib.cn_comm_set_push_exchange(ctx.h, 1))
        gg.copy_(src * f)
        torch.cuda.synchronize()
        dist.barrier()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(gg, want_g), rep
    ctx.gemm_check()
    # TdotMPI with a sharded B: the row-major batch as a transposed operand, through the fused gather
    M, K, N = 128, 2048, 2048 + 8 * world
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    W = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    s0, c0 = ctx.shard_cols(N, rank, world)
    dW = ctx.colmajor(np.ascontiguousarray(W[:, s0:s0 + c0]))
    want = ctx.dotmpi(ctx.colmajor(A), dW, N)
    rm = torch.from_numpy(A).cuda()
    got = ctx.sym_empty(M, N)
    epi = cn.Epilogue(None, 0, 0, None)
    cn.check(ctx.lib.cn_tdotmpi_f32(ctx.h, M, K, N, rm.data_ptr(), K, dW.data_ptr(), got.data_ptr(), ctypes.byref(epi), _lib.GEMM_3XTF32, 0,
                                    ctx.stream_ptr()))
    ctx.gemm_check()
    assert torch.equal(got, want)
    # ... and the same product from planes made ahead of it (cn_gemm_prepare), through the fused gather: bit-identical
    hp = ctypes.c_void_p()
    cn.check(ctx.lib.cn_gemm_prepare_create(ctx.h, M, K, _lib.GEMM_3XTF32, ctypes.byref(hp)))
    cn.check(ctx.lib.cn_gemm_prepare(ctx.h, hp, 1, rm.data_ptr(), K, ctx.stream_ptr()))
    got_p = ctx.sym_empty(M, N)
    cn.check(ctx.lib.cn_dotmpi_prepared_f32(ctx.h, hp, N, dW.data_ptr(), got_p.data_ptr(), ctypes.byref(epi), 0, ctx.stream_ptr()))
    ctx.gemm_check()
    torch.cuda.synchronize()
    assert torch.equal(got_p, want)
    dist.barrier()
    ctx.lib.cn_gemm_prepare_destroy(hp)
    # batch allocator with the sharded upload: every rank holds the data set and uploads 1/G of each batch's rows; the
    # blocks are exchanged over NVLink; every rank then sees every batch whole (tests/batchAllocator_test.cu:40-114 form)
    rows, cols_x, B = 1000, 36, 128
    X = np.arange(rows * cols_x, dtype=np.float32).reshape(rows, cols_x)
    y = np.arange(rows, dtype=np.float32).reshape(rows, 1) + 0.5
    hX, hy = torch.from_numpy(X).pin_memory(), torch.from_numpy(y).pin_memory()
    for flags in (_lib.BATCH_SHARDED_UPLOAD, _lib.BATCH_SHARDED_UPLOAD | _lib.BATCH_NO_COL_MAJOR,
                  _lib.BATCH_SHARDED_UPLOAD | _lib.BATCH_NO_COL_MAJOR | _lib.BATCH_PUSH_BY_KERNEL,
                  _lib.BATCH_SHARDED_UPLOAD | _lib.BATCH_NO_COL_MAJOR | _lib.BATCH_LOOKAHEAD):
        bh = ctypes.c_void_p()
        cn.check(ctx.lib.cn_batch_create_ex(ctx.h, hX.data_ptr(), hy.data_ptr(), rows, cols_x, 1, B, 0, flags, ctypes.byref(bh)))
        ora = oracle.BatchOracle(rows, B, False)
        px, py, n, prm = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int64(), ctypes.c_void_p()
        cn.check(ctx.lib.cn_batch_current(bh, ctypes.byref(px), ctypes.byref(py), ctypes.byref(n)))
        start, cnt = ora.current
        rt = ctypes.CDLL("libcudart.so.12")
        for step in range(2 * ora.total + 2):
            cn.check(ctx.lib.cn_batch_copy_next_async(bh))
            cn.check(ctx.lib.cn_batch_current_row_major(bh, ctypes.byref(prm), ctypes.byref(n)))
            torch.cuda.synchronize()
            assert n.value == cnt
            buf = torch.empty((cnt, cols_x), device="cuda")
            assert rt.cudaMemcpy(ctypes.c_void_p(buf.data_ptr()), prm, ctypes.c_size_t(cnt * cols_x * 4), 3) == 0
            assert np.array_equal(buf.cpu().numpy(), X[start:start + cnt]), (flags, step)
            if not (flags & _lib.BATCH_NO_COL_MAJOR):
                cm = torch.empty((cols_x, cnt), device="cuda")
                assert rt.cudaMemcpy(ctypes.c_void_p(cm.data_ptr()), px, ctypes.c_size_t(cnt * cols_x * 4), 3) == 0
                assert np.array_equal(cm.cpu().numpy().T, X[start:start + cnt])
            cn.check(ctx.lib.cn_batch_swap(bh, ctx.stream_ptr(), ctypes.byref(px), ctypes.byref(py), ctypes.byref(n)))
            start, cnt = ora.advance()
        ctx.gemm_check()
        torch.cuda.synchronize()
        dist.barrier()
        ctx.lib.cn_batch_destroy(bh)
        dist.barrier()
    # scalar gather and all-reduce
    v = torch.zeros(world, device="cuda")
    v[rank] = rank + 1.5
    cn.check(ctx.lib.cn_allgather_scalar_f32(ctx.h, v.data_ptr(), ctx.stream_ptr()))
    t = torch.full((1000,), float(rank + 1), device="cuda")
    cn.check(ctx.lib.cn_allreduce_sum_f32(ctx.h, t.data_ptr(), t.numel(), ctx.stream_ptr()))
    torch.cuda.synchronize()
    assert v.tolist() == [r + 1.5 for r in range(world)]
    assert float(t[0]) == world * (world + 1) / 2
    dist.barrier()
    ctx.sym_free_all()

    # ---- bounded host wait and recovery.  No rank fails here: the stream is kept busy by a plain delay kernel, the
    # short limit runs out on every rank, cn_comm_sync aborts the (idle, healthy) communicator, later collectives are
    # refused, and a new communicator is made on the same context.
    assert ctx.lib.cn_comm_sync(ctx.h, ctx.stream_ptr(), 2000) == 0
    torch.cuda._sleep(int(0.4 * 1.9e9))                      # ~0.2-0.4 s of device time, then the stream drains by itself
    assert ctx.lib.cn_comm_sync(ctx.h, ctx.stream_ptr(), 20) == _lib.CN_ERR_TIMEOUT
    assert b"communicator aborted" in ctx.lib.cn_last_error()
    torch.cuda.synchronize()
    assert ctx.lib.cn_allreduce_sum_f32(ctx.h, t.data_ptr(), t.numel(), ctx.stream_ptr()) == _lib.CN_ERR_NCCL
    assert b"cn_comm_destroy" in ctx.lib.cn_last_error()
    dist.barrier()
    cn.check(ctx.lib.cn_comm_destroy(ctx.h))
    ids = [ctx.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    ctx.comm_init(ids[0], rank, world)
    t.fill_(float(rank + 1))
    cn.check(ctx.lib.cn_allreduce_sum_f32(ctx.h, t.data_ptr(), t.numel(), ctx.stream_ptr()))
    cn.check(ctx.lib.cn_comm_sync(ctx.h, ctx.stream_ptr(), 10000))
    assert float(t[0]) == world * (world + 1) / 2
    dist.barrier()
    cn.check(ctx.lib.cn_comm_destroy(ctx.h))
    if rank == 0:
        print("NCCL-OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    run_gloo() if sys.argv[1] == "gloo" else run_nccl()
