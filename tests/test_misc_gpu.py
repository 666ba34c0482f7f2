"""Layout boundary, random numbers / weight creation, batch allocator, timers — on the GPU through the C ABI."""
import ctypes

import numpy as np
import pytest
import torch

import clusternet_b200 as cn
from clusternet_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 1), (2, 3), (31, 33), (128, 784), (1000, 17), (5, 4099)])
def test_layout_round_trip(ctx, rows, cols):
    """tests/basicOps_test.cu:20-57: to_gpu (row-major -> col-major) and to_host are inverse; device order is col-major."""
    a = np.arange(rows * cols, dtype=np.float32).reshape(rows, cols)
    d = ctx.colmajor(a)
    assert np.array_equal(d.cpu().numpy().ravel(), a.T.ravel())      # memory = column-major
    assert np.array_equal(ctx.to_numpy(d), a)


def test_fill(ctx):
    t = torch.empty(100003, device="cuda")
    cn.check(ctx.lib.cn_fill_f32(ctx.h, t.data_ptr(), t.numel(), 1.7, ctx.stream_ptr()))
    assert float(t.min()) == float(t.max()) == np.float32(1.7)


def test_rand_is_deterministic_and_in_range(ctx):
    """tests/clusterNet_test.cu:177-255: same seed -> same numbers, values in (0,1], mean 0.5, different seeds differ."""
    a = ctx.rand(100, 1000, seed=42)
    b = ctx.rand(100, 1000, seed=42)
    c = ctx.rand(100, 1000, seed=43)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert float(a.min()) > 0.0 and float(a.max()) <= 1.0
    assert abs(float(a.mean()) - 0.5) < 0.01
    # a stream does not depend on how it is cut: the second half equals a separate launch with an offset
    whole = ctx.rand(1, 4096, seed=7)
    part = ctx.rand(1, 2048, seed=7, offset=512)      # offset counts groups of four values
    assert torch.equal(whole.flatten()[2048:], part.flatten())
    n = ctx.randn(200, 1000, seed=1, mean=1.0, std=2.0)
    assert abs(float(n.mean()) - 1.0) < 0.02 and abs(float(n.std()) - 2.0) < 0.02


def test_rand_int_range(ctx):
    t = torch.empty(200000, device="cuda")
    cn.check(ctx.lib.cn_rand_int(ctx.h, t.data_ptr(), t.numel(), 3, 9, 5, 0, ctx.stream_ptr()))
    assert float(t.min()) == 3.0 and float(t.max()) == 9.0 and bool((t == t.round()).all())
    counts = torch.bincount(t.long())[3:]
    assert float(counts.float().std() / counts.float().mean()) < 0.02


@pytest.mark.parametrize("rows,cols,total", [(784, 1200, 1200), (100, 40, 320), (5, 5, 5)])
def test_uniform_sqrt_weight_range(ctx, rows, cols, total):
    """tests/clusterNet_test.cu:279-314,499-577: weights lie within +-4*sqrt(6/(in+out)) and fill that range."""
    w = ctx.uniform_sqrt_weight(rows, cols, seed=3, fan_out_total=total)
    lim = float(oracle.sqrt_weight_limit(rows, total))
    assert float(w.max()) <= lim and float(w.min()) >= -lim
    if rows * cols > 10000:
        assert float(w.max()) > 0.99 * lim and float(w.min()) < -0.99 * lim and abs(float(w.mean())) < 0.02 * lim


def test_dropout_rate_and_values(ctx):
    """tests/clusterNet_test.cu:467-495: about `rate` of the entries become zero, the rest are unchanged (no rescale)."""
    a = ctx.rand(500, 1000, seed=9) + 1.0
    for rate in (0.2, 0.5, 0.8):
        d = ctx.dropout(a, rate, seed=11)
        zero = (d == 0)
        assert abs(float(zero.float().mean()) - rate) < 0.01
        assert torch.equal(d[~zero], a[~zero])


def _copy_from_device_pointer(ptr, count):
    """Device-to-device copy out of a raw pointer owned by the library (cudaMemcpyDeviceToDevice = 3)."""
    out = torch.empty(count, dtype=torch.float32, device="cuda")
    rt = ctypes.CDLL("libcudart.so.12")
    assert rt.cudaMemcpy(ctypes.c_void_p(out.data_ptr()), ptr, ctypes.c_size_t(count * 4), 3) == 0
    return out


def _batch_epochs(ctx, rows, cols_x, cols_y, B, skip_last=False, epochs=2, flags=0, pinned=False):
    X = np.arange(rows * cols_x, dtype=np.float32).reshape(rows, cols_x)
    y = np.arange(rows * cols_y, dtype=np.float32).reshape(rows, cols_y) + 0.5
    hX, hy = torch.from_numpy(X), torch.from_numpy(y)
    if pinned:
        hX, hy = hX.pin_memory(), hy.pin_memory()
    h = ctypes.c_void_p()
    if flags:
        cn.check(ctx.lib.cn_batch_create_ex(ctx.h, hX.data_ptr(), hy.data_ptr(), rows, cols_x, cols_y, B, int(skip_last), flags, ctypes.byref(h)))
    else:
        cn.check(ctx.lib.cn_batch_create(ctx.h, hX.data_ptr(), hy.data_ptr(), rows, cols_x, cols_y, B, int(skip_last), ctypes.byref(h)))
    keep_rm = bool(flags & (_lib.BATCH_KEEP_ROW_MAJOR | _lib.BATCH_NO_COL_MAJOR | _lib.BATCH_LOOKAHEAD))
    prm, nrm = ctypes.c_void_p(), ctypes.c_int64()
    prev_rm = None
    ora = oracle.BatchOracle(rows, B, skip_last)
    assert ctx.lib.cn_batch_total_batches(h) == ora.total
    px, py, n = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int64()
    cn.check(ctx.lib.cn_batch_current(h, ctypes.byref(px), ctypes.byref(py), ctypes.byref(n)))
    start, cnt = ora.current
    total = 0.0
    for step in range(epochs * ora.total + 3):
        assert n.value == cnt
        # current batch on the device is column-major n x cols
        torch.cuda.synchronize()
        if flags & _lib.BATCH_NO_COL_MAJOR:
            assert not px.value
        else:
            bx = _copy_from_device_pointer(px, cols_x * n.value).reshape(cols_x, n.value)
            assert np.array_equal(bx.cpu().numpy().T, X[start:start + cnt])
            total += float(bx.double().sum())
        by = _copy_from_device_pointer(py, cols_y * n.value).reshape(cols_y, n.value)
        assert np.array_equal(by.cpu().numpy().T, y[start:start + cnt])
        cn.check(ctx.lib.cn_batch_copy_next_async(h))
        if keep_rm:
            # the row-major copy of the CURRENT batch must survive the copy of the next one that was just queued
            cn.check(ctx.lib.cn_batch_current_row_major(h, ctypes.byref(prm), ctypes.byref(nrm)))
            torch.cuda.synchronize()
            assert nrm.value == cnt and prm.value != prev_rm
            rm = _copy_from_device_pointer(prm, cols_x * cnt).reshape(cnt, cols_x)
            assert np.array_equal(rm.cpu().numpy(), X[start:start + cnt])
            prev_rm = prm.value
        cn.check(ctx.lib.cn_batch_swap(h, ctx.stream_ptr(), ctypes.byref(px), ctypes.byref(py), ctypes.byref(n)))
        start, cnt = ora.advance()
    ctx.lib.cn_batch_destroy(h)


def test_batch_allocator_epochs_with_partial_last_batch(ctx):
    """tests/batchAllocator_test.cu:40-114: arange data, every element of every batch equals a running counter, the last
    batch of an epoch is short, the counter wraps around."""
    _batch_epochs(ctx, rows=1000, cols_x=17, cols_y=1, B=128)


def test_batch_allocator_exact_multiple_and_skip_last(ctx):
    _batch_epochs(ctx, rows=512, cols_x=8, cols_y=2, B=128)
    _batch_epochs(ctx, rows=1000, cols_x=5, cols_y=1, B=128, skip_last=True)


@pytest.mark.parametrize("flags", [_lib.BATCH_KEEP_ROW_MAJOR, _lib.BATCH_NO_COL_MAJOR, _lib.BATCH_SHARDED_UPLOAD, _lib.BATCH_LOOKAHEAD,
                                   _lib.BATCH_LOOKAHEAD | _lib.BATCH_NO_COL_MAJOR])
@pytest.mark.parametrize("pinned", [False, True])
def test_batch_allocator_options(ctx, flags, pinned):
    """cn_batch_create_ex: the row-major copy of the current batch stays valid (two buffers alternate), X is not
    transposed when that is switched off, the sharded upload is the plain one on a single rank, and with two copies in
    flight (three buffers) the batches still come in the reference's order - also when the short last batch is skipped
    and when the data set holds no more batches than the ring has buffers."""
    _batch_epochs(ctx, rows=1000, cols_x=20, cols_y=1, B=128, flags=flags, pinned=pinned)
    if flags & _lib.BATCH_LOOKAHEAD:
        _batch_epochs(ctx, rows=1000, cols_x=6, cols_y=1, B=128, skip_last=True, flags=flags, pinned=pinned)
        _batch_epochs(ctx, rows=200, cols_x=6, cols_y=1, B=128, flags=flags, pinned=pinned, epochs=4)      # 2 batches
        _batch_epochs(ctx, rows=300, cols_x=6, cols_y=2, B=128, flags=flags, pinned=pinned, epochs=4)      # 3 batches
    h = ctypes.c_void_p()
    x = torch.zeros(256, 4)
    assert ctx.lib.cn_batch_create_ex(ctx.h, x.data_ptr(), x.data_ptr(), 256, 4, 4, 128, 0, 64, ctypes.byref(h)) == _lib.CN_ERR_ARG


@pytest.mark.parametrize("flags", [0, _lib.BATCH_LOOKAHEAD])
def test_skip_last_switched_while_copies_are_in_flight(ctx, flags):
    """SKIP_LAST_BATCH is a public member the reference's users flip between epochs (source/batchAllocator.h); a copy that
    was started under the old setting and no longer lies on the sequence is dropped, not delivered."""
    rows, cols, B = 1000, 4, 128                       # 8 batches, the last one short
    X = np.arange(rows * cols, dtype=np.float32).reshape(rows, cols)
    y = np.arange(rows, dtype=np.float32).reshape(rows, 1)
    hX, hy = torch.from_numpy(X).pin_memory(), torch.from_numpy(y).pin_memory()
    h = ctypes.c_void_p()
    cn.check(ctx.lib.cn_batch_create_ex(ctx.h, hX.data_ptr(), hy.data_ptr(), rows, cols, 1, B, 0, flags | _lib.BATCH_KEEP_ROW_MAJOR, ctypes.byref(h)))
    px, py, n, prm = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int64(), ctypes.c_void_p()
    seen = []
    for step in range(14):
        cn.check(ctx.lib.cn_batch_copy_next_async(h))
        if step == 5:      # current batch is number 5; with two copies in flight, 6 and 7 are under way and 7 must go
            cn.check(ctx.lib.cn_batch_set_skip_last(h, 1))
        cn.check(ctx.lib.cn_batch_swap(h, ctx.stream_ptr(), ctypes.byref(px), ctypes.byref(py), ctypes.byref(n)))
        cn.check(ctx.lib.cn_batch_current_row_major(h, ctypes.byref(prm), ctypes.byref(n)))
        torch.cuda.synchronize()
        first = float(_copy_from_device_pointer(prm, cols)[0].item())
        lab = float(_copy_from_device_pointer(py, 1)[0].item())
        assert first == lab * cols                     # X and the labels belong to the same batch
        seen.append(int(lab) // B)
    assert seen == [1, 2, 3, 4, 5, 6, 0, 1, 2, 3, 4, 5, 6, 0]
    ctx.lib.cn_batch_destroy(h)


def test_row_major_batch_feeds_the_product_as_a_transposed_operand(ctx):
    """The batch as the host holds it (row-major M x K) is the transposed operand of TdotMPI (source/clusterNet.cpp:510):
    the product equals the one computed from the column-major copy, bit for bit, also for K that is not a multiple of 4
    and for a leading dimension above K."""
    rng = np.random.default_rng(9)
    for (M, K, N, pad) in [(128, 4096, 512, 0), (128, 1000, 384, 0), (100, 1002, 256, 0), (64, 512, 256, 8), (7, 33, 64, 1)]:
        A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        W = rng.uniform(-1, 1, (K, N)).astype(np.float32)
        dW = ctx.colmajor(W)
        want = ctx.gemm(ctx.colmajor(A), dW)
        lda = K + pad
        rm = torch.zeros((M, lda), device="cuda")
        rm[:, :K] = torch.from_numpy(A).cuda()
        got = ctx.empty(M, N)
        epi = cn.Epilogue(None, 0, 0, None)
        cn.check(ctx.lib.cn_tdotmpi_f32(ctx.h, M, K, N, rm.data_ptr(), lda, dW.data_ptr(), got.data_ptr(), ctypes.byref(epi),
                                        _lib.GEMM_3XTF32, 0, ctx.stream_ptr()))
        ctx.gemm_check()
        assert torch.equal(got, want), (M, K, N, pad)
        ref = oracle.gemm_f64(A, W)
        assert np.abs(ctx.to_numpy(got) - ref).max() / np.abs(ref).max() < 1e-5


def test_packed_gradient_exchange_is_a_no_op_on_one_rank(ctx):
    g = torch.randn(1000, device="cuda")
    keep = g.clone()
    seg = (ctypes.c_int64 * 3)(300, 0, 700)
    cn.check(ctx.lib.cn_grad_sync_8bit_multi(ctx.h, g.data_ptr(), seg, 3, 0.0, ctx.stream_ptr()))
    assert torch.equal(g, keep)
    seg = (ctypes.c_int64 * 1)(-1)
    assert ctx.lib.cn_grad_sync_8bit_multi(ctx.h, g.data_ptr(), seg, 1, 0.0, ctx.stream_ptr()) == _lib.CN_ERR_ARG


def test_batch_size_larger_than_data_is_rejected(ctx):
    x = torch.zeros(10, 4)
    h = ctypes.c_void_p()
    st = ctx.lib.cn_batch_create(ctx.h, x.data_ptr(), x.data_ptr(), 10, 4, 4, 128, 0, ctypes.byref(h))
    assert st == _lib.CN_ERR_SHAPE and b"Batch size must be smaller" in ctx.lib.cn_last_error()


def test_tick_tock_accumulates(ctx):
    ctx.tick("t")
    a = ctx.rand(1000, 1000, seed=1)
    first = ctx.tock("t")
    ctx.tick("t")
    a = ctx.rand(1000, 1000, seed=2)
    second = ctx.tock("t")
    assert first > 0 and second > first
    with pytest.raises(cn.CnError):
        ctx.tock("never-ticked")


def test_kernel_launch_counter_moves(ctx):
    n0 = ctx.lib.cn_kernel_launches()
    ctx.rand(10, 10, seed=1)
    assert ctx.lib.cn_kernel_launches() == n0 + 1


def test_single_rank_dotmpi_equals_dot(ctx):
    """tests/clusterNet_test.cu:257-276 at one rank: dotMPI == dot on 0.3*ones(200x400) . 1.1748345*ones(400x800)."""
    A = ctx.colmajor(np.full((200, 400), 0.3, np.float32))
    W = ctx.colmajor(np.full((400, 800), 1.1748345, np.float32))
    C1 = ctx.gemm(A, W)
    C2 = ctx.dotmpi(A, W, 800)
    ctx.gemm_check()
    assert torch.equal(C1, C2)
    want = np.float64(np.float32(0.3)) * np.float64(np.float32(1.1748345)) * 400
    assert np.abs(ctx.to_numpy(C2) - want).max() / want < 1e-5


def test_coded_chain_on_one_rank_is_exact(ctx):
    """With one rank the whole matrix is the rank's own block, kept in fp32: the coded chain equals the plain chain."""
    rng = np.random.default_rng(11)
    A = ctx.colmajor(rng.uniform(-1, 1, (128, 320)).astype(np.float32))
    W1 = ctx.colmajor(rng.uniform(-1, 1, (320, 512)).astype(np.float32))
    W2 = ctx.colmajor(rng.uniform(-1, 1, (512, 256)).astype(np.float32))
    ref = ctx.gemm(ctx.gemm(A, W1, activation=_lib.ACT_RELU), W2)
    coded, keep = ctx.dotmpi_to_coded(A, W1, 512, activation=_lib.ACT_RELU)
    got = ctx.dotmpi_from_coded(coded, W2, 256)
    ctx.gemm_check()
    assert torch.equal(got, ref)
    # the codes are the compressor's output for the fp32 block with its absmax as the scale
    codes, scales, own = keep
    p = float(scales[0].item())
    assert p == float(own.abs().max().item())
    assert np.array_equal(codes.cpu().numpy().ravel(), oracle.compress(ctx.codebook, own.cpu().numpy().ravel(), p))


def test_bounded_wait_surfaces_as_timeout_status(ctx):
    """A device-side wait for a signal that never arrives (a peer that died between steps) ends by itself after its
    cycle limit and is reported by the next status check; the context stays usable."""
    ctx.gemm_check()                                                    # clean before
    cn.check(ctx.lib.cn_diag_wait_probe(ctx.h, 2_000_000, ctx.stream_ptr()))      # ~1 ms
    with pytest.raises(cn.CnError) as e:
        ctx.gemm_check()
    assert e.value.status == _lib.CN_ERR_TIMEOUT
    ctx.gemm_check()                                                    # the status word was cleared
    a = ctx.rand(4, 4, seed=1)                                          # and the GPU still works
    assert float(a.sum()) > 0


def test_comm_sync_is_a_bounded_wait_without_a_communicator(ctx):
    """cn_comm_sync: done at once on an idle stream; CN_ERR_TIMEOUT while a (finite) delay kernel runs; fine again after."""
    sp = ctx.stream_ptr()
    assert ctx.lib.cn_comm_sync(ctx.h, sp, 1000) == 0
    torch.cuda._sleep(int(0.3 * 1.9e9))
    assert ctx.lib.cn_comm_sync(ctx.h, sp, 10) == _lib.CN_ERR_TIMEOUT
    assert b"still busy" in ctx.lib.cn_last_error() and b"aborted" not in ctx.lib.cn_last_error()
    assert ctx.lib.cn_comm_sync(ctx.h, sp, 20000) == 0
    assert ctx.lib.cn_comm_sync(ctx.h, sp, 0) == _lib.CN_ERR_ARG
    x = torch.ones(1024, device="cuda")
    assert float(ctx.absmax(x).item()) == 1.0          # the context is still usable
