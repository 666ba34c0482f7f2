"""Data-parallel training step: each elementwise kernel against its numpy restatement, the 8-bit gradient sync at one
rank, and the facade's Layer chain (forward / backward on the config-4 MLP shape) against an fp64 restatement."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

import clusternet_b200 as cn
from clusternet_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_softmax_and_t_matrix(ctx):
    rng = np.random.default_rng(0)
    for rows, cols in [(128, 10), (1, 3), (1000, 37)]:
        A = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
        d = ctx.colmajor(A)
        out = ctx.empty(rows, cols)
        cn.check(ctx.lib.cn_softmax(ctx.h, d.data_ptr(), out.data_ptr(), rows, cols, ctx.stream_ptr()))
        got = ctx.to_numpy(out)
        assert np.abs(got - oracle.softmax_rows(A)).max() < 2e-6      # __expf vs libm exp
        assert np.abs(got.sum(1) - 1).max() < 1e-5
        labels = rng.integers(0, cols, rows).astype(np.float32)
        t = ctx.empty(rows, cols)
        t.fill_(7.0)
        cn.check(ctx.lib.cn_create_t_matrix(ctx.h, torch.from_numpy(labels).cuda().data_ptr(), t.data_ptr(), rows, cols, ctx.stream_ptr()))
        assert np.array_equal(ctx.to_numpy(t), oracle.t_matrix(labels, cols))
        # the fused output layer (softmax + one-hot + sub in one pass) gives the same bits as the three calls
        want_err = ctx.empty(rows, cols)
        cn.check(ctx.lib.cn_sub(ctx.h, out.data_ptr(), t.data_ptr(), want_err.data_ptr(), rows * cols, ctx.stream_ptr()))
        prob, err = ctx.empty(rows, cols), ctx.empty(rows, cols)
        cn.check(ctx.lib.cn_softmax_error(ctx.h, d.data_ptr(), torch.from_numpy(labels).cuda().data_ptr(), prob.data_ptr(), err.data_ptr(),
                                          rows, cols, ctx.stream_ptr()))
        assert torch.equal(prob, out) and torch.equal(err, want_err)


def test_elementwise_and_activation_gradients(ctx):
    rng = np.random.default_rng(1)
    a = rng.standard_normal(100003).astype(np.float32)
    b = rng.standard_normal(100003).astype(np.float32)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    out = torch.empty_like(da)
    sp = ctx.stream_ptr()
    for fn, want in [(ctx.lib.cn_add, a + b), (ctx.lib.cn_sub, a - b), (ctx.lib.cn_mul, a * b)]:
        cn.check(fn(ctx.h, da.data_ptr(), db.data_ptr(), out.data_ptr(), a.size, sp))
        assert np.array_equal(out.cpu().numpy(), want)
    cn.check(ctx.lib.cn_scalar_mul(ctx.h, da.data_ptr(), 0.5, out.data_ptr(), a.size, sp))
    assert np.array_equal(out.cpu().numpy(), a * np.float32(0.5))
    for act, want in [(_lib.ACT_RELU, (a > 0).astype(np.float32)), (_lib.ACT_LOGISTIC, a * (np.float32(1) - a)),
                      (_lib.ACT_DOUBLE_RELU, ((a > 0) & (a < 1)).astype(np.float32))]:
        cn.check(ctx.lib.cn_activation_gradient(ctx.h, da.data_ptr(), act, out.data_ptr(), a.size, sp))
        assert np.array_equal(out.cpu().numpy(), want)
        # error * f'(activation) in one pass == the two calls
        prod, g2, fused = torch.empty_like(da), torch.empty_like(da), torch.empty_like(da)
        cn.check(ctx.lib.cn_mul(ctx.h, db.data_ptr(), out.data_ptr(), prod.data_ptr(), a.size, sp))
        cn.check(ctx.lib.cn_mul_activation_gradient(ctx.h, db.data_ptr(), da.data_ptr(), act, g2.data_ptr(), fused.data_ptr(), a.size, sp))
        assert torch.equal(fused, prod) and torch.equal(g2, out)
        cn.check(ctx.lib.cn_mul_activation_gradient(ctx.h, db.data_ptr(), da.data_ptr(), act, None, fused.data_ptr(), a.size, sp))
        assert torch.equal(fused, prod)
    assert ctx.lib.cn_activation_gradient(ctx.h, da.data_ptr(), _lib.ACT_LINEAR, out.data_ptr(), a.size, sp) == _lib.CN_ERR_ARG
    assert ctx.lib.cn_mul_activation_gradient(ctx.h, db.data_ptr(), da.data_ptr(), _lib.ACT_LINEAR, None, out.data_ptr(), a.size, sp) == _lib.CN_ERR_ARG


def test_abs_div_square_scalar_add_and_seeded_max(ctx):
    rng = np.random.default_rng(7)
    a = rng.standard_normal(70001).astype(np.float32)
    b = (rng.standard_normal(70001).astype(np.float32) + np.float32(3.0))
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    out = torch.empty_like(da)
    sp = ctx.stream_ptr()
    cn.check(ctx.lib.cn_abs(ctx.h, da.data_ptr(), out.data_ptr(), a.size, sp))
    assert np.array_equal(out.cpu().numpy(), np.abs(a))
    cn.check(ctx.lib.cn_square(ctx.h, da.data_ptr(), out.data_ptr(), a.size, sp))
    sq = (a.astype(np.float64) ** 2)              # the reference squares with powf(x, 2.0f): within 2 ulp of the product
    assert np.all(np.abs(out.cpu().numpy() - sq) <= 2 * np.spacing((a * a).astype(np.float32)))
    cn.check(ctx.lib.cn_scalar_add(ctx.h, da.data_ptr(), 0.1748345, out.data_ptr(), a.size, sp))
    assert np.array_equal(out.cpu().numpy(), a + np.float32(0.1748345))
    cn.check(ctx.lib.cn_div(ctx.h, da.data_ptr(), db.data_ptr(), out.data_ptr(), a.size, sp))
    want = a / b                                  # the reference divides with fdividef: 2 ulp
    assert np.abs(out.cpu().numpy() - want).max() <= 3e-7 * np.abs(want).max() + 1e-30
    assert np.all(np.abs(out.cpu().numpy() - want) <= 4 * np.spacing(np.abs(want)))
    res = torch.full((1,), 99.0, device="cuda")
    for arr in (a, -np.abs(a) - np.float32(2.0), a[:1], a[:33], np.full(5000, -0.25, np.float32)):
        d = torch.from_numpy(np.ascontiguousarray(arr)).cuda()
        cn.check(ctx.lib.cn_max_f32(ctx.h, d.data_ptr(), arr.size, res.data_ptr(), sp))
        assert res.item() == oracle.max_seeded(arr)
    cn.check(ctx.lib.cn_max_f32(ctx.h, None, 0, res.data_ptr(), sp))
    assert res.item() == -1.0


def test_nesterov_update(ctx):
    rng = np.random.default_rng(8)
    n = 30011
    g, w, m = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    dg, dw, dm = (torch.from_numpy(x.copy()).cuda() for x in (g, w, m))
    cn.check(ctx.lib.cn_nesterov_update(ctx.h, dg.data_ptr(), dw.data_ptr(), dm.data_ptr(), 0.003, 128, 0.9, n, ctx.stream_ptr()))
    w_want, m_want = oracle.nesterov_update(g, w, m, 0.003, 128, 0.9)
    assert np.abs(dw.cpu().numpy() - w_want).max() <= 1e-6
    assert np.abs(dm.cpu().numpy() - m_want).max() <= 1e-6
    assert ctx.lib.cn_nesterov_update(ctx.h, dg.data_ptr(), dw.data_ptr(), dm.data_ptr(), 0.003, 0, 0.9, n, ctx.stream_ptr()) == _lib.CN_ERR_ARG


def test_rmsprop_update(ctx):
    rng = np.random.default_rng(2)
    n = 50001
    rms = np.abs(rng.standard_normal(n)).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    w = rng.standard_normal(n).astype(np.float32)
    drms, dg, dw = (torch.from_numpy(x.copy()).cuda() for x in (rms, g, w))
    cn.check(ctx.lib.cn_rmsprop_update(ctx.h, drms.data_ptr(), dg.data_ptr(), dw.data_ptr(), 0.9, 0.006, n, ctx.stream_ptr()))
    r_want, w_want = oracle.rmsprop_update(rms, g, w, 0.9, 0.006)
    assert np.abs(drms.cpu().numpy() - r_want).max() <= 1e-6 * np.abs(r_want).max()
    assert np.abs(dw.cpu().numpy() - w_want).max() <= 2e-6


def test_grad_sync_is_identity_on_one_rank(ctx):
    g = torch.randn(10000, device="cuda")
    ref = g.clone()
    cn.check(ctx.lib.cn_grad_sync_8bit(ctx.h, g.data_ptr(), g.numel(), 1.0, ctx.stream_ptr()))
    assert torch.equal(g, ref)
    # ... and the exchange with the update inside is the plain update there
    rms, w = torch.rand(10000, device="cuda"), torch.randn(10000, device="cuda")
    rms2, w2 = rms.clone(), w.clone()
    seg = (ctypes.c_int64 * 2)(4000, 6000)
    cn.check(ctx.lib.cn_grad_sync_8bit_rmsprop(ctx.h, g.data_ptr(), seg, 2, 0.0, rms.data_ptr(), w.data_ptr(), 0.9, 0.006, ctx.stream_ptr()))
    cn.check(ctx.lib.cn_rmsprop_update(ctx.h, rms2.data_ptr(), g.data_ptr(), w2.data_ptr(), 0.9, 0.006, 10000, ctx.stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(g, ref) and torch.equal(rms, rms2) and torch.equal(w, w2)
    assert ctx.lib.cn_grad_sync_8bit_rmsprop(ctx.h, g.data_ptr(), seg, 2, 0.0, None, w.data_ptr(), 0.9, 0.006, ctx.stream_ptr()) == _lib.CN_ERR_ARG


def test_layer_chain_gradients_and_training(built_lib, tmp_path):
    """Config-4 MLP shape 784-1200-1200-10, batch 128, through the C++ facade's Layer class: probabilities and the three
    weight gradients of one step against the fp64 restatement, then 40 RMSprop steps must cut the training error."""
    exe = str(tmp_path / "layer_test")
    libdir = os.path.join(ROOT, "clusternet_b200")
    subprocess.check_call(["/usr/local/cuda/bin/nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a",
                           os.path.join(ROOT, "tests", "layer_test.cu"), "-o", exe, f"-L{libdir}", "-lclusternet_b200",
                           "-Xlinker", f"-rpath={libdir}"])
    r = subprocess.run([exe, os.path.join(ROOT, "tests", "golden", "codebook_126.f32"), "784", "1200", "10", "128", "40", str(tmp_path)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "All tests passed" in r.stdout, r.stdout + r.stderr

    def load(name, rows, cols):
        return np.fromfile(tmp_path / name, dtype=np.float32).reshape(rows, cols)
    X, y = load("X.bin", 128, 784), load("y.bin", 128, 1)
    W = [load("w0.bin", 784, 1200), load("w1.bin", 1200, 1200), load("w2.bin", 1200, 10)]
    probs, grads = oracle.mlp_step_gradients(X, y, W)
    # the logits reach +-50 with the reference's 4x weight range, so their 1e-6 relative error shows up as 1e-5..1e-4 in
    # the saturated softmax and, through the error term, in the gradients
    assert np.abs(load("probs.bin", 128, 10) - probs).max() < 2e-4
    for name, g in zip(("g0.bin", "g1.bin", "g2.bin"), grads):
        got = load(name, *g.shape)
        assert np.abs(got - g).max() / np.abs(g).max() < 5e-4, name
