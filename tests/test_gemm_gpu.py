"""GEMM parity: the reference's known-answer tests, an fp64 host GEMM as accuracy yardstick, fused epilogues."""
import ctypes

import numpy as np
import pytest
import torch

import clusternet_b200 as cn
from clusternet_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu

TOL_3XTF32 = 1e-5      # max |C - C64| / max |C64|, the bound the 3xTF32 mode has to meet
TOL_TF32 = 2e-3        # looser bound of the single-pass TF32 mode (10-bit mantissa operands)


def normwise(got, ref):
    return float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-300))


def test_dot_known_answers(ctx):
    """The reference's own known-answer vectors (tests/clusterNet_test.cu:16-36,67-84,106-129,158-165), which it
    checks with float equality."""
    import json
    import os
    kat = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "gemm_kat.json")))
    mats = {k: np.array(kat[k]["data"], np.float32).reshape(kat[k]["rows"], kat[k]["cols"]) for k in ("m1", "m2")}
    for case in kat["cases"]:
        A, B = ctx.colmajor(mats[case["a"]]), ctx.colmajor(mats[case["b"]])
        C = ctx.to_numpy(ctx.gemm(A, B, transA=case["op"] == "Tdot", transB=case["op"] == "dotT"))
        assert ctx.gemm_last_path() == "simt_fp32"
        want = np.array(case["expect"], np.float32).reshape(case["rows"], case["cols"])
        assert C.shape == want.shape
        assert np.array_equal(C, want), (case["op"], C, want)


def test_shape_mismatch_is_an_error(ctx):
    from clusternet_b200 import CnError
    A = ctx.colmajor(np.ones((4, 5), np.float32))
    B = ctx.colmajor(np.ones((6, 3), np.float32))
    with pytest.raises(CnError) as e:
        ctx.gemm(A, B)
    assert e.value.status == _lib.CN_ERR_SHAPE


@pytest.mark.parametrize("M,K,N", [(128, 32, 128), (128, 64, 128), (128, 256, 128), (128, 784, 1024), (64, 128, 256),
                                   (1, 64, 16), (128, 1200, 10), (128, 12, 1200), (3, 4, 8), (130, 100, 200), (256, 512, 384), (300, 1000, 520), (128, 4096, 2304)])
@pytest.mark.parametrize("mode", [_lib.GEMM_3XTF32, _lib.GEMM_TF32])
def test_tensor_core_gemm_vs_fp64(ctx, M, K, N, mode):
    rng = np.random.default_rng(M * 7 + K * 3 + N)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    C = ctx.gemm(ctx.colmajor(A), ctx.colmajor(B), mode=mode)
    ctx.gemm_check()
    assert ctx.gemm_last_path() == ("tcgen05_3xtf32" if mode == _lib.GEMM_3XTF32 else "tcgen05_tf32")
    err = normwise(ctx.to_numpy(C), oracle.gemm_f64(A, B))
    assert err < (TOL_3XTF32 if mode == _lib.GEMM_3XTF32 else TOL_TF32), err


@pytest.mark.parametrize("M,K,N", [(128, 100000, 1024), (128, 100000, 5000), (128, 40000, 2500), (128, 100000, 2304)])
@pytest.mark.parametrize("mode", [_lib.GEMM_3XTF32, _lib.GEMM_TF32])
def test_long_inner_dimension_vs_fp64_on_sampled_columns(ctx, M, K, N, mode):
    """The regime of the README benchmark (source/test.cu, README.md:22-32): K = 100000 and the per-rank shapes of its two
    layers at 8 ranks.  Inputs as there (batch uniform [0,1), weights uniform +-4*sqrt(6/(in+out))); the accumulation runs
    over 3125 K blocks, i.e. hundreds of TMEM chains and several K splits.  Checked on sampled columns (both ends, tile
    edges, random) against an fp64 host product."""
    g = torch.Generator(device="cuda")
    g.manual_seed(K + N)
    lim = 4.0 * np.sqrt(6.0 / (K + 8 * N))
    A = torch.rand((K, M), device="cuda", generator=g)                          # column-major M x K
    W = (torch.rand((N, K), device="cuda", generator=g) * 2 - 1) * lim         # column-major K x N
    C = ctx.gemm(A, W, mode=mode)
    ctx.gemm_check()
    assert ctx.gemm_last_path() == ("tcgen05_3xtf32" if mode == _lib.GEMM_3XTF32 else "tcgen05_tf32")
    rng = np.random.default_rng(N)
    cols = np.unique(np.concatenate([[0, 1, 127, 128, 129, 255, 256, 257, N - 2, N - 1], rng.integers(0, N, 40)]))
    ci = torch.from_numpy(cols).cuda()
    ref = A.T.double().cpu().numpy() @ W[ci].double().cpu().numpy().T          # (M, ncols) in fp64 on the host
    got = C[ci].double().cpu().numpy().T
    err = float(np.abs(got - ref).max() / float(C.abs().max()))
    assert err < (TOL_3XTF32 if mode == _lib.GEMM_3XTF32 else TOL_TF32), err
    # the same launch twice gives the same bits (split-K partials are added in split order)
    C2 = ctx.gemm(A, W, mode=mode)
    assert torch.equal(C, C2)


@pytest.mark.parametrize("transA,transB", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,K,N", [(128, 1200, 1200), (784, 128, 1200), (200, 96, 333 * 4), (128, 4096, 1024)])
def test_transposed_operands_on_the_tensor_path(ctx, transA, transB, M, K, N):
    """Tdot / dotT shapes of the backward pass (source/Layer.cpp:327,334): op(A) M x K, op(B) K x N."""
    rng = np.random.default_rng(M + K + N + transA * 2 + transB)
    A = rng.uniform(-1, 1, (K, M) if transA else (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (N, K) if transB else (K, N)).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    C = ctx.gemm(ctx.colmajor(A), ctx.colmajor(B), transA=transA, transB=transB, bias=torch.from_numpy(bias).cuda(),
                 activation=_lib.ACT_RELU)
    ctx.gemm_check()
    assert ctx.gemm_last_path() == "tcgen05_3xtf32"
    ref = np.maximum(oracle.gemm_f64(A, B, transA, transB) + bias, 0)
    assert normwise(ctx.to_numpy(C), ref) < TOL_3XTF32


@pytest.mark.parametrize("mode", [_lib.GEMM_3XTF32, _lib.GEMM_TF32])
@pytest.mark.parametrize("row_major", [False, True])
@pytest.mark.parametrize("M,K,N", [(128, 4100, 1024), (96, 1000, 2304)])
def test_planes_made_ahead_give_the_same_product(ctx, mode, row_major, M, K, N):
    """cn_gemm_prepare + cn_dotmpi_prepared_f32 == cn_dotmpi_f32 / cn_tdotmpi_f32 bit for bit (the product only skips its own
    pass over the activations), the planes made on another stream and handed over through an event; a handle of another
    shape or mode is refused."""
    rng = np.random.default_rng(M + K + N + mode)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    W = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    bias = torch.from_numpy(rng.uniform(-1, 1, N).astype(np.float32)).cuda()
    dW = ctx.colmajor(W)
    a_dev = torch.from_numpy(A).cuda() if row_major else ctx.colmajor(A)      # row-major M x K == column-major K x M
    epi = cn.Epilogue(bias.data_ptr(), _lib.ACT_RELU, 0, None)
    want = ctx.empty(M, N)
    if row_major:
        cn.check(ctx.lib.cn_tdotmpi_f32(ctx.h, M, K, N, a_dev.data_ptr(), K, dW.data_ptr(), want.data_ptr(), ctypes.byref(epi), mode, 0, ctx.stream_ptr()))
    else:
        cn.check(ctx.lib.cn_dotmpi_f32(ctx.h, M, K, N, a_dev.data_ptr(), dW.data_ptr(), want.data_ptr(), ctypes.byref(epi), mode, 0, ctx.stream_ptr()))
    h = ctypes.c_void_p()
    cn.check(ctx.lib.cn_gemm_prepare_create(ctx.h, M, K, mode, ctypes.byref(h)))
    got = ctx.empty(M, N)
    # not filled yet
    assert ctx.lib.cn_dotmpi_prepared_f32(ctx.h, h, N, dW.data_ptr(), got.data_ptr(), ctypes.byref(epi), 0, ctx.stream_ptr()) == _lib.CN_ERR_ARG
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    cn.check(ctx.lib.cn_gemm_prepare(ctx.h, h, 1 if row_major else 0, a_dev.data_ptr(), K if row_major else M, ctypes.c_void_p(side.cuda_stream)))
    ev = torch.cuda.Event()
    ev.record(side)
    torch.cuda.current_stream().wait_event(ev)
    a_cm, scratch_out = ctx.colmajor(A), ctx.empty(M, N)
    n0 = ctx.lib.cn_kernel_launches()
    cn.check(ctx.lib.cn_dotmpi_prepared_f32(ctx.h, h, N, dW.data_ptr(), got.data_ptr(), ctypes.byref(epi), 0, ctx.stream_ptr()))
    n1 = ctx.lib.cn_kernel_launches()
    cn.check(ctx.lib.cn_dotmpi_f32(ctx.h, M, K, N, a_cm.data_ptr(), dW.data_ptr(), scratch_out.data_ptr(), ctypes.byref(epi), mode, 0, ctx.stream_ptr()))
    n2 = ctx.lib.cn_kernel_launches()
    ctx.gemm_check()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert (n1 - n0) == (n2 - n1) - 1               # one launch less: no pass over the activations
    ref = np.maximum(oracle.gemm_f64(A, W, False, False) + bias.cpu().numpy(), 0)
    assert normwise(ctx.to_numpy(got), ref) < (TOL_3XTF32 if mode == _lib.GEMM_3XTF32 else TOL_TF32)
    # a leading dimension below the stored rows, and a mode without planes, are refused
    assert ctx.lib.cn_gemm_prepare(ctx.h, h, 0, a_cm.data_ptr(), M - 1, ctx.stream_ptr()) == _lib.CN_ERR_SHAPE
    assert ctx.lib.cn_gemm_prepare_create(ctx.h, M, K, _lib.GEMM_FP32_SIMT, ctypes.byref(ctypes.c_void_p())) == _lib.CN_ERR_ARG
    torch.cuda.synchronize()
    ctx.lib.cn_gemm_prepare_destroy(h)


def test_config1_dot_bias_relu(ctx):
    """Single-layer dot: A 128x784, B 784x1024 uniform(-1,1) seed 0, + bias + ReLU, vs fp64."""
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (128, 784)).astype(np.float32)
    B = rng.uniform(-1, 1, (784, 1024)).astype(np.float32)
    bias = rng.uniform(-1, 1, 1024).astype(np.float32)
    dbias = torch.from_numpy(bias).cuda()
    ref = np.maximum(oracle.gemm_f64(A, B) + bias, 0)
    for mode, tol, path in [(_lib.GEMM_3XTF32, TOL_3XTF32, "tcgen05_3xtf32"), (_lib.GEMM_TF32, TOL_TF32, "tcgen05_tf32"),
                            (_lib.GEMM_FP32_SIMT, 3e-6, "simt_fp32")]:
        C = ctx.gemm(ctx.colmajor(A), ctx.colmajor(B), bias=dbias, activation=_lib.ACT_RELU, mode=mode)
        ctx.gemm_check()
        assert ctx.gemm_last_path() == path
        err = normwise(ctx.to_numpy(C), ref)
        assert err < tol, (mode, err)


@pytest.mark.parametrize("splits,nt", [(1, 1), (3, 1), (7, 1), (1, 2), (4, 2)])
def test_split_k_and_tile_variants(ctx, splits, nt):
    from clusternet_b200 import check
    check(ctx.lib.cn_gemm_set_tuning(ctx.h, nt, splits, 0))
    try:
        _split_k_and_tile_variant(ctx, splits, nt)
    finally:
        check(ctx.lib.cn_gemm_set_tuning(ctx.h, 0, 0, 0))


def _split_k_and_tile_variant(ctx, splits, nt):
    rng = np.random.default_rng(splits * 10 + nt)
    M, K, N = 128, 2048, 640
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    bias = rng.uniform(-1, 1, N).astype(np.float32)
    dA, dB, db = ctx.colmajor(A), ctx.colmajor(B), torch.from_numpy(bias).cuda()
    C1 = ctx.gemm(dA, dB, bias=db, activation=_lib.ACT_RELU)
    C2 = ctx.gemm(dA, dB, bias=db, activation=_lib.ACT_RELU)
    ctx.gemm_check()
    assert torch.equal(C1, C2), "split-K reduction must be reproducible"
    ref = np.maximum(oracle.gemm_f64(A, B) + bias, 0)
    assert normwise(ctx.to_numpy(C1), ref) < TOL_3XTF32


@pytest.mark.parametrize("act", [_lib.ACT_LINEAR, _lib.ACT_RELU, _lib.ACT_LOGISTIC, _lib.ACT_DOUBLE_RELU])
def test_fused_epilogue_matches_unfused(ctx, act):
    rng = np.random.default_rng(act)
    A = rng.uniform(-1, 1, (128, 160)).astype(np.float32)
    B = rng.uniform(-1, 1, (160, 256)).astype(np.float32)
    bias = rng.uniform(-1, 1, 256).astype(np.float32)
    dA, dB, db = ctx.colmajor(A), ctx.colmajor(B), torch.from_numpy(bias).cuda()
    plain = ctx.gemm(dA, dB)
    fused = ctx.gemm(dA, dB, bias=db, activation=act)
    unfused = ctx.bias_activation(plain, db, act)
    ctx.gemm_check()
    assert torch.equal(fused, unfused)
    want = oracle.bias_activation(ctx.to_numpy(plain), bias, act)
    got = ctx.to_numpy(fused)
    if act == _lib.ACT_LOGISTIC:
        assert np.abs(got - want).max() <= 2.4e-7   # expf differs by an ulp or two between libm and CUDA
    else:
        assert np.array_equal(got, want)


@pytest.mark.parametrize("level", [2, 4, 8, 32, 3, 5])
def test_maxout_fused_and_standalone(ctx, level):
    rng = np.random.default_rng(level)
    N = {2: 256, 4: 256, 8: 256, 32: 256, 3: 240, 5: 160}[level]
    A = rng.uniform(-1, 1, (128, 96)).astype(np.float32)
    B = rng.uniform(-1, 1, (96, N)).astype(np.float32)
    dA, dB = ctx.colmajor(A), ctx.colmajor(B)
    plain = ctx.gemm(dA, dB)
    arg = ctx.empty(128, N // level)
    out = ctx.gemm(dA, dB, maxout_level=level, argmax_out=arg)
    ctx.gemm_check()
    wv, wi = oracle.maxout(ctx.to_numpy(plain), level)
    assert np.array_equal(ctx.to_numpy(out), wv)
    assert np.array_equal(ctx.to_numpy(arg), wi)
    sv, si = ctx.maxout(plain, level)
    assert np.array_equal(ctx.to_numpy(sv), wv) and np.array_equal(ctx.to_numpy(si), wi)
