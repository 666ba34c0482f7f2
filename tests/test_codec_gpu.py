"""Parity of the CUDA 8-bit codec with the CPU restatement of the reference kernels (bit-exact) and, where the
recompiled reference kernels are present (oracle/_ref), with the reference's own GPU output."""
import ctypes
import os

import numpy as np
import pytest
import torch

import clusternet_b200 as cn
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def adversarial(tbl, p):
    """Table entries, decision boundaries and specials, scaled by precision p, with +-2 ulp neighbours."""
    vals = [tbl.astype(np.float64) * p, (tbl[:-1].astype(np.float64) + tbl[1:]) * 0.5 * p,
            np.array([0.0000015, 0.995703, 1.0, 0.5, 2.0, 1e-8, 1e-30, 1e30]) * p]
    v = np.concatenate(vals).astype(np.float32)
    bits = v.view(np.uint32).astype(np.int64)
    nb = np.concatenate([bits + d for d in (-2, -1, 0, 1, 2)])
    nb = np.clip(nb, 0, 0x7F7FFFFF).astype(np.uint32).view(np.float32)
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45, 3.4e38, -3.4e38], np.float32)
    return np.concatenate([nb, -nb, special])


def run_compress(ctx, x, p):
    d = torch.from_numpy(x).cuda()
    out = ctx.compress(d, p)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 127, 128, 129, 1023, 4096, 100003, 1 << 20])
def test_compress_sizes_bit_exact(ctx, n):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 0.1).astype(np.float32)
    p = float(np.abs(x).max()) if n else 1.0
    got = run_compress(ctx, x, p)
    assert np.array_equal(got, oracle.compress(ctx.codebook, x, p))


@pytest.mark.parametrize("p", [1.0, 0.1, 0.37251, 3.0e-5, 7.77e7, -0.25, 1.9999999, 1.0000001, 2.0 ** -99, 2.0 ** 99])
def test_compress_adversarial_fast_path(ctx, p):
    x = adversarial(ctx.codebook, abs(p))
    got = run_compress(ctx, x, p)
    want = oracle.compress(ctx.codebook, x, p)
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, (x[bad[:8]], got[bad[:8]], want[bad[:8]])


@pytest.mark.parametrize("p", [0.0, -0.0, float("inf"), float("nan"), 1e-40, 1e-37, 3e38, 2.0 ** -101])
def test_compress_generic_path_precisions(ctx, p):
    """Precisions for which the in-kernel boundary table is not built: per-element IEEE division instead."""
    rng = np.random.default_rng(5)
    base = 1.0 if not np.isfinite(p) or p == 0 else abs(p)
    x = np.concatenate([adversarial(ctx.codebook, base), (rng.standard_normal(5000) * base).astype(np.float32)])
    with np.errstate(all="ignore"):
        got = run_compress(ctx, x, p)
        want = oracle.compress(ctx.codebook, x, p)
    assert np.array_equal(got, want)


def test_compress_config2_full_size(ctx):
    """4096 x 4096 ~ N(0, 0.1), seed 1, precision = absmax: bit-exact codes, then decode round trip."""
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(4096 * 4096) * 0.1).astype(np.float32)
    d = torch.from_numpy(x).cuda()
    pm = ctx.absmax(d)
    codes = ctx.compress(d, pm)
    back = ctx.decompress(codes, pm)
    torch.cuda.synchronize()
    p = float(pm.item())
    assert p == oracle.absmax(x)
    want = oracle.compress(ctx.codebook, x, p, threads=True)
    got = codes.cpu().numpy()
    assert np.array_equal(got, want)
    assert np.array_equal(back.cpu().numpy(), oracle.decompress(ctx.codebook, want, p, threads=True))
    # the host-scalar and device-scalar entry points agree
    codes2 = ctx.compress(d, p)
    torch.cuda.synchronize()
    assert torch.equal(codes, codes2)


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 2047, 8192, 100003, 1 << 20, (4 << 20) - 1, 4096 * 4096 + 2])
def test_fused_absmax_compress_equals_the_two_calls(ctx, n):
    """cn_absmax_compress_8bit (one cooperative launch: reduce, grid barrier, code) gives the scale and the codes of
    cn_absmax_f32 followed by cn_compress_8bit_dp, on consecutive calls and for a buffer that is not 16-byte aligned
    (two-call fallback)."""
    rng = np.random.default_rng(n + 1)
    for rep in range(3):
        x = torch.from_numpy((rng.standard_normal(n + 1) * rng.uniform(1e-3, 30)).astype(np.float32)).cuda()
        a = x[:n] if rep < 2 else x[1:n + 1]
        pm = ctx.absmax(a)
        want = ctx.compress(a, pm)
        got, scale = ctx.absmax_compress(a)
        torch.cuda.synchronize()
        ctx.gemm_check()
        assert scale.item() == pm.item()
        assert torch.equal(got, want), (n, rep)
    if n:
        p = float(pm.item())
        assert np.array_equal(got.cpu().numpy(), oracle.compress(ctx.codebook, a.cpu().numpy(), p))


def test_fused_absmax_compress_replays_from_a_cuda_graph(ctx):
    """The one-launch form keeps its grid barrier's state on the device only, so a recorded launch can be replayed: every
    replay must wait for ITS maxima.  The data shrink from replay to replay - a barrier that let a CTA through early would
    fold a stale, larger maximum of the replay before into the scale."""
    n = 1_000_003 + 1                                     # the one-launch form (at most 4 Mi elements), with a ragged end
    rng = np.random.default_rng(99)
    base = torch.from_numpy((rng.standard_normal(n) * 5).astype(np.float32)).cuda()
    a = base.clone()
    codes = torch.empty(n, dtype=torch.uint8, device="cuda")
    scale = torch.zeros(1, device="cuda")
    cn.check(ctx.lib.cn_absmax_compress_8bit(ctx.h, a.data_ptr(), n, scale.data_ptr(), codes.data_ptr(), ctx.stream_ptr()))   # warm-up
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        cn.check(ctx.lib.cn_absmax_compress_8bit(ctx.h, a.data_ptr(), n, scale.data_ptr(), codes.data_ptr(),
                                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    for rep, f in enumerate((1.0, 0.5, 0.01, 3.0, 0.001)):
        a.copy_(base * f)
        g.replay()
        torch.cuda.synchronize()
        pm = ctx.absmax(a)
        want = ctx.compress(a, pm)
        torch.cuda.synchronize()
        assert scale.item() == pm.item(), (rep, f)
        assert torch.equal(codes, want), (rep, f)
    # ... and calls outside the graph still work afterwards
    got, sc = ctx.absmax_compress(a)
    torch.cuda.synchronize()
    assert sc.item() == pm.item() and torch.equal(got, want)
    ctx.gemm_check()


def test_unaligned_buffers_take_scalar_path(ctx):
    rng = np.random.default_rng(7)
    x = (rng.standard_normal(10007) * 0.3).astype(np.float32)
    big = torch.zeros(10007 + 8, dtype=torch.float32, device="cuda")
    big[1:1 + x.size] = torch.from_numpy(x).cuda()
    src = big[1:1 + x.size]          # 4-byte aligned only
    outbuf = torch.zeros(10007 + 8, dtype=torch.uint8, device="cuda")
    dst = outbuf[3:3 + x.size]       # 1-byte aligned only
    ctx.compress(src, 1.0, out=dst)
    torch.cuda.synchronize()
    want = oracle.compress(ctx.codebook, x, 1.0)
    assert np.array_equal(dst.cpu().numpy(), want)
    fl = torch.zeros(10007 + 8, dtype=torch.float32, device="cuda")
    ctx.decompress(dst, 0.5, out=fl[1:1 + x.size])
    torch.cuda.synchronize()
    assert np.array_equal(fl[1:1 + x.size].cpu().numpy(), oracle.decompress(ctx.codebook, want, 0.5))
    assert float(fl[0]) == 0.0 and float(fl[1 + x.size]) == 0.0


@pytest.mark.parametrize("p", [1.0, 0.1, -3.5, 0.0, float("inf")])
def test_decompress_all_codes(ctx, p):
    codes = np.arange(256, dtype=np.uint8).repeat(5)
    d = torch.from_numpy(codes).cuda()
    out = ctx.decompress(d, p)
    torch.cuda.synchronize()
    with np.errstate(all="ignore"):
        want = oracle.decompress(ctx.codebook, codes, p)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("extra", [0, 517])
def test_decompress_large_tensor_takes_the_sixteen_codes_kernel(ctx, extra):
    """From 2^26 codes on (16-byte aligned) a warp decodes 512 codes per load and exchanges words by shuffles; every element
    must still be table[code], the ragged end (no whole warp, no whole 16 bytes) included.  The 256-entry table itself is
    pinned against the oracle, so a gather through it on the device is the full-size check."""
    n = (1 << 26) + extra
    g = torch.Generator(device="cuda").manual_seed(11 + extra)
    codes = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=g)
    p = 0.37
    table = ctx.decompress(torch.arange(256, dtype=torch.uint8, device="cuda"), p)
    torch.cuda.synchronize()
    want_tbl = oracle.decompress(ctx.codebook, np.arange(256, dtype=np.uint8), p)
    assert np.array_equal(table.cpu().numpy().view(np.uint32), want_tbl.view(np.uint32))
    out = ctx.decompress(codes, p)
    pd = torch.tensor([p], device="cuda")
    out_dp = torch.empty_like(out)
    cn.check(ctx.lib.cn_decompress_8bit_dp(ctx.h, codes.data_ptr(), pd.data_ptr(), n, out_dp.data_ptr(), ctx.stream_ptr()))
    torch.cuda.synchronize()
    step = 1 << 24                                  # gather in pieces: the int64 index of the whole tensor would take 512 MiB
    for lo in range(0, n, step):
        want = table[codes[lo:lo + step].long()]
        assert torch.equal(out[lo:lo + step].view(torch.int32), want.view(torch.int32)), lo
        assert torch.equal(out_dp[lo:lo + step].view(torch.int32), want.view(torch.int32)), lo


@pytest.mark.parametrize("n", [0, 1, 5, 1000, 65537, 1 << 22])
def test_absmax(ctx, n):
    rng = np.random.default_rng(n + 1)
    x = (rng.standard_normal(n) * 3).astype(np.float32)
    d = torch.from_numpy(x).cuda()
    for _ in range(2):   # twice: the ticket counter must be back at zero
        got = float(ctx.absmax(d).item())
        assert got == oracle.absmax(x)


def _ref_lib():
    path = os.path.join(ROOT, "oracle", "_ref", "libcnref.so")
    if not os.path.exists(path):
        pytest.skip("reference kernels not built (oracle/_ref)")
    L = ctypes.CDLL(path)
    L.ref_absmax.restype = ctypes.c_float
    return L


def test_against_reference_kernels_on_this_gpu(ctx):
    """The reference's kCompression_8bit / kDecompression_8bit, recompiled for sm_100a, on the same buffers.
    Inputs in the band where the reference reads an unwritten shared-memory word are excluded and counted."""
    L = _ref_lib()
    rng = np.random.default_rng(1)
    n = 1 << 22
    x = (rng.standard_normal(n) * 0.1).astype(np.float32)
    adv = adversarial(ctx.codebook, float(np.abs(x).max()))
    adv = adv[np.isfinite(adv)]
    x[:adv.size] = adv
    p = float(np.abs(x).max())
    d = torch.from_numpy(x).cuda()
    tbl = torch.from_numpy(ctx.codebook).cuda()
    ref_codes = torch.zeros(n, dtype=torch.uint8, device="cuda")
    fp = ctypes.c_void_p
    assert L.ref_compression_8bit(fp(tbl.data_ptr()), fp(d.data_ptr()), ctypes.c_float(p), n, fp(ref_codes.data_ptr())) == 0
    mine = ctx.compress(d, p)
    torch.cuda.synchronize()
    band = oracle.undefined_band_mask(ctx.codebook, x, p)
    nan = np.isnan(x)
    a, b = mine.cpu().numpy(), ref_codes.cpu().numpy()
    keep = ~band
    assert np.array_equal(a[keep], b[keep]), f"{(a[keep] != b[keep]).sum()} codes differ from the reference kernel"
    print(f"reference-kernel comparison: {n} values, {int(band.sum())} in the undefined band, {int(nan.sum())} NaN")
    ref_out = torch.zeros(n, dtype=torch.float32, device="cuda")
    assert L.ref_decompression_8bit(fp(tbl.data_ptr()), fp(mine.data_ptr()), ctypes.c_float(p), n, fp(ref_out.data_ptr())) == 0
    out = ctx.decompress(mine, p)
    torch.cuda.synchronize()
    assert torch.equal(out, ref_out)
    tmp = torch.empty_like(d)
    assert L.ref_absmax(fp(d.data_ptr()), fp(tmp.data_ptr()), n) == float(ctx.absmax(d).item())
