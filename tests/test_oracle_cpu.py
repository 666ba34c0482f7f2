"""The CPU oracle against the golden vectors: (a) outputs of the reference's own kernels recompiled for sm_100a and run
on a B200 (tests/golden/codec_ref_golden.npz, made by tests/golden/make_codec_golden.py), (b) properties of the codec
that follow from the reference source, (c) the reference's batch-allocator expectations."""
import os

import numpy as np
import pytest

from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "codec_ref_golden.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def test_oracle_compress_equals_reference_kernel_output(codebook, golden):
    x, p = golden["x"], float(golden["precision"])
    keep = ~golden["undefined_band"]
    got = oracle.compress(codebook, x, p)
    assert keep.sum() > 62000
    assert np.array_equal(got[keep], golden["codes"][keep])
    # the band the reference leaves undefined is exactly where the oracle says it is, and the oracle answers 125 there
    band = oracle.undefined_band_mask(codebook, x, p)
    assert np.array_equal(band, golden["undefined_band"])
    assert set(np.unique(got[band] & 0x7F)) <= {125}


def test_oracle_decompress_and_absmax_equal_reference_kernel_output(codebook, golden):
    p = float(golden["precision"])
    got = oracle.decompress(codebook, golden["codes"], p)
    assert np.array_equal(got.view(np.uint32), golden["decoded"].view(np.uint32))
    lut = oracle.decompress(codebook, np.arange(256, dtype=np.uint8), p)
    assert np.array_equal(lut.view(np.uint32), golden["decode_lut"].view(np.uint32))
    assert oracle.absmax(golden["x"][:60000]) == float(golden["absmax"]) == p


def test_special_inputs_follow_the_kernel_source(codebook):
    x = np.array([0.0, -0.0, 1e-9, -1e-9, np.inf, -np.inf, np.nan, 1.0, -1.0, 0.9957, 0.99571], np.float32)
    got = oracle.compress(codebook, x, 1.0)
    assert list(got[:9]) == [254, 254, 254, 254, 127, 255, 1, 127, 255]
    assert got[9] == 125 and got[10] == 127
    with np.errstate(all="ignore"):
        z = oracle.compress(codebook, np.array([1.0, -1.0, 0.0], np.float32), 0.0)
    assert list(z) == [127, 255, 1]          # x/0 = +-inf, 0/0 = NaN
    lut = oracle.decompress(codebook, np.arange(256, dtype=np.uint8), 0.5)
    assert lut[126] == lut[127] == lut[254] == 0.5 and lut[255] == -0.5
    assert np.array_equal(lut[:126], codebook * np.float32(0.5)) and np.array_equal(lut[128:254], -lut[:126])


def test_codes_are_scale_invariant_and_round_trip_is_stable(codebook):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(200000) * 0.1).astype(np.float32)
    p = oracle.absmax(x)
    c1 = oracle.compress(codebook, x, p)
    c2 = oracle.compress(codebook, (x * np.float32(4.0)), p * 4.0)   # exact power-of-two rescale
    assert np.array_equal(c1, c2)
    d = oracle.decompress(codebook, c1, p)
    keep = (c1 != 254) & ((c1 & 0x7F) != 127)     # specials decode to +-precision, not to themselves
    # Re-encoding a decoded value lands on the same table entry or, for an odd entry, on the even entry just below it:
    # the search never compares against its final (even) pivot, so an input equal to an odd entry resolves downwards.
    c3 = oracle.compress(codebook, d, p)
    delta = (c1[keep] & 0x7F).astype(int) - (c3[keep] & 0x7F).astype(int)
    assert set(np.unique(delta)) <= {0, 1}
    assert np.all((delta == 0) | ((c1[keep] & 1) == 1))
    assert np.array_equal(c3[keep] & 0x80, c1[keep] & 0x80)
    # an input just below an odd entry still maps to the even entry below it: the error can reach one table step (0.0172)
    assert np.abs(d[keep] - x[keep]).max() <= 0.0175 * p


def test_batch_oracle_reproduces_reference_test_totals():
    """tests/batchAllocator_test.cu:22-114: arange(10000 x 784) data, 20 % cross-validation, batch 128: every element of
    every batch equals a running counter; two epochs."""
    rows, cols, B = 10000, 784, 128
    train = int(np.ceil(rows * (1.0 - 0.2)))
    b = oracle.BatchOracle(train, B)
    assert b.total == 63 and train == 8000
    seen = 0
    start, n = b.current
    for epoch in range(2):
        for i in range(b.total):
            assert start == (i * B) and n == (B if i < b.total - 1 else train % B)
            seen += n * cols
            start, n = b.advance()
    assert seen == 2 * 6272000     # 6 272 000 training values per epoch in the reference's test


def test_maxout_oracle_tree_and_ties():
    C = np.array([[1, 5, 5, 2, 7, 7, 7, 0]], np.float32)
    v, i = oracle.maxout(C, 4)
    assert list(v[0]) == [5, 7]
    # tree order of the 32-slot reduction: at offset 2 slot 0 takes slot 2 only when strictly smaller, etc.
    assert list(i[0]) == [2.0, 4.0] or list(i[0]) == [1.0, 4.0]
    rng = np.random.default_rng(0)
    X = rng.standard_normal((50, 96)).astype(np.float32)
    v, i = oracle.maxout(X, 8)
    assert np.array_equal(v, X.reshape(50, 12, 8).max(-1))
    assert np.array_equal(i, (X.reshape(50, 12, 8).argmax(-1) + np.arange(12) * 8).astype(np.float32))
