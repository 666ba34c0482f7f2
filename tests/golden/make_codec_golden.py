"""Generates golden vectors for the 8-bit codec by running the REFERENCE's own kernels (kCompression_8bit,
kDecompression_8bit, abs + max), recompiled for sm_100a into oracle/_ref/libcnref.so, on a GPU.

    python tests/golden/make_codec_golden.py output.npz        (needs a GPU and oracle/_ref/libcnref.so)

Inputs: 60000 values ~ N(0, 0.1) from numpy's default_rng(1) plus every codebook entry, every midpoint of adjacent
entries, the two range thresholds and a few magnitudes, each with its +-2 ulp neighbours and both signs, plus
zeros / infinities / NaN / denormals; precision = the largest finite |x| of the random part.  Stored: the inputs,
the precision, the reference kernel's codes, its decode of those codes, its absmax, and a mask of the inputs for which
the reference reads an unwritten shared-memory word (tbl[125] < |x/precision| <= 0.995703), whose reference output
is not defined and must not be compared.
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402


def inputs(tbl):
    rng = np.random.default_rng(1)
    rnd = (rng.standard_normal(60000) * 0.1).astype(np.float32)
    p = float(np.abs(rnd).max())
    vals = np.concatenate([tbl.astype(np.float64) * p, (tbl[:-1].astype(np.float64) + tbl[1:]) * 0.5 * p,
                           np.array([0.0000015, 0.995703, 1.0, 0.5, 2.0, 1e-8]) * p]).astype(np.float32)
    bits = vals.view(np.uint32).astype(np.int64)
    nb = np.concatenate([bits + d for d in (-2, -1, 0, 1, 2)]).astype(np.uint32).view(np.float32)
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45, 3.4e38, -3.4e38], np.float32)
    return np.concatenate([rnd, nb, -nb, special]), p


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    out_path = sys.argv[1]
    L = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libcnref.so"))
    L.ref_absmax.restype = ctypes.c_float
    tbl = np.fromfile(os.path.join(ROOT, "tests", "golden", "codebook_126.f32"), dtype="<f4")
    x, p = inputs(tbl)
    n = x.size
    fp = ctypes.c_void_p
    d_tbl, d_x = torch.from_numpy(tbl).cuda(), torch.from_numpy(x).cuda()
    d_codes = torch.zeros(n, dtype=torch.uint8, device="cuda")
    d_out = torch.zeros(n, dtype=torch.float32, device="cuda")
    d_tmp = torch.zeros(60000, dtype=torch.float32, device="cuda")
    assert L.ref_compression_8bit(fp(d_tbl.data_ptr()), fp(d_x.data_ptr()), ctypes.c_float(p), n, fp(d_codes.data_ptr())) == 0
    assert L.ref_decompression_8bit(fp(d_tbl.data_ptr()), fp(d_codes.data_ptr()), ctypes.c_float(p), n, fp(d_out.data_ptr())) == 0
    amax = L.ref_absmax(fp(d_x.data_ptr()), fp(d_tmp.data_ptr()), 60000)
    all_codes = torch.arange(256, dtype=torch.uint8, device="cuda")
    d_lut = torch.zeros(256, dtype=torch.float32, device="cuda")
    assert L.ref_decompression_8bit(fp(d_tbl.data_ptr()), fp(all_codes.data_ptr()), ctypes.c_float(p), 256, fp(d_lut.data_ptr())) == 0
    band = oracle.undefined_band_mask(tbl, x, p)
    os.makedirs(os.path.dirname(out_path), exist_ok=True)
    np.savez_compressed(out_path, x=x, precision=np.float32(p), codes=d_codes.cpu().numpy(), decoded=d_out.cpu().numpy(),
                        absmax=np.float32(amax), decode_lut=d_lut.cpu().numpy(), undefined_band=band)
    mine = oracle.compress(tbl, x, p)
    keep = ~band
    print(f"wrote {out_path}: {n} values, {int(band.sum())} in the undefined band, oracle agrees on "
          f"{int((mine[keep] == d_codes.cpu().numpy()[keep]).sum())}/{int(keep.sum())} defined codes")


if __name__ == "__main__":
    main()
