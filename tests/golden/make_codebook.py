"""Extracts the 126-entry dynamic-float codebook from the reference's HDF5 file into a raw
little-endian float32 dump (504 bytes), checking both sha256 sums.

    python tests/golden/make_codebook.py <reference tree>/source/8bit_floats.hdf5

The file is a version-0 HDF5 container; its only dataset (/Default, 126 x 1 float32, contiguous) is the
last 504 bytes.  The dump is written to tests/golden/codebook_126.f32 and to clusternet_b200/data/.
"""
import hashlib
import os
import sys

FILE_SHA = "d584e1a65e8d1f0b48e53dcf814ea2d3bd43982b6088c7c1159e616e4418ae7b"
PAYLOAD_SHA = "c2dbfffe982a2fc5430f56cbb44857fe8e6b610b4445f3dae2a64b0b6c977a37"

if len(sys.argv) != 2:
    sys.exit(__doc__)
src = sys.argv[1]
blob = open(src, "rb").read()
assert hashlib.sha256(blob).hexdigest() == FILE_SHA, "unexpected codebook file"
assert blob[:8] == b"\x89HDF\r\n\x1a\n" and len(blob) == 2648
payload = blob[-504:]
assert hashlib.sha256(payload).hexdigest() == PAYLOAD_SHA
here = os.path.dirname(os.path.abspath(__file__))
for dst in (os.path.join(here, "codebook_126.f32"), os.path.join(here, "..", "..", "clusternet_b200", "data", "8bit_floats.f32")):
    with open(dst, "wb") as f:
        f.write(payload)
    print("wrote", os.path.normpath(dst))
