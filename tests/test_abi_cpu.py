"""CPU-only checks of the C ABI: the library loads, exports every symbol the header declares, and its host-only
entry points (codebook loader, threshold builder, shard arithmetic, error reporting) behave."""
import ctypes
import os

import numpy as np
import pytest

import clusternet_b200
from clusternet_b200 import _lib
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_lib):
    names = _lib.declared_symbols()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(built_lib, n)]
    assert not missing, missing
    unbound = [n for n in names if n not in _lib._SIGNATURES]
    assert not unbound, f"declared but not bound in _lib.py: {unbound}"
    assert built_lib.cn_compiled_arch() == 100
    assert built_lib.cn_status_string(5).decode() == "CN_ERR_TIMEOUT"


def test_python_constants_equal_the_header(built_lib):
    """The ctypes binding repeats the header's status codes and option bits by value: they must not drift apart."""
    import re
    text = open(os.path.join(ROOT, "include", "clusternet_b200.h")).read()
    defines = {m.group(1): int(m.group(2), 0) for m in re.finditer(r"^#define\s+(CN_[A-Z0-9_]+)\s+(\d+|0x[0-9a-fA-F]+)\s*$", text, re.M)}
    enums = {m.group(1): int(m.group(2)) for m in re.finditer(r"^\s+(CN_[A-Z0-9_]+)\s*=\s*(\d+)\s*,?", text, re.M)}
    for name in ("KEEP_ROW_MAJOR", "NO_COL_MAJOR", "SHARDED_UPLOAD", "PUSH_BY_KERNEL", "LOOKAHEAD"):
        assert defines["CN_BATCH_" + name] == getattr(_lib, "BATCH_" + name), name
    bits = [defines["CN_BATCH_" + n] for n in ("KEEP_ROW_MAJOR", "NO_COL_MAJOR", "SHARDED_UPLOAD", "PUSH_BY_KERNEL", "LOOKAHEAD")]
    assert len(set(bits)) == 5 and all(b & (b - 1) == 0 for b in bits)        # distinct single bits
    for name in ("CN_OK", "CN_ERR_ARG", "CN_ERR_SHAPE", "CN_ERR_CUDA", "CN_ERR_NCCL", "CN_ERR_TIMEOUT", "CN_ERR_UNSUPPORTED", "CN_ERR_NOMEM"):
        assert enums[name] == getattr(_lib, name), name
        assert built_lib.cn_status_string(enums[name]).decode() == name
    for name in ("3XTF32", "TF32", "FP32_SIMT"):
        assert enums.get("CN_GEMM_" + name, defines.get("CN_GEMM_" + name)) == getattr(_lib, "GEMM_" + name), name


def test_codebook_loader_reads_raw_and_hdf5_container(built_lib, codebook, tmp_path):
    tbl = np.zeros(126, np.float32)
    raw = os.path.join(ROOT, "tests", "golden", "codebook_126.f32")
    assert built_lib.cn_codebook_load(raw.encode(), tbl.ctypes.data) == 0
    assert np.array_equal(tbl, codebook)
    # an HDF5 file with the table as its 126 x 1 /Default dataset (the reference file's layout)
    fake = tmp_path / "c.hdf5"
    clusternet_b200.write_hdf5(fake, codebook.reshape(126, 1))
    tbl2 = np.zeros(126, np.float32)
    assert built_lib.cn_codebook_load(str(fake).encode(), tbl2.ctypes.data) == 0
    assert np.array_equal(tbl2, codebook)
    assert np.array_equal(oracle.load_codebook(str(fake)), codebook)
    bad = tmp_path / "bad.bin"
    bad.write_bytes(bytes(777))
    assert built_lib.cn_codebook_load(str(bad).encode(), tbl2.ctypes.data) == _lib.CN_ERR_ARG
    assert b"neither" in built_lib.cn_last_error()
    # the packaged copy is the same table
    assert np.array_equal(clusternet_b200.load_codebook(), codebook)


def test_hdf5_reader_on_the_reference_fixture_and_round_trips(built_lib, tmp_path):
    # the reference's own check (tests/util_test.cu:18-20): element i of numpy_arange_as_h5py.hdf5 is i (float64 on disk)
    a = clusternet_b200.read_hdf5(os.path.join(ROOT, "tests", "golden", "numpy_arange_as_h5py.hdf5"))
    assert a.dtype == np.float32 and a.shape == (10, 50)
    assert np.array_equal(a.ravel(), np.arange(500, dtype=np.float32))
    rng = np.random.default_rng(5)
    for shape in [(1, 1), (7, 1), (1, 9), (33, 17), (500, 784)]:
        x = rng.standard_normal(shape).astype(np.float32)
        path = tmp_path / f"m{shape[0]}x{shape[1]}.hdf5"
        clusternet_b200.write_hdf5(path, x)
        assert np.array_equal(clusternet_b200.read_hdf5(path), x)
        assert os.path.getsize(path) == 2048 + x.nbytes
    # shape query and conversion into a caller's buffer
    import ctypes
    r, c = ctypes.c_int64(), ctypes.c_int64()
    assert built_lib.cn_hdf5_dims(str(path).encode(), b"/Default", ctypes.byref(r), ctypes.byref(c)) == 0
    assert (r.value, c.value) == x.shape
    buf = np.full(x.size + 3, -7.0, np.float32)
    assert built_lib.cn_hdf5_read_f32_into(str(path).encode(), b"/Default", buf.ctypes.data, buf.size) == 0
    assert np.array_equal(buf[:x.size].reshape(x.shape), x) and np.all(buf[x.size:] == -7.0)
    assert built_lib.cn_hdf5_read_f32_into(str(path).encode(), b"/Default", buf.ctypes.data, x.size - 1) == _lib.CN_ERR_SHAPE
    clusternet_b200.write_hdf5(tmp_path / "named.hdf5", x, "/labels")
    assert np.array_equal(clusternet_b200.read_hdf5(tmp_path / "named.hdf5", "labels"), x)
    with pytest.raises(_lib.CnError, match="not found"):
        clusternet_b200.read_hdf5(tmp_path / "named.hdf5")


def test_sparse_hdf5_reader_on_the_reference_fixture(built_lib):
    # the reference's own (commented) check, tests/util_test.cu:22-44: a 10 x 50 arange stored as scipy CSR through h5py
    data, indices, indptr, shape = clusternet_b200.read_sparse_hdf5(os.path.join(ROOT, "tests", "golden", "scipy_sparse_arange_as_h5py.hdf5"))
    assert shape == (10, 50) and data.dtype == np.float32 and indices.dtype == np.int32 and indptr.dtype == np.int32
    assert np.array_equal(data, np.arange(1, 500, dtype=np.float32))
    assert np.array_equal(indices, np.arange(1, 500, dtype=np.int32) % 50)
    assert np.array_equal(indptr, np.array([0] + [50 * r - 1 for r in range(1, 11)], np.int32))
    dense = np.zeros(shape, np.float32)
    for r in range(shape[0]):
        dense[r, indices[indptr[r]:indptr[r + 1]]] = data[indptr[r]:indptr[r + 1]]
    assert np.array_equal(dense, np.arange(500, dtype=np.float32).reshape(10, 50))
    with pytest.raises(TypeError):
        clusternet_b200.read_hdf5(os.path.join(ROOT, "tests", "golden", "numpy_arange_as_h5py.hdf5"), dtype=np.float64)


def test_hdf5_reader_rejects_damaged_files(built_lib, tmp_path):
    good = open(os.path.join(ROOT, "tests", "golden", "numpy_arange_as_h5py.hdf5"), "rb").read()
    cases = {
        "short": good[:64],
        "nosig": b"\0" * 8 + good[8:],
        "truncated_data": good[:3000],
        "truncated_meta": good[:700],
        "v2_superblock": good[:8] + b"\x02" + good[9:],
    }
    for name, blob in cases.items():
        path = tmp_path / (name + ".hdf5")
        path.write_bytes(blob)
        with pytest.raises(_lib.CnError):
            clusternet_b200.read_hdf5(path)
    # every single-byte corruption of the metadata is either read consistently or refused, never a crash
    rng = np.random.default_rng(11)
    for _ in range(300):
        blob = bytearray(good)
        off = int(rng.integers(8, 1400))
        blob[off] = int(rng.integers(0, 256))
        path = tmp_path / "fuzz.hdf5"
        path.write_bytes(bytes(blob))
        try:
            out = clusternet_b200.read_hdf5(path)
            assert out.ndim == 2
        except _lib.CnError:
            pass
    with pytest.raises(_lib.CnError):
        clusternet_b200.read_hdf5(tmp_path / "missing.hdf5")


def test_hdf5_datasets_of_the_reference_when_mounted(built_lib):
    from conftest import reference_dir
    if not reference_dir():
        pytest.skip("reference tree not mounted")
    ref = os.path.join(reference_dir(), "tests")
    X = clusternet_b200.read_hdf5(os.path.join(ref, "mnist_mini_X.hdf5"))
    y = clusternet_b200.read_hdf5(os.path.join(ref, "mnist_mini_y.hdf5"))
    assert X.shape == (500, 784) and y.shape == (500, 1)
    assert X.min() >= 0.0 and X.max() <= 1.0 and set(np.unique(y)) <= set(range(10))
    assert list(y[:5, 0]) == [5, 0, 4, 1, 9]      # the first MNIST labels


def test_codebook_matches_reference_file_when_mounted(codebook):
    from conftest import reference_dir
    if not reference_dir():
        pytest.skip("reference tree not mounted")
    ref = os.path.join(reference_dir(), "source", "8bit_floats.hdf5")
    import hashlib
    blob = open(ref, "rb").read()
    assert hashlib.sha256(blob).hexdigest() == "d584e1a65e8d1f0b48e53dcf814ea2d3bd43982b6088c7c1159e616e4418ae7b"
    assert np.array_equal(oracle.load_codebook(ref), codebook)


def test_threshold_table_equals_the_restated_kernel_for_every_float(built_lib, codebook):
    """The product derives 127 thresholds from the codebook; 'number of thresholds <= |a|' must reproduce the restated
    kCompression_8bit decision for EVERY non-negative fp32 (0 .. +inf: 2 139 095 041 bit patterns)."""
    thr = np.zeros(127, np.uint32)
    lc = np.zeros(128, np.uint8)
    assert built_lib.cn_codec_build_thresholds(codebook.ctypes.data, thr.ctypes.data, lc.ctypes.data) == 0
    assert np.all(np.diff(thr.astype(np.int64)) > 0)
    assert list(lc) == [254] + list(range(126)) + [127]
    bad, first = oracle.sweep_thresholds(codebook, thr, lc)
    assert bad == 0, hex(first)


def test_threshold_builder_rejects_a_broken_codebook(built_lib, codebook):
    thr = np.zeros(127, np.uint32)
    lc = np.zeros(128, np.uint8)
    broken = codebook.copy()
    broken[10] = broken[9]
    assert built_lib.cn_codec_build_thresholds(broken.ctypes.data, thr.ctypes.data, lc.ctypes.data) == _lib.CN_ERR_ARG


@pytest.mark.parametrize("n,g", [(40000, 8), (20000, 8), (1024, 3), (10, 4), (7, 7), (5, 8), (0, 2)])
def test_shard_cols_matches_reference_split(built_lib, n, g):
    """split = N / G, remainder to the last rank (source/clusterNet.cpp:515-516,926-931)."""
    total = 0
    for r in range(g):
        a, b = ctypes.c_int64(), ctypes.c_int64()
        assert built_lib.cn_shard_cols(n, r, g, ctypes.byref(a), ctypes.byref(b)) == 0
        assert (a.value, b.value) == oracle.shard_cols(n, r, g)
        assert a.value == total
        total += b.value
    assert total == n
    assert built_lib.cn_shard_cols(10, 4, 4, None, None) == _lib.CN_ERR_ARG


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


@pytest.mark.parametrize("program", ["facade_test", "layer_test", "readme_test", "batch_test"])
def test_facade_programs_compile_and_link(built_lib, tmp_path, program):
    """The header-only facade and the programs written against it build without a GPU (they run in the GPU tests)."""
    import subprocess
    libdir = os.path.join(ROOT, "clusternet_b200")
    r = subprocess.run(["/usr/local/cuda/bin/nvcc", "-std=c++17", "-O0", "-gencode", "arch=compute_100a,code=sm_100a",
                        os.path.join(ROOT, "tests", program + ".cu"), "-o", str(tmp_path / program), f"-L{libdir}", "-lclusternet_b200"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
