"""Thin Python harness over the C ABI: torch tensors hold device memory, raw pointers go down.

Matrices follow the reference's convention: a logical rows x cols matrix is stored on the device in
column-major order (leading dimension = rows).  Here such a matrix is a contiguous torch tensor of
shape (cols, rows) — its memory is exactly the column-major array — and `colmajor()` / `to_numpy()`
convert from and to ordinary row-major numpy arrays.
"""
import ctypes
import os

import numpy as np
import torch

from . import _lib
from ._lib import Epilogue, check, load

HERE = os.path.dirname(os.path.abspath(__file__))


def codebook_path():
    """Codebook file: $CN_CODEBOOK (the reference's 8bit_floats.hdf5 or a raw dump), else the packaged dump."""
    return os.environ.get("CN_CODEBOOK", os.path.join(HERE, "data", "8bit_floats.f32"))


def load_codebook(path=None):
    lib = load()
    tbl = np.zeros(126, np.float32)
    check(lib.cn_codebook_load((path or codebook_path()).encode(), tbl.ctypes.data))
    return tbl


def read_hdf5(path, dataset="/Default", dtype=np.float32):
    """Dense dataset of an HDF5 file as a (rows, cols) array, float32 (read_hdf5 of the reference,
    source/util.cu:100-131) or int32 (the index datasets of its CSR files)."""
    import ctypes
    lib = load()
    dtype = np.dtype(dtype)
    if dtype not in (np.dtype(np.float32), np.dtype(np.int32)):
        raise TypeError("read_hdf5 returns float32 or int32")
    fn, ctype = (lib.cn_hdf5_read_f32, ctypes.c_float) if dtype == np.float32 else (lib.cn_hdf5_read_i32, ctypes.c_int32)
    p, r, c = ctypes.c_void_p(), ctypes.c_int64(), ctypes.c_int64()
    check(fn(str(path).encode(), dataset.encode(), ctypes.byref(p), ctypes.byref(r), ctypes.byref(c)))
    try:
        flat = np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctype)), shape=(r.value * c.value,))
        return flat.reshape(r.value, c.value).copy()
    finally:
        lib.cn_host_free(p)


def read_sparse_hdf5(path):
    """CSR matrix written by scipy + h5py (read_sparse_hdf5 of the reference, source/util.cu:133-198):
    returns (data float32, indices int32, indptr int32, (rows, cols))."""
    data = read_hdf5(path, "/data").ravel()
    indices = read_hdf5(path, "/indices", np.int32).ravel()
    indptr = read_hdf5(path, "/indptr", np.int32).ravel()
    shape = read_hdf5(path, "/shape", np.int32).ravel()
    return data, indices, indptr, (int(shape[0]), int(shape[1]))


def write_hdf5(path, a, dataset="/Default"):
    """write_hdf5 of the reference (source/util.cu:202-216): one float32 rank-2 dataset in a new file."""
    a = np.ascontiguousarray(a, np.float32)
    if a.ndim == 1:
        a = a.reshape(-1, 1)
    check(load().cn_hdf5_write_f32(str(path).encode(), dataset.encode(), a.ctypes.data, a.shape[0], a.shape[1]))


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        return t.data_ptr()
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    return int(t)


class Context:
    """One cn_context bound to one CUDA device."""

    def __init__(self, device=0, codebook=None):
        self.lib = load()
        if not torch.cuda.is_available():
            raise RuntimeError("clusternet_b200 needs a CUDA device (sm_100a); none is visible")
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.codebook = np.ascontiguousarray(codebook if codebook is not None else load_codebook(), np.float32)
        h = ctypes.c_void_p()
        check(self.lib.cn_context_create(device, self.codebook.ctypes.data, ctypes.byref(h)))
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.lib.cn_context_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def stream_ptr(stream=None):
        s = stream if stream is not None else torch.cuda.current_stream()
        return ctypes.c_void_p(s.cuda_stream)

    def empty(self, rows, cols):
        """Device matrix rows x cols, column-major (tensor shape (cols, rows))."""
        return torch.empty((cols, rows), dtype=torch.float32, device=self.device)

    def colmajor(self, a):
        """Row-major numpy (rows x cols) -> device column-major matrix, through the library's own upload path."""
        a = np.ascontiguousarray(a, np.float32)
        rows, cols = a.shape
        host = torch.from_numpy(a).pin_memory()
        stage = torch.empty((rows, cols), dtype=torch.float32, device=self.device)
        out = self.empty(rows, cols)
        check(self.lib.cn_upload_row_major(self.h, _ptr(host), _ptr(stage), _ptr(out), rows, cols, self.stream_ptr()))
        torch.cuda.current_stream().synchronize()
        return out

    def to_numpy(self, m):
        """Device column-major matrix (tensor (cols, rows)) -> row-major numpy, through the download path."""
        cols, rows = m.shape
        stage = torch.empty((rows, cols), dtype=torch.float32, device=self.device)
        host = torch.empty((rows, cols), dtype=torch.float32).pin_memory()
        check(self.lib.cn_download_row_major(self.h, _ptr(m), _ptr(stage), _ptr(host), rows, cols, self.stream_ptr()))
        torch.cuda.current_stream().synchronize()
        return host.numpy().copy()

    # ------------------------------------------------------------------ codec
    def absmax(self, a, out=None):
        out = out if out is not None else torch.empty(1, dtype=torch.float32, device=self.device)
        check(self.lib.cn_absmax_f32(self.h, _ptr(a), a.numel(), _ptr(out), self.stream_ptr()))
        return out

    def compress(self, a, precision, out=None):
        out = out if out is not None else torch.empty(a.shape, dtype=torch.uint8, device=self.device)
        if isinstance(precision, torch.Tensor):
            check(self.lib.cn_compress_8bit_dp(self.h, _ptr(a), _ptr(precision), a.numel(), _ptr(out), self.stream_ptr()))
        else:
            check(self.lib.cn_compress_8bit(self.h, _ptr(a), float(precision), a.numel(), _ptr(out), self.stream_ptr()))
        return out

    def absmax_compress(self, a, scale=None, out=None):
        """scale = max |a|; codes = compress(a, scale) in one launch; returns (codes, scale tensor)."""
        out = out if out is not None else torch.empty(a.shape, dtype=torch.uint8, device=self.device)
        scale = scale if scale is not None else torch.empty(1, dtype=torch.float32, device=self.device)
        check(self.lib.cn_absmax_compress_8bit(self.h, _ptr(a), a.numel(), _ptr(scale), _ptr(out), self.stream_ptr()))
        return out, scale

    def decompress(self, codes, precision, out=None):
        out = out if out is not None else torch.empty(codes.shape, dtype=torch.float32, device=self.device)
        if isinstance(precision, torch.Tensor):
            check(self.lib.cn_decompress_8bit_dp(self.h, _ptr(codes), _ptr(precision), codes.numel(), _ptr(out), self.stream_ptr()))
        else:
            check(self.lib.cn_decompress_8bit(self.h, _ptr(codes), float(precision), codes.numel(), _ptr(out), self.stream_ptr()))
        return out

    # ------------------------------------------------------------------ GEMM
    def gemm(self, A, B, out=None, transA=False, transB=False, bias=None, activation=_lib.ACT_LINEAR, maxout_level=0,
             argmax_out=None, mode=_lib.GEMM_3XTF32):
        """C = act(op(A).op(B) + bias); A, B, C are column-major device matrices (tensor shape (cols, rows))."""
        a_cols, a_rows = A.shape
        b_cols, b_rows = B.shape
        M, K = (a_cols, a_rows) if transA else (a_rows, a_cols)
        K2, N = (b_cols, b_rows) if transB else (b_rows, b_cols)
        if K != K2:
            raise _lib.CnError(_lib.CN_ERR_SHAPE, f"inner dimensions differ: {K} vs {K2}")
        L = maxout_level if maxout_level and maxout_level > 1 else 1
        if out is None:
            out = self.empty(M, N // L)
        epi = Epilogue(_ptr(bias), int(activation), int(maxout_level), _ptr(argmax_out))
        check(self.lib.cn_gemm_f32(self.h, int(transA), int(transB), M, N, K, _ptr(A), a_rows, _ptr(B), b_rows, _ptr(out), M,
                                   ctypes.byref(epi), int(mode), self.stream_ptr()))
        return out

    def gemm_check(self):
        check(self.lib.cn_gemm_check_status(self.h, self.stream_ptr()))

    def gemm_last_path(self):
        return self.lib.cn_gemm_last_path(self.h).decode()

    def bias_activation(self, A, bias, activation, out=None):
        cols, rows = A.shape
        out = out if out is not None else torch.empty_like(A)
        check(self.lib.cn_bias_activation(self.h, _ptr(A), _ptr(bias), int(activation), _ptr(out), rows, cols, self.stream_ptr()))
        return out

    def maxout(self, A, level):
        cols, rows = A.shape
        out = self.empty(rows, cols // level)
        arg = self.empty(rows, cols // level)
        check(self.lib.cn_maxout(self.h, _ptr(A), _ptr(out), _ptr(arg), rows, cols, int(level), self.stream_ptr()))
        return out, arg

    # ------------------------------------------------------------------ random numbers / weights
    def rand(self, rows, cols, seed, offset=0):
        out = self.empty(rows, cols)
        check(self.lib.cn_rand_uniform(self.h, _ptr(out), out.numel(), seed, offset, self.stream_ptr()))
        return out

    def randn(self, rows, cols, seed, mean=0.0, std=1.0, offset=0):
        out = self.empty(rows, cols)
        check(self.lib.cn_rand_normal(self.h, _ptr(out), out.numel(), mean, std, seed, offset, self.stream_ptr()))
        return out

    def uniform_sqrt_weight(self, rows, cols, seed, fan_out_total=None, offset=0):
        out = self.empty(rows, cols)
        check(self.lib.cn_uniform_sqrt_weight(self.h, _ptr(out), out.numel(), rows, fan_out_total or cols, seed, offset,
                                              self.stream_ptr()))
        return out

    def dropout(self, A, rate, seed, offset=0):
        out = torch.empty_like(A)
        check(self.lib.cn_dropout(self.h, _ptr(A), _ptr(out), A.numel(), float(rate), seed, offset, self.stream_ptr()))
        return out

    # ------------------------------------------------------------------ communicator
    def comm_init(self, unique_id, rank, nranks):
        buf = (ctypes.c_char * 128).from_buffer_copy(unique_id)
        check(self.lib.cn_comm_init_rank(self.h, buf, rank, nranks))

    def unique_id(self):
        buf = (ctypes.c_char * 128)()
        check(self.lib.cn_comm_get_unique_id(buf))
        return bytes(buf)

    def shard_cols(self, n_total, rank, nranks):
        a, b = ctypes.c_int64(), ctypes.c_int64()
        check(self.lib.cn_shard_cols(n_total, rank, nranks, ctypes.byref(a), ctypes.byref(b)))
        return a.value, b.value

    def sym_empty(self, rows, cols):
        """Column-major rows x cols matrix in a symmetric buffer (collective call; see cn_sym_alloc)."""
        p = ctypes.c_void_p()
        nbytes = rows * cols * 4
        check(self.lib.cn_sym_alloc(self.h, nbytes, ctypes.byref(p)))

        class _Raw:
            __cuda_array_interface__ = {"shape": (cols, rows), "typestr": "<f4", "data": (p.value, False), "version": 2, "strides": None}
        t = torch.as_tensor(_Raw(), device=self.device)
        self._sym = getattr(self, "_sym", [])
        self._sym.append(p)
        return t

    def sym_free_all(self):
        for p in getattr(self, "_sym", []):
            self.lib.cn_sym_free(self.h, p)
        self._sym = []

    def bcast(self, t, root=0):
        check(self.lib.cn_bcast_f32(self.h, _ptr(t), t.numel(), root, self.stream_ptr()))
        return t

    def dotmpi(self, A, Wshard, n_total, out=None, bias=None, activation=_lib.ACT_LINEAR, mode=_lib.GEMM_3XTF32, exchange=0):
        K, M = A.shape
        out = out if out is not None else self.empty(M, n_total)
        epi = Epilogue(_ptr(bias), int(activation), 0, None)
        check(self.lib.cn_dotmpi_f32(self.h, M, K, n_total, _ptr(A), _ptr(Wshard), _ptr(out), ctypes.byref(epi), int(mode),
                                     int(exchange), self.stream_ptr()))
        return out

    def dotmpi_to_coded(self, A, Wshard, n_total, bias=None, activation=_lib.ACT_LINEAR, mode=_lib.GEMM_3XTF32, rank=0, nranks=1):
        """Sharded product whose gathered output stays 8-bit coded; returns (Coded struct, the tensors that back it)."""
        K, M = A.shape
        _, cnt = self.shard_cols(n_total, rank, nranks)
        codes = torch.empty((n_total, M), dtype=torch.uint8, device=self.device)
        scales = torch.zeros(max(nranks, 1), dtype=torch.float32, device=self.device)
        own = torch.empty((cnt, M), dtype=torch.float32, device=self.device)
        c = _lib.Coded(_ptr(codes), _ptr(scales), _ptr(own), M, n_total)
        epi = Epilogue(_ptr(bias), int(activation), 0, None)
        check(self.lib.cn_dotmpi_to_coded_f32(self.h, M, K, n_total, _ptr(A), _ptr(Wshard), ctypes.byref(c), ctypes.byref(epi), int(mode),
                                              self.stream_ptr()))
        return c, (codes, scales, own)

    def dotmpi_from_coded(self, coded, Wshard, n_total, out=None, bias=None, activation=_lib.ACT_LINEAR, mode=_lib.GEMM_3XTF32, exchange=0):
        out = out if out is not None else self.empty(coded.rows, n_total)
        epi = Epilogue(_ptr(bias), int(activation), 0, None)
        check(self.lib.cn_dotmpi_from_coded_f32(self.h, ctypes.byref(coded), n_total, _ptr(Wshard), _ptr(out), ctypes.byref(epi), int(mode),
                                                int(exchange), self.stream_ptr()))
        return out

    def dottmpi(self, A, Bshard, out=None, mode=_lib.GEMM_3XTF32):
        """out (M x R) = A (M x n_total) . B^T with B column-sharded (this rank: R x cols_local)."""
        n_total, M = A.shape
        _, R = Bshard.shape
        out = out if out is not None else self.empty(M, R)
        check(self.lib.cn_dottmpi_f32(self.h, M, n_total, R, _ptr(A), _ptr(Bshard), _ptr(out), int(mode), self.stream_ptr()))
        return out

    def dot_sharded_out(self, A, B, out_shard, transA=False, mode=_lib.GEMM_3XTF32):
        """out_shard (M x cols_local) = op(A) . B[:, shard]."""
        a_cols, a_rows = A.shape
        M, K = (a_cols, a_rows) if transA else (a_rows, a_cols)
        n_total = B.shape[0]
        check(self.lib.cn_dot_sharded_out_f32(self.h, int(transA), M, K, n_total, _ptr(A), _ptr(B), _ptr(out_shard), int(mode),
                                              self.stream_ptr()))
        return out_shard

    # ------------------------------------------------------------------ timers
    def tick(self, name="default"):
        check(self.lib.cn_tick(self.h, name.encode(), self.stream_ptr()))

    def tock(self, name="default"):
        ms = ctypes.c_float()
        check(self.lib.cn_tock(self.h, name.encode(), self.stream_ptr(), ctypes.byref(ms)))
        return ms.value
