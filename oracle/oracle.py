"""TEST INFRASTRUCTURE — numpy / ctypes front of the CPU oracle.

Only tests/, __graft_entry__.smoke() and the CPU-baseline / reference legs of bench.py import this module; the
product never does.  The codec functions call the C restatement in oracle/codec_oracle.c; the rest restates,
in numpy, the reference semantics at the boundary of the hot path:

  gemm_f64           fp64 host GEMM, the accuracy yardstick for ClusterNet::dot (source/clusterNet.cpp:404-487)
  bias_activation    kAddMatrixVector + activation kernels (source/clusterKernels.cu:706-718,803-811,382-390,823-844)
  maxout             kMaxout + reduceToMaxAndArgMax, same comparison tree (source/clusterKernels.cu:1432-1458,563-604)
  shard_cols         column split of dotMPI / distributed weights (source/clusterNet.cpp:515-516,926-931)
  sqrt_weight_limit  kCreateRdmSqrtWeight_Logistic's bound (source/clusterKernels.cu:126-138)
  BatchOracle        BatchAllocator's dense batching (source/batchAllocator.cpp:101-139,399-425,977-1053)
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(HERE, "_build", "liboracle.so")
        if not os.path.exists(path):
            subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
        L = ctypes.CDLL(path)
        L.oracle_absmax.restype = ctypes.c_float
        L.oracle_count_undefined_band.restype = ctypes.c_int64
        L.oracle_sweep_thresholds.restype = ctypes.c_int64
        L.oracle_code_of_magnitude.restype = ctypes.c_ubyte
        L.oracle_code_of_magnitude.argtypes = [ctypes.c_void_p, ctypes.c_float]
        _LIB = L
    return _LIB


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def load_codebook(path):
    tbl = np.zeros(126, np.float32)
    rc = lib().oracle_load_codebook(path.encode(), _p(tbl))
    if rc != 0:
        raise RuntimeError(f"oracle_load_codebook({path}) = {rc}")
    return tbl


def compress(tbl, x, precision, threads=False):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    fn = lib().oracle_compress_8bit_mt if threads else lib().oracle_compress_8bit
    fn(_p(tbl), _p(x), ctypes.c_float(precision), ctypes.c_int64(x.size), _p(out))
    return out


def decompress(tbl, codes, precision, threads=False):
    codes = np.ascontiguousarray(codes, np.uint8)
    out = np.empty(codes.shape, np.float32)
    fn = lib().oracle_decompress_8bit_mt if threads else lib().oracle_decompress_8bit
    fn(_p(tbl), _p(codes), ctypes.c_float(precision), ctypes.c_int64(codes.size), _p(out))
    return out


def absmax(x):
    x = np.ascontiguousarray(x, np.float32)
    return float(lib().oracle_absmax(_p(x), ctypes.c_int64(x.size)))


def undefined_band_mask(tbl, x, precision):
    x = np.ascontiguousarray(x, np.float32)
    mask = np.zeros(x.shape, np.uint8)
    lib().oracle_count_undefined_band(_p(tbl), _p(x), ctypes.c_float(precision), ctypes.c_int64(x.size), _p(mask))
    return mask.astype(bool)


def sweep_thresholds(tbl, thr, level_codes, lo_bits=0, hi_bits=0x7F800000):
    """Exhaustive check of a threshold table against the restated kernel; returns (mismatches, first bad bits)."""
    thr = np.ascontiguousarray(thr, np.uint32)
    level_codes = np.ascontiguousarray(level_codes, np.uint8)
    fb = ctypes.c_uint32()
    bad = lib().oracle_sweep_thresholds(_p(tbl), _p(thr), ctypes.c_int(thr.size), _p(level_codes), ctypes.c_uint32(lo_bits),
                                        ctypes.c_uint32(hi_bits), ctypes.byref(fb))
    return int(bad), fb.value


# ---------------------------------------------------------------------------------------------- GEMM and epilogue
def gemm_f64(A, B, transA=False, transB=False):
    a = A.astype(np.float64)
    b = B.astype(np.float64)
    return (a.T if transA else a) @ (b.T if transB else b)


def bias_activation(C, bias=None, activation=0):
    c = np.array(C, np.float32, copy=True)
    if bias is not None:
        c = (c + np.asarray(bias, np.float32)[None, :]).astype(np.float32)
    if activation == 1:
        c = np.where(c > 0, c, np.float32(0)).astype(np.float32)
    elif activation == 2:
        with np.errstate(over="ignore"):
            c = (1.0 / (1.0 + np.exp(-c).astype(np.float32).astype(np.float64))).astype(np.float32)
    elif activation == 3:
        c = np.minimum(np.where(c > 0, c, np.float32(0)), np.float32(1)).astype(np.float32)
    return c


def maxout(C, level):
    """Value and absolute argmax column (as float) over groups of `level` consecutive columns."""
    rows, cols = C.shape
    assert cols % level == 0 and level <= 32
    g = cols // level
    vals = np.full((rows, g, 32), -np.finfo(np.float32).max, np.float32)
    idx = np.full((rows, g, 32), -1.0, np.float32)
    vals[:, :, :level] = C.reshape(rows, g, level)
    idx[:, :, :level] = (np.arange(g)[:, None] * level + np.arange(level)[None, :]).astype(np.float32)[None]
    off = 16
    while off > 0:
        take = vals[:, :, :off] < vals[:, :, off:2 * off]
        vals[:, :, :off] = np.where(take, vals[:, :, off:2 * off], vals[:, :, :off])
        idx[:, :, :off] = np.where(take, idx[:, :, off:2 * off], idx[:, :, :off])
        off >>= 1
    return vals[:, :, 0].copy(), idx[:, :, 0].copy()


def shard_cols(n_total, rank, nranks):
    split = n_total // nranks
    return split * rank, (n_total - split * (nranks - 1)) if rank == nranks - 1 else split


def sqrt_weight_limit(fan_in, fan_out_total):
    return np.float32(4.0) * np.sqrt(np.float32(6.0) / (np.float32(fan_in) + np.float32(fan_out_total)), dtype=np.float32)


class BatchOracle:
    """Row ranges the reference's dense BatchAllocator serves, batch after batch, over epochs."""

    def __init__(self, rows, batch_size, skip_last_batch=False):
        self.rows, self.batch, self.skip = rows, batch_size, skip_last_batch
        self.total = -(-rows // batch_size)
        self.next = 1            # init leaves batch 0 current and the counter at 1
        self.current = (0, batch_size)

    def rows_of(self, idx):
        return self.rows % self.batch if self.batch * (idx + 1) > self.rows else self.batch

    def advance(self):
        idx = self.next
        self.current = (idx * self.batch, self.rows_of(idx))
        self.next += 1
        if self.next + 1 == self.total and self.skip:
            self.next = 0
        if self.next >= self.total:
            self.next = 0
        return self.current


# ---------------------------------------------------------------------------------------------- training step
def softmax_rows(A):
    """kSoftMax (source/clusterKernels.cu:651-688): per row, subtract the maximum, exponentiate, divide by the sum."""
    a = A.astype(np.float32)
    e = np.exp((a - a.max(axis=1, keepdims=True)).astype(np.float32)).astype(np.float32)
    return (e / e.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)


def t_matrix(labels, classes):
    """kCreate_t_matrix (source/clusterKernels.cu:775-790): one-hot rows from float labels."""
    out = np.zeros((labels.size, classes), np.float32)
    out[np.arange(labels.size), labels.astype(np.int64).ravel()] = 1.0
    return out


def rmsprop_update(rms, grad, w, rms_mult, lr):
    """kRMSprop_with_weight_update (source/clusterKernels.cu:1306-1325) in fp32."""
    rms, grad, w = rms.astype(np.float32), grad.astype(np.float32), w.astype(np.float32)
    r = (np.float32(rms_mult) * rms + (grad * grad) * np.float32(1.0 - rms_mult)).astype(np.float32)
    return r, (w - np.float32(lr) * (grad / (np.sqrt(r) + np.float32(1.0e-08)))).astype(np.float32)


def nesterov_update(grad, w, m, lr, batch_size, momentum):
    """kNesterov_weight_update (source/clusterKernels.cu:1064-1077) in fp32: returns the new (w, m)."""
    grad, w, m = grad.astype(np.float32), w.astype(np.float32), m.astype(np.float32)
    g = (np.float32(lr) * (grad / np.float32(batch_size))).astype(np.float32)
    return (w - g).astype(np.float32), (np.float32(momentum) * m - g).astype(np.float32)


def max_seeded(a):
    """max (source/basicOps.cu:1076-1081): a maximum reduction seeded with -1.0f."""
    a = np.asarray(a, np.float32).ravel()
    return np.float32(max(np.float32(-1.0), a.max())) if a.size else np.float32(-1.0)


def mlp_step_gradients(X, y, weights, dropout=0.0):
    """Forward / backward of the reference's Layer chain (source/Layer.cpp:250-261,314-339) for ReLU hidden layers and a
    softmax output, biases zero, dropout rate 0 (activations pass unchanged): returns the softmax output and the weight
    gradients Tdot(activation_l, error_{l+1}) of every layer, computed in float64."""
    acts = [X.astype(np.float64)]
    for W in weights[:-1]:
        acts.append(np.maximum(acts[-1] @ W.astype(np.float64), 0.0))
    z = acts[-1] @ weights[-1].astype(np.float64)
    e = np.exp(z - z.max(axis=1, keepdims=True))
    probs = e / e.sum(axis=1, keepdims=True)
    err = probs - t_matrix(y, z.shape[1])
    grads = [None] * len(weights)
    for l in range(len(weights) - 1, -1, -1):
        grads[l] = acts[l].T @ err
        if l > 0:
            err = (err @ weights[l].astype(np.float64).T) * (acts[l] > 0)
    return probs, grads
