"""ctypes binding of libclusternet_b200.so (the C ABI declared in include/clusternet_b200.h).

The library is the product: there is no Python or CPU fallback.  `load()` raises when the shared
object is missing or does not export a symbol the header declares.
"""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libclusternet_b200.so")
HEADER_PATH = os.path.join(HERE, "..", "include", "clusternet_b200.h")

c_void_p, c_int, c_int64, c_float, c_char_p = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_char_p
c_uint64 = ctypes.c_uint64

CN_OK, CN_ERR_ARG, CN_ERR_SHAPE, CN_ERR_CUDA, CN_ERR_NCCL, CN_ERR_TIMEOUT, CN_ERR_UNSUPPORTED, CN_ERR_NOMEM = range(8)
GEMM_3XTF32, GEMM_TF32, GEMM_FP32_SIMT = 0, 1, 2
ACT_LINEAR, ACT_RELU, ACT_LOGISTIC, ACT_DOUBLE_RELU = 0, 1, 2, 3
BATCH_KEEP_ROW_MAJOR, BATCH_NO_COL_MAJOR, BATCH_SHARDED_UPLOAD, BATCH_PUSH_BY_KERNEL, BATCH_LOOKAHEAD = 1, 2, 4, 8, 16


class Coded(ctypes.Structure):
    _fields_ = [("codes", c_void_p), ("scales", c_void_p), ("own_fp32", c_void_p), ("rows", c_int64), ("cols", c_int64)]


class Epilogue(ctypes.Structure):
    _fields_ = [("bias", c_void_p), ("activation", c_int), ("maxout_level", c_int), ("argmax_out", c_void_p)]


_SIGNATURES = {
    "cn_last_error": (c_char_p, []),
    "cn_status_string": (c_char_p, [c_int]),
    "cn_version": (c_int, []),
    "cn_compiled_arch": (c_int, []),
    "cn_kernel_launches": (c_uint64, []),
    "cn_diag_wait_probe": (c_int, [c_void_p, c_int64, c_void_p]),
    "cn_gemm_profile_enable": (c_int, [c_void_p, c_int]),
    "cn_gemm_set_tuning": (c_int, [c_void_p, c_int, c_int, c_int]),
    "cn_gemm_profile_read": (c_int, [c_void_p, c_void_p, c_int, ctypes.POINTER(c_int)]),
    "cn_context_create": (c_int, [c_int, c_void_p, ctypes.POINTER(c_void_p)]),
    "cn_context_destroy": (c_int, [c_void_p]),
    "cn_context_device": (c_int, [c_void_p]),
    "cn_codebook_load": (c_int, [c_char_p, c_void_p]),
    "cn_hdf5_read_f32": (c_int, [c_char_p, c_char_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64), ctypes.POINTER(c_int64)]),
    "cn_hdf5_dims": (c_int, [c_char_p, c_char_p, ctypes.POINTER(c_int64), ctypes.POINTER(c_int64)]),
    "cn_hdf5_read_f32_into": (c_int, [c_char_p, c_char_p, c_void_p, c_int64]),
    "cn_hdf5_read_i32": (c_int, [c_char_p, c_char_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64), ctypes.POINTER(c_int64)]),
    "cn_host_free": (None, [c_void_p]),
    "cn_hdf5_write_f32": (c_int, [c_char_p, c_char_p, c_void_p, c_int64, c_int64]),
    "cn_codec_build_thresholds": (c_int, [c_void_p, c_void_p, c_void_p]),
    "cn_absmax_f32": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "cn_absmax_f32_noalloc": (c_int, [c_void_p, c_int64, c_void_p, c_void_p]),
    "cn_compress_8bit": (c_int, [c_void_p, c_void_p, c_float, c_int64, c_void_p, c_void_p]),
    "cn_compress_8bit_dp": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "cn_absmax_compress_8bit": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "cn_decompress_8bit": (c_int, [c_void_p, c_void_p, c_float, c_int64, c_void_p, c_void_p]),
    "cn_decompress_8bit_dp": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "cn_to_col_major": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_to_row_major": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_upload_row_major": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_download_row_major": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_fill_f32": (c_int, [c_void_p, c_void_p, c_int64, c_float, c_void_p]),
    "cn_arange_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "cn_gemm_f32": (c_int, [c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                            c_void_p, c_int64, ctypes.POINTER(Epilogue), c_int, c_void_p]),
    "cn_gemm_last_path": (c_char_p, [c_void_p]),
    "cn_gemm_check_status": (c_int, [c_void_p, c_void_p]),
    "cn_bias_activation": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_maxout": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "cn_rand_uniform": (c_int, [c_void_p, c_void_p, c_int64, c_uint64, c_uint64, c_void_p]),
    "cn_rand_normal": (c_int, [c_void_p, c_void_p, c_int64, c_float, c_float, c_uint64, c_uint64, c_void_p]),
    "cn_rand_int": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_uint64, c_uint64, c_void_p]),
    "cn_uniform_sqrt_weight": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_uint64, c_uint64, c_void_p]),
    "cn_dropout": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_float, c_uint64, c_uint64, c_void_p]),
    "cn_dropout_dp": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_float, c_void_p, c_uint64, c_void_p]),
    "cn_seed_advance": (c_int, [c_void_p, c_void_p, c_void_p]),
    "cn_comm_get_unique_id": (c_int, [c_void_p]),
    "cn_comm_init_rank": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "cn_comm_init_all": (c_int, [ctypes.POINTER(c_void_p), c_int]),
    "cn_group_start": (c_int, []),
    "cn_group_end": (c_int, []),
    "cn_context_make_current": (c_int, [c_void_p]),
    "cn_comm_sync": (c_int, [c_void_p, c_void_p, c_int]),
    "cn_comm_destroy": (c_int, [c_void_p]),
    "cn_comm_rank": (c_int, [c_void_p]),
    "cn_comm_size": (c_int, [c_void_p]),
    "cn_shard_cols": (c_int, [c_int64, c_int, c_int, ctypes.POINTER(c_int64), ctypes.POINTER(c_int64)]),
    "cn_bcast_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "cn_allgather_cols_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_allgather_cols_u8": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_allgather_scalar_f32": (c_int, [c_void_p, c_void_p, c_void_p]),
    "cn_allreduce_sum_f32": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "cn_sym_alloc": (c_int, [c_void_p, ctypes.c_size_t, ctypes.POINTER(c_void_p)]),
    "cn_sym_free": (c_int, [c_void_p, c_void_p]),
    "cn_dotmpi_f32": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, ctypes.POINTER(Epilogue),
                              c_int, c_int, c_void_p]),
    "cn_tdotmpi_f32": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p, ctypes.POINTER(Epilogue),
                               c_int, c_int, c_void_p]),
    "cn_dotmpi_to_coded_f32": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, ctypes.POINTER(Coded),
                                       ctypes.POINTER(Epilogue), c_int, c_void_p]),
    "cn_dotmpi_from_coded_f32": (c_int, [c_void_p, ctypes.POINTER(Coded), c_int64, c_void_p, c_void_p, ctypes.POINTER(Epilogue),
                                         c_int, c_int, c_void_p]),
    "cn_dottmpi_f32": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "cn_dot_sharded_out_f32": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "cn_softmax": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_create_t_matrix": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_add": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "cn_sub": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "cn_mul": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "cn_scalar_mul": (c_int, [c_void_p, c_void_p, c_float, c_void_p, c_int64, c_void_p]),
    "cn_div": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "cn_scalar_add": (c_int, [c_void_p, c_void_p, c_float, c_void_p, c_int64, c_void_p]),
    "cn_abs": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "cn_square": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "cn_max_f32": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "cn_nesterov_update": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int64, c_float, c_int64, c_void_p]),
    "cn_activation_gradient": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p]),
    "cn_mul_activation_gradient": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p]),
    "cn_softmax_error": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "cn_rmsprop_update": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_int64, c_void_p]),
    "cn_grad_sync_8bit": (c_int, [c_void_p, c_void_p, c_int64, c_float, c_void_p]),
    "cn_grad_sync_8bit_multi": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    "cn_comm_set_push_exchange": (c_int, [c_void_p, c_int]),
    "cn_grad_sync_8bit_rmsprop": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_float, c_float, c_void_p]),
    "cn_batch_create": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, ctypes.POINTER(c_void_p)]),
    "cn_batch_create_ex": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, ctypes.POINTER(c_void_p)]),
    "cn_batch_current_row_major": (c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64)]),
    "cn_batch_profile": (c_int, [c_void_p, c_int, c_void_p]),
    "cn_batch_next_row_major": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "cn_gemm_prepare_create": (c_int, [c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "cn_gemm_prepare": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p]),
    "cn_dotmpi_prepared_f32": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "cn_gemm_prepare_destroy": (c_int, [c_void_p]),
    "cn_batch_destroy": (c_int, [c_void_p]),
    "cn_batch_total_batches": (c_int64, [c_void_p]),
    "cn_batch_current": (c_int, [c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64)]),
    "cn_batch_set_skip_last": (c_int, [c_void_p, c_int]),
    "cn_batch_copy_next_async": (c_int, [c_void_p]),
    "cn_batch_swap": (c_int, [c_void_p, c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64)]),
    "cn_tick": (c_int, [c_void_p, c_char_p, c_void_p]),
    "cn_tock": (c_int, [c_void_p, c_char_p, c_void_p, ctypes.POINTER(c_float)]),
}

_lib = None


def declared_symbols():
    """Names of all functions declared in the public header."""
    text = open(HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cn_[a-z0-9_]+)\s*\(", text)))


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libclusternet_b200.so is missing: build it with `python -m clusternet_b200.build` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError here = the library does not match the header
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class CnError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"{message} [{status}]")
        self.status = status


def check(status):
    if status != CN_OK:
        lib = load()
        raise CnError(status, f"{lib.cn_status_string(status).decode()}: {lib.cn_last_error().decode()}")
