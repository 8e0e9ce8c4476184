"""ctypes binding of libmixedgemm_b200.so (the C ABI declared in include/mixedgemm_c.h).

The library is the product path: there is no Python or CPU fallback.  If the shared
library is missing, importing this module raises with the build command.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libmixedgemm_b200.so")

MG_OK = 0
STATUS_NAMES = {0: "MG_OK", 1: "MG_ERR_SHAPE", 2: "MG_ERR_NULL", 3: "MG_ERR_ALIGN", 4: "MG_ERR_WORKSPACE",
                5: "MG_ERR_CUDA", 6: "MG_ERR_DEVICE", 7: "MG_ERR_TIMEOUT", 8: "MG_ERR_NCCL"}

# every symbol include/*.h declares, with its prototype
_vp, _i, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
PROTOTYPES = {
    "mg_strerror": (ctypes.c_char_p, [_i]),
    "mg_last_cuda_error": (_i, []),
    "mg_version": (_i, []),
    "mg_device_status": (_i, [ctypes.POINTER(_i), _vp]),
    "mg_set_wait_limit_us": (_i, [ctypes.c_longlong]),
    "mg_set_option": (_i, [ctypes.c_char_p, _i]),
    "mg_get_option": (_i, [ctypes.c_char_p, ctypes.POINTER(_i)]),
    "mg_reset_options": (None, []),
    "mg_matmul_multi": (_i, [_i, _vp, _vp]),
    "mg_pair_schedule": (_i, [_i, _vp, _vp, _i, ctypes.POINTER(_i), _vp, _vp]),
    "mg_reorder_quantize_multi": (_i, [_i, _i, _vp, _vp]),
    "mg_push_block": (_i, [_i, _i, _vp, _sz, _sz, _sz, _vp, _vp, _i, _vp]),
    "mg_push_block_to": (_i, [_i, _i, ctypes.c_uint, _vp, _sz, _sz, _sz, _vp, _vp, _i, _vp]),
    "mg_push_shard_to": (_i, [_i, _i, ctypes.c_uint, _vp, _vp, _vp, _i, _sz, _vp, _vp]),
    "mg_dist_unique_id": (_i, [_vp]),
    "mg_dist_init": (_i, [ctypes.POINTER(_vp), _vp, _i, _i]),
    "mg_dist_destroy": (_i, [_vp]),
    "mg_bcast_activations": (_i, [_vp, _i, _vp, _vp, _i, _vp]),
    "mg_allgather_inplace": (_i, [_vp, _vp, _vp, _i, _vp]),
    "mg_allgather_output": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "mg_xbuf_alloc": (_i, [ctypes.POINTER(_vp), _sz]),
    "mg_xbuf_free": (_i, [_vp]),
    "mg_ipc_export": (_i, [_vp, _vp]),
    "mg_ipc_import": (_i, [_vp, ctypes.POINTER(_vp)]),
    "mg_ipc_close": (_i, [_vp]),
    "mg_epoch_bump": (_i, [_vp, _vp]),
    "mg_push_shard": (_i, [_i, _i, _vp, _vp, _vp, _i, _sz, _vp, _vp]),
    "mg_sf_bytes": (_sz, [_i, _i]),
    "mg_reorder_quantize_x": (_i, [_vp, _i, _i, _vp, _i, _i, _i] + [_vp] * 6 + [_vp]),
    "mg_reorder_quantize_w": (_i, [_vp, _i, _i, _vp, _i, _i, _i] + [_vp] * 6 + [_vp]),
    "mg_matmul_workspace_bytes": (_sz, [_i] * 5),
    "mg_matmul": (_i, [_vp] * 6 + [_i] * 5 + [_vp, _vp, _i] + [_vp] * 6 + [_vp, _sz, _vp]),
    "mg_code_pitch": (_sz, [_i, _i, _i]),
    "mg_reorder_quantize_pitched": (_i, [_i, _vp, _i, _i, _vp, _i, _i, _i] + [_vp] * 3 + [_vp] + [_vp] * 3 + [_vp]),
    "mg_matmul_pitched_workspace_bytes": (_sz, [_i] * 5 + [_vp]),
    "mg_matmul_pitched": (_i, [_vp] * 6 + [_vp, _i] + [_i] * 5 + [_vp, _vp, _i] + [_vp] * 6 + [_vp, _sz, _vp]),
    "mg_reorder_index": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "mg_matmul_group_pitched": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp, _vp,
                                     _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "mg_matmul_f32": (_i, [_vp] * 6 + [_i] * 5 + [_vp, _vp, _i] + [_vp] * 6 + [_vp, _sz, _vp]),
    "mg_matmul_static_ws": (_i, [_vp] * 6 + [_i] * 5 + [_vp, _vp, _i] + [_vp] * 6 + [_vp]),
    "mg_matmul_fp4": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "mg_matmul_fp6": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "mg_matmul_fp8": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
}



class QuantProblem(ctypes.Structure):
    """mg_quant_problem_t of include/mixedgemm_c.h."""
    _fields_ = [("X", _vp), ("rows", _i), ("K", _i), ("idx", _vp), ("KN", _i), ("KS", _i), ("KO", _i),
                ("C4", _vp), ("C6", _vp), ("C8", _vp), ("pitch", _sz * 3), ("SF4", _vp), ("SF6", _vp), ("SF8", _vp)]


class Problem(ctypes.Structure):
    """mg_problem_t of include/mixedgemm_c.h."""
    _fields_ = ([(n, _vp) for n in ("AN", "AS", "AO", "SFAN", "SFAS", "SFAO")] + [("pitch_a", _sz * 3)] +
                [(n, _vp) for n in ("BN", "BS", "BO", "SFBN", "SFBS", "SFBO")] + [("pitch_b", _sz * 3)] +
                [(n, _i) for n in ("M", "N", "KN", "KS", "KO")] + [("D_bf16", _vp), ("ldd", _i),
                                                                  ("ready_flags", _vp), ("ready_count", _i),
                                                                  ("ready_epoch", _vp), ("ready_value", _i),
                                                                  ("ready_rows", _i), ("first_row", _i),
                                                                  ("a_shard_rows", _i), ("a_shard_stride", _sz * 3),
                                                                  ("sfa_shard_stride", _sz * 3)])


_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "libmixedgemm_b200.so is not built; run `python -m mixedgemm_b200.build` "
                "(nvcc for sm_100a).  There is no fallback path.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class MixedGemmError(RuntimeError):
    def __init__(self, status, where):
        lib = load()
        msg = lib.mg_strerror(status).decode()
        extra = ""
        if status == 5:
            extra = " (cudaError %d)" % lib.mg_last_cuda_error()
        super().__init__("%s: %s [%s]%s" % (where, msg, STATUS_NAMES.get(status, status), extra))
        self.status = status


def check(status, where):
    if status != MG_OK:
        raise MixedGemmError(status, where)
