"""ctypes binding of libendia_b200.so (the C ABI declared in include/endia_b200.h).

There is no CPU fallback: importing this module without the built library raises, and every
compute call on a machine without an sm_100 device raises EndiaError.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libendia_b200.so")

MAX_DIMS = 8


class EndiaError(RuntimeError):
    """Raised for a non-zero status of the device library (Endia ops `raise "string"`)."""

    def __init__(self, status, message):
        super().__init__("endia_b200 status %d: %s" % (status, message))
        self.status = status


class Tensor(C.Structure):
    """Mirror of `endia_b200_tensor`."""
    _fields_ = [
        ("data", C.c_void_p),
        ("shape", C.c_int64 * MAX_DIMS),
        ("stride", C.c_int64 * MAX_DIMS),
        ("offset", C.c_int64),
        ("ndim", C.c_int32),
        ("is_complex", C.c_int32),
    ]


class Epilogue(C.Structure):
    """Mirror of `endia_b200_epilogue`."""
    _fields_ = [
        ("alpha", C.c_float),
        ("beta", C.c_float),
        ("bias", C.c_void_p),
        ("act", C.c_int32),
        ("dact", C.c_int32),
        ("dact_src", C.c_void_p),
        ("ld_dact", C.c_int64),
        ("colsum", C.c_void_p),
        ("colsum_scratch", C.c_void_p),
        ("a_lo", C.c_void_p),
        ("b_lo", C.c_void_p),
        ("a16", C.c_void_p),
        ("b16", C.c_void_p),
        ("c16", C.c_void_p),
    ]


class FftFusion(C.Structure):
    """Mirror of `endia_b200_fft_fusion`."""
    _fields_ = [
        ("scale_dev", C.c_void_p),
        ("reduce", C.c_int32),
        ("reduce_w", C.c_void_p),
        ("reduce_out", C.c_void_p),
        ("reduce_scale", C.c_float),
        ("reduce_scratch", C.c_void_p),
    ]


# status codes
OK, EINVAL, ECUDA, ENODEV, ENOMEM, ESHAPE, EPOW2, ETIMEOUT, ELIMIT = 0, -1, -2, -3, -4, -5, -6, -7, -8
ACT_NONE, ACT_RELU, ACT_TANH, ACT_SIGMOID = 0, 1, 2, 3
GEMM_AUTO, GEMM_FFMA, GEMM_3XTF32, GEMM_TF32_BF16X2 = 0, 1, 2, 3
(UN_COPY, UN_NEG, UN_RELU, UN_TANH, UN_SIGMOID, UN_SQUARE, UN_SQRT, UN_ABS, UN_SIGN, UN_CONJ,
 UN_EXP, UN_LOG, UN_SIN, UN_COS, UN_RECIPROCAL, UN_SINH, UN_COSH, UN_TAN, UN_ASIN, UN_ACOS,
 UN_ATAN) = range(21)
(BIN_ADD, BIN_SUB, BIN_MUL, BIN_DIV, BIN_POW, BIN_GREATER, BIN_RELU_BWD, BIN_TANH_BWD,
 BIN_SIGMOID_BWD, BIN_COMPLEX, BIN_ABS_BWD, BIN_SQUARE_BWD, BIN_GREATER_EQUAL, BIN_LESS,
 BIN_LESS_EQUAL, BIN_EQUAL, BIN_NOT_EQUAL, BIN_TANH_OUT_BWD, BIN_TANH_OUT_BWD2) = range(19)

_vp, _i64, _i32, _f32, _sz = C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_size_t
_TP = C.POINTER(Tensor)

# name -> (restype, argtypes); every symbol the header declares.
SIGNATURES = {
    "endia_b200_init": (C.c_int, [C.c_int]),
    "endia_b200_shutdown": (C.c_int, []),
    "endia_b200_last_error": (C.c_char_p, []),
    "endia_b200_version": (C.c_int, []),
    "endia_b200_has_tcgen05": (C.c_int, []),
    "endia_b200_launch_count": (C.c_uint64, []),
    "endia_b200_device_status": (C.c_int, [_vp]),
    "endia_b200_selftest_wait_timeout": (C.c_int, [_i32, _vp]),
    "endia_b200_malloc": (C.c_int, [C.POINTER(_vp), _sz, _vp]),
    "endia_b200_set_malloc_quota": (C.c_int, [_sz]),
    "endia_b200_free": (C.c_int, [_vp, _vp]),
    "endia_b200_memset0": (C.c_int, [_vp, _sz, _vp]),
    "endia_b200_h2d": (C.c_int, [_vp, _vp, _sz, _vp]),
    "endia_b200_d2h": (C.c_int, [_vp, _vp, _sz, _vp]),
    "endia_b200_d2d": (C.c_int, [_vp, _vp, _sz, _vp]),
    "endia_b200_stream_create": (C.c_int, [C.POINTER(_vp)]),
    "endia_b200_stream_destroy": (C.c_int, [_vp]),
    "endia_b200_stream_sync": (C.c_int, [_vp]),
    "endia_b200_event_create": (C.c_int, [C.POINTER(_vp)]),
    "endia_b200_event_destroy": (C.c_int, [_vp]),
    "endia_b200_event_record": (C.c_int, [_vp, _vp]),
    "endia_b200_stream_wait_event": (C.c_int, [_vp, _vp]),
    "endia_b200_event_elapsed_ms": (C.c_int, [_vp, _vp, C.POINTER(_f32)]),
    "endia_b200_gemm_colsum_scratch_bytes": (_sz, [_i64, _i64]),
    "endia_b200_gemm": (C.c_int, [C.c_int, C.c_int, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp,
                                  _i64, _i64, _i64, _i64, _i64, C.POINTER(Epilogue), C.c_int, _vp]),
    "endia_b200_tf32_split": (C.c_int, [_vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "endia_b200_gemm_complex": (C.c_int, [C.c_int, C.c_int, _i64, _i64, _i64, _vp, _i64, _vp, _i64,
                                          _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "endia_b200_ew_unary": (C.c_int, [C.c_int, _TP, _TP, _vp]),
    "endia_b200_ew_binary": (C.c_int, [C.c_int, _TP, _TP, _TP, _vp]),
    "endia_b200_fill": (C.c_int, [_vp, _i64, C.c_int, _f32, _f32, _vp]),
    "endia_b200_eye": (C.c_int, [_vp, _i64, _vp]),
    "endia_b200_reduce_scratch_bytes": (_sz, [_TP, C.c_uint32]),
    "endia_b200_reduce_add": (C.c_int, [_TP, C.c_uint32, _vp, _vp, _vp]),
    "endia_b200_reduce_mul": (C.c_int, [_TP, C.c_uint32, _vp, _vp, _vp]),
    "endia_b200_mse_scratch_bytes": (_sz, [_i64]),
    "endia_b200_mse_fwd_bwd": (C.c_int, [_vp, _vp, _i64, _f32, _vp, _vp, _vp, _vp]),
    "endia_b200_mse_fwd_bwd_noalloc": (C.c_int, [_vp, _vp, _i64, _f32, _vp, _vp, _vp]),
    "endia_b200_act_bwd_colsum_scratch_bytes": (_sz, [_i64, _i64]),
    "endia_b200_act_bwd_colsum": (C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp]),
    "endia_b200_act_bwd_colsum_parts": (C.c_int, [C.c_int, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "endia_b200_adam_step_multi": (C.c_int, [_i32, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                             C.POINTER(_vp), C.POINTER(_i64), _f32, _f32, _f32,
                                             _f32, _f32, _f32, _vp]),
    "endia_b200_adam_step_multi_lo": (C.c_int, [_i32, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                                C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i64), _f32, _f32,
                                                _f32, _f32, _f32, _f32, _vp]),
    "endia_b200_adam_step_multi_bf16": (C.c_int, [_i32, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                                  C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i64), _f32, _f32,
                                                  _f32, _f32, _f32, _f32, _vp]),
    "endia_b200_adam_step_multi_graph": (C.c_int, [_i32, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                                   C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i64), _f32, _f32,
                                                   _f32, _f32, _vp, _i32, _f32, _vp]),
    "endia_b200_bf16_split": (C.c_int, [_vp, _vp, _i64, _vp]),
    "endia_b200_mlp_small_step": (C.c_int, [_i32, C.POINTER(_i32), _i32, _i32, _vp, _vp] + [C.POINTER(_vp)] * 8 +
                                  [_vp, _i32, _f32, _f32, _f32, _f32, _f32, _vp]),
    "endia_b200_fft_scratch_bytes": (_sz, [_TP, C.POINTER(_i32), _i32]),
    "endia_b200_fft_c2c": (C.c_int, [_TP, _TP, C.POINTER(_i32), _i32, C.c_int, _f32, _vp, _vp]),
    "endia_b200_fft_fusion_scratch_bytes": (_sz, []),
    "endia_b200_fft_c2c_fused": (C.c_int, [_TP, _TP, C.POINTER(_i32), _i32, C.c_int, _f32, _vp,
                                           C.POINTER(FftFusion), _vp]),
    "endia_b200_fft_loss_term": (C.c_int, [_TP, C.c_int, _vp, _vp, _f32, _vp, _vp]),
    "endia_b200_sgd_step_multi": (C.c_int, [_i32, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                            C.POINTER(_i64), _f32, _f32, _f32, _f32, _vp]),
    "endia_b200_rmsprop_step_multi": (C.c_int, [_i32, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                                C.POINTER(_i64), _f32, _f32, _f32, _f32, _vp]),
    "endia_b200_adagrad_step_multi": (C.c_int, [_i32, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                                C.POINTER(_i64), _f32, _f32, _f32, _vp]),
    "endia_b200_copy_strided": (C.c_int, [_TP, _TP, _vp]),
    "endia_b200_gather_slices": (C.c_int, [_vp, _vp, _i64, _i32, _i32, _vp, _vp]),
    "endia_b200_ipc_alloc": (C.c_int, [_sz, C.POINTER(_vp), _vp]),
    "endia_b200_ipc_open": (C.c_int, [_vp, C.POINTER(_vp)]),
    "endia_b200_ipc_close": (C.c_int, [_vp]),
    "endia_b200_ipc_free": (C.c_int, [_vp]),
    "endia_b200_comm_unique_id": (C.c_int, [_vp]),
    "endia_b200_comm_init": (C.c_int, [_i32, _i32, _vp, C.POINTER(_vp)]),
    "endia_b200_comm_destroy": (C.c_int, [_vp]),
    "endia_b200_allreduce_sum_f32": (C.c_int, [_vp, _vp, _vp, _i64, _vp]),
    "endia_b200_alltoall_bytes": (C.c_int, [_vp, _vp, _vp, _i64, _vp]),
}


def _load():
    # Rebuild when the sources changed and a compiler is at hand; a box without nvcc uses the
    # library that travelled with the tree.
    if os.environ.get("ENDIA_B200_NO_AUTOBUILD") != "1":
        import shutil
        if os.path.exists("/usr/local/cuda/bin/nvcc") or shutil.which("nvcc"):
            from . import build as _build
            _build.build()
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "endia_b200: %s is missing. Build it with `python -m endia_b200.build` "
            "(nvcc, sm_100a); there is no CPU fallback." % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(status):
    """Turn a non-zero status into an EndiaError carrying the library's message."""
    if status != 0:
        raise EndiaError(status, lib.endia_b200_last_error().decode(errors="replace"))


def call(name, *args):
    check(getattr(lib, name)(*args))
