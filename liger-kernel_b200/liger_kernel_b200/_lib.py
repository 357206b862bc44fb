"""ctypes binding of libflce_b200.so (declared in include/flce_b200.h).

There is no fallback: if the shared library is missing, importing this module raises.
"""

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# LIGER_B200_LIB selects another build of the same library (e.g. the cycle-accounting build, `build.py --trace`)
LIB_PATH = os.environ.get("LIGER_B200_LIB") or os.path.join(_HERE, "libflce_b200.so")

FLCE_BF16, FLCE_FP16, FLCE_FP32 = 0, 1, 2
FLCE_MEAN, FLCE_SUM, FLCE_NONE = 0, 1, 2
PHASE_FORWARD, PHASE_BACKWARD, PHASE_FUSED, PHASE_BACKWARD_SPLIT = 0, 1, 2, 3
ROWSTAT_PLANES = 6
FLAG_ARGMAX = 1
# flce_status_t
FLCE_OK, FLCE_ERR_INVALID_ARGUMENT, FLCE_ERR_UNSUPPORTED, FLCE_ERR_WORKSPACE, FLCE_ERR_CUDA, FLCE_ERR_DEVICE_TIMEOUT = range(6)

EXPORTS = (
    "flce_b200_workspace_bytes",
    "flce_b200_count",
    "flce_b200_forward_stats",
    "flce_b200_forward_stats_static",
    "flce_b200_forward_finalize",
    "flce_b200_forward",
    "flce_b200_backward",
    "flce_b200_backward_plan",
    "flce_b200_forward_backward_plan",
    "flce_b200_forward_backward",
    "flce_b200_scale_gradient",
    "flce_b200_split_fp32",
    "flce_b200_compact_rows",
    "flce_b200_scatter_rows",
    "flce_b200_compact_rows_rmsnorm",
    "flce_b200_rmsnorm_partial_floats",
    "flce_b200_rmsnorm_scatter_backward",
    "flce_b200_ce_forward",
    "flce_b200_ce_backward",
    "flce_b200_ce_forward_backward",
    "flce_b200_ce_scale_gradient",
    "flce_b200_gemm",
    "flce_b200_gemm_accumulate",
    "flce_b200_selftest_wait_expiry",
    "flce_b200_scaled_ce_rows",
    "flce_b200_scaled_ce_grad",
    "flce_b200_jsd_rows",
    "flce_b200_sce_workspace_bytes",
    "flce_b200_sce_forward",
    "flce_b200_sce_backward",
    "flce_b200_check_device_status",
    "flce_b200_profile_enable",
    "flce_b200_profile_read",
    "flce_b200_kernel_launches",
    "flce_b200_set_option",
    "flce_b200_status_string",
    "flce_b200_last_error",
    "flce_b200_version",
)


class Problem(C.Structure):
    _fields_ = [
        ("n_rows", C.c_int64), ("hidden", C.c_int64), ("vocab", C.c_int64),
        ("vocab_total", C.c_int64), ("vocab_offset", C.c_int64),
        ("ld_x", C.c_int64), ("ld_w", C.c_int64),
        ("dtype", C.c_int32), ("reduction", C.c_int32),
        ("ignore_index", C.c_int64),
        ("label_smoothing", C.c_float), ("lse_square_scale", C.c_float), ("softcap", C.c_float),
        ("use_token_scaling", C.c_int32), ("flags", C.c_int32),
        ("x", C.c_void_p), ("w", C.c_void_p), ("target", C.c_void_p),
        ("bias", C.c_void_p), ("ce_weight", C.c_void_p), ("active_rows", C.c_void_p),
    ]


class ForwardOut(C.Structure):
    _fields_ = [
        ("lse", C.c_void_p), ("target_prob", C.c_void_p), ("loss_rows", C.c_void_p),
        ("z_loss_rows", C.c_void_p), ("correct_rows", C.c_void_p), ("predicted_tokens", C.c_void_p),
        ("scalars", C.c_void_p),
    ]


class BackwardArgs(C.Structure):
    _fields_ = [
        ("lse", C.c_void_p), ("target_prob", C.c_void_p), ("norm", C.c_void_p), ("grad_output", C.c_void_p),
        ("grad_output_per_row", C.c_int32), ("grad_dtype", C.c_int32),
        ("grad_input", C.c_void_p), ("grad_weight", C.c_void_p), ("grad_bias", C.c_void_p),
        ("slab_begin", C.c_int32), ("slab_end", C.c_int32),
        ("proj_x", C.c_void_p), ("proj_x_cols", C.c_int64), ("ld_proj_x", C.c_int64),
        ("proj_w", C.c_void_p), ("proj_w_cols", C.c_int64), ("ld_proj_w", C.c_int64),
        ("split_logit_grad", C.c_int32), ("lo_cols_x", C.c_int64), ("lo_cols_w", C.c_int64),
    ]


class CeProblem(C.Structure):
    _fields_ = [
        ("n_rows", C.c_int64), ("vocab", C.c_int64), ("ld", C.c_int64),
        ("dtype", C.c_int32), ("reduction", C.c_int32), ("ignore_index", C.c_int64),
        ("label_smoothing", C.c_float), ("lse_square_scale", C.c_float), ("softcap", C.c_float), ("flags", C.c_int32),
        ("logits", C.c_void_p), ("target", C.c_void_p), ("ce_weight", C.c_void_p),
    ]


class SceProblem(C.Structure):
    _fields_ = [
        ("n_rows", C.c_int64), ("hidden", C.c_int64), ("vocab", C.c_int64), ("ld_x", C.c_int64), ("ld_w", C.c_int64),
        ("dtype", C.c_int32), ("reserved", C.c_int32), ("ignore_index", C.c_int64),
        ("temperature", C.c_float), ("reserved2", C.c_float),
        ("x", C.c_void_p), ("w", C.c_void_p), ("target", C.c_void_p),
    ]


class FusedArgs(C.Structure):
    _fields_ = [
        ("out", C.POINTER(ForwardOut)), ("norm", C.c_void_p), ("grad_dtype", C.c_int32),
        ("grad_input", C.c_void_p), ("grad_weight", C.c_void_p), ("grad_bias", C.c_void_p),
        ("norm_given", C.c_int32), ("store_mode", C.c_int32),
        ("after_grad_weight", C.c_void_p), ("after_grad_weight_user", C.c_void_p), ("reserve_sms", C.c_int32),
        ("exchange_shift", C.c_void_p), ("exchange_rowstats", C.c_void_p), ("after_grad_input", C.c_void_p),
        ("exchange_user", C.c_void_p),
    ]


AFTER_GRAD_WEIGHT_FN = C.CFUNCTYPE(None, C.c_void_p)
EXCHANGE_SHIFT_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int64)
EXCHANGE_ROWSTATS_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64)
AFTER_GRAD_INPUT_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64)


STORE_AUTO, STORE_LOGITS, STORE_EXP = 0, 1, 2


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python liger-kernel_b200/build.py` "
            "(nvcc, sm_100a). This package has no CPU or PyTorch fallback."
        )
    lib = C.CDLL(LIB_PATH)
    P, A, F = C.POINTER(Problem), C.POINTER(BackwardArgs), C.POINTER(ForwardOut)
    vp, sz, i32, i64 = C.c_void_p, C.c_size_t, C.c_int32, C.c_int64
    lib.flce_b200_workspace_bytes.argtypes = [P, C.c_int, sz]
    lib.flce_b200_workspace_bytes.restype = sz
    lib.flce_b200_count.argtypes = [P, vp, vp]
    lib.flce_b200_forward_stats.argtypes = [P, vp, vp, sz, vp]
    lib.flce_b200_forward_stats_static.argtypes = [P, vp, vp]
    lib.flce_b200_forward_stats_static.restype = C.c_int
    lib.flce_b200_forward_finalize.argtypes = [P, vp, vp, F, vp]
    lib.flce_b200_forward.argtypes = [P, vp, vp, F, vp, sz, vp]
    lib.flce_b200_backward.argtypes = [P, A, vp, sz, sz, vp]
    lib.flce_b200_forward_backward.argtypes = [P, C.POINTER(FusedArgs), vp, sz, sz, vp]
    lib.flce_b200_forward_backward.restype = C.c_int
    lib.flce_b200_scale_gradient.argtypes = [vp, i64, i32, vp, vp]
    lib.flce_b200_scale_gradient.restype = C.c_int
    lib.flce_b200_split_fp32.argtypes = [vp, i64, i64, i64, vp, i64, i64, C.POINTER(C.c_int32), i32, i32, vp]
    lib.flce_b200_split_fp32.restype = C.c_int
    CP = C.POINTER(CeProblem)
    lib.flce_b200_ce_forward.argtypes = [CP, vp, vp, F, vp]
    lib.flce_b200_ce_forward.restype = C.c_int
    lib.flce_b200_ce_backward.argtypes = [CP, vp, vp, vp, i32, vp, i64, vp, vp]
    lib.flce_b200_ce_backward.restype = C.c_int
    lib.flce_b200_ce_forward_backward.argtypes = [CP, vp, vp, F, vp, i64, vp]
    lib.flce_b200_ce_forward_backward.restype = C.c_int
    lib.flce_b200_ce_scale_gradient.argtypes = [vp, i64, i64, i64, i32, vp, i32, vp]
    lib.flce_b200_ce_scale_gradient.restype = C.c_int
    lib.flce_b200_compact_rows.argtypes = [P, vp, vp, vp, vp, vp]
    lib.flce_b200_compact_rows.restype = C.c_int
    lib.flce_b200_scatter_rows.argtypes = [vp, i64, vp, vp, i64, vp, vp]
    lib.flce_b200_scatter_rows.restype = C.c_int
    f32 = C.c_float
    lib.flce_b200_compact_rows_rmsnorm.argtypes = [P, vp, f32, f32, i32, vp, vp, vp, vp, vp, vp]
    lib.flce_b200_compact_rows_rmsnorm.restype = C.c_int
    lib.flce_b200_rmsnorm_partial_floats.argtypes = [i64]
    lib.flce_b200_rmsnorm_partial_floats.restype = C.c_int64
    lib.flce_b200_rmsnorm_scatter_backward.argtypes = [vp, i64, vp, i64, i32, i64, i64, vp, vp, vp, vp, f32, i32, vp, i64, vp, vp, vp]
    lib.flce_b200_rmsnorm_scatter_backward.restype = C.c_int
    lib.flce_b200_backward_plan.argtypes = [P, sz, C.POINTER(C.c_int32), C.POINTER(C.c_int64)]
    lib.flce_b200_backward_plan.restype = C.c_int
    lib.flce_b200_forward_backward_plan.argtypes = [P, sz, C.POINTER(C.c_int32), C.POINTER(C.c_int64)]
    lib.flce_b200_forward_backward_plan.restype = C.c_int
    lib.flce_b200_gemm.argtypes = [vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, i32, i32, i32, vp]
    f32 = C.c_float
    lib.flce_b200_gemm_accumulate.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i32, i32, i32, i32, i32, vp]
    lib.flce_b200_gemm_accumulate.restype = C.c_int
    lib.flce_b200_scaled_ce_rows.argtypes = [vp, i64, i32, i64, i64, vp, i64, f32, vp, vp, vp, vp]
    lib.flce_b200_scaled_ce_rows.restype = C.c_int
    lib.flce_b200_scaled_ce_grad.argtypes = [vp, i64, i32, i64, i64, vp, i64, f32, vp, vp, vp, vp, vp]
    lib.flce_b200_scaled_ce_grad.restype = C.c_int
    lib.flce_b200_jsd_rows.argtypes = [vp, i64, vp, i64, i32, i64, i64, vp, i64, f32, f32, vp, f32, vp, vp]
    lib.flce_b200_jsd_rows.restype = C.c_int
    SP = C.POINTER(SceProblem)
    lib.flce_b200_sce_workspace_bytes.argtypes = [SP, C.c_int, sz]
    lib.flce_b200_sce_workspace_bytes.restype = sz
    lib.flce_b200_sce_forward.argtypes = [SP, vp, vp, vp, vp, sz, vp]
    lib.flce_b200_sce_forward.restype = C.c_int
    lib.flce_b200_sce_backward.argtypes = [SP, vp, vp, vp, vp, i32, vp, vp, vp, sz, sz, vp]
    lib.flce_b200_sce_backward.restype = C.c_int
    lib.flce_b200_check_device_status.argtypes = [vp]
    lib.flce_b200_selftest_wait_expiry.argtypes = [i64, vp, vp]
    lib.flce_b200_selftest_wait_expiry.restype = C.c_int
    lib.flce_b200_set_option.argtypes = [C.c_char_p, i64]
    lib.flce_b200_profile_enable.argtypes = [C.c_int]
    lib.flce_b200_profile_enable.restype = C.c_int
    lib.flce_b200_profile_read.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_int64), C.c_int]
    lib.flce_b200_profile_read.restype = C.c_int
    lib.flce_b200_kernel_launches.argtypes = []
    lib.flce_b200_kernel_launches.restype = C.c_int64
    for name in ("flce_b200_count", "flce_b200_forward_stats", "flce_b200_forward_finalize", "flce_b200_forward",
                 "flce_b200_backward", "flce_b200_gemm", "flce_b200_check_device_status", "flce_b200_set_option"):
        getattr(lib, name).restype = C.c_int
    for name in ("flce_b200_status_string", "flce_b200_last_error", "flce_b200_version"):
        getattr(lib, name).restype = C.c_char_p
    lib.flce_b200_status_string.argtypes = [C.c_int]
    return lib


lib = _load()


class FlceError(RuntimeError):
    pass


def check(status):
    if status != 0:
        raise FlceError(
            f"libflce_b200: {lib.flce_b200_status_string(status).decode()}: {lib.flce_b200_last_error().decode()}"
        )


KERNEL_KINDS = ("stats", "dz", "dw", "dx", "gemm")


def profile_enable(on=True):
    check(lib.flce_b200_profile_enable(int(on)))


def profile_read(reset=True):
    """{kind: (milliseconds, launches)} of the tensor-core kernels recorded since the last reset."""
    ms = (C.c_double * len(KERNEL_KINDS))()
    n = (C.c_int64 * len(KERNEL_KINDS))()
    check(lib.flce_b200_profile_read(ms, n, int(reset)))
    return {k: (ms[i], n[i]) for i, k in enumerate(KERNEL_KINDS)}


def set_option(name, value):
    check(lib.flce_b200_set_option(name.encode(), int(value)))
