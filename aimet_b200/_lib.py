"""ctypes binding of ``libaimet_b200.so`` (the C ABI declared in ``include/aimet_b200.h``).

There is no CPU or PyTorch fallback: if the library is missing, importing this module raises.
Build it with ``python -m aimet_b200.build`` (needs nvcc; cross-compiles for sm_100a without a GPU).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
#: the in-tree build, unless AIMET_B200_LIB names another build of the same library
LIB_PATH = os.environ.get("AIMET_B200_LIB") or os.path.join(_HERE, "lib", "libaimet_b200.so")

AQ_OK = 0
AQ_F32, AQ_F16, AQ_BF16 = 0, 1, 2
AQ_V2_OUT_QDQ, AQ_V2_OUT_CODES = 0, 1
AQ_PDF_SIZE = 512
AQ_TFE_HIST_MANY = 16
AQ_V2HIST_MAX_BINS = 4096
V2HIST_HEAD_BYTES = 16


class AqEncoding(C.Structure):
    """Mirror of ``aq_encoding_t`` / DlQuantization::TfEncoding."""
    _fields_ = [("min", C.c_double), ("max", C.c_double), ("delta", C.c_double), ("offset", C.c_double),
                ("bw", C.c_int)]


class AqTfeState(C.Structure):
    """Mirror of ``aq_tfe_state_t`` (lives in device memory; this type is only used for its size/offsets)."""
    _fields_ = [("x_left", C.c_double * AQ_PDF_SIZE), ("bucket_size", C.c_float), ("pdf_offset", C.c_float),
                ("initialized", C.c_int32), ("reserved", C.c_int32)]


TFE_STATE_BYTES = C.sizeof(AqTfeState)

_vp, _i64, _i32, _f64 = C.c_void_p, C.c_int64, C.c_int, C.c_double

#: name -> (restype, argtypes); the complete export list of include/aimet_b200.h
SIGNATURES = {
    "aq_version": (_i32, []),
    "aq_status_string": (C.c_char_p, [_i32]),
    "aq_last_cuda_error": (C.c_char_p, []),
    "aq_launch_count": (_i64, []),
    "aq_fill_encoding": (_i32, [_i32, _f64, _f64, C.POINTER(AqEncoding)]),
    "aq_computed_encodings": (_i32, [_i32, _f64, _f64, _i32, _i32, _i32, C.POINTER(AqEncoding)]),
    "aq_minmax_encoding": (_i32, [_i32, _f64, _f64, _i32, _i32, _i32, C.POINTER(AqEncoding)]),
    "aq_qdq_per_tensor": (_i32, [_vp, _vp, _i64, _f64, _f64, _i32, _i32, _vp]),
    "aq_quantize_per_tensor": (_i32, [_vp, _vp, _i64, _f64, _f64, _i32, _i32, _i32, _vp]),
    "aq_v2_minmax_encoding": (_i32, [_vp, _vp, _i32, _i32, _i64, _f64, _i32, _f64, _vp, _vp]),
    "aq_qdq_fp16": (_i32, [_vp, _vp, _i64, _vp]),
    "aq_quantize_packed": (_i32, [_vp, _vp, _i64, _f64, _f64, _i32, _i32, _i32, _vp]),
    "aq_dequantize_packed": (_i32, [_vp, _vp, _i64, _f64, _f64, _i32, _i32, _vp]),
    "aq_qdq_per_channel": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _f64, _i32, _vp]),
    "aq_qdq_broadcast": (_i32, [_vp, _vp, _i64, _i64, C.POINTER(_i64), C.POINTER(_i64), _vp, _vp, _vp, _vp, _vp]),
    "aq_ste_backward_v1": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp]),
    "aq_v2_quantize": (_i32, [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _vp, _vp, _f64, _f64, _i32, _i32, _vp]),
    "aq_v2_dequantize": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _vp, _vp, _i32, _vp]),
    "aq_v2_qdq_backward": (_i32, [_vp, _vp, _vp, _i32, _i64, _vp]),
    "aq_v2_qdq_backward_params": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _vp, _vp, _f64, _f64, _vp]),
    "aq_v2_qdq_backward_params_reduced": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _vp, _vp, _f64, _f64,
                                                 _vp]),
    "aq_minmax_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "aq_minmax": (_i32, [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _i32, _i32, _vp, _i64, _vp]),
    "aq_minmax_static": (_i32, [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _i32, _vp]),
    "aq_tfe_init_grid": (_i32, [_vp, _vp, _vp]),
    "aq_tfe_histogram": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp]),
    "aq_tfe_histogram_many": (_i32, [C.POINTER(_vp), C.POINTER(_i64), _i32, _i64, _vp, _vp, _vp, _vp, _vp]),
    "aq_tfe_offer_grid_workspace_bytes": (_i64, []),
    "aq_tfe_offer_grid": (_i32, [_vp, _i64, _vp, _vp, _i32, _vp, _i64, _vp]),
    "aq_tfe_select_grid": (_i32, [_vp, _i32, _i32, _vp, _vp, _vp]),
    "aq_tfe_pdf_replay": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp]),
    "aq_tfe_search_workspace_bytes": (_i64, []),
    "aq_tfe_search": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _i64, _vp]),
    "aq_tfe_mse_workspace_bytes": (_i64, []),
    "aq_tfe_mse_encoding": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _i64, _vp]),
    "aq_tfe_percentile_encoding": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _i32, _vp, _f64, _i32, _i32, _i32, _i32, _vp, _vp]),
    "aq_v2hist_scratch_bytes": (_i64, []),
    "aq_v2hist_collect": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp, _vp]),
    "aq_v2hist_merge": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp, _i32, _vp, _vp, _vp]),
    "aq_v2hist_collect_rows": (_i32, [_vp, _i32, _i64, _i32, _i32, _vp, _i64, _vp, _vp]),
    "aq_v2hist_merge_rows": (_i32, [_vp, _i32, _i64, _i32, _i32, _vp, _vp, _i64, _i32, _vp, _vp, _vp]),
    "aq_v2hist_update_rows": (_i32, [_vp, _i32, _i64, _i32, _i32, _vp, _vp, _i64, _i32, _vp, _vp, _vp]),
    "aq_v2hist_range_rows": (_i32, [_vp, _i32, _i64, _i32, _vp, _vp, _vp]),
    "aq_v2hist_plan_batches": (_i32, [_vp, _i32, _i32, _i32, _vp, _vp]),
    "aq_v2hist_count_rows": (_i32, [_vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp]),
    "aq_v2hist_range_many": (_i32, [_vp, _i32, _i32, _i64, _i32, _vp, _i64, _vp, _vp]),
    "aq_v2hist_count_many": (_i32, [_vp, _i32, _i32, _i64, _i32, _i32, _vp, _i64, _vp, _i64, _vp]),
    "aq_v2hist_replay_batches": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp, _i64, _vp]),
    "aq_v2hist_sqnr_rows": (_i32, [_vp, _i64, _i32, _i32, _f64, _i32, _i32, _vp, _i32, _f64, _vp, _vp, _i64, _vp]),
    "aq_v2hist_sqnr_encode_rows": (_i32, [_vp, _i64, _i32, _i32, _f64, _i32, _i32, _vp, _i32, _f64, _i32, _f64, _vp, _vp,
                                          _i64, _vp]),
    "aq_v2hist_sqnr_workspace_bytes": (_i64, []),
    "aq_v2hist_sqnr": (_i32, [_vp, _i32, _f64, _i32, _i32, _vp, _i32, _f64, _vp, _vp, _i64, _vp]),
    "aq_tfe_compute_encoding": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _i64,
                                       _vp]),
}


class AimetB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: the CUDA library is required (there is no CPU fallback). "
            "Build it with `python -m aimet_b200.build`.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if an export is missing
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(status: int, what: str = "") -> None:
    if status != AQ_OK:
        msg = lib.aq_status_string(status).decode()
        if status == -3:
            msg += ": " + lib.aq_last_cuda_error().decode()
        raise AimetB200Error(f"aimet_b200 {what} failed: {msg} (status {status})")


def launch_count() -> int:
    return int(lib.aq_launch_count())
