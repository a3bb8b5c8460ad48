"""ctypes view of the C-ABI library (``libmsda_sm100.so``, include/msda_sm100.h and
include/conv_ops_sm100.h).

This is the same boundary a non-Python host would bind. The torch extension
``_C`` links against the library directly; this module exists for callers that
hold raw device pointers (tests, the benchmark's kernel-only timing, other
runtimes). Loading fails loudly when the library has not been built.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmsda_sm100.so")
# the same library compiled with -DMSDA_DEBUG_BOUNDS (every computed row offset checked)
DEBUG_LIB_PATH = os.path.join(_HERE, "libmsda_sm100_dbg.so")

F32, F16, BF16 = 0, 1, 2
TUNE_STAGE, TUNE_CTAS_PER_SM, TUNE_CTAS_PER_SM_BWD, TUNE_INTERLEAVE, TUNE_SPIN_LIMIT = 0, 1, 2, 3, 4
TUNE_PRECISE_AMP, TUNE_DEBUG_ROW_LIMIT, TUNE_PACK_ROWS = 5, 6, 7

# name -> (restype, argtypes); kept in step with the headers under include/
_vp, _ip, _i, _sz = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
_DIMS7 = [_i] * 7
SIGNATURES = {
    "msda_sm100_forward": (_i, [_vp, _ip, _ip, _vp, _vp, _vp] + _DIMS7 + [_i, _vp]),
    "msda_sm100_backward": (_i, [_vp, _ip, _ip, _vp, _vp, _vp, _vp, _vp, _vp] + _DIMS7 + [_i, _vp]),
    "msda_sm100_backward_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "msda_sm100_backward_ws": (_i, [_vp, _ip, _ip, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz]
                               + _DIMS7 + [_i, _vp]),
    "msda_sm100_fused_forward": (_i, [_vp, _ip, _ip, _vp, _vp, _vp, _vp] + _DIMS7 + [_i, _vp]),
    "msda_sm100_fused_backward_ws": (_i, [_vp, _ip, _ip, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                         _vp, _sz] + _DIMS7 + [_i, _vp]),
    "gka_sm100_forward": (_i, [_vp, _ip, _ip, _vp, _vp, _vp] + _DIMS7 + [_i, _vp]),
    "gka_sm100_backward_ws": (_i, [_vp, _ip, _ip, _vp, _vp, _vp, _vp, _vp, _vp, _sz] + _DIMS7
                              + [_i, _vp]),
    "da_sm100_forward": (_i, [_vp, _ip, _ip, _vp, _vp, _vp] + [_i] * 8 + [_vp]),
    "da_sm100_backward": (_i, [_vp, _ip, _ip, _vp, _vp, _vp, _vp, _vp, _vp] + [_i] * 8 + [_vp]),
    "da_sm100_last_cuda_error": (_i, []),
    "msda_sm100_static_scratch_bytes": (_sz, []),
    "msda_sm100_backward_static": (_i, [_vp, _ip, _ip, _vp, _vp, _vp, _vp, _vp, _vp] + _DIMS7
                                   + [_i, _vp]),
    "addrelu_sm100_forward": (_i, [_vp, _vp, _sz, _i, _vp]),
    "addrelu_sm100_backward": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "maxpool_sm100_forward": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "dcn_sm100_columns_bytes": (_sz, [_vp]),
    "dcn_sm100_backward_workspace_bytes": (_sz, [_vp]),
    "dcn_sm100_forward": (_i, [_vp] * 7 + [_vp, _vp]),
    "dcn_sm100_backward": (_i, [_vp] * 11 + [_vp, _sz, _vp, _vp]),
    "dcn_sm100_use_tensor_cores": (_i, [_i]),
    "gemm_tn_sm100_f32": (_i, [_vp, ctypes.c_longlong, _vp, ctypes.c_longlong, _vp,
                               ctypes.c_longlong, _i, _i, _i, _i, _vp]),
    "gemm_nt_sm100_f32": (_i, [_vp, ctypes.c_longlong, _vp, ctypes.c_longlong, _vp,
                               ctypes.c_longlong, _vp, _i, _i, _i, _i, _vp]),
    "msda_sm100_forward_bytes": (_sz, _DIMS7 + [_i]),
    "msda_sm100_backward_bytes": (_sz, _DIMS7 + [_i]),
    "msda_sm100_probe_row_rates": (_i, [_vp, _sz, _i, _i, ctypes.POINTER(ctypes.c_double),
                                        ctypes.POINTER(ctypes.c_double), _vp]),
    "msda_sm100_device_status": (_i, [_i]),
    "msda_sm100_tune": (_i, [_i, _i]),
    "msda_sm100_profile_events": (None, [_vp, _vp, _vp, _vp]),
    "msda_sm100_launch_count": (ctypes.c_longlong, []),
    "msda_sm100_strerror": (ctypes.c_char_p, [_i]),
    "msda_sm100_last_cuda_error": (_i, []),
    "msda_sm100_abi_version": (_i, []),
    "msda_sm100_debug_bounds": (_i, []),
}



class DcnShape(ctypes.Structure):
    """``dcn_shape`` of include/conv_ops_sm100.h."""
    _fields_ = [(n, ctypes.c_int) for n in (
        "N", "H", "W", "C", "Ho", "Wo", "Co", "kh", "kw", "stride_h", "stride_w", "pad_h",
        "pad_w", "dil_h", "dil_w", "groups", "deform_groups")]


_lib = None
_debug_lib = None


def _open(path):
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is not built; run `python -m drivingsdk_b200.build`. "
            "There is no CPU fallback.")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


def load():
    """Returns the loaded library with argument types set; raises if it is not built."""
    global _lib
    if _lib is None:
        _lib = _open(LIB_PATH)
    return _lib


def load_debug():
    """The bounds-checking build of the same library (its own status word and knobs)."""
    global _debug_lib
    if _debug_lib is None:
        _debug_lib = _open(DEBUG_LIB_PATH)
    return _debug_lib


def dtype_code(torch_dtype) -> int:
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[torch_dtype]


def check(rc: int, what: str) -> None:
    if rc != 0:
        lib = load()
        msg = lib.msda_sm100_strerror(rc).decode()
        raise RuntimeError(f"{what}: {msg} (status {rc}, cuda error {lib.msda_sm100_last_cuda_error()})")
