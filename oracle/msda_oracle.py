"""ctypes front end of the C oracle (``msda_oracle.c``). TEST INFRASTRUCTURE ONLY.

The oracle restates the reference's CPU golden
(tests/torch/test_multi_scale_deformable_attn.py:34-76) and the device kernel's
sample/corner rules (kernels/multi_scale_deformable_attn/op_kernel/msda.h:367-390)
in double precision. Inputs are numpy float32 arrays that already hold the values
of the dtype under test; results are float64.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libmsda_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (through the Makefile next to this file)."""
    src = os.path.join(_HERE, "msda_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(_LIB_PATH)
        f32 = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
        f64 = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
        i32 = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
        dims = [ctypes.c_int] * 7
        lib.msda_oracle_forward.argtypes = [f32, i32, i32, f32, f32, f64] + dims
        lib.msda_oracle_forward.restype = None
        lib.msda_oracle_backward.argtypes = [f32, i32, i32, f32, f32, f32, f64, f64, f64] + dims
        lib.msda_oracle_backward.restype = None
        lib.gka_oracle_forward.argtypes = [f32, i32, i32, f32, f32, f64] + dims
        lib.gka_oracle_forward.restype = None
        lib.gka_oracle_backward.argtypes = [f32, i32, i32, f32, f32, f32, f64, f64] + dims
        lib.gka_oracle_backward.restype = None
        d8 = [ctypes.c_int] * 8
        lib.da_oracle_forward.argtypes = [f32, i32, i32, f32, f32, f64] + d8
        lib.da_oracle_forward.restype = None
        lib.da_oracle_backward.argtypes = [f32, i32, i32, f32, f32, f32, f64, f64, f64] + d8
        lib.da_oracle_backward.restype = None
        lib.msda_oracle_kink_distance.argtypes = [i32, f32, f64] + [ctypes.c_int] * 5
        lib.msda_oracle_kink_distance.restype = None
        lib.msda_oracle_set_threads.argtypes = [ctypes.c_int]
        lib.msda_oracle_set_threads.restype = None
        _lib = lib
    return _lib


def set_threads(n: int) -> None:
    _load().msda_oracle_set_threads(int(n))


def _prep(value, shapes, starts, loc, attn):
    value = np.ascontiguousarray(value, dtype=np.float32)
    loc = np.ascontiguousarray(loc, dtype=np.float32)
    attn = np.ascontiguousarray(attn, dtype=np.float32)
    shapes = np.ascontiguousarray(shapes, dtype=np.int32).reshape(-1, 2)
    starts = np.ascontiguousarray(starts, dtype=np.int32).reshape(-1)
    B, K, H, D = value.shape
    _, Q, H2, L, P, two = loc.shape
    if H2 != H or two != 2 or attn.shape != (B, Q, H, L, P) or shapes.shape[0] != L:
        raise ValueError("inconsistent MSDA operand shapes")
    if int((shapes[:, 0] * shapes[:, 1]).sum()) > K and int(starts[-1] + shapes[-1, 0] * shapes[-1, 1]) > K:
        raise ValueError("levels do not fit in value")
    return value, shapes, starts, loc, attn, (B, K, H, D, L, Q, P)


def forward(value, shapes, starts, loc, attn):
    """output[B, Q, H*D] in float64."""
    value, shapes, starts, loc, attn, dims = _prep(value, shapes, starts, loc, attn)
    B, K, H, D, L, Q, P = dims
    out = np.empty((B, Q, H * D), dtype=np.float64)
    _load().msda_oracle_forward(value, shapes, starts, loc, attn, out, *dims)
    return out


def backward(value, shapes, starts, loc, attn, grad_out):
    """(grad_value, grad_loc, grad_attn) in float64, shaped like value / loc / attn."""
    value, shapes, starts, loc, attn, dims = _prep(value, shapes, starts, loc, attn)
    B, K, H, D, L, Q, P = dims
    grad_out = np.ascontiguousarray(grad_out, dtype=np.float32).reshape(B, Q, H * D)
    gv = np.empty(value.shape, dtype=np.float64)
    gl = np.empty(loc.shape, dtype=np.float64)
    ga = np.empty(attn.shape, dtype=np.float64)
    _load().msda_oracle_backward(value, shapes, starts, loc, attn, grad_out, gv, gl, ga, *dims)
    return gv, gl, ga


def kink_distance(shapes, loc):
    """Per sample, distance (in pixels) of (x, y) to the nearest cell boundary.

    grad_sampling_loc is a one-sided derivative at a boundary; comparisons mask
    samples whose distance is below float rounding of the pixel coordinate.
    """
    loc = np.ascontiguousarray(loc, dtype=np.float32)
    shapes = np.ascontiguousarray(shapes, dtype=np.int32).reshape(-1, 2)
    B, Q, H, L, P, _ = loc.shape
    dist = np.empty((B, Q, H, L, P), dtype=np.float64)
    _load().msda_oracle_kink_distance(shapes, loc, dist, B, H, L, Q, P)
    return dist


def gka_forward(value, shapes, starts, loc, attn):
    """Geometric kernel attention, output[B, Q, H*D] in float64 (loc = pixel coordinates)."""
    value, shapes, starts, loc, attn, dims = _prep(value, shapes, starts, loc, attn)
    B, K, H, D, L, Q, P = dims
    out = np.empty((B, Q, H * D), dtype=np.float64)
    _load().gka_oracle_forward(value, shapes, starts, loc, attn, out, *dims)
    return out


def gka_backward(value, shapes, starts, loc, attn, grad_out):
    """(grad_value, grad_attn) in float64."""
    value, shapes, starts, loc, attn, dims = _prep(value, shapes, starts, loc, attn)
    B, K, H, D, L, Q, P = dims
    grad_out = np.ascontiguousarray(grad_out, dtype=np.float32).reshape(B, Q, H * D)
    gv = np.empty(value.shape, dtype=np.float64)
    ga = np.empty(attn.shape, dtype=np.float64)
    _load().gka_oracle_backward(value, shapes, starts, loc, attn, grad_out, gv, ga, *dims)
    return gv, ga


def _da_prep(feat, shapes, starts, loc, wts):
    feat = np.ascontiguousarray(feat, dtype=np.float32)
    loc = np.ascontiguousarray(loc, dtype=np.float32)
    wts = np.ascontiguousarray(wts, dtype=np.float32)
    shapes = np.ascontiguousarray(shapes, dtype=np.int32)
    starts = np.ascontiguousarray(starts, dtype=np.int32)
    B, F, C = feat.shape
    _, A, Pts, cams, scales, G = wts.shape
    if loc.shape != (B, A, Pts, cams, 2) or shapes.shape != (cams, scales, 2) or \
            starts.shape != (cams, scales) or C % G != 0:
        raise ValueError("inconsistent deformable-aggregation operand shapes")
    return feat, shapes, starts, loc, wts, (B, F, C, A, Pts, cams, scales, G)


def da_forward(feat, shapes, starts, loc, wts):
    """Deformable aggregation, out[B, A, C] in float64."""
    feat, shapes, starts, loc, wts, dims = _da_prep(feat, shapes, starts, loc, wts)
    out = np.empty((dims[0], dims[3], dims[2]), dtype=np.float64)
    _load().da_oracle_forward(feat, shapes, starts, loc, wts, out, *dims)
    return out


def da_backward(feat, shapes, starts, loc, wts, grad_out):
    """(grad_feat, grad_loc, grad_wts) in float64."""
    feat, shapes, starts, loc, wts, dims = _da_prep(feat, shapes, starts, loc, wts)
    grad_out = np.ascontiguousarray(grad_out, dtype=np.float32).reshape(dims[0], dims[3], dims[2])
    gf = np.empty(feat.shape, dtype=np.float64)
    gl = np.empty(loc.shape, dtype=np.float64)
    gw = np.empty(wts.shape, dtype=np.float64)
    _load().da_oracle_backward(feat, shapes, starts, loc, wts, grad_out, gf, gl, gw, *dims)
    return gf, gl, gw
