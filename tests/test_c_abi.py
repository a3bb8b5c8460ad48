"""The C-ABI library: loads, exports everything the header declares, validates arguments.
No kernel is launched here (CPU only)."""
import ctypes
import os
import re

from drivingsdk_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include")


def declared_functions():
    names = set()
    for header in sorted(os.listdir(INCLUDE)):
        if not header.endswith(".h"):
            continue
        text = open(os.path.join(INCLUDE, header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b([a-z][a-z0-9_]*_sm100_\w+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported():
    lib = ctypes.CDLL(capi.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} is declared under include/ but not exported"


def test_python_signature_table_matches_header():
    assert sorted(capi.SIGNATURES) == declared_functions()


def test_abi_version_and_messages():
    lib = capi.load()
    assert lib.msda_sm100_abi_version() == 1
    assert lib.msda_sm100_strerror(0) == b"ok"
    for code in range(-7, 0):
        assert lib.msda_sm100_strerror(code) not in (b"ok", b"unknown status")
    assert lib.msda_sm100_strerror(-99) == b"unknown status"


def test_argument_validation_needs_no_device():
    lib = capi.load()
    dims = (1, 4, 2, 8, 1, 3, 2)
    one = ctypes.c_void_p(16)  # non-null dummy; validation fails before it is ever used
    # null pointer
    assert lib.msda_sm100_forward(None, one, one, one, one, one, *dims, capi.F32, None) == -1
    # unknown dtype
    assert lib.msda_sm100_forward(one, one, one, one, one, one, *dims, 9, None) == -5
    # non-positive dimension
    assert lib.msda_sm100_forward(one, one, one, one, one, one, 0, 4, 2, 8, 1, 3, 2, capi.F32, None) == -2
    # D > 256
    assert lib.msda_sm100_forward(one, one, one, one, one, one, 1, 4, 2, 257, 1, 3, 2, capi.F32, None) == -3
    # L * P > 64
    assert lib.msda_sm100_forward(one, one, one, one, one, one, 1, 4, 2, 8, 5, 3, 13, capi.F32, None) == -3
    # backward: same checks
    assert lib.msda_sm100_backward(one, one, one, one, one, None, one, one, one, *dims, capi.F32, None) == -1
    assert lib.msda_sm100_backward_ws(one, one, one, one, one, one, one, one, one, None, 0,
                                      1, 4, 2, 300, 1, 3, 2, capi.BF16, None) == -3


def test_byte_counts_follow_the_roofline_formulas():
    lib = capi.load()
    B, K, H, D, L, Q, P = 6, 30825, 8, 32, 4, 2500, 8
    v, s, o = B * K * H * D, B * Q * H * L * P, B * Q * H * D
    assert lib.msda_sm100_forward_bytes(B, K, H, D, L, Q, P, capi.F32) == 4 * (v + 3 * s + o)
    assert lib.msda_sm100_backward_bytes(B, K, H, D, L, Q, P, capi.F32) == 4 * (2 * v + 6 * s + o)
    assert lib.msda_sm100_forward_bytes(B, K, H, D, L, Q, P, capi.BF16) == 2 * (v + 3 * s + o)
    assert lib.msda_sm100_backward_workspace_bytes(B, K, H, D, capi.F32) == 0
    assert lib.msda_sm100_backward_workspace_bytes(B, K, H, D, capi.BF16) == 4 * v


def test_tuning_knobs_round_trip():
    lib = capi.load()
    old = lib.msda_sm100_tune(capi.TUNE_STAGE, 0)
    assert lib.msda_sm100_tune(capi.TUNE_STAGE, -1) == 0
    lib.msda_sm100_tune(capi.TUNE_STAGE, old)
    assert lib.msda_sm100_tune(capi.TUNE_STAGE, -1) == old
    assert lib.msda_sm100_tune(99, 1) == -2


def test_deformable_convolution_shape_validation_needs_no_device():
    """dcn_sm100_*: sizes are derived and checked on the host before anything is launched."""
    lib = capi.load()
    ok = capi.DcnShape(2, 7, 9, 8, 7, 9, 16, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1)
    assert lib.dcn_sm100_columns_bytes(ctypes.byref(ok)) == 4 * 2 * 7 * 9 * 9 * 8
    assert lib.dcn_sm100_backward_workspace_bytes(ctypes.byref(ok)) >= 4 * 2 * 7 * 9 * 9 * 8
    wrong_out = capi.DcnShape(2, 7, 9, 8, 6, 9, 16, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1)   # Ho != conv size
    assert lib.dcn_sm100_columns_bytes(ctypes.byref(wrong_out)) == 0
    bad_groups = capi.DcnShape(2, 7, 9, 8, 7, 9, 16, 3, 3, 1, 1, 1, 1, 1, 1, 3, 1)  # 8 % 3 != 0
    assert lib.dcn_sm100_columns_bytes(ctypes.byref(bad_groups)) == 0
    one = ctypes.c_void_p(16)
    assert lib.dcn_sm100_forward(None, one, None, one, None, one, one, ctypes.byref(ok), None) == -1
    assert lib.dcn_sm100_forward(one, one, None, one, None, one, one, ctypes.byref(wrong_out), None) == -2
    # mask without grad_mask (or the reverse) is refused
    assert lib.dcn_sm100_backward(one, one, one, one, one, one, one, one, None, one, None, one, 1 << 30,
                                  ctypes.byref(ok), None) == -1
    assert lib.dcn_sm100_use_tensor_cores(-1) in (0, 1, 2)
    assert lib.gemm_nt_sm100_f32(one, 8, one, 8, one, 4, None, 4, 4, 16, 1, None) == -2   # lda < K
    assert lib.addrelu_sm100_forward(None, one, 4, capi.F32, None) == -1
    assert lib.addrelu_sm100_forward(one, one, 0, capi.F32, None) == 0
    assert lib.addrelu_sm100_forward(one, one, 4, 9, None) == -5
    assert lib.maxpool_sm100_forward(one, one, 1, 1, -1, 4, capi.F32, None) == -2
