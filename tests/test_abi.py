"""CPU checks of the C-ABI boundary: the library builds, loads without a GPU, exports every symbol
the header declares, and rejects bad arguments without touching a device."""
import ctypes
import os
import re

from kernl_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "kernl_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kb_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    build.build()
    lib = ctypes.CDLL(build.LIB_PATH)
    names = declared_functions()
    assert "kb_attention_fwd" in names and "kb_linear_fwd" in names and "kb_norm_fwd" in names
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/kernl_b200.h but not exported"
    for name in _lib.EXPORTED_SYMBOLS:
        assert name in names


def test_version_and_status_strings():
    lib = _lib.load()
    assert lib.kb_version() >= 100
    assert _lib.status_str(0) == "ok"
    for code in range(-6, 0):
        assert _lib.status_str(code) != "unknown status"


def test_bad_arguments_are_rejected_before_any_device_call():
    lib = _lib.load()
    assert lib.kb_norm_fwd(None, None) == -1
    assert lib.kb_linear_fwd(None, None) == -1
    assert lib.kb_attention_fwd(None, None) == -1
    p = _lib.LinearParams(x=16, w=16, y=16, M=4, N=4, K=0)
    assert lib.kb_linear_fwd(p, None) == -1
    p = _lib.LinearParams(x=16, w=16, y=16, M=4, N=4, K=12, x_row_stride=12, y_row_stride=4)
    assert lib.kb_linear_fwd(p, None) == -2  # K not a multiple of 8
    gated = _lib.ACTIVATIONS["swiglu"]
    p = _lib.LinearParams(x=16, w=16, y=16, M=4, N=24, K=16, x_row_stride=16, y_row_stride=12, activation=gated)
    assert lib.kb_linear_fwd(p, None) == -1  # gate/up rows come in blocks of eight: N a multiple of 16
    p = _lib.LinearParams(x=16, w=16, y=16, act_inputs=16, M=4, N=32, K=16, x_row_stride=16, y_row_stride=16,
                          activation=gated)
    assert lib.kb_linear_fwd(p, None) == -1  # no pre-activation output with the gated epilogue
    p = _lib.LinearParams(x=16, w=16, y=16, M=4, N=32, K=16, x_row_stride=16, y_row_stride=16, activation=7)
    assert lib.kb_linear_fwd(p, None) == -1
    assert lib.kb_attention_decode_scratch_bytes(2, 3, 1, 1500, 64) == 2 * 3 * 1 * 12 * 66 * 4
    assert lib.kb_attention_decode_scratch_bytes(1, 1, 1, 128 * 256 + 1, 64) == 129 * 66 * 4


def test_struct_layouts_match_the_header():
    # sizes follow from the field lists in include/kernl_b200.h (LP64)
    assert ctypes.sizeof(_lib.NormParams) == 6 * 8 + 6 * 8 + 3 * 4 + 4 + 2 * 8
    assert ctypes.sizeof(_lib.LinearParams) == 5 * 8 + 5 * 8 + 2 * 4 + 2 * 8
    assert ctypes.sizeof(_lib.AttnParams) == 5 * 8 + 5 * 8 + 5 * 32 + 4 * 4
