"""ctypes binding of libkernl_b200.so (the C ABI declared in include/kernl_b200.h).

There is no fallback: if the library is missing or a kernel reports an error, the caller gets an
exception. The library itself loads without a GPU (it links the CUDA runtime statically), which
lets CPU-only checks verify the exported symbols.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_float, c_int32, c_int64, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libkernl_b200.so")

KB_OK = 0
KB_F16, KB_BF16, KB_F32 = 0, 1, 2
ACTIVATIONS = {"": 0, None: 0, "tanh": 1, "gelu": 2, "fast_gelu": 3, "relu": 4, "silu": 5, "swiglu": 6}

EXPORTED_SYMBOLS = [
    "kb_norm_fwd",
    "kb_linear_fwd",
    "kb_linear_workspace_bytes",
    "kb_silu_mul",
    "kb_attention_fwd",
    "kb_attention_decode_scratch_bytes",
    "kb_attention_decode_fwd",
    "kb_rope_kv_write",
    "kb_allreduce_residual_fwd",
    "kb_peer_alloc", "kb_peer_free", "kb_peer_export", "kb_peer_open", "kb_peer_close",
    "kb_attention_decode_static_max_bytes",
    "kb_attention_decode_fwd_static",
    "kb_device_status_read",
    "kb_gemm_sm_limit",
    "kb_status_str",
    "kb_version",
]


class NormParams(Structure):
    _fields_ = [
        ("x", c_void_p), ("y", c_void_p), ("gamma", c_void_p), ("beta", c_void_p),
        ("mean", c_void_p), ("rstd", c_void_p),
        ("rows", c_int64), ("cols", c_int64),
        ("x_row_stride", c_int64), ("x_col_stride", c_int64),
        ("y_row_stride", c_int64), ("y_col_stride", c_int64),
        ("eps", c_float), ("is_rms", c_int32), ("dtype", c_int32),
        ("residual", c_void_p), ("sum_out", c_void_p),
    ]


class LinearParams(Structure):
    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("y", c_void_p), ("act_inputs", c_void_p),
        ("M", c_int64), ("N", c_int64), ("K", c_int64),
        ("x_row_stride", c_int64), ("y_row_stride", c_int64),
        ("activation", c_int32), ("dtype", c_int32),
        ("workspace", c_void_p), ("workspace_bytes", c_int64),
    ]


class AttnParams(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("mask", c_void_p),
        ("B", c_int64), ("H", c_int64), ("M", c_int64), ("N", c_int64), ("D", c_int64),
        ("q_strides", c_int64 * 4), ("k_strides", c_int64 * 4), ("v_strides", c_int64 * 4),
        ("o_strides", c_int64 * 4), ("mask_strides", c_int64 * 4),
        ("sm_scale", c_float), ("is_causal", c_int32), ("dtype", c_int32), ("mask_dtype", c_int32),
        ("kv_group", c_int32), ("kv_len_dev", c_void_p),
    ]


class RopeParams(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("q_out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
        ("cos", c_void_p), ("sin", c_void_p), ("pos_dev", c_void_p), ("pos_host", c_int64),
        ("B", c_int64), ("S", c_int64), ("H", c_int64), ("D", c_int64), ("max_seq", c_int64),
        ("dtype", c_int32),
    ]


class AllReduceParams(Structure):
    _fields_ = [
        ("partials", c_void_p * 8), ("flags", c_void_p * 8), ("residual", c_void_p), ("out", c_void_p),
        ("count", c_int64), ("rank", c_int32), ("world", c_int32), ("dtype", c_int32),
        ("norm_weight", c_void_p), ("norm_out", c_void_p), ("cols", c_int64), ("eps", c_float),
    ]


_lib = None


def load() -> ctypes.CDLL:
    """Load the CUDA library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m kernl_b200.build` (needs nvcc). "
            "kernl_b200 has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.kb_norm_fwd.argtypes = [POINTER(NormParams), c_void_p]
    lib.kb_norm_fwd.restype = ctypes.c_int
    lib.kb_linear_fwd.argtypes = [POINTER(LinearParams), c_void_p]
    lib.kb_linear_fwd.restype = ctypes.c_int
    lib.kb_linear_workspace_bytes.argtypes = [c_int64, c_int64]
    lib.kb_linear_workspace_bytes.restype = c_int64
    lib.kb_silu_mul.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p]
    lib.kb_silu_mul.restype = ctypes.c_int
    lib.kb_attention_fwd.argtypes = [POINTER(AttnParams), c_void_p]
    lib.kb_attention_fwd.restype = ctypes.c_int
    lib.kb_attention_decode_scratch_bytes.argtypes = [c_int64] * 5
    lib.kb_attention_decode_scratch_bytes.restype = c_int64
    lib.kb_attention_decode_fwd.argtypes = [POINTER(AttnParams), c_void_p, c_int64, c_void_p]
    lib.kb_attention_decode_fwd.restype = ctypes.c_int
    lib.kb_attention_decode_static_max_bytes.argtypes = []
    lib.kb_attention_decode_static_max_bytes.restype = c_int64
    lib.kb_attention_decode_fwd_static.argtypes = [POINTER(AttnParams), c_void_p]
    lib.kb_attention_decode_fwd_static.restype = ctypes.c_int
    lib.kb_rope_kv_write.argtypes = [POINTER(RopeParams), c_void_p]
    lib.kb_rope_kv_write.restype = ctypes.c_int
    lib.kb_allreduce_residual_fwd.argtypes = [POINTER(AllReduceParams), c_void_p]
    lib.kb_allreduce_residual_fwd.restype = ctypes.c_int
    lib.kb_peer_alloc.argtypes = [c_int64, POINTER(c_void_p)]
    lib.kb_peer_export.argtypes = [c_void_p, ctypes.c_char_p]
    lib.kb_peer_open.argtypes = [ctypes.c_char_p, POINTER(c_void_p)]
    lib.kb_peer_free.argtypes = [c_void_p]
    lib.kb_peer_close.argtypes = [c_void_p]
    for name in ("kb_peer_alloc", "kb_peer_export", "kb_peer_open", "kb_peer_free", "kb_peer_close"):
        getattr(lib, name).restype = ctypes.c_int
    lib.kb_gemm_sm_limit.argtypes = [ctypes.c_int]
    lib.kb_gemm_sm_limit.restype = ctypes.c_int
    lib.kb_device_status_read.argtypes = [POINTER(c_int32)]
    lib.kb_device_status_read.restype = ctypes.c_int
    lib.kb_status_str.argtypes = [ctypes.c_int]
    lib.kb_status_str.restype = ctypes.c_char_p
    lib.kb_version.restype = ctypes.c_int
    # unstable test hooks (include/kernl_b200_debug.h)
    for hook in ("kb_debug_force_bn", "kb_debug_force_splits", "kb_debug_pdl", "kb_debug_split_tiles", "kb_debug_attention_persistent", "kb_debug_linear_pair"):
        if hasattr(lib, hook):
            getattr(lib, hook).argtypes = [ctypes.c_int]
            getattr(lib, hook).restype = None
    if hasattr(lib, "kb_debug_wait_limit"):
        lib.kb_debug_wait_limit.argtypes = [c_int64, c_int64]
        lib.kb_debug_wait_limit.restype = ctypes.c_int
    if os.environ.get("KERNL_B200_PDL", "1") == "0" and hasattr(lib, "kb_debug_pdl"):
        lib.kb_debug_pdl(0)  # launch every kernel with plain stream ordering (A/B measurements)
    _lib = lib
    return lib


def status_str(status: int) -> str:
    return load().kb_status_str(status).decode()


def check(status: int, what: str) -> None:
    if status != KB_OK:
        raise RuntimeError(f"kernl_b200: {what} failed: {status_str(status)} (status {status})")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return KB_F16
    if dtype == torch.bfloat16:
        return KB_BF16
    if dtype == torch.float32:
        return KB_F32
    raise AssertionError(f"unsupported dtype {dtype}")


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_expiry_hooks = []


def on_wait_expired(hook) -> None:
    """Register a callable that `device_status` runs when it finds that a bounded wait expired
    (front-ends use it to put scratch that a cut-short kernel may have left dirty back in order)."""
    _expiry_hooks.append(hook)


def device_status() -> list:
    """Synchronise the device and return (and clear) the kernels' status word; raises when a
    bounded device-side wait expired. Kernels launched between the expiry and this call did no
    work, so call it at every point where results leave the GPU (end of a generation loop, after
    replaying captured graphs, before closing peer buffers)."""
    out = (c_int32 * 4)()
    st = load().kb_device_status_read(out)
    vals = list(out)
    if st != KB_OK:
        for hook in _expiry_hooks:
            hook()
        raise RuntimeError(f"kernl_b200 device status: {status_str(st)}; word = {vals}")
    return vals
