"""Fused linear front-end (reference: src/kernl/implementations/linear_layer.py)."""
from typing import Optional

import torch

from kernl_b200 import _lib
from kernl_b200.implementations._autocast import cast_if_autocast


_WORKSPACE_BYTES = 32 * 1024 * 1024
_workspaces = {}
_padded_weights = {}


def _workspace(device: torch.device) -> torch.Tensor:
    """A zero-initialised scratch buffer for split-K partial sums per (device, stream), allocated on
    first use and kept (a stable address, so CUDA graphs that captured it stay valid). The kernel
    leaves it zero after every call. Calls on different streams get different buffers, so they may
    overlap on the GPU; a graph replayed on a stream other than the one it was captured on keeps
    using the capture stream's buffer."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        with torch.inference_mode(False):  # an ordinary tensor: it is zeroed in place again after an expired wait
            ws = torch.zeros(_WORKSPACE_BYTES // 4, dtype=torch.float32, device=device)
        _workspaces[key] = ws
    return ws


def _rezero_workspaces() -> None:
    """A GEMM whose wait expired may have left partial sums behind; split-K needs zeros."""
    for ws in _workspaces.values():
        ws.zero_()


_lib.on_wait_expired(_rezero_workspaces)


def _aligned(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """The kernels read weights and biases with 16-byte accesses. A tensor that starts elsewhere
    (a graph input that the CUDA-graph arena placed on an 8-byte boundary, a slice) is copied."""
    if t is None or t.data_ptr() % 16 == 0:
        return t
    return t.clone(memory_format=torch.contiguous_format)


def _k_padded_weight(weight: torch.Tensor, pad: int) -> torch.Tensor:
    """Weight with `pad` zero columns appended, built once per weight (and again when the weight
    is modified in place) rather than on every call."""
    key = (weight.data_ptr(), tuple(weight.shape), weight.dtype, weight.device)
    hit = _padded_weights.get(key)
    if hit is not None and hit[0] == weight._version:
        return hit[1]
    if len(_padded_weights) >= 256:
        _padded_weights.clear()
    padded = torch.nn.functional.pad(weight, (0, pad))
    _padded_weights[key] = (weight._version, padded)
    return padded


def linear_layer(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    activation="",
    act_inputs: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """activation(x @ weight.T + bias) on the tcgen05 GEMM kernel.

    Same contract as the reference's `linear_layer` (linear_layer.py:285-292 →
    LinearLayer.forward :213-282): x is 2-D or 3-D (flattened over its first two dims), weight is
    [N, K] contiguous, bias [N] contiguous or None, activation in {"", "tanh", "gelu",
    "fast_gelu", "relu"} (plus "silu", and "swiglu": weight rows interleaved by
    `interleave_gate_up`, result [M, N/2] = silu(gate) * up); `act_inputs`, if given, receives the
    pre-activation values. Returns [M, N], or [x.shape[0], -1, N] for 3-D x. fp32 inputs (tf32 in the
    reference) are not supported: fp16/bf16 only. `out` (an extension over the reference's
    signature) lets the caller provide the [M, N] result buffer (unit column stride, any row stride),
    e.g. a peer-mapped one or a column slice of a wider tensor.
    """
    x, weight, bias = cast_if_autocast(x, weight, bias)
    x_ = x if x.ndim == 2 else x.flatten(0, 1)
    assert x.dtype == weight.dtype, f"Input and weight must have the same dtype, got {x.dtype} and {weight.dtype}"
    if bias is not None:
        assert x.dtype == bias.dtype, f"Input and bias must have the same dtype, got {x.dtype} and {bias.dtype}"
    assert x.dtype in (torch.float16, torch.bfloat16), f"Only float16 and bfloat16 are supported, got {x.dtype}"
    assert x_.shape[1] == weight.shape[1], f"Incompatible dimensions: {x_.shape} - {weight.shape}"
    assert bias is None or bias.is_contiguous()
    assert bias is None or bias.shape[0] == weight.shape[0], "Incompatible dimensions in between weight and bias"
    assert weight.is_contiguous()
    assert activation in _lib.ACTIVATIONS, f"Unknown activation: {activation}"
    assert x.is_cuda, "kernl_b200 ops run on a CUDA (sm_100a) device only"

    M, K = x_.shape
    N = weight.shape[0]
    gated = activation == "swiglu"
    if gated:
        assert N % 16 == 0 and act_inputs is None, "swiglu wants gate/up rows in blocks of eight and no act_inputs"
    n_out = N // 2 if gated else N
    # The TMA path wants unit K stride and 16-byte aligned rows; anything else is copied once.
    if x_.stride(1) != 1 or x_.stride(0) % 8 != 0 or x_.data_ptr() % 16 != 0:
        x_ = x_.contiguous()
    if K % 8 != 0:
        # K is padded with zeros to the next multiple of 8 (16-byte rows for TMA); zeros add nothing.
        pad = 8 - K % 8
        x_ = torch.nn.functional.pad(x_, (0, pad))
        weight = _k_padded_weight(weight, pad)
        K += pad
    weight, bias = _aligned(weight), _aligned(bias)
    if out is not None:
        assert out.shape == (M, n_out) and out.dtype == x.dtype and out.stride(1) == 1 and out.device == x.device
        outputs = out
    else:
        outputs = torch.empty((M, n_out), device=x.device, dtype=x.dtype)
    if act_inputs is not None:
        assert act_inputs.shape == (M, N) and act_inputs.dtype == x.dtype and act_inputs.is_contiguous()
    if M > 0:
        ws = _workspace(x.device) if _lib.load().kb_linear_workspace_bytes(M, N) <= _WORKSPACE_BYTES else None
        p = _lib.LinearParams(
            x=x_.data_ptr(), w=weight.data_ptr(), bias=bias.data_ptr() if bias is not None else None,
            y=outputs.data_ptr(), act_inputs=act_inputs.data_ptr() if act_inputs is not None else None,
            M=M, N=N, K=K, x_row_stride=x_.stride(0), y_row_stride=outputs.stride(0),
            activation=_lib.ACTIVATIONS[activation], dtype=_lib.dtype_code(x.dtype),
            workspace=ws.data_ptr() if ws is not None else None,
            workspace_bytes=ws.numel() * 4 if ws is not None else 0,
        )
        with torch.cuda.device(x.device):
            _lib.check(_lib.load().kb_linear_fwd(p, _lib.current_stream(x.device)), "linear_layer")
    return outputs if x.ndim == 2 else outputs.reshape(x.shape[0], -1, n_out)


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[F, K] gate and up projection weights → the [2F, K] layout that activation="swiglu" reads:
    blocks of eight gate rows alternate with the matching eight up rows, so that one CTA (whatever
    its tile width) holds both halves of every output column it produces. F a multiple of 8.
    Works on biases ([F]) too."""
    assert w_gate.shape == w_up.shape and w_gate.shape[0] % 8 == 0
    f = w_gate.shape[0]
    rest = w_gate.shape[1:]
    both = torch.stack((w_gate.reshape(f // 8, 8, *rest), w_up.reshape(f // 8, 8, *rest)), dim=1)
    return both.reshape(2 * f, *rest).contiguous()


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for gate_up = [..., 2*N] laid out as [gate | up] (SwiGLU feed-forward)."""
    assert gate_up.dtype in (torch.float16, torch.bfloat16) and gate_up.is_contiguous()
    n2 = gate_up.shape[-1]
    assert n2 % 16 == 0
    n = n2 // 2
    m = gate_up.numel() // n2
    out = torch.empty(gate_up.shape[:-1] + (n,), dtype=gate_up.dtype, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        _lib.check(
            _lib.load().kb_silu_mul(gate_up.data_ptr(), out.data_ptr(), m, n, _lib.dtype_code(gate_up.dtype),
                                    _lib.current_stream(gate_up.device)),
            "silu_mul",
        )
    return out
