"""LayerNorm / RMSNorm forward front-end (reference: src/kernl/implementations/layer_norm.py)."""
from typing import Optional

import torch

from kernl_b200 import _lib
from kernl_b200.implementations._autocast import cast_if_autocast


def _aligned(t: torch.Tensor) -> torch.Tensor:
    """gamma, beta and the residual are read with 16-byte accesses; a tensor that starts on another
    boundary (e.g. a graph input placed by the 8-byte-aligned CUDA-graph arena) is copied."""
    return t if t.data_ptr() % 16 == 0 else t.clone(memory_format=torch.contiguous_format)


def pytorch_naive_layernorm(a: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float):
    """Eager LayerNorm used by benchmarks (reference: layer_norm.py:28-38; note the unbiased
    `var` there — kept, since this function only serves as a comparison point)."""
    mean = a.mean(dim=-1, keepdim=True)
    var = a.var(dim=-1, keepdim=True)
    rstd = 1 / torch.sqrt(var + eps)
    return (a - mean) * rstd * weight + bias


def pytorch_naive_rmsnorm(a: torch.Tensor, weight: torch.Tensor, eps: float):
    """Eager RMSNorm (reference: layer_norm.py:41-57). Unlike the reference it does not modify
    its input in place."""
    variance = a.to(torch.float32).pow(2).mean(-1, keepdim=True)
    a = a * torch.rsqrt(variance + eps)
    if weight.dtype in [torch.float16, torch.bfloat16]:
        a = a.to(weight.dtype)
    return weight * a


def layer_norm(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    eps: float,
    implementation=None,
    use_rms_norm: bool = False,
    residual: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
):
    """y = LayerNorm(x) or RMSNorm(x) over the last dimension on the sm_100a kernel.

    Same contract as the reference's `layer_norm` (layer_norm.py:338-346 → LayerNorm.forward
    :279-335): x/weight/bias share a dtype, fp16 inputs clamp eps to 1.6e-5 (:295-296), a new
    tensor shaped like x is returned. `implementation` selected one of several Triton kernels in
    the reference; there is a single CUDA implementation here, so it is accepted and ignored.
    `residual` (an extension for pre-norm decoders): normalise x + residual in the same kernel and
    return the pair (y, x + residual). `out` (an extension as well): a caller-provided result tensor
    shaped like x, written instead of a new one.
    """
    x, weight, bias, residual = cast_if_autocast(x, weight, bias, residual)
    assert x.dtype == weight.dtype, f"input and weight bias must have the same dtype: {x.dtype}, {weight.dtype}"
    if bias is not None:
        assert x.dtype == bias.dtype, f"input and bias must have the same dtype: {x.dtype}, {bias.dtype}"
    assert x.dtype in (torch.float16, torch.bfloat16), f"Only float16 and bfloat16 are supported, got {x.dtype}"
    assert x.is_cuda, "kernl_b200 ops run on a CUDA (sm_100a) device only"
    if x.dtype == torch.float16:
        eps = max(eps, 1.6e-5)
    n = x.shape[-1]
    assert weight.shape[-1] == n and weight.numel() == n
    weight = _aligned(weight.contiguous())
    bias = _aligned(bias.contiguous()) if bias is not None else None
    if out is not None:
        assert out.shape == x.shape and out.dtype == x.dtype and out.device == x.device and out.is_contiguous()
    if x.dim() == 2:
        out = torch.empty_like(x) if out is None else out
        x2, out2 = x, out
    else:
        x2 = x.reshape(-1, n)
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device) if out is None else out
        out2 = out.view(-1, n)
    rows = x2.shape[0]
    sum_out = None
    if residual is not None:
        assert residual.shape == x.shape and residual.dtype == x.dtype
        x2 = x2.contiguous()
        residual = _aligned(residual.contiguous())
        sum_out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    if rows == 0:
        return out if residual is None else (out, sum_out)
    p = _lib.NormParams(
        x=x2.data_ptr(), y=out2.data_ptr(), gamma=weight.data_ptr(),
        beta=bias.data_ptr() if bias is not None else None, mean=None, rstd=None,
        rows=rows, cols=n,
        x_row_stride=x2.stride(0), x_col_stride=x2.stride(1),
        y_row_stride=out2.stride(0), y_col_stride=out2.stride(1),
        eps=float(eps), is_rms=1 if use_rms_norm else 0, dtype=_lib.dtype_code(x.dtype),
        residual=residual.data_ptr() if residual is not None else None,
        sum_out=sum_out.data_ptr() if sum_out is not None else None,
    )
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().kb_norm_fwd(p, _lib.current_stream(x.device)), "layer_norm")
    return out if residual is None else (out, sum_out)
