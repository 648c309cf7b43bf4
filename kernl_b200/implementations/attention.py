"""Fused attention front-end (reference: src/kernl/implementations/attention.py)."""
import math
from typing import List, Optional, Union

import torch

from kernl_b200 import _lib
from kernl_b200.implementations._autocast import cast_if_autocast


def attention_reference(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    output: torch.Tensor,
    sm_scale: float,
    is_causal: bool,
    attention_mask: Union[torch.Tensor, None],
) -> torch.Tensor:
    """Eager attention, the ground truth of the reference's tests (attention.py:29-61):
    softmax(q·kᵀ·sm_scale + mask, causal → -inf above the top-left-aligned diagonal)·v, written
    into `output`. The reference builds its causal mask on "cuda" (:57); here it follows q.device
    so that the same function also runs on CPU.
    """
    p = torch.matmul(q, k.transpose(2, 3)) * sm_scale
    if attention_mask is not None:
        p += attention_mask
    if is_causal:
        m_size, n_size = q.size(2), k.size(2)
        keep = torch.tril(torch.ones((m_size, n_size), device=q.device))
        p = torch.where(keep == 0, float("-inf"), p)
    p = torch.nn.functional.softmax(p, dim=-1)
    return torch.matmul(p.to(v.dtype), v, out=output)


def closest_power_of_2(n: int, min_range: int = 16, max_range: int = 128) -> List[int]:
    """Powers of two around n clamped to [min_range, max_range] (reference: attention.py:64-70)."""
    n = max(min(n, max_range), min_range)
    lo = math.floor(math.log2(n - 1))
    hi = math.ceil(math.log2(n + 1))
    return [2**i for i in range(lo, hi + 1)]


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """q/k/v feed TMA: unit stride on the head dimension, other strides multiples of 8 elements,
    16-byte aligned base. Tensors laid out differently (e.g. column-major q) are copied once."""
    ok = t.stride(3) == 1 and t.data_ptr() % 16 == 0
    for d in range(3):
        if t.size(d) > 1 and t.stride(d) % 8 != 0:
            ok = False
    return t if ok else t.contiguous()


def _check_mask(attention_mask, batch, heads, m_size, n_size):
    assert attention_mask.size(0) == batch or attention_mask.size(0) == 1, "Incompatible broadcast batch dimension"
    assert attention_mask.size(1) == heads or attention_mask.size(1) == 1, "Incompatible broadcast heads dimension"
    assert attention_mask.size(2) == m_size or attention_mask.size(2) == 1, "Incompatible broadcast m_size dimension"
    assert attention_mask.size(3) == n_size, "Last size of mask must broadcast on QK^t"


def kv_group_of(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> int:
    """Query heads per K/V head: 1 for ordinary attention; grouped-query models pass k/v with fewer
    heads (query head h then reads K/V head h // group) instead of repeating them."""
    heads, kv_heads = q.size(1), k.size(1)
    assert v.size(1) == kv_heads and k.size(0) == q.size(0) and v.size(0) == q.size(0), "Incompatible q/k/v shapes"
    assert kv_heads > 0 and heads % kv_heads == 0, f"{heads} query heads cannot share {kv_heads} key/value heads"
    return heads // kv_heads


def make_params(q, k, v, output, sm_scale, is_causal, attention_mask, kv_len=None) -> "_lib.AttnParams":
    batch, heads, m_size, dhead = q.size()
    n_size = k.size(2)
    p = _lib.AttnParams()
    p.kv_group = kv_group_of(q, k, v)
    p.kv_len_dev = kv_len.data_ptr() if kv_len is not None else None
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), output.data_ptr()
    p.B, p.H, p.M, p.N, p.D = batch, heads, m_size, n_size, dhead
    for i in range(4):
        p.q_strides[i], p.k_strides[i] = q.stride(i), k.stride(i)
        p.v_strides[i], p.o_strides[i] = v.stride(i), output.stride(i)
    if attention_mask is not None:
        p.mask = attention_mask.data_ptr()
        for i in range(4):
            # a broadcast (size-1) dimension never advances
            p.mask_strides[i] = attention_mask.stride(i) if attention_mask.size(i) > 1 else 0
        p.mask_dtype = _lib.dtype_code(attention_mask.dtype)
    else:
        p.mask = None
        p.mask_dtype = _lib.KB_F32
    p.sm_scale = float(sm_scale)
    p.is_causal = 1 if is_causal else 0
    p.dtype = _lib.dtype_code(q.dtype)
    return p


def _attention_other_head_dim(q, k, v, output, sm_scale, is_causal, attention_mask):
    """Head dimensions that are not a multiple of 8 (their rows cannot be addressed by a tensor map:
    TMA wants 16-byte strides) run as the next multiple of 8 with zero columns appended to q, k and v:
    zeros add nothing to q·kᵀ, and the extra output columns (zeros) are dropped. Costs one padded copy
    of the operands; the reference's kernel takes powers of two from 16 (attention.py:122-135), all of
    which run natively."""
    dhead = q.shape[-1]
    assert dhead < 128, f"head dimension above 128 is not supported, got {dhead}"
    extra = (-dhead) % 8
    qp, kp, vp = (torch.nn.functional.pad(t, (0, extra)) for t in (q, k, v))
    padded_out = torch.empty(qp.shape, dtype=output.dtype, device=output.device)
    attention_forward(qp, kp, vp, padded_out, sm_scale, is_causal, attention_mask)
    output.copy_(padded_out[..., :dhead])
    return output


def attention_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    output: torch.Tensor,
    sm_scale: float,
    is_causal: bool = False,
    attention_mask: Optional[torch.Tensor] = None,
):
    """Flash attention on the tcgen05 kernel, written into `output` (which is returned).

    Same contract as the reference's `attention_forward` (attention.py:532-541 →
    Attention.forward :438-529): q [B,H,M,D], k/v [B,H,N,D], all fp16 or all bf16;
    attention_mask additive, broadcastable over batch / heads / rows with last size N; -inf mask
    entries behave as the lowest finite value of the mask dtype; `is_causal` keeps col <= row.
    Head dimensions that are multiples of 8 up to 128 run natively (the kernels compute on 64 or 128
    columns; the tensor maps end at the real head dimension and TMA fills the rest with zeros). Beyond the reference:
    k/v may carry fewer heads than q (grouped-query attention, see `kv_group_of`).
    """
    q, k, v, output, attention_mask = cast_if_autocast(q, k, v, output, attention_mask)
    assert q.shape[-1] == k.shape[-1]
    assert (
        q.dtype == k.dtype == v.dtype == output.dtype
    ), f"All tensors must have the same dtype: {q.dtype}, {k.dtype}, {v.dtype}, {output.dtype}"
    assert q.dtype in [torch.float16, torch.bfloat16], f"Only float16 and bfloat16 are supported, got {q.dtype}"
    assert q.is_cuda, "kernl_b200 ops run on a CUDA (sm_100a) device only"
    batch, heads, m_size, dhead = q.size()
    n_size = k.size(2)
    if dhead % 8 != 0 or dhead > 128:
        return _attention_other_head_dim(q, k, v, output, sm_scale, is_causal, attention_mask)
    if attention_mask is not None:
        _check_mask(attention_mask, batch, heads, m_size, n_size)
        assert attention_mask.dtype in (torch.float16, torch.bfloat16, torch.float32)
    qc, kc, vc = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    p = make_params(qc, kc, vc, output, sm_scale, is_causal, attention_mask)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().kb_attention_fwd(p, _lib.current_stream(q.device)), "attention_forward")
    return output
