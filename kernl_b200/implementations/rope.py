"""Rotary embedding + KV-cache write front-end (kb_rope_kv_write)."""
from typing import Optional, Union

import torch

from kernl_b200 import _lib


def rope_kv_write(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                  pos: Union[int, torch.Tensor], batch: int, seq: int) -> torch.Tensor:
    """qkv: [batch*seq, 3*H*D] (fused projection output, laid out [3][H][D] per token);
    k_cache / v_cache: [batch, H, max_seq, D] contiguous; cos / sin: fp32 [max_seq, D/2];
    pos: start position (int, or a 1-element int64 device tensor for captured decode steps).
    Returns q rotated, [batch, seq, H, D]; k (rotated) and v are written into the caches."""
    B, H, max_seq, D = k_cache.shape
    assert B == batch and v_cache.shape == k_cache.shape and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert qkv.is_contiguous() and qkv.shape == (batch * seq, 3 * H * D) and qkv.dtype == k_cache.dtype
    assert cos.dtype == torch.float32 and cos.is_contiguous() and cos.shape == (max_seq, D // 2) and sin.shape == cos.shape
    q_out = torch.empty((batch, seq, H, D), dtype=qkv.dtype, device=qkv.device)
    p = _lib.RopeParams(
        qkv=qkv.data_ptr(), q_out=q_out.data_ptr(), k_cache=k_cache.data_ptr(), v_cache=v_cache.data_ptr(),
        cos=cos.data_ptr(), sin=sin.data_ptr(),
        pos_dev=pos.data_ptr() if isinstance(pos, torch.Tensor) else None,
        pos_host=0 if isinstance(pos, torch.Tensor) else int(pos),
        B=batch, S=seq, H=H, D=D, max_seq=max_seq, dtype=_lib.dtype_code(qkv.dtype),
    )
    if isinstance(pos, torch.Tensor):
        assert pos.dtype == torch.int64 and pos.numel() == 1 and pos.device == qkv.device
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.load().kb_rope_kv_write(p, _lib.current_stream(qkv.device)), "rope_kv_write")
    return q_out
