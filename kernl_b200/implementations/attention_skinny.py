"""Decode-shape attention front-end (reference: src/kernl/implementations/attention_skinny.py)."""
from typing import Optional

import torch

from kernl_b200 import _lib
from kernl_b200.implementations._autocast import cast_if_autocast
from kernl_b200.implementations.attention import _check_mask, make_params


def skinny_attention_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    output: torch.Tensor,
    sm_scale: float,
    is_causal: bool = False,
    attention_mask: Optional[torch.Tensor] = None,
    kv_len: Optional[torch.Tensor] = None,
):
    """Split-KV attention for few query rows and many keys, written into `output`.

    Same contract as the reference's `skinny_attention_forward` (attention_skinny.py:539-548 →
    SkinnyAttention.forward :369-536). The scratch for the per-chunk partial results is taken
    from the torch caching allocator per call, as the reference does (:416-441), which keeps the
    call capturable in a CUDA graph after one warm-up. Beyond the reference: k/v may carry fewer
    heads than q (grouped-query attention), and `kv_len` — a one-element int64 tensor on the device —
    says how many of the keys exist (a KV cache filled up to that slot): keys beyond it are neither
    loaded nor scored, and because the kernel reads the count, a captured graph follows a growing
    cache (the `start_position` of experimental/llama-v2/kernel/fused_kernel_attention.py:30,63,76).
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
    assert dhead <= 256, "head dimension above 256 is not supported"
    if attention_mask is not None:
        _check_mask(attention_mask, batch, heads, m_size, n_size)
    lib = _lib.load()
    nbytes = lib.kb_attention_decode_scratch_bytes(batch, heads, m_size, n_size, dhead)
    scratch = torch.empty((max(nbytes, 4) + 3) // 4, dtype=torch.float32, device=q.device)
    if kv_len is not None:
        assert kv_len.dtype == torch.int64 and kv_len.numel() == 1 and kv_len.device == q.device
    p = make_params(q, k, v, output, sm_scale, is_causal, attention_mask, kv_len)
    with torch.cuda.device(q.device):
        _lib.check(
            lib.kb_attention_decode_fwd(p, scratch.data_ptr(), scratch.numel() * 4, _lib.current_stream(q.device)),
            "skinny_attention_forward",
        )
    return output
