"""The allocation-free decode-attention entry point, kb_attention_decode_fwd_static.

Some hosts of this library cannot hand it a scratch buffer because they have no device allocator of
their own (a plugin that only ever receives tensors from its runtime, or a process whose GPU memory
is already reserved by someone else's pool). For them the library carries a fixed 4 MiB scratch
array; this test calls that entry point through the C ABI, twice in a row on different inputs
(the array keeps the previous call's contents, which must not leak into the next result), and
compares each output with the regular entry point that takes caller-provided scratch. The file
name sorts last on purpose, so a run that stops at the first failure has already run everything
else.
"""
import pytest
import torch

from kernl_b200 import _lib
from kernl_b200.implementations.attention import make_params

pytestmark = pytest.mark.gpu


def _decode_both_ways(lib, q, k, v, mask, sm_scale):
    B, H, M, D = q.shape
    N = k.shape[2]
    stream = _lib.current_stream(q.device)
    # regular entry point: scratch from the caller
    nbytes = lib.kb_attention_decode_scratch_bytes(B, H, M, N, D)
    scratch = torch.empty((nbytes + 3) // 4, dtype=torch.float32, device=q.device)
    expected = torch.empty_like(q)
    _lib.check(lib.kb_attention_decode_fwd(make_params(q, k, v, expected, sm_scale, False, mask), scratch.data_ptr(),
                                           scratch.numel() * 4, stream), "kb_attention_decode_fwd")
    # allocation-free entry point: inputs and output only
    out = torch.empty_like(q)
    _lib.check(lib.kb_attention_decode_fwd_static(make_params(q, k, v, out, sm_scale, False, mask), stream),
               "kb_attention_decode_fwd_static")
    torch.cuda.synchronize()
    return out, expected


def test_static_scratch_entry_point_matches_regular_one(lib):
    from oracle import kernl_oracle as O

    assert lib.kb_attention_decode_static_max_bytes() == 4 << 20
    g = torch.Generator().manual_seed(0)
    # two calls in a row; the second is smaller and masked, so stale partial results of the first
    # call sit in the array right behind the slots the second call uses
    cases = [
        (5, 20, 1, 1500, 64, torch.float16, False),
        (2, 3, 1, 700, 128, torch.bfloat16, True),
    ]
    for (B, H, M, N, D, dtype, with_mask) in cases:
        q = torch.randn((B, H, M, D), generator=g).to(dtype).cuda()
        k = torch.randn((B, H, N, D), generator=g).to(dtype).cuda()
        v = torch.randn((B, H, N, D), generator=g).to(dtype).cuda()
        mask = torch.rand((B, H, M, N), generator=g).to(dtype).cuda() if with_mask else None
        out, expected = _decode_both_ways(lib, q, k, v, mask, D ** -0.5)
        # same kernels, same order of operations: the results agree to the tolerance of this
        # build's tests (they are in fact bit-identical)
        O.assert_parity(out, expected, max_abs=1e-2 if dtype == torch.float16 else 3e-2)
        O.assert_parity(out, O.attention(q, k, v, D ** -0.5, False, mask), max_abs=1e-2 if dtype == torch.float16 else 3e-2)


def test_static_scratch_entry_point_rejects_oversized_problems(lib):
    """Beyond the fixed 4 MiB the call must refuse with KB_ERR_TOO_LARGE and launch nothing."""
    B, H, M, N, D = 64, 32, 1, 4096, 128
    assert lib.kb_attention_decode_scratch_bytes(B, H, M, N, D) > lib.kb_attention_decode_static_max_bytes()
    q = torch.zeros((B, H, M, D), dtype=torch.float16, device="cuda")
    kv = torch.zeros((1, 1, 1, D), dtype=torch.float16, device="cuda").expand(B, H, N, D)  # never read
    out = torch.full_like(q, 7.0)
    status = lib.kb_attention_decode_fwd_static(make_params(q, kv, kv, out, 1.0, False, None), _lib.current_stream(q.device))
    assert status == -6
    assert "maximum" in _lib.status_str(status)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())
