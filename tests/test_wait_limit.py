"""A bounded device-side wait that runs out: the kernel gives up, records it, and returns.

One GPU, one kernel, no fault: rank 0 of a two-rank all-reduce is launched alone with a wait limit
of a few thousand cycles, so the flag that its (absent) peer would set never arrives and the wait
expires. The kernel neither traps nor hangs; the host finds KB_ERR_TIMEOUT in the status word,
kernels launched before the word is read do no work, and after the read everything works again.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _params(bufs, flags, residual, out, rank=0):
    from kernl_b200 import _lib

    p = _lib.AllReduceParams()
    for r in range(2):
        p.partials[r] = bufs[r].data_ptr()
        p.flags[r] = flags[r].data_ptr()
    p.residual, p.out, p.count = residual.data_ptr(), out.data_ptr(), out.numel()
    p.rank, p.world, p.dtype = rank, 2, _lib.KB_BF16
    return p


def test_expired_wait_sets_the_status_word_and_the_library_recovers(lib):
    from kernl_b200 import _lib
    from kernl_b200.implementations.attention import attention_forward
    from oracle import kernl_oracle as O

    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(0)
    bufs = [torch.randn(4096, generator=g).bfloat16().to(dev) for _ in range(2)]
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]  # "rank 1" is just more memory here
    residual = torch.randn(4096, generator=g).bfloat16().to(dev)
    out = torch.zeros(4096, dtype=torch.bfloat16, device=dev)
    stream = _lib.current_stream(dev)
    _lib.device_status()
    assert lib.kb_debug_wait_limit(20000, 20000) == 0
    try:
        # rank 0 alone: nobody sets its "ready" flag, the wait of ~20 000 cycles runs out
        assert lib.kb_allreduce_residual_fwd(_params(bufs, flags, residual, out), stream) == 0
        # a kernel launched while the word is set skips its work
        q = torch.randn((1, 2, 128, 64), generator=g).half().to(dev)
        sentinel = torch.full_like(q, 7.0)
        attention_forward(q, q, q, sentinel, 0.125, False, None)
        with pytest.raises(RuntimeError, match="wait expired") as info:
            _lib.device_status()
        word = [int(x) for x in info.value.args[0].split("word = ")[1].strip("[]").split(",")]
        assert word[0] == 1 and 500 <= word[1] < 600, word  # the all-reduce's flag waits are sites 500..579
        assert torch.equal(sentinel, torch.full_like(q, 7.0)), "a kernel ran although a wait had expired"
    finally:
        assert lib.kb_debug_wait_limit(0, 0) == 0  # defaults back
    assert _lib.device_status()[0] == 0
    # after the read: ordinary kernels work again ...
    fresh = attention_forward(q, q, q, torch.empty_like(q), 0.125, False, None)
    O.assert_parity(fresh, O.attention(q.cpu(), q.cpu(), q.cpu(), 0.125))
    # ... and so does the all-reduce once its peer's flags arrive. The peer is played by the host:
    # the call that gave up closed epoch 1, so the next one waits for 2 in "ready" and "done".
    assert int(flags[0][16]) == 1
    flags[0][1] = 2
    flags[0][8 + 1] = 2
    torch.cuda.synchronize()
    assert lib.kb_allreduce_residual_fwd(_params(bufs, flags, residual, out), stream) == 0
    assert _lib.device_status()[0] == 0
    want = (bufs[0].float() + bufs[1].float() + residual.float()).bfloat16()
    assert torch.equal(out, want)
