"""Attention for operands that live in pinned HOST memory, as a two-deep pipeline.

A caller that keeps q, k, v and the mask on the host (a pre-processing thread fills pinned buffers,
a post-processing thread reads the result) pays, per call, the host→device copy of the operands,
the kernel, and the device→host copy of the result. At the headline shape ([8, 12, 512, 64] fp16:
18.9 MB in, 6.3 MB out) the copies take more than ten times as long as the kernel, so what matters
is that the two copy directions — separate DMA engines on a full-duplex link — run at the same
time: the result of call i goes back while the operands of call i + 1 come in.

    pipe = HostAttentionPipeline(q_shape, k_shape, mask_shape, dtype, device)
    for batch in batches:                       # pinned host tensors
        pipe.submit(hq, hk, hv, hmask, hout, sm_scale)   # returns at once
    pipe.synchronize()                          # every hout is now valid

`submit` enqueues on two streams of its own (operands + kernel on one, results on the other) and two
sets of device buffers; events order the reuse of a set (the operands of call i + 2 wait for the
kernel of call i, the kernel of call i + 2 waits for the result copy of call i). The kernel call
is the package's `attention_forward` (reference contract: src/kernl/implementations/attention.py:532-541).
"""
from typing import Optional, Sequence

import torch

from kernl_b200.implementations.attention import attention_forward


class HostAttentionPipeline:
    def __init__(self, q_shape: Sequence[int], kv_shape: Sequence[int], mask_shape: Optional[Sequence[int]],
                 dtype: torch.dtype, device, depth: int = 2):
        assert depth >= 1
        self.device = torch.device(device)
        assert self.device.type == "cuda", "kernl_b200 ops run on a CUDA (sm_100a) device only"
        self.depth = depth
        self.sets = []
        for _ in range(depth):
            self.sets.append({
                "q": torch.empty(tuple(q_shape), dtype=dtype, device=self.device),
                "k": torch.empty(tuple(kv_shape), dtype=dtype, device=self.device),
                "v": torch.empty(tuple(kv_shape), dtype=dtype, device=self.device),
                "mask": torch.empty(tuple(mask_shape), dtype=dtype, device=self.device) if mask_shape is not None else None,
                "o": torch.empty(tuple(q_shape), dtype=dtype, device=self.device),
                "kernel_done": torch.cuda.Event(),
                "result_out": torch.cuda.Event(),
                "used": False,
            })
        self.in_stream = torch.cuda.Stream(self.device)
        self.out_stream = torch.cuda.Stream(self.device)
        self.calls = 0

    def submit(self, hq: torch.Tensor, hk: torch.Tensor, hv: torch.Tensor, hmask: Optional[torch.Tensor],
               hout: torch.Tensor, sm_scale: float, is_causal: bool = False) -> None:
        """Enqueue one attention over host operands; `hout` (pinned) is valid after `synchronize()`
        — or after any later `submit` that reuses the same device set has been enqueued and the
        out stream has drained. Host tensors must stay untouched until then."""
        for t in (hq, hk, hv, hout) + ((hmask,) if hmask is not None else ()):
            assert t.device.type == "cpu" and t.is_pinned(), "host operands must be pinned for asynchronous copies"
        s = self.sets[self.calls % self.depth]
        assert (hmask is None) == (s["mask"] is None), "the pipeline was built with / without a mask"
        self.calls += 1
        with torch.cuda.stream(self.in_stream):
            if s["used"]:
                # the result of the call that last used this set must have left before o is rewritten
                # (q/k/v are safe already: that call's kernel ran earlier on this very stream)
                self.in_stream.wait_event(s["result_out"])
            s["q"].copy_(hq, non_blocking=True)
            s["k"].copy_(hk, non_blocking=True)
            s["v"].copy_(hv, non_blocking=True)
            if hmask is not None:
                s["mask"].copy_(hmask, non_blocking=True)
            attention_forward(s["q"], s["k"], s["v"], s["o"], sm_scale, is_causal, s["mask"])
            s["kernel_done"].record(self.in_stream)
        with torch.cuda.stream(self.out_stream):
            self.out_stream.wait_event(s["kernel_done"])
            hout.copy_(s["o"], non_blocking=True)
            s["result_out"].record(self.out_stream)
        s["used"] = True

    def synchronize(self) -> None:
        self.in_stream.synchronize()
        self.out_stream.synchronize()
