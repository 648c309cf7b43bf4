"""Tensor-parallel communication for the row-parallel linears: all-reduce + residual add.

`PeerAllReduce` is the B200-native path for the latency-bound decode messages: every rank's GEMM
writes its partial sum into a symmetric (peer-mapped) buffer and ONE kernel of the library
(`kb_allreduce_residual_fwd`) signals, pulls the peers' partials over NVLink with plain loads, adds
the residual and stores the result. Messages above 1 MiB (prefill) fall back to NCCL through
`torch.distributed`. Symmetric memory comes from `torch.distributed._symmetric_memory` (allocation
and handle exchange only — no kernel of that module is called); NVLS / multimem is not used.
"""
from typing import Optional

import torch

from kernl_b200 import _lib

MAX_BYTES = 1 << 20


class NcclAllReduce:
    """Baseline: NCCL all-reduce, then the residual add as a separate elementwise op."""

    def __init__(self, world: int):
        self.world = world

    def partial_buffer(self, rows: int, cols: int, dtype, device) -> Optional[torch.Tensor]:
        return None  # the GEMM allocates its own output

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t

    def reduce_add(self, partial: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        return residual + self.all_reduce(partial)


class PeerAllReduce(NcclAllReduce):
    def __init__(self, rank: int, world: int, device, dtype, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        super().__init__(world)
        assert 1 < world <= 8
        self.rank, self.device, self.dtype = rank, torch.device(device), dtype
        group = group if group is not None else dist.group.WORLD
        self.buf = symm_mem.empty(MAX_BYTES // 2, dtype=dtype, device=self.device)
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=self.device)
        self.flags.zero_()
        torch.cuda.synchronize(self.device)
        self._buf_handle = symm_mem.rendezvous(self.buf, group)
        self._flag_handle = symm_mem.rendezvous(self.flags, group)
        self.buf_ptrs = [int(p) for p in self._buf_handle.buffer_ptrs]
        self.flag_ptrs = [int(p) for p in self._flag_handle.buffer_ptrs]
        dist.barrier()

    def partial_buffer(self, rows: int, cols: int, dtype, device) -> Optional[torch.Tensor]:
        """Where the GEMM should write its partial result, or None when the message is too large
        for the one-shot kernel."""
        if rows * cols * 2 > MAX_BYTES or (rows * cols) % 8 != 0 or dtype != self.dtype:
            return None
        return self.buf[: rows * cols].view(rows, cols)

    def reduce_add(self, partial: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        if partial.data_ptr() != self.buf.data_ptr():
            return super().reduce_add(partial, residual)
        out = torch.empty_like(residual)
        p = _lib.AllReduceParams()
        for r in range(self.world):
            p.partials[r] = self.buf_ptrs[r]
            p.flags[r] = self.flag_ptrs[r]
        p.residual = residual.data_ptr()
        p.out = out.data_ptr()
        p.count = partial.numel()
        p.rank, p.world = self.rank, self.world
        p.dtype = _lib.dtype_code(partial.dtype)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().kb_allreduce_residual_fwd(p, _lib.current_stream(self.device)), "allreduce_residual")
        return out
