"""Tensor-parallel communication for the row-parallel linears: all-reduce + residual add.

`PeerAllReduce` is the B200-native path for the latency-bound decode messages: every rank's GEMM
writes its partial sum into a peer-mapped buffer and ONE kernel of the library
(`kb_allreduce_residual_fwd`) signals, pulls the peers' partials over NVLink with plain loads, adds
the residual and stores the result. Messages above 1 MiB (prefill) go through NCCL
(`torch.distributed`). The peer mapping is plain CUDA IPC (`kb_peer_*`): handles are exchanged with
`all_gather_object`; no NVLS / multimem / multicast object is created.
"""
import ctypes
from typing import Optional

import torch

from kernl_b200 import _lib

MAX_BYTES = 1 << 20
_FLAG_BYTES = 256


class _DevicePtr:
    """Exposes raw device memory to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


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

    def reduce_add_norm(self, partial, residual, weight, eps, ops):
        """x = residual + all_reduce(partial); returns (x, rms_norm(x) * weight). After NCCL the add
        and the norm are one kernel."""
        h, x = ops.add_rms_norm(self.all_reduce(partial), residual, weight, eps)
        return x, h


class PeerAllReduce(NcclAllReduce):
    def __init__(self, rank: int, world: int, device, dtype):
        import torch.distributed as dist

        super().__init__(world)
        assert 1 < world <= 8
        self.rank, self.device, self.dtype = rank, torch.device(device), dtype
        lib = _lib.load()
        self._lib = lib
        with torch.cuda.device(self.device):
            buf, flags = ctypes.c_void_p(), ctypes.c_void_p()
            _lib.check(lib.kb_peer_alloc(MAX_BYTES, ctypes.byref(buf)), "kb_peer_alloc")
            _lib.check(lib.kb_peer_alloc(_FLAG_BYTES, ctypes.byref(flags)), "kb_peer_alloc")
            handles = []
            for p in (buf, flags):
                h = ctypes.create_string_buffer(64)
                _lib.check(lib.kb_peer_export(p, h), "kb_peer_export")
                handles.append(h.raw)
            gathered = [None] * world
            dist.all_gather_object(gathered, handles)
            self.buf_ptrs, self.flag_ptrs, self._opened = [], [], []
            for r in range(world):
                if r == rank:
                    self.buf_ptrs.append(buf.value)
                    self.flag_ptrs.append(flags.value)
                    continue
                for which, dst in ((0, self.buf_ptrs), (1, self.flag_ptrs)):
                    out = ctypes.c_void_p()
                    _lib.check(lib.kb_peer_open(gathered[r][which], ctypes.byref(out)), "kb_peer_open")
                    dst.append(out.value)
                    self._opened.append(out.value)
            self._own = (buf.value, flags.value)
            self.buf = torch.as_tensor(_DevicePtr(buf.value, MAX_BYTES), device=self.device).view(dtype)
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
        return self._launch(partial, residual, None, 0.0)[0]

    def reduce_add_norm(self, partial, residual, weight, eps, ops):
        """All-reduce, residual add and the following RMSNorm in ONE kernel over peer memory."""
        if partial.data_ptr() != self.buf.data_ptr() or partial.shape[-1] > 8192 or partial.shape[-1] % 8:
            return super().reduce_add_norm(partial, residual, weight, eps, ops)
        return self._launch(partial, residual, weight, eps)

    def _launch(self, partial, residual, weight, eps):
        residual = residual.contiguous()
        out = torch.empty_like(residual)
        normed = torch.empty_like(residual) if weight is not None else None
        p = _lib.AllReduceParams()
        if weight is not None:
            p.norm_weight = weight.data_ptr()
            p.norm_out = normed.data_ptr()
            p.cols = partial.shape[-1]
            p.eps = float(eps)
        for r in range(self.world):
            p.partials[r] = self.buf_ptrs[r]
            p.flags[r] = self.flag_ptrs[r]
        p.residual = residual.data_ptr()
        p.out = out.data_ptr()
        p.count = partial.numel()
        p.rank, p.world = self.rank, self.world
        p.dtype = _lib.dtype_code(partial.dtype)
        with torch.cuda.device(self.device):
            _lib.check(self._lib.kb_allreduce_residual_fwd(p, _lib.current_stream(self.device)), "allreduce_residual")
        return out, normed

    def close(self):
        """Unmap the peers' buffers and free this rank's. Call on every rank, between steps, after a
        barrier, with no kernel in flight."""
        torch.cuda.synchronize(self.device)
        try:
            with torch.cuda.device(self.device):
                _lib.device_status()  # a flag wait that expired during this communicator's life shows here
        finally:
            self._release()

    def _release(self):
        for ptr in self._opened:
            self._lib.kb_peer_close(ptr)
        self._opened = []
        for ptr in self._own:
            self._lib.kb_peer_free(ptr)
        self._own = ()
