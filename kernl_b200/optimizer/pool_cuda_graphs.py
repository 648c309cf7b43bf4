"""Static-address arena for CUDA-graph inputs (reference: src/kernl/optimizer/pool_cuda_graphs.py).

A captured graph reads its inputs from fixed device addresses, so every call first copies the
caller's tensors into an arena at deterministic offsets. The arena is a flat int8 tensor; tensors
are bump-allocated with 8-byte alignment and viewed with their own dtype, sizes and strides.
"""
import torch


def get_aligned_size(t: torch.Tensor, alignment: int = 8) -> int:
    """Bytes of t's storage rounded up to `alignment` (reference: pool_cuda_graphs.py:55-64)."""
    nbytes = len(t.untyped_storage())
    return -(-nbytes // alignment) * alignment


class CudaGraphPool:
    """Bump allocator over one int8 buffer (reference: pool_cuda_graphs.py:4-52)."""

    def __init__(self, size, device="cuda"):
        assert (size > 0) and (size % 8 == 0), f"Size must be positive and multiple of 8, got {size}"
        self.pool: torch.Tensor = torch.empty(size, dtype=torch.int8, device=device)
        self.size = len(self.pool.untyped_storage())
        self.offset = 0

    def can_store(self, t: torch.Tensor) -> bool:
        return (self.pool.device == t.device) and (self.size - self.offset >= get_aligned_size(t))

    def copy_to_pool(self, t: torch.Tensor) -> torch.Tensor:
        """Copy t into the arena; the returned tensor is a view of the arena with t's geometry.
        Zero strides (expanded tensors) become 1 so that the copy has distinct elements to write
        (reference: pool_cuda_graphs.py:31)."""
        assert t.device == self.pool.device
        assert self.can_store(t)
        strides = tuple(s if s > 0 else 1 for s in t.stride())
        view = torch.as_strided(
            self.pool.view(t.dtype), size=t.size(), stride=strides, storage_offset=self.offset // t.element_size()
        )
        view.copy_(t)
        self.offset += get_aligned_size(t)
        return view

    def reset(self):
        self.offset = 0
