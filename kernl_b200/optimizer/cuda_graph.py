"""CUDA-graph capture wrapper (reference: src/kernl/optimizer/cuda_graph.py).

Same semantics as the reference: the callable is captured once for the shapes of its example
inputs; every call copies the new inputs into a static arena (first-fit-decreasing bin packing
over a global list of pools) and replays the graph; the outputs are static tensors that the next
call overwrites, returned as a list (callers index [0]). The reference goes through
`torch._inductor.compile_fx.cudagraphify_impl`; this implementation captures with
`torch.cuda.CUDAGraph` directly: warm-up on a side stream, capture, replay.
"""
import math
from typing import Callable, Iterable, Optional, Union

import torch
from torch._subclasses import FakeTensor

from kernl_b200.optimizer.pool_cuda_graphs import CudaGraphPool, get_aligned_size

static_inputs_pool = []


def get_pool_size(inputs: list, existing_pools: list) -> int:
    """Size of a new pool: at least the sum of the aligned inputs and at least the largest
    existing pool; below 1 GiB rounded up to a power of two so that small pools stay reusable
    (reference: cuda_graph.py:29-44)."""
    size = sum(get_aligned_size(p) for p in inputs)
    size = max([size] + [p.size for p in existing_pools])
    if size < 1024 * 1024 * 1024:
        size = 2 ** math.ceil(math.log2(size))
    return max(size, 8)


def argsort(iterable: Iterable, key: Callable) -> list:
    """Indices that sort `iterable` by `key` (stable) (reference: cuda_graph.py:47-54)."""
    return [i for i, _ in sorted(enumerate(iterable), key=lambda pair: key(pair[1]))]


def prepare_inputs(inputs: list, pools: list, static_input_idxs: Iterable[int] = ()) -> list:
    """Copy `inputs` into the pools and return the copies, in input order.

    Deterministic, so that the same shapes always land on the same addresses: pools are reset and
    sorted by size ascending, inputs are visited by storage size ascending, each goes into the
    first pool with room; the leftovers share one new pool (reference: cuda_graph.py:57-100).
    Inputs named by `static_input_idxs` are passed through untouched: they take no room in the
    pools and are not copied (see `cuda_graphs_wrapper`).
    """
    for p in pools:
        p.reset()
    pools.sort(key=lambda p: p.size)
    static = set(static_input_idxs)
    order = [i for i in argsort(inputs, key=lambda t: t.untyped_storage().size()) if i not in static]
    copies: list = [inputs[i] if i in static else None for i in range(len(inputs))]
    leftovers = []
    for idx in order:
        t = inputs[idx]
        for pool in pools:
            if pool.can_store(t):
                copies[idx] = pool.copy_to_pool(t)
                break
        else:
            leftovers.append(idx)
    if leftovers:
        new_pool = CudaGraphPool(
            get_pool_size([inputs[i] for i in leftovers], existing_pools=pools), device=inputs[leftovers[0]].device
        )
        pools.append(new_pool)
        for idx in leftovers:
            assert new_pool.can_store(inputs[idx])
            copies[idx] = new_pool.copy_to_pool(inputs[idx])
    return copies


def _capture(model: Callable, static_inputs: list) -> Callable:
    """Warm up on a side stream, capture one graph, return a replay function."""
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        model(*static_inputs)
    side.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        static_outputs = model(*static_inputs)
    if not isinstance(static_outputs, (list, tuple)):
        static_outputs = (static_outputs,)
    static_outputs = list(static_outputs)

    def replay():
        graph.replay()
        return static_outputs

    # The captured graph holds device ADDRESSES, not references: everything it reads must outlive
    # it. The rewritten GraphModule owns tensors that exist nowhere else (stacked / transposed /
    # interleaved weights built by the rewrites), and nothing else may be holding it once the
    # backend has returned — without this reference a garbage collection frees those weights and
    # later replays read whatever was allocated in their place.
    replay.keep_alive = (model, static_inputs)
    return replay


def _static_idxs(inputs, static_input_idxs) -> tuple:
    """Inputs that keep their address from call to call: those the caller names, and every
    `torch.nn.Parameter` (weights that TorchDynamo lifts into graph inputs)."""
    named = set(static_input_idxs or ())
    assert all(0 <= i < len(inputs) for i in named), f"static_input_idxs out of range: {sorted(named)}"
    params = {i for i, t in enumerate(inputs) if isinstance(t, torch.nn.Parameter)}
    return tuple(sorted(named | params))


def _check_static(args, static, addresses) -> None:
    for i in static:
        assert args[i].data_ptr() == addresses[i], (
            f"input {i} was declared static (captured by address) but arrived at another address")


def cuda_graphs_wrapper(model: Callable, inputs: Union[list, tuple], static_input_idxs: Optional[Iterable[int]] = None,
                        defer_capture: Optional[bool] = None) -> Callable:
    """Run `model` through a CUDA graph (reference: cuda_graph.py:103-138).

    With real example inputs the graph is captured now (after one extra eager call, because
    kernels may mutate their inputs during warm-up). With FakeTensor inputs, or when the caller
    asks for it (`defer_capture=True`: `optimize_model` does, whatever kind of example inputs
    TorchDynamo hands over), the first real call runs eagerly and the second one captures, with the
    RNG state preserved around warm-up and capture.

    The reference copies every input into the arena on every call (cuda_graph.py:115-119), which
    for a decoder means copying its whole KV cache per generated token. Here the inputs listed in
    `static_input_idxs` — large tensors whose address does not change between calls, such as a KV
    cache updated in place — and all `torch.nn.Parameter` inputs are captured by address instead:
    no arena space, no per-call copy. Passing a different tensor at such a position later raises
    an AssertionError (the graph would silently read the old one).
    """
    assert isinstance(inputs, (list, tuple))
    if any(not isinstance(inp, torch.Tensor) for inp in inputs):
        # A graph traced with symbolic sizes takes integers as inputs: one capture cannot serve the
        # shapes it stands for. Such a graph runs as it is (`optimize_model` asks TorchDynamo for
        # static shapes, so this is a safety net, not the normal path).
        return model
    if defer_capture is None:
        defer_capture = any(isinstance(inp, FakeTensor) for inp in inputs)
    assert defer_capture or not any(isinstance(inp, FakeTensor) for inp in inputs), "FakeTensor inputs cannot be captured now"
    if not defer_capture:
        static = _static_idxs(inputs, static_input_idxs)
        addresses = {i: inputs[i].data_ptr() for i in static}
        static_inputs = prepare_inputs(inputs=list(inputs), pools=static_inputs_pool, static_input_idxs=static)
        model(*static_inputs)
        replay = _capture(model, static_inputs)

        def run_now(*args):
            _check_static(args, static, addresses)
            prepare_inputs(inputs=list(args), pools=static_inputs_pool, static_input_idxs=static)
            return replay()

        return run_now

    replay: Optional[Callable] = None
    static: tuple = ()
    addresses: dict = {}
    calls = 0

    def run(*new_inputs):
        nonlocal replay, static, addresses, calls
        calls += 1
        if calls == 1:
            # The first call runs eagerly and captures nothing. A model is usually cut into several
            # graphs, and the wrappers convert fp32 parameters to fp16 in place the first time they
            # run (optimizer/linear.py, optimizer/layer_norm.py): a graph captured during the first
            # forward would keep the address of a parameter that a LATER graph of the same forward
            # replaces (tied embedding / output weights), and read freed memory on replay. After
            # one whole forward every parameter has its final storage.
            return model(*new_inputs)
        if replay is None:
            static = _static_idxs(new_inputs, static_input_idxs)
            addresses = {i: new_inputs[i].data_ptr() for i in static}
        else:
            _check_static(new_inputs, static, addresses)
        static_inputs = prepare_inputs(inputs=list(new_inputs), pools=static_inputs_pool, static_input_idxs=static)
        if replay is None:
            cpu_state = torch.get_rng_state()
            cuda_state = torch.cuda.get_rng_state()
            model(*static_inputs)
            replay = _capture(model, static_inputs)
            torch.set_rng_state(cpu_state)
            torch.cuda.set_rng_state(cuda_state)
        return replay()

    return run
