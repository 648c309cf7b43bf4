"""`optimize_model`: the one-call entry point (reference: src/kernl/model_optimization.py)."""
from typing import List

import torch

from kernl_b200.optimizer.cuda_graph import cuda_graphs_wrapper, static_inputs_pool
from kernl_b200.optimizer.dynamo_backend import dynamo_backend_ofi


# Module-level on purpose: compiled graphs are then shared by every forward that goes through
# this backend, e.g. the encoder and the decoder of one model (reference: model_optimization.py:25-29).
def _compiler(gm: torch.fx.GraphModule, example_inputs: List[torch.Tensor]):
    dynamo_backend_ofi(gm)
    # Capture is put off to the second call: a model is cut into several graphs, and a graph
    # captured while the first forward is still under way could hold the address of a parameter that
    # a later graph of that forward converts to fp16 in place (tied embedding / output weights).
    return cuda_graphs_wrapper(gm, example_inputs, defer_capture=True)


def optimize_model(model) -> None:
    """Replace `model.forward` by a TorchDynamo-traced version whose attention, linear and
    normalisation sub-graphs call the sm_100a kernels, wrapped in a CUDA graph per input shape.
    The original forward stays available as `model.forward_original`.

        model = AutoModel.from_pretrained(...).eval().cuda()
        optimize_model(model)
        with torch.inference_mode(), torch.autocast("cuda", dtype=torch.float16):
            model(**inputs)

    Same contract as the reference (model_optimization.py:32-66), with the device check moved
    from "Ampere or newer" to "compute capability 10.x": there is no other code path.
    """
    assert torch.cuda.is_available(), "CUDA capacity is required to use Kernl"
    major, _ = torch.cuda.get_device_capability()
    if major != 10:
        raise RuntimeError("GPU compute capability 10.x (Blackwell B200, sm_100a) is required to use kernl_b200")
    assert next(model.parameters()).device.type == "cuda", "Model must be on GPU"
    static_inputs_pool.clear()
    # The rewrites match `call_module` nodes by module type; recent TorchDynamo inlines built-in
    # modules (parameters become graph inputs) unless told otherwise.
    torch._dynamo.config.inline_inbuilt_nn_modules = False
    # One CUDA graph per input shape, as in the reference: every new shape is a new static trace
    # (symbolic sizes would reach the graph wrapper as integer inputs that a captured graph cannot
    # follow), and a generation loop meets one shape per decoded token — far more than TorchDynamo's
    # default of 8 variants per frame (the reference raises the same limit: conftest.py:37-39, tutorial/t5 e2e.ipynb).
    torch._dynamo.config.automatic_dynamic_shapes = False
    torch._dynamo.config.cache_size_limit = max(torch._dynamo.config.cache_size_limit, 512)
    model.forward_original = model.forward

    @torch._dynamo.optimize(_compiler)
    def run(*args, **kwargs):
        return model.forward_original(*args, **kwargs)

    model.forward = run
