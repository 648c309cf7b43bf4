"""kernl_b200: B200 (sm_100a) kernels behind the ELS-RD/kernl operator API.

The public surface mirrors the reference package `kernl`:
  kernl_b200.model_optimization.optimize_model
  kernl_b200.optimizer.{dynamo_backend, attention, linear, layer_norm, dropout, normalizer, cuda_graph, pool_cuda_graphs}
  kernl_b200.implementations.{attention, attention_skinny, linear_layer, layer_norm}
  kernl_b200.utils.extended_matcher.replace_pattern
Every op dispatches to the hand-written CUDA library libkernl_b200.so through its C ABI
(include/kernl_b200.h); there is no Triton, no PyTorch and no CPU fallback for the ops.
"""
__version__ = "0.1.0"
