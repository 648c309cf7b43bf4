"""The ordered rewrite pipeline applied to each TorchDynamo graph
(reference: src/kernl/optimizer/dynamo_backend.py:25-34)."""
import torch

from kernl_b200.optimizer.attention import (
    fuse_attention_pattern_1,
    fuse_attention_pattern_2,
    fuse_attention_pattern_3,
    fuse_attention_sdpa,
)
from kernl_b200.optimizer.dropout import remove_dropout
from kernl_b200.optimizer.layer_norm import fuse_add_layer_norm, replace_layer_norm, replace_layer_norm_rms
from kernl_b200.optimizer.linear import fuse_parallel_linears, replace_all_linear
from kernl_b200.optimizer.normalizer import normalize_operators, replace_scalar_tensor_constants


def dynamo_backend_ofi(gm: torch.fx.GraphModule, assume_causal=False):
    """Order matters: operators are normalised and dropout removed before the attention patterns
    are looked for, and linears are fused with their activation before bare linears are replaced.
    `assume_causal` sets the causal flag of every attention replacement, on top of whatever
    additive mask the model passes."""
    normalize_operators(gm)
    replace_scalar_tensor_constants(gm)
    remove_dropout(gm)
    fuse_attention_pattern_1(gm, assume_causal)
    fuse_attention_pattern_2(gm, assume_causal)
    fuse_attention_pattern_3(gm, assume_causal)
    fuse_attention_sdpa(gm, assume_causal)
    replace_all_linear(gm)
    fuse_parallel_linears(gm)
    replace_layer_norm(gm)
    fuse_add_layer_norm(gm)
    replace_layer_norm_rms(gm)
    return gm
