"""The ordered rewrite pipeline applied to each TorchDynamo graph
(reference: src/kernl/optimizer/dynamo_backend.py:25-34)."""
import torch

from kernl_b200.optimizer.attention import (
    fuse_attention_pattern_1,
    fuse_attention_pattern_2,
    fuse_attention_pattern_3,
    fuse_attention_sdpa,
    fuse_repeat_kv,
)
from kernl_b200.optimizer.dropout import remove_dropout
from kernl_b200.optimizer.layer_norm import (
    fuse_add_layer_norm,
    fuse_add_rms_norm,
    replace_layer_norm,
    replace_layer_norm_rms,
    replace_rms_norm_any_eps,
)
from kernl_b200.optimizer.linear import fuse_gated_feed_forward, fuse_parallel_linears, replace_all_linear
from kernl_b200.optimizer.normalizer import normalize_operators, replace_scalar_tensor_constants


def rewrite_passes(assume_causal: bool):
    """The passes in the order they run. Operators are normalised and dropout removed before the
    attention patterns are looked for; linears are fused with their activation before bare linears
    are replaced; gate/up pairs of gated feed-forwards are merged and what is left is stacked; the
    residual add is folded into a LayerNorm / RMSNorm only once the norm itself has been replaced."""
    attention = [fuse_attention_pattern_1, fuse_attention_pattern_2, fuse_attention_pattern_3, fuse_attention_sdpa]
    return (
        [normalize_operators, replace_scalar_tensor_constants, remove_dropout]
        + [lambda gm, rewrite=rewrite: rewrite(gm, assume_causal) for rewrite in attention]
        + [fuse_repeat_kv]
        + [replace_all_linear, fuse_gated_feed_forward, fuse_parallel_linears]
        + [replace_layer_norm, fuse_add_layer_norm, replace_layer_norm_rms, replace_rms_norm_any_eps, fuse_add_rms_norm]
    )


def dynamo_backend_ofi(gm: torch.fx.GraphModule, assume_causal=False):
    """Rewrites one TorchDynamo graph in place and returns it. `assume_causal` sets the causal flag
    of every attention replacement, on top of whatever additive mask the model passes."""
    for rewrite in rewrite_passes(assume_causal):
        rewrite(gm)
    return gm
