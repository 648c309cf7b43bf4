"""CPU checks of the oracle itself: against the golden vectors produced by the reference's own
eager functions (tests/golden/make_golden.py), and against an independent tile-by-tile
restatement of the fused kernel's loop."""
import os

import numpy as np
import pytest
import torch

from oracle import kernl_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def attn_golden():
    return np.load(os.path.join(GOLDEN, "attention_reference.npz"))


@pytest.fixture(scope="module")
def norm_golden():
    return np.load(os.path.join(GOLDEN, "norm_reference.npz"))


@pytest.mark.parametrize("name", ["nomask", "pad", "bias", "cross", "d128"])
def test_attention_matches_reference_golden(attn_golden, name):
    g = attn_golden
    q, k, v = (torch.from_numpy(g[f"{name}_{t}"]) for t in "qkv")
    mask = torch.from_numpy(g[f"{name}_mask"]) if f"{name}_mask" in g.files else None
    out = O.attention(q, k, v, float(g[f"{name}_scale"]), False, mask)
    assert torch.allclose(out, torch.from_numpy(g[f"{name}_out"]), atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("name", ["nomask", "pad", "bias", "cross", "d128"])
def test_blockwise_matches_reference_golden(attn_golden, name):
    g = attn_golden
    q, k, v = (torch.from_numpy(g[f"{name}_{t}"]) for t in "qkv")
    mask = torch.from_numpy(g[f"{name}_mask"]) if f"{name}_mask" in g.files else None
    out = O.attention_blockwise(q, k, v, float(g[f"{name}_scale"]), False, mask, block_m=16, block_n=16)
    assert torch.allclose(out, torch.from_numpy(g[f"{name}_out"]), atol=1e-5, rtol=1e-4)


CAUSAL_GOLDEN = ["causal_square", "causal_morekeys", "causal_morequeries", "causal_bias", "causal_pad", "causal_d128"]


@pytest.mark.parametrize("name", CAUSAL_GOLDEN)
def test_causal_matches_reference_golden(attn_golden, name):
    """The causal branch against outputs of the reference's own `attention_reference(is_causal=True)`
    (fixtures made by tests/golden/make_golden.py): dense restatement and tile loop."""
    g = attn_golden
    q, k, v = (torch.from_numpy(g[f"{name}_{t}"]) for t in "qkv")
    mask = torch.from_numpy(g[f"{name}_mask"]) if f"{name}_mask" in g.files else None
    want = torch.from_numpy(g[f"{name}_out"])
    out = O.attention(q, k, v, float(g[f"{name}_scale"]), True, mask)
    assert torch.allclose(out, want, atol=2e-6, rtol=1e-5)
    out = O.attention_blockwise(q, k, v, float(g[f"{name}_scale"]), True, mask, block_m=16, block_n=16)
    assert torch.allclose(out, want, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("m,n", [(1, 24), (33, 33), (40, 17), (17, 40), (129, 257)])
@pytest.mark.parametrize("mask_kind", [None, "bias", "pad"])
def test_causal_oracle_matches_blockwise(m, n, mask_kind):
    """Beyond the golden cases: the dense and the tile-loop restatement agree on more causal
    shapes."""
    torch.manual_seed(0)
    q, k, v = torch.randn(2, 2, m, 64), torch.randn(2, 2, n, 64), torch.randn(2, 2, n, 64)
    mask = None
    if mask_kind == "bias":
        mask = torch.rand(2, 2, m, n)
    elif mask_kind == "pad":
        valid = torch.randint(1, n + 1, (2,))
        mask = torch.where(valid[:, None] > torch.arange(n)[None, :], 0.0, float("-inf")).reshape(2, 1, 1, n)
    a = O.attention(q, k, v, 0.3, True, mask)
    b = O.attention_blockwise(q, k, v, 0.3, True, mask, block_m=32, block_n=32)
    assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)


def test_mask_clamp_keeps_fully_masked_rows_finite():
    q, k, v = torch.randn(1, 1, 4, 64), torch.randn(1, 1, 8, 64), torch.randn(1, 1, 8, 64)
    mask = torch.full((1, 1, 1, 8), float("-inf"), dtype=torch.float16)
    out = O.attention(q, k, v, 1.0, False, mask)
    assert torch.isfinite(out).all()
    # every key is lowered by the same -65504, so the result is the plain softmax of q·k up to the
    # fp32 rounding of (score - 65504), whose ulp is 2^-8
    assert torch.allclose(out, O.attention(q, k, v, 1.0, False, None), atol=2e-2)


@pytest.mark.parametrize("n", [128, 250, 768])
def test_norms_match_reference_golden(norm_golden, n):
    g = norm_golden
    x, w, b = (torch.from_numpy(g[f"n{n}_{t}"]) for t in "xwb")
    assert torch.allclose(O.layer_norm(x, w, b, 1e-5), torch.from_numpy(g[f"n{n}_f_ln"]), atol=2e-5, rtol=1e-5)
    assert torch.allclose(O.rms_norm(x, w, 1e-6), torch.from_numpy(g[f"n{n}_rms"]), atol=2e-5, rtol=1e-5)
    # the reference's naive LayerNorm uses the unbiased variance: same result up to n/(n-1)
    naive = torch.from_numpy(g[f"n{n}_naive_ln"])
    assert (O.layer_norm(x, w, b, 1e-5) - naive).abs().max() < 0.05


@pytest.mark.parametrize("act", ["", "tanh", "gelu", "relu", "fast_gelu", "silu"])
def test_linear_oracle_against_torch(act):
    torch.manual_seed(0)
    x, w, b = torch.randn(9, 40), torch.randn(24, 40) * 0.1, torch.randn(24)
    ref = torch.nn.functional.linear(x, w, b)
    ref = {
        "": lambda z: z, "tanh": torch.tanh, "gelu": torch.nn.functional.gelu, "relu": torch.relu,
        "fast_gelu": lambda z: torch.nn.functional.gelu(z, approximate="tanh"), "silu": torch.nn.functional.silu,
    }[act](ref)
    assert torch.allclose(O.linear(x, w, b, act), ref, atol=1e-5, rtol=1e-5)


def test_kernel_eps_clamp():
    assert O.kernel_eps(1e-12, torch.float16) == 1.6e-5
    assert O.kernel_eps(1e-12, torch.bfloat16) == 1e-12
    assert O.kernel_eps(1e-3, torch.float16) == 1e-3


def test_zero_padding_the_head_dimension_changes_nothing():
    """What the attention front-end relies on for head dimensions other than 64 / 128."""
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(2, 3, 17, 32, generator=g) for _ in range(3))
    mask = torch.rand(2, 1, 1, 17, generator=g)
    want = O.attention(q, k, v, 0.2, True, mask)
    pad = lambda t: torch.nn.functional.pad(t, (0, 32))
    got = O.attention(pad(q), pad(k), pad(v), 0.2, True, mask)
    assert torch.allclose(got[..., :32], want, atol=1e-6) and float(got[..., 32:].abs().max()) == 0.0


# ------------------------------------------------------------------------------------------------
# Llama pieces against vectors from the reference's experimental eager code
# ------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def llama_golden():
    return np.load(os.path.join(GOLDEN, "llama_reference.npz"))


def test_rotary_matches_reference_golden(llama_golden):
    from kernl_b200.llama_tp import apply_rope

    x, cos, sin = (torch.from_numpy(llama_golden[k]) for k in ("rope_x", "rope_cos", "rope_sin"))
    expected = torch.from_numpy(llama_golden["rope_out"])
    assert torch.allclose(O.rotary(x, cos, sin), expected, atol=1e-6, rtol=0)
    # the host-side helper of the decoder (used where no kernel runs) follows the same convention
    assert torch.allclose(apply_rope(x, cos, sin), expected, atol=1e-6, rtol=0)


def test_gated_feed_forward_matches_reference_golden(llama_golden):
    from kernl_b200.implementations.linear_layer import interleave_gate_up

    x, rms_w, w1, w3 = (torch.from_numpy(llama_golden[k]) for k in ("ff_x", "ff_rms_w", "ff_w1", "ff_w3"))
    x_norm = O.rms_norm(x, rms_w, 1e-6)
    assert torch.allclose(x_norm, torch.from_numpy(llama_golden["ff_x_norm"]), atol=1e-6, rtol=0)
    expected = torch.from_numpy(llama_golden["ff_out"])
    assert torch.allclose(O.gated_feed_forward(x_norm, w1, w3), expected, atol=1e-5, rtol=0)
    # the interleaved weight layout the gated GEMM epilogue reads: block 2j = gate rows 8j .. 8j+7,
    # block 2j+1 = the matching up rows; evaluated block-wise it gives the same numbers
    w = interleave_gate_up(w1, w3)
    z = x_norm @ w.t()
    z = z.reshape(z.shape[0], -1, 2, 8)
    out = (torch.nn.functional.silu(z[:, :, 0]) * z[:, :, 1]).reshape(z.shape[0], -1)
    assert torch.allclose(out, expected, atol=1e-5, rtol=0)

