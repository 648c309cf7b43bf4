"""Generates tests/golden/*.npz from the reference's own eager functions.

Run where the reference tree is checked out and point KERNL_REFERENCE_ROOT at it: it imports `attention_reference`, `pytorch_naive_layernorm` and
`pytorch_naive_rmsnorm` from the reference's sources, evaluates them on seeded CPU inputs and
stores inputs and outputs. The fixtures are small (a few hundred KB in total) and committed; the
tests only read the .npz files, never the reference tree.

The Llama pieces (RMSNorm, rotary embedding on interleaved pairs, gated feed-forward) come from the
reference's experimental eager code, `experimental/llama-v2/kernel/pytorch_reference.py`
(`rms_norm_pytorch`, `apply_rotary_emb_pytorch`), loaded by file path; the feed-forward is composed
from `rms_norm_pytorch` exactly as `ff_pytorch` in `fused_kernel_ff.py:130-134` composes it (that
file runs Triton kernels at import and cannot be loaded on a CPU-only box).

The causal branch of `attention_reference` builds its triangular mask with a literal
`device="cuda"` (src/kernl/implementations/attention.py:57). The function is still run unmodified:
a `TorchFunctionMode` redirects that one factory call's `device="cuda"` to the CPU, everything else
(the masking rule `row >= col`, top-left aligned when M != N; the order scale -> mask -> causal ->
softmax) is the reference's own code. Cases: square, more keys than queries, more queries than
keys, with an additive bias, with a padding mask, and head dimension 128.

Not covered (and why): the reference's `linear_layer` module does not import under the installed
Triton (`triton.ops` is gone), and its tests use plain `F.linear` + activation as ground truth anyway.
"""
import os
import sys

import numpy as np
import torch
from torch.overrides import TorchFunctionMode

REF_ROOT = os.environ.get("KERNL_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference"))
sys.path.insert(0, os.path.join(REF_ROOT, "src"))
HERE = os.path.dirname(os.path.abspath(__file__))


class _CudaFactoriesOnCpu(TorchFunctionMode):
    """Runs factory calls that name `device="cuda"` on the CPU (this box has no GPU)."""

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = dict(kwargs or {})
        if kwargs.get("device") == "cuda":
            kwargs["device"] = "cpu"
        return func(*args, **kwargs)


def main():
    from kernl.implementations.attention import attention_reference
    from kernl.implementations.layer_norm import pytorch_naive_layernorm, pytorch_naive_rmsnorm

    # ---- attention, non-causal: no mask / broadcast padding mask / full bias mask / row-broadcast
    cases = {}
    g = torch.Generator().manual_seed(0)
    for name, (B, H, M, N, D, kind, scale) in {
        "nomask": (2, 3, 33, 33, 64, None, 0.3),
        "pad": (2, 2, 40, 40, 64, "pad", 0.125),
        "bias": (1, 2, 24, 50, 64, "bias", 0.3),
        "cross": (1, 8, 1, 24, 64, "rowvec", 1.0),
        "d128": (1, 2, 17, 29, 128, "bias", 0.0883883),
    }.items():
        q = torch.randn(B, H, M, D, generator=g)
        k = torch.randn(B, H, N, D, generator=g)
        v = torch.randn(B, H, N, D, generator=g)
        mask = None
        if kind == "pad":
            valid = torch.randint(1, N, (B,), generator=g)
            mask = torch.where(valid[:, None] > torch.arange(N)[None, :], 0.0, float("-inf")).reshape(B, 1, 1, N)
        elif kind == "bias":
            mask = torch.rand(B, H, M, N, generator=g)
        elif kind == "rowvec":
            mask = torch.rand(B, H, 1, N, generator=g)
        out = attention_reference(q, k, v, torch.empty_like(q), scale, False, mask)
        cases[f"{name}_q"], cases[f"{name}_k"], cases[f"{name}_v"] = q.numpy(), k.numpy(), v.numpy()
        if mask is not None:
            cases[f"{name}_mask"] = mask.numpy()
        cases[f"{name}_scale"] = np.float32(scale)
        cases[f"{name}_out"] = out.numpy()
    # ---- attention, causal branch (own generator: the arrays above keep their values)
    gc = torch.Generator().manual_seed(1)
    for name, (B, H, M, N, D, kind, scale) in {
        "causal_square": (2, 2, 48, 48, 64, None, 0.125),
        "causal_morekeys": (1, 3, 20, 45, 64, None, 0.3),
        "causal_morequeries": (1, 2, 45, 20, 64, None, 0.3),
        "causal_bias": (1, 2, 33, 33, 64, "bias", 0.125),
        "causal_pad": (2, 2, 40, 40, 64, "pad", 0.125),
        "causal_d128": (1, 2, 37, 37, 128, None, 0.0883883),
    }.items():
        q = torch.randn(B, H, M, D, generator=gc)
        k = torch.randn(B, H, N, D, generator=gc)
        v = torch.randn(B, H, N, D, generator=gc)
        mask = None
        if kind == "pad":
            valid = torch.randint(1, N, (B,), generator=gc)
            mask = torch.where(valid[:, None] > torch.arange(N)[None, :], 0.0, float("-inf")).reshape(B, 1, 1, N)
        elif kind == "bias":
            mask = torch.rand(B, H, M, N, generator=gc)
        with _CudaFactoriesOnCpu():
            out = attention_reference(q, k, v, torch.empty_like(q), scale, True, mask)
        cases[f"{name}_q"], cases[f"{name}_k"], cases[f"{name}_v"] = q.numpy(), k.numpy(), v.numpy()
        if mask is not None:
            cases[f"{name}_mask"] = mask.numpy()
        cases[f"{name}_scale"] = np.float32(scale)
        cases[f"{name}_out"] = out.numpy()
    np.savez_compressed(os.path.join(HERE, "attention_reference.npz"), **cases)

    # ---- norms: x = -20 + 0.5*randn as in the reference's test (test/test_layer_norm.py:58)
    cases = {}
    for n in (128, 250, 768):
        x = -20 + 0.5 * torch.randn(16, n, generator=g)
        w = torch.rand(n, generator=g) + 0.5
        b = torch.randn(n, generator=g) * 0.1
        cases[f"n{n}_x"], cases[f"n{n}_w"], cases[f"n{n}_b"] = x.numpy(), w.numpy(), b.numpy()
        # pytorch_naive_layernorm uses the unbiased variance (torch.var default); stored as is,
        # next to F.layer_norm which the reference's tests use as ground truth.
        cases[f"n{n}_naive_ln"] = pytorch_naive_layernorm(x.clone(), w, b, 1e-5).numpy()
        cases[f"n{n}_f_ln"] = torch.nn.functional.layer_norm(x, (n,), w, b, 1e-5).numpy()
        cases[f"n{n}_rms"] = pytorch_naive_rmsnorm(x.clone(), w, 1e-6).numpy()
    np.savez_compressed(os.path.join(HERE, "norm_reference.npz"), **cases)

    # ---- Llama pieces from the reference's experimental eager code
    import importlib.util

    spec = importlib.util.spec_from_file_location(
        "kernl_llama_eager", os.path.join(REF_ROOT, "experimental", "llama-v2", "kernel", "pytorch_reference.py"))
    eager = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(eager)
    cases = {}
    B, S, H, D = 2, 7, 3, 16
    x = torch.randn(B, S, H, D, generator=g)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = (torch.arange(S, dtype=torch.float32) + 5)[:, None] * inv[None, :]  # positions 5 .. 5 + S - 1
    cos, sin = torch.cos(ang), torch.sin(ang)
    cases["rope_x"], cases["rope_cos"], cases["rope_sin"] = x.numpy(), cos.numpy(), sin.numpy()
    cases["rope_out"] = eager.apply_rotary_emb_pytorch(x, cos, sin).numpy()
    hid, ffn = 48, 40
    xf = torch.randn(5, hid, generator=g)
    rms_w = torch.rand(hid, generator=g) + 0.5
    w1 = torch.randn(ffn, hid, generator=g) * 0.2
    w3 = torch.randn(ffn, hid, generator=g) * 0.2
    x_norm = eager.rms_norm_pytorch(xf, rms_w, eps=1e-6)
    cases["ff_x"], cases["ff_rms_w"], cases["ff_w1"], cases["ff_w3"] = xf.numpy(), rms_w.numpy(), w1.numpy(), w3.numpy()
    cases["ff_x_norm"] = x_norm.numpy()
    cases["ff_out"] = (torch.nn.functional.silu(torch.matmul(x_norm, w1.t())) * torch.matmul(x_norm, w3.t())).numpy()
    np.savez_compressed(os.path.join(HERE, "llama_reference.npz"), **cases)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
