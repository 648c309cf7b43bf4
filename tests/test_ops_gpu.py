"""GPU parity tests: the CUDA kernels, called through the Python front-ends (ctypes → C ABI),
against the CPU oracle on the same seeded inputs. Shapes, input distributions and edge cases
follow the reference's op tests (test/test_attention.py, test/test_linear_layer.py,
test/test_layer_norm.py); the pass bar is the tolerance of this build — max-abs <= 1e-2 and
cosine >= 0.9995 for fp16 (bf16 outputs carry 8 mantissa bits, so their max-abs bound scales
with the output magnitude and is stated per test).
"""
import os

import numpy as np
import pytest
import torch

from oracle import kernl_oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _cuda(*ts):
    return tuple(t.cuda() if t is not None else None for t in ts)


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------
def _mask(kind, B, H, M, N, dtype, g):
    if kind == "none":
        return None
    if kind == "bias":  # test/test_attention.py:52-55
        return torch.rand((B, H, M, N), generator=g).to(dtype)
    if kind == "pad":  # test/test_attention.py:39-49
        valid = torch.randint(1, max(N, 2), (B,), generator=g)
        m = torch.where(valid[:, None] > torch.arange(N)[None, :], 0.0, float("-inf"))
        return m.reshape(B, 1, 1, N).to(dtype)
    raise ValueError(kind)


def _run_attention(B, H, M, N, D, dtype, causal, mask_kind, sm_scale, mask_dtype=None, fn=None):
    from kernl_b200.implementations.attention import attention_forward

    fn = fn or attention_forward
    g = torch.Generator().manual_seed(0)
    q = (torch.rand((B, H, M, D), generator=g) * 2).to(dtype)  # rand*2 as test/test_attention.py:92-96
    k = (torch.rand((B, H, N, D), generator=g) * 2).to(dtype)
    v = (torch.rand((B, H, N, D), generator=g) * 2).to(dtype)
    mask = _mask(mask_kind, B, H, M, N, mask_dtype or dtype, g)
    expected = O.attention(q, k, v, sm_scale, causal, mask)
    qc, kc, vc, mc = _cuda(q, k, v, mask)
    out = torch.empty_like(qc)
    ret = fn(qc, kc, vc, out, sm_scale, causal, mc)
    assert ret.data_ptr() == out.data_ptr()
    return out, expected


@pytest.mark.parametrize("seq", [8, 16, 32, 33, 64, 128, 256, 257, 384, 512])
@pytest.mark.parametrize("mask_kind", ["none", "pad", "bias"])
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_attention_reference_shapes(lib, seq, mask_kind, causal):
    out, expected = _run_attention(2, 12, seq, seq, 64, torch.float16, causal, mask_kind, 0.3)
    O.assert_parity(out, expected, what=f"attention seq={seq} {mask_kind} causal={causal}")


@pytest.mark.parametrize("shape", [(8, 1, 1500, 64), (1, 48, 512, 64), (3, 5, 130, 64)], ids=str)
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_attention_more_shapes(lib, shape, causal):
    B, H, S, D = shape
    out, expected = _run_attention(B, H, S, S, D, torch.float16, causal, "pad", 0.3)
    O.assert_parity(out, expected, what=f"attention {shape}")


@pytest.mark.parametrize("m,n", [(1, 24), (100, 300), (300, 100), (129, 1000)])
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_attention_rectangular(lib, m, n, causal):
    out, expected = _run_attention(2, 3, m, n, 64, torch.float16, causal, "bias", 0.3)
    O.assert_parity(out, expected, what=f"attention {m}x{n}")


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 1e-2), (torch.bfloat16, 3e-2)], ids=["fp16", "bf16"])
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_attention_head_dim_128(lib, dtype, tol, causal):
    # bf16 outputs near 1.0 have an ulp of 2^-8 = 3.9e-3 and P is rounded to bf16 as well
    out, expected = _run_attention(2, 4, 320, 320, 128, dtype, causal, "none", 128**-0.5)
    O.assert_parity(out, expected, max_abs=tol, what="attention d=128")


@pytest.mark.parametrize("d,dtype,tol", [(64, torch.float16, 1e-2), (64, torch.bfloat16, 3e-2), (128, torch.float16, 1e-2), (128, torch.bfloat16, 3e-2)],
                         ids=["d64_fp16", "d64_bf16", "d128_fp16", "d128_bf16"])
@pytest.mark.parametrize("mask_kind,causal,m,n", [("none", False, 512, 512), ("pad", False, 300, 300), ("bias", True, 257, 257),
                                                  ("none", True, 640, 640), ("bias", False, 100, 700), ("none", False, 1, 24)])
def test_attention_both_head_dims(lib, d, dtype, tol, mask_kind, causal, m, n):
    """Both fused kernels (head dimension 64: 64-key blocks, two threads per query row; head
    dimension 128: 128-key blocks) on every dtype, mask form and shape class."""
    out, expected = _run_attention(2, 3, m, n, d, dtype, causal, mask_kind, d ** -0.5)
    O.assert_parity(out, expected, max_abs=tol, what=f"d={d}")


@pytest.mark.parametrize("d", [16, 32, 40, 96, 20])
@pytest.mark.parametrize("mask_kind,causal,m,n", [("none", False, 300, 300), ("pad", False, 130, 520), ("bias", True, 257, 257), ("none", False, 1, 24)])
def test_attention_other_head_dims(lib, d, mask_kind, causal, m, n):
    """Head dimensions other than 64 / 128 (the reference takes powers of two from 16): multiples of 8
    run natively — tensor maps that end at the real head dimension under a 64-column box, output
    columns beyond it never written — and anything else (20) through the front-end's zero padding."""
    out, expected = _run_attention(2, 3, m, n, d, torch.float16, causal, mask_kind, d ** -0.5)
    assert out.shape[-1] == d
    O.assert_parity(out, expected, what=f"d={d}")


def test_attention_small_head_dim_leaves_neighbours_alone(lib):
    """The output of a head-dimension-16 call is a [.., 16] view into a wider buffer: the columns next
    to it must keep their contents (the kernel computes 64 columns and may store only 16)."""
    from kernl_b200.implementations.attention import attention_forward

    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn((1, 2, 200, 16), generator=g).half().cuda() for _ in range(3))
    wide = torch.full((1, 2, 200, 64), 7.0, dtype=torch.float16, device="cuda")
    out = wide[..., 8:24]
    attention_forward(q, k, v, out, 0.25)
    torch.cuda.synchronize()
    assert torch.all(wide[..., :8] == 7.0) and torch.all(wide[..., 24:] == 7.0)
    expected = O.attention(q.cpu(), k.cpu(), v.cpu(), 0.25)
    O.assert_parity(out.cpu(), expected, what="d=16 into a strided view")


@pytest.mark.parametrize("d,dtype,tol", [(64, torch.float16, 1e-2), (128, torch.bfloat16, 3e-2)], ids=["d64_fp16", "d128_bf16"])
@pytest.mark.parametrize("group", [2, 4, 8])
@pytest.mark.parametrize("m,n,causal,mask_kind", [(300, 300, True, "none"), (130, 520, False, "pad"), (1, 700, False, "none")])
def test_attention_grouped_query(lib, d, dtype, tol, group, m, n, causal, mask_kind):
    """k/v with H / group heads: query head h reads K/V head h // group — in the fused kernels and,
    for one query row, in the decode kernel — against the oracle on explicitly repeated K/V."""
    from kernl_b200.implementations.attention import attention_forward
    from kernl_b200.implementations.attention_skinny import skinny_attention_forward

    g = torch.Generator().manual_seed(group)
    B, H = 2, 8
    q = torch.randn((B, H, m, d), generator=g).to(dtype)
    k = torch.randn((B, H // group, n, d), generator=g).to(dtype)
    v = torch.randn((B, H // group, n, d), generator=g).to(dtype)
    mask = _mask(mask_kind, B, H, m, n, dtype, g)
    scale = d ** -0.5
    expected = O.attention(q, k.repeat_interleave(group, 1), v.repeat_interleave(group, 1), scale, causal, mask)
    qc, kc, vc, mc = _cuda(q, k, v, mask)
    fn = skinny_attention_forward if m == 1 else attention_forward
    out = fn(qc, kc, vc, torch.empty_like(qc), scale, causal, mc)
    O.assert_parity(out, expected, max_abs=tol, what=f"group {group}")
    O.assert_parity(out, O.attention(q, k, v, scale, causal, mask), max_abs=tol, what="oracle's own head expansion")


@pytest.mark.parametrize("tiles", [1, 2], ids=["one_tile_per_cta", "two_tiles_per_cta"])
@pytest.mark.parametrize("dtype,tol", [(torch.float16, 1e-2), (torch.bfloat16, 3e-2)], ids=["fp16", "bf16"])
@pytest.mark.parametrize("mask_kind,causal,m,n", [("none", False, 512, 512), ("pad", False, 300, 300), ("bias", True, 257, 257),
                                                  ("none", True, 640, 640), ("bias", False, 100, 700), ("none", False, 1, 24),
                                                  ("pad", False, 1100, 1100)])
def test_attention_split_rows_both_cta_shapes(lib, tiles, dtype, tol, mask_kind, causal, m, n):
    """The head-dimension-64 kernel in both of its CTA shapes (one query tile per CTA, two CTAs per
    SM — the dispatcher's choice; two tiles per CTA, kept selectable)."""
    try:
        lib.kb_debug_split_tiles(tiles)
        out, expected = _run_attention(2, 3, m, n, 64, dtype, causal, mask_kind, 0.125)
    finally:
        lib.kb_debug_split_tiles(0)
    O.assert_parity(out, expected, max_abs=tol, what=f"split rows, {tiles} tile(s) per CTA")


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 1e-2), (torch.bfloat16, 3e-2)], ids=["fp16", "bf16"])
@pytest.mark.parametrize("mask_kind,causal,m,n", [("none", False, 512, 512), ("pad", False, 300, 300), ("bias", True, 257, 257),
                                                  ("none", True, 640, 640), ("bias", False, 100, 700), ("none", False, 1, 24),
                                                  ("pad", False, 1100, 1100), ("pad", True, 384, 384)])
def test_attention_persistent_scheduling_small_launches(lib, dtype, tol, mask_kind, causal, m, n):
    """The head-dimension-64 kernel with persistent CTAs drawing query tiles from the device-side
    queue, forced on launches of a few tiles (every CTA draws one tile and then finds the queue
    empty) up to a few tiles per CTA."""
    try:
        lib.kb_debug_attention_persistent(1)
        out, expected = _run_attention(2, 3, m, n, 64, dtype, causal, mask_kind, 0.125)
    finally:
        lib.kb_debug_attention_persistent(-1)
    O.assert_parity(out, expected, max_abs=tol, what="persistent CTAs")


@pytest.mark.parametrize("kind", ["none", "pad", "causal", "bias", "pad_causal"])
@pytest.mark.parametrize("shape", [(16, 12, 512), (40, 12, 128), (3, 16, 4096), (8, 12, 512)], ids=str)
def test_attention_persistent_scheduling_equals_one_cta_per_tile(lib, shape, kind):
    """Launches of more query tiles than CTA slots (what the dispatcher gives to the persistent
    kernel): every tile goes through the same arithmetic in both forms of the kernel, so the outputs
    must be bit-identical whatever CTA computed a tile and in whatever order; sampled (batch, head)
    slices are checked against the oracle as well. Repeated, because the tile-to-CTA assignment
    depends on timing."""
    from kernl_b200.implementations.attention import attention_forward

    B, H, S = shape
    g = torch.Generator().manual_seed(B * 1000 + S)
    q, k, v = (torch.randn((B, H, S, 64), generator=g).half() for _ in range(3))
    mask = None
    if kind.startswith("pad"):
        valid = torch.randint(min(64, S), S + 1, (B,), generator=g)
        valid[0] = S // 3
        mask = torch.where(valid[:, None] > torch.arange(S)[None, :], 0.0, float("-inf")).reshape(B, 1, 1, S).half()
    elif kind == "bias":
        if B * H * S * S * 2 > (1 << 31):
            pytest.skip("bias mask of this shape is larger than needed here")
        mask = torch.rand((B, H, S, S), generator=g).half()
    causal = kind.endswith("causal")
    qc, kc, vc, mc = _cuda(q, k, v, mask)
    outs = {}
    for mode in (0, 1, 1, 1):
        try:
            lib.kb_debug_attention_persistent(mode)
            out = attention_forward(qc, kc, vc, torch.empty_like(qc), 0.125, causal, mc)
        finally:
            lib.kb_debug_attention_persistent(-1)
        if mode in outs:
            assert torch.equal(out, outs[mode]), "two runs of the persistent kernel differ"
        outs[mode] = out
    assert torch.equal(outs[0], outs[1]), "persistent CTAs and one CTA per tile disagree"
    default = attention_forward(qc, kc, vc, torch.empty_like(qc), 0.125, causal, mc)
    assert torch.equal(default, outs[1])
    for b, h in [(0, 0), (B - 1, H - 1), (B // 2, 5)]:
        exp = O.attention(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], 0.125, causal,
                          None if mask is None else mask[b:b + 1, (h if mask.shape[1] > 1 else 0):(h if mask.shape[1] > 1 else 0) + 1])
        O.assert_parity(outs[1][b:b + 1, h:h + 1], exp, what=f"batch {b} head {h}")


@pytest.mark.parametrize("fill", [float("-inf"), -65504.0, -10000.0], ids=["neg_inf", "fp16_lowest", "minus_1e4"])
@pytest.mark.parametrize("causal", [False, True], ids=["full", "causal"])
def test_attention_padding_mask_with_fully_masked_key_blocks(lib, fill, causal):
    """Row-broadcast masks that blank out whole 64-key blocks: the head-dimension-64 kernel does not
    visit such blocks. Right padding, left padding, a hole in the middle, a single live key, and one
    fully masked sequence (where nothing may be skipped) in one batch."""
    from kernl_b200.implementations.attention import attention_forward

    g = torch.Generator().manual_seed(5)
    B, H, S, D = 6, 2, 448, 64
    q, k, v = (torch.randn((B, H, S, D), generator=g).half() for _ in range(3))
    mask = torch.zeros((B, 1, 1, S))
    mask[0, ..., 200:] = fill          # right padding: blocks 4..6 blank
    mask[1, ..., :130] = fill          # left padding: blocks 0..1 blank
    mask[2, ..., 64:320] = fill        # hole: blocks 1..4 blank
    mask[3, ..., :] = fill
    mask[3, ..., 257] = 0.0            # one live key
    mask[4, ..., :] = fill             # fully masked sequence
    mask = mask.half()
    expected = O.attention(q, k, v, 0.125, causal, mask)
    qc, kc, vc, mc = _cuda(q, k, v, mask)
    out = attention_forward(qc, kc, vc, torch.empty_like(qc), 0.125, causal, mc)
    assert torch.isfinite(out).all()
    O.assert_parity(out, expected, max_abs=2e-2 if fill != -10000.0 else 1e-2, cos=0.999)


def test_attention_fp32_mask_and_row_broadcast(lib):
    out, expected = _run_attention(2, 4, 200, 200, 64, torch.float16, False, "pad", 0.125, mask_dtype=torch.float32)
    O.assert_parity(out, expected)
    # T5-style position bias: batch-broadcast [1,H,M,N]
    from kernl_b200.implementations.attention import attention_forward

    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn((2, 4, 150, 64), generator=g).half() for _ in range(3))
    bias = torch.randn((1, 4, 150, 150), generator=g).half()
    expected = O.attention(q, k, v, 1.0, False, bias)
    qc, kc, vc, bc = _cuda(q, k, v, bias)
    out = attention_forward(qc, kc, vc, torch.empty_like(qc), 1.0, False, bc)
    O.assert_parity(out, expected)


def test_attention_fully_masked_row_is_finite(lib):
    """-inf mask entries act as the lowest finite value (reference attention.py:380), so a fully
    padded sequence gives a plain softmax instead of NaN."""
    from kernl_b200.implementations.attention import attention_forward

    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn((1, 2, 64, 64), generator=g).half() for _ in range(3))
    mask = torch.full((1, 1, 1, 64), float("-inf"), dtype=torch.float16)
    expected = O.attention(q, k, v, 0.125, False, mask)
    qc, kc, vc, mc = _cuda(q, k, v, mask)
    out = attention_forward(qc, kc, vc, torch.empty_like(qc), 0.125, False, mc)
    O.assert_parity(out, expected, max_abs=3e-2)  # (score - 65504) is rounded to 2^-8 in fp32 on both sides


def test_attention_mixed_stride(lib):
    """Column-major q, interleaved-batch k, transposed mask (test/test_attention.py:110-129)."""
    from kernl_b200.implementations.attention import attention_forward

    g = torch.Generator().manual_seed(0)
    q = torch.rand((2, 6, 64, 256), generator=g).half().cuda().transpose(-1, -2)
    k = torch.rand((6, 2, 256, 64), generator=g).half().cuda().transpose(0, 1)
    v = torch.rand((2, 6, 256, 64), generator=g).half().cuda()
    mask = torch.rand((6, 2, 256, 256), generator=g).half().cuda().transpose(0, 1).transpose(-1, -2)
    assert not q.is_contiguous() and not k.is_contiguous() and not mask.is_contiguous()
    expected = O.attention(q, k, v, 0.3, False, mask)
    out = torch.empty_like(q)  # keeps q's column-major strides
    attention_forward(q, k, v, out, 0.3, attention_mask=mask)
    O.assert_parity(out, expected)


def test_attention_cross_attention(lib):
    """M=1, N=24 through the fused kernel (test/test_attention.py:132-145)."""
    out, expected = _run_attention(1, 8, 1, 24, 64, torch.float16, False, "bias", 1.0)
    O.assert_parity(out, expected)


@pytest.mark.parametrize("name", ["nomask", "pad", "bias", "cross", "d128"])
def test_attention_against_reference_golden(lib, name):
    from kernl_b200.implementations.attention import attention_forward

    g = np.load(os.path.join(GOLDEN, "attention_reference.npz"))
    q, k, v = (torch.from_numpy(g[f"{name}_{t}"]).half() for t in "qkv")
    mask = torch.from_numpy(g[f"{name}_mask"]).half() if f"{name}_mask" in g.files else None
    # the golden output was computed from fp32 inputs; recompute the expectation from the rounded
    # inputs with the oracle AND keep the raw golden as a looser second check
    expected = O.attention(q, k, v, float(g[f"{name}_scale"]), False, mask)
    qc, kc, vc, mc = _cuda(q, k, v, mask)
    out = attention_forward(qc, kc, vc, torch.empty_like(qc), float(g[f"{name}_scale"]), False, mc)
    O.assert_parity(out, expected)
    O.assert_parity(out, torch.from_numpy(g[f"{name}_out"]), max_abs=5e-2, cos=0.999)


@pytest.mark.parametrize("name", ["causal_square", "causal_morekeys", "causal_morequeries", "causal_bias", "causal_pad", "causal_d128"])
def test_attention_causal_against_reference_golden(lib, name):
    """The kernels' causal branch against outputs of the reference's own
    `attention_reference(is_causal=True)` (src/kernl/implementations/attention.py:29-61)."""
    from kernl_b200.implementations.attention import attention_forward

    g = np.load(os.path.join(GOLDEN, "attention_reference.npz"))
    q, k, v = (torch.from_numpy(g[f"{name}_{t}"]).half() for t in "qkv")
    mask = torch.from_numpy(g[f"{name}_mask"]).half() if f"{name}_mask" in g.files else None
    expected = O.attention(q, k, v, float(g[f"{name}_scale"]), True, mask)
    qc, kc, vc, mc = _cuda(q, k, v, mask)
    out = attention_forward(qc, kc, vc, torch.empty_like(qc), float(g[f"{name}_scale"]), True, mc)
    O.assert_parity(out, expected)
    O.assert_parity(out, torch.from_numpy(g[f"{name}_out"]), max_abs=5e-2, cos=0.999)


@pytest.mark.parametrize("kind", ["full", "causal", "pad"])
@pytest.mark.parametrize("seq", [2048, 4096])
@pytest.mark.parametrize("d,dtype,tol", [(64, torch.float16, 1e-2), (128, torch.bfloat16, 3e-2)], ids=["d64_fp16", "d128_bf16"])
def test_attention_long_sequences_sampled_rows(lib, d, dtype, tol, seq, kind):
    """The sizes the benchmark sweep quotes (4096 tokens split into sequences of 2048 / 4096 keys,
    both head dimensions): 128-row query tiles sampled from the first, a middle and the last part
    of several (batch, head) pairs against the oracle evaluated on those rows alone (a causal
    row only needs the keys up to itself, so the oracle gets the row offset through a bias-free
    slice: queries [r0, r0+128) against keys [0, r0+128) with a top-left mask shifted by r0)."""
    from kernl_b200.implementations.attention import attention_forward

    g = torch.Generator().manual_seed(seq + d)
    B, H = 4096 // seq if d == 64 else 2, 12 if d == 64 else 32
    B = max(B, 2)
    q, k, v = (torch.randn((B, H, seq, d), generator=g).to(dtype) for _ in range(3))
    mask = None
    valid = torch.full((B,), seq)
    if kind == "pad":
        valid = torch.randint(64, seq + 1, (B,), generator=g)
        mask = torch.where(valid[:, None] > torch.arange(seq)[None, :], 0.0, float("-inf")).reshape(B, 1, 1, seq).to(dtype)
    scale = d ** -0.5
    qc, kc, vc, mc = _cuda(q, k, v, mask)
    out = attention_forward(qc, kc, vc, torch.empty_like(qc), scale, kind == "causal", mc).cpu()
    for b, h, r0 in [(0, 0, 0), (B - 1, H - 1, seq - 128), (B - 1, 3, seq // 2 - 64), (0, H // 2, seq // 2 + 128)]:
        rows = slice(r0, r0 + 128)
        qs = q[b:b + 1, h:h + 1, rows]
        if kind == "causal":
            # rows r0.. see keys 0..row: evaluate against keys [0, r0+128) with an additive mask
            n = r0 + 128
            tri = torch.where(torch.arange(n)[None, :] <= (torch.arange(128) + r0)[:, None], 0.0, float("-inf")).reshape(1, 1, 128, n)
            exp = O.attention(qs, k[b:b + 1, h:h + 1, :n], v[b:b + 1, h:h + 1, :n], scale, False, tri)
        else:
            exp = O.attention(qs, k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], scale, False, mask[b:b + 1] if mask is not None else None)
        O.assert_parity(out[b:b + 1, h:h + 1, rows], exp, max_abs=tol, what=f"b{b} h{h} rows {r0}")


def test_attention_full_size_properties(lib):
    """Config-size check ([8,12,512,64], padding mask) through properties that need no CPU
    oracle at that size plus a sampled oracle comparison: rows of softmax sum to one (V = ones
    gives ones), linearity in V, and independence of padded keys."""
    from kernl_b200.implementations.attention import attention_forward

    g = torch.Generator().manual_seed(0)
    B, H, S, D = 8, 12, 512, 64
    q, k, v = (torch.randn((B, H, S, D), generator=g).half().cuda() for _ in range(3))
    valid = torch.randint(64, S + 1, (B,), generator=g)
    mask = torch.where(valid[:, None] > torch.arange(S)[None, :], 0.0, float("-inf")).reshape(B, 1, 1, S).half().cuda()
    run = lambda vv, kk=k: attention_forward(q, kk, vv, torch.empty_like(q), 0.125, False, mask)
    ones = run(torch.ones_like(v))
    assert (ones.float() - 1).abs().max() < 2e-3
    v2 = torch.randn((B, H, S, D), generator=g).half().cuda()
    lin = run((0.5 * v.float() + 0.25 * v2.float()).half())
    assert (lin.float() - (0.5 * run(v).float() + 0.25 * run(v2).float())).abs().max() < 5e-3
    k_junk, v_junk = k.clone(), v.clone()
    for b in range(B):
        k_junk[b, :, valid[b]:] = 7.0
        v_junk[b, :, valid[b]:] = -9.0
    assert torch.equal(run(v_junk, k_junk), run(v))
    # two (batch, head) slices against the oracle
    for b, h in [(0, 0), (7, 11)]:
        exp = O.attention(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], 0.125, False, mask[b:b + 1])
        O.assert_parity(run(v)[b:b + 1, h:h + 1], exp)


# ------------------------------------------------------------------------------------------------
# skinny (decode-shape) attention
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("beam,heads", [(1, 6), (5, 20), (1, 16)])
@pytest.mark.parametrize("mask_kind", ["none", "bias"])
def test_skinny_attention_whisper_shapes(lib, beam, heads, mask_kind):
    """(beam, heads, 1500, 64) with one query row (test/test_attention.py:176-208)."""
    from kernl_b200.implementations.attention_skinny import skinny_attention_forward

    out, expected = _run_attention(beam, heads, 1, 1500, 64, torch.float16, False, mask_kind, 0.3, fn=skinny_attention_forward)
    O.assert_parity(out, expected)


@pytest.mark.parametrize("m,n,d,dtype", [(1, 51, 64, torch.float16), (3, 700, 64, torch.float16), (1, 2049, 128, torch.bfloat16), (2, 40000, 64, torch.float16)])
def test_skinny_attention_shapes(lib, m, n, d, dtype):
    from kernl_b200.implementations.attention_skinny import skinny_attention_forward

    out, expected = _run_attention(2, 3, m, n, d, dtype, False, "pad", 0.3, fn=skinny_attention_forward)
    O.assert_parity(out, expected, max_abs=1e-2 if dtype == torch.float16 else 3e-2)


@pytest.mark.parametrize("d,dtype,tol", [(64, torch.float16, 1e-2), (128, torch.bfloat16, 3e-2)], ids=["d64_fp16", "d128_bf16"])
@pytest.mark.parametrize("live", [1, 127, 128, 129, 1000, 2304])
def test_skinny_attention_device_side_key_count(lib, d, dtype, tol, live):
    """A KV cache of 2304 slots of which `live` are filled (the count lives on the device): the
    result equals attention over the first `live` keys, whatever the other slots hold, and the
    same captured call follows the count when it changes."""
    from kernl_b200.implementations.attention_skinny import skinny_attention_forward

    g = torch.Generator().manual_seed(live)
    B, H, N = 2, 4, 2304
    q = torch.randn((B, H, 1, d), generator=g).to(dtype)
    k = torch.randn((B, H, N, d), generator=g).to(dtype)
    v = torch.randn((B, H, N, d), generator=g).to(dtype)
    k[:, :, live:] = 50.0   # stale slots must not matter
    v[:, :, live:] = -70.0
    qc, kc, vc = _cuda(q, k, v)
    count = torch.tensor([live], dtype=torch.int64, device="cuda")
    out = skinny_attention_forward(qc, kc, vc, torch.empty_like(qc), d ** -0.5, False, None, kv_len=count)
    O.assert_parity(out, O.attention(q, k[:, :, :live], v[:, :, :live], d ** -0.5), max_abs=tol, what=f"{live} live keys")
    if live > 1:
        count.fill_(live - 1)
        out = skinny_attention_forward(qc, kc, vc, torch.empty_like(qc), d ** -0.5, False, None, kv_len=count)
        O.assert_parity(out, O.attention(q, k[:, :, :live - 1], v[:, :, :live - 1], d ** -0.5), max_abs=tol)


@pytest.mark.parametrize("d,dtype,tol", [(64, torch.float16, 1e-2), (128, torch.bfloat16, 3e-2)], ids=["d64_fp16", "d128_bf16"])
def test_skinny_attention_right_behind_a_long_kernel(lib, d, dtype, tol):
    """Many (batch, head) problems launched while the GPU is still draining a large fill: the first
    wave of CTAs then sees slow asynchronous copies, which is what exposes a missing wait on the
    staged K/V tiles (this case failed once with errors of 1e18)."""
    from kernl_b200.implementations.attention_skinny import skinny_attention_forward

    g = torch.Generator().manual_seed(0)
    B, H, N = 8, 32, 1500
    q = (torch.rand((B, H, 1, d), generator=g) * 2).to(dtype)
    k = (torch.rand((B, H, N, d), generator=g) * 2).to(dtype)
    v = (torch.rand((B, H, N, d), generator=g) * 2).to(dtype)
    expected = O.attention(q, k, v, 0.3, False, None)
    qc, kc, vc = _cuda(q, k, v)
    for _ in range(4):
        junk = torch.full((64 * 1024 * 1024,), float("nan"), device="cuda")
        out = torch.empty_like(qc)
        skinny_attention_forward(qc, kc, vc, out, 0.3, False, None)
        del junk
        O.assert_parity(out, expected, max_abs=tol)


def test_skinny_matches_fused_kernel(lib):
    from kernl_b200.implementations.attention import attention_forward
    from kernl_b200.implementations.attention_skinny import skinny_attention_forward

    a, _ = _run_attention(2, 4, 1, 777, 64, torch.float16, False, "bias", 0.3, fn=skinny_attention_forward)
    b, _ = _run_attention(2, 4, 1, 777, 64, torch.float16, False, "bias", 0.3, fn=attention_forward)
    assert (a.float() - b.float()).abs().max() < 4e-3


# ------------------------------------------------------------------------------------------------
# linear
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("contiguous", [True, False], ids=["contiguous", "non-contiguous"])
@pytest.mark.parametrize("bias", [True, False], ids=["with_bias", "no_bias"])
@pytest.mark.parametrize("activation", ["", "tanh", "gelu", "relu", "fast_gelu", "silu"])
@pytest.mark.parametrize("shape", [(1, 8, 8, 8), (1, 16, 768, 768), (16, 128, 768, 768), (1, 512, 768, 768)], ids=str)
def test_linear_reference_shapes(lib, shape, activation, bias, contiguous):
    """Shapes and layout of test/test_linear_layer.py:48-99: x is a transposed view of a
    [batch, K, M] tensor; weights drawn N(0,1) as there (the 1e-2 bound is scaled by the output
    magnitude, sqrt(K), because fp16 outputs of size ~30 have an ulp of 1.6e-2)."""
    from kernl_b200.implementations.linear_layer import linear_layer

    batch, M, N, K = shape
    g = torch.Generator().manual_seed(0)
    x = torch.randn((batch, K, M), generator=g).half().mT
    if contiguous:
        x = x.contiguous()
    w = torch.randn((N, K), generator=g).half()
    b = torch.randn((N,), generator=g).half() if bias else None
    expected = O.linear(x.reshape(-1, K), w, b, activation).reshape(batch, M, N)
    xc, wc, bc = _cuda(x, w, b)
    out = linear_layer(xc, wc, bc, activation)
    assert out.shape == (batch, M, N)
    O.assert_parity(out, expected, max_abs=1e-2 * max(1.0, K**0.5))


@pytest.mark.parametrize("M", [16, 128, 1024])
@pytest.mark.parametrize("kn", [(768, 768), (768, 3072), (3072, 768), (4096, 11008), (11008, 4096)], ids=str)
@pytest.mark.parametrize("activation", ["", "gelu", "relu"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_linear_config_shapes(lib, M, kn, activation, dtype):
    """X ~ N(0,1), W ~ N(0,0.02), bias ~ N(0,0.02): outputs are O(1), so the plain bound applies
    to fp16; bf16 outputs of magnitude up to ~8 have an ulp of 3.1e-2."""
    from kernl_b200.implementations.linear_layer import linear_layer

    K, N = kn
    g = torch.Generator().manual_seed(0)
    x = torch.randn((M, K), generator=g).to(dtype)
    w = (torch.randn((N, K), generator=g) * 0.02).to(dtype)
    b = (torch.randn((N,), generator=g) * 0.02).to(dtype)
    expected = O.linear(x, w, b, activation)
    xc, wc, bc = _cuda(x, w, b)
    out = linear_layer(xc, wc, bc, activation)
    O.assert_parity(out, expected, max_abs=1e-2 if dtype == torch.float16 else 4e-2)


def test_linear_largest_config_against_sampled_oracle(lib):
    """M=8192, (K,N)=(4096,11008): full output checked on sampled rows/columns against the oracle,
    plus linearity in x over the whole output."""
    from kernl_b200.implementations.linear_layer import linear_layer

    g = torch.Generator().manual_seed(0)
    M, K, N = 8192, 4096, 11008
    x = torch.randn((M, K), generator=g).half()
    w = (torch.randn((N, K), generator=g) * 0.02).half()
    b = (torch.randn((N,), generator=g) * 0.02).half()
    xc, wc, bc = _cuda(x, w, b)
    out = linear_layer(xc, wc, bc, "")
    rows = torch.tensor([0, 1, 127, 128, 4095, 8191])
    expected = O.linear(x[rows], w, b, "")
    O.assert_parity(out[rows.cuda()], expected)
    half_out = linear_layer((xc.float() * 0.5).half(), wc, None, "")
    assert (half_out.float() * 2 + bc.float() - out.float()).abs().max() < 1e-2


def test_linear_ragged_shapes_and_act_inputs(lib):
    from kernl_b200.implementations.linear_layer import linear_layer

    g = torch.Generator().manual_seed(0)
    for (M, K, N) in [(1, 8, 8), (100, 200, 72), (300, 520, 136), (129, 72, 257), (5, 12, 3)]:
        x = torch.randn((M, K), generator=g).half()
        w = (torch.randn((N, K), generator=g) * 0.1).half()
        b = torch.randn((N,), generator=g).half()
        xc, wc, bc = _cuda(x, w, b)
        pre = torch.empty((M, N), dtype=torch.float16, device="cuda")
        out = linear_layer(xc, wc, bc, "gelu", pre)
        O.assert_parity(out, O.linear(x, w, b, "gelu"), what=f"{M}x{K}x{N}")
        O.assert_parity(pre, O.linear(x, w, b, ""), what=f"act_inputs {M}x{K}x{N}")


def test_linear_every_tile_width(lib):
    from kernl_b200.implementations.linear_layer import linear_layer

    g = torch.Generator().manual_seed(0)
    x = torch.randn((300, 520), generator=g).half()
    w = (torch.randn((392, 520), generator=g) * 0.05).half()
    b = torch.randn((392,), generator=g).half()
    expected = O.linear(x, w, b, "relu")
    xc, wc, bc = _cuda(x, w, b)
    try:
        for bn in (32, 64, 128, 256):
            lib.kb_debug_force_bn(bn)
            O.assert_parity(linear_layer(xc, wc, bc, "relu"), expected, what=f"BN={bn}")
    finally:
        lib.kb_debug_force_bn(0)


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 1e-2), (torch.bfloat16, 6e-2)], ids=["fp16", "bf16"])
@pytest.mark.parametrize("activation", ["", "gelu", "swiglu"])
@pytest.mark.parametrize("shape", [(2048, 512, 2560), (2000, 264, 2512), (513, 1024, 9488), (4096, 256, 1280)], ids=str)
@pytest.mark.parametrize("width", [256, 192])
def test_linear_cta_pairs(lib, shape, activation, dtype, tol, width):
    """Problems large enough for the CTA-pair kernel (256-row tiles of 256 or 192 columns,
    `tcgen05.mma.cta_group::2`), with ragged edges in every dimension, against the oracle and against
    the one-CTA-per-tile kernel. Gelu runs once with a pre-activation output (the epilogue's
    thread-per-row path) and, in `test_linear_cta_pairs_staged_gelu`, once without."""
    from kernl_b200.implementations.linear_layer import linear_layer

    M, K, N = shape
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn((M, K), generator=g).to(dtype)
    w = (torch.randn((N, K), generator=g) * 0.05).to(dtype)
    b = (torch.randn((N,), generator=g) * 0.1).to(dtype)
    xc, wc, bc = _cuda(x, w, b)
    pre = torch.empty((M, N), dtype=dtype, device="cuda") if activation == "gelu" else None
    try:
        lib.kb_debug_linear_pair(width)
        out = linear_layer(xc, wc, bc, activation, act_inputs=pre)
        lib.kb_debug_linear_pair(0)
        single = linear_layer(xc, wc, bc, activation)
    finally:
        lib.kb_debug_linear_pair(1)
    if activation == "swiglu":
        z = O.linear(x, w, b, "").reshape(M, N // 16, 2, 8)
        expected = (torch.nn.functional.silu(z[:, :, 0]) * z[:, :, 1]).reshape(M, N // 2)
    else:
        expected = O.linear(x, w, b, activation)
    if dtype == torch.bfloat16:  # 8 mantissa bits: one ulp of the largest result
        tol = max(tol, float(expected.abs().max()) * 2.0 ** -7)
    O.assert_parity(out, expected, max_abs=tol, what="pair kernel vs oracle")
    # the two kernels add the same products in the same k order: they may differ by a rounding of the
    # 16-bit result here and there, not more (compared in double precision: the fp32 cosine of
    # several million values is itself only good to ~1e-4)
    diff = out.double().cpu() - single.double().cpu()
    rel_rms = float(diff.norm() / single.double().cpu().norm())
    print(f"pair vs one CTA per tile: relative rms difference {rel_rms:.3e}, max abs {float(diff.abs().max()):.3e}")
    assert rel_rms < (5e-4 if dtype == torch.float16 else 4e-3), rel_rms
    if pre is not None:
        O.assert_parity(pre, O.linear(x, w, b, ""), max_abs=tol, what="pre-activation output")


@pytest.mark.parametrize("width", [256, 192, 1])
@pytest.mark.parametrize("activation", ["gelu", "fast_gelu", "tanh", "silu"])
@pytest.mark.parametrize("shape", [(8192, 768, 3072), (1000, 520, 1400)], ids=str)
def test_linear_cta_pairs_staged_epilogue(lib, shape, activation, width):
    """The pair kernel's staged epilogue (results through shared memory, sixteen warps) with every
    activation and both tile widths (1 = the dispatcher's own choice), without bias as well."""
    from kernl_b200.implementations.linear_layer import linear_layer

    M, K, N = shape
    g = torch.Generator().manual_seed(N)
    x = torch.randn((M, K), generator=g).half()
    w = (torch.randn((N, K), generator=g) * 0.05).half()
    b = (torch.randn((N,), generator=g) * 0.5).half()
    xc, wc, bc = _cuda(x, w, b)
    try:
        lib.kb_debug_linear_pair(width)
        with_bias = linear_layer(xc, wc, bc, activation)
        without = linear_layer(xc, wc, None, activation)
    finally:
        lib.kb_debug_linear_pair(1)
    O.assert_parity(with_bias, O.linear(x, w, b, activation), what=f"{activation} with bias, width {width}")
    O.assert_parity(without, O.linear(x, w, None, activation), what=f"{activation} without bias, width {width}")


@pytest.mark.parametrize("limit", [100, 32, 3])
@pytest.mark.parametrize("shape", [(4096, 512, 5120), (2048, 768, 768)], ids=str)  # (more than 1024 rows: no split-K, whose atomics add in no fixed order)
def test_linear_with_an_sm_limit(lib, shape, limit):
    """`kb_gemm_sm_limit(n)`: the persistent GEMMs run on at most n SMs (what the two-stream prefill of
    the tensor-parallel decoder sets while a collective shares the GPU) and give the same bits."""
    from kernl_b200.implementations.linear_layer import linear_layer

    M, K, N = shape
    g = torch.Generator().manual_seed(limit)
    x, w, b = (torch.randn((M, K), generator=g).half(), (torch.randn((N, K), generator=g) * 0.05).half(),
               torch.randn((N,), generator=g).half())
    xc, wc, bc = _cuda(x, w, b)
    full = linear_layer(xc, wc, bc, "relu")
    try:
        assert lib.kb_gemm_sm_limit(limit) == 0
        limited = linear_layer(xc, wc, bc, "relu")
    finally:
        lib.kb_gemm_sm_limit(0)
    assert lib.kb_gemm_sm_limit(-1) != 0
    torch.cuda.synchronize()
    assert torch.equal(full, limited)
    O.assert_parity(limited, O.linear(x, w, b, "relu"), what=f"linear on {limit} SMs")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("shape", [(1, 4096, 4096), (5, 520, 1000), (8, 11008, 4096), (9, 264, 17), (16, 8, 40), (13, 4096, 12288)], ids=str)
def test_linear_few_rows(lib, shape, dtype):
    """M <= 16 goes to the weight-streaming kernel: ragged N, K tails that are not a multiple of 32,
    a row-strided x, the pre-activation side output, and an output written into a strided view."""
    from kernl_b200.implementations.linear_layer import linear_layer

    M, K, N = shape
    g = torch.Generator().manual_seed(2)
    xfull = torch.randn((M, K + 24), generator=g).to(dtype)
    w = (torch.randn((N, K), generator=g) * 0.02).to(dtype)
    b = (torch.randn((N,), generator=g) * 0.02).to(dtype)
    x = xfull[:, 8:8 + K]  # row stride K + 24, 16-byte aligned start
    tol = 1e-2 if dtype == torch.float16 else 4e-2
    xc, wc, bc = _cuda(xfull, w, b)
    xv = xc[:, 8:8 + K]
    pre = torch.empty((M, N), dtype=dtype, device="cuda")
    out = linear_layer(xv, wc, bc, "gelu", act_inputs=pre)
    O.assert_parity(out, O.linear(x, w, b, "gelu"), max_abs=tol)
    O.assert_parity(pre, O.linear(x, w, b, ""), max_abs=tol)
    O.assert_parity(linear_layer(xv, wc, None, ""), O.linear(x, w, None, ""), max_abs=tol)


@pytest.mark.parametrize("shape", [(16, 768, 768), (128, 3072, 768), (40, 4096, 1000), (8, 11008, 4096), (300, 520, 392)], ids=str)
@pytest.mark.parametrize("splits", [0, 2, 5])
def test_linear_split_k(lib, shape, splits):
    """Split-K (fp32 atomics into the workspace + finishing kernel) against the oracle, with the
    heuristic (0) and forced split counts; act_inputs must hold the pre-activation values."""
    from kernl_b200.implementations.linear_layer import linear_layer

    M, K, N = shape
    g = torch.Generator().manual_seed(0)
    x = torch.randn((M, K), generator=g).half()
    w = (torch.randn((N, K), generator=g) * 0.02).half()
    b = (torch.randn((N,), generator=g) * 0.02).half()
    xc, wc, bc = _cuda(x, w, b)
    pre = torch.empty((M, N), dtype=torch.float16, device="cuda")
    try:
        lib.kb_debug_force_splits(splits)
        for _ in range(2):  # twice: the workspace is reused and must be cleared by the call
            out = linear_layer(xc, wc, bc, "gelu", pre)
    finally:
        lib.kb_debug_force_splits(0)
    O.assert_parity(out, O.linear(x, w, b, "gelu"))
    O.assert_parity(pre, O.linear(x, w, b, ""))


def test_host_attention_pipeline_keeps_calls_apart(lib):
    """Six calls with different pinned host operands through the two-deep host pipeline: each
    result buffer must hold its own call's attention (set reuse is ordered by events), equal to
    the direct call on device tensors bit for bit."""
    from kernl_b200.host_pipeline import HostAttentionPipeline
    from kernl_b200.implementations.attention import attention_forward

    g = torch.Generator().manual_seed(3)
    B, H, S, D = 2, 3, 200, 64
    pipe = HostAttentionPipeline((B, H, S, D), (B, H, S, D), (B, 1, 1, S), torch.float16, "cuda")
    calls = []
    for i in range(6):
        hq, hk, hv = (torch.randn((B, H, S, D), generator=g).half().pin_memory() for _ in range(3))
        valid = torch.randint(1, S, (B,), generator=g)
        hm = torch.where(valid[:, None] > torch.arange(S)[None, :], 0.0, float("-inf")).reshape(B, 1, 1, S).half().pin_memory()
        hout = torch.full((B, H, S, D), float("nan"), dtype=torch.float16).pin_memory()
        calls.append((hq, hk, hv, hm, hout))
        pipe.submit(hq, hk, hv, hm, hout, 0.125)
    pipe.synchronize()
    for i, (hq, hk, hv, hm, hout) in enumerate(calls):
        q, k, v, m = hq.cuda(), hk.cuda(), hv.cuda(), hm.cuda()
        direct = attention_forward(q, k, v, torch.empty_like(q), 0.125, False, m)
        assert torch.equal(hout, direct.cpu()), f"call {i}"
    O.assert_parity(calls[-1][4], O.attention(calls[-1][0], calls[-1][1], calls[-1][2], 0.125, False, calls[-1][3]))


def _gated_case(m, k, f, dtype, with_bias, seed=0):
    from kernl_b200.implementations.linear_layer import interleave_gate_up

    g = torch.Generator().manual_seed(seed)
    x = torch.randn((m, k), generator=g).to(dtype)
    wg = (torch.randn((f, k), generator=g) * 0.05).to(dtype)
    wu = (torch.randn((f, k), generator=g) * 0.05).to(dtype)
    bg = (torch.randn((f,), generator=g) * 0.1).to(dtype) if with_bias else None
    bu = (torch.randn((f,), generator=g) * 0.1).to(dtype) if with_bias else None
    expected = torch.nn.functional.silu(O.linear(x, wg, bg)) * O.linear(x, wu, bu)
    w = interleave_gate_up(wg, wu).cuda()
    b = interleave_gate_up(bg, bu).cuda() if with_bias else None
    return x.cuda(), w, b, expected


@pytest.mark.parametrize("m", [1, 8, 13, 16, 100, 300, 1100])
@pytest.mark.parametrize("f", [8, 176, 1376])
@pytest.mark.parametrize("with_bias", [False, True], ids=["nobias", "bias"])
def test_linear_gated_epilogue(lib, m, f, with_bias):
    """activation="swiglu": silu(x·Wgᵀ) * (x·Wuᵀ) out of one GEMM over the interleaved weight, on
    the few-row kernel (m <= 16), the tensor-core kernel, and its split-K form (chosen by the
    planner for the middle sizes), against the two projections evaluated separately in fp32."""
    from kernl_b200.implementations.linear_layer import linear_layer

    x, w, b, expected = _gated_case(m, 264, f, torch.bfloat16, with_bias)
    for _ in range(2):  # twice: a split-K workspace must come back clean
        out = linear_layer(x, w, b, activation="swiglu")
    assert out.shape == (m, f)
    O.assert_parity(out, expected, max_abs=3e-2)


@pytest.mark.parametrize("bn", [32, 64, 128, 256])
@pytest.mark.parametrize("splits", [1, 3])
def test_linear_gated_epilogue_every_tile_width(lib, bn, splits):
    from kernl_b200.implementations.linear_layer import linear_layer

    x, w, b, expected = _gated_case(200, 512, 328, torch.float16, True, seed=1)
    try:
        lib.kb_debug_force_bn(bn)
        lib.kb_debug_force_splits(splits)
        for _ in range(2):
            out = linear_layer(x, w, b, activation="swiglu")
    finally:
        lib.kb_debug_force_bn(0)
        lib.kb_debug_force_splits(0)
    O.assert_parity(out, expected, max_abs=3e-2)


def test_linear_gated_epilogue_rejects_bad_shapes(lib):
    from kernl_b200.implementations.linear_layer import linear_layer

    x = torch.zeros((4, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(AssertionError):
        linear_layer(x, torch.zeros((24, 64), dtype=torch.float16, device="cuda"), None, activation="swiglu")


def test_silu_mul(lib):
    from kernl_b200.implementations.linear_layer import silu_mul

    g = torch.Generator().manual_seed(0)
    gu = torch.randn((37, 2 * 176), generator=g).bfloat16()
    out = silu_mul(gu.cuda())
    gate, up = gu[:, :176].float(), gu[:, 176:].float()
    O.assert_parity(out, torch.nn.functional.silu(gate) * up, max_abs=3e-2)


# ------------------------------------------------------------------------------------------------
# norms
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [128, 512, 1024, 2048, 4096, 768, 250, 5120, 8192])
@pytest.mark.parametrize("rms", [False, True], ids=["layernorm", "rmsnorm"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
def test_norm_reference_shapes(lib, n, rms, dtype):
    """x = -20 + 0.5*randn stresses the mean subtraction (test/test_layer_norm.py:58)."""
    from kernl_b200.implementations.layer_norm import layer_norm

    g = torch.Generator().manual_seed(0)
    rows = min(n, 512)
    x = (-20 + 0.5 * torch.randn((rows, n), generator=g)).to(dtype)
    w = (torch.rand((n,), generator=g) + 0.5).to(dtype)
    b = (torch.randn((n,), generator=g) * 0.1).to(dtype)
    eps = O.kernel_eps(1e-5, dtype)
    expected = O.rms_norm(x, w, eps) if rms else O.layer_norm(x, w, b, eps)
    xc, wc, bc = _cuda(x, w, b)
    out = layer_norm(xc, wc, None if rms else bc, 1e-5, use_rms_norm=rms)
    # bf16: outputs up to ~5 in magnitude, ulp 3.1e-2
    O.assert_parity(out, expected, max_abs=1e-2 if dtype == torch.float16 else 4e-2)


def test_norm_stride_and_3d(lib):
    """Transposed 250x250 input (test/test_layer_norm.py:110-123) and a 3-D input."""
    from kernl_b200.implementations.layer_norm import layer_norm

    g = torch.Generator().manual_seed(0)
    x = torch.randn((250, 250), generator=g).half().cuda().t()
    w, b = torch.rand((250,), generator=g).half().cuda(), torch.randn((250,), generator=g).half().cuda()
    out = layer_norm(x, w, b, 1e-5)
    O.assert_parity(out, O.layer_norm(x, w, b, 1.6e-5))
    x3 = torch.randn((3, 17, 768), generator=g).half().cuda()
    w3, b3 = torch.rand((768,), generator=g).half().cuda(), torch.randn((768,), generator=g).half().cuda()
    out3 = layer_norm(x3, w3, b3, 1e-12)
    assert out3.shape == x3.shape
    O.assert_parity(out3, O.layer_norm(x3, w3, b3, 1.6e-5))


@pytest.mark.parametrize("n", [128, 250, 768])
def test_norm_against_reference_golden(lib, n):
    from kernl_b200.implementations.layer_norm import layer_norm

    g = np.load(os.path.join(GOLDEN, "norm_reference.npz"))
    x, w, b = (torch.from_numpy(g[f"n{n}_{t}"]).half() for t in "xwb")
    xc, wc, bc = _cuda(x, w, b)
    O.assert_parity(layer_norm(xc, wc, bc, 1e-5), O.layer_norm(x, w, b, 1.6e-5))
    O.assert_parity(layer_norm(xc, wc, None, 1e-6, use_rms_norm=True), O.rms_norm(x, w, 1.6e-5))
    # raw golden outputs (computed from fp32 inputs): x = -20 ± 0.5 loses ~1e-2 when rounded to
    # fp16, which (x-mean)*rstd amplifies by 1/0.5, hence the looser bound
    O.assert_parity(layer_norm(xc, wc, bc, 1e-5), torch.from_numpy(g[f"n{n}_f_ln"]), max_abs=8e-2, cos=0.999)


def test_norm_full_size_properties(lib):
    """[16384, 4096] rows: output of LayerNorm with gamma=1, beta=0 has zero mean and unit
    variance per row; RMSNorm output has unit mean square; sampled rows match the oracle."""
    from kernl_b200.implementations.layer_norm import layer_norm

    g = torch.Generator().manual_seed(0)
    x = torch.randn((16384, 4096), generator=g).half().cuda()
    one, zero = torch.ones(4096).half().cuda(), torch.zeros(4096).half().cuda()
    y = layer_norm(x, one, zero, 1e-5).float()
    assert y.mean(-1).abs().max() < 2e-3 and (y.var(-1, unbiased=False) - 1).abs().max() < 5e-3
    r = layer_norm(x, one, None, 1e-5, use_rms_norm=True).float()
    assert (r.pow(2).mean(-1) - 1).abs().max() < 5e-3
    rows = torch.tensor([0, 1, 8191, 16383])
    O.assert_parity(y[rows.cuda()], O.layer_norm(x[rows.cuda()].cpu(), one.cpu(), zero.cpu(), 1.6e-5))


@pytest.mark.parametrize("rows,cols", [(16384, 768), (9001, 768), (40000, 256), (8200, 1000), (5000, 1024)])
@pytest.mark.parametrize("rms", [False, True], ids=["layernorm", "rmsnorm"])
@pytest.mark.parametrize("with_residual", [False, True], ids=["plain", "residual"])
def test_norm_many_short_rows(lib, rows, cols, rms, with_residual):
    """Many rows of at most 1024 columns (one warp per row, four rows per CTA): every row against the
    oracle, ragged row counts included, with and without the fused residual add."""
    from kernl_b200.implementations.layer_norm import layer_norm

    g = torch.Generator().manual_seed(rows)
    x = (1.5 * torch.randn((rows, cols), generator=g) + 0.3).half()
    res = torch.randn((rows, cols), generator=g).half() if with_residual else None
    w = (torch.rand((cols,), generator=g) + 0.5).half()
    b = (torch.randn((cols,), generator=g) * 0.1).half()
    xc, wc, bc = _cuda(x, w, b)
    if with_residual:
        y, s = layer_norm(xc, wc, None if rms else bc, 1e-5, use_rms_norm=rms, residual=res.cuda())
        base = (x.float() + res.float()).half()
        assert torch.equal(s.cpu(), base)
    else:
        y = layer_norm(xc, wc, None if rms else bc, 1e-5, use_rms_norm=rms)
        base = x
    expected = O.rms_norm(base, w, 1.6e-5) if rms else O.layer_norm(base, w, b, 1.6e-5)
    O.assert_parity(y, expected, what=f"{rows} x {cols}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(8, 4096), (3, 7, 768), (1, 8), (513, 6144)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_with_residual(lib, shape, rms, dtype):
    """Fused pre-norm add: the returned sum is the exactly rounded x + residual, the normed output
    matches the oracle applied to that sum."""
    from kernl_b200.implementations.layer_norm import layer_norm

    g = torch.Generator().manual_seed(3)
    x = torch.randn(shape, generator=g).to(dtype)
    res = (2 * torch.randn(shape, generator=g)).to(dtype)
    n = shape[-1]
    w = (torch.rand((n,), generator=g) + 0.5).to(dtype)
    b = (torch.randn((n,), generator=g) * 0.1).to(dtype)
    xc, rc, wc, bc = _cuda(x, res, w, b)
    y, s = layer_norm(xc, wc, None if rms else bc, 1e-5, use_rms_norm=rms, residual=rc)
    want_sum = (x.float() + res.float()).to(dtype)
    assert torch.equal(s.cpu(), want_sum)
    eps = O.kernel_eps(1e-5, dtype)
    expected = O.rms_norm(want_sum, w, eps) if rms else O.layer_norm(want_sum, w, b, eps)
    O.assert_parity(y, expected, max_abs=1e-2 if dtype == torch.float16 else 4e-2)
    # the plain call on the sum gives the same bits
    assert torch.equal(y, layer_norm(s, wc, None if rms else bc, 1e-5, use_rms_norm=rms))


def test_eps_clamp_only_for_fp16(lib):
    """fp16 clamps eps to 1.6e-5 (reference layer_norm.py:295-296); bf16 does not."""
    from kernl_b200.implementations.layer_norm import layer_norm

    x = torch.full((4, 128), 3e-3).cuda()
    x[:, ::2] = -3e-3  # variance 9e-6, comparable to the clamp
    w, b = torch.ones(128).cuda(), torch.zeros(128).cuda()
    out16 = layer_norm(x.half(), w.half(), b.half(), 1e-12).float()
    outbf = layer_norm(x.bfloat16(), w.bfloat16(), b.bfloat16(), 1e-12).float()
    assert abs(out16.abs().max().item() - (3e-3 / (9e-6 + 1.6e-5) ** 0.5)) < 2e-2
    assert abs(outbf.abs().max().item() - 1.0) < 2e-2
