"""Input casting shared by the op front-ends.

The reference decorates every op's forward with `custom_fwd(cast_inputs=torch.float16)`
(src/kernl/implementations/attention.py:440, linear_layer.py:215, layer_norm.py:281): under
`torch.autocast` every floating-point tensor argument is cast to fp16 — the mask and the
caller-provided output included — and autocast is switched off inside; outside autocast the
arguments pass through unchanged.
"""
import torch


def autocast_active() -> bool:
    return torch.is_autocast_enabled()


def cast_if_autocast(*tensors):
    if not autocast_active():
        return tensors
    out = []
    for t in tensors:
        if isinstance(t, torch.Tensor) and t.is_floating_point() and t.dtype != torch.float16:
            t = t.to(torch.float16)
        out.append(t)
    return tuple(out)
