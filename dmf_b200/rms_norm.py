"""Per-head RMS norm of q / k as one kernel, with forward-mode (JVP) support.

The reference normalises q and k with ``RMSNorm`` (models/layers.py:33-42, applied at
layers.py:148) written in elementwise PyTorch ops; under ``torch.func.jvp`` forward-mode AD turns
those into a dozen kernels over (B, L, H, D) tensors.  ``rms_norm(x, weight, eps)`` computes the
same function - ``x * rsqrt(mean(x^2, -1) + eps) * weight`` - in one pass, and when ``x`` is a
forward-AD dual tensor its tangent in the same pass.

Like the attention op (flash_attn_jvp.py), ``backward`` differentiates the primal output only:
gradients arriving for the tangent output are dropped and ``None`` is returned for the tangent
input.  That is exact for the reference's losses, which detach everything computed from the
tangent (loss.py:171-173).  ``weight`` is treated as a constant by forward mode (the reference
never seeds a parameter tangent) and receives its gradient in backward.

Arithmetic is fp32 with one rounding of the result; the reference rounds to the 16-bit type after
each elementwise step, so results agree to a few 16-bit ulps, not bit for bit.
"""

from __future__ import annotations

import torch
import torch.autograd.forward_ad as fwAD

from . import ops  # noqa: F401  (registers the custom ops)


class RmsNormFunc(torch.autograd.Function):

    @staticmethod
    def forward(x, tx, weight, eps):
        if tx is not None:
            y, ty = torch.ops.dmf_b200.rmsnorm_fwd_dual(x, tx, weight, float(eps))
        else:
            y, ty = torch.ops.dmf_b200.rmsnorm_fwd(x, weight, float(eps)), None
        return y, ty

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        x, tx, weight, eps = inputs
        _, ty = outputs
        ctx.save_for_backward(x, weight)
        if tx is not None:
            ctx.save_for_forward(ty)
        ctx.eps = float(eps)

    @staticmethod
    def backward(ctx, dy, *args):
        # *args: the gradient of the tangent output - ignored on purpose
        x, weight = ctx.saved_tensors
        dx, dw = torch.ops.dmf_b200.rmsnorm_bwd(dy, x, weight, ctx.eps)
        return dx, None, dw.to(weight.dtype), None

    @staticmethod
    def jvp(ctx, *args):
        saved = getattr(ctx, "saved_forward", ())
        return (saved[0] if len(saved) > 0 else None), None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm over the last dim of a (B, L, H, D) tensor; a dual tensor in gives a dual tensor out."""
    primal, tangent = fwAD.unpack_dual(x)
    if tangent is not None:
        w, _ = fwAD.unpack_dual(weight)
        y, ty = RmsNormFunc.apply(primal, tangent, w, eps)
        return fwAD.make_dual(y, ty)
    y, _ = RmsNormFunc.apply(x, None, weight, eps)
    return y
