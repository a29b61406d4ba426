"""Drop-in for the reference's flash_attn_func with forward-mode (JVP) support.

Same surface as models/flash_attention_2_jvp.py and models/flash_attention_3_jvp.py:

* ``flash_attn_func(q, k, v, softmax_scale=None)`` on (B, L, H, D) tensors.  When
  any of q, k, v is a forward-AD dual tensor the fused forward + tangent kernel
  runs and a dual tensor comes back; otherwise the plain forward runs
  (flash_attention_2_jvp.py:294-319).
* ``FlashAttnFunc`` - a new-style autograd.Function (forward without ctx +
  setup_context, so functorch transforms accept it) that takes the tangents as
  ordinary inputs and returns ``(o, lse, to)`` (flash_attention_2_jvp.py:177-282).
  ``backward`` differentiates the primal output only: gradients arriving for
  ``lse`` and for the tangent output are dropped and ``None`` is returned for the
  tangent inputs and the scale - the stop-gradient-on-tangent behaviour that
  loss.py:171-173 relies on.  ``jvp`` hands back the saved tangent output.

* ``flash_attn_qkvpacked_func(qkv, softmax_scale=None)`` on the (B, L, 3, H, D) view of the packed projection
  (models/layers.py:143-146 builds q, k, v as its slices): the same computation, but the backward writes dq, dk, dv
  straight into one packed gradient instead of three tensors that autograd then copies together.

Every compute step is a kernel of the sm_100a library; there is no Triton, no
PyTorch fallback and no CPU path.
"""

from __future__ import annotations

import torch
import torch.autograd.forward_ad as fwAD

from . import ops


class FlashAttnFunc(torch.autograd.Function):

    @staticmethod
    def forward(q, k, v, tq, tk, tv, softmax_scale):
        # q, k, v: (B, L, H, D); default scale uses the true head dim (flash_attention_2_jvp.py:182-183)
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        enable_jvp = (tq is not None) and (tk is not None) and (tv is not None)
        if enable_jvp:
            o, to, m = torch.ops.dmf_b200.attn_fwd_dual(q, k, v, tq, tk, tv, float(softmax_scale))
        else:
            to = None
            o, m = torch.ops.dmf_b200.attn_fwd(q, k, v, float(softmax_scale))
        return o, m, to

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        q, k, v, tq, tk, tv, softmax_scale = inputs
        o, m, to = outputs
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        ctx.save_for_backward(q, k, v, o, m)
        if tq is not None and tk is not None and tv is not None:
            ctx.save_for_forward(to)
        ctx.softmax_scale = softmax_scale

    @staticmethod
    def backward(ctx, dout, *args):
        # *args: gradients w.r.t. lse and the tangent output - ignored on purpose
        q, k, v, o, m = ctx.saved_tensors
        dq, dk, dv = torch.ops.dmf_b200.attn_bwd(dout, q, k, v, o, m, float(ctx.softmax_scale))
        return dq, dk, dv, None, None, None, None

    @staticmethod
    def jvp(ctx, *args):
        t_saved = getattr(ctx, "saved_forward", ())
        to = t_saved[0] if len(t_saved) > 0 else None
        return to, None, None


def _is_dual_mode(*tensors):
    """True if any tensor carries a forward-AD tangent (flash_attention_2_jvp.py:285-291)."""
    for tensor in tensors:
        _, tangent = fwAD.unpack_dual(tensor)
        if tangent is not None:
            return True
    return False


def flash_attn_func(q, k, v, softmax_scale=None):
    if _is_dual_mode(q, k, v):
        primals, tangents = [], []
        for tensor in (q, k, v):
            primal, tangent = fwAD.unpack_dual(tensor)
            primals.append(primal)
            tangents.append(torch.zeros_like(primal) if tangent is None else tangent)
        out, _, t_out = FlashAttnFunc.apply(*primals, *tangents, softmax_scale)
        return fwAD.make_dual(out, t_out)
    out, _, _ = FlashAttnFunc.apply(q, k, v, None, None, None, softmax_scale)
    return out


class FlashAttnQKVPackedFunc(torch.autograd.Function):
    """FlashAttnFunc on the (B, L, 3, H, D) packed projection; the gradient comes back packed."""

    @staticmethod
    def forward(qkv, tqkv, softmax_scale):
        if softmax_scale is None:
            softmax_scale = qkv.shape[-1] ** (-0.5)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if tqkv is not None:
            o, to, m = torch.ops.dmf_b200.attn_fwd_dual(q, k, v, tqkv[:, :, 0], tqkv[:, :, 1], tqkv[:, :, 2],
                                                        float(softmax_scale))
        else:
            to = None
            o, m = torch.ops.dmf_b200.attn_fwd(q, k, v, float(softmax_scale))
        return o, m, to

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        qkv, tqkv, softmax_scale = inputs
        o, m, to = outputs
        ctx.save_for_backward(qkv, o, m)
        if tqkv is not None:
            ctx.save_for_forward(to)
        ctx.softmax_scale = qkv.shape[-1] ** (-0.5) if softmax_scale is None else softmax_scale

    @staticmethod
    def backward(ctx, dout, *args):
        qkv, o, m = ctx.saved_tensors
        return torch.ops.dmf_b200.attn_bwd_qkvpacked(dout, qkv, o, m, float(ctx.softmax_scale)), None, None

    @staticmethod
    def jvp(ctx, *args):
        t_saved = getattr(ctx, "saved_forward", ())
        return (t_saved[0] if len(t_saved) > 0 else None), None, None


def flash_attn_qkvpacked_func(qkv, softmax_scale=None):
    if qkv.dim() != 5 or qkv.shape[2] != 3:
        raise ValueError("expected a (B, L, 3, H, D) tensor")
    primal, tangent = fwAD.unpack_dual(qkv)
    if tangent is not None:
        out, _, t_out = FlashAttnQKVPackedFunc.apply(primal, tangent, softmax_scale)
        return fwAD.make_dual(out, t_out)
    return FlashAttnQKVPackedFunc.apply(qkv, None, softmax_scale)[0]
