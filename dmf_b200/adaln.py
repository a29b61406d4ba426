"""adaLN-Zero elementwise ops of the DiT block as single kernels, with forward-mode (JVP) support.

The reference's block (models/layers.py:195-201) computes

    x = x + gate * branch(modulate(norm(x), shift, scale))        modulate: x * (1 + scale) + shift

with ``norm`` a LayerNorm without affine parameters.  Under ``torch.func.jvp`` (loss.py:149-166)
forward-mode AD runs ``modulate(norm(x), ...)`` and ``x + gate * h`` as about twenty elementwise and
reduction kernels each.  ``ln_modulate`` and ``gate_residual`` compute the same functions in one
pass over the rows, and when an input is a forward-AD dual tensor the tangent in the same pass.

Like the attention op (flash_attn_jvp.py), ``backward`` differentiates the primal outputs only:
gradients arriving for a tangent output are dropped and tangent inputs get ``None``.  That is exact
for the reference's losses, which detach everything computed from the tangent (loss.py:171-173).

dtypes: the residual stream ``x`` is fp32 (training under bf16 autocast) or bf16 (a bf16 model);
what feeds a matmul or leaves one (``ln_modulate``'s result, ``h``) is bf16, or fp32 with an fp32
stream; shift / scale / gate are bf16 or fp32.  ``ln_modulate`` writes its result directly in the
autocast dtype when autocast is on - the cast autocast would insert before the next Linear.
Arithmetic is fp32 with one rounding of each result (the reference rounds after every op).

There is no other implementation behind these functions: without the CUDA library they raise.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.autograd.forward_ad as fwAD

from . import _lib
from . import ops as _ops

WIDTHS = (384, 768, 1024, 1152)   # hidden sizes the row kernels are compiled for (DMFT-S/B/L/XL)
_ADA = {torch.bfloat16: _lib.ADALN_BF16, torch.float32: _lib.ADALN_F32}
_PAIRS = {(torch.float32, torch.float32), (torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16)}


def _rows_ok(t: torch.Tensor) -> torch.Tensor:
    """Rows the kernels can read as 4-element vectors: unit channel stride, 16-byte aligned base, row strides
    that are multiples of 4 elements."""
    if not t.is_cuda:
        raise RuntimeError("dmf_b200 adaLN ops run on CUDA (sm_100a) only; there is no CPU path")
    if t.dim() != 3:
        raise ValueError("expected a (B, L, C) tensor")
    if t.stride(-1) != 1 or t.data_ptr() % 16 or any(s % 4 for s in t.stride()[:-1]):
        return t.contiguous()
    return t


def _mod_ok(t: torch.Tensor, B: int, Cn: int, dtype: torch.dtype) -> torch.Tensor:
    """A (B, C) or (B, 1, C) modulation tensor as a 2-D view with unit channel stride."""
    if t.dim() == 3:
        if t.shape[1] != 1:
            raise ValueError("shift / scale / gate must be (B, C) or (B, 1, C)")
        t = t[:, 0]
    if t.shape != (B, Cn):
        raise ValueError(f"shift / scale / gate must have shape ({B}, {Cn}), got {tuple(t.shape)}")
    if t.dtype != dtype:
        t = t.to(dtype)
    if t.stride(-1) != 1 or t.data_ptr() % 16 or t.stride(0) % 4:
        t = t.contiguous()
    return t


def _rows(t: Optional[torch.Tensor]) -> _lib.Rows:
    return _lib.Rows(None, 0, 0) if t is None else _lib.Rows(t.data_ptr(), t.stride(0), t.stride(1))


def _mod(t: Optional[torch.Tensor]) -> _lib.Mod:
    return _lib.Mod(None, 0) if t is None else _lib.Mod(t.data_ptr(), t.stride(0))


def _head(a, x: torch.Tensor, narrow: torch.dtype, mod: torch.dtype) -> None:
    if not x.is_cuda:
        raise RuntimeError("dmf_b200 adaLN ops run on CUDA (sm_100a) only; there is no CPU path")
    if (x.dtype, narrow) not in _PAIRS or mod not in _ADA:
        raise TypeError(f"unsupported dtypes: stream {x.dtype}, matmul side {narrow}, modulation {mod}")
    a.batch, a.seqlen, a.channels = x.shape
    a.wide_dtype, a.narrow_dtype, a.mod_dtype = _ADA[x.dtype], _ADA[narrow], _ADA[mod]
    a.stream = torch.cuda.current_stream(x.device).cuda_stream


def _mod_dtype(*mods) -> torch.dtype:
    return torch.float32 if any(m is not None and m.dtype == torch.float32 for m in mods) else torch.bfloat16


def _workspace(x: torch.Tensor):
    B, L, Cn = x.shape
    nbytes = _lib.load().dmf_adaln_bwd_workspace_bytes(B, L, Cn)
    return torch.empty((nbytes,), dtype=torch.uint8, device=x.device), nbytes


def ln_modulate_fwd_raw(x, tx, shift, scale, tshift, tscale, eps: float, out_dtype: torch.dtype):
    """y (and ty when tx is given) of LayerNorm(x) * (1 + scale) + shift; one kernel."""
    x = _rows_ok(x)
    B, L, Cn = x.shape
    md = _mod_dtype(shift, scale, tshift, tscale)
    shift, scale = _mod_ok(shift, B, Cn, md), _mod_ok(scale, B, Cn, md)
    if tx is not None:
        tx = _rows_ok(tx.to(x.dtype))
        if (tshift is None) != (tscale is None):   # the kernel takes the two modulation tangents together
            tshift = torch.zeros_like(shift) if tshift is None else tshift
            tscale = torch.zeros_like(scale) if tscale is None else tscale
        if tshift is not None:
            tshift, tscale = _mod_ok(tshift, B, Cn, md), _mod_ok(tscale, B, Cn, md)
    with torch.cuda.device(x.device):
        y = torch.empty((B, L, Cn), dtype=out_dtype, device=x.device)
        ty = None if tx is None else torch.empty((B, L, Cn), dtype=out_dtype, device=x.device)
        a = _lib.LnModulateArgs()
        _head(a, x, out_dtype, md)
        a.eps = float(eps)
        a.x, a.tx, a.y, a.ty = _rows(x), _rows(tx), _rows(y), _rows(ty)
        a.shift, a.scale = _mod(shift), _mod(scale)
        a.tshift, a.tscale = (_mod(tshift), _mod(tscale)) if tx is not None else (_mod(None), _mod(None))
        _lib.check(_lib.load().dmf_ln_modulate_fwd(C.byref(a)))
        _ops.launch_count += 1
    return y, ty


def ln_modulate_bwd_raw(dy, x, scale, eps: float):
    """dx (like x), dshift and dscale ((B, C) fp32) of y = LayerNorm(x) * (1 + scale) + shift."""
    x, dy = _rows_ok(x), _rows_ok(dy)
    B, L, Cn = x.shape
    md = _mod_dtype(scale)
    scale = _mod_ok(scale, B, Cn, md)
    with torch.cuda.device(x.device):
        dx = torch.empty((B, L, Cn), dtype=x.dtype, device=x.device)
        dmod = torch.empty((2, B, Cn), dtype=torch.float32, device=x.device)
        ws, nbytes = _workspace(x)
        a = _lib.LnModulateBwdArgs()
        _head(a, x, dy.dtype, md)
        a.eps = float(eps)
        a.dy, a.x, a.dx, a.scale = _rows(dy), _rows(x), _rows(dx), _mod(scale)
        a.dshift, a.dscale = dmod[0].data_ptr(), dmod[1].data_ptr()
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
        _lib.check(_lib.load().dmf_ln_modulate_bwd(C.byref(a)))
        _ops.launch_count += 2
    return dx, dmod[0], dmod[1]


def gate_residual_fwd_raw(x, tx, h, th, gate, tgate):
    """out (and tout when tx / th are given) of x + gate * h; one kernel."""
    x, h = _rows_ok(x), _rows_ok(h)
    B, L, Cn = x.shape
    if h.shape != x.shape:
        raise ValueError("x and h must have the same shape")
    md = _mod_dtype(gate, tgate)
    gate = _mod_ok(gate, B, Cn, md)
    dual = tx is not None or th is not None or tgate is not None
    if dual:
        tx = _rows_ok(torch.zeros_like(x) if tx is None else tx.to(x.dtype))
        th = _rows_ok(torch.zeros_like(h) if th is None else th.to(h.dtype))
        tgate = None if tgate is None else _mod_ok(tgate, B, Cn, md)
    with torch.cuda.device(x.device):
        out = torch.empty((B, L, Cn), dtype=x.dtype, device=x.device)
        tout = torch.empty((B, L, Cn), dtype=x.dtype, device=x.device) if dual else None
        a = _lib.GateResidualArgs()
        _head(a, x, h.dtype, md)
        a.x, a.h, a.out, a.gate = _rows(x), _rows(h), _rows(out), _mod(gate)
        a.tx, a.th, a.tout, a.tgate = _rows(tx if dual else None), _rows(th if dual else None), _rows(tout), _mod(tgate if dual else None)
        _lib.check(_lib.load().dmf_gate_residual_fwd(C.byref(a)))
        _ops.launch_count += 1
    return out, tout


def gate_residual_bwd_raw(dout, h, gate):
    """dh (like h) and dgate ((B, C) fp32) of out = x + gate * h (dx is dout itself)."""
    dout, h = _rows_ok(dout), _rows_ok(h)
    B, L, Cn = h.shape
    md = _mod_dtype(gate)
    gate = _mod_ok(gate, B, Cn, md)
    with torch.cuda.device(h.device):
        dh = torch.empty((B, L, Cn), dtype=h.dtype, device=h.device)
        dgate = torch.empty((B, Cn), dtype=torch.float32, device=h.device)
        ws, nbytes = _workspace(h)
        a = _lib.GateResidualBwdArgs()
        _head(a, dout, h.dtype, md)
        a.dout, a.h, a.dh, a.gate = _rows(dout), _rows(h), _rows(dh), _mod(gate)
        a.dgate = dgate.data_ptr()
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
        _lib.check(_lib.load().dmf_gate_residual_bwd(C.byref(a)))
        _ops.launch_count += 2
    return dh, dgate


def _like(grad: torch.Tensor, ref_shape, ref_dtype) -> torch.Tensor:
    return grad.to(ref_dtype).reshape(ref_shape)


class LnModulateFunc(torch.autograd.Function):

    @staticmethod
    def forward(x, tx, shift, scale, tshift, tscale, eps, out_dtype):
        return ln_modulate_fwd_raw(x, tx, shift, scale, tshift, tscale, eps, out_dtype)

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        x, _, shift, scale, _, _, eps, _ = inputs
        ctx.save_for_backward(x, scale)
        if outputs[1] is not None:
            ctx.save_for_forward(outputs[1])
        ctx.eps = float(eps)
        ctx.mod_meta = (shift.shape, shift.dtype, scale.shape, scale.dtype)

    @staticmethod
    def backward(ctx, dy, *unused):
        # *unused: the gradient of the tangent output - ignored on purpose
        x, scale = ctx.saved_tensors
        dx, dshift, dscale = ln_modulate_bwd_raw(dy, x, scale, ctx.eps)
        s_shape, s_dtype, c_shape, c_dtype = ctx.mod_meta
        return dx, None, _like(dshift, s_shape, s_dtype), _like(dscale, c_shape, c_dtype), None, None, None, None

    @staticmethod
    def jvp(ctx, *tangents):
        # the tangent was computed in forward from the tangents passed as plain inputs (like FlashAttnFunc.jvp)
        saved = getattr(ctx, "saved_forward", ())
        return (saved[0] if len(saved) > 0 else None), None


class GateResidualFunc(torch.autograd.Function):

    @staticmethod
    def forward(x, tx, h, th, gate, tgate):
        return gate_residual_fwd_raw(x, tx, h, th, gate, tgate)

    @staticmethod
    def setup_context(ctx, inputs, outputs):
        _, _, h, _, gate, _ = inputs
        ctx.save_for_backward(h, gate)
        if outputs[1] is not None:
            ctx.save_for_forward(outputs[1])
        ctx.gate_meta = (gate.shape, gate.dtype)

    @staticmethod
    def backward(ctx, dout, *unused):
        h, gate = ctx.saved_tensors
        dh, dgate = gate_residual_bwd_raw(dout, h, gate)
        return dout, None, dh, None, _like(dgate, *ctx.gate_meta), None

    @staticmethod
    def jvp(ctx, *tangents):
        saved = getattr(ctx, "saved_forward", ())
        return (saved[0] if len(saved) > 0 else None), None


def usable(x: torch.Tensor, h_dtype: Optional[torch.dtype] = None) -> bool:
    """Whether the kernels cover this residual stream: CUDA, (B, L, C) with a compiled width, fp32 or bf16,
    and (under autocast) bf16 as the autocast dtype."""
    if not (x.is_cuda and x.dim() == 3 and x.shape[-1] in WIDTHS and x.dtype in (torch.float32, torch.bfloat16)):
        return False
    if torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") != torch.bfloat16:
        return False
    return h_dtype is None or (x.dtype, h_dtype) in _PAIRS


def ln_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``F.layer_norm(x, (C,), eps=eps) * (1 + scale) + shift`` for x (B, L, C) and shift / scale (B, C) or
    (B, 1, C); dual tensors in give a dual tensor out.  The result has ``out_dtype`` (default: the autocast
    dtype when autocast is on, else x's dtype)."""
    if out_dtype is None:
        out_dtype = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else x.dtype
    xp, xt = fwAD.unpack_dual(x)
    sp, st = fwAD.unpack_dual(shift)
    cp, ct = fwAD.unpack_dual(scale)
    if xt is None and st is None and ct is None:
        return LnModulateFunc.apply(x, None, shift, scale, None, None, eps, out_dtype)[0]
    if xt is None:
        xt = torch.zeros_like(xp)
    y, ty = LnModulateFunc.apply(xp, xt, sp, cp, st, ct, eps, out_dtype)
    return fwAD.make_dual(y, ty)


def gate_residual(x: torch.Tensor, gate: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
    """``x + gate * h`` for x, h (B, L, C) and gate (B, C) or (B, 1, C); the result has x's dtype; dual tensors
    in give a dual tensor out."""
    xp, xt = fwAD.unpack_dual(x)
    hp, ht = fwAD.unpack_dual(h)
    gp, gt = fwAD.unpack_dual(gate)
    if xt is None and ht is None and gt is None:
        return GateResidualFunc.apply(x, None, h, None, gate, None)[0]
    out, tout = GateResidualFunc.apply(xp, xt, hp, ht, gp, gt)
    return fwAD.make_dual(out, tout)
