"""CPU oracle of the adaLN-Zero elementwise ops of the DiT block (test infrastructure, not a product path).

``modulate`` / ``block_branch`` restate the reference's formulas (models/layers.py:28-29 ``modulate``, :195-201
``DiTBlock.forward``, :217-221 ``FinalLayer.forward``) in plain PyTorch, so that ``torch.func.jvp`` and autograd
through them are the reference's own arithmetic; the ``*_closed_form`` functions are the fp64 formulas the CUDA
kernels implement, pinned against autodiff of the restated forms in tests/test_oracle.py.  The DiT block as a whole
is also pinned by the model fixtures generated from the reference's DMFT (tests/golden/make_golden_model.py).

Only tests/, the smoke test and the CPU-baseline leg of the bench may import this file.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def modulate(x, shift, scale):
    """models/layers.py:28-29."""
    return x * (1 + scale) + shift


def ln_modulate(x, shift, scale, eps: float = 1e-6):
    """modulate(norm(x), shift, scale) with norm = LayerNorm(C, elementwise_affine=False, eps):
    models/layers.py:196-197, 219.  shift / scale are (B, 1, C)."""
    return modulate(F.layer_norm(x, (x.shape[-1],), eps=eps), shift, scale)


def gate_residual(x, gate, h):
    """x + gate * h, models/layers.py:196-197."""
    return x + gate * h


def ln_modulate_jvp_closed_form(x, tx, shift, scale, tshift, tscale, eps: float = 1e-6):
    """fp64 (y, ty): n = (x - mean x) r, r = rsqrt(var x + eps) (biased variance),
    y = n (1 + scale) + shift,  tn = r (tx - mean tx - n mean(n tx_c)),  ty = tn (1 + scale) + n tscale + tshift."""
    xd, td = x.double(), tx.double()
    sh, sc, tsh, tsc = (t.double() for t in (shift, scale, tshift, tscale))
    xc = xd - xd.mean(-1, keepdim=True)
    r = torch.rsqrt(xc.pow(2).mean(-1, keepdim=True) + eps)
    n = xc * r
    tc = td - td.mean(-1, keepdim=True)
    tn = r * (tc - n * (n * tc).mean(-1, keepdim=True))
    return n * (1 + sc) + sh, tn * (1 + sc) + n * tsc + tsh


def ln_modulate_bwd_closed_form(dy, x, scale, eps: float = 1e-6):
    """fp64 (dx, dshift, dscale) of y = LayerNorm(x) (1 + scale) + shift; dshift / dscale are (B, 1, C)."""
    xd, gy, sc = x.double(), dy.double(), scale.double()
    xc = xd - xd.mean(-1, keepdim=True)
    r = torch.rsqrt(xc.pow(2).mean(-1, keepdim=True) + eps)
    n = xc * r
    g = gy * (1 + sc)
    dx = r * (g - g.mean(-1, keepdim=True) - n * (g * n).mean(-1, keepdim=True))
    return dx, gy.sum(1, keepdim=True), (gy * n).sum(1, keepdim=True)


def gate_residual_jvp_closed_form(x, tx, h, th, gate, tgate):
    """fp64 (out, tout) of x + gate h."""
    xd, td, hd, thd, g, tg = (t.double() for t in (x, tx, h, th, gate, tgate))
    return xd + g * hd, td + tg * hd + g * thd


def gate_residual_bwd_closed_form(dout, h, gate):
    """fp64 (dx, dh, dgate) of out = x + gate h; dgate is (B, 1, C)."""
    go, hd, g = dout.double(), h.double(), gate.double()
    return go, g * go, (go * hd).sum(1, keepdim=True)
