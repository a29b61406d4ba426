"""CPU oracle for the end of an optimisation step.  TEST INFRASTRUCTURE ONLY (never imported by ``dmf_b200``).

Restates in float64 what train_dmf.py:331-338 computes after backward: ``clip_grad_norm_`` (scale by
``min(1, max_norm / (norm + 1e-6))``), one step of ``torch.optim.AdamW`` (train_dmf.py:221-228; decoupled weight
decay, bias-corrected moments), ``zero_grad`` and ``update_ema`` (train_dmf.py:54-99: ``ema = ema * decay +
p * (1 - decay)``).  Pinned in tests/test_oracle.py against those very library calls on CPU.
"""

from __future__ import annotations

import math

import torch


def step_tail(grad, param, exp_avg, exp_avg_sq, ema, *, step: int, lr=1e-4, betas=(0.9, 0.95), eps=1e-8,
              weight_decay=0.0, max_grad_norm=1.0, ema_decay=0.9999):
    """Returns (param, exp_avg, exp_avg_sq, ema) after the step, all float64; ``step`` counts from 1."""
    g, p, m, v = grad.double(), param.double(), exp_avg.double(), exp_avg_sq.double()
    if max_grad_norm is not None:
        g = g * min(1.0, max_grad_norm / (float(g.norm(2)) + 1e-6))
    p = p * (1.0 - lr * weight_decay)
    m = m + (1.0 - betas[0]) * (g - m)
    v = betas[1] * v + (1.0 - betas[1]) * g * g
    denom = v.sqrt() / math.sqrt(1.0 - betas[1] ** step) + eps
    p = p - (lr / (1.0 - betas[0] ** step)) * m / denom
    e = None if ema is None else ema.double() * ema_decay + p * (1.0 - ema_decay)
    return p, m, v, e
