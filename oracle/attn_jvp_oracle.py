"""CPU oracle for the attention forward-mode JVP path.  TEST INFRASTRUCTURE ONLY.

This module is the checker that the CUDA kernels are compared against.  It is
never imported by the product package (``dmf_b200``); only the tests, the
smoke entry and the CPU-baseline / reference arm of the benchmark use it.

It restates, on CPU, what the reference computes on this path:

* ``base_attention``       - the ``'base'`` branch of ``attn_op``
                             (models/layers.py:100-114): scale q, q @ k^T,
                             softmax, @ v, on (B, L, H, D) tensors.
* ``raw_attention``        - the in-test oracle ``raw_attn_func``
                             (models/flash_attention_2_jvp.py:322-336): same
                             math with the division by sqrt(D) after the matmul.
* ``attn_jvp_base``        - ``torch.func.jvp`` through ``base_attention``,
                             which is how loss.py:165-170 reaches the op.
* ``attn_jvp_closed_form`` - the explicit formula in float64:
                               S  = s * Q K^T,  P = softmax(S),  O = P V
                               dS = s * (dQ K^T + Q dK^T)
                               dP = P * (dS - rowsum(P * dS))
                               dO = dP V + P dV
                             plus LSE = logsumexp(S) (natural log), the quantity
                             the reference stores in ``m``
                             (models/triton_utils.py:346-348).
* ``attn_jvp_online``      - the single-pass online-softmax recurrence over KV
                             blocks (models/triton_utils.py:51-127), written in
                             its un-normalised form, optionally with the same
                             rounding points as the bf16 kernel (bf16 P and
                             P*dS before the V products).
* ``attn_bwd_base``        - primal backward through autograd of
                             ``base_attention`` (what ``test_jvp`` compares
                             against, flash_attention_2_jvp.py:361-369).
* ``rms_norm``             - per-head RMSNorm of q/k (models/layers.py:33-42).

Parity pin: the reference holds no stored golden vectors for this path (its one
test is differential on unseeded CUDA randoms).  The pin used here is the
reference's own Python code imported from its source tree and run on seeded CPU
inputs; ``tests/golden/make_golden.py`` generates those vectors and
``tests/test_oracle.py`` checks every function above against them.
"""

from __future__ import annotations

import math
from functools import partial
from typing import Optional, Tuple

import torch

LOG2E = 1.4426950408889634


# ----------------------------------------------------------------------------
# reference restatements
# ----------------------------------------------------------------------------

def base_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """'base' branch of attn_op, models/layers.py:100-114.  (B, L, H, D) in/out."""
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    scale = q.shape[-1] ** -0.5
    q = q * scale
    attn = q @ k.transpose(-2, -1)
    attn = attn.softmax(dim=-1)
    x = attn @ v
    return x.transpose(1, 2)


def raw_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """raw_attn_func, models/flash_attention_2_jvp.py:322-336."""
    q, k, v = q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3)
    scores = torch.matmul(q, k.transpose(-2, -1)) / (q.shape[-1] ** 0.5)
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, v).permute(0, 2, 1, 3)


def attn_jvp_base(q, k, v, tq, tk, tv) -> Tuple[torch.Tensor, torch.Tensor]:
    """torch.func.jvp over the 'base' path; returns (O, dO), both (B, L, H, D)."""
    return torch.func.jvp(base_attention, (q, k, v), (tq, tk, tv))


def attn_jvp_closed_form(q, k, v, tq, tk, tv, softmax_scale: Optional[float] = None,
                         dtype=torch.float64):
    """Explicit JVP formula.  Returns (O, dO, LSE) with LSE of shape (B, H, Lq)."""
    d = q.shape[-1]
    s = d ** -0.5 if softmax_scale is None else softmax_scale
    Q, K, V, dQ, dK, dV = (x.to(dtype).transpose(1, 2) for x in (q, k, v, tq, tk, tv))
    S = s * (Q @ K.transpose(-2, -1))
    lse = torch.logsumexp(S, dim=-1)
    P = torch.exp(S - lse[..., None])
    O = P @ V
    dS = s * (dQ @ K.transpose(-2, -1) + Q @ dK.transpose(-2, -1))
    dP = P * (dS - (P * dS).sum(-1, keepdim=True))
    dO = dP @ V + P @ dV
    return O.transpose(1, 2), dO.transpose(1, 2), lse


def attn_fwd_closed_form(q, k, v, softmax_scale: Optional[float] = None, dtype=torch.float64):
    """Plain forward: (O, LSE)."""
    z = torch.zeros_like(q)
    o, _, lse = attn_jvp_closed_form(q, k, v, z, torch.zeros_like(k), torch.zeros_like(v),
                                     softmax_scale, dtype)
    return o, lse


def _round(x: torch.Tensor, emulate_bf16: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(x.dtype) if emulate_bf16 else x


def attn_jvp_online(q, k, v, tq, tk, tv, softmax_scale: Optional[float] = None,
                    block_kv: int = 128, emulate_bf16: bool = False, dtype=torch.float64):
    """Single-pass online softmax over KV blocks (models/triton_utils.py:51-127).

    Un-normalised form: running (m, l, mu, Oacc, Tacc); on a max change all four
    sums are scaled by alpha; epilogue O = Oacc/l, dO = Tacc/l - (mu/l) O,
    LSE = m + ln l.  With ``emulate_bf16`` P and P*dS are rounded to bf16 before
    the products with V / dV, as the reference kernel does
    (models/triton_utils.py:104-111).
    """
    d = q.shape[-1]
    s = d ** -0.5 if softmax_scale is None else softmax_scale
    Q, K, V, dQ, dK, dV = (x.to(dtype).transpose(1, 2) for x in (q, k, v, tq, tk, tv))
    B, H, Lq, D = Q.shape
    Lk = K.shape[2]
    m = torch.full((B, H, Lq), -math.inf, dtype=dtype)
    l = torch.zeros((B, H, Lq), dtype=dtype)
    mu = torch.zeros((B, H, Lq), dtype=dtype)
    Oacc = torch.zeros((B, H, Lq, D), dtype=dtype)
    Tacc = torch.zeros((B, H, Lq, D), dtype=dtype)
    for j in range(0, Lk, block_kv):
        Kj, Vj, dKj, dVj = (x[:, :, j:j + block_kv] for x in (K, V, dK, dV))
        S = s * (Q @ Kj.transpose(-2, -1))
        m_new = torch.maximum(m, S.amax(-1))
        alpha = torch.exp(m - m_new)
        P = torch.exp(S - m_new[..., None])
        dS = s * (dQ @ Kj.transpose(-2, -1) + Q @ dKj.transpose(-2, -1))
        G = P * dS
        l = l * alpha + P.sum(-1)
        mu = mu * alpha + G.sum(-1)
        Pr, Gr = _round(P, emulate_bf16), _round(G, emulate_bf16)
        Oacc = Oacc * alpha[..., None] + Pr @ Vj
        Tacc = Tacc * alpha[..., None] + Gr @ Vj + Pr @ dVj
        m = m_new
    O = Oacc / l[..., None]
    dO = Tacc / l[..., None] - (mu / l)[..., None] * O
    lse = m + torch.log(l)
    return O.transpose(1, 2), dO.transpose(1, 2), lse


def attn_jvp_online_lazy(q, k, v, tq, tk, tv, softmax_scale: Optional[float] = None, block_kv: int = 128,
                         threshold_log2: float = 8.0, emulate_bf16: bool = True, dtype=torch.float64):
    """The same recurrence with the operand roundings of the sm_100a kernel, evaluated in fp64.

    This is the comparison partner for the kernel's fp32-output checking mode: it rounds where the kernel
    rounds and nowhere else, so the difference that remains is the kernel's accumulation error.

    * exponents are taken in base 2 relative to a LAZILY updated maximum: the first block sets it to the
      block's row maximum; afterwards it only moves (to the block's maximum) when that exceeds it by more
      than ``threshold_log2``, and only then are the running sums rescaled.  bf16 rounding is not invariant
      under a change of the reference point unless the change is a power of two, so P has to be formed the
      way the kernel forms it;
    * l sums the unrounded P; P is then rounded to bf16;
    * G = bf16(P) * dS (dS carries the softmax scale), mu sums the unrounded G; G is then rounded to bf16;
    * O += bf16(P) V,  T += bf16(P) dV + bf16(G) V;  o = O / l,  to = T / l - (mu / l) o,
      lse = ln 2 * (m + log2 l).
    """
    d = q.shape[-1]
    s = d ** -0.5 if softmax_scale is None else softmax_scale
    Q, K, V, dQ, dK, dV = (x.to(dtype).transpose(1, 2) for x in (q, k, v, tq, tk, tv))
    B, H, Lq, D = Q.shape
    Lk = K.shape[2]
    m = None
    l = torch.zeros((B, H, Lq), dtype=dtype)
    mu = torch.zeros((B, H, Lq), dtype=dtype)
    Oacc = torch.zeros((B, H, Lq, D), dtype=dtype)
    Tacc = torch.zeros((B, H, Lq, D), dtype=dtype)
    for j in range(0, Lk, block_kv):
        Kj, Vj, dKj, dVj = (x[:, :, j:j + block_kv] for x in (K, V, dK, dV))
        S2 = (s * LOG2E) * (Q @ Kj.transpose(-2, -1))          # scores in log2 units
        m_blk = S2.amax(-1)
        if m is None:
            m = m_blk
        else:
            need = m_blk > m + threshold_log2
            alpha = torch.where(need, torch.exp2(m - m_blk), torch.ones_like(m))
            m = torch.where(need, m_blk, m)
            l, mu = l * alpha, mu * alpha
            Oacc, Tacc = Oacc * alpha[..., None], Tacc * alpha[..., None]
        P = torch.exp2(S2 - m[..., None])
        l = l + P.sum(-1)
        Pr = _round(P, emulate_bf16)
        dS = s * (dQ @ Kj.transpose(-2, -1) + Q @ dKj.transpose(-2, -1))
        G = Pr * dS
        mu = mu + G.sum(-1)
        Gr = _round(G, emulate_bf16)
        Oacc = Oacc + Pr @ Vj
        Tacc = Tacc + Gr @ Vj + Pr @ dVj
    O = Oacc / l[..., None]
    dO = Tacc / l[..., None] - (mu / l)[..., None] * O
    lse = (m + torch.log2(l)) * math.log(2.0)
    return O.transpose(1, 2), dO.transpose(1, 2), lse


def attn_bwd_base(q, k, v, dout):
    """Primal backward through autograd of the 'base' path: (dq, dk, dv)."""
    q, k, v = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
    out = base_attention(q, k, v)
    out.backward(dout)
    return q.grad, k.grad, v.grad


def attn_bwd_closed_form(q, k, v, dout, softmax_scale: Optional[float] = None, dtype=torch.float64):
    """Explicit backward: dV = P^T dO; dP = dO V^T; dS = P*(dP - rowsum(dO*O)); dQ = s dS K; dK = s dS^T Q."""
    d = q.shape[-1]
    s = d ** -0.5 if softmax_scale is None else softmax_scale
    Q, K, V, dO = (x.to(dtype).transpose(1, 2) for x in (q, k, v, dout))
    S = s * (Q @ K.transpose(-2, -1))
    P = torch.softmax(S, dim=-1)
    O = P @ V
    dV = P.transpose(-2, -1) @ dO
    dP = dO @ V.transpose(-2, -1)
    delta = (dO * O).sum(-1, keepdim=True)
    dS = P * (dP - delta)
    dQ = s * (dS @ K)
    dK = s * (dS.transpose(-2, -1) @ Q)
    return dQ.transpose(1, 2), dK.transpose(1, 2), dV.transpose(1, 2)


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm.forward, models/layers.py:39-42 (weight initialised to ones)."""
    norm_x = torch.rsqrt(x.pow(2).mean(-1, keepdim=True, dtype=torch.float32) + eps)
    w = torch.ones(x.shape[-1], dtype=x.dtype) if weight is None else weight.to(x.dtype)
    return x * norm_x.to(dtype=x.dtype) * w


def rms_norm_jvp_closed_form(x, tx, weight, eps: float = 1e-6):
    """fp64 closed form of RMSNorm (models/layers.py:39-42) and of its tangent with respect to x:
    r = rsqrt(mean(x^2) + eps), y = x r w, ty = (tx r - x r^3 mean(x tx)) w.  The weight is rounded
    to x's dtype first, as the reference casts it.  Returns (y, ty) in fp64."""
    w = weight.to(x.dtype).double()
    xd, td = x.double(), tx.double()
    r = torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps)
    y = xd * r * w
    ty = (td * r - xd * r.pow(3) * (xd * td).mean(-1, keepdim=True)) * w
    return y, ty


def rms_norm_bwd_closed_form(dy, x, weight, eps: float = 1e-6):
    """fp64 gradients of y = RMSNorm(x) w with respect to x and w (autograd of the formula above)."""
    w = weight.to(x.dtype).double()
    xd, g = x.double(), dy.double() * w
    r = torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps)
    dx = r * g - xd * r.pow(3) * (xd * g).mean(-1, keepdim=True)
    dw = (dy.double() * xd * r).reshape(-1, x.shape[-1]).sum(0)
    return dx, dw


# ----------------------------------------------------------------------------
# seeded synthetic inputs with the shapes / distributions of the named configs
# ----------------------------------------------------------------------------

CONFIGS = {
    # name: (B, L, H, D, tangent_scale, qk_norm)
    "C1": (8, 256, 12, 64, 1.0, False),
    "C2": (256, 256, 16, 72, 0.1, False),
    "C3": (64, 1024, 16, 72, 0.1, True),
}


def make_inputs(B: int, L: int, H: int, D: int, *, seed: int = 0, tangent_scale: float = 1.0,
                qk_norm: bool = False, n_extra: int = 0, dtype=torch.float32):
    """Draw q, k, v, dq, dk, dv (then ``n_extra`` more tensors, e.g. dO for the
    backward) in that fixed order from one CPU generator, each randn(B, L, H, D).

    With ``qk_norm`` q and k and their tangents go through ``rms_norm`` by
    forward-mode AD, as Attention.forward does (models/layers.py:143-148).
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    draws = [torch.randn(B, L, H, D, generator=g, dtype=torch.float32) for _ in range(6 + n_extra)]
    q, k, v, tq, tk, tv = draws[:6]
    tq, tk, tv = tq * tangent_scale, tk * tangent_scale, tv * tangent_scale
    if qk_norm:
        q, tq = torch.func.jvp(rms_norm, (q,), (tq,))
        k, tk = torch.func.jvp(rms_norm, (k,), (tk,))
    out = [q, k, v, tq, tk, tv] + draws[6:]
    return [x.to(dtype) for x in out]


def make_config_inputs(name: str, *, batch: Optional[int] = None, n_extra: int = 0, dtype=torch.float32):
    B, L, H, D, ts, qkn = CONFIGS[name]
    return make_inputs(batch or B, L, H, D, seed=0, tangent_scale=ts, qk_norm=qkn,
                       n_extra=n_extra, dtype=dtype)


# ----------------------------------------------------------------------------
# error metrics
# ----------------------------------------------------------------------------

def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def max_rel(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / max|b|."""
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-300))


def flops_dual_fwd(B, H, Lq, Lk, D) -> float:
    return 12.0 * B * H * Lq * Lk * D


def flops_fwd(B, H, Lq, Lk, D) -> float:
    return 4.0 * B * H * Lq * Lk * D


def flops_bwd(B, H, Lq, Lk, D) -> float:
    return 10.0 * B * H * Lq * Lk * D
