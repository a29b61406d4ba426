"""Parity of the fused per-head RMS norm (+ tangent, + backward) with the oracle.

The oracle is the closed form in fp64 (pinned in test_oracle.py against torch.func.jvp / autograd through
the reference's own RMSNorm.forward restated in oracle.rms_norm); the reference's 16-bit evaluation of the
same function, which rounds after every elementwise step, is compared as well.
"""

import pytest
import torch

from dmf_b200 import ops
from dmf_b200.rms_norm import rms_norm
from oracle import attn_jvp_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 3e-3        # rel-L2 vs fp64 on the same 16-bit inputs: one rounding of the result (2^-9 / sqrt(3) ~ 1.1e-3)
TOL_REF = 8e-3    # vs the reference's own 16-bit evaluation (three roundings)


def _inputs(B, L, H, D, seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, L, H, D, generator=g).to(dtype)
    tx = (0.1 * torch.randn(B, L, H, D, generator=g)).to(dtype)
    w = 1.0 + 0.2 * torch.randn(D, generator=g)
    dy = torch.randn(B, L, H, D, generator=g).to(dtype)
    return x, tx, w, dy


@pytest.mark.parametrize("D", [8, 24, 40, 64, 72, 88, 96, 104, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_forward_dual_matches_oracle(D, dtype):
    x, tx, w, _ = _inputs(3, 200, 5, D, seed=D, dtype=dtype)   # ragged row count: 3000 rows, not a multiple of 16
    y, ty = ops.rmsnorm_fwd_raw(x.to(DEV), tx.to(DEV), w.to(DEV), 1e-6)
    y_ref, ty_ref = orc.rms_norm_jvp_closed_form(x, tx, w)
    assert orc.rel_l2(y.float().cpu(), y_ref) < TOL
    assert orc.rel_l2(ty.float().cpu(), ty_ref) < TOL
    y_plain, none = ops.rmsnorm_fwd_raw(x.to(DEV), None, w.to(DEV), 1e-6)
    assert none is None and torch.equal(y_plain, y)


def test_strided_views_of_packed_qkv():
    x, tx, w, _ = _inputs(2, 256, 16, 72, seed=1)
    qkv = torch.stack([x, x * 0.5, x * 0.25], dim=2).to(DEV)      # (B, L, 3, H, D)
    tqkv = torch.stack([tx, tx, tx], dim=2).to(DEV)
    y, ty = ops.rmsnorm_fwd_raw(qkv[:, :, 0], tqkv[:, :, 0], w.to(DEV), 1e-6)
    y0, ty0 = ops.rmsnorm_fwd_raw(x.to(DEV), tx.to(DEV), w.to(DEV), 1e-6)
    assert torch.equal(y, y0) and torch.equal(ty, ty0)


def test_backward_matches_oracle_and_is_reproducible():
    x, _, w, dy = _inputs(4, 384, 16, 72, seed=2)
    dx, dw = ops.rmsnorm_bwd_raw(dy.to(DEV), x.to(DEV), w.to(DEV), 1e-6)
    dx_ref, dw_ref = orc.rms_norm_bwd_closed_form(dy, x, w)
    assert orc.rel_l2(dx.float().cpu(), dx_ref) < TOL
    assert orc.rel_l2(dw.cpu().double(), dw_ref) < 1e-5
    dx2, dw2 = ops.rmsnorm_bwd_raw(dy.to(DEV), x.to(DEV), w.to(DEV), 1e-6)
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)  # fixed-order reduction, no atomics


@pytest.mark.parametrize("D", [8, 40, 64, 72, 128])
@pytest.mark.parametrize("shape", [(1, 1, 1), (1, 7, 3), (5, 333, 7), (2, 4096, 16)])
def test_every_row_grouping_and_ragged_row_counts(D, shape):
    """Rows per warp differ with the head dim (32 // (D / 8)); row counts below one warp, below one block
    slice, and above one pass of the grid."""
    B, L, H = shape
    x, tx, w, dy = _inputs(B, L, H, D, seed=B * L + D)
    y, ty = ops.rmsnorm_fwd_raw(x.to(DEV), tx.to(DEV), w.to(DEV), 1e-6)
    y0, none = ops.rmsnorm_fwd_raw(x.to(DEV), None, w.to(DEV), 1e-6)
    assert none is None and torch.equal(y0, y)                     # the plain kernel computes the same primal
    y_ref, ty_ref = orc.rms_norm_jvp_closed_form(x, tx, w)
    assert orc.rel_l2(y.float().cpu(), y_ref) < TOL and orc.rel_l2(ty.float().cpu(), ty_ref) < TOL
    dx, dw = ops.rmsnorm_bwd_raw(dy.to(DEV), x.to(DEV), w.to(DEV), 1e-6)
    dx_ref, dw_ref = orc.rms_norm_bwd_closed_form(dy, x, w)
    assert orc.rel_l2(dx.float().cpu(), dx_ref) < TOL
    assert orc.rel_l2(dw.double().cpu(), dw_ref) < 1e-4


def test_offsets_beyond_31_bits_take_the_64_bit_path():
    """Tensors whose element offsets fit 31 bits are indexed with 32-bit arithmetic; a batch stride of 2^31 + 64
    elements (a view of a 4.3 GB buffer) must give the same rows through the 64-bit kernels."""
    L, H, D = 40, 3, 72
    x, tx, w, dy = _inputs(2, L, H, D, seed=11)
    stride_b = 2 ** 31 + 64
    base = torch.empty(stride_b + L * H * D, dtype=torch.bfloat16, device=DEV)
    big = base.as_strided((2, L, H, D), (stride_b, H * D, D, 1))
    big.copy_(x.to(DEV))
    y_big, ty_big = ops.rmsnorm_fwd_raw(big, tx.to(DEV), w.to(DEV), 1e-6)
    y, ty = ops.rmsnorm_fwd_raw(x.to(DEV), tx.to(DEV), w.to(DEV), 1e-6)
    assert torch.equal(y_big, y) and torch.equal(ty_big, ty)
    dx_big, dw_big = ops.rmsnorm_bwd_raw(dy.to(DEV), big, w.to(DEV), 1e-6)
    dx, dw = ops.rmsnorm_bwd_raw(dy.to(DEV), x.to(DEV), w.to(DEV), 1e-6)
    assert torch.equal(dx_big, dx) and torch.equal(dw_big, dw)


def test_full_size_properties():
    """At the benchmark's size (q and k views of a packed 64 x 1024 x 3 x 16 x 72 projection): the tangent is linear
    in the input tangent (a factor 2 is exact in every rounding), dual and plain kernels give the same primal, rows
    have unit mean square for a unit weight, and dweight matches a column sum."""
    B, L, H, D = 64, 1024, 16, 72
    g = torch.Generator(device=DEV).manual_seed(0)
    qkv = torch.randn(B, L, 3, H, D, device=DEV, generator=g).bfloat16()
    tqkv = (0.1 * torch.randn(B, L, 3, H, D, device=DEV, generator=g)).bfloat16()
    w = torch.ones(D, device=DEV)
    for i in (0, 1):
        x, tx = qkv[:, :, i], tqkv[:, :, i]
        y, ty = ops.rmsnorm_fwd_raw(x, tx, w, 1e-6)
        y2, ty2 = ops.rmsnorm_fwd_raw(x, 2 * tx, w, 1e-6)
        assert torch.equal(y2, y) and torch.equal(ty2, 2 * ty)
        assert torch.equal(ops.rmsnorm_fwd_raw(x, None, w, 1e-6)[0], y)
        assert float((y.float().square().mean(-1) - 1).abs().max()) < 1e-2      # bf16 rounding of 72 values
        assert float((y.float() * ty.float()).mean(-1).abs().max()) < 2e-2        # the tangent is orthogonal to the row
    dy = torch.randn(B, L, H, D, device=DEV, generator=g).bfloat16()
    x = qkv[:, :, 0]
    dx, dw = ops.rmsnorm_bwd_raw(dy, x, w, 1e-6)
    r = torch.rsqrt(x.double().square().mean(-1, keepdim=True) + 1e-6)
    assert orc.rel_l2(dw.double(), (dy.double() * x.double() * r).sum((0, 1, 2))) < 1e-5
    assert float((dx.float() * x.float()).mean(-1).abs().max()) < 5e-2            # dx is orthogonal to x (weight 1)


def test_jvp_and_backward_through_the_wrapper_like_the_reference_module():
    """torch.func.jvp through rms_norm vs through the reference's RMSNorm.forward (restated in the oracle),
    both on the GPU in bf16, and the primal gradient vs autograd through the reference form."""
    x, tx, w, dy = _inputs(2, 256, 16, 72, seed=3)
    xd, txd, dyd = x.to(DEV), tx.to(DEV), dy.to(DEV)
    wd = w.to(DEV).requires_grad_(True)
    y, ty = torch.func.jvp(lambda a: rms_norm(a, wd), (xd,), (txd,))
    y_ref, ty_ref = torch.func.jvp(lambda a: orc.rms_norm(a, wd.detach()), (xd,), (txd,))
    assert orc.rel_l2(y.detach().float().cpu(), y_ref.float().cpu()) < TOL_REF
    assert orc.rel_l2(ty.detach().float().cpu(), ty_ref.float().cpu()) < TOL_REF
    xg = xd.clone().requires_grad_(True)
    out = rms_norm(xg, wd)
    out.backward(dyd)
    dx_ref, dw_ref = orc.rms_norm_bwd_closed_form(dy, x, w)
    assert orc.rel_l2(xg.grad.float().cpu(), dx_ref) < TOL
    assert orc.rel_l2(wd.grad.detach().cpu().double(), dw_ref) < 1e-4


def test_rejects_bad_arguments():
    x, tx, w, _ = _inputs(1, 16, 2, 72)
    with pytest.raises(RuntimeError):
        ops.rmsnorm_fwd_raw(x, tx, w, 1e-6)                       # CPU tensors: no CPU path
    with pytest.raises(Exception):
        ops.rmsnorm_fwd_raw(x[..., :68].to(DEV), None, w[:68].to(DEV), 1e-6)   # head_dim not a multiple of 8
