"""Parity of the CUDA forward kernels (dual and plain) with the CPU oracle, through
the C ABI.  Tolerances: the bar for bf16 is rel-L2(O), rel-L2(dO) <= 2e-2 against
the fp32 'base' oracle; the kernels sit near the bf16 rounding floor (~2.5e-3), so
the asserts use 6e-3 against an oracle fed the same bf16-rounded inputs and 8e-3
against the un-rounded one - a miss means a bug, not noise."""

import numpy as np
import pytest
import torch

from oracle import attn_jvp_oracle as orc
from tests import _cabi
from tests.conftest import GOLDEN
from tests.golden.make_golden import CASES

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

TOL_SAME_INPUTS = 6e-3
TOL_BAR = 2e-2
TOL_LSE = 1e-4   # half of the exponentials use a cubic with 7.5e-5 relative error, which moves ln(l) by up to that much


def _inputs(B, L, H, D, *, seed=0, ts=0.5, dtype=torch.bfloat16, qk_norm=False):
    ins = orc.make_inputs(B, L, H, D, seed=seed, tangent_scale=ts, qk_norm=qk_norm)
    return [x.to(dtype) for x in ins]


def _to_dev(ins, layout):
    """layout: 'contig' | 'packed' (strided views of a (B,L,3,H,D) buffer) | 'qknorm' (q,k contiguous, v strided)."""
    if layout == "contig":
        return [x.to(DEV) for x in ins]
    qkv = torch.stack(ins[:3], dim=2).to(DEV)
    tqkv = torch.stack(ins[3:6], dim=2).to(DEV)
    g = [qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], tqkv[:, :, 0], tqkv[:, :, 1], tqkv[:, :, 2]]
    if layout == "qknorm":
        for i in (0, 1, 3, 4):
            g[i] = g[i].contiguous()
    return g


def _check_dual(ins, g, tol=TOL_SAME_INPUTS):
    o, to, lse, _ = _cabi.fwd(*g)
    o_ref, do_ref, lse_ref = orc.attn_jvp_closed_form(*[x.float() for x in ins])
    assert not torch.isnan(o).any() and not torch.isnan(to).any() and not torch.isnan(lse).any()
    assert orc.rel_l2(o.float().cpu(), o_ref) < tol
    assert orc.rel_l2(to.float().cpu(), do_ref) < tol
    assert float((lse.cpu().double() - lse_ref).abs().max()) < TOL_LSE
    return o, to, lse


@pytest.mark.parametrize("D", [64, 72, 80, 96, 128])
@pytest.mark.parametrize("L", [128, 256, 1024])
def test_dual_matches_oracle(D, L):
    ins = _inputs(2, L, 3, D, seed=D + L)
    _check_dual(ins, _to_dev(ins, "contig"))


@pytest.mark.parametrize("layout", ["packed", "qknorm"])
@pytest.mark.parametrize("D", [64, 72])
def test_dual_strided_layouts(layout, D):
    ins = _inputs(3, 256, 4, D, seed=7, ts=0.1, qk_norm=(layout == "qknorm"))
    _check_dual(ins, _to_dev(ins, layout))


@pytest.mark.parametrize("D", [64, 72, 96, 128])
def test_strided_outputs(D):
    """o and to as strided halves of one buffer (the stores go through TMA maps built from the strides);
    the dual pass and the plain forward must agree with the contiguous call bit for bit."""
    ins = _inputs(2, 256, 3, D, seed=11, ts=0.2)
    g = _to_dev(ins, "contig")
    o0, to0, lse0, _ = _cabi.fwd(*g)
    o1, to1, lse1, _ = _cabi.fwd(*g, packed_out=True)
    assert not o1.is_contiguous()
    assert torch.equal(o0, o1) and torch.equal(to0, to1) and torch.equal(lse0, lse1)
    p0, _, pl0, _ = _cabi.fwd(*g[:3])
    p1, _, pl1, _ = _cabi.fwd(*g[:3], packed_out=True)
    assert torch.equal(p0, p1) and torch.equal(pl0, pl1)
    assert not torch.isnan(p1).any()


def test_dual_fp16():
    ins = _inputs(2, 256, 2, 72, seed=3, dtype=torch.float16)
    _check_dual(ins, _to_dev(ins, "contig"), tol=1e-3)


def test_dual_cross_attention_lengths():
    """seqlen_q != seqlen_kv (the reference kernel takes both, flash_attention_2_jvp.py:189-190)."""
    q, _, _, tq, _, _ = _inputs(2, 128, 2, 72, seed=11)
    _, k, v, _, tk, tv = _inputs(2, 384, 2, 72, seed=12)
    ins = [q, k, v, tq, tk, tv]
    _check_dual(ins, [x.to(DEV) for x in ins])


def test_dual_custom_scale_and_large_logits():
    """A sharp softmax (large scale) drives the running max up block after block: the
    lazy rescale of the accumulators must keep O, dO and LSE right."""
    ins = _inputs(1, 1024, 2, 64, seed=5)
    # keys sorted so that later blocks hold larger logits for every row
    ins[1] = ins[1] * torch.linspace(0.2, 3.0, 1024).view(1, 1024, 1, 1).to(ins[1].dtype)
    g = [x.to(DEV) for x in ins]
    o, to, lse, _ = _cabi.fwd(*g, scale=0.7)
    o_ref, do_ref, lse_ref = orc.attn_jvp_closed_form(*[x.float() for x in ins], softmax_scale=0.7)
    assert orc.rel_l2(o.float().cpu(), o_ref) < TOL_SAME_INPUTS
    assert orc.rel_l2(to.float().cpu(), do_ref) < 1e-2
    assert float((lse.cpu().double() - lse_ref).abs().max()) < 1e-4


@pytest.mark.parametrize("D", [64, 72, 96, 128])
def test_plain_forward_matches_oracle_and_dual(D):
    ins = _inputs(2, 512, 3, D, seed=D)
    g = _to_dev(ins, "packed")
    o, _, lse, _ = _cabi.fwd(*g[:3])
    o_ref, lse_ref = orc.attn_fwd_closed_form(*[x.float() for x in ins[:3]])
    assert orc.rel_l2(o.float().cpu(), o_ref) < TOL_SAME_INPUTS
    assert float((lse.cpu().double() - lse_ref).abs().max()) < TOL_LSE
    # the primal half of the dual pass computes the same numbers
    o2, _, lse2, _ = _cabi.fwd(*g)
    assert orc.rel_l2(o2.float(), o.float()) < 2e-3
    assert float((lse2 - lse).abs().max()) < TOL_LSE


def test_many_tiles_per_cta():
    """More tiles than SMs: every CTA walks several tiles through the same barriers."""
    ins = _inputs(40, 256, 12, 64, seed=9)
    g = _to_dev(ins, "contig")
    _check_dual(ins, g)
    o, _, lse, _ = _cabi.fwd(*g[:3])
    o_ref, lse_ref = orc.attn_fwd_closed_form(*[x.float() for x in ins[:3]])
    assert orc.rel_l2(o.float().cpu(), o_ref) < TOL_SAME_INPUTS
    assert float((lse.cpu().double() - lse_ref).abs().max()) < TOL_LSE


@pytest.mark.parametrize("name", list(CASES))
def test_against_reference_golden_vectors(name):
    """Kernel vs the outputs of the reference's own code (tests/golden)."""
    B, L, H, D, ts, qkn, seed = CASES[name]
    g = np.load(GOLDEN / f"{name}.npz")
    ins32 = orc.make_inputs(B, L, H, D, seed=seed, tangent_scale=ts, qk_norm=qkn)
    ins = [x.bfloat16().to(DEV) for x in ins32]
    o, to, lse, _ = _cabi.fwd(*ins)
    assert orc.rel_l2(o.float().cpu(), torch.from_numpy(g["base_o"])) < 8e-3 < TOL_BAR
    assert orc.rel_l2(to.float().cpu(), torch.from_numpy(g["base_do"])) < 8e-3 < TOL_BAR
    assert float((lse.cpu() - torch.from_numpy(g["tri_lse"])).abs().max()) < 2e-2   # bf16 input rounding moves S


def test_config_c1_shape():
    """B=8, H=12, N=256, D=64, tangents N(0,1): the CPU-runnable reference case."""
    ins32 = orc.make_config_inputs("C1")
    o_ref, do_ref = orc.attn_jvp_base(*ins32)
    g = [x.bfloat16().to(DEV) for x in ins32]
    o, to, lse, _ = _cabi.fwd(*g)
    assert o.transpose(1, 2).shape == (8, 12, 256, 64)
    assert orc.rel_l2(o.float().cpu(), o_ref) < 8e-3 < TOL_BAR
    assert orc.rel_l2(to.float().cpu(), do_ref) < 8e-3 < TOL_BAR


@pytest.mark.parametrize("cfg", ["C2", "C3"])
def test_full_size_properties(cfg):
    """At the full benchmark sizes the oracle is too slow for every element, so check:
    a batch slice against the oracle, bitwise determinism, convexity of O, zero
    tangents -> zero dO, and linearity of dO in the tangents."""
    B, L, H, D, ts, qkn = orc.CONFIGS[cfg]
    gen = torch.Generator(device=DEV).manual_seed(0)
    qkv = torch.randn(B, L, 3, H, D, device=DEV, dtype=torch.bfloat16, generator=gen)
    tqkv = torch.randn(B, L, 3, H, D, device=DEV, dtype=torch.bfloat16, generator=gen) * ts
    if qkn:
        nrm = lambda x: (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(x.dtype)
        q, k = nrm(qkv[:, :, 0]), nrm(qkv[:, :, 1])
    else:
        q, k = qkv[:, :, 0], qkv[:, :, 1]
    v, tq, tk, tv = qkv[:, :, 2], tqkv[:, :, 0], tqkv[:, :, 1], tqkv[:, :, 2]
    o, to, lse, _ = _cabi.fwd(q, k, v, tq, tk, tv)
    assert not torch.isnan(o).any() and not torch.isnan(to).any() and not torch.isnan(lse).any()
    # (1) slices against the oracle
    for b in (0, B - 1):
        sl = [x[b:b + 1].float().cpu() for x in (q, k, v, tq, tk, tv)]
        o_ref, do_ref, lse_ref = orc.attn_jvp_closed_form(*sl)
        assert orc.rel_l2(o[b:b + 1].float().cpu(), o_ref) < TOL_SAME_INPUTS
        assert orc.rel_l2(to[b:b + 1].float().cpu(), do_ref) < TOL_SAME_INPUTS
        assert float((lse[b:b + 1].cpu().double() - lse_ref).abs().max()) < TOL_LSE
    # (2) determinism
    o2, to2, lse2, _ = _cabi.fwd(q, k, v, tq, tk, tv)
    assert torch.equal(o, o2) and torch.equal(to, to2) and torch.equal(lse, lse2)
    # (3) O is a convex combination of the rows of V
    vmax = v.float().amax(dim=1, keepdim=True)
    vmin = v.float().amin(dim=1, keepdim=True)
    assert bool((o.float() <= vmax + 2e-2).all()) and bool((o.float() >= vmin - 2e-2).all())
    # (4) zero tangents give a zero output tangent and the same primal
    z = torch.zeros_like(q)
    o3, to3, _, _ = _cabi.fwd(q, k, v, z, torch.zeros_like(k), torch.zeros_like(v))
    assert torch.equal(o3, o) and float(to3.float().abs().max()) == 0.0
    # (5) dO is linear in the tangents (powers of two scale bf16 exactly)
    _, to4, _, _ = _cabi.fwd(q, k, v, tq * 2, tk * 2, tv * 2)
    assert orc.rel_l2(to4.float(), 2 * to.float()) < 3e-3


def test_arguments_rejected_before_launch():
    q = torch.randn(1, 100, 1, 64, device=DEV, dtype=torch.bfloat16)
    _cabi.fwd(q, q, q, expect=4)                                  # seqlen not a multiple of 128
    q = torch.randn(1, 128, 1, 48, device=DEV, dtype=torch.bfloat16)
    _cabi.fwd(q, q, q, expect=3)                                  # head dim
    from dmf_b200 import ops
    q = torch.randn(1, 128, 1, 64, device=DEV, dtype=torch.float32)
    with pytest.raises(TypeError):
        ops.fwd_raw(q, q, q, 0.125)
