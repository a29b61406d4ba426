"""The CPU oracle against the golden vectors produced by the reference's own code
(tests/golden/make_golden.py).  Everything here runs without a GPU."""

import numpy as np
import pytest
import torch

from oracle import attn_jvp_oracle as orc
from tests.conftest import GOLDEN
from tests.golden.make_golden import CASES


def _load(name):
    B, L, H, D, ts, qkn, seed = CASES[name]
    g = np.load(GOLDEN / f"{name}.npz")
    ins = orc.make_inputs(B, L, H, D, seed=seed, tangent_scale=ts, qk_norm=qkn, n_extra=1)
    # the generator must reproduce the inputs the golden outputs were made from
    chk = np.array([float(x.double().sum()) for x in ins])
    np.testing.assert_allclose(chk, g["checksum"], rtol=0, atol=1e-3)
    return g, ins


@pytest.mark.parametrize("name", list(CASES))
def test_base_jvp_matches_reference(name):
    g, (q, k, v, tq, tk, tv, dout) = _load(name)
    o, do = orc.attn_jvp_base(q, k, v, tq, tk, tv)
    # same code path, same machine arithmetic: fp32 round-off only
    np.testing.assert_allclose(o.numpy(), g["base_o"], rtol=0, atol=2e-6)
    np.testing.assert_allclose(do.numpy(), g["base_do"], rtol=0, atol=2e-6)
    assert g["raw_vs_base_maxabs"].max() < 5e-6


@pytest.mark.parametrize("name", list(CASES))
def test_closed_form_matches_reference(name):
    g, (q, k, v, tq, tk, tv, dout) = _load(name)
    o, do, lse = orc.attn_jvp_closed_form(q, k, v, tq, tk, tv)
    assert orc.rel_l2(o, torch.from_numpy(g["base_o"])) < 2e-6
    assert orc.rel_l2(do, torch.from_numpy(g["base_do"])) < 2e-6
    # the reference Triton kernels (CPU interpreter, fp32) as a third witness, incl. LSE
    assert orc.rel_l2(o, torch.from_numpy(g["tri_o"])) < 2e-6
    assert orc.rel_l2(do, torch.from_numpy(g["tri_do"])) < 2e-6
    np.testing.assert_allclose(lse.float().numpy(), g["tri_lse"], rtol=0, atol=5e-6)


@pytest.mark.parametrize("name", list(CASES))
def test_online_recurrence_matches_reference_kernel(name):
    g, (q, k, v, tq, tk, tv, dout) = _load(name)
    o, do, lse = orc.attn_jvp_online(q, k, v, tq, tk, tv, block_kv=128)
    assert orc.rel_l2(o, torch.from_numpy(g["tri_o"])) < 2e-6
    assert orc.rel_l2(do, torch.from_numpy(g["tri_do"])) < 2e-6
    np.testing.assert_allclose(lse.float().numpy(), g["tri_lse"], rtol=0, atol=5e-6)
    # block size must not matter
    o2, do2, lse2 = orc.attn_jvp_online(q, k, v, tq, tk, tv, block_kv=64)
    assert orc.rel_l2(o2, o) < 1e-12 and orc.rel_l2(do2, do) < 1e-12


@pytest.mark.parametrize("name", list(CASES))
def test_backward_matches_reference(name):
    g, (q, k, v, tq, tk, tv, dout) = _load(name)
    dq, dk, dv = orc.attn_bwd_base(q, k, v, dout)
    for got, key in ((dq, "raw_dq"), (dk, "raw_dk"), (dv, "raw_dv")):
        assert orc.rel_l2(got, torch.from_numpy(g[key])) < 2e-6
    dq2, dk2, dv2 = orc.attn_bwd_closed_form(q, k, v, dout)
    for got, key in ((dq2, "raw_dq"), (dk2, "raw_dk"), (dv2, "raw_dv")):
        assert orc.rel_l2(got, torch.from_numpy(g[key])) < 2e-6


def test_rms_norm_matches_reference():
    name = "d72_l256_qknorm"
    g, (q, k, v, tq, tk, tv, dout) = _load(name)
    np.testing.assert_allclose(q.numpy(), g["normed_q"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(tq.numpy(), g["normed_tq"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(k.numpy(), g["normed_k"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(tk.numpy(), g["normed_tk"], rtol=0, atol=1e-6)


def test_bf16_emulation_floor():
    """The rounding points of the bf16 kernel leave a wide margin under the 2e-2 bar."""
    q, k, v, tq, tk, tv = orc.make_inputs(1, 256, 2, 72, seed=5, tangent_scale=0.1)
    qb, kb, vb, tqb, tkb, tvb = (x.bfloat16().float() for x in (q, k, v, tq, tk, tv))
    o_ref, do_ref, _ = orc.attn_jvp_closed_form(q, k, v, tq, tk, tv)
    o, do, _ = orc.attn_jvp_online(qb, kb, vb, tqb, tkb, tvb, emulate_bf16=True, dtype=torch.float32)
    assert orc.rel_l2(o.bfloat16(), o_ref) < 1e-2
    assert orc.rel_l2(do.bfloat16(), do_ref) < 1e-2


def test_config_shapes_and_flops():
    assert orc.CONFIGS["C2"][:4] == (256, 256, 16, 72)
    assert orc.CONFIGS["C3"][:4] == (64, 1024, 16, 72)
    assert abs(orc.flops_dual_fwd(256, 16, 256, 256, 72) - 231.9e9) < 0.1e9
    assert abs(orc.flops_dual_fwd(64, 16, 1024, 1024, 72) - 927.7e9) < 0.1e9
    assert abs(orc.flops_dual_fwd(8, 12, 256, 256, 64) - 4.83e9) < 0.01e9


def test_rms_norm_closed_forms_match_autodiff_of_the_reference_form():
    """rms_norm restates RMSNorm.forward (models/layers.py:39-42; pinned against the reference's own output by
    the qk-norm golden case above); the fp64 closed forms of its tangent and gradients must agree with
    torch.func.jvp / autograd through it."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 8, 3, 72, generator=g, dtype=torch.float64)
    tx = torch.randn(2, 8, 3, 72, generator=g, dtype=torch.float64)
    w = (1 + 0.2 * torch.randn(72, generator=g)).double()
    dy = torch.randn(2, 8, 3, 72, generator=g, dtype=torch.float64)
    y, ty = torch.func.jvp(lambda a: orc.rms_norm(a, w), (x,), (tx,))
    y2, ty2 = orc.rms_norm_jvp_closed_form(x, tx, w)
    assert float((y - y2).abs().max()) < 1e-5 and float((ty - ty2).abs().max()) < 1e-5   # the reference form means in fp32
    xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    orc.rms_norm(xg, wg).backward(dy)
    dx, dw = orc.rms_norm_bwd_closed_form(dy, x, w)
    assert float((xg.grad - dx).abs().max()) < 1e-5 and float((wg.grad - dw).abs().max()) < 1e-5


def test_adaln_closed_forms_match_autodiff_of_the_reference_forms():
    """oracle/adaln_oracle.py restates modulate(norm(x)) and x + gate * h (models/layers.py:28-29, 195-201); the fp64
    closed forms the kernels implement must agree with torch.func.jvp / autograd through the restated forms."""
    from oracle import adaln_oracle as ada
    g = torch.Generator().manual_seed(11)
    B, L, Cn = 2, 5, 384
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    x, tx, h, th, dy = rn(B, L, Cn) * 2 + 0.3, rn(B, L, Cn), rn(B, L, Cn), rn(B, L, Cn), rn(B, L, Cn)
    sh, sc, gt, tsh, tsc, tgt = (0.3 * rn(B, 1, Cn) for _ in range(6))
    y, ty = torch.func.jvp(ada.ln_modulate, (x, sh, sc), (tx, tsh, tsc))
    y2, ty2 = ada.ln_modulate_jvp_closed_form(x, tx, sh, sc, tsh, tsc)
    assert float((y - y2).abs().max()) < 1e-10 and float((ty - ty2).abs().max()) < 1e-10
    xs = [t.clone().requires_grad_(True) for t in (x, sh, sc)]
    ada.ln_modulate(*xs).backward(dy)
    for got, want in zip([t.grad for t in xs], [ada.ln_modulate_bwd_closed_form(dy, x, sc)[i] for i in (0, 1, 2)]):
        assert float((got - want).abs().max()) < 1e-10
    o, to = torch.func.jvp(ada.gate_residual, (x, gt, h), (tx, tgt, th))
    o2, to2 = ada.gate_residual_jvp_closed_form(x, tx, h, th, gt, tgt)
    assert float((o - o2).abs().max()) < 1e-12 and float((to - to2).abs().max()) < 1e-12
    xs = [t.clone().requires_grad_(True) for t in (x, gt, h)]
    ada.gate_residual(*xs).backward(dy)
    dx, dh, dg = ada.gate_residual_bwd_closed_form(dy, h, gt)
    for got, want in zip([t.grad for t in xs], [dx, dg, dh]):
        assert float((got - want).abs().max()) < 1e-10


def test_lazy_rescale_variant_is_the_same_function_and_shows_why_it_exists():
    """Without rounding, moving the reference point of the exponent lazily changes nothing; with bf16 rounding of P
    it does, at the size of one bf16 rounding, which is why the fp32-output check of the kernel needs this variant."""
    q, k, v, tq, tk, tv = orc.make_inputs(1, 512, 2, 72, seed=9, tangent_scale=0.1)
    # large logits in a few rows, so that the lazy maximum really moves between blocks
    q[:, :7] *= 6.0
    o_ref, do_ref, lse_ref = orc.attn_jvp_closed_form(q, k, v, tq, tk, tv)
    o, do, lse = orc.attn_jvp_online_lazy(q, k, v, tq, tk, tv, emulate_bf16=False)
    assert orc.max_rel(o, o_ref) < 1e-12 and orc.max_rel(do, do_ref) < 1e-11 and orc.max_rel(lse, lse_ref) < 1e-12
    o0, do0, _ = orc.attn_jvp_online_lazy(q, k, v, tq, tk, tv, threshold_log2=0.0, emulate_bf16=False)
    assert orc.max_rel(o0, o_ref) < 1e-12 and orc.max_rel(do0, do_ref) < 1e-11
    # rounded: both schedules stay within the bf16 floor of the exact result, but differ from each other
    ob, dob, _ = orc.attn_jvp_online_lazy(q, k, v, tq, tk, tv, emulate_bf16=True)
    oe, doe, _ = orc.attn_jvp_online(q, k, v, tq, tk, tv, emulate_bf16=True)
    assert orc.rel_l2(ob, o_ref) < 6e-3 and orc.rel_l2(dob, do_ref) < 6e-3
    assert 1e-5 < orc.max_rel(ob, oe) < 1e-2


def test_step_tail_oracle_matches_the_library_calls_of_the_reference_step():
    """clip_grad_norm_ + torch.optim.AdamW + the EMA formula, three steps on CPU, against the fp64 restatement."""
    from oracle import step_oracle as so
    g = torch.Generator().manual_seed(3)
    p = torch.nn.Parameter(torch.randn(1000, generator=g))
    ema = p.detach().clone()
    opt = torch.optim.AdamW([p], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.05, eps=1e-8)
    po, m, v, eo = p.detach().double().clone(), torch.zeros(1000).double(), torch.zeros(1000).double(), ema.double().clone()
    for t in range(1, 4):
        grad = torch.randn(1000, generator=g) * (3.0 if t == 2 else 0.01)     # one step clips, the others do not
        p.grad = grad.clone()
        torch.nn.utils.clip_grad_norm_([p], 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        ema.mul_(0.999).add_(p.detach(), alpha=1 - 0.999)
        po, m, v, eo = so.step_tail(grad, po, m, v, eo, step=t, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.05,
                                    max_grad_norm=1.0, ema_decay=0.999)
        assert orc.max_rel(p.detach(), po) < 1e-6 and orc.max_rel(ema, eo) < 1e-6
        st = opt.state[p]
        assert orc.max_rel(st["exp_avg"], m) < 1e-6 and orc.max_rel(st["exp_avg_sq"], v) < 1e-6
