"""dmf_step_tail (clip + AdamW + EMA + zero-grad in one pass) against the library calls the reference step makes
(train_dmf.py:331-338: clip_grad_norm_, fused torch.optim.AdamW, zero_grad, update_ema) and against the fp64 oracle."""

import copy
from functools import partial

import pytest
import torch

from dmf_b200 import ops
from dmf_b200.step import FlatAdamW
from oracle import attn_jvp_oracle as orc
from oracle import step_oracle as so

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = 2e-6   # max|a - b| / max|b|: fp32 arithmetic in a different order of operations


@pytest.mark.parametrize("n,wd,with_ema", [(1_000_003, 0.0, True), (4096, 0.05, True), (777, 0.0, False)])
def test_step_tail_matches_torch_and_the_oracle(n, wd, with_ema):
    g = torch.Generator(device=DEV).manual_seed(n)
    p0 = torch.randn(n, device=DEV, generator=g)
    ref_p = torch.nn.Parameter(p0.clone())
    ref_ema = p0.clone()
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=wd, fused=True)
    flat_p, flat_ema = p0.clone(), (p0.clone() if with_ema else None)
    flat_opt = FlatAdamW(flat_p, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=wd)
    po, mo, vo, eo = p0.double().cpu(), torch.zeros(n).double(), torch.zeros(n).double(), p0.double().cpu()
    for t in range(1, 4):
        scale = 3.0 / n ** 0.5 if t == 2 else 0.1 / n ** 0.5          # norm 3 (clipped) or 0.1 (not clipped)
        grad = torch.randn(n, device=DEV, generator=g) * scale
        ref_p.grad = grad.clone()
        torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        ref_ema.mul_(0.999).add_(ref_p.detach(), alpha=1 - 0.999)
        flat_g = grad.clone()
        flat_opt.step_tail(flat_g, flat_p, flat_ema, flat_g.norm(2), max_grad_norm=1.0, ema_decay=0.999)
        po, mo, vo, eo = so.step_tail(grad.cpu(), po, mo, vo, eo, step=t, lr=1e-3, betas=(0.9, 0.95), eps=1e-8,
                                      weight_decay=wd, max_grad_norm=1.0, ema_decay=0.999)
        assert float(flat_g.abs().max()) == 0.0                        # gradients are zeroed
        st = opt.state[ref_p]
        assert orc.max_rel(flat_p, ref_p.detach()) < TOL and orc.max_rel(flat_p.cpu(), po) < TOL
        assert orc.max_rel(flat_opt.exp_avg, st["exp_avg"]) < TOL and orc.max_rel(flat_opt.exp_avg.cpu(), mo) < TOL
        assert orc.max_rel(flat_opt.exp_avg_sq, st["exp_avg_sq"]) < TOL and orc.max_rel(flat_opt.exp_avg_sq.cpu(), vo) < TOL
        if with_ema:
            assert orc.max_rel(flat_ema, ref_ema) < TOL and orc.max_rel(flat_ema.cpu(), eo) < TOL
    # the update itself (param - start), where a wrong step size or moment would show at full size
    assert orc.max_rel(flat_p - p0, ref_p.detach() - p0) < 1e-4


def test_graphed_train_step_with_fused_tail_matches_the_library_tail():
    from dmf_b200.harness import train as T
    states = []
    for fused in (True, False):
        st = T.build_train_state(DEV, name="DMFT-S/2", input_size=32, dmf_depth=8, attn_func="fa3", seed=0,
                                 zero_init=False, graphs=True, fused_tail=fused)
        gen = torch.Generator(device=DEV).manual_seed(5)
        eps = torch.randn(4, 4, 32, 32, device=DEV, generator=gen)
        t = torch.rand(4, 1, 1, 1, device=DEV, generator=gen) * 0.5 + 0.5
        r = torch.rand(4, 1, 1, 1, device=DEV, generator=gen) * 0.5

        def fixed_loss(model, raw, x, y, eps=eps, t=t, r=r):
            x_t, v = (1 - t) * x + t * eps, eps - x
            (u, lv), (du, _) = torch.func.jvp(partial(raw, y=y, return_logvar=True), (x_t, t, r),
                                              (v, torch.ones_like(t), torch.zeros_like(r)))
            return ((u - (v + (r - t) * du).detach()) ** 2).mean(dim=(1, 2, 3)) + lv.flatten(), {}

        st.loss_fn = fixed_loss
        w0 = torch.cat([p.detach().flatten().clone() for p in st.model.parameters() if p.requires_grad])
        bgen = torch.Generator(device=DEV).manual_seed(9)
        for _ in range(3):
            T.train_step(st, [T.synthetic_batch(st, 4, generator=bgen)])
        w = torch.cat([p.detach().flatten() for p in st.model.parameters() if p.requires_grad])
        e = torch.cat([q.detach().flatten() for q, p in zip(st.ema.parameters(), st.model.parameters()) if p.requires_grad])
        states.append((w - w0, e, st))
    (dw_f, e_f, st_f), (dw_l, e_l, _) = states
    assert st_f.flat_opt is not None and st_f.flat_opt.step_count == 3
    p = next(q for q in st_f.model.parameters() if q.requires_grad)
    assert p.data_ptr() == st_f.flat_param.data_ptr() and float(st_f.flat_grad.abs().max()) == 0.0
    assert float(dw_l.abs().max()) > 0
    assert orc.rel_l2(dw_f, dw_l) < 1e-3          # three Adam updates from bit-identical gradients
    assert orc.max_rel(e_f, e_l) < 1e-6
    ops.check_device_status(DEV)
