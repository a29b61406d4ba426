"""Parity of the fused adaLN-Zero ops (LayerNorm + modulate, gate + residual; tangents and backwards) with the oracle.

The oracle is the fp64 closed form (pinned in test_oracle.py against torch.func.jvp / autograd through the reference's
formulas restated in oracle/adaln_oracle.py); the wrapper tests also compare with the reference formulas evaluated on
the GPU under torch.func.jvp and autograd, in the dtypes the training step (fp32 stream under bf16 autocast) and the
bf16 sampler use.
"""

import pytest
import torch

from dmf_b200 import adaln
from oracle import adaln_oracle as ada
from oracle import attn_jvp_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16 = torch.float32, torch.bfloat16
# rel-L2 against fp64 on the same inputs: one rounding of the result to its dtype
TOL = {F32: 2e-6, BF16: 3e-3}


def _inputs(B, L, Cn, wide, narrow, mod, seed=0):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    d = dict(
        x=(2.0 * rn(B, L, Cn) + 0.5).to(wide), tx=(0.3 * rn(B, L, Cn)).to(wide),
        h=rn(B, L, Cn).to(narrow), th=(0.3 * rn(B, L, Cn)).to(narrow),
        dy=rn(B, L, Cn).to(narrow), dout=rn(B, L, Cn).to(wide),
    )
    mods = (0.5 * rn(B, 1, 6 * Cn)).to(mod)          # the adaLN projection: chunks are strided views
    tmods = (0.1 * rn(B, 1, 6 * Cn)).to(mod)
    d["shift"], d["scale"], d["gate"] = mods.chunk(6, dim=-1)[:3]
    d["tshift"], d["tscale"], d["tgate"] = tmods.chunk(6, dim=-1)[:3]
    d["_mods"], d["_tmods"] = mods, tmods
    return d


def _dev(d):
    mods, tmods = d["_mods"].to(DEV), d["_tmods"].to(DEV)
    out = {k: v.to(DEV) for k, v in d.items() if not k.startswith("_")}
    out["shift"], out["scale"], out["gate"] = mods.chunk(6, dim=-1)[:3]      # keep them views of one buffer
    out["tshift"], out["tscale"], out["tgate"] = tmods.chunk(6, dim=-1)[:3]
    return out


COMBOS = [(F32, F32, F32), (F32, BF16, BF16), (BF16, BF16, BF16), (F32, BF16, F32)]


@pytest.mark.parametrize("Cn", adaln.WIDTHS)
@pytest.mark.parametrize("wide,narrow,mod", COMBOS)
def test_ln_modulate_forward_and_backward_match_oracle(Cn, wide, narrow, mod):
    B, L = 3, 77                                       # ragged: 231 rows, the last backward block holds 13 rows
    c = _inputs(B, L, Cn, wide, narrow, mod, seed=Cn)
    g = _dev(c)
    y, ty = adaln.ln_modulate_fwd_raw(g["x"], g["tx"], g["shift"], g["scale"], g["tshift"], g["tscale"], 1e-6, narrow)
    y_ref, ty_ref = ada.ln_modulate_jvp_closed_form(c["x"], c["tx"], c["shift"], c["scale"], c["tshift"], c["tscale"])
    assert y.dtype == narrow and orc.rel_l2(y.double().cpu(), y_ref) < TOL[narrow]
    assert orc.rel_l2(ty.double().cpu(), ty_ref) < TOL[narrow]
    y0, none = adaln.ln_modulate_fwd_raw(g["x"], None, g["shift"], g["scale"], None, None, 1e-6, narrow)
    assert none is None and torch.equal(y0, y)         # the plain kernel computes the same primal
    # zero modulation tangents: the kernel's short path
    _, ty1 = adaln.ln_modulate_fwd_raw(g["x"], g["tx"], g["shift"], g["scale"], None, None, 1e-6, narrow)
    zero = torch.zeros_like(c["tshift"])
    _, ty1_ref = ada.ln_modulate_jvp_closed_form(c["x"], c["tx"], c["shift"], c["scale"], zero, zero)
    assert orc.rel_l2(ty1.double().cpu(), ty1_ref) < TOL[narrow]
    dx, dshift, dscale = adaln.ln_modulate_bwd_raw(g["dy"], g["x"], g["scale"], 1e-6)
    dx_ref, dshift_ref, dscale_ref = ada.ln_modulate_bwd_closed_form(c["dy"], c["x"], c["scale"])
    assert dx.dtype == wide and orc.rel_l2(dx.double().cpu(), dx_ref) < TOL[wide]
    assert orc.rel_l2(dshift.double().cpu(), dshift_ref[:, 0]) < 2e-6
    assert orc.rel_l2(dscale.double().cpu(), dscale_ref[:, 0]) < 2e-6
    again = adaln.ln_modulate_bwd_raw(g["dy"], g["x"], g["scale"], 1e-6)
    assert all(torch.equal(a, b) for a, b in zip((dx, dshift, dscale), again))   # fixed-order reductions


@pytest.mark.parametrize("Cn", adaln.WIDTHS)
@pytest.mark.parametrize("wide,narrow,mod", COMBOS)
def test_gate_residual_forward_and_backward_match_oracle(Cn, wide, narrow, mod):
    B, L = 2, 130
    c = _inputs(B, L, Cn, wide, narrow, mod, seed=Cn + 1)
    g = _dev(c)
    out, tout = adaln.gate_residual_fwd_raw(g["x"], g["tx"], g["h"], g["th"], g["gate"], g["tgate"])
    out_ref, tout_ref = ada.gate_residual_jvp_closed_form(c["x"], c["tx"], c["h"], c["th"], c["gate"], c["tgate"])
    assert out.dtype == wide and orc.rel_l2(out.double().cpu(), out_ref) < TOL[wide]
    assert orc.rel_l2(tout.double().cpu(), tout_ref) < TOL[wide]
    out0, none = adaln.gate_residual_fwd_raw(g["x"], None, g["h"], None, g["gate"], None)
    assert none is None and torch.equal(out0, out)
    _, tout1 = adaln.gate_residual_fwd_raw(g["x"], g["tx"], g["h"], g["th"], g["gate"], None)
    _, tout1_ref = ada.gate_residual_jvp_closed_form(c["x"], c["tx"], c["h"], c["th"], c["gate"], torch.zeros_like(c["tgate"]))
    assert orc.rel_l2(tout1.double().cpu(), tout1_ref) < TOL[wide]
    dh, dgate = adaln.gate_residual_bwd_raw(g["dout"], g["h"], g["gate"])
    _, dh_ref, dgate_ref = ada.gate_residual_bwd_closed_form(c["dout"], c["h"], c["gate"])
    assert dh.dtype == narrow and orc.rel_l2(dh.double().cpu(), dh_ref) < TOL[narrow]
    assert orc.rel_l2(dgate.double().cpu(), dgate_ref[:, 0]) < 2e-6
    assert torch.equal(adaln.gate_residual_bwd_raw(g["dout"], g["h"], g["gate"])[1], dgate)


def test_gate_residual_forward_takes_any_width_that_is_a_multiple_of_four():
    c = _inputs(2, 9, 100, F32, BF16, BF16, seed=3)
    g = _dev(c)
    out, tout = adaln.gate_residual_fwd_raw(g["x"], g["tx"], g["h"], g["th"], g["gate"].contiguous(), g["tgate"].contiguous())
    out_ref, tout_ref = ada.gate_residual_jvp_closed_form(c["x"], c["tx"], c["h"], c["th"], c["gate"], c["tgate"])
    assert orc.rel_l2(out.double().cpu(), out_ref) < TOL[F32] and orc.rel_l2(tout.double().cpu(), tout_ref) < TOL[F32]


@pytest.mark.parametrize("autocast", [True, False])
def test_block_through_the_wrappers_like_the_reference_block(autocast):
    """x -> x + gate * W(modulate(norm(x))) under torch.func.jvp and autograd: the fused ops against the reference
    formulas on the GPU, with an fp32 stream under bf16 autocast (training) and all-bf16 (sampling)."""
    B, L, Cn = 2, 64, 384
    wide = F32 if autocast else BF16
    c = _inputs(B, L, Cn, wide, BF16, BF16, seed=9)
    g = _dev(c)
    lin = torch.nn.Linear(Cn, Cn).to(DEV).to(F32 if autocast else BF16)

    def fused(x, shift, scale, gate):
        return adaln.gate_residual(x, gate, lin(adaln.ln_modulate(x, shift, scale)))

    lin32 = torch.nn.Linear(Cn, Cn).to(DEV)
    lin32.load_state_dict({k: v.float() for k, v in lin.state_dict().items()})

    def plain(x, shift, scale, gate):
        # under autocast: the reference's own dtypes; for the all-bf16 model: the same formulas in fp32
        return ada.gate_residual(x, gate, (lin if autocast else lin32)(ada.ln_modulate(x, shift, scale)))

    prim = (g["x"], g["shift"], g["scale"], g["gate"])
    tang = (g["tx"], g["tshift"], g["tscale"], g["tgate"])
    res = {}
    for name, fn in (("fused", fused), ("plain", plain)):
        up = (lambda t: t.float()) if (name == "plain" and not autocast) else (lambda t: t)
        leaves = [up(t.detach().clone()).requires_grad_(True) for t in prim]
        with torch.autocast("cuda", dtype=BF16, enabled=autocast):
            out, tout = torch.func.jvp(fn, tuple(leaves), tuple(up(t) for t in tang))
            (out.float().square().mean() + tout.detach().float().mean()).backward()
        res[name] = [out.detach(), tout.detach()] + [t.grad for t in leaves]
    tol = 2e-2                                          # the reference form rounds to bf16 after every op
    for a, b in zip(res["fused"], res["plain"]):
        assert a.shape == b.shape and (a.dtype == b.dtype or not autocast)
        assert orc.rel_l2(a.float().cpu(), b.float().cpu()) < tol


def test_full_size_properties():
    """At the benchmark's size (64 x 1024 tokens of width 1152), through properties that need no oracle run:
    the tangent is linear in the input tangents (a factor 2 is exact in every rounding), the dual and plain kernels
    give the same primal, LayerNorm rows have mean 0 and variance 1, the gradient sums match column sums."""
    B, L, Cn = 64, 1024, 1152
    g = torch.Generator(device=DEV).manual_seed(0)
    rn = lambda *s: torch.randn(*s, device=DEV, generator=g)
    x, tx = 3.0 * rn(B, L, Cn) + 1.0, rn(B, L, Cn)
    mods, tmods = (0.3 * rn(B, 1, 6 * Cn)).bfloat16(), (0.1 * rn(B, 1, 6 * Cn)).bfloat16()
    sh, sc, gt = mods.chunk(6, dim=-1)[:3]
    tsh, tsc, tgt = tmods.chunk(6, dim=-1)[:3]
    y, ty = adaln.ln_modulate_fwd_raw(x, tx, sh, sc, tsh, tsc, 1e-6, BF16)
    y2, ty2 = adaln.ln_modulate_fwd_raw(x, 2 * tx, sh, sc, 2 * tsh, 2 * tsc, 1e-6, BF16)
    assert torch.equal(y2, y) and torch.equal(ty2, 2 * ty)
    assert torch.equal(adaln.ln_modulate_fwd_raw(x, None, sh, sc, None, None, 1e-6, BF16)[0], y)
    zero = torch.zeros_like(mods[..., :Cn])
    n, _ = adaln.ln_modulate_fwd_raw(x, None, zero, zero, None, None, 1e-6, F32)
    assert float(n.mean(-1).abs().max()) < 1e-5 and float((n.var(-1, unbiased=False) - 1).abs().max()) < 1e-4
    h, th = rn(B, L, Cn).bfloat16(), rn(B, L, Cn).bfloat16()
    out, tout = adaln.gate_residual_fwd_raw(x, tx, h, th, gt, tgt)
    out2, tout2 = adaln.gate_residual_fwd_raw(x, 2 * tx, h, 2 * th, gt, 2 * tgt)
    assert torch.equal(out2, out) and torch.equal(tout2, 2 * tout)
    dy = rn(B, L, Cn).bfloat16()
    dx, dshift, dscale = adaln.ln_modulate_bwd_raw(dy, x, sc, 1e-6)
    assert orc.rel_l2(dshift.double(), dy.double().sum(1)) < 1e-6
    assert orc.rel_l2(dscale.double(), (dy.double() * n.double()).sum(1)) < 1e-5
    assert float(dx.mean(-1).abs().max()) < 1e-4                      # a LayerNorm gradient has zero row mean
    dh, dgate = adaln.gate_residual_bwd_raw(x, h, gt)
    assert orc.rel_l2(dgate.double(), (x.double() * h.double()).sum(1)) < 1e-6
    assert torch.equal(dh, (gt.float() * x).to(BF16))


def test_rejects_what_the_kernels_do_not_cover():
    c = _inputs(1, 8, 384, F32, BF16, BF16)
    with pytest.raises(RuntimeError):
        adaln.ln_modulate_fwd_raw(c["x"], None, c["shift"], c["scale"], None, None, 1e-6, BF16)      # CPU tensors
    g = _dev(c)
    with pytest.raises(TypeError):
        adaln.ln_modulate_fwd_raw(g["x"].half(), None, g["shift"], g["scale"], None, None, 1e-6, torch.float16)
    bad = _dev(_inputs(1, 8, 256, F32, BF16, BF16))
    with pytest.raises(RuntimeError):                                                               # width not compiled
        adaln.ln_modulate_fwd_raw(bad["x"], None, bad["shift"], bad["scale"], None, None, 1e-6, BF16)
    assert not adaln.usable(bad["x"]) and adaln.usable(g["x"], BF16) and not adaln.usable(c["x"])
