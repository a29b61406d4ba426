"""The reference-facing Python surface on a GPU: flash_attn_func under torch.func.jvp,
autograd through the primal, stop-gradient on the tangent, the drop-in shim.  Mirrors
the reference's own test_jvp (models/flash_attention_2_jvp.py:339-376) with seeded inputs
and the CPU oracle in place of the unseeded CUDA randoms."""

import sys

import pytest
import torch
import torch.autograd.forward_ad as fwAD

from dmf_b200 import FlashAttnFunc, flash_attn_func, flash_attn_qkvpacked_func
from oracle import attn_jvp_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ins(B, L, H, D, seed=0, std=0.5):
    xs = orc.make_inputs(B, L, H, D, seed=seed, n_extra=1)
    return [(x * std).bfloat16().to(DEV) for x in xs]


@pytest.mark.parametrize("L", [256, 1024])
@pytest.mark.parametrize("H", [16])
@pytest.mark.parametrize("D", [64, 72, 96, 128])
def test_jvp_and_backward_like_reference_test(L, H, D):
    """b=2, inputs N(0, 0.5^2), bf16: u, du and dq, dk, dv against naive attention;
    the reference asserts atol 1.2e-3 against a bf16 naive result, we assert against
    the fp64 oracle (on the same bf16 inputs) with atol for bf16 output rounding."""
    q, k, v, dq, dk, dv, do = _ins(2, L, H, D, seed=L + D)
    q, k, v = (x.requires_grad_(True) for x in (q, k, v))
    u, du = torch.func.jvp(flash_attn_func, (q, k, v), (dq, dk, dv))
    u.backward(do)
    ref = [x.detach().float().cpu() for x in (q, k, v, dq, dk, dv)]
    u_ref, du_ref, _ = orc.attn_jvp_closed_form(*ref)
    gq, gk, gv = orc.attn_bwd_closed_form(*ref[:3], do.float().cpu())
    atol = 4e-3
    torch.testing.assert_close(u.detach().float().cpu(), u_ref.float(), atol=atol, rtol=0)
    torch.testing.assert_close(du.detach().float().cpu(), du_ref.float(), atol=atol, rtol=0)
    torch.testing.assert_close(q.grad.float().cpu(), gq.float(), atol=atol, rtol=0)
    torch.testing.assert_close(k.grad.float().cpu(), gk.float(), atol=atol, rtol=0)
    torch.testing.assert_close(v.grad.float().cpu(), gv.float(), atol=atol, rtol=0)
    for got, want in ((u, u_ref), (du, du_ref), (q.grad, gq), (k.grad, gk), (v.grad, gv)):
        assert orc.rel_l2(got.detach().float().cpu(), want) < 2e-2


def test_non_dual_path_and_default_scale():
    q, k, v, *_ = _ins(2, 256, 4, 72, seed=1)
    out = flash_attn_func(q, k, v)
    o_ref, _ = orc.attn_fwd_closed_form(*[x.float().cpu() for x in (q, k, v)])
    assert orc.rel_l2(out.float().cpu(), o_ref) < 6e-3
    out2 = flash_attn_func(q, k, v, softmax_scale=0.2)
    o_ref2, _ = orc.attn_fwd_closed_form(*[x.float().cpu() for x in (q, k, v)], softmax_scale=0.2)
    assert orc.rel_l2(out2.float().cpu(), o_ref2) < 6e-3
    assert fwAD.unpack_dual(out).tangent is None


def test_missing_tangents_become_zeros():
    """Only q carries a tangent: k and v tangents are zero-filled (flash_attention_2_jvp.py:303-304)."""
    q, k, v, tq, *_ = _ins(1, 256, 2, 64, seed=2)
    with fwAD.dual_level():
        out = flash_attn_func(fwAD.make_dual(q, tq), k, v)
        o, to = fwAD.unpack_dual(out)
    z = torch.zeros_like(k).float().cpu()
    _, do_ref, _ = orc.attn_jvp_closed_form(q.float().cpu(), k.float().cpu(), v.float().cpu(), tq.float().cpu(), z, z)
    assert to is not None and orc.rel_l2(to.float().cpu(), do_ref) < 6e-3


def test_stop_gradient_on_tangent():
    """Back-propagating through the tangent output reaches neither primals nor tangents:
    FlashAttnFunc.backward ignores the gradient of `to` (flash_attention_2_jvp.py:260-276)."""
    q, k, v, tq, tk, tv, do = _ins(1, 256, 2, 72, seed=3)
    q, k, v, tq, tk, tv = (x.requires_grad_(True) for x in (q, k, v, tq, tk, tv))
    o, m, to = FlashAttnFunc.apply(q, k, v, tq, tk, tv, None)
    assert m.shape == (1, 2, 256) and m.dtype == torch.float32
    (to.float() * do.float()).sum().backward()
    for x in (q, k, v):
        assert x.grad is not None and float(x.grad.float().abs().max()) == 0.0
    for x in (tq, tk, tv):
        assert x.grad is None
    # while the primal output does propagate
    o2, _, _ = FlashAttnFunc.apply(q, k, v, tq, tk, tv, None)
    o2.backward(do)
    assert float(q.grad.float().abs().max()) > 0


def test_jvp_staticmethod_returns_saved_tangent():
    class Ctx:
        saved_forward = ("T",)
    assert FlashAttnFunc.jvp(Ctx()) == ("T", None, None)
    assert FlashAttnFunc.jvp(object()) == (None, None, None)


def test_dropin_modules_resolve_to_this_package():
    import dmf_b200.dropin as dropin
    saved = {n: sys.modules.pop(n, None) for n in dropin._NAMES}
    try:
        dropin.install()
        import importlib
        m2 = importlib.import_module("models.flash_attention_2_jvp")
        m3 = importlib.import_module("models.flash_attention_3_jvp")
        assert m2.flash_attn_func is flash_attn_func and m3.flash_attn_func is flash_attn_func
        q, k, v, *_ = _ins(1, 128, 1, 64, seed=4)
        assert m3.flash_attn_func(q, k, v).shape == q.shape
    finally:
        dropin.uninstall()
        for n, mod in saved.items():
            if mod is not None:
                sys.modules[n] = mod


def test_torch_compile_traces_the_plain_path():
    q, k, v, *_ = _ins(1, 256, 2, 64, seed=5)
    f = torch.compile(lambda a, b, c: flash_attn_func(a, b, c) * 2, fullgraph=False, dynamic=True)
    out = f(q, k, v)
    assert orc.rel_l2(out.float(), 2 * flash_attn_func(q, k, v).float()) < 1e-6


@pytest.mark.parametrize("D", [64, 72])
def test_qkvpacked_is_the_same_computation_with_a_packed_gradient(D):
    """flash_attn_qkvpacked_func on the (B, L, 3, H, D) projection against flash_attn_func on its slices: outputs,
    tangents and gradients bit for bit (the same kernels on the same views; only where dq, dk, dv land differs)."""
    q, k, v, dq, dk, dv, do = _ins(2, 256, 4, D, seed=D)
    qkv = torch.stack([q, k, v], dim=2)
    tqkv = torch.stack([dq, dk, dv], dim=2)
    a = qkv.clone().requires_grad_(True)
    u1, du1 = torch.func.jvp(flash_attn_qkvpacked_func, (a,), (tqkv,))
    u1.backward(do)
    b = qkv.clone().requires_grad_(True)
    u2, du2 = torch.func.jvp(lambda t: flash_attn_func(t[:, :, 0], t[:, :, 1], t[:, :, 2]), (b,), (tqkv,))
    u2.backward(do)
    assert torch.equal(u1, u2) and torch.equal(du1, du2) and torch.equal(a.grad, b.grad)
    assert a.grad.shape == qkv.shape and a.grad.is_contiguous()
    c = qkv.clone().requires_grad_(True)
    u3 = flash_attn_qkvpacked_func(c)                    # no tangent: the plain forward
    u3.backward(do)
    assert torch.equal(u3, u1) and torch.equal(c.grad, a.grad)
    with pytest.raises(ValueError):
        flash_attn_qkvpacked_func(q)


def test_long_sequence_backward_replays_in_a_cuda_graph():
    """Forward + backward at three tiles (the backward's long-sequence kernels: a memset, the pre-kernel, the main
    kernel, the conversion; the workspace comes from the graph's memory pool) captured once and replayed: dk, dv
    bit-identical to the eager call, dq equal up to the order of its fp32 additions."""
    q, k, v, _, _, _, do = _ins(2, 384, 3, 72, seed=7)
    a, b_, c = (x.clone().requires_grad_(True) for x in (q, k, v))
    flash_attn_func(a, b_, c).backward(do)
    eager = [x.grad.clone() for x in (a, b_, c)]
    sq, sk, sv = (x.clone().requires_grad_(True) for x in (q, k, v))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):          # warm-up outside the capture
        flash_attn_func(sq, sk, sv).backward(do)
    torch.cuda.current_stream().wait_stream(side)
    for x in (sq, sk, sv):
        x.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        flash_attn_func(sq, sk, sv).backward(do)
    for _ in range(2):
        for x in (sq, sk, sv):
            x.grad.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(sk.grad, eager[1]) and torch.equal(sv.grad, eager[2])
        assert orc.rel_l2(sq.grad.float().cpu(), eager[0].float().cpu()) < 1e-3
