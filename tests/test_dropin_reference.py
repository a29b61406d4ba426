"""The reference's REAL attention block over this package's drop-in.

``models/layers.py`` of the reference (an unmodified copy under baseline/_ref, staged by __graft_entry__.build() where
the reference tree is present) is imported with ``dmf_b200.dropin.install()`` in effect, so that its
``from .flash_attention_2_jvp import flash_attn_func`` lines (models/layers.py:23-24) resolve to this package, and its
own ``Attention`` module (models/layers.py:118-154) is run:

* on CPU, with this package's ``flash_attn_func`` replaced by a recorder: the module hands over (B, L, H, D) tensors in
  exactly the layouts the kernels are written for - q, k contiguous after the qk-norm, v (and everything without a
  qk-norm) as strided views of the packed projection with strides (L*3*H*D, 3*H*D, D, 1);
* on a GPU, under torch.func.jvp and autograd, against the same module with ``attn_func='base'`` (naive attention).

Skipped where the copy of the reference files is absent.
"""

import importlib
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

needs_ref = pytest.mark.skipif(not (REF / "models" / "layers.py").exists(),
                               reason="no copy of the reference's models/layers.py under baseline/_ref")


@pytest.fixture
def ref_layers():
    """The reference's models.layers imported over the drop-in; restores sys.modules / sys.path afterwards."""
    import dmf_b200.dropin as dropin
    saved = {n: m for n, m in sys.modules.items() if n == "models" or n.startswith("models.")}
    for n in saved:
        del sys.modules[n]
    sys.path.insert(0, str(REF))
    try:
        dropin.install()
        layers = importlib.import_module("models.layers")
        assert Path(layers.__file__).resolve() == (REF / "models" / "layers.py").resolve()
        yield layers
    finally:
        sys.path.remove(str(REF))
        for n in [n for n in sys.modules if n == "models" or n.startswith("models.")]:
            del sys.modules[n]
        sys.modules.update(saved)


@needs_ref
@pytest.mark.parametrize("qk_norm", [True, False])
@pytest.mark.parametrize("selector", ["fa2", "fa3"])
def test_reference_attention_hands_the_dropin_the_layouts_it_expects(ref_layers, monkeypatch, qk_norm, selector):
    import dmf_b200
    assert ref_layers.fa2_func is dmf_b200.flash_attn_func and ref_layers.fa3_func is dmf_b200.flash_attn_func
    seen = {}

    def recorder(q, k, v, softmax_scale=None):
        seen.update(q=q, k=k, v=v, scale=softmax_scale)
        return torch.zeros(q.shape, dtype=q.dtype)

    # attn_op looks the two names up in the module at call time (models/layers.py:96-99)
    monkeypatch.setattr(ref_layers, "fa2_func", recorder)
    monkeypatch.setattr(ref_layers, "fa3_func", recorder)
    B, L, Hh, D = 2, 128, 2, 72
    attn = ref_layers.Attention(dim=Hh * D, num_heads=Hh, qkv_bias=True, qk_norm=qk_norm, attn_func=selector)
    out = attn(torch.randn(B, L, Hh * D))
    assert out.shape == (B, L, Hh * D) and seen["scale"] is None
    packed = (L * 3 * Hh * D, 3 * Hh * D, D, 1)
    for name in ("q", "k", "v"):
        assert tuple(seen[name].shape) == (B, L, Hh, D), name
    assert tuple(seen["v"].stride()) == packed
    for name in ("q", "k"):
        if qk_norm:
            assert seen[name].is_contiguous(), name
        else:
            assert tuple(seen[name].stride()) == packed, name


@needs_ref
@pytest.mark.gpu
@pytest.mark.parametrize("qk_norm", [True, False])
def test_reference_attention_over_the_dropin_matches_its_base_path_on_gpu(ref_layers, qk_norm):
    from dmf_b200 import ops
    dev = torch.device("cuda:0")
    B, L, Hh, D = 2, 256, 2, 72
    torch.manual_seed(0)
    fa = ref_layers.Attention(dim=Hh * D, num_heads=Hh, qkv_bias=True, qk_norm=qk_norm, attn_func="fa3").to(dev)
    base = ref_layers.Attention(dim=Hh * D, num_heads=Hh, qkv_bias=True, qk_norm=qk_norm, attn_func="base").to(dev)
    base.load_state_dict(fa.state_dict())
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(B, L, Hh * D, device=dev, generator=g)
    tx = 0.1 * torch.randn(B, L, Hh * D, device=dev, generator=g)
    dy = torch.randn(B, L, Hh * D, device=dev, generator=g)
    n0 = ops.launch_count
    res = []
    for m in (fa, base):
        m.zero_grad()
        # the kernels under bf16 autocast (how training runs them); the naive path in fp32, as the parity bar is stated
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=m is fa):
            y, ty = torch.func.jvp(m, (x,), (tx,))
        y.float().backward(dy)
        res.append((y.float(), ty.float(), m.qkv.weight.grad.clone()))
    assert ops.launch_count - n0 == 3          # one fused forward + tangent launch, two backward launches
    rel = lambda a, b: float((a - b).norm() / b.norm())
    assert rel(res[0][0], res[1][0]) <= 2e-2    # O through the block
    assert rel(res[0][1], res[1][1]) <= 2e-2    # its tangent
    assert rel(res[0][2], res[1][2]) <= 3e-2    # primal backward into the qkv projection
    ops.check_device_status(dev)
