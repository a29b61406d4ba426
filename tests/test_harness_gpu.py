"""Whole-model check on a GPU: the harness DMFT with attn_func='fa3' (the sm_100a kernels)
against the same weights with attn_func='base' (naive attention), through forward,
torch.func.jvp, the DMF loss and its backward; plus one train step and a sampler run."""

import copy

import pytest
import torch

from dmf_b200 import ops
from dmf_b200.harness import train as T
from dmf_b200.harness.loss import DMFLoss
from dmf_b200.harness.model import DMFT, build_dmft
from dmf_b200.harness.sampler import euler_sampler

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _pair(qk_norm):
    torch.manual_seed(0)
    kw = dict(input_size=32, patch_size=2, in_channels=4, hidden_size=144, depth=3, num_heads=2, dmf_depth=2,
              use_logvar=True, num_classes=1000, qk_norm=qk_norm)   # 256 tokens, head dim 72
    fa = DMFT(**kw, attn_func="fa3")
    fa.initialize_weights(zero_init=False)   # zero-initialised gates would hide the attention output
    base = DMFT(**kw, attn_func="base")
    base.load_state_dict(fa.state_dict())
    return fa.to(DEV), base.to(DEV)


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("qk_norm", [False, True])
def test_model_jvp_and_loss_gradients_match_base_attention(qk_norm):
    fa, base = _pair(qk_norm)
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(4, 4, 32, 32, device=DEV, generator=g)
    y = torch.randint(0, 1000, (4,), device=DEV, generator=g)
    t = torch.rand(4, 1, 1, 1, device=DEV, generator=g)
    r = t * torch.rand(4, 1, 1, 1, device=DEV, generator=g)
    v = torch.randn(4, 4, 32, 32, device=DEV, generator=g)
    outs = []
    for m in (fa, base):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            (u, lv), (du, _) = torch.func.jvp(lambda a, b, c: m(a, b, c, y=y, return_logvar=True), (x, t, r),
                                              (v, torch.ones_like(t), torch.zeros_like(r)))
        outs.append((u, du))
    assert _rel(outs[0][0], outs[1][0]) < 2e-2
    assert _rel(outs[0][1], outs[1][1]) < 3e-2
    grads = []
    for m in (fa, base):
        torch.manual_seed(5)
        m.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss, _ = DMFLoss()(m, m, x, y)
        loss.mean().backward()
        grads.append((float(loss.mean()), m.blocks[0].attn.qkv.weight.grad.clone(), m.blocks[2].mlp.fc1.weight.grad.clone()))
    assert abs(grads[0][0] - grads[1][0]) < 2e-2 * max(1.0, abs(grads[1][0]))
    assert _rel(grads[0][1], grads[1][1]) < 5e-2
    assert _rel(grads[0][2], grads[1][2]) < 5e-2
    ops.check_device_status(DEV)


def test_train_step_and_sampler_run():
    st = T.build_train_state(DEV, name="DMFT-S/2", input_size=32, dmf_depth=8, attn_func="fa3", seed=0,
                             zero_init=False)
    before = copy.deepcopy(st.model.state_dict())
    n0 = ops.launch_count
    loss = T.train_step(st, [T.synthetic_batch(st, 4), T.synthetic_batch(st, 4)])
    assert torch.isfinite(loss)
    # per micro-batch, two passes over 12 blocks (plain + dual), each backpropagated (a backward call = 2 kernels):
    # attention 24 forwards, LayerNorm-modulate 2 per block + the final layer = 50, gate-residual 2 per block = 48
    assert ops.launch_count - n0 == 2 * (24 + 50 + 48) * (1 + 2)
    assert any(not torch.equal(v, before[k]) for k, v in st.model.state_dict().items())
    model = st.model.to(torch.bfloat16).eval()
    z = torch.randn(4, 4, 32, 32, device=DEV, dtype=torch.bfloat16)
    y = torch.randint(0, 1000, (4,), device=DEV)
    out = euler_sampler(model, z, y, num_steps=4, shift=1.5)
    assert out.shape == (4, 4, 32, 32) and out.dtype == torch.float64 and bool(torch.isfinite(out).all())
    ops.check_device_status(DEV)


def test_graphed_micro_step_gives_the_eager_gradients():
    """Forward + backward replayed as a CUDA graph against the same computation launched eagerly, with a loss whose
    random draws are fixed tensors (a captured graph owns its own RNG offsets, so DMFLoss's draws would differ)."""
    from functools import partial
    st = T.build_train_state(DEV, name="DMFT-S/2", input_size=32, dmf_depth=8, attn_func="fa3", seed=0,
                             zero_init=False, graphs=True)
    gen = torch.Generator(device=DEV).manual_seed(5)
    x, y = T.synthetic_batch(st, 4, generator=gen)
    eps = torch.randn(4, 4, 32, 32, device=DEV, generator=gen)
    t = torch.rand(4, 1, 1, 1, device=DEV, generator=gen) * 0.5 + 0.5
    r = torch.rand(4, 1, 1, 1, device=DEV, generator=gen) * 0.5

    def fixed_loss(model, raw, x, y):
        x_t, v = (1 - t) * x + t * eps, eps - x
        (u, _), (du, _) = torch.func.jvp(partial(raw, y=y, return_logvar=True), (x_t, t, r),
                                         (v, torch.ones_like(t), torch.zeros_like(r)))
        return ((u - (v + (r - t) * du).detach()) ** 2).mean(dim=(1, 2, 3)), {}

    st.loss_fn = fixed_loss
    step = T.GraphedMicroStep(st, 4, 1, torch.bfloat16)
    grads = []
    for _ in range(2):                                   # two replays: identical, and nothing leaks between them
        st.flat_grad.zero_()
        n0 = ops.launch_count
        loss = step(x, y)
        assert ops.launch_count - n0 == (12 + 25 + 24) * 3   # one dual pass over 12 blocks, backpropagated
        grads.append((float(loss), st.flat_grad.clone()))
    assert grads[0][0] == grads[1][0] and torch.equal(grads[0][1], grads[1][1])
    st.flat_grad.zero_()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        eager, _ = fixed_loss(st.model, st.model, x, y)
    eager.mean().backward()
    assert abs(float(eager.mean()) - grads[0][0]) < 1e-3 * max(1.0, abs(grads[0][0]))
    assert _rel(st.flat_grad, grads[0][1]) < 1e-3
    # a whole graphed optimisation step with the real loss: runs, moves the weights, keeps p.grad views of the buffer
    st = T.build_train_state(DEV, name="DMFT-S/2", input_size=32, dmf_depth=8, attn_func="fa3", seed=0,
                             zero_init=False, graphs=True)
    w0 = st.model.blocks[3].attn.qkv.weight.detach().clone()
    for _ in range(2):
        loss = T.train_step(st, [T.synthetic_batch(st, 4), T.synthetic_batch(st, 4)])
    assert torch.isfinite(loss) and not torch.equal(w0, st.model.blocks[3].attn.qkv.weight)
    p = next(q for q in st.model.parameters() if q.requires_grad)
    assert p.grad.data_ptr() == st.flat_grad.data_ptr() and float(st.flat_grad.abs().max()) == 0.0
    ops.check_device_status(DEV)


def test_graphed_sampler_matches_the_eager_loop():
    from dmf_b200.harness.sampler import GraphedSampler
    torch.manual_seed(0)
    model = build_dmft("DMFT-S/2", input_size=32, dmf_depth=8, use_logvar=False, num_classes=1000, attn_func="fa3",
                       qk_norm=True)
    model.initialize_weights(zero_init=False)
    model = model.to(DEV).to(torch.bfloat16).eval()
    z = torch.randn(4, 4, 32, 32, device=DEV, dtype=torch.bfloat16)
    y = torch.randint(0, 1000, (4,), device=DEV)
    want = euler_sampler(model, z, y, num_steps=4, shift=1.5)
    g = GraphedSampler(model, 4, (4, 32, 32), torch.bfloat16, DEV, num_steps=4, shift=1.5)
    n0 = ops.launch_count
    got = g(z, y).clone()
    # per step: 12 attention forwards, 24 q/k norms, 25 LayerNorm-modulates, 24 gate-residuals
    assert ops.launch_count - n0 == 4 * (12 + 24 + 25 + 24)
    assert got.dtype == torch.float64 and _rel(got, want) < 1e-3
    assert torch.equal(g(z, y), got)                     # replays are deterministic
    z2 = torch.randn_like(z)
    assert _rel(g(z2, y), euler_sampler(model, z2, y, num_steps=4, shift=1.5)) < 1e-3
    ops.check_device_status(DEV)
