"""The measurement harness (DMFT model, DMF loss, Euler sampler, train step) on CPU against
golden vectors produced by the reference's own model / loss / sampler code, and the
data-parallel train step on two gloo ranks."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from dmf_b200.harness.loss import DMFLoss
from dmf_b200.harness.model import DMFT, build_dmft
from dmf_b200.harness.sampler import euler_sampler, get_tsteps
from tests.conftest import GOLDEN
from tests.golden.make_golden_model import TINY, tiny_inputs


def _model(qk_norm):
    torch.manual_seed(7)
    m = DMFT(**TINY, attn_func="base", qk_norm=qk_norm)
    m.initialize_weights(zero_init=False)
    return m


@pytest.mark.parametrize("qk_norm", [False, True])
def test_model_loss_sampler_match_reference(qk_norm):
    g = np.load(GOLDEN / "dmft_tiny.npz")
    tag = "qkn" if qk_norm else "plain"
    m = _model(qk_norm)
    x, y, t, r = tiny_inputs()
    with torch.no_grad():
        o, lv = m(x, t, r, y, return_logvar=True)
    np.testing.assert_allclose(o.numpy(), g[f"{tag}_fwd"], rtol=0, atol=2e-6)
    np.testing.assert_allclose(lv.numpy(), g[f"{tag}_logvar"], rtol=0, atol=2e-6)
    # the loss consumes the global CPU generator in the reference's order when times are drawn on the host
    torch.manual_seed(11)
    loss, ld = DMFLoss(sample_on_device=False)(m, m, x, y)
    loss.mean().backward()
    np.testing.assert_allclose(loss.detach().numpy(), g[f"{tag}_loss"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(ld["mf_loss"].detach().numpy(), g[f"{tag}_mf_loss"], rtol=1e-4, atol=1e-5)
    gn = torch.stack([p.grad.norm() for p in m.parameters() if p.grad is not None])
    np.testing.assert_allclose(gn.numpy(), g[f"{tag}_grad_norms"], rtol=2e-4, atol=1e-7)
    np.testing.assert_allclose(m.blocks[0].attn.qkv.weight.grad.numpy(), g[f"{tag}_grad_qkv0"], rtol=0, atol=2e-6)
    gen = torch.Generator().manual_seed(5)
    z = torch.randn(4, 4, 8, 8, generator=gen)
    out = euler_sampler(m, z, y, num_steps=4, shift=1.5)
    assert out.dtype == torch.float64
    np.testing.assert_allclose(out.numpy(), g[f"{tag}_euler"], rtol=0, atol=1e-5)


def test_xl2_parameter_count_and_time_grid():
    with torch.device("meta"):
        m = build_dmft("DMFT-XL/2", input_size=32, dmf_depth=20, use_logvar=True, num_classes=1000)
    n_all = sum(p.numel() for p in m.parameters())
    n_train = sum(p.numel() for p in m.parameters() if p.requires_grad)
    assert n_all == 675_111_441 and n_train == 674_816_529
    ts = get_tsteps(4, shift=1.5)
    assert ts[0] == 1.0 and ts[-1] == 0.0 and torch.all(ts[:-1] > ts[1:])
    assert abs(float(ts[2]) - 1.5 * 0.5 / (1 + 0.5 * 0.5)) < 1e-12


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _ddp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from dmf_b200.harness import train as T
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dev = torch.device("cpu")
        st = T.build_train_state(dev, name="DMFT-S/2", input_size=8, dmf_depth=8, attn_func="base", seed=3,
                                 zero_init=False)
        # shrink: 2 blocks are enough for the plumbing
        gen = torch.Generator().manual_seed(100 + rank)
        batches = [T.synthetic_batch(st, 2, generator=gen) for _ in range(2)]   # 2 micro-batches per rank
        torch.manual_seed(50 + rank)
        before = [p.detach().clone() for p in st.model.parameters()]
        loss = T.train_step(st, batches, autocast_dtype=torch.bfloat16)
        after = torch.cat([p.detach().flatten() for p in st.model.parameters()])
        moved = float(sum((a - b).abs().sum() for a, b in zip(st.model.parameters(), before)))
        # every rank must hold identical parameters after the all-reduced step
        gathered = [torch.zeros_like(after) for _ in range(world)]
        dist.all_gather(gathered, after)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        ema_moved = float(sum((a - b).abs().sum() for a, b in zip(st.ema.parameters(), before)))
        out[rank] = (bool(torch.isfinite(loss)), moved > 0, same, ema_moved > 0)
    finally:
        dist.destroy_process_group()


def test_train_step_two_gloo_ranks():
    world, port = 2, _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_ddp_worker, args=(world, port, out), nprocs=world, join=True)
    for rank in range(world):
        finite, moved, same, ema_moved = out[rank]
        assert finite and moved and same and ema_moved


def _failing_worker(rank, world, port, out):
    """Rank 1 fails on the host before the gradient all-reduce (it never enters the step); rank 0 must not hang:
    its step ends with an exception within the process group's timeout and the group is torn down."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    from dmf_b200.harness import train as T
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    dev = torch.device("cpu")
    st = T.build_train_state(dev, name="DMFT-S/2", input_size=8, dmf_depth=8, attn_func="base", seed=3, zero_init=False)
    gen = torch.Generator().manual_seed(100 + rank)
    batches = [T.synthetic_batch(st, 2, generator=gen)]
    dist.barrier()                      # both ranks are up and the model is wrapped
    if rank == 1:
        out[rank] = "raised before the all-reduce"
        raise RuntimeError("injected host-side failure on rank 1")
    t0 = time.time()
    try:
        T.train_step(st, batches)
        out[rank] = "no error"
    except Exception as e:              # gloo: peer closed the connection, or the collective timed out
        out[rank] = f"error after {time.time() - t0:.1f} s: {type(e).__name__}"
    try:
        dist.destroy_process_group()
        out["teardown"] = "ok"
    except Exception as e:
        out["teardown"] = f"failed: {e!r}"


def test_a_rank_that_fails_before_the_allreduce_ends_the_other_ranks_step_with_an_error():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    out = mgr.dict()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
        p.join(timeout=30)
    assert not hung, "a rank hung"
    assert procs[1].exitcode != 0                       # the injected failure
    assert procs[0].exitcode == 0
    assert out[1] == "raised before the all-reduce"
    assert out[0].startswith("error after"), out[0]
    assert float(out[0].split()[2]) < 60.0
    assert out["teardown"] == "ok"
