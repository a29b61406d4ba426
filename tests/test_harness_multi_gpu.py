"""The data-parallel training step on two GPUs over NCCL: the CUDA-graphed step with its bucketed all-reduce inside the
last micro-batch's graph, the graphed step with one all-reduce after it, and the eager DistributedDataParallel step
(what the reference runs, train_dmf.py:285-287, 330) must produce the same averaged gradients, and every rank must
hold the same parameters after an optimisation step.  Needs two GPUs; skipped otherwise."""

import datetime
import os
import socket
import traceback
from functools import partial

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")          # plain ring / tree: nothing of this test binds multicast memory
    import torch.distributed as dist
    from dmf_b200 import ops
    from dmf_b200.harness import train as T
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # a collective that cannot complete ends with an error after a minute instead of blocking the test
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        gen = torch.Generator(device=dev).manual_seed(5 + rank)      # every rank has its own data and noise
        eps = torch.randn(4, 4, 32, 32, device=dev, generator=gen)
        t = torch.rand(4, 1, 1, 1, device=dev, generator=gen) * 0.5 + 0.5
        r = torch.rand(4, 1, 1, 1, device=dev, generator=gen) * 0.5

        def fixed_loss(model, raw, x, y):    # the DMF loss with its random draws fixed (a captured graph owns its RNG offsets)
            x_t, v = (1 - t) * x + t * eps, eps - x
            # flow-matching term through `model` (the DDP wrapper in the eager mode: its forward is what arms the
            # gradient reducer), MeanFlow term through the raw module under torch.func.jvp, as DMFLoss does
            v_fm, lv_fm = model(x_t, t, t, y, return_logvar=True)
            (u, lv_mf), (du, _) = torch.func.jvp(partial(raw, y=y, return_logvar=True), (x_t, t, r),
                                                 (v, torch.ones_like(t), torch.zeros_like(r)))
            fm = ((v_fm - v) ** 2).mean(dim=(1, 2, 3))
            mf = ((u - (v + (r - t) * du).detach()) ** 2).mean(dim=(1, 2, 3))
            # the log-variance heads take part too (every parameter receives a gradient, as DDP expects)
            return 0.5 * (fm / lv_fm.flatten().exp() + lv_fm.flatten() + mf / lv_mf.flatten().exp() + lv_mf.flatten()), {}

        grads, losses = {}, {}
        say = lambda *a: print(f"[rank {rank}]", *a, flush=True)
        for mode in ("overlap", "single", "ddp"):
            say("mode", mode)
            st = T.build_train_state(dev, name="DMFT-S/2", input_size=32, dmf_depth=8, attn_func="fa3", seed=0,
                                     zero_init=False, graphs=(mode != "ddp"), overlap=(mode == "overlap"), n_buckets=4)
            st.loss_fn = fixed_loss
            bgen = torch.Generator(device=dev).manual_seed(100 + rank)
            batches = [T.synthetic_batch(st, 4, generator=bgen) for _ in range(2)]
            if mode == "ddp":
                loss = T.accumulate_eager(st, batches)
                flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).flatten()
                                  for p in st.model.parameters() if p.requires_grad])
            else:
                loss = T.accumulate_graphed(st, batches)
                flat = st.flat_grad.clone()
                if mode == "overlap":       # the last micro-batch ran the graph that carries the collectives
                    assert any(k[3] for k in st.graphed) and any(not k[3] for k in st.graphed)
            torch.cuda.synchronize(dev)
            grads[mode], losses[mode] = flat, float(loss)
            both = [torch.empty_like(flat) for _ in range(world)]
            dist.all_gather(both, flat)
            assert torch.equal(both[0], both[1]), f"{mode}: ranks hold different reduced gradients"
        rel = lambda a, b: float((a - b).norm() / b.norm())
        res = {"overlap_vs_ddp": rel(grads["overlap"], grads["ddp"]), "single_vs_ddp": rel(grads["single"], grads["ddp"]),
               "loss_overlap": losses["overlap"], "loss_ddp": losses["ddp"],
               "grad_norm": float(grads["ddp"].norm())}
        say("gradients compared", res)
        # one whole optimisation step with the real loss on the overlapped path: parameters stay identical across ranks
        st = T.build_train_state(dev, name="DMFT-S/2", input_size=32, dmf_depth=8, attn_func="fa3", seed=0,
                                 zero_init=False, graphs=True, overlap=True, n_buckets=4)
        torch.manual_seed(50 + rank)
        w0 = torch.cat([p.detach().flatten() for p in st.model.parameters()])
        for _ in range(2):
            loss = T.train_step(st, [T.synthetic_batch(st, 4)])
        w1 = torch.cat([p.detach().flatten() for p in st.model.parameters()])
        both = [torch.empty_like(w1) for _ in range(world)]
        dist.all_gather(both, w1)
        res["params_equal"] = bool(torch.equal(both[0], both[1]))
        res["params_moved"] = bool((w1 != w0).any())
        res["loss_finite"] = bool(torch.isfinite(loss))
        ops.check_device_status(dev)
        out[rank] = res
        say("done")
    except BaseException:
        # report, and leave without tearing the process group down: after a failure in the middle of a sequence of
        # collectives the teardown itself can block on the other rank
        out[rank] = {"error": traceback.format_exc()}
        os._exit(1)
    # Graphs that hold captured collectives must be gone before the communicator is (the teardown otherwise waits for
    # them for ever); and if the teardown still does not return, leave anyway: the results are already with the parent.
    import gc
    import threading
    del st
    gc.collect()
    torch.cuda.synchronize(dev)
    threading.Timer(20.0, lambda: os._exit(0)).start()
    dist.destroy_process_group()
    os._exit(0)


def test_graphed_allreduce_matches_ddp_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    out = mgr.dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=200)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:                      # never leave a rank behind on the GPU
        p.terminate()
        p.join(timeout=30)
    errors = {r: out[r]["error"] for r in range(world) if r in out and "error" in out[r]}
    assert not errors, "\n".join(f"rank {r}:\n{e}" for r, e in errors.items())
    assert not hung, "a rank hung"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for rank in range(world):
        res = out[rank]
        print(rank, res)
        assert res["grad_norm"] > 0
        assert res["overlap_vs_ddp"] < 1e-3 and res["single_vs_ddp"] < 1e-3
        assert abs(res["loss_overlap"] - res["loss_ddp"]) < 1e-3 * max(1.0, abs(res["loss_ddp"]))
        assert res["params_equal"] and res["params_moved"] and res["loss_finite"]
