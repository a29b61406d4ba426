"""One optimisation step of DMF fine-tuning, as train_dmf.py:320-338 runs it:
bf16 autocast, DMF loss (flow-matching forward + JVP forward), backward, gradient
all-reduce (DDP over NCCL when world size > 1), clip to 1.0, fused AdamW, EMA 0.9999.

The reference reaches DDP through HF accelerate; here it is plain
torch.nn.parallel.DistributedDataParallel.  A global batch that does not fit one
GPU in a single pass is split into micro-batches with gradient accumulation
(``no_sync`` on all but the last), so that every world size runs the same
micro-batch shape.

With ``graphs=True`` (CUDA only) the forward + backward of a micro-batch is captured once in a CUDA
graph and replayed: eager PyTorch needs about 6300 kernel launches per micro-batch of DMFT-XL/2
(forward-mode AD decomposes into small kernels) and is bound by the host at ~37 us per launch,
about twice the GPU time.  Gradients then live in one flat fp32 buffer (each ``p.grad`` is a view
of it) that the captured backward accumulates into.  Across ranks the buffer is averaged by NCCL in
place of the DDP wrapper, in one of two ways:

* ``overlap=True`` (default): the buffer is cut into a few contiguous buckets, last parameters
  first (the order in which backward finishes them).  The graph of a rank's LAST micro-batch carries
  one all-reduce per bucket on a second stream, each starting as soon as the bucket's last gradient
  has been accumulated, so the collective runs under the rest of the backward pass (what DDP's
  bucketed reducer does, train_dmf.py:285-287, captured instead of launched from hooks every step);
* ``overlap=False``: a single all-reduce of the whole buffer after the last micro-batch.

Either way the mean over ranks is taken by scaling the loss by 1 / world size before backward (a
power of two on 2, 4, 8 GPUs: exact), not by a pass over the reduced buffer.  With ``fused_tail=True``
(default) parameters, AdamW moments and EMA copies live in flat buffers as well and the rest of the
step - clipping, AdamW, EMA, zeroing of the gradients - is one norm reduction plus ONE kernel
(``dmf_step_tail``); otherwise torch's fused AdamW (with the clipping coefficient as its grad_scale)
and two foreach EMA calls.

Graphs that hold captured collectives must be released (drop the TrainState) before the process
group is destroyed; the teardown otherwise waits for them.
"""

from __future__ import annotations

import contextlib
import copy
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

from .. import ops as _ops
from ..step import FlatAdamW
from .loss import DMFLoss
from .model import build_dmft


@torch.no_grad()
def update_ema(ema, model, decay: float = 0.9999):
    """EMA of the trainable parameters, buffers copied (train_dmf.py:54-99), as two foreach calls."""
    src = [p for p in model.parameters() if p.requires_grad]
    dst = [q for q, p in zip(ema.parameters(), model.parameters()) if p.requires_grad]
    torch._foreach_mul_(dst, decay)
    torch._foreach_add_(dst, src, alpha=1.0 - decay)
    for b_ema, b in zip(ema.buffers(), model.buffers()):
        b_ema.copy_(b)


@dataclass
class TrainState:
    model: torch.nn.Module       # raw module
    wrapped: torch.nn.Module     # DDP wrapper (or the raw module on one process)
    ema: torch.nn.Module
    opt: torch.optim.Optimizer
    loss_fn: DMFLoss
    device: torch.device
    input_size: int
    graphs: bool = False
    flat_grad: torch.Tensor | None = None   # graphs: all gradients, one buffer
    graphed: dict | None = None             # graphs: (batch, n_micro, dtype, reduces?) -> GraphedMicroStep
    overlap: bool = True                    # graphs, world > 1: bucketed all-reduce inside the last micro-batch's graph
    n_buckets: int = 8
    bucket_bounds: list | None = None       # [(lo, hi, [parameters])] over flat_grad, in launch order
    comm_stream: torch.cuda.Stream | None = None
    pool: object | None = None              # memory pool shared by this state's graphs (they never run concurrently)
    timing: dict | None = None              # set to {} to have train_step record CUDA events around its phases
    steps_done: int = 0
    flat_param: torch.Tensor | None = None  # graphs + fused tail: all trainable parameters, one buffer (p.data are views)
    flat_ema: torch.Tensor | None = None    # ... and their EMA copies
    flat_opt: FlatAdamW | None = None       # ... and the AdamW moments; None: torch's fused AdamW + foreach EMA


def build_train_state(device, *, name: str = "DMFT-XL/2", input_size: int = 32, dmf_depth: int = 20,
                      attn_func: str = "fa3", qk_norm: bool = False, seed: int = 0, lr: float = 1e-4,
                      zero_init: bool = True, graphs: bool = False, overlap: bool = True,
                      n_buckets: int = 8, fused_tail: bool = True) -> TrainState:
    torch.manual_seed(seed)  # same initial weights on every rank
    model = build_dmft(name, input_size=input_size, dmf_depth=dmf_depth, use_logvar=True, num_classes=1000,
                       attn_func=attn_func, qk_norm=qk_norm)
    if not zero_init:
        model.initialize_weights(zero_init=False)
    model = model.to(device)
    ema = copy.deepcopy(model).requires_grad_(False)
    wrapped = model
    graphs = graphs and torch.device(device).type == "cuda"
    if not graphs and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        wrapped = DDP(model, device_ids=[device.index] if device.type == "cuda" else None)
    opt = torch.optim.AdamW((p for p in model.parameters() if p.requires_grad), lr=lr, betas=(0.9, 0.95),
                            weight_decay=0.0, eps=1e-8, fused=(device.type == "cuda"))
    state = TrainState(model, wrapped, ema, opt, DMFLoss(), device, input_size, graphs=graphs)
    if graphs:
        params = [p for p in model.parameters() if p.requires_grad]
        state.flat_grad = torch.zeros(sum(p.numel() for p in params), dtype=torch.float32, device=device)
        off = 0
        for p in params:
            assert p.dtype == torch.float32
            p.grad = state.flat_grad[off:off + p.numel()].view_as(p)
            off += p.numel()
        state.graphed = {}
        state.overlap, state.n_buckets = overlap, n_buckets
        state.bucket_bounds = _make_buckets(params, n_buckets)
        state.comm_stream = torch.cuda.Stream(device=device)
        # the clipping coefficient reaches the fused AdamW kernel as its grad_scale (it divides by it)
        opt.grad_scale = torch.ones((), dtype=torch.float32, device=device)
        if fused_tail:
            # parameters and their EMA copies move into flat buffers too (each tensor becomes a view), so that clipping,
            # AdamW, the EMA and the zeroing of the gradients are one pass of one kernel over five buffers
            def flatten(tensors):
                flat = torch.empty(sum(t.numel() for t in tensors), dtype=torch.float32, device=device)
                o = 0
                for t in tensors:
                    flat[o:o + t.numel()].copy_(t.detach().reshape(-1))
                    t.data = flat[o:o + t.numel()].view_as(t)
                    o += t.numel()
                return flat
            state.flat_param = flatten(params)
            state.flat_ema = flatten([q for q, p in zip(ema.parameters(), model.parameters()) if p.requires_grad])
            state.flat_opt = FlatAdamW(state.flat_param, lr=lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    return state


def _make_buckets(params, n_buckets: int):
    """Cut the flat gradient buffer into at most ``n_buckets`` contiguous ranges of about equal size, at parameter
    boundaries, listed from the END of the buffer: backward produces the gradients of the last layers first."""
    sizes = [p.numel() for p in params]
    total = sum(sizes)
    target = -(-total // max(1, n_buckets))
    bounds, hi, acc, members = [], total, 0, []
    for p, n in zip(reversed(params), reversed(sizes)):
        acc += n
        members.append(p)
        if acc >= target:
            bounds.append((hi - acc, hi, members))
            hi, acc, members = hi - acc, 0, []
    if members:
        bounds.append((hi - acc, hi, members))
    assert bounds[-1][0] == 0 and sum(b[1] - b[0] for b in bounds) == total
    return bounds


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


class GraphedMicroStep:
    """loss(x, y) / (n_micro * world) and its backward (accumulating into the existing ``p.grad``), captured in a CUDA
    graph.  With ``reduce_in_graph`` the capture also holds the bucketed all-reduce of the flat gradient buffer on the
    state's second stream (see the module docstring); such a graph is only replayed for a rank's last micro-batch."""

    def __init__(self, state: TrainState, batch: int, n_micro: int, autocast_dtype, reduce_in_graph: bool = False):
        dev, S = state.device, state.input_size
        self.x = torch.zeros(batch, 4, S, S, device=dev)
        self.y = torch.zeros(batch, dtype=torch.long, device=dev)
        self.n_micro, self.autocast_dtype, self.state = n_micro, autocast_dtype, state
        self.loss_div = float(n_micro * _world())
        self.reduce_in_graph = reduce_in_graph
        keep = state.flat_grad.clone()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):        # warm-up outside the capture: lazy initialisations, allocator
            for _ in range(3):
                self._fwd_bwd(False)
        torch.cuda.current_stream(dev).wait_stream(side)
        if reduce_in_graph:
            # NCCL sets a transport up the first time a collective needs it (which one depends on the message size):
            # that involves allocations and a handshake between the ranks, neither of which may happen inside a
            # capture.  So every bucket is all-reduced once here, at its real size (flat_grad is restored below).
            for lo, hi, _ in state.bucket_bounds:
                dist.all_reduce(state.flat_grad[lo:hi])
            torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        launches0 = _ops.launch_count
        with torch.cuda.graph(self.graph, pool=state.pool):
            self.loss = self._fwd_bwd(reduce_in_graph)
        if state.pool is None:
            state.pool = self.graph.pool()
        self.launches = _ops.launch_count - launches0   # kernels of this package inside the graph
        state.flat_grad.copy_(keep)          # the warm-up passes accumulated; the capture itself ran nothing

    def _fwd_bwd(self, reduce_buckets: bool):
        st = self.state
        with torch.autocast(device_type="cuda", dtype=self.autocast_dtype):
            loss, _ = st.loss_fn(st.model, st.model, self.x, self.y)
        loss = loss.mean() / self.loss_div
        if not reduce_buckets:
            loss.backward()
            return loss.detach()
        # Bucketed all-reduce under the backward pass.  A hook on every parameter counts its bucket down once the
        # gradient has been accumulated; buckets are launched strictly in list order (a bucket that completes early
        # waits for the ones before it), so every rank issues the same sequence of collectives.
        main, comm = torch.cuda.current_stream(st.device), st.comm_stream
        pending = [len(b[2]) for b in st.bucket_bounds]
        nxt = [0]

        def launch_ready():
            while nxt[0] < len(pending) and pending[nxt[0]] == 0:
                lo, hi, _ = st.bucket_bounds[nxt[0]]
                comm.wait_stream(main)          # inside a capture this forks the graph onto the second stream
                with torch.cuda.stream(comm):
                    dist.all_reduce(st.flat_grad[lo:hi])
                nxt[0] += 1

        handles = []
        for k, (_, _, members) in enumerate(st.bucket_bounds):
            for p in members:
                def hook(_p, k=k):
                    pending[k] -= 1
                    launch_ready()
                handles.append(p.register_post_accumulate_grad_hook(hook))
        try:
            loss.backward()
        finally:
            for h in handles:
                h.remove()
        # parameters that took no part in this loss never fire their hook: whatever is left goes now, in order
        for k in range(len(pending)):
            pending[k] = 0
        launch_ready()
        main.wait_stream(comm)                  # join: the graph's tail depends on every collective
        return loss.detach()

    def __call__(self, x, y):
        self.x.copy_(x)
        self.y.copy_(y)
        self.graph.replay()
        _ops.launch_count += self.launches
        return self.loss


def _mark(state: TrainState, name: str):
    """Record a CUDA event under ``name`` when the state collects timings (bench runs); no cost otherwise."""
    if state.timing is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(state.device))
        state.timing.setdefault(name, []).append(ev)


def accumulate_graphed(state: TrainState, micro_batches, autocast_dtype=torch.bfloat16):
    """Forward + backward of every micro-batch (graph replays) and the gradient all-reduce; afterwards
    ``state.flat_grad`` holds the mean gradient over all micro-batches and ranks.  Returns this rank's mean loss."""
    n = len(micro_batches)
    world = _world()
    total = None
    for i, (x, y) in enumerate(micro_batches):
        in_graph = world > 1 and state.overlap and i == n - 1
        key = (x.shape[0], n, autocast_dtype, in_graph)
        step = state.graphed.get(key)
        if step is None:
            step = state.graphed[key] = GraphedMicroStep(state, x.shape[0], n, autocast_dtype, reduce_in_graph=in_graph)
        loss = step(x, y) * float(world)        # the graph divides by n_micro * world; report the mean over this rank
        total = loss if total is None else total + loss
    _mark(state, "backward_done")
    if world > 1 and not state.overlap:
        dist.all_reduce(state.flat_grad)        # one collective for all gradients (already scaled by 1 / world)
    _mark(state, "allreduce_done")
    return total


def _train_step_graphed(state: TrainState, micro_batches, max_grad_norm, ema_decay, autocast_dtype):
    _mark(state, "step_start")
    total = accumulate_graphed(state, micro_batches, autocast_dtype)
    flat = state.flat_grad
    if state.flat_opt is not None:
        # one reduction for the norm, then clip + AdamW + EMA + zeroing of the gradients in one pass over the buffers
        state.flat_opt.step_tail(flat, state.flat_param, state.flat_ema, flat.norm(2), max_grad_norm=max_grad_norm,
                                 ema_decay=ema_decay)
        for b_ema, b in zip(state.ema.buffers(), state.model.buffers()):
            b_ema.copy_(b)
    else:
        # clip_grad_norm_ on the flat buffer without a host sync and without a pass of its own: the coefficient
        # min(1, max_norm / (norm + 1e-6)) goes to the fused AdamW kernel, which divides every gradient by grad_scale
        coef = torch.clamp(max_grad_norm / (flat.norm(2) + 1e-6), max=1.0)
        state.opt.grad_scale.copy_(1.0 / coef)
        state.opt.step()
        flat.zero_()                            # p.grad stay views of the buffer
        update_ema(state.ema, state.model, ema_decay)
    _mark(state, "tail_done")
    state.steps_done += 1
    _ops.poll_device_status(state.device)       # a kernel that gave up a wait is reported one step later, no sync
    return total


def synthetic_batch(state: TrainState, batch: int, generator=None):
    """Latents iid N(0,1) of shape (batch, 4, S, S), labels uniform over 1000 classes."""
    x = torch.randn(batch, 4, state.input_size, state.input_size, device=state.device, generator=generator)
    y = torch.randint(0, 1000, (batch,), device=state.device, generator=generator)
    return x, y


def train_step(state: TrainState, micro_batches, *, max_grad_norm: float = 1.0, ema_decay: float = 0.9999,
               autocast_dtype=torch.bfloat16):
    """micro_batches: list of (x, y) for THIS rank; gradients are averaged over all of them and,
    through DDP, over ranks.  Returns the mean loss (a device tensor; no host sync)."""
    if state.graphs:
        return _train_step_graphed(state, micro_batches, max_grad_norm, ema_decay, autocast_dtype)
    total = accumulate_eager(state, micro_batches, autocast_dtype)
    torch.nn.utils.clip_grad_norm_(state.model.parameters(), max_grad_norm)
    state.opt.step()
    state.opt.zero_grad(set_to_none=True)
    update_ema(state.ema, state.model, ema_decay)
    state.steps_done += 1
    if state.device.type == "cuda":
        _ops.poll_device_status(state.device)
    return total


def accumulate_eager(state: TrainState, micro_batches, autocast_dtype=torch.bfloat16):
    """The same without graphs: eager launches, gradients in ``p.grad``, averaged over ranks by the DDP wrapper during
    the last micro-batch's backward.  Returns this rank's mean loss."""
    n = len(micro_batches)
    total = None
    for i, (x, y) in enumerate(micro_batches):
        last = i == n - 1
        sync_ctx = contextlib.nullcontext() if (last or state.wrapped is state.model) else state.wrapped.no_sync()
        with sync_ctx:
            with torch.autocast(device_type=state.device.type, dtype=autocast_dtype):
                loss, _ = state.loss_fn(state.wrapped, state.model, x, y)
            loss = loss.mean() / n
            loss.backward()
        total = loss.detach() if total is None else total + loss.detach()
    return total
