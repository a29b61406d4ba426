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
of it) that the captured backward accumulates into; across ranks it is averaged by a single NCCL
all-reduce of that buffer after the last micro-batch, in place of the DDP wrapper.
"""

from __future__ import annotations

import contextlib
import copy
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

from .. import ops as _ops
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
    graphed: dict | None = None             # graphs: (batch, n_micro) -> GraphedMicroStep


def build_train_state(device, *, name: str = "DMFT-XL/2", input_size: int = 32, dmf_depth: int = 20,
                      attn_func: str = "fa3", qk_norm: bool = False, seed: int = 0, lr: float = 1e-4,
                      zero_init: bool = True, graphs: bool = False) -> TrainState:
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
    return state


class GraphedMicroStep:
    """loss(x, y) / n_micro and its backward (accumulating into the existing ``p.grad``), captured in a CUDA graph."""

    def __init__(self, state: TrainState, batch: int, n_micro: int, autocast_dtype):
        dev, S = state.device, state.input_size
        self.x = torch.zeros(batch, 4, S, S, device=dev)
        self.y = torch.zeros(batch, dtype=torch.long, device=dev)
        self.n_micro, self.autocast_dtype, self.state = n_micro, autocast_dtype, state
        keep = state.flat_grad.clone()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):        # warm-up outside the capture: lazy initialisations, allocator
            for _ in range(3):
                self._fwd_bwd()
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        launches0 = _ops.launch_count
        with torch.cuda.graph(self.graph):
            self.loss = self._fwd_bwd()
        self.launches = _ops.launch_count - launches0   # kernels of this package inside the graph
        state.flat_grad.copy_(keep)          # the warm-up passes accumulated; the capture itself ran nothing

    def _fwd_bwd(self):
        st = self.state
        with torch.autocast(device_type="cuda", dtype=self.autocast_dtype):
            loss, _ = st.loss_fn(st.model, st.model, self.x, self.y)
        loss = loss.mean() / self.n_micro
        loss.backward()
        return loss.detach()

    def __call__(self, x, y):
        self.x.copy_(x)
        self.y.copy_(y)
        self.graph.replay()
        _ops.launch_count += self.launches
        return self.loss


def _train_step_graphed(state: TrainState, micro_batches, max_grad_norm, ema_decay, autocast_dtype):
    n = len(micro_batches)
    total = None
    for x, y in micro_batches:
        key = (x.shape[0], n, autocast_dtype)
        step = state.graphed.get(key)
        if step is None:
            step = state.graphed[key] = GraphedMicroStep(state, x.shape[0], n, autocast_dtype)
        loss = step(x, y)
        total = loss.clone() if total is None else total + loss
    flat = state.flat_grad
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(flat)                                  # one collective for all gradients
        flat.div_(dist.get_world_size())
    # clip_grad_norm_ on the flat buffer: scale by min(1, max_norm / (norm + 1e-6)), no host sync
    flat.mul_(torch.clamp(max_grad_norm / (flat.norm(2) + 1e-6), max=1.0))
    state.opt.step()
    flat.zero_()                                               # p.grad stay views of the buffer
    update_ema(state.ema, state.model, ema_decay)
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
    torch.nn.utils.clip_grad_norm_(state.model.parameters(), max_grad_norm)
    state.opt.step()
    state.opt.zero_grad(set_to_none=True)
    update_ema(state.ema, state.model, ema_decay)
    return total
