"""One optimisation step of DMF fine-tuning, as train_dmf.py:320-338 runs it:
bf16 autocast, DMF loss (flow-matching forward + JVP forward), backward, gradient
all-reduce (DDP over NCCL when world size > 1), clip to 1.0, fused AdamW, EMA 0.9999.

The reference reaches DDP through HF accelerate; here it is plain
torch.nn.parallel.DistributedDataParallel.  A global batch that does not fit one
GPU in a single pass is split into micro-batches with gradient accumulation
(``no_sync`` on all but the last), so that every world size runs the same
micro-batch shape.
"""

from __future__ import annotations

import contextlib
import copy
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

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


def build_train_state(device, *, name: str = "DMFT-XL/2", input_size: int = 32, dmf_depth: int = 20,
                      attn_func: str = "fa3", qk_norm: bool = False, seed: int = 0, lr: float = 1e-4,
                      zero_init: bool = True) -> TrainState:
    torch.manual_seed(seed)  # same initial weights on every rank
    model = build_dmft(name, input_size=input_size, dmf_depth=dmf_depth, use_logvar=True, num_classes=1000,
                       attn_func=attn_func, qk_norm=qk_norm)
    if not zero_init:
        model.initialize_weights(zero_init=False)
    model = model.to(device)
    ema = copy.deepcopy(model).requires_grad_(False)
    wrapped = model
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        wrapped = DDP(model, device_ids=[device.index] if device.type == "cuda" else None)
    opt = torch.optim.AdamW((p for p in model.parameters() if p.requires_grad), lr=lr, betas=(0.9, 0.95),
                            weight_decay=0.0, eps=1e-8, fused=(device.type == "cuda"))
    return TrainState(model, wrapped, ema, opt, DMFLoss(), device, input_size)


def synthetic_batch(state: TrainState, batch: int, generator=None):
    """Latents iid N(0,1) of shape (batch, 4, S, S), labels uniform over 1000 classes."""
    x = torch.randn(batch, 4, state.input_size, state.input_size, device=state.device, generator=generator)
    y = torch.randint(0, 1000, (batch,), device=state.device, generator=generator)
    return x, y


def train_step(state: TrainState, micro_batches, *, max_grad_norm: float = 1.0, ema_decay: float = 0.9999,
               autocast_dtype=torch.bfloat16):
    """micro_batches: list of (x, y) for THIS rank; gradients are averaged over all of them and,
    through DDP, over ranks.  Returns the mean loss (a device tensor; no host sync)."""
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
