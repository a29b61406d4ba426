"""The end of an optimisation step - gradient clipping, AdamW, EMA of the weights, zeroing of the gradients - as ONE
kernel over flat fp32 buffers (`dmf_step_tail`, include/dmf_step.h), in place of the calls train_dmf.py:331-338 makes
(`clip_grad_norm_`, fused `AdamW.step`, `zero_grad`, `update_ema`), which read and write the buffers about 16 times.
"""

from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from . import ops as _ops


class FlatAdamW:
    """AdamW state for parameters that live in one flat fp32 buffer: both moments flat, the step count on the host."""

    def __init__(self, flat_param: torch.Tensor, *, lr: float = 1e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.0):
        if flat_param.dtype != torch.float32 or not flat_param.is_cuda or not flat_param.is_contiguous():
            raise ValueError("FlatAdamW needs a contiguous fp32 CUDA buffer")
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.exp_avg = torch.zeros_like(flat_param)
        self.exp_avg_sq = torch.zeros_like(flat_param)
        self.step_count = 0

    def step_tail(self, flat_grad: torch.Tensor, flat_param: torch.Tensor, flat_ema, grad_norm, *,
                  max_grad_norm: float = 1.0, ema_decay: float = 0.9999) -> None:
        """One optimisation step.  ``grad_norm``: 0-dim fp32 device tensor with the 2-norm of ``flat_grad`` (or None for
        no clipping); ``flat_ema``: the EMA buffer or None.  ``flat_grad`` is zero afterwards."""
        self.step_count += 1
        t = self.step_count
        a = _lib.StepTailArgs()
        a.count = flat_param.numel()
        a.grad, a.param = flat_grad.data_ptr(), flat_param.data_ptr()
        a.exp_avg, a.exp_avg_sq = self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr()
        a.ema = None if flat_ema is None else flat_ema.data_ptr()
        a.grad_norm = None if grad_norm is None else grad_norm.data_ptr()
        a.max_grad_norm = float(max_grad_norm)
        a.lr, a.beta1, a.beta2, a.eps = float(self.lr), float(self.betas[0]), float(self.betas[1]), float(self.eps)
        a.weight_decay = float(self.weight_decay)
        # bias corrections in double on the host, as torch's fused kernel forms them from its step counter
        a.step_size = float(self.lr / (1.0 - self.betas[0] ** t))
        a.bias_correction2_sqrt = float(math.sqrt(1.0 - self.betas[1] ** t))
        a.ema_decay = float(ema_decay)
        with torch.cuda.device(flat_param.device):
            a.stream = torch.cuda.current_stream(flat_param.device).cuda_stream
            _lib.check(_lib.load().dmf_step_tail(C.byref(a)))
        _ops.launch_count += 1
