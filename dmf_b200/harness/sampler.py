"""Few-step Euler sampler of the mean-velocity model (samplers.py:60-100 of the reference):
float64 state, shifted time grid, one model call per step with (t_cur, r = t_next).

``GraphedSampler`` captures the whole loop for one (batch, latent shape, step count) in a CUDA graph and replays it:
the time grid is known on the host, so nothing in the loop depends on device results.
"""

from __future__ import annotations

import torch

from .. import ops as _ops


def get_tsteps(num_steps: int, t_start: float = 1.0, t_end: float = 0.0, shift: float = 1.0):
    t = torch.linspace(t_start, t_end, num_steps + 1, dtype=torch.float64)
    return t if shift == 1.0 else shift * t / (1 + (shift - 1.0) * t)


@torch.no_grad()
def euler_sampler(model, latents, y, num_steps: int = 4, cfg_scale: float = 1.0, g_min: float = 0.0,
                  g_max: float = 1.0, shift: float = 1.0, null_label: int = 1000):
    dtype, device = latents.dtype, latents.device
    y_null = torch.full_like(y, null_label) if cfg_scale > 1.0 else None
    t_steps = get_tsteps(num_steps, shift=shift)
    x = latents.to(torch.float64)
    for t_cur, t_nxt in zip(t_steps[:-1], t_steps[1:]):
        guided = cfg_scale > 1.0 and g_min <= t_cur <= g_max
        inp = torch.cat([x, x], dim=0) if guided else x
        lab = torch.cat([y, y_null], dim=0) if guided else y
        inp = inp.to(dtype)
        t_in = torch.full((inp.shape[0],), float(t_cur), device=device, dtype=dtype)
        r_in = torch.full((inp.shape[0],), float(t_nxt), device=device, dtype=dtype)
        d = model(inp, t_in, r_in, lab).to(torch.float64)
        if guided:
            d_c, d_u = d.chunk(2)
            d = d_u + cfg_scale * (d_c - d_u)
        x = x + float(t_nxt - t_cur) * d   # a host float64: no host tensor enters the device arithmetic
    if x.is_cuda and not torch.cuda.is_current_stream_capturing():
        _ops.poll_device_status(x.device)  # a kernel that gave up a wait is reported at the next call, no sync
    return x


class GraphedSampler:
    """euler_sampler for fixed shapes, replayed as one CUDA graph.  ``sampler(z, y)`` copies the inputs into the
    graph's static buffers, replays, and returns the static float64 output (overwritten by the next call)."""

    def __init__(self, model, batch: int, latent_shape=(4, 64, 64), dtype=torch.bfloat16, device="cuda", **kwargs):
        dev = torch.device(device)
        self.z = torch.zeros(batch, *latent_shape, device=dev, dtype=dtype)
        self.y = torch.zeros(batch, dtype=torch.long, device=dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):        # warm-up outside the capture: lazy initialisations, allocator
            for _ in range(2):
                euler_sampler(model, self.z, self.y, **kwargs)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        launches0 = _ops.launch_count
        with torch.cuda.graph(self.graph):
            self.out = euler_sampler(model, self.z, self.y, **kwargs)
        self.launches = _ops.launch_count - launches0   # kernels of this package inside the graph

    def __call__(self, z, y):
        self.z.copy_(z, non_blocking=True)
        self.y.copy_(y, non_blocking=True)
        self.graph.replay()
        _ops.launch_count += self.launches
        _ops.poll_device_status(self.z.device)
        return self.out
