"""Few-step Euler sampler of the mean-velocity model (samplers.py:60-100 of the reference):
float64 state, shifted time grid, one model call per step with (t_cur, r = t_next)."""

from __future__ import annotations

import torch


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
        x = x + (t_nxt - t_cur) * d
    return x
