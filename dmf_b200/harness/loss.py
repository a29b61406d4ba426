"""DMF objective (loss.py:98-181 of the reference), ``g_type='default'`` only.

Per batch: class-label dropout, three logit-normal time draws, a flow-matching term on
``model(x_t, t, t, y)`` and a MeanFlow term whose target needs d u / d t, taken with
``torch.func.jvp`` through the raw model with tangents (v, 1, 0) - this is where dual
tensors reach ``flash_attn_func``.  Only the primal u carries gradient; the target
``v + (r - t) du/dt`` is detached (loss.py:171-173).
"""

from __future__ import annotations

from functools import partial

import torch


def interpolant(x, t):
    """Linear path (loss.py:7-23): x_t = (1-t) x + t eps, v_t = eps - x."""
    eps = torch.randn_like(x)
    return (1 - t) * x + t * eps, eps - x


def log_lv_loss(x, y, lv, eps: float = 0.01):
    """loss.py:30-35."""
    dims = list(range(1, x.dim()))
    err = (x - y) ** 2
    mean_loss = err.mean(dim=dims)
    return err.sum(dim=dims), torch.log(mean_loss / lv.exp() + eps) + lv


class DMFLoss:
    def __init__(self, P_mean: float = -0.4, P_std: float = 1.0, P_mean_t: float = 0.4, P_std_t: float = 1.0,
                 P_mean_r: float = -1.2, P_std_r: float = 1.0, cfg_prob: float = 0.1, null_label: int = 1000,
                 sample_on_device: bool = True):
        self.P_mean, self.P_std = P_mean, P_std
        self.P_mean_t, self.P_std_t = P_mean_t, P_std_t
        self.P_mean_r, self.P_std_r = P_mean_r, P_std_r
        self.cfg_prob, self.null_label = cfg_prob, null_label
        # the reference draws the times on the CPU and copies them (loss.py:135-140, 149); drawing on
        # the device removes a host sync per step without changing the distribution
        self.sample_on_device = sample_on_device

    def cond_drop(self, y):
        drop = torch.rand(y.shape[0], device=y.device) < self.cfg_prob
        return torch.where(drop, self.null_label, y), drop

    def sample_times(self, bsz: int, device):
        dev = device if self.sample_on_device else "cpu"
        z = lambda: torch.randn((bsz, 1, 1, 1), device=dev)
        t_fm = torch.sigmoid(z() * self.P_std + self.P_mean)
        a = torch.sigmoid(z() * self.P_std_t + self.P_mean_t)
        b = torch.sigmoid(z() * self.P_std_r + self.P_mean_r)
        t_mf, r_mf = torch.maximum(a, b), torch.minimum(a, b)   # r <= t by swap
        return t_fm.to(device), t_mf.to(device), r_mf.to(device)

    def __call__(self, model, raw_model, x, y):
        y, _ = self.cond_drop(y)
        t_fm, t_mf, r_mf = self.sample_times(x.shape[0], x.device)
        # flow matching term (through `model`, which may be the DDP / compiled wrapper)
        x_t, v_t = interpolant(x, t_fm)
        v_fm, lv_fm = model(x_t, t_fm, t_fm, y, return_logvar=True)
        fm_mse, fm_lp = log_lv_loss(v_fm, v_t.detach(), lv_fm)
        # MeanFlow term: JVP through the raw module
        x_t, v_t = interpolant(x, t_mf)
        v_tgt = v_t.detach()
        unwrapped = raw_model.module if hasattr(raw_model, "module") else raw_model
        fn = partial(unwrapped, y=y, return_logvar=True)
        (u, lv_mf), (du_dt, _) = torch.func.jvp(fn, (x_t, t_mf, r_mf),
                                                (v_tgt, torch.ones_like(t_mf), torch.zeros_like(r_mf)))
        u_tgt = (v_tgt + (r_mf - t_mf) * du_dt).detach()
        mf_mse, mf_lp = log_lv_loss(u, u_tgt, lv_mf)
        loss = 0.5 * (fm_lp + mf_lp)
        return loss, {"fm_loss": fm_mse, "fm_p_loss": fm_lp, "mf_p_loss": mf_lp, "mf_loss": mf_mse}
