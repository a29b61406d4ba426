"""Generate the golden vectors under tests/golden/ from the reference itself.

Run once, in a container that holds the reference source tree:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference /path/to/dmf

It imports the reference's own Python code (nothing is copied), runs it on CPU
with seeded inputs and stores the OUTPUTS as .npz.  Inputs are not stored: they
are re-drawn from the same seeded CPU generator by
``oracle.attn_jvp_oracle.make_inputs``; a float64 checksum of every input is
stored so that a change of the generator is detected instead of silently
comparing different data.

Witnesses stored per case:
  base_o, base_do   torch.func.jvp(partial(attn_op, op="base"))   models/layers.py:100-114
  raw_vs_base_*     max|raw_attn_func - 'base'| under the same jvp   models/flash_attention_2_jvp.py:322-336
  raw_dq/dk/dv      autograd of raw_attn_func with a seeded dout   models/flash_attention_2_jvp.py:361-369
  tri_o, tri_do,    the reference Triton kernels _attn_fwd_dual / _attn_fwd_dual_split run by
  tri_lse           the Triton CPU interpreter in fp32              models/triton_utils.py:258-500
  (qk-norm case)    q, k and tangents pass through the reference RMSNorm first, models/layers.py:33-42
"""

import argparse
import os
import sys
import types
from functools import partial
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

CASES = {
    # name: (B, L, H, D, tangent_scale, qk_norm, seed)
    "d64_l256": (1, 256, 1, 64, 1.0, False, 0),
    "d72_l256": (1, 256, 1, 72, 0.1, False, 1),
    "d72_l256_qknorm": (1, 256, 1, 72, 0.1, True, 2),
    "d96_l128": (1, 128, 1, 96, 0.5, False, 3),
    "d128_l128": (1, 128, 1, 128, 0.5, False, 4),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference source tree")
    args = ap.parse_args()
    os.environ.setdefault("TRITON_INTERPRET", "1")

    sys.path.insert(0, args.reference)
    for name in ("flash_attn_3", "flash_attn_3._C"):  # Hopper-only module, absent here
        sys.modules.setdefault(name, types.ModuleType(name))
    from models.layers import attn_op, RMSNorm
    from models.flash_attention_2_jvp import raw_attn_func
    from models.triton_utils import _attn_fwd_dual, _attn_fwd_dual_split, split_head_dim

    from oracle.attn_jvp_oracle import make_inputs

    for name, (B, L, H, D, ts, qkn, seed) in CASES.items():
        # un-normalised draws; the reference RMSNorm is applied below for the qk-norm case
        q, k, v, tq, tk, tv, dout = make_inputs(B, L, H, D, seed=seed, tangent_scale=ts,
                                                qk_norm=False, n_extra=1)
        out = {}
        if qkn:
            norm = RMSNorm(D)
            with torch.no_grad():
                q, tq = torch.func.jvp(norm, (q,), (tq,))
                k, tk = torch.func.jvp(norm, (k,), (tk,))
            out["normed_q"], out["normed_tq"] = q.numpy(), tq.numpy()
            out["normed_k"], out["normed_tk"] = k.numpy(), tk.numpy()
        out["checksum"] = np.array([float(x.double().sum()) for x in (q, k, v, tq, tk, tv, dout)])

        o, do = torch.func.jvp(partial(attn_op, op="base"), (q, k, v), (tq, tk, tv))
        out["base_o"], out["base_do"] = o.numpy(), do.numpy()
        o2, do2 = torch.func.jvp(raw_attn_func, (q, k, v), (tq, tk, tv))
        # raw_attn_func differs from 'base' only in where the scale is applied; store the gap, not the copy
        out["raw_vs_base_maxabs"] = np.array([float((o2 - o).abs().max()), float((do2 - do).abs().max())])

        qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
        raw_attn_func(qg, kg, vg).backward(dout)
        out["raw_dq"], out["raw_dk"], out["raw_dv"] = qg.grad.numpy(), kg.grad.numpy(), vg.grad.numpy()

        # the reference Triton kernels under the CPU interpreter (fp32), launched exactly as
        # FlashAttnFunc.forward does (flash_attention_2_jvp.py:186-230)
        o_t, to_t = torch.empty_like(q), torch.empty_like(tq)
        m_t = torch.empty((B, H, L), dtype=torch.float32)
        tile, tail = split_head_dim(D)
        strides = []
        for x in (q, k, v, tq, tk, tv, o_t, to_t):
            strides += [x.stride(0), x.stride(1), x.stride(2), x.stride(3)]
        grid = (L // 128, B * H, 1)
        if tail > 0:
            _attn_fwd_dual_split[grid](q, k, v, tq, tk, tv, m_t, o_t, to_t, D ** -0.5, *strides,
                                       H, L, L, D, tile, tail, block_q=128, block_kv=128)
        else:
            _attn_fwd_dual[grid](q, k, v, tq, tk, tv, m_t, o_t, to_t, D ** -0.5, *strides,
                                 H, L, L, D, block_q=128, block_kv=128)
        out["tri_o"], out["tri_do"], out["tri_lse"] = o_t.numpy(), to_t.numpy(), m_t.numpy()

        path = HERE / f"{name}.npz"
        np.savez(path, **out)
        print(f"{name}: wrote {path.name} ({path.stat().st_size / 1024:.0f} KiB); "
              f"|tri_o - base_o|max = {np.abs(out['tri_o'] - out['base_o']).max():.2e}, "
              f"|tri_do - base_do|max = {np.abs(out['tri_do'] - out['base_do']).max():.2e}")


if __name__ == "__main__":
    main()
