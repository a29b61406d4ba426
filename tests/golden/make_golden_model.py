"""Golden vectors for the measurement harness (dmf_b200/harness), from the reference itself.

    python tests/golden/make_golden_model.py --reference /path/to/dmf

A tiny DMFT is initialised by the harness under a fixed seed, its state dict is loaded
(strict) into the reference's own ``models.dmft.DMFT`` (``timm``'s PatchEmbed, which is not
installed here, is replaced by a two-line stand-in), and the reference computes: a forward
with log-variance, the DMF loss (``loss.DMFLoss``, which takes torch.func.jvp through the
model) and its parameter gradients, and a 4-step ``samplers.euler_sampler`` run.  Outputs
are stored; inputs and weights are re-created from the seeds by the test.
"""

import argparse
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

TINY = dict(input_size=8, patch_size=2, in_channels=4, hidden_size=64, depth=3, num_heads=2, dmf_depth=2,
            use_logvar=True, num_classes=1000)


def tiny_inputs():
    g = torch.Generator().manual_seed(123)
    x = torch.randn(4, 4, 8, 8, generator=g)
    y = torch.randint(0, 1000, (4,), generator=g)
    t = torch.rand(4, generator=g)
    r = t * torch.rand(4, generator=g)
    return x, y, t, r


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference source tree")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    for name in ("flash_attn_3", "flash_attn_3._C"):
        sys.modules.setdefault(name, types.ModuleType(name))
    # stand-in for timm.models.vision_transformer.PatchEmbed (only .proj and .num_patches are used)
    import torch.nn as nn

    class PatchEmbed(nn.Module):
        def __init__(self, img_size, patch_size, in_chans, embed_dim, bias=True):
            super().__init__()
            self.num_patches = (img_size // patch_size) ** 2
            self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=patch_size, stride=patch_size, bias=bias)

        def forward(self, x):
            return self.proj(x).flatten(2).transpose(1, 2)

    timm = types.ModuleType("timm"); timm.models = types.ModuleType("timm.models")
    vt = types.ModuleType("timm.models.vision_transformer"); vt.PatchEmbed = PatchEmbed
    sys.modules.update({"timm": timm, "timm.models": timm.models, "timm.models.vision_transformer": vt})

    from models.dmft import DMFT as RefDMFT
    from loss import DMFLoss as RefLoss
    from samplers import euler_sampler as ref_euler

    from dmf_b200.harness.model import DMFT

    out = {}
    for qk_norm in (False, True):
        tag = "qkn" if qk_norm else "plain"
        torch.manual_seed(7)
        mine = DMFT(**TINY, attn_func="base", qk_norm=qk_norm)
        mine.initialize_weights(zero_init=False)
        ref = RefDMFT(**TINY, attn_func="base", qk_norm=qk_norm)
        ref.load_state_dict(mine.state_dict(), strict=True)
        x, y, t, r = tiny_inputs()
        with torch.no_grad():
            o, lv = ref(x, t, r, y, return_logvar=True)
        out[f"{tag}_fwd"], out[f"{tag}_logvar"] = o.numpy(), lv.numpy()
        # DMF loss + gradients (reference defaults of train_dmf.py: P_mean -0.4, P_mean_t 0.4, P_mean_r -1.2)
        torch.manual_seed(11)
        loss_fn = RefLoss(P_mean=-0.4, P_std=1.0, P_mean_t=0.4, P_std_t=1.0, P_mean_r=-1.2, P_std_r=1.0)
        loss, ld = loss_fn(ref, ref, x, y)
        loss.mean().backward()
        out[f"{tag}_loss"] = loss.detach().numpy()
        out[f"{tag}_mf_loss"] = ld["mf_loss"].detach().numpy()
        gn = torch.stack([p.grad.norm() for p in ref.parameters() if p.grad is not None])
        out[f"{tag}_grad_norms"] = gn.numpy()
        out[f"{tag}_grad_qkv0"] = ref.blocks[0].attn.qkv.weight.grad.numpy()
        # sampler
        g = torch.Generator().manual_seed(5)
        z = torch.randn(4, 4, 8, 8, generator=g)
        out[f"{tag}_euler"] = ref_euler(ref, z, y, num_steps=4, shift=1.5).numpy()
    path = HERE / "dmft_tiny.npz"
    np.savez(path, **out)
    print("wrote", path, path.stat().st_size // 1024, "KiB")


if __name__ == "__main__":
    main()
