"""Zero-edit drop-in for the reference tree.

``models/layers.py:23-24`` imports ``flash_attn_func`` from
``models.flash_attention_2_jvp`` (as ``fa2_func``) and from
``models.flash_attention_3_jvp`` (as ``fa3_func``).  ``install()`` registers
modules under exactly those names in ``sys.modules`` *before* ``models.layers`` is
imported, so both selector strings (``attn_func='fa2'`` and ``'fa3'``) resolve to
the sm_100a kernels and neither ``layers.py`` nor ``dmft.py`` needs an edit.  It
also removes the hard dependency on ``flash_attn_2_cuda`` / ``flash_attn_3`` /
Triton that importing the original two modules has.

    import dmf_b200.dropin as dropin
    dropin.install()            # before `from models.dmft import DMFT_models`
"""

from __future__ import annotations

import sys
import types

from . import flash_attn_jvp as _impl

_NAMES = ("models.flash_attention_2_jvp", "models.flash_attention_3_jvp")


def _make_module(name: str) -> types.ModuleType:
    m = types.ModuleType(name)
    m.__doc__ = f"{name}: provided by dmf_b200 (sm_100a kernels)"
    m.flash_attn_func = _impl.flash_attn_func
    m.FlashAttnFunc = _impl.FlashAttnFunc
    m._is_dual_mode = _impl._is_dual_mode
    m.__dmf_b200__ = True
    return m


def install(force: bool = False) -> None:
    """Make the reference's two attention modules resolve to this package."""
    for name in _NAMES:
        existing = sys.modules.get(name)
        if existing is not None and not getattr(existing, "__dmf_b200__", False) and not force:
            raise RuntimeError(f"{name} is already imported from the reference; call install() before "
                               f"importing models.layers (or pass force=True and re-import it)")
        sys.modules[name] = _make_module(name)


def uninstall() -> None:
    for name in _NAMES:
        if getattr(sys.modules.get(name), "__dmf_b200__", False):
            del sys.modules[name]
