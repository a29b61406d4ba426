"""Measurement harness around the attention kernels: the callers of the hot path.

These modules restate, with the reference's parameter names and step semantics,
the pieces of kyungmnlee/dmf that reach ``flash_attn_func`` - the DMFT model
(models/dmft.py), the DMF loss that takes ``torch.func.jvp`` through it
(loss.py:142-181), the few-step Euler sampler (samplers.py:69-100) and the
optimisation step of train_dmf.py:320-338 - so that the whole-model configurations
(DMFT-XL/2 training step, 4-step sampling) can be measured without the reference
tree, ``timm``, ``accelerate`` or ``diffusers``.  They are callers, not kernels:
all attention work goes through ``dmf_b200.flash_attn_func``.
"""
