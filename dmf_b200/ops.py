"""Tensor-level wrappers of the C ABI and their registration as torch custom ops.

Three ops, named after the entry points they call:

    dmf_b200::attn_fwd_dual(q, k, v, tq, tk, tv, scale) -> (o, to, lse)
    dmf_b200::attn_fwd(q, k, v, scale)                  -> (o, lse)
    dmf_b200::attn_bwd(dout, q, k, v, o, lse, scale)    -> (dq, dk, dv)

All tensors are (B, L, H, D); lse is (B, H, Lq) fp32.  The ops own no weights and
allocate only their outputs (and the backward workspace) through torch's caching
allocator; the kernels run on torch's current CUDA stream.  Fake (meta)
implementations let torch.compile trace through them, as the reference's
register_fake does (models/flash_attention_2_jvp.py:64-88, 143-174).
"""

from __future__ import annotations

import ctypes as C
import os
from typing import Tuple

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.BF16, torch.float16: _lib.FP16}

# Kernel launches made through this module since import (a backward call launches two kernels).
launch_count = 0

# One int32 per device that kernels write to when a device-side wait runs out.
_status_words: dict[int, torch.Tensor] = {}
# DMF_ATTN_CHECK=1 reads the status word back after every call (synchronises; for tests and debugging).
_CHECK_EVERY_CALL = os.environ.get("DMF_ATTN_CHECK", "0") == "1"


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[idx] = w
    return w


def check_device_status(device=None) -> None:
    """Raise if any kernel launched so far on ``device`` gave up a wait.  Synchronises."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _status_word(device)
    raw = C.c_int32(0)
    st = _lib.load().dmf_attn_check_status_word(w.data_ptr(), torch.cuda.current_stream(device).cuda_stream,
                                                C.byref(raw))
    if st != 0:
        w.zero_()
        raise _lib.DmfAttnError(st, f"status word = {raw.value} (role*100 + barrier index)")


# device index -> [pinned host copy of the status word, event recorded behind the copy, copy in flight?]
_status_polls: dict[int, list] = {}


def poll_device_status(device=None) -> None:
    """check_device_status without a synchronisation, one call late: every call looks at the value the PREVIOUS
    call read back (if that copy has finished) and queues a new asynchronous copy of the status word to pinned host
    memory on the current stream.  Meant for once per optimisation step or sampler call: a kernel that gave up a
    wait is reported at the next step instead of its output being used silently from then on."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_word(device)
    slot = _status_polls.get(idx)
    if slot is None:
        slot = _status_polls[idx] = [torch.zeros(1, dtype=torch.int32).pin_memory(), torch.cuda.Event(), False]
    host, ev, pending = slot
    if pending:
        if not ev.query():
            return                      # the previous read-back is still queued behind running work
        slot[2] = False
        raw = int(host[0])
        if raw != 0:
            w.zero_()
            raise _lib.DmfAttnError(12, f"status word = {raw} (role*100 + barrier index)")
    host.copy_(w, non_blocking=True)
    ev.record(torch.cuda.current_stream(device))
    slot[2] = True


def _prep(x: torch.Tensor) -> torch.Tensor:
    """Make a tensor consumable without changing its values: unit stride on D,
    16-byte aligned base and strides (maybe_contiguous in the reference,
    models/flash_attention_2_jvp.py:24-25, is the first of these)."""
    if x.stride(-1) != 1 or x.data_ptr() % 16 != 0 or any((s * x.element_size()) % 16 for s in x.stride()[:-1]):
        return x.contiguous()
    return x


def _t4(x: torch.Tensor) -> _lib.Tensor4:
    return _lib.Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2))


def _check_inputs(*tensors: torch.Tensor) -> None:
    ref = tensors[0]
    if not ref.is_cuda:
        raise RuntimeError("dmf_b200 attention runs on CUDA (sm_100a) only; there is no CPU path")
    if ref.dtype not in _DTYPES:
        raise TypeError(f"dmf_b200 attention supports bf16 and fp16, got {ref.dtype}")
    for t in tensors:
        if t.dim() != 4:
            raise ValueError("expected (B, L, H, D) tensors")
        if t.dtype != ref.dtype or t.device != ref.device:
            raise ValueError("all tensors must share dtype and device")


def _fill_common(a, q, k, scale, device):
    B, Lq, H, D = q.shape
    a.batch, a.seqlen_q, a.seqlen_kv, a.heads, a.head_dim = B, Lq, k.shape[1], H, D
    a.dtype = _DTYPES[q.dtype]
    a.softmax_scale = float(scale)
    a.status_word = _status_word(device).data_ptr()
    a.stream = torch.cuda.current_stream(device).cuda_stream


def fwd_dual_raw(q, k, v, tq, tk, tv, scale: float):
    _check_inputs(q, k, v, tq, tk, tv)
    if not (q.shape == tq.shape and k.shape == tk.shape and v.shape == tv.shape and k.shape == v.shape
            and q.shape[0] == k.shape[0] and q.shape[2:] == k.shape[2:]):
        raise ValueError("shape mismatch between q/k/v and their tangents")
    q, k, v, tq, tk, tv = (_prep(x) for x in (q, k, v, tq, tk, tv))
    B, Lq, H, D = q.shape
    with torch.cuda.device(q.device):
        o = torch.empty((B, Lq, H, D), dtype=q.dtype, device=q.device)
        to = torch.empty((B, Lq, H, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        a = _lib.FwdArgs()
        _fill_common(a, q, k, scale, q.device)
        a.q, a.k, a.v, a.tq, a.tk, a.tv, a.o, a.to = (_t4(x) for x in (q, k, v, tq, tk, tv, o, to))
        a.lse = lse.data_ptr()
        _lib.check(_lib.load().dmf_attn_fwd_dual(C.byref(a)))
        global launch_count
        launch_count += 1
        if _CHECK_EVERY_CALL:
            check_device_status(q.device)
    return o, to, lse


def fwd_raw(q, k, v, scale: float):
    _check_inputs(q, k, v)
    if not (k.shape == v.shape and q.shape[0] == k.shape[0] and q.shape[2:] == k.shape[2:]):
        raise ValueError("shape mismatch between q, k and v")
    q, k, v = (_prep(x) for x in (q, k, v))
    B, Lq, H, D = q.shape
    with torch.cuda.device(q.device):
        o = torch.empty((B, Lq, H, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        a = _lib.FwdArgs()
        _fill_common(a, q, k, scale, q.device)
        a.q, a.k, a.v, a.o = (_t4(x) for x in (q, k, v, o))
        a.lse = lse.data_ptr()
        _lib.check(_lib.load().dmf_attn_fwd(C.byref(a)))
        global launch_count
        launch_count += 1
        if _CHECK_EVERY_CALL:
            check_device_status(q.device)
    return o, lse


def bwd_raw(dout, q, k, v, o, lse, scale: float, packed_out: bool = False):
    """dq, dk, dv; with ``packed_out`` the three are the [:, :, i] views of one (B, L, 3, H, D) buffer, which is
    returned instead (self-attention: q, k, v of equal shape)."""
    _check_inputs(dout, q, k, v, o)
    dout, q, k, v, o = (_prep(x) for x in (dout, q, k, v, o))
    lse = lse.contiguous()
    B, Lq, H, D = q.shape
    Lk = k.shape[1]
    lib = _lib.load()
    with torch.cuda.device(q.device):
        if packed_out:
            if not (q.shape == k.shape == v.shape):
                raise ValueError("a packed gradient needs q, k, v of one shape")
            dqkv = torch.empty((B, Lq, 3, H, D), dtype=q.dtype, device=q.device)
            dq, dk, dv = dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]
        else:
            dq, dk, dv = torch.empty_like(q, memory_format=torch.contiguous_format), \
                torch.empty_like(k, memory_format=torch.contiguous_format), \
                torch.empty_like(v, memory_format=torch.contiguous_format)
        ws_bytes = lib.dmf_attn_bwd_workspace_bytes(B, Lq, Lk, H, D)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=q.device)
        a = _lib.BwdArgs()
        _fill_common(a, q, k, scale, q.device)
        a.dout, a.q, a.k, a.v, a.o, a.dq, a.dk, a.dv = (_t4(x) for x in (dout, q, k, v, o, dq, dk, dv))
        a.lse = lse.data_ptr()
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws_bytes
        _lib.check(lib.dmf_attn_bwd(C.byref(a)))
        global launch_count
        launch_count += 2
        if _CHECK_EVERY_CALL:
            check_device_status(q.device)
    return dqkv if packed_out else (dq, dk, dv)


# ---- torch custom ops --------------------------------------------------------

@torch.library.custom_op("dmf_b200::attn_fwd_dual", mutates_args=(), device_types="cuda")
def attn_fwd_dual(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tq: torch.Tensor, tk: torch.Tensor,
                  tv: torch.Tensor, softmax_scale: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return fwd_dual_raw(q, k, v, tq, tk, tv, softmax_scale)


@torch.library.register_fake("dmf_b200::attn_fwd_dual")
def _attn_fwd_dual_fake(q, k, v, tq, tk, tv, softmax_scale):
    B, Lq, H, D = q.shape
    o = q.new_empty((B, Lq, H, D))
    return o, q.new_empty((B, Lq, H, D)), q.new_empty((B, H, Lq), dtype=torch.float32)


@torch.library.custom_op("dmf_b200::attn_fwd", mutates_args=(), device_types="cuda")
def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
             softmax_scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    return fwd_raw(q, k, v, softmax_scale)


@torch.library.register_fake("dmf_b200::attn_fwd")
def _attn_fwd_fake(q, k, v, softmax_scale):
    B, Lq, H, D = q.shape
    return q.new_empty((B, Lq, H, D)), q.new_empty((B, H, Lq), dtype=torch.float32)


@torch.library.custom_op("dmf_b200::attn_bwd", mutates_args=(), device_types="cuda")
def attn_bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor,
             lse: torch.Tensor, softmax_scale: float) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return bwd_raw(dout, q, k, v, o, lse, softmax_scale)


@torch.library.register_fake("dmf_b200::attn_bwd")
def _attn_bwd_fake(dout, q, k, v, o, lse, softmax_scale):
    return (q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape))


@torch.library.custom_op("dmf_b200::attn_bwd_qkvpacked", mutates_args=(), device_types="cuda")
def attn_bwd_qkvpacked(dout: torch.Tensor, qkv: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                       softmax_scale: float) -> torch.Tensor:
    return bwd_raw(dout, qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], o, lse, softmax_scale, packed_out=True)


@torch.library.register_fake("dmf_b200::attn_bwd_qkvpacked")
def _attn_bwd_qkvpacked_fake(dout, qkv, o, lse, softmax_scale):
    return qkv.new_empty(qkv.shape)


# ---- per-head RMS norm of q / k with its tangent (models/layers.py:33-42 under forward-mode AD) ----

def _rms_weight(weight: torch.Tensor, device) -> torch.Tensor:
    w = weight.detach()
    if w.dtype != torch.float32 or w.device != device or not w.is_contiguous():
        w = w.to(device=device, dtype=torch.float32).contiguous()
    return w


def rmsnorm_fwd_raw(x, tx, weight, eps: float):
    """y (and ty if tx is given) for (B, L, H, D) tensors; one kernel, every row read and written once."""
    tensors = (x,) if tx is None else (x, tx)
    _check_inputs(*tensors)
    if tx is not None and tx.shape != x.shape:
        raise ValueError("shape mismatch between x and its tangent")
    x = _prep(x)
    tx = None if tx is None else _prep(tx)
    B, L, H, D = x.shape
    with torch.cuda.device(x.device):
        w = _rms_weight(weight, x.device)
        y = torch.empty((B, L, H, D), dtype=x.dtype, device=x.device)
        ty = None if tx is None else torch.empty((B, L, H, D), dtype=x.dtype, device=x.device)
        a = _lib.RmsNormArgs()
        a.batch, a.seqlen, a.heads, a.head_dim = B, L, H, D
        a.dtype = _DTYPES[x.dtype]
        a.eps = float(eps)
        a.x, a.y = _t4(x), _t4(y)
        if tx is not None:
            a.tx, a.ty = _t4(tx), _t4(ty)
        a.weight = w.data_ptr()
        a.stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(_lib.load().dmf_rmsnorm_fwd(C.byref(a)))
        global launch_count
        launch_count += 1
    return y, ty


def rmsnorm_bwd_raw(dy, x, weight, eps: float):
    """dx (like x) and dweight (D, fp32) of y = rmsnorm(x) * weight."""
    _check_inputs(dy, x)
    dy, x = _prep(dy), _prep(x)
    B, L, H, D = x.shape
    with torch.cuda.device(x.device):
        w = _rms_weight(weight, x.device)
        dx = torch.empty((B, L, H, D), dtype=x.dtype, device=x.device)
        dw = torch.empty((D,), dtype=torch.float32, device=x.device)
        lib = _lib.load()
        nbytes = lib.dmf_rmsnorm_bwd_workspace_bytes(D)
        ws = torch.empty((nbytes,), dtype=torch.uint8, device=x.device)
        a = _lib.RmsNormBwdArgs()
        a.batch, a.seqlen, a.heads, a.head_dim = B, L, H, D
        a.dtype = _DTYPES[x.dtype]
        a.eps = float(eps)
        a.dy, a.x, a.dx = _t4(dy), _t4(x), _t4(dx)
        a.weight, a.dweight = w.data_ptr(), dw.data_ptr()
        a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
        a.stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(lib.dmf_rmsnorm_bwd(C.byref(a)))
        global launch_count
        launch_count += 2
    return dx, dw


@torch.library.custom_op("dmf_b200::rmsnorm_fwd_dual", mutates_args=(), device_types="cuda")
def rmsnorm_fwd_dual(x: torch.Tensor, tx: torch.Tensor, weight: torch.Tensor,
                     eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    return rmsnorm_fwd_raw(x, tx, weight, eps)


@torch.library.register_fake("dmf_b200::rmsnorm_fwd_dual")
def _rmsnorm_fwd_dual_fake(x, tx, weight, eps):
    return x.new_empty(x.shape), x.new_empty(x.shape)


@torch.library.custom_op("dmf_b200::rmsnorm_fwd", mutates_args=(), device_types="cuda")
def rmsnorm_fwd(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rmsnorm_fwd_raw(x, None, weight, eps)[0]


@torch.library.register_fake("dmf_b200::rmsnorm_fwd")
def _rmsnorm_fwd_fake(x, weight, eps):
    return x.new_empty(x.shape)


@torch.library.custom_op("dmf_b200::rmsnorm_bwd", mutates_args=(), device_types="cuda")
def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    return rmsnorm_bwd_raw(dy, x, weight, eps)


@torch.library.register_fake("dmf_b200::rmsnorm_bwd")
def _rmsnorm_bwd_fake(dy, x, weight, eps):
    return x.new_empty(x.shape), x.new_empty((x.shape[-1],), dtype=torch.float32)
