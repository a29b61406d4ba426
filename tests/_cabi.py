"""Test-side helper: call the C ABI directly (ctypes) on torch CUDA tensors, with
outputs poison-filled so that any row a kernel fails to write shows up as NaN."""

import ctypes as C

import torch

from dmf_b200 import _lib

_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.FP16}


def t4(x):
    return _lib.Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2))


def status_word(device):
    return torch.zeros(1, dtype=torch.int32, device=device)


def fwd(q, k, v, tq=None, tk=None, tv=None, scale=None, expect=0, packed_out=False):
    """dmf_attn_fwd_dual if tangents are given, else dmf_attn_fwd.  Returns (o, to, lse, status).
    packed_out: o and to are the two strided halves of one (B, L, 2, H, D) buffer."""
    dual = tq is not None
    B, Lq, H, D = q.shape
    dev = q.device
    nan = float("nan")
    if packed_out:
        both = torch.full((B, Lq, 2, H, D), nan, dtype=q.dtype, device=dev)
        o, to = both[:, :, 0], (both[:, :, 1] if dual else None)
    else:
        o = torch.full((B, Lq, H, D), nan, dtype=q.dtype, device=dev)
        to = torch.full((B, Lq, H, D), nan, dtype=q.dtype, device=dev) if dual else None
    lse = torch.full((B, H, Lq), nan, dtype=torch.float32, device=dev)
    sw = status_word(dev)
    a = _lib.FwdArgs()
    a.batch, a.seqlen_q, a.seqlen_kv, a.heads, a.head_dim = B, Lq, k.shape[1], H, D
    a.dtype = _DT[q.dtype]
    a.softmax_scale = float(D ** -0.5 if scale is None else scale)
    a.q, a.k, a.v, a.o = t4(q), t4(k), t4(v), t4(o)
    if dual:
        a.tq, a.tk, a.tv, a.to = t4(tq), t4(tk), t4(tv), t4(to)
    a.lse = lse.data_ptr()
    a.status_word = sw.data_ptr()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    lib = _lib.load()
    st = (lib.dmf_attn_fwd_dual if dual else lib.dmf_attn_fwd)(C.byref(a))
    assert st == expect, f"status {st}: {lib.dmf_attn_status_string(st).decode()}"
    if st == 0:
        raw = C.c_int32(0)
        st2 = lib.dmf_attn_check_status_word(sw.data_ptr(), a.stream, C.byref(raw))
        assert st2 == 0, f"device-side wait gave up: status word {raw.value}"
    return o, to, lse, st


def bwd(dout, q, k, v, o, lse, scale=None, expect=0, packed_out=False, min_workspace=False):
    """dmf_attn_bwd.  Returns (dq, dk, dv, status).
    packed_out (self-attention shapes only): dq, dk, dv are strided views of one (B, L, 3, H, D) buffer.
    min_workspace: pass only the two fp32 rows per query every kernel needs (8 * B * H * Lq bytes) instead of
    what dmf_attn_bwd_workspace_bytes reports; the long-sequence one-pass kernel, which wants an fp32 dQ
    accumulator behind them, then leaves the call to the two-launch kernels."""
    B, Lq, H, D = q.shape
    dev = q.device
    nan = float("nan")
    if packed_out:
        assert q.shape == k.shape
        grads = torch.full((B, Lq, 3, H, D), nan, dtype=q.dtype, device=dev)
        dq, dk, dv = grads[:, :, 0], grads[:, :, 1], grads[:, :, 2]
    else:
        dq = torch.full(q.shape, nan, dtype=q.dtype, device=dev)
        dk = torch.full(k.shape, nan, dtype=q.dtype, device=dev)
        dv = torch.full(v.shape, nan, dtype=q.dtype, device=dev)
    lib = _lib.load()
    nbytes = lib.dmf_attn_bwd_workspace_bytes(B, Lq, k.shape[1], H, D)
    if min_workspace:
        assert nbytes >= 8 * B * H * Lq
        nbytes = 8 * B * H * Lq
    ws = torch.full((max(nbytes, 16),), 0xFF, dtype=torch.uint8, device=dev)  # garbage on purpose
    sw = status_word(dev)
    a = _lib.BwdArgs()
    a.batch, a.seqlen_q, a.seqlen_kv, a.heads, a.head_dim = B, Lq, k.shape[1], H, D
    a.dtype = _DT[q.dtype]
    a.softmax_scale = float(D ** -0.5 if scale is None else scale)
    a.dout, a.q, a.k, a.v, a.o = t4(dout), t4(q), t4(k), t4(v), t4(o)
    a.dq, a.dk, a.dv = t4(dq), t4(dk), t4(dv)
    a.lse = lse.data_ptr()
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    a.status_word = sw.data_ptr()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    st = lib.dmf_attn_bwd(C.byref(a))
    assert st == expect, f"status {st}: {lib.dmf_attn_status_string(st).decode()}"
    if st == 0:
        raw = C.c_int32(0)
        st2 = lib.dmf_attn_check_status_word(sw.data_ptr(), a.stream, C.byref(raw))
        assert st2 == 0, f"device-side wait gave up: status word {raw.value}"
    return dq, dk, dv, st


def fwd_dual_f32out(q, k, v, tq, tk, tv, scale=None, expect=0):
    """dmf_attn_fwd_dual_f32out: o and to as fp32 tensors (the accumulators before the 16-bit rounding).
    Returns (o, to, lse, status)."""
    B, Lq, H, D = q.shape
    dev = q.device
    nan = float("nan")
    o = torch.full((B, Lq, H, D), nan, dtype=torch.float32, device=dev)
    to = torch.full((B, Lq, H, D), nan, dtype=torch.float32, device=dev)
    lse = torch.full((B, H, Lq), nan, dtype=torch.float32, device=dev)
    sw = status_word(dev)
    a = _lib.FwdArgs()
    a.batch, a.seqlen_q, a.seqlen_kv, a.heads, a.head_dim = B, Lq, k.shape[1], H, D
    a.dtype = _DT[q.dtype]
    a.softmax_scale = float(D ** -0.5 if scale is None else scale)
    a.q, a.k, a.v, a.o = t4(q), t4(k), t4(v), t4(o)
    a.tq, a.tk, a.tv, a.to = t4(tq), t4(tk), t4(tv), t4(to)
    a.lse = lse.data_ptr()
    a.status_word = sw.data_ptr()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    lib = _lib.load()
    st = lib.dmf_attn_fwd_dual_f32out(C.byref(a))
    assert st == expect, f"status {st}: {lib.dmf_attn_status_string(st).decode()}"
    if st == 0:
        raw = C.c_int32(0)
        st2 = lib.dmf_attn_check_status_word(sw.data_ptr(), a.stream, C.byref(raw))
        assert st2 == 0, f"device-side wait gave up: status word {raw.value}"
    return o, to, lse, st
