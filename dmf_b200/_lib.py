"""ctypes binding of the C ABI in include/dmf_attn.h and include/dmf_adaln.h.

The library is the only compute path of this package: if it cannot be loaded the
import fails; nothing falls back to PyTorch or to the CPU.
"""

from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

from . import build as _build

ABI_VERSION = 1
BF16, FP16 = 0, 1

STATUS_NAMES = {
    0: "OK", 1: "ERR_NULL", 2: "ERR_DTYPE", 3: "ERR_HEAD_DIM", 4: "ERR_SEQLEN", 5: "ERR_SHAPE",
    6: "ERR_STRIDE", 7: "ERR_ALIGN", 8: "ERR_DEVICE", 9: "ERR_TENSOR_MAP", 10: "ERR_LAUNCH",
    11: "ERR_WORKSPACE", 12: "ERR_TIMEOUT", 13: "ERR_TOO_LARGE",
}

# every symbol include/dmf_attn.h and include/dmf_adaln.h declare
EXPORTS = (
    "dmf_attn_abi_version", "dmf_attn_status_string", "dmf_attn_fwd_dual", "dmf_attn_fwd",
    "dmf_attn_bwd", "dmf_attn_bwd_static", "dmf_attn_bwd_workspace_bytes", "dmf_attn_check_status_word",
    "dmf_attn_validate_fwd", "dmf_attn_validate_bwd",
    "dmf_attn_fwd_dual_f32out", "dmf_attn_selftest_wait_limit", "dmf_attn_kernel_name",
    "dmf_rmsnorm_fwd", "dmf_rmsnorm_bwd", "dmf_rmsnorm_bwd_workspace_bytes",
    "dmf_ln_modulate_fwd", "dmf_ln_modulate_bwd", "dmf_adaln_bwd_workspace_bytes",
    "dmf_gate_residual_fwd", "dmf_gate_residual_bwd",
    "dmf_step_tail",
)
ADALN_BF16, ADALN_F32 = 0, 2


class Tensor4(C.Structure):
    """dmf_attn_tensor: base pointer + element strides of a (B, L, H, D) tensor."""
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_l", C.c_int64), ("stride_h", C.c_int64)]


class FwdArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("seqlen_q", C.c_int32), ("seqlen_kv", C.c_int32), ("heads", C.c_int32),
        ("head_dim", C.c_int32), ("dtype", C.c_int32), ("softmax_scale", C.c_float), ("reserved", C.c_int32),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4),
        ("tq", Tensor4), ("tk", Tensor4), ("tv", Tensor4),
        ("o", Tensor4), ("to", Tensor4),
        ("lse", C.c_void_p), ("status_word", C.c_void_p), ("stream", C.c_void_p),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("seqlen_q", C.c_int32), ("seqlen_kv", C.c_int32), ("heads", C.c_int32),
        ("head_dim", C.c_int32), ("dtype", C.c_int32), ("softmax_scale", C.c_float), ("reserved", C.c_int32),
        ("dout", Tensor4), ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4),
        ("lse", C.c_void_p),
        ("dq", Tensor4), ("dk", Tensor4), ("dv", Tensor4),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status_word", C.c_void_p), ("stream", C.c_void_p),
    ]


class RmsNormArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("seqlen", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("dtype", C.c_int32), ("eps", C.c_float),
        ("x", Tensor4), ("tx", Tensor4), ("y", Tensor4), ("ty", Tensor4),
        ("weight", C.c_void_p), ("stream", C.c_void_p),
    ]


class RmsNormBwdArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("seqlen", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("dtype", C.c_int32), ("eps", C.c_float),
        ("dy", Tensor4), ("x", Tensor4), ("dx", Tensor4),
        ("weight", C.c_void_p), ("dweight", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class Rows(C.Structure):
    """dmf_rows: a (B, L, C) tensor, element strides of B and L."""
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_l", C.c_int64)]


class Mod(C.Structure):
    """dmf_mod: a (B, C) tensor, element stride of B."""
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64)]


_ADA_HEAD = [("batch", C.c_int32), ("seqlen", C.c_int32), ("channels", C.c_int32),
             ("wide_dtype", C.c_int32), ("narrow_dtype", C.c_int32), ("mod_dtype", C.c_int32)]


class LnModulateArgs(C.Structure):
    _fields_ = _ADA_HEAD + [
        ("eps", C.c_float), ("reserved", C.c_int32),
        ("x", Rows), ("tx", Rows), ("shift", Mod), ("scale", Mod), ("tshift", Mod), ("tscale", Mod),
        ("y", Rows), ("ty", Rows), ("stream", C.c_void_p),
    ]


class LnModulateBwdArgs(C.Structure):
    _fields_ = _ADA_HEAD + [
        ("eps", C.c_float), ("reserved", C.c_int32),
        ("dy", Rows), ("x", Rows), ("scale", Mod), ("dx", Rows),
        ("dshift", C.c_void_p), ("dscale", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class GateResidualArgs(C.Structure):
    _fields_ = _ADA_HEAD + [
        ("x", Rows), ("tx", Rows), ("h", Rows), ("th", Rows), ("gate", Mod), ("tgate", Mod),
        ("out", Rows), ("tout", Rows), ("stream", C.c_void_p),
    ]


class GateResidualBwdArgs(C.Structure):
    _fields_ = _ADA_HEAD + [
        ("dout", Rows), ("h", Rows), ("gate", Mod), ("dh", Rows), ("dgate", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class StepTailArgs(C.Structure):
    """dmf_step_tail_args (include/dmf_step.h)."""
    _fields_ = [
        ("count", C.c_int64),
        ("grad", C.c_void_p), ("param", C.c_void_p), ("exp_avg", C.c_void_p), ("exp_avg_sq", C.c_void_p),
        ("ema", C.c_void_p), ("grad_norm", C.c_void_p),
        ("max_grad_norm", C.c_float), ("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
        ("eps", C.c_float), ("weight_decay", C.c_float), ("step_size", C.c_float),
        ("bias_correction2_sqrt", C.c_float), ("ema_decay", C.c_float), ("reserved", C.c_int32),
        ("stream", C.c_void_p),
    ]


class DmfAttnError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"dmf_attn: {STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


_lock = threading.Lock()
_lib = None


def library_path() -> Path:
    return _build.LIB


def load() -> C.CDLL:
    """Load (building first if the in-tree .so is missing or stale) and type the library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.build()
        lib = C.CDLL(str(path))
        lib.dmf_attn_abi_version.restype = C.c_int
        lib.dmf_attn_status_string.restype = C.c_char_p
        lib.dmf_attn_status_string.argtypes = [C.c_int]
        lib.dmf_attn_selftest_wait_limit.restype = C.c_int
        lib.dmf_attn_selftest_wait_limit.argtypes = [C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.dmf_attn_kernel_name.restype = C.c_int
        lib.dmf_attn_kernel_name.argtypes = [C.c_int32] * 5 + [C.c_char_p, C.c_size_t]
        for name in ("dmf_attn_fwd_dual", "dmf_attn_fwd", "dmf_attn_fwd_dual_f32out"):
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(FwdArgs)]
        for name in ("dmf_attn_bwd", "dmf_attn_bwd_static"):
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(BwdArgs)]
        lib.dmf_attn_bwd_workspace_bytes.restype = C.c_size_t
        lib.dmf_attn_bwd_workspace_bytes.argtypes = [C.c_int32] * 5
        lib.dmf_attn_check_status_word.restype = C.c_int
        lib.dmf_attn_check_status_word.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
        lib.dmf_attn_validate_fwd.restype = C.c_int
        lib.dmf_attn_validate_fwd.argtypes = [C.POINTER(FwdArgs), C.c_int]
        lib.dmf_attn_validate_bwd.restype = C.c_int
        lib.dmf_attn_validate_bwd.argtypes = [C.POINTER(BwdArgs)]
        lib.dmf_rmsnorm_fwd.restype = C.c_int
        lib.dmf_rmsnorm_fwd.argtypes = [C.POINTER(RmsNormArgs)]
        lib.dmf_rmsnorm_bwd.restype = C.c_int
        lib.dmf_rmsnorm_bwd.argtypes = [C.POINTER(RmsNormBwdArgs)]
        lib.dmf_rmsnorm_bwd_workspace_bytes.restype = C.c_size_t
        lib.dmf_rmsnorm_bwd_workspace_bytes.argtypes = [C.c_int32]
        for name, args in (("dmf_ln_modulate_fwd", LnModulateArgs), ("dmf_ln_modulate_bwd", LnModulateBwdArgs),
                           ("dmf_gate_residual_fwd", GateResidualArgs), ("dmf_gate_residual_bwd", GateResidualBwdArgs)):
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(args)]
        lib.dmf_step_tail.restype = C.c_int
        lib.dmf_step_tail.argtypes = [C.POINTER(StepTailArgs)]
        lib.dmf_adaln_bwd_workspace_bytes.restype = C.c_size_t
        lib.dmf_adaln_bwd_workspace_bytes.argtypes = [C.c_int32] * 3
        got = lib.dmf_attn_abi_version()
        if got != ABI_VERSION:
            raise ImportError(f"libdmf_attn.so has ABI version {got}, this package expects {ABI_VERSION}")
        _lib = lib
        return lib


def kernel_name(op: str, seqlen_q: int, seqlen_kv: int, head_dim: int, dtype: int = BF16) -> str:
    """The kernel template instance the launcher picks for this problem (op: 'dual', 'fwd' or 'bwd')."""
    buf = C.create_string_buffer(256)
    check(load().dmf_attn_kernel_name({"dual": 0, "fwd": 1, "bwd": 2}[op], seqlen_q, seqlen_kv, head_dim, dtype,
                                      buf, len(buf)))
    return buf.value.decode()


def check(status: int) -> None:
    if status != 0:
        raise DmfAttnError(status, load().dmf_attn_status_string(status).decode())
