"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, and rejects bad arguments with the documented status codes."""

import ctypes as C
import re
from pathlib import Path

import pytest

from dmf_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = "".join(h.read_text() for h in sorted((ROOT / "include").glob("*.h")))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dmf_[a-z_0-9]+)\s*\(", text)))


def test_library_loads_and_exports_header_symbols():
    lib = _lib.load()
    declared = _declared_symbols()
    assert set(declared) == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.dmf_attn_abi_version() == _lib.ABI_VERSION


def test_status_strings():
    lib = _lib.load()
    seen = set()
    for code in _lib.STATUS_NAMES:
        s = lib.dmf_attn_status_string(code).decode()
        assert s and s not in seen
        seen.add(s)
    assert lib.dmf_attn_status_string(999).decode() == "unknown status"


def _good_args(dual=True):
    a = _lib.FwdArgs()
    a.batch, a.seqlen_q, a.seqlen_kv, a.heads, a.head_dim = 2, 256, 256, 4, 72
    a.dtype, a.softmax_scale = _lib.BF16, 72 ** -0.5
    fake = 0x10000  # never dereferenced by validation
    for name in ("q", "k", "v", "tq", "tk", "tv", "o", "to"):
        setattr(a, name, _lib.Tensor4(fake, 256 * 4 * 72, 4 * 72, 72))
    a.lse = fake
    return a


def test_validation_accepts_reference_layouts():
    lib = _lib.load()
    a = _good_args()
    assert lib.dmf_attn_validate_fwd(C.byref(a), 1) == 0
    # strided views of a packed (B, L, 3, H, D) qkv projection
    for name, off in (("q", 0), ("k", 4 * 72 * 2), ("v", 2 * 4 * 72 * 2)):
        setattr(a, name, _lib.Tensor4(0x10000 + off, 256 * 3 * 4 * 72, 3 * 4 * 72, 72))
    assert lib.dmf_attn_validate_fwd(C.byref(a), 1) == 0
    assert lib.dmf_attn_validate_fwd(C.byref(a), 0) == 0


def test_backward_workspace_sizes():
    """Two fp32 rows per query for every backward kernel; where the long-sequence one-pass kernel applies (more
    than two tiles in a length, head_dim <= 80), an fp32 dQ accumulator behind them, 256-byte aligned."""
    lib = _lib.load()
    rows = lambda B, H, L: 8 * B * H * L
    assert lib.dmf_attn_bwd_workspace_bytes(256, 256, 256, 16, 72) == rows(256, 16, 256)     # two tiles: cluster kernel
    assert lib.dmf_attn_bwd_workspace_bytes(4, 1024, 1024, 16, 128) == rows(4, 16, 1024)     # head_dim above 80
    assert lib.dmf_attn_bwd_workspace_bytes(64, 1024, 1024, 16, 72) == rows(64, 16, 1024) + 4 * 64 * 16 * 1024 * 72
    assert lib.dmf_attn_bwd_workspace_bytes(1, 128, 384, 3, 64) == 3072 + 4 * 3 * 128 * 64   # 3072 is already aligned
    assert lib.dmf_attn_bwd_workspace_bytes(1, 128, 384, 1, 64) == 1024 + 4 * 128 * 64
    assert lib.dmf_attn_bwd_workspace_bytes(1, 100, 128, 1, 64) == 0                         # not a valid problem


@pytest.mark.parametrize("field,value,status", [
    ("dtype", 7, 2),
    ("head_dim", 48, 3), ("head_dim", 76, 3), ("head_dim", 136, 3),
    ("seqlen_q", 100, 4), ("seqlen_kv", 0, 4), ("seqlen_kv", 130, 4),
    ("batch", 0, 5), ("heads", 0, 5),
])
def test_validation_rejects_bad_sizes(field, value, status):
    lib = _lib.load()
    a = _good_args()
    setattr(a, field, value)
    assert lib.dmf_attn_validate_fwd(C.byref(a), 1) == status


def test_validation_rejects_bad_pointers_and_strides():
    lib = _lib.load()
    a = _good_args()
    a.q = _lib.Tensor4(0, 1, 1, 1)
    assert lib.dmf_attn_validate_fwd(C.byref(a), 1) == 1          # NULL
    a = _good_args()
    a.k = _lib.Tensor4(0x10008, 256 * 4 * 72, 4 * 72, 72)
    assert lib.dmf_attn_validate_fwd(C.byref(a), 1) == 7          # misaligned base
    a = _good_args()
    a.v = _lib.Tensor4(0x10000, 256 * 4 * 72, 4 * 72 + 4, 72)
    assert lib.dmf_attn_validate_fwd(C.byref(a), 1) == 6          # stride not a multiple of 16 bytes
    a = _good_args()
    a.tq = _lib.Tensor4(0, 1, 1, 1)
    assert lib.dmf_attn_validate_fwd(C.byref(a), 1) == 1          # tangents required by the dual pass
    assert lib.dmf_attn_validate_fwd(C.byref(a), 0) == 0          # ... and ignored by the plain one
    a = _good_args()
    a.lse = None
    assert lib.dmf_attn_validate_fwd(C.byref(a), 0) == 1
    assert lib.dmf_attn_validate_fwd(None, 0) == 1


def test_compute_entry_points_fail_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    lib = _lib.load()
    a = _good_args()
    # no device: a status, not a crash and not a silent CPU computation
    assert lib.dmf_attn_fwd_dual(C.byref(a)) == 8
    assert lib.dmf_attn_fwd(C.byref(a)) == 8
    from dmf_b200 import flash_attn_func
    q = torch.randn(1, 128, 1, 64)
    with pytest.raises(Exception):
        flash_attn_func(q, q, q)


def test_adaln_entry_points_reject_bad_arguments_without_a_gpu():
    lib = _lib.load()
    fake = 0x10000
    a = _lib.LnModulateArgs()
    a.batch, a.seqlen, a.channels = 2, 16, 1152
    a.wide_dtype, a.narrow_dtype, a.mod_dtype = _lib.ADALN_F32, _lib.ADALN_BF16, _lib.ADALN_BF16
    a.x, a.y = _lib.Rows(fake, 16 * 1152, 1152), _lib.Rows(fake, 16 * 1152, 1152)
    a.shift, a.scale = _lib.Mod(fake, 6 * 1152), _lib.Mod(fake, 6 * 1152)
    assert lib.dmf_ln_modulate_fwd(None) == 1
    a.channels = 1000
    assert lib.dmf_ln_modulate_fwd(C.byref(a)) == 5          # width not compiled
    a.channels = 1152
    a.wide_dtype, a.narrow_dtype = _lib.ADALN_BF16, _lib.ADALN_F32
    assert lib.dmf_ln_modulate_fwd(C.byref(a)) == 2          # a bf16 stream with fp32 matmul side
    a.wide_dtype, a.narrow_dtype = _lib.ADALN_F32, _lib.ADALN_BF16
    a.x = _lib.Rows(fake + 4, 16 * 1152, 1152)
    assert lib.dmf_ln_modulate_fwd(C.byref(a)) == 7          # base not 16-byte aligned
    a.x = _lib.Rows(fake, 16 * 1152, 1150)
    assert lib.dmf_ln_modulate_fwd(C.byref(a)) == 6          # row stride not a multiple of 4 elements
    a.x = _lib.Rows(fake, 16 * 1152, 1152)
    a.scale = _lib.Mod(None, 0)
    assert lib.dmf_ln_modulate_fwd(C.byref(a)) == 1
    a.scale = _lib.Mod(fake, 6 * 1152)
    assert lib.dmf_ln_modulate_fwd(C.byref(a)) == 8          # all checks pass: no device here
    assert lib.dmf_adaln_bwd_workspace_bytes(4, 100, 1152) == 4 * 13 * 2 * 1152 * 4      # small problem: 8 rows per block
    assert lib.dmf_adaln_bwd_workspace_bytes(64, 1024, 1152) == 64 * 32 * 2 * 1152 * 4  # 32 rows per block
    b = _lib.GateResidualBwdArgs()
    b.batch, b.seqlen, b.channels = 2, 16, 768
    b.wide_dtype, b.narrow_dtype, b.mod_dtype = _lib.ADALN_F32, _lib.ADALN_BF16, _lib.ADALN_BF16
    b.dout, b.h, b.dh = (_lib.Rows(fake, 16 * 768, 768) for _ in range(3))
    b.gate, b.dgate = _lib.Mod(fake, 768), fake
    assert lib.dmf_gate_residual_bwd(C.byref(b)) == 11       # no workspace


def test_python_surface_has_no_cpu_path():
    """Every op of the package raises on CPU tensors instead of computing somewhere else."""
    import torch
    from dmf_b200 import adaln, flash_attn_func, flash_attn_qkvpacked_func
    from dmf_b200.rms_norm import rms_norm
    q = torch.randn(1, 128, 2, 64).bfloat16()
    with pytest.raises(Exception):
        flash_attn_func(q, q, q)
    with pytest.raises(Exception):
        flash_attn_qkvpacked_func(torch.stack([q, q, q], dim=2))
    with pytest.raises(ValueError):
        flash_attn_qkvpacked_func(q)                       # not a (B, L, 3, H, D) tensor
    with pytest.raises(Exception):
        rms_norm(q, torch.ones(64))
    x = torch.randn(2, 8, 384)
    mod = torch.zeros(2, 1, 384)
    assert not adaln.usable(x)
    with pytest.raises(RuntimeError):
        adaln.ln_modulate(x, mod, mod)
    with pytest.raises(RuntimeError):
        adaln.gate_residual(x, mod, x)
