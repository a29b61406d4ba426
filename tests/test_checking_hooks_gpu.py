"""The library's checking hooks on a GPU:

* the fp32-output mode of the fused forward + tangent kernel against an fp64 evaluation that rounds its
  operands where the kernel does - the "max relative error <= 1e-3 for fp32-accumulated outputs" criterion;
* the bounded device-side wait: a wait that nothing ever satisfies gives up after its limit, reports which
  wait it was, and leaves the context usable (no trap, no fault, no endless loop anywhere);
* the host side of that report: a non-zero status word becomes DmfAttnError(ERR_TIMEOUT) and is cleared.
"""

import ctypes as C

import pytest
import torch

from dmf_b200 import _lib, ops
from oracle import attn_jvp_oracle as orc
from tests import _cabi

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")

# Tolerance of the fp32-accumulated outputs, as max|a - b| / max|b| against the fp64 evaluation with the same
# operand roundings (bf16 inputs, bf16 P, bf16 P*dS).  What is left is the kernel's own arithmetic: fp32 sums, fp32
# rescaling, and the few P or P*dS elements (about one in 10^4) that an fp32 exponent argument and ex2.approx put
# on the other side of a bf16 rounding boundary than the fp64 evaluation; one such element of a heavy key is worth
# up to a few 1e-4 in this max-norm metric, which is why the observed values sit near 1e-4 and not near 1e-6.
TOL_F32_OUT = 1e-3
# the same comparison in relative L2, where isolated rounding flips do not dominate
TOL_F32_OUT_L2 = 3e-4


@pytest.mark.parametrize("B,L,H,D,qk_norm,big_rows", [
    (2, 256, 3, 64, False, False),
    (2, 1024, 2, 64, False, True),
    (2, 256, 3, 72, False, True),
    (1, 1024, 4, 72, True, False),
    (1, 1024, 2, 72, False, True),
])
def test_fp32_accumulated_outputs_within_1e_3(B, L, H, D, qk_norm, big_rows):
    ins = orc.make_inputs(B, L, H, D, seed=31 + D + L, tangent_scale=0.1, qk_norm=qk_norm)
    if big_rows:
        ins[0][:, 5:37] *= 8.0           # rows with large logits: the lazily updated maximum moves between blocks
    dev_in = [x.bfloat16().to(DEV) for x in ins]
    o, to, lse, _ = _cabi.fwd_dual_f32out(*dev_in)
    assert o.dtype == torch.float32 and not torch.isnan(o).any() and not torch.isnan(to).any()
    ref_in = [x.float().cpu() for x in dev_in]                      # the bf16 values the kernel saw
    o_ref, to_ref, lse_ref = orc.attn_jvp_online_lazy(*ref_in, emulate_bf16=True)
    e_o, e_to = orc.max_rel(o.cpu(), o_ref), orc.max_rel(to.cpu(), to_ref)
    e_lse = orc.max_rel(lse.cpu(), lse_ref)
    l2_o, l2_to = orc.rel_l2(o.cpu(), o_ref), orc.rel_l2(to.cpu(), to_ref)
    print(f"fp32-out D={D} L={L} qk_norm={qk_norm} big_rows={big_rows}: max-rel o {e_o:.2e} to {e_to:.2e} "
          f"lse {e_lse:.2e}; rel-L2 o {l2_o:.2e} to {l2_to:.2e}")
    assert e_o <= TOL_F32_OUT and e_to <= TOL_F32_OUT and e_lse <= TOL_F32_OUT
    assert l2_o <= TOL_F32_OUT_L2 and l2_to <= TOL_F32_OUT_L2
    # the 16-bit entry point computes the same thing up to its own output rounding (and its faster exponentials)
    o16, to16, lse16, _ = _cabi.fwd(*dev_in)
    assert orc.rel_l2(o16.float(), o) < 4e-3 and orc.rel_l2(to16.float(), to) < 4e-3
    assert orc.max_rel(lse16, lse) < 1e-4


def test_fp32_out_rejects_what_it_does_not_cover():
    ins = [x.bfloat16().to(DEV) for x in orc.make_inputs(1, 128, 1, 64, seed=1)]   # one query tile: no tile pair
    _cabi.fwd_dual_f32out(*ins, expect=3)
    ins = [x.bfloat16().to(DEV) for x in orc.make_inputs(1, 256, 1, 96, seed=1)]   # head_dim above 80
    _cabi.fwd_dual_f32out(*ins, expect=3)


def test_a_wait_that_runs_out_reports_and_leaves_the_context_usable():
    lib = _lib.load()
    sw = torch.zeros(1, dtype=torch.int32, device=DEV)
    res = torch.full((4,), -1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream(DEV).cuda_stream
    limit = 200_000                                                   # SM cycles: about 0.1 ms
    assert lib.dmf_attn_selftest_wait_limit(limit, sw.data_ptr(), res.data_ptr(), stream) == 0
    raw = C.c_int32(0)
    assert lib.dmf_attn_check_status_word(sw.data_ptr(), stream, C.byref(raw)) == 12      # DMF_ATTN_ERR_TIMEOUT
    assert raw.value == 901                                           # role 900 (self-test), barrier 1
    first, second, signalled, cycles = res.tolist()
    assert first == 0          # the wait on the barrier nobody signals gave up ...
    assert cycles >= limit     # ... after its limit, not before
    assert cycles < 50 * limit
    assert second == 0         # the other waiter saw the abort flag long before its own (64 x) limit
    assert signalled == 1      # an ordinary wait still succeeds
    # limits outside the allowed range launch nothing
    assert lib.dmf_attn_selftest_wait_limit(10, sw.data_ptr(), res.data_ptr(), stream) == 5
    assert lib.dmf_attn_selftest_wait_limit(10**10, sw.data_ptr(), res.data_ptr(), stream) == 5
    # the context is intact: a normal call right afterwards is correct
    ins = orc.make_inputs(1, 256, 2, 72, seed=3, tangent_scale=0.1)
    dev_in = [x.bfloat16().to(DEV) for x in ins]
    o, to, _, _ = _cabi.fwd(*dev_in)
    o_ref, to_ref, _ = orc.attn_jvp_closed_form(*[x.float().cpu() for x in dev_in])
    assert orc.rel_l2(o.float().cpu(), o_ref) < 6e-3 and orc.rel_l2(to.float().cpu(), to_ref) < 6e-3


def test_nonzero_status_word_raises_and_is_cleared():
    w = ops._status_word(DEV)
    torch.cuda.synchronize()
    w.fill_(307)                                                      # what a softmax-role wait on barrier 7 would leave
    with pytest.raises(_lib.DmfAttnError) as ei:
        ops.check_device_status(DEV)
    assert ei.value.status == 12 and "307" in str(ei.value)
    assert int(w.item()) == 0                                         # cleared: the next check passes
    ops.check_device_status(DEV)
    # the non-blocking form reports one call late, without synchronising
    w.fill_(205)
    ops.poll_device_status(DEV)                                       # starts the read-back
    torch.cuda.synchronize()
    with pytest.raises(_lib.DmfAttnError):
        ops.poll_device_status(DEV)                                   # sees the value read back by the first call
    assert int(w.item()) == 0
    torch.cuda.synchronize()
    ops.poll_device_status(DEV)
    torch.cuda.synchronize()
    ops.poll_device_status(DEV)
