"""lq4_linear_decode_noalloc: the entry point for callers that may not allocate device memory
(an engine that gave all of it to its own pool, or a decode loop that cannot take the
device-wide synchronisation cudaMalloc implies).  It must give what lq4_linear gives.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  The test owns no state from the others and passes alone in a fresh process too.
"""
import ctypes as C

import numpy as np
import pytest

from lattice_b200 import _lib
from tests._cases import make_case, tol_ratio

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _run_both(be, case, bf16=False):
    """Returns (y from lq4_linear, y from lq4_linear_decode_noalloc) for one projection."""
    from lattice_b200 import Q4WeightBuf
    from lattice_b200._lib import LinearArgs, LoraDesc, RotDesc
    L = _lib.lib()
    qw = Q4WeightBuf.from_host_payload(case["payload"], case["n"], case["k"])
    x = _dev(case["x"]).to(torch.bfloat16) if bf16 else _dev(case["x"])
    keep, lora, rot = [], None, None
    if case["lora"] is not None:
        a, b, s = case["lora"]
        ad, bd = _dev(a), _dev(b)
        keep += [ad, bd]
        lora = LoraDesc(ad.data_ptr(), bd.data_ptr(), case["rank"], s)
    if case["signs"] is not None:
        sd = _dev(case["signs"])
        keep.append(sd)
        rot = RotDesc(sd.data_ptr(), sd.numel())
    stream = torch.cuda.current_stream().cuda_stream
    m, n, k = case["m"], case["n"], case["k"]
    y_ref = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    be.dispatch_gemm_q4(x, 0, qw, y_ref, 0, m, n, k, lora=lora, rot=rot)
    y_new = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    args = LinearArgs(x.data_ptr(), _lib.DTYPE_BF16 if bf16 else _lib.DTYPE_F32, m, n, k, qw.payload_ptr,
                      y_new.data_ptr(), 0, C.pointer(lora) if lora is not None else None,
                      C.pointer(rot) if rot is not None else None, 0)
    _lib.check(L.lq4_linear_decode_noalloc(C.byref(args), stream))
    # the entry point has no context: its bounded waits report through the built-in array's own status word
    _lib.check(L.lq4_noalloc_check(stream))
    be.check_device_status()
    out = (y_ref.cpu().numpy(), y_new.cpu().numpy())
    qw.free()
    return out


def test_noalloc_entry_point_matches_lq4_linear_on_two_calls_in_a_row():
    from lattice_b200 import CudaQ4Backend
    be = CudaQ4Backend(0)
    try:
        # two different shapes back to back: whatever the first call leaves in the shared
        # scratch (partial sums, tickets, LoRA partials) must not leak into the second
        cases = [make_case(3, 1, 5120, 1024, rank=16, alpha=32.0, extra=41),      # split-k tiles + LoRA
                 make_case(5, 2, 1024, 300, quarot=True, extra=42)]   # rotation, ragged n
        for rep in range(2):
            for case in cases:
                y_old, y_new = _run_both(be, case)
                assert tol_ratio(y_new, y_old) <= 1.0
                assert tol_ratio(y_new, case["y_ref"]) <= 1.0
    finally:
        be.close()


def test_noalloc_entry_point_multi_token_variants_twice_in_a_row():
    """The entry point is the only caller of the resident kernel with 2..4 tokens: adapters with several
    tokens (the projection messages of every token), the fast in-register rotation per row, bf16 rows."""
    from lattice_b200 import CudaQ4Backend
    be = CudaQ4Backend(0)
    try:
        cases = [(make_case(2, 3, 1024, 300, rank=16, alpha=32.0, extra=51), False),     # ragged n, adapter, 3 tokens
                 (make_case(2, 4, 1024, 1000, rank=16, alpha=32.0, extra=52), False),    # 4 tokens, n % 128 != 0
                 (make_case(5, 2, 2048, 384, quarot=True, extra=53), False),             # rotation, K >= 2048
                 (make_case(2, 4, 1024, 512, bf16_x=True, extra=54), True)]              # bf16 rows
        for rep in range(2):
            for case, bf16 in cases:
                y_old, y_new = _run_both(be, case, bf16=bf16)
                assert tol_ratio(y_new, y_old) <= 1.0
                assert tol_ratio(y_new, case["y_ref"]) <= 1.0
    finally:
        be.close()


def test_noalloc_check_reports_nothing_after_clean_calls():
    L = _lib.lib()
    assert L.lq4_noalloc_check(torch.cuda.current_stream().cuda_stream) == _lib.OK


def test_noalloc_entry_point_rejects_what_exceeds_its_fixed_scratch():
    from lattice_b200._lib import LinearArgs, LoraDesc
    L = _lib.lib()
    x = torch.zeros((8, 65536), device="cuda")
    w = torch.zeros(64 * 32 * 20, dtype=torch.uint8, device="cuda")
    y = torch.zeros((8, 64), device="cuda")

    def call(m=1, n=64, k=1024, lora=None):
        args = LinearArgs(x.data_ptr(), 0, m, n, k, w.data_ptr(), y.data_ptr(), 0,
                          C.pointer(lora) if lora is not None else None, None, 0)
        return L.lq4_linear_decode_noalloc(C.byref(args), None)

    assert call(m=5) == _lib.ERR_NOSPACE and b"at most 4 tokens" in L.lq4_last_error()
    assert call(n=40000) == _lib.ERR_NOSPACE
    assert call(m=4, k=65536) == _lib.ERR_NOSPACE     # the activation rows no longer fit in shared memory
    big = LoraDesc(x.data_ptr(), x.data_ptr(), 65, 1.0)
    assert call(lora=big) == _lib.ERR_NOSPACE
    assert call(k=96) == _lib.ERR_ALIGN
    odd = LoraDesc(x.data_ptr() + 2, x.data_ptr(), 16, 1.0)      # a factor pointer lq4_linear refuses too
    assert call(lora=odd) == _lib.ERR_ALIGN
    assert call(k=40) == _lib.ERR_K
    assert call(m=0) == _lib.OK
    assert L.lq4_linear_decode_noalloc(None, None) == _lib.ERR_NULL
