"""dqmoe_quant_fp8_tensor_static: the per-tensor FP8 quantiser for callers that may not
allocate (its amax scratch is a static device array inside the library). Checked through the
C ABI against dqmoe_quant_fp8_tensor, bit for bit, on two calls in a row: the second call
sees the first call's maxima in the shared array and must clear them."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import bits

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _both(lib, check, x, e):
    numel_per = x.numel() // e
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    q_ref = torch.zeros(x.shape, dtype=torch.uint8, device=DEV)
    s_ref = torch.zeros(e, dtype=torch.float32, device=DEV)
    scratch = torch.zeros(e, dtype=torch.float32, device=DEV)
    check(lib.dqmoe_quant_fp8_tensor(p(x), e, numel_per, p(q_ref), p(s_ref), p(scratch), stream))
    q_new = torch.zeros(x.shape, dtype=torch.uint8, device=DEV)
    s_new = torch.zeros(e, dtype=torch.float32, device=DEV)
    check(lib.dqmoe_quant_fp8_tensor_static(p(x), e, numel_per, p(q_new), p(s_new), stream))
    torch.cuda.synchronize()
    return q_ref, s_ref, q_new, s_new


def test_static_scratch_entry_point_matches_the_allocating_one_twice():
    from dqmoe_b200 import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(17)
    big = (torch.randn(8, 96, 1024, generator=g) * 3.0).to(torch.bfloat16).to(DEV)      # per-expert, large maxima
    small = (torch.randn(8, 96, 1024, generator=g) * 0.01).to(torch.bfloat16).to(DEV)   # smaller maxima afterwards
    for x, e in ((big, 8), (small, 8), (small, 1)):
        q_ref, s_ref, q_new, s_new = _both(lib, _lib.check, x, e)
        assert np.array_equal(bits(s_new), bits(s_ref))
        assert torch.equal(q_new, q_ref)
        assert float(s_new.max()) > 0.0


def test_static_scratch_entry_point_rejects_more_slices_than_it_holds():
    from dqmoe_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(1025 * 8, dtype=torch.bfloat16, device=DEV)
    q = torch.zeros(1025 * 8, dtype=torch.uint8, device=DEV)
    s = torch.zeros(1025, dtype=torch.float32, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.dqmoe_quant_fp8_tensor_static(p(x), 1025, 8, p(q), p(s), None)
    assert rc == 1
    assert "exceeds the 1024 slices" in lib.dqmoe_last_error().decode()
    # the largest size it accepts still works
    _lib.check(lib.dqmoe_quant_fp8_tensor_static(p(x), 1024, 8, p(q), p(s), None))
    torch.cuda.synchronize()
