"""Host logic of the drop-in `moe_test` module that needs no GPU."""
import glob
import importlib.util
import os

import pytest
import torch

import moe_test as _shim

_EXT = glob.glob(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "dqmoe_b200", "dropin_ext",
                              "moe_test*.so"))


@pytest.fixture(params=["ctypes module", "pybind11 extension"])
def moe_test(request):
    """Both builds of the drop-in module: dqmoe_b200/dropin/moe_test.py and the compiled
    dqmoe_b200/dropin_ext/moe_test*.so (python -m dqmoe_b200.build --ext)."""
    if request.param == "ctypes module":
        return _shim
    if not _EXT:
        pytest.skip("the pybind11 extension is not built")
    spec = importlib.util.spec_from_file_location("moe_test", _EXT[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_get_mn_major_tma_aligned_tensor_matches_reference_strides(moe_test):
    # csrc/torch_help.h:37-52: same values, strides (mn*sf_k, 1, mn); identity when already so
    sf = torch.arange(2 * 5 * 3, dtype=torch.float32).view(2, 5, 3)
    out = moe_test.get_mn_major_tma_aligned_tensor(sf)
    assert out.shape == sf.shape and out.stride() == (15, 1, 5)
    assert torch.equal(out, sf)
    again = moe_test.get_mn_major_tma_aligned_tensor(out)
    assert again.data_ptr() == out.data_ptr()
    sf2 = torch.arange(12, dtype=torch.float32).view(4, 3)
    out2 = moe_test.get_mn_major_tma_aligned_tensor(sf2)
    assert out2.shape == (4, 3) and out2.stride() == (1, 4) and torch.equal(out2, sf2)
    with pytest.raises(RuntimeError, match="ASSERT FAILED"):
        moe_test.get_mn_major_tma_aligned_tensor(sf.double())
    with pytest.raises(RuntimeError, match="ASSERT FAILED"):
        moe_test.get_mn_major_tma_aligned_tensor(torch.zeros(3))


def _args(T=4, H=64, I=32, E=2, k=2, idx_dtype=torch.int32):
    a = torch.zeros(T, H, dtype=torch.bfloat16)
    b = torch.zeros(E, 2 * I, H, dtype=torch.bfloat16)
    b1 = torch.zeros(E, H, I, dtype=torch.bfloat16)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16)
    mi = torch.zeros(T, k, dtype=idx_dtype)
    ws = torch.zeros(1024, dtype=torch.uint8)
    one = torch.ones(1)
    return (a, one), (b, one), (b1, one), d, mi, ws


def test_shape_and_dtype_checks_raise_like_the_reference(moe_test):
    a, b, b1, d, mi, ws = _args()
    bad_b1 = (torch.zeros(2, 64, 48, dtype=torch.bfloat16), b1[1])  # inter_size*2 != rows of b
    with pytest.raises(RuntimeError, match=r"\[ASSERT FAILED\].*inter_size \* 2 == inter_size_2"):
        moe_test.m_grouped_moe_nt_contiguous_bf16(a, b, bad_b1, d, mi, ws, 0)
    a, b, b1, d, mi, ws = _args(idx_dtype=torch.int64)
    with pytest.raises(RuntimeError, match=r"m_indices.scalar_type\(\) == torch::kInt"):
        moe_test.m_grouped_moe_nt_contiguous_bf16(a, b, b1, d, mi, ws, 0)
    a, b, b1, d, mi, ws = _args()
    with pytest.raises(RuntimeError, match="ASSERT FAILED"):  # bf16 data through the FP8 entry point
        moe_test.m_grouped_moe_nt_contiguous_fp8_bf16(a, b, b1, d, mi, ws, 1024)


def test_zero_tokens_returns_silently(moe_test):
    a, b, b1, d, mi, ws = _args(T=0)
    assert moe_test.m_grouped_moe_nt_contiguous_bf16(a, b, b1, d, mi, ws, 0) is None


def test_cpu_tensors_are_rejected_not_computed(moe_test):
    a, b, b1, d, mi, ws = _args()
    with pytest.raises(RuntimeError):
        moe_test.m_grouped_moe_nt_contiguous_bf16(a, b, b1, d, mi, ws, 0)
