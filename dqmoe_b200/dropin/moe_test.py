"""Drop-in replacement of the reference's `moe_test` extension module.

Put this directory on sys.path (or copy/symlink this file next to the
reference's test/torch_test.py, where develop.sh:12-15 puts the built
extension) and `import moe_test` resolves here. The three functions have the
names, arguments and error behaviour of csrc/pybind11_register.h:153-163; the
work is done by libdqmoe_b200.so through its C ABI.
"""
from __future__ import annotations

import os
import sys

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    # at the end: the importing script's own modules (the reference's test/bench.py, test/util.py) must keep
    # winning over same-named files at the root of this repository
    sys.path.append(_ROOT)

from dqmoe_b200 import ops as _ops  # noqa: E402


def _fail(cond: str, info: str = "") -> None:
    msg = f"[ASSERT FAILED] moe_test.py  Condition: {cond}"
    if info:
        msg += f"  Info: {info}"
    raise RuntimeError(msg)


def _run(a, b, b1, d, m_indices, workspace, quant_mode_value, fused, fp8):
    a0, sfa = a
    b0, sfb = b
    b10, sfb1 = b1
    # shape checks of csrc/pybind11_register.h:108-123
    if a0.dim() != 2 or b0.dim() != 3 or b10.dim() != 3 or d.dim() != 3 or m_indices.dim() != 2:
        _fail("a [T,H], b [E,2I,H], b1 [E,H,I], d [T,k,H], m_indices [T,k]")
    T, H = a0.shape
    E, I2, H_ = b0.shape
    T_, k, H__ = d.shape
    E_, H___, I = b10.shape
    T___, k_ = m_indices.shape
    if not (T == T_ and E == E_ and H == H_ and H == H__ and H == H___ and I * 2 == I2):
        _fail("num_tokens == num_tokens_ and num_groups == num_groups_ and hidden_size == hidden_size_ and "
              "hidden_size == hidden_size__ and hidden_size == hidden_size___ and inter_size * 2 == inter_size_2")
    if T___ != T or k_ != k:
        _fail("m_indices.shape == (num_tokens, topk)")
    if m_indices.dtype != torch.int32:
        _fail("m_indices.scalar_type() == torch::kInt")
    if T == 0:
        return
    want = torch.float8_e4m3fn if fp8 else torch.bfloat16
    if a0.dtype != want or b0.dtype != want or b10.dtype != want:
        _fail(f"a, b, b1 data tensors are {want}")
    if d.dtype != torch.bfloat16:
        _fail("d.scalar_type() == torch::kBFloat16")
    if fp8:
        if quant_mode_value not in (256, 512, 1024, 2048):
            _fail("quant_mode_value in (256, 512, 1024, 2048)", f"got {quant_mode_value}")
        # 2048 = MXFP8, an added mode (include/dqmoe.h): its scale tensors hold UE8M0 bytes
        want_s = torch.uint8 if quant_mode_value == 2048 else torch.float32
        for name, s in (("sfa", sfa), ("sfb", sfb), ("sfb1", sfb1)):
            if s.dtype != want_s or not s.is_contiguous() or not s.is_cuda:
                _fail(f"{name} is a contiguous {want_s} CUDA tensor")
        mode = quant_mode_value
    else:
        # the scale halves are dummy tensors in this mode (test/util.py:232-234) and are not read
        sfa = sfb = sfb1 = None
        mode = 0
    if workspace.data_ptr() % 256 != 0:
        _fail("is_aligned(workspace.data_ptr(), CUDA_MEM_ALIGN)",
              f"workspace pointer {hex(workspace.data_ptr())} is not aligned!")
    _ops.moe_forward(a0, sfa, b0, sfb, b10, sfb1, d, m_indices, workspace, mode, fused)


def m_grouped_moe_nt_contiguous_fp8_bf16(a, b, b1, d, m_indices, workspace, quant_mode_value, fused=True):
    """FP8 E4M3 layer, bf16 output (csrc/pybind11_register.h:156-159)."""
    _run(a, b, b1, d, m_indices, workspace, int(quant_mode_value), bool(fused), True)


def m_grouped_moe_nt_contiguous_bf16(a, b, b1, d, m_indices, workspace, quant_mode_value, fused=True):
    """bf16 layer (csrc/pybind11_register.h:160-162); quant_mode_value is ignored like the scales."""
    _run(a, b, b1, d, m_indices, workspace, 0, bool(fused), False)


def get_mn_major_tma_aligned_tensor(sf: torch.Tensor) -> torch.Tensor:
    """Scale tensor with MN-major strides (mn*sf_k, 1, mn); csrc/torch_help.h:37-52."""
    if sf.dim() not in (2, 3):
        _fail("dim == 2 or dim == 3")
    if sf.dtype != torch.float32:
        _fail("sf.scalar_type() == torch::kFloat")
    dim = sf.dim()
    batched = sf.unsqueeze(0) if dim == 2 else sf
    g, mn, sf_k = batched.shape
    if (batched.stride(0) == mn * sf_k or dim == 2) and batched.stride(1) == 1 and batched.stride(2) == mn:
        return batched.squeeze(0) if dim == 2 else batched
    out = torch.empty_strided((g, mn, sf_k), (mn * sf_k, 1, mn), dtype=batched.dtype, device=batched.device)
    out.copy_(batched)
    return out.squeeze(0) if dim == 2 else out
