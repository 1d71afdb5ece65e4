"""Shared helpers of the tests: seeded inputs, golden-file access, bit views."""
from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def make_inputs(seed, T, H, I, E, k, act_std=1.0, w_std=0.02):
    """Same generator as tests/golden/make_golden.py:make_inputs (CPU tensors)."""
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(T, H, generator=g) * act_std).to(torch.bfloat16)
    b = (torch.randn(E, 2 * I, H, generator=g) * w_std).to(torch.bfloat16)
    b1 = (torch.randn(E, H, I, generator=g) * w_std).to(torch.bfloat16)
    scores = torch.randn(T, E, generator=g)
    m_indices = torch.topk(scores, k, dim=1).indices.to(torch.int32)
    return a, b, b1, scores, m_indices


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


def bf16_from_bits(arr: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(arr).view(np.int16)).view(torch.bfloat16)


def fp8_from_bits(arr: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(arr)).view(torch.float8_e4m3fn)


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()
