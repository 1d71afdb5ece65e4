"""Generate the golden fixtures of tests/golden/ from the reference's own torch code.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's test/util.py (with util.device = "cpu"), feeds it seeded
inputs and stores the inputs and the reference's outputs as .npz files. The tests
never import the reference; they read these files. bf16 tensors are stored as their
uint16 bit patterns, e4m3 tensors as uint8.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_util(ref_root: str):
    spec = importlib.util.spec_from_file_location("ref_util", os.path.join(ref_root, "test", "util.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.device = "cpu"
    return mod


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def make_inputs(seed: int, T: int, H: int, I: int, E: int, k: int, act_std: float, w_std: float):
    """Seeded layer inputs; the same function is used by the tests (tests/helpers.py mirrors it)."""
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(T, H, generator=g) * act_std).to(torch.bfloat16)
    b = (torch.randn(E, 2 * I, H, generator=g) * w_std).to(torch.bfloat16)
    b1 = (torch.randn(E, H, I, generator=g) * w_std).to(torch.bfloat16)
    scores = torch.randn(T, E, generator=g)
    m_indices = torch.topk(scores, k, dim=1).indices.to(torch.int32)
    return a, b, b1, scores, m_indices


def quantizer_cases(util):
    out = {}
    g = torch.Generator().manual_seed(11)
    # shapes: a multiple of 128, ragged tails, fewer than one group, a zero row/block (amax floor)
    x2 = torch.randn(37, 320, generator=g).to(torch.bfloat16)
    x2[5] = 0
    x2[7, :128] = 0
    x2[9] *= 1e-6  # below the 1e-4 amax floor
    x3 = (torch.randn(3, 200, 144, generator=g) * 0.02).to(torch.bfloat16)
    x3[1, :128, :128] = 0
    out["x2"] = bits(x2)
    out["x3"] = bits(x3)
    q, s = util.per_token_cast_to_fp8(x2)
    out["token_q"], out["token_s"] = bits(q), bits(s)
    q, s = util.per_channel_cast_to_fp8(x3)
    out["channel_q"], out["channel_s"] = bits(q), bits(s)
    q, s = util.per_token_block_cast_to_fp8(x2)
    out["block1x128_q"], out["block1x128_s"] = bits(q), bits(s)
    q, s = util.per_block_cast_to_fp8(x3)
    out["block128_q"], out["block128_s"] = bits(q), bits(s)
    x16 = torch.randn(4, 16, generator=g).to(torch.bfloat16)
    out["x16"] = bits(x16)
    q, s = util.per_token_block_cast_to_fp8(x16)
    out["x16_block_q"], out["x16_block_s"] = bits(q), bits(s)
    return out


def layer_case(util, seed, T, H, I, E, k, act_std, w_std, store_inputs):
    a, b, b1, scores, m_indices = make_inputs(seed, T, H, I, E, k, act_std, w_std)
    out = {"shape": np.array([T, H, I, E, k], dtype=np.int64), "seed": np.array([seed]),
           "std": np.array([act_std, w_std])}
    if store_inputs:
        out.update(a=bits(a), b=bits(b), b1=bits(b1))
    # checksums let the tests detect a drift of the seeded generator
    out["a_sum"] = np.array([a.double().sum().item()])
    out["b_sum"] = np.array([b.double().sum().item()])
    out["b1_sum"] = np.array([b1.double().sum().item()])
    out["m_indices"] = bits(m_indices)
    # bf16 layer: torch_moe_grouped
    ref_d = torch.zeros((T, k, H), dtype=torch.bfloat16)
    util.torch_moe_grouped(a, b, b1, ref_d, m_indices, E)
    out["d_bf16"] = bits(ref_d)
    # block FP8 layer: the reference's generators quantise with these functions
    a_q = util.per_token_block_cast_to_fp8(a)
    b_q = util.per_block_cast_to_fp8(b)
    b1_q = util.per_block_cast_to_fp8(b1)
    d_blk = torch.zeros((T, k, H), dtype=torch.bfloat16)
    util.fp8_blockwise_torch_moe_grouped(a_q, b_q, b1_q, d_blk, m_indices, E)
    out["d_block"] = bits(d_blk)
    out["a_q_sum"] = np.array([a_q[0].float().double().sum().item(), a_q[1].double().sum().item()])
    # per-expert row selection order of torch.where (the stable order of the expert sort)
    order = []
    for e in range(E):
        tok, slot = torch.where(m_indices == e)
        order.append((tok * k + slot).to(torch.int32))
    out["dest_to_src"] = torch.cat(order).numpy()
    return out


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DQMOE_REFERENCE_ROOT", "")
    if not ref_root or not os.path.isdir(ref_root):
        raise SystemExit("usage: make_golden.py <checkout of the reference repository>  (or DQMOE_REFERENCE_ROOT)")
    util = load_reference_util(ref_root)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    np.savez_compressed(os.path.join(HERE, "quantizers.npz"), **quantizer_cases(util))
    # small ragged layer: H and I are not multiples of 128 and the gate/value split (row I of b)
    # falls inside a 128x128 weight-scale block, as in the reference's 2880 shape
    np.savez_compressed(os.path.join(HERE, "layer_small.npz"),
                        **layer_case(util, 21, T=24, H=192, I=160, E=3, k=2, act_std=1.0, w_std=0.05,
                                     store_inputs=True))
    # the CPU-runnable headline configuration: T=64, H=1024, I=2048, E=8, top-2 (inputs from the seed)
    np.savez_compressed(os.path.join(HERE, "layer_c1.npz"),
                        **layer_case(util, 1, T=64, H=1024, I=2048, E=8, k=2, act_std=1.0, w_std=0.02,
                                     store_inputs=False))
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
