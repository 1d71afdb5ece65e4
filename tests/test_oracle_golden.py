"""The CPU oracle against the golden vectors produced by the reference's own torch code
(tests/golden/make_golden.py). Bit-exact: these pin the oracle before it checks any kernel."""
import numpy as np
import torch

from helpers import bf16_from_bits, bits, golden, make_inputs
from oracle import moe_oracle as orc


def test_quantizers_bit_exact():
    g = golden("quantizers.npz")
    x2 = bf16_from_bits(g["x2"])
    x3 = bf16_from_bits(g["x3"])
    x16 = bf16_from_bits(g["x16"])
    for fn, x, key in (
        (orc.quant_rowwise, x2, "token"),
        (orc.quant_rowwise, x3, "channel"),
        (orc.quant_block_1x128, x2, "block1x128"),
        (orc.quant_block_128x128, x3, "block128"),
        (orc.quant_block_1x128, x16, "x16_block"),
    ):
        q, s = fn(x)
        assert np.array_equal(bits(q), g[key + "_q"]), key
        assert np.array_equal(bits(s), g[key + "_s"]), key


def _layer_inputs(g):
    T, H, I, E, k = (int(v) for v in g["shape"])
    act_std, w_std = (float(v) for v in g["std"])
    a, b, b1, _, m_indices = make_inputs(int(g["seed"][0]), T, H, I, E, k, act_std, w_std)
    # the seeded generator must reproduce what the fixture was made from
    assert a.double().sum().item() == g["a_sum"][0]
    assert b.double().sum().item() == g["b_sum"][0]
    assert b1.double().sum().item() == g["b1_sum"][0]
    assert np.array_equal(bits(m_indices), g["m_indices"])
    if "a" in g:
        assert np.array_equal(bits(a), g["a"]) and np.array_equal(bits(b), g["b"]) and np.array_equal(bits(b1), g["b1"])
    return a, b, b1, m_indices, E


def _check_layer(name):
    g = golden(name)
    a, b, b1, m_indices, E = _layer_inputs(g)
    d = orc.moe_layer_bf16(a, b, b1, m_indices, E)
    assert np.array_equal(bits(d), g["d_bf16"])
    qs = orc.quantize_inputs(a, b, b1, orc.QUANT_BLOCK)
    assert qs[0].float().double().sum().item() == g["a_q_sum"][0]
    assert qs[1].double().sum().item() == g["a_q_sum"][1]
    d_blk = orc.moe_layer_fp8(*qs, m_indices, E, orc.QUANT_BLOCK)
    assert np.array_equal(bits(d_blk), g["d_block"])
    _, _, d2s, s2d = orc.route_sort(m_indices, E)
    assert np.array_equal(d2s.numpy(), g["dest_to_src"])
    n = m_indices.numel()
    assert np.array_equal(s2d.numpy()[d2s.numpy()], np.arange(n))


def test_layer_small_bit_exact():
    _check_layer("layer_small.npz")


def test_layer_c1_bit_exact():
    _check_layer("layer_c1.npz")


def test_route_sort_drops_out_of_range_ids():
    m = torch.tensor([[0, 5], [2, -1], [2, 0], [7, 1]], dtype=torch.int32)
    counts, offsets, d2s, s2d = orc.route_sort(m, 3)
    assert counts.tolist() == [2, 1, 2]
    assert offsets.tolist() == [0, 2, 3, 5]
    assert d2s.tolist() == [0, 5, 7, 2, 4, -1, -1, -1]
    assert s2d.tolist() == [0, -1, 3, -1, 4, 1, -1, 2]


def test_router_matches_torch_topk_without_ties():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(50, 64, generator=g)
    idx, w = orc.route_topk(logits, 6, "softmax")
    ref_w, ref_idx = torch.topk(torch.softmax(logits, dim=1), 6, dim=1)
    assert torch.equal(idx.long(), ref_idx)
    torch.testing.assert_close(w, ref_w / ref_w.sum(1, keepdim=True), rtol=1e-5, atol=1e-7)
    idx, w = orc.route_topk(logits, 8, "sigmoid")
    ref_w, ref_idx = torch.topk(torch.sigmoid(logits), 8, dim=1)
    assert torch.equal(idx.long(), ref_idx)
    torch.testing.assert_close(w, ref_w / ref_w.sum(1, keepdim=True), rtol=1e-5, atol=1e-7)


def test_fp8_layers_track_the_bf16_layer():
    # the three FP8-simulating layers stay close to the unquantised layer on the same inputs
    a, b, b1, _, m_indices = make_inputs(5, 16, 256, 128, 4, 2, 1.0, 0.05)
    ref = orc.moe_layer_bf16(a, b, b1, m_indices, 4)
    for mode in (orc.QUANT_TENSOR, orc.QUANT_CHANNEL, orc.QUANT_BLOCK):
        d = orc.moe_layer_fp8(*orc.quantize_inputs(a, b, b1, mode), m_indices, 4, mode)
        assert orc.cosine(d, ref) > 0.99, mode


def test_block_with_shared_experts_is_routed_block_plus_dense_expert():
    """moe_block(n_shared=1): the appended expert sees every token with weight 1, i.e. the result is the routed
    block's fp32 sum plus that expert applied densely (one rounding to bf16 at the end)."""
    E, T, H, I, k = 4, 12, 128, 128, 2
    a, b, b1, _, _ = make_inputs(3, T, H, I, E + 1, k, 1.0, 0.05)
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(1))
    idx, w = orc.route_topk(logits, k, "softmax")
    d_routed = orc.moe_layer_bf16(a, b[:E], b1[:E], idx, E)                       # [T, k, H]
    everyone = torch.zeros(T, 1, dtype=torch.int32)
    d_shared = orc.moe_layer_bf16(a, b[E:], b1[E:], everyone, 1)                  # [T, 1, H]
    want = orc.finalize_weighted(torch.cat([d_routed, d_shared], dim=1),
                                 torch.cat([w, torch.ones(T, 1)], dim=1))
    got = orc.moe_block(a, logits, b, b1, k, "softmax", 0, n_shared=1)
    assert torch.equal(got, want)
    assert not torch.equal(got, orc.moe_block(a, logits, b[:E], b1[:E], k, "softmax", 0))
