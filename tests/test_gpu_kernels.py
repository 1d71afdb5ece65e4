"""GPU parity of the streaming kernels against the CPU oracle (bit-exact: indices, maps,
FP8 bytes and scales), through the C ABI."""
import numpy as np
import pytest
import torch

from helpers import bf16_from_bits, bits, golden
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from dqmoe_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("T,k,E", [(1, 1, 1), (5, 2, 3), (300, 3, 8), (1024, 2, 8), (1025, 2, 8), (4096, 2, 8),
                                   (8192, 8, 256), (16384, 8, 128), (3000, 4, 1000), (35456, 1, 4)])
def test_route_sort_bit_exact(ops, T, k, E):
    g = torch.Generator().manual_seed(T * 31 + E)
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    if T > 4:  # out-of-range ids are dropped
        ids[1, 0] = -1
        ids[3, k - 1] = E + 5
    got = ops.route_sort(ids.to(DEV), E)
    want = orc.route_sort(ids, E)
    for name, a, b in zip(("counts", "offsets", "dest_to_src", "src_to_dest"), got, want):
        assert torch.equal(a.cpu(), b), name
    assert ops.device_status() == 0


def test_route_sort_skewed_and_empty_experts(ops):
    ids = torch.zeros(5000, 2, dtype=torch.int32)  # every row to expert 0, experts 1..6 empty
    ids[:, 1] = 7
    got = ops.route_sort(ids.to(DEV), 8)
    want = orc.route_sort(ids, 8)
    for a, b in zip(got, want):
        assert torch.equal(a.cpu(), b)


@pytest.mark.parametrize("E,k,scoring", [(8, 2, "softmax"), (256, 8, "sigmoid"), (128, 8, "softmax"),
                                         (64, 6, "softmax"), (1000, 6, "sigmoid"), (3, 3, "softmax")])
def test_route_topk(ops, E, k, scoring):
    g = torch.Generator().manual_seed(E + k)
    logits = torch.randn(777, E, generator=g)
    idx, w = ops.route_topk(logits.to(DEV), k, scoring)
    ref_idx, ref_w = orc.route_topk(logits, k, scoring)
    assert torch.equal(idx.cpu(), ref_idx)  # fp32 logits: ties have measure zero
    torch.testing.assert_close(w.cpu(), ref_w, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(w.sum(1).cpu(), torch.ones(777), rtol=1e-5, atol=1e-6)


def test_route_topk_ties_prefer_lower_expert_id(ops):
    logits = torch.zeros(4, 16)
    logits[:, 9] = 1.0
    idx, w = ops.route_topk(logits.to(DEV), 3, "softmax")
    assert idx.cpu().tolist() == [[9, 0, 1]] * 4


def test_quantizers_match_reference_golden_vectors(ops):
    g = golden("quantizers.npz")
    x2 = bf16_from_bits(g["x2"]).to(DEV)
    x3 = bf16_from_bits(g["x3"]).to(DEV)
    x16 = bf16_from_bits(g["x16"]).to(DEV)
    for fn, x, key in ((ops.per_token_cast_to_fp8, x2, "token"), (ops.per_channel_cast_to_fp8, x3, "channel"),
                       (ops.per_token_block_cast_to_fp8, x2, "block1x128"), (ops.per_block_cast_to_fp8, x3, "block128"),
                       (ops.per_token_block_cast_to_fp8, x16, "x16_block")):
        q, s = fn(x)
        assert np.array_equal(bits(q), g[key + "_q"]), key
        assert np.array_equal(bits(s), g[key + "_s"]), key


@pytest.mark.parametrize("rows,cols", [(1, 16), (513, 4096), (64, 2880), (7, 136), (2048, 7168)])
def test_quantizers_bit_exact_vs_oracle(ops, rows, cols):
    g = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=g).to(torch.bfloat16)
    x[0, : min(cols, 128)] = 0
    for fn, ofn in ((ops.per_token_cast_to_fp8, orc.quant_rowwise), (ops.per_token_block_cast_to_fp8, orc.quant_block_1x128),
                    (ops.per_block_cast_to_fp8, orc.quant_block_128x128), (ops.per_tensor_cast_to_fp8, orc.quant_tensor)):
        q, s = fn(x.to(DEV))
        rq, rs = ofn(x)
        assert np.array_equal(bits(q).reshape(-1), bits(rq).reshape(-1)), fn.__name__
        assert np.array_equal(bits(s).reshape(-1), bits(rs).reshape(-1)), fn.__name__


def test_quantize_weights_per_expert_and_channel(ops):
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(3, 200, 144, generator=g) * 0.02).to(torch.bfloat16)
    for fn, ofn in ((ops.per_channel_cast_to_fp8, orc.quant_rowwise), (ops.per_block_cast_to_fp8, orc.quant_block_128x128),
                    (lambda t: ops.per_tensor_cast_to_fp8(t, per_expert=True), lambda t: orc.quant_tensor(t, per_expert=True))):
        q, s = fn(w.to(DEV))
        rq, rs = ofn(w)
        assert np.array_equal(bits(q), bits(rq))
        assert np.array_equal(bits(s).reshape(-1), bits(rs).reshape(-1))


@pytest.mark.parametrize("T,H,k,E,dtype", [(100, 256, 2, 8, torch.bfloat16), (1, 16, 1, 1, torch.bfloat16),
                                           (777, 2880, 3, 64, torch.float8_e4m3fn), (4096, 4096, 2, 8, torch.float8_e4m3fn)])
def test_permute_scatter_round_trip(ops, T, H, k, E, dtype):
    g = torch.Generator().manual_seed(T + H)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    a = torch.randn(T, H, generator=g).to(torch.bfloat16)
    if dtype != torch.bfloat16:
        a = a.to(dtype)
    scale = torch.rand(T, (H + 127) // 128, generator=g)
    _, _, d2s, _ = ops.route_sort(ids.to(DEV), E)
    p, ps = ops.moe_permute(a.to(DEV), d2s, k, scale.to(DEV))
    assert np.array_equal(bits(p), bits(orc.permute_rows(a, d2s.cpu(), k)))
    assert torch.equal(ps.cpu(), orc.permute_rows(scale, d2s.cpu(), k))
    # gather then scatter puts every token's row into each of its k slots
    d = torch.zeros(T * k, H, dtype=dtype, device=DEV) if dtype == torch.bfloat16 else torch.zeros(T * k, H, dtype=torch.uint8, device=DEV).view(dtype)
    ops.finalize_scatter(p, d2s, d)
    assert np.array_equal(bits(d).reshape(T, k, H), np.broadcast_to(bits(a)[:, None, :], (T, k, H)))


def test_permute_quant_fused_equals_quant_then_permute(ops):
    g = torch.Generator().manual_seed(9)
    T, H, k, E = 333, 2880, 3, 16
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    _, _, d2s, _ = ops.route_sort(ids.to(DEV), E)
    q, s = ops.moe_permute_quant_block(x.to(DEV), d2s, k)
    rq, rs = orc.quant_block_1x128(orc.permute_rows(x, d2s.cpu(), k))
    assert np.array_equal(bits(q), bits(rq)) and np.array_equal(bits(s), bits(rs))


def test_finalize_weighted(ops):
    g = torch.Generator().manual_seed(2)
    d = torch.randn(257, 8, 2048, generator=g).to(torch.bfloat16)
    w = torch.rand(257, 8, generator=g)
    w[3, 2] = 0.0
    out = ops.finalize_weighted(d.to(DEV), w.to(DEV))
    ref = orc.finalize_weighted(d, w)
    # fp32 accumulation in the same slot order: results agree to one bf16 rounding
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1e-2, atol=1e-3)
    assert (out.cpu() != ref).float().mean().item() < 0.01


@pytest.mark.parametrize("rows,cols", [(1, 8), (37, 24), (300, 768), (64, 2880), (1025, 1000)])
def test_requant_from_amax_bit_exact(ops, rows, cols):
    """The second pass of the tensor / channel modes (dqmoe_requant_from_amax): with the amax that stage 1
    collects, its bytes and scales equal the oracle's row-wise and per-tensor quantisers."""
    x = (torch.randn(rows, cols, generator=torch.Generator().manual_seed(rows + cols)) * 3).to(torch.bfloat16)
    x[0, 0] = 0.0
    if rows > 2:
        x[2] = 0.0  # an all-zero row: scale 1e-4 / 448
    xd = x.to(DEV)
    q, s = ops.requant_from_amax(xd, xd.abs().float().amax(dim=1).contiguous(), per_row=True)
    rq, rs = orc.quant_rowwise(x)
    assert np.array_equal(bits(q), bits(rq))
    assert torch.equal(s.cpu(), rs.reshape(-1))
    q, s = ops.requant_from_amax(xd, xd.abs().float().amax().reshape(1), per_row=False)
    rq, rs = orc.quant_tensor(x)
    assert np.array_equal(bits(q), bits(rq))
    assert torch.equal(s.cpu(), rs.reshape(-1))


def test_requant_row_count_read_on_the_device(ops):
    """dqmoe_requant_from_amax_dev: only the first *n_rows_device rows are quantised (an expert-parallel rank
    learns how many rows it received on the device only); the rest of the output is left alone."""
    rows, cols, live = 200, 256, 77
    x = (torch.randn(rows, cols, generator=torch.Generator().manual_seed(3)) * 2).to(torch.bfloat16)
    xd = x.to(DEV)
    q = torch.full((rows, cols), 0x7b, dtype=torch.uint8, device=DEV).view(torch.float8_e4m3fn)
    s = torch.full((rows,), -1.0, device=DEV)
    count = torch.tensor([live], dtype=torch.int32, device=DEV)
    ops.requant_from_amax(xd, xd.abs().float().amax(dim=1).contiguous(), True, n_rows_device=count, out=(q, s))
    rq, rs = orc.quant_rowwise(x)
    assert np.array_equal(bits(q[:live]), bits(rq[:live]))
    assert torch.equal(s[:live].cpu(), rs.reshape(-1)[:live])
    assert (q[live:].view(torch.uint8) == 0x7b).all() and (s[live:] == -1.0).all()
