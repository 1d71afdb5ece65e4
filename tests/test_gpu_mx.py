"""The MXFP8 mode (e4m3 with one UE8M0 power-of-two scale per 32 elements; block-scaled tensor-core instruction)
against the oracle: quantisers bit for bit, the grouped GEMM and the layer within the layer tolerance. The format
has no counterpart in the reference, so the oracle functions used here are marked "parity unpinned"."""
import numpy as np
import pytest
import torch

from helpers import bits, make_inputs
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, REL_MAX = 0.999, 2e-2  # the layer tolerance: cosine and max|x - ref| / max|ref|
MX = 2048


@pytest.fixture(scope="module")
def ops():
    from dqmoe_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("rows,cols,std", [(1, 32, 1.0), (513, 4096, 1.0), (64, 2880 + 32, 0.05), (7, 160, 30.0), (2048, 7168, 1.0)])
def test_mx_quantiser_bit_exact_vs_oracle(ops, rows, cols, std):
    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=g) * std).to(torch.bfloat16)
    x[0, :32] = 0                      # an all-zero group: the amax floor decides its scale
    if rows > 2:
        x[1, 0] = 448.0                # exactly at the top of the e4m3 range: scale 1
        x[2, 5] = 2.0 ** -20
    q_ref, s_ref = orc.quant_mx(x)
    q, s = ops.mx_cast_to_fp8(x.to(DEV))
    assert np.array_equal(bits(s), s_ref.numpy())
    assert np.array_equal(bits(q), bits(q_ref))


def test_mx_quantiser_on_weight_shaped_tensors(ops):
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(3, 200, 256, generator=g) * 0.02).to(torch.bfloat16)
    q_ref, s_ref = orc.quant_mx(w)
    q, s = ops.mx_cast_to_fp8(w.to(DEV))
    assert s.shape == (3, 200, 8)
    assert np.array_equal(bits(s), s_ref.numpy()) and np.array_equal(bits(q), bits(q_ref))


def test_mx_permute_quant_fused_equals_quant_then_permute(ops):
    T, H, k, E = 300, 1024, 3, 8
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    idx = torch.topk(torch.randn(T, E, generator=g), k, dim=1).indices.to(torch.int32)
    idx[7, 1] = -1
    _, _, d2s, _ = ops.route_sort(idx.to(DEV), E)
    q, s = ops.mx_cast_to_fp8(x)
    fq, fs = ops.moe_permute_quant_mx(x, d2s, k)
    kept = int((d2s >= 0).sum())
    src = (d2s[:kept] // k).long()
    assert torch.equal(fq[:kept].view(torch.uint8), q[src].view(torch.uint8))
    assert torch.equal(fs[:kept], s[src])


def _groups(counts):
    offs = np.zeros(len(counts) + 1, dtype=np.int32)
    offs[1:] = np.cumsum(counts)
    return offs


RAGGED = [0, 1, 127, 128, 129, 300, 0, 5]
LARGE = [700, 64, 1500, 3]
@pytest.mark.parametrize("counts,N,K", [(RAGGED, 384, 640), (LARGE, 512, 1024), ([40] * 40, 1280, 256)], ids=["ragged", "large", "many"])
@pytest.mark.parametrize("gated", [False, True])
def test_grouped_gemm_mx_ragged_groups(ops, gated, counts, N, K):
    E, n = len(counts), int(sum(counts))
    offs = _groups(counts)
    g = torch.Generator().manual_seed(11)
    a = torch.randn(n, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, 2 * N if gated else N, K, generator=g) * 0.05).to(torch.bfloat16)
    aq, asf = orc.quant_mx(a)
    wq, wsf = orc.quant_mx(w)
    offsets = torch.from_numpy(offs).to(DEV)
    mt = ops.mtile_prefix(offsets)
    da, dw = orc.dequant_mx(aq, asf), orc.dequant_mx(wq, wsf)
    if gated:
        out = torch.zeros(n, N, dtype=torch.uint8, device=DEV)
        out_sf = torch.zeros(n, N // 32, dtype=torch.uint8, device=DEV)
        ops.grouped_gemm_mx(aq.to(DEV), asf.to(DEV), wq.to(DEV), wsf.to(DEV), offsets, mt, N, True, out, out_sf)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        got = orc.dequant_mx(out.cpu().view(torch.float8_e4m3fn), out_sf.cpu())
        ref = torch.zeros(n, N)
        for e in range(E):
            lo, hi = offs[e], offs[e + 1]
            if hi > lo:
                inter = torch.nn.functional.linear(da[lo:hi], dw[e]).to(torch.bfloat16)
                gate, value = inter.chunk(2, dim=-1)
                act = torch.nn.functional.silu(gate) * value
                ref[lo:hi] = orc.dequant_mx(*orc.quant_mx(act))
    else:
        out = torch.zeros(n, N, dtype=torch.bfloat16, device=DEV)
        ops.grouped_gemm_mx(aq.to(DEV), asf.to(DEV), wq.to(DEV), wsf.to(DEV), offsets, mt, N, False, out)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        got = out.cpu().float()
        ref = torch.zeros(n, N)
        for e in range(E):
            lo, hi = offs[e], offs[e + 1]
            if hi > lo:
                ref[lo:hi] = torch.nn.functional.linear(da[lo:hi], dw[e]).to(torch.bfloat16).float()
    assert orc.cosine(got, ref) >= 0.9999, orc.cosine(got, ref)
    assert orc.max_rel_err(got, ref) <= (REL_MAX if gated else 5e-3), orc.max_rel_err(got, ref)


SHAPES = [(8, 96, 512, 384, 2), (4, 700, 384, 640, 2), (8, 64, 1024, 2048, 2), (3, 5, 256, 128, 2), (2, 3000, 512, 1024, 2),
          (1, 1, 128, 128, 1)]
@pytest.mark.parametrize("E,T,H,I,k", SHAPES)
def test_layer_mx_matches_oracle(ops, E, T, H, I, k):
    a, b, b1, _, idx = make_inputs(7, T, H, I, E, k, 1.0, 0.05)
    if T > 10:
        idx[3, 0] = -1   # a dropped row
    q = orc.quantize_inputs(a, b, b1, MX)
    ref = orc.moe_layer_fp8(*q, idx, E, MX)
    qd = [t.to(DEV).contiguous() for t in q]
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, MX) + 256, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward(*qd, d, idx.to(DEV), ws, MX)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = d.cpu()
    assert orc.cosine(got, ref) >= COS_MIN, orc.cosine(got, ref)
    assert orc.max_rel_err(got, ref) <= REL_MAX, orc.max_rel_err(got, ref)
    if T > 10:
        assert torch.count_nonzero(got[3, 0]) == 0
    # deterministic
    d2 = torch.zeros_like(d)
    ops.moe_forward(*qd, d2, idx.to(DEV), ws, MX)
    assert torch.equal(d, d2)


def test_layer_mx_with_biases(ops):
    E, T, H, I, k = 4, 300, 384, 640, 2
    a, b, b1, _, idx = make_inputs(9, T, H, I, E, k, 1.0, 0.05)
    g = torch.Generator().manual_seed(1)
    bias1, bias2 = torch.randn(E, 2 * I, generator=g) * 0.5, torch.randn(E, H, generator=g) * 0.5
    q = orc.quantize_inputs(a, b, b1, MX)
    ref = orc.moe_layer_fp8(*q, idx, E, MX, bias1=bias1, bias2=bias2)
    qd = [t.to(DEV).contiguous() for t in q]
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, MX) + 256, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward(*qd, d, idx.to(DEV), ws, MX, bias1=bias1.to(DEV), bias2=bias2.to(DEV))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert orc.cosine(d.cpu(), ref) >= COS_MIN and orc.max_rel_err(d.cpu(), ref) <= REL_MAX


def test_moe_block_mx(ops):
    E, T, H, I, k = 8, 200, 512, 384, 2
    a, b, b1, logits, _ = make_inputs(13, T, H, I, E, k, 1.0, 0.05)
    bq, bs = orc.quant_mx(b)
    b1q, b1s = orc.quant_mx(b1)
    ref = orc.moe_block(a, logits, b, b1, k, "softmax", MX, quantized=(*orc.quant_mx(a), bq, bs, b1q, b1s))
    out = ops.moe_block(a.to(DEV), logits.to(DEV), bq.to(DEV), bs.to(DEV), b1q.to(DEV), b1s.to(DEV), k, "softmax", MX)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert orc.cosine(out.cpu(), ref) >= COS_MIN and orc.max_rel_err(out.cpu(), ref) <= REL_MAX


def test_mx_mode_rejects_shapes_it_cannot_tile(ops):
    E, T, H, I, k = 2, 8, 160, 128, 1
    a, b, b1, _, idx = make_inputs(15, T, H, I, E, k)
    q = [t.to(DEV).contiguous() for t in orc.quantize_inputs(a, b, b1, MX)]
    ws = torch.empty(1 << 20, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="multiples of 128 in the MXFP8 mode"):
        ops.moe_forward(*q, d, idx.to(DEV), ws, MX)


def test_mixtral_shape_mx_full_size_sample(ops):
    """T=4096, H=4096, I=14336, E=8, top-2 in the MXFP8 mode: a sample of tokens against the oracle at full H and I,
    and the same sample as a small batch bit for bit."""
    T, H, I, E, k = 4096, 4096, 14336, 8, 2
    g = torch.Generator(device=DEV).manual_seed(77)
    x = torch.randn(T, H, generator=g, device=DEV).to(torch.bfloat16)
    idx, _ = ops.route_topk(torch.randn(T, E, generator=g, device=DEV), k, "softmax")
    b = (torch.randn(E, 2 * I, H, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    bq, bs = ops.mx_cast_to_fp8(b)
    del b
    b1 = (torch.randn(E, H, I, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    b1q, b1s = ops.mx_cast_to_fp8(b1)
    del b1
    aq, as_ = ops.mx_cast_to_fp8(x)
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, MX), dtype=torch.uint8, device=DEV)
    d = torch.empty(T, k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward(aq, as_, bq, bs, b1q, b1s, d, idx, ws, MX)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.isfinite(d.float()).all() and (d.float().abs().amax(dim=2) > 0).all()
    rows = torch.arange(3, T, 17, device=DEV)[:200]
    small = torch.empty(rows.numel(), k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward(aq[rows].contiguous(), as_[rows].contiguous(), bq, bs, b1q, b1s, small, idx[rows].contiguous(), ws, MX)
    assert torch.equal(small, d[rows])
    srows = torch.arange(5, T, 127, device=DEV)[:16]
    ref = orc.moe_layer_fp8(aq[srows].cpu(), as_[srows].cpu(), bq.cpu(), bs.cpu(), b1q.cpu(), b1s.cpu(), idx[srows].cpu(), E, MX)
    got = d[srows].cpu()
    assert orc.cosine(got, ref) >= COS_MIN and orc.max_rel_err(got, ref) <= REL_MAX
