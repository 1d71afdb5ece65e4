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


def _untile(tiled, cols, offsets=None):
    """Tiled scale bytes (see dqmoe_mx_tile_scales) back to row-major [rows, cols/32], in numpy: the inverse the
    tests need. offsets [E+1]: expert-sorted rows (blocks by tile); None: rows form blocks by their index."""
    t = np.asarray(tiled.cpu()).reshape(-1)
    kblocks = cols // 128
    if offsets is None:
        rows = t.size // (cols // 32)
        block = np.arange(rows) // 128
        rit = np.arange(rows) % 128
    else:
        offs = np.asarray(offsets.cpu()).astype(np.int64)
        counts = np.diff(offs)
        mt = np.concatenate([[0], np.cumsum((counts + 127) // 128)])
        rows = int(offs[-1])
        e = np.searchsorted(offs, np.arange(rows), side="right") - 1
        local = np.arange(rows) - offs[e]
        block, rit = mt[e] + local // 128, local % 128
    base = block * kblocks * 512 + (rit % 32) * 16 + (rit // 32) * 4
    g = np.arange(cols // 32)
    idx = base[:, None] + (g // 4)[None, :] * 512 + (g % 4)[None, :]
    return torch.from_numpy(t[idx].astype(np.uint8))


def test_mx_tiled_scale_layout_round_trip(ops):
    g = torch.Generator().manual_seed(4)
    s = torch.randint(0, 255, (3 * 256, 512 // 32), generator=g, dtype=torch.uint8)
    tiled = ops.mx_tile_scales(s.to(DEV), 512)
    assert tiled.numel() == s.numel()
    assert torch.equal(_untile(tiled, 512), s)
    # block 0, K block 0: row r at byte (r % 32) * 16 + (r // 32) * 4
    t = tiled.cpu()
    assert t[0] == s[0, 0] and t[4] == s[32, 0] and t[16] == s[1, 0] and t[17] == s[1, 1] and t[512 + 3] == s[0, 7]
    # expert-sorted rows: ragged experts start new blocks
    counts = [5, 0, 130, 128, 1]
    offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
    n = int(offs[-1])
    rows = torch.randint(0, 255, (n, 256 // 32), generator=g, dtype=torch.uint8)
    tiled = ops.mx_tile_scales(rows.to(DEV), 256, offsets=offs, mtile_pref=ops.mtile_prefix(offs))
    assert tiled.numel() >= (1 + 0 + 2 + 1 + 1) * 2 * 512
    assert torch.equal(_untile(tiled, 256, offs), rows)


def test_mx_permute_quant_fused_equals_quant_then_permute(ops):
    T, H, k, E = 300, 1024, 3, 8
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    idx = torch.topk(torch.randn(T, E, generator=g), k, dim=1).indices.to(torch.int32)
    idx[7, 1] = -1
    _, offsets, d2s, _ = ops.route_sort(idx.to(DEV), E)
    mt = ops.mtile_prefix(offsets)
    q, s = ops.mx_cast_to_fp8(x)
    fq, fs = ops.moe_permute_quant_mx(x, d2s, k, offsets, mt)
    kept = int((d2s >= 0).sum())
    src = (d2s[:kept] // k).long()
    assert torch.equal(fq[:kept].view(torch.uint8), q[src].view(torch.uint8))
    assert torch.equal(_untile(fs, H, offsets), s[src].cpu())
    # the unfused path gives the same tiled bytes for the kept rows
    gathered = ops.mx_tile_scales(s, H, offsets=offsets, mtile_pref=mt, dest_to_src=d2s, k=k)
    assert torch.equal(_untile(gathered, H, offsets), s[src].cpu())


def _groups(counts):
    offs = np.zeros(len(counts) + 1, dtype=np.int32)
    offs[1:] = np.cumsum(counts)
    return offs


RAGGED = [0, 1, 127, 128, 129, 300, 0, 5]
LARGE = [700, 64, 1500, 3]
def _device_inputs(ops, q, H, I):
    """Oracle-quantised layer inputs on the device, weight scales converted to the tiled layout the layer takes."""
    aq, as_, bq, bs, b1q, b1s = [t.to(DEV).contiguous() for t in q]
    return [aq, as_, bq, ops.mx_tile_scales(bs, H), b1q, ops.mx_tile_scales(b1s, I)]


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
    asf_t = ops.mx_tile_scales(asf.to(DEV), K, offsets=offsets, mtile_pref=mt)
    wsf_t = ops.mx_tile_scales(wsf.to(DEV), K)
    if gated:
        out = torch.zeros(n, N, dtype=torch.uint8, device=DEV)
        out_sf = torch.zeros(asf_t.numel() // K * N + 512, dtype=torch.uint8, device=DEV)
        ops.grouped_gemm_mx(aq.to(DEV), asf_t, wq.to(DEV), wsf_t, offsets, mt, N, True, out, out_sf)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        got = orc.dequant_mx(out.cpu().view(torch.float8_e4m3fn), _untile(out_sf, N, offsets))
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
        ops.grouped_gemm_mx(aq.to(DEV), asf_t, wq.to(DEV), wsf_t, offsets, mt, N, False, out)
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
    qd = _device_inputs(ops, q, H, I)
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
    qd = _device_inputs(ops, q, H, I)
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
    out = ops.moe_block(a.to(DEV), logits.to(DEV), bq.to(DEV), ops.mx_tile_scales(bs.to(DEV), H), b1q.to(DEV),
                        ops.mx_tile_scales(b1s.to(DEV), I), k, "softmax", MX)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert orc.cosine(out.cpu(), ref) >= COS_MIN and orc.max_rel_err(out.cpu(), ref) <= REL_MAX


def test_mx_through_the_drop_in_module_and_the_plugin_front_end(ops):
    """quant_mode_value 2048 through moe_test.m_grouped_moe_nt_contiguous_fp8_bf16 (scale halves of the tuples hold
    UE8M0 bytes) and through the plugin-shaped entry points with HALF output."""
    import moe_test
    from dqmoe_b200 import plugin
    E, T, H, I, k = 8, 96, 512, 384, 2
    a, b, b1, _, idx = make_inputs(21, T, H, I, E, k, 1.0, 0.05)
    q = orc.quantize_inputs(a, b, b1, MX)
    ref = orc.moe_layer_fp8(*q, idx, E, MX)
    aq, as_, bq, bs, b1q, b1s = _device_inputs(ops, q, H, I)
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, MX) + 256, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    moe_test.m_grouped_moe_nt_contiguous_fp8_bf16((aq, as_), (bq, bs), (b1q, b1s), d, idx.to(DEV), ws, MX)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert orc.cosine(d.cpu(), ref) >= COS_MIN and orc.max_rel_err(d.cpu(), ref) <= REL_MAX
    with pytest.raises(RuntimeError, match="ASSERT FAILED"):  # fp32 scale tensors in the byte-scaled mode
        moe_test.m_grouped_moe_nt_contiguous_fp8_bf16((aq, as_.float()), (bq, bs), (b1q, b1s), d, idx.to(DEV), ws, MX)
    p = plugin.MoePlugin(E, k, H, I, max_num_tokens=128, type=plugin.DT_FP8, output_type=plugin.DT_HALF, quant_mode=MX)
    out = p.enqueue([aq, bq, b1q, idx.to(DEV), None, None, as_, bs, b1s])
    torch.cuda.synchronize()
    assert out.dtype == torch.float16 and torch.equal(out.float(), d.float())
    with pytest.raises(RuntimeError, match="multiples of 128 in the MXFP8 mode"):
        plugin.MoePlugin(E, k, 160, I, 128, type=plugin.DT_FP8, quant_mode=MX)


def test_mx_mode_rejects_shapes_it_cannot_tile(ops):
    E, T, H, I, k = 2, 8, 160, 128, 1
    a, b, b1, _, idx = make_inputs(15, T, H, I, E, k)
    q = [t.to(DEV).contiguous() for t in orc.quantize_inputs(a, b, b1, MX)]  # (rejected before any scale is read)
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
    bq, bs_rows = ops.mx_cast_to_fp8(b)
    bs = ops.mx_tile_scales(bs_rows, H)
    del b
    b1 = (torch.randn(E, H, I, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    b1q, b1s_rows = ops.mx_cast_to_fp8(b1)
    b1s = ops.mx_tile_scales(b1s_rows, I)
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
    ref = orc.moe_layer_fp8(aq[srows].cpu(), as_[srows].cpu(), bq.cpu(), bs_rows.cpu(), b1q.cpu(), b1s_rows.cpu(),
                            idx[srows].cpu(), E, MX)
    got = d[srows].cpu()
    assert orc.cosine(got, ref) >= COS_MIN and orc.max_rel_err(got, ref) <= REL_MAX
