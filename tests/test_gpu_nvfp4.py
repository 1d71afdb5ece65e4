"""The NVFP4 mode (e2m1 pairs with one UE4M3 scale per 16 elements and an fp32 global scale; block-scaled tensor-core
instruction kind::mxf4nvf4) against the oracle: the quantiser bit for bit, the grouped GEMM and the layer within
the layer tolerance. The reference names the format without code for it, so the oracle functions used here are
marked "parity unpinned"."""
import numpy as np
import pytest
import torch

from helpers import make_inputs
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, REL_MAX = 0.999, 2e-2  # the layer tolerance: cosine and max|x - ref| / max|ref|


@pytest.fixture(scope="module")
def ops():
    from dqmoe_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("rows,cols,std", [(1, 16, 1.0), (7, 64, 1.0), (300, 512, 0.02), (129, 2048, 30.0)])
def test_nvfp4_quantiser_bit_exact_vs_oracle(ops, rows, cols, std):
    g = torch.Generator().manual_seed(rows * 1000 + cols)
    x = (torch.randn(rows, cols, generator=g) * std).to(torch.bfloat16)
    x[0, :16] = 0                      # an all-zero group: scale byte 0, zero nibbles
    if rows > 2:
        x[1, 3] = 1000.0 * std         # an outlier that sets the global scale: other groups get tiny scale bytes
        x[2, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, 6.0, 7.0, -7.0, 0.5, 1.0, 1.5, 3.0]) * std
    gs = orc.nvfp4_global_scale(x)
    q_ref, s_ref = orc.quant_nvfp4(x, gs)
    q, s = ops.nvfp4_cast(x.to(DEV), gs.to(DEV))
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu(), q_ref)


def test_nvfp4_quantiser_per_expert_global_scales(ops):
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(3, 128, 256, generator=g) * torch.tensor([0.02, 1.0, 40.0]).view(3, 1, 1)).to(torch.bfloat16)
    gs = torch.cat([orc.nvfp4_global_scale(w[e]) for e in range(3)])
    q_ref, s_ref = orc.quant_nvfp4(w, gs)
    q, s = ops.nvfp4_cast(w.to(DEV), gs.to(DEV))
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    q2, s_tiled, g2 = ops.nvfp4_cast_weights(w.to(DEV))   # computes the global scales itself
    assert torch.allclose(g2.cpu(), gs, rtol=1e-6)
    q_ref, s_ref = orc.quant_nvfp4(w, g2.cpu())
    assert torch.equal(q2.cpu(), q_ref)
    # tiled layout: block [row block][64-column block], row r at (r % 32) * 16 + (r / 32) * 4, four bytes in column order
    t = s_tiled.cpu().numpy().reshape(3, 256 // 64, 32, 4, 4)   # [row block = expert (128 rows each), K block, r % 32, r / 32, byte]
    back = t.transpose(0, 3, 2, 1, 4).reshape(3, 128, 256 // 16)
    assert np.array_equal(back, s_ref.numpy())


def _groups(counts):
    offs = np.zeros(len(counts) + 1, dtype=np.int32)
    offs[1:] = np.cumsum(counts)
    return offs


def _mtile_prefix(offs):
    counts = np.diff(offs)
    mt = np.zeros(len(offs), dtype=np.int32)
    mt[1:] = np.cumsum((counts + 127) // 128)
    return mt


RAGGED = [0, 1, 127, 128, 129, 300, 0, 5]


@pytest.mark.parametrize("counts,N,K", [(RAGGED, 384, 512), ([700, 64, 1500, 3], 512, 1024), ([40] * 24, 1280, 256)],
                         ids=["ragged", "large", "many"])
@pytest.mark.parametrize("gated", [False, True])
def test_grouped_gemm_nvfp4_ragged_groups(ops, gated, counts, N, K):
    E = len(counts)
    offs = _groups(counts)
    n = int(offs[-1])
    g = torch.Generator().manual_seed(n + N + K + int(gated))
    a = torch.randn(n, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, (2 if gated else 1) * N, K, generator=g) * 0.05).to(torch.bfloat16)
    a_g = orc.nvfp4_global_scale(a)
    w_g = torch.cat([orc.nvfp4_global_scale(w[e]) for e in range(E)])
    a_q, a_s = orc.quant_nvfp4(a, a_g)
    w_q, w_s = orc.quant_nvfp4(w, w_g)
    a_f, w_f = orc.dequant_nvfp4(a_q, a_s, a_g), orc.dequant_nvfp4(w_q, w_s, w_g)
    offs_t, mt_t = torch.from_numpy(offs).to(DEV), torch.from_numpy(_mtile_prefix(offs)).to(DEV)
    a_sf = ops.mx_tile_scales(a_s.to(DEV), 2 * K, offs_t, mt_t)
    w_sf = ops.mx_tile_scales(w_s.to(DEV), 2 * K)
    if gated:
        refs = []
        for e in range(E):
            rows = slice(int(offs[e]), int(offs[e + 1]))
            inter = torch.nn.functional.linear(a_f[rows], w_f[e]).to(torch.bfloat16)
            refs.append(orc._swiglu_bf16(inter))
        act = torch.cat(refs)
        out_g = orc.nvfp4_global_scale(act)
        q_ref, s_ref = orc.quant_nvfp4(act, out_g)
        out = torch.zeros(n, N // 2, dtype=torch.uint8, device=DEV)
        out_sf = torch.zeros(int(ops._lib.load().dqmoe_mx_tiled_scale_bytes(n, E, 2 * N)), dtype=torch.uint8, device=DEV)
        ops.grouped_gemm_nvfp4(a_q.to(DEV), a_sf, a_g.to(DEV), w_q.to(DEV), w_sf, w_g.to(DEV), offs_t, mt_t, N, True, out, out_sf,
                               out_g.to(DEV))
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        # compare dequantised: a summation-order difference may flip a 4-bit code here and there, never the bulk
        want_sf = ops.mx_tile_scales(s_ref.to(DEV), 2 * N, offs_t, mt_t)
        got = out.cpu()
        same = (got == q_ref).float().mean().item()
        assert same > 0.995, same
        # the scale bytes of rows that exist agree almost everywhere as well
        # (rows of a tile past its expert's last row hold bytes of no meaning: compare where real rows sit)
        real = ops.mx_tile_scales(torch.ones_like(s_ref).to(DEV), 2 * N, offs_t, mt_t).cpu() != 0
        agree = (out_sf.cpu()[real] == want_sf.cpu()[real]).float().mean().item()
        assert agree > 0.995, agree
    else:
        ref = torch.cat([torch.nn.functional.linear(a_f[int(offs[e]):int(offs[e + 1])], w_f[e]) for e in range(E)]).to(torch.bfloat16)
        out = torch.zeros(n, N, dtype=torch.bfloat16, device=DEV)
        ops.grouped_gemm_nvfp4(a_q.to(DEV), a_sf, a_g.to(DEV), w_q.to(DEV), w_sf, w_g.to(DEV), offs_t, mt_t, N, False, out)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        assert orc.cosine(out.cpu(), ref) >= 0.99999, orc.cosine(out.cpu(), ref)
        assert orc.max_rel_err(out.cpu(), ref) <= 5e-3, orc.max_rel_err(out.cpu(), ref)


def _layer_inputs(ops, seed, T, H, I, E, k):
    a, b, b1, _, idx = make_inputs(seed, T, H, I, E, k, 1.0, 0.05)
    a_g = orc.nvfp4_global_scale(a)
    b_g = torch.cat([orc.nvfp4_global_scale(b[e]) for e in range(E)])
    b1_g = torch.cat([orc.nvfp4_global_scale(b1[e]) for e in range(E)])
    a_q, a_s = orc.quant_nvfp4(a, a_g)
    b_q, b_s = orc.quant_nvfp4(b, b_g)
    b1_q, b1_s = orc.quant_nvfp4(b1, b1_g)
    # the global scale of the intermediate: a calibration constant; here from the bf16 layer's own intermediate
    act_amax = 0.0
    for e in range(E):
        tok, _ = torch.where(idx == e)
        if tok.numel():
            act_amax = max(act_amax, orc._swiglu_bf16(torch.nn.functional.linear(a[tok], b[e])).float().abs().amax().item())
    act_g = torch.tensor([max(act_amax, 1e-4) / (448.0 * 6.0)], dtype=torch.float32)
    cpu = (a_q, a_s, a_g, b_q, b_s, b_g, b1_q, b1_s, b1_g, act_g)
    dev = (a_q.to(DEV), a_s.to(DEV), a_g.to(DEV), b_q.to(DEV), ops.mx_tile_scales(b_s.to(DEV), 2 * H), b_g.to(DEV), b1_q.to(DEV),
           ops.mx_tile_scales(b1_s.to(DEV), 2 * I), b1_g.to(DEV), act_g.to(DEV))
    return cpu, dev, idx


SHAPES = [(8, 96, 512, 512, 2), (4, 700, 256, 768, 2), (8, 64, 1024, 2048, 2), (3, 5, 256, 256, 2), (2, 3000, 512, 1024, 2),
          (1, 1, 256, 256, 1)]


@pytest.mark.parametrize("E,T,H,I,k", SHAPES)
def test_layer_nvfp4_matches_oracle(ops, E, T, H, I, k):
    cpu, dev, idx = _layer_inputs(ops, 11, T, H, I, E, k)
    if T > 10:
        idx[3, 0] = -1   # a dropped row
    ref = orc.moe_layer_nvfp4(*cpu, idx, E)
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, orc.QUANT_NVFP4) + 256, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward_nvfp4(*dev, d, idx.to(DEV), ws)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = d.cpu()
    assert orc.cosine(got, ref) >= COS_MIN, orc.cosine(got, ref)
    assert orc.max_rel_err(got, ref) <= REL_MAX, orc.max_rel_err(got, ref)
    if T > 10:
        assert torch.count_nonzero(got[3, 0]) == 0
    d2 = torch.zeros_like(d)
    ops.moe_forward_nvfp4(*dev, d2, idx.to(DEV), ws)
    assert torch.equal(d, d2)   # deterministic


def test_layer_nvfp4_with_biases(ops):
    E, T, H, I, k = 4, 200, 512, 256, 2
    cpu, dev, idx = _layer_inputs(ops, 13, T, H, I, E, k)
    g = torch.Generator().manual_seed(2)
    bias1, bias2 = torch.randn(E, 2 * I, generator=g) * 0.5, torch.randn(E, H, generator=g) * 0.5
    ref = orc.moe_layer_nvfp4(*cpu, idx, E, bias1=bias1, bias2=bias2)
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, orc.QUANT_NVFP4) + 256, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward_nvfp4(*dev, d, idx.to(DEV), ws, bias1=bias1.to(DEV), bias2=bias2.to(DEV))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert orc.cosine(d.cpu(), ref) >= COS_MIN and orc.max_rel_err(d.cpu(), ref) <= REL_MAX


def test_nvfp4_mode_rejects_shapes_it_cannot_tile(ops):
    E, T, H, I, k = 2, 8, 128, 256, 1
    ws = torch.empty(1 << 20, dtype=torch.uint8, device=DEV)
    z = lambda *s: torch.zeros(*s, dtype=torch.uint8, device=DEV)
    f = lambda n: torch.ones(n, dtype=torch.float32, device=DEV)
    with pytest.raises(RuntimeError, match="multiples of 256 in the NVFP4 mode"):
        ops.moe_forward_nvfp4(z(T, H // 2), z(T, H // 16), f(1), z(E, 2 * I, H // 2), z(4096), f(E), z(E, H, I // 2), z(4096), f(E),
                              f(1), torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV),
                              torch.zeros(T, k, dtype=torch.int32, device=DEV), ws)


def test_mixtral_shape_nvfp4_full_size_sample(ops):
    """T=4096, H=4096, I=14336, E=8, top-2 in the NVFP4 mode: a sample of tokens against the oracle at full H and I,
    and the same sample as a small batch bit for bit."""
    T, H, I, E, k = 4096, 4096, 14336, 8, 2
    g = torch.Generator(device=DEV).manual_seed(78)
    x = torch.randn(T, H, generator=g, device=DEV).to(torch.bfloat16)
    idx, _ = ops.route_topk(torch.randn(T, E, generator=g, device=DEV), k, "softmax")
    b = (torch.randn(E, 2 * I, H, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    b_g = (b.float().abs().amax(dim=(1, 2)) / torch.full((), 2688.0, device=DEV)).contiguous()
    bq, bs_rows = ops.nvfp4_cast(b, b_g)
    bs = ops.mx_tile_scales(bs_rows, 2 * H)
    del b
    b1 = (torch.randn(E, H, I, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    b1_g = (b1.float().abs().amax(dim=(1, 2)) / torch.full((), 2688.0, device=DEV)).contiguous()
    b1q, b1s_rows = ops.nvfp4_cast(b1, b1_g)
    b1s = ops.mx_tile_scales(b1s_rows, 2 * I)
    del b1
    a_g = ops.nvfp4_global_scale(x)
    aq, a_sf = ops.nvfp4_cast(x, a_g)
    act_g = torch.tensor([64.0 / 2688.0], dtype=torch.float32, device=DEV)
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, orc.QUANT_NVFP4), dtype=torch.uint8, device=DEV)
    d = torch.empty(T, k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward_nvfp4(aq, a_sf, a_g, bq, bs, b_g, b1q, b1s, b1_g, act_g, d, idx, ws)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.isfinite(d.float()).all() and (d.float().abs().amax(dim=2) > 0).all()
    rows = torch.arange(3, T, 17, device=DEV)[:200]
    small = torch.empty(rows.numel(), k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward_nvfp4(aq[rows].contiguous(), a_sf[rows].contiguous(), a_g, bq, bs, b_g, b1q, b1s, b1_g, act_g, small,
                          idx[rows].contiguous(), ws)
    assert torch.equal(small, d[rows])
    srows = torch.arange(5, T, 127, device=DEV)[:16]
    ref = orc.moe_layer_nvfp4(aq[srows].cpu(), a_sf[srows].cpu(), a_g.cpu(), bq.cpu(), bs_rows.cpu(), b_g.cpu(), b1q.cpu(),
                              b1s_rows.cpu(), b1_g.cpu(), act_g.cpu(), idx[srows].cpu(), E)
    got = d[srows].cpu()
    assert orc.cosine(got, ref) >= COS_MIN and orc.max_rel_err(got, ref) <= REL_MAX
