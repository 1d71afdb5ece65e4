"""GPU parity of the grouped GEMM and of the whole layer through the drop-in `moe_test`
module. Tolerance for layer outputs (floating point): cosine >= 0.999 and
max|x - ref| / max|ref| <= 2e-2 against the FP8-simulating CPU oracle."""
import numpy as np
import pytest
import torch

import moe_test
from helpers import bf16_from_bits, bits, golden, make_inputs
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, REL_MAX = 0.999, 2e-2


@pytest.fixture(scope="module")
def ops():
    from dqmoe_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def workspace():
    return torch.empty(1 << 30, dtype=torch.uint8, device=DEV)


def run_layer(a, b, b1, m_indices, mode, workspace, fused=True):
    T, k = m_indices.shape
    H = a.shape[1]
    E = b.shape[0]
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    if mode == 0:
        ref = orc.moe_layer_bf16(a, b, b1, m_indices, E)
        # the scale halves are dummies in this mode, as in test/util.py:232-234
        moe_test.m_grouped_moe_nt_contiguous_bf16((a.to(DEV), torch.ones_like(a).to(DEV)), (b.to(DEV), torch.ones(1, device=DEV)),
                                                  (b1.to(DEV), torch.ones(1, device=DEV)), d, m_indices.to(DEV), workspace, 0, fused)
    else:
        qs = orc.quantize_inputs(a, b, b1, mode)
        ref = orc.moe_layer_fp8(*qs, m_indices, E, mode)
        q = [t.to(DEV).contiguous() for t in qs]
        moe_test.m_grouped_moe_nt_contiguous_fp8_bf16((q[0], q[1]), (q[2], q[3]), (q[4], q[5]), d, m_indices.to(DEV),
                                                      workspace, mode, fused)
    return d, ref


def assert_close(d, ref):
    cos, rel = orc.cosine(d.cpu(), ref), orc.max_rel_err(d.cpu(), ref)
    assert cos >= COS_MIN and rel <= REL_MAX, (cos, rel)


# the reference's own small shapes (test/torch_test.py:19-25) plus ragged ones
SHAPES = [(1, 1, 16, 16, 1), (2, 1, 256, 32, 1), (3, 24, 192, 160, 2), (8, 64, 1024, 2048, 2), (8, 300, 512, 384, 3),
          (4, 130, 2880, 2880, 1), (64, 257, 256, 128, 6)]


@pytest.mark.parametrize("mode", [0, 256, 512, 1024])
@pytest.mark.parametrize("E,T,H,I,k", SHAPES)
def test_layer_matches_oracle(ops, workspace, mode, E, T, H, I, k):
    a, b, b1, _, m_indices = make_inputs(7, T, H, I, E, k, 1.0, 0.05)
    d, ref = run_layer(a, b, b1, m_indices, mode, workspace)
    assert ops.device_status() == 0
    assert_close(d, ref)


def test_layer_matches_reference_golden_outputs(ops, workspace):
    # outputs of the reference's torch_moe_grouped / fp8_blockwise_torch_moe_grouped (tests/golden)
    for name in ("layer_small.npz", "layer_c1.npz"):
        g = golden(name)
        T, H, I, E, k = (int(v) for v in g["shape"])
        a, b, b1, _, m_indices = make_inputs(int(g["seed"][0]), T, H, I, E, k, float(g["std"][0]), float(g["std"][1]))
        assert np.array_equal(bits(m_indices), g["m_indices"])
        d, _ = run_layer(a, b, b1, m_indices, 0, workspace)
        assert_close(d, bf16_from_bits(g["d_bf16"]))
        d, _ = run_layer(a, b, b1, m_indices, 1024, workspace)
        assert_close(d, bf16_from_bits(g["d_block"]))
    assert ops.device_status() == 0


def test_block_mode_intermediate_bytes_and_scales(ops, workspace):
    """The re-quantised intermediate (FP8 bytes + 1x128 scales) against the oracle's: the scales
    depend on a bf16-rounded fp32 sum whose order differs, so a small fraction may differ by one step."""
    import ctypes
    from dqmoe_b200 import _lib
    E, T, H, I, k = 4, 200, 512, 384, 2
    a, b, b1, _, m_indices = make_inputs(11, T, H, I, E, k, 1.0, 0.05)
    qs = orc.quantize_inputs(a, b, b1, 1024)
    _, inter = orc.moe_layer_fp8(*qs, m_indices, E, 1024, return_intermediate=True)
    run_layer(a, b, b1, m_indices, 1024, workspace)
    torch.cuda.synchronize()
    lib = _lib.load()
    n = T * k
    base = workspace.data_ptr()
    act_off = lib.dqmoe_moe_workspace_ptr(ctypes.c_void_p(base), 4, T, H, I, E, k, 1024) - base
    sc_off = lib.dqmoe_moe_workspace_ptr(ctypes.c_void_p(base), 5, T, H, I, E, k, 1024) - base
    act = workspace[act_off:act_off + n * I].view(torch.float8_e4m3fn).view(n, I).cpu()
    sc = workspace[sc_off:sc_off + n * 3 * 4].view(torch.float32).view(n, 3).cpu()
    ref_q = torch.cat([inter[e][0] for e in sorted(inter)])
    ref_s = torch.cat([inter[e][1] for e in sorted(inter)])
    assert (sc != ref_s).float().mean().item() < 0.02
    torch.testing.assert_close(sc, ref_s, rtol=1e-2, atol=0)
    assert (bits(act) != bits(ref_q)).mean() < 0.02


def test_fused_flag_gives_equal_results(ops, workspace):
    a, b, b1, _, m_indices = make_inputs(3, 100, 256, 128, 4, 2, 1.0, 0.05)
    d1, _ = run_layer(a, b, b1, m_indices, 512, workspace, fused=True)
    d2, _ = run_layer(a, b, b1, m_indices, 512, workspace, fused=False)
    assert torch.equal(d1, d2)


def test_layer_is_deterministic(ops, workspace):
    a, b, b1, _, m_indices = make_inputs(4, 700, 512, 256, 8, 2, 1.0, 0.05)
    for mode in (0, 512, 1024):
        d1, _ = run_layer(a, b, b1, m_indices, mode, workspace)
        d2, _ = run_layer(a, b, b1, m_indices, mode, workspace)
        assert torch.equal(d1, d2), mode


def test_dropped_rows_and_empty_experts(ops, workspace):
    E, T, H, I, k = 6, 50, 256, 128, 2
    a, b, b1, _, m_indices = make_inputs(5, T, H, I, E, k, 1.0, 0.05)
    m_indices = m_indices.clone()
    m_indices[m_indices == 2] = 4     # expert 2 receives nothing
    m_indices[7, 0] = -1              # dropped rows keep what d held before the call
    m_indices[9, 1] = E
    for mode in (0, 1024):
        d, ref = run_layer(a, b, b1, m_indices, mode, workspace)
        assert torch.count_nonzero(d[7, 0]) == 0 and torch.count_nonzero(d[9, 1]) == 0
        keep = (m_indices >= 0) & (m_indices < E)
        assert_close(d[keep.to(DEV)], ref[keep])
    assert ops.device_status() == 0


def test_errors_raise_runtime_error(ops, workspace):
    a, b, b1, _, m_indices = make_inputs(5, 8, 64, 32, 2, 2, 1.0, 0.05)
    d = torch.zeros(8, 2, 64, dtype=torch.bfloat16, device=DEV)
    one = torch.ones(1, device=DEV)
    args = ((a.to(DEV), one), (b.to(DEV), one), (b1.to(DEV), one), d, m_indices.to(DEV))
    with pytest.raises(RuntimeError, match="is not aligned"):
        moe_test.m_grouped_moe_nt_contiguous_bf16(*args, workspace[8:], 0)
    with pytest.raises(RuntimeError, match="workspace has"):
        moe_test.m_grouped_moe_nt_contiguous_bf16(*args, workspace[:256], 0)
    with pytest.raises(RuntimeError, match="torch::kInt"):
        moe_test.m_grouped_moe_nt_contiguous_bf16(*args[:4], m_indices.long().to(DEV), workspace, 0)
    # the context is still usable afterwards
    moe_test.m_grouped_moe_nt_contiguous_bf16(*args, workspace, 0)
    assert ops.device_status() == 0


RAGGED = [0, 1, 127, 128, 129, 0, 300, 5]
# mean rows per expert >= 512: the non-block modes run on CTA pairs (256-row tiles, odd tile counts included)
LARGE = [641, 0, 1300, 129]


# many experts and wide outputs: enough tiles for the 256-column single-CTA kernel (few tiles select 128 columns)
MANY = [200, 131, 0, 256, 77, 300, 128, 129, 1, 255, 190, 260, 140, 222, 180, 250]


@pytest.mark.parametrize("counts,N,K", [(RAGGED, 384, 640), (LARGE, 384, 640), (MANY, 1280, 256)],
                         ids=["ragged-narrow", "pairs", "many-wide"])
@pytest.mark.parametrize("mode,gated", [(0, False), (0, True), (256, True), (512, False), (512, True), (1024, False), (1024, True)])
def test_grouped_gemm_ragged_groups(ops, mode, gated, counts, N, K):
    """dqmoe_grouped_gemm alone on ragged expert sizes (0, 1, 127, 128, 129 rows ...); the three
    shape sets reach the three tile configurations (128-column, CTA-pair and 256-column tiles)."""
    E = len(counts)
    n = sum(counts)
    g = torch.Generator().manual_seed(mode + gated)
    a = torch.randn(n, K, generator=g).to(torch.bfloat16)
    wrows = 2 * N if gated else N
    w = (torch.randn(E, wrows, K, generator=g) * 0.05).to(torch.bfloat16)
    offsets = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32)
    off_d = offsets.to(DEV)
    mt = ops.mtile_prefix(off_d)
    if mode == 0:
        aq, asc, wq, wsc = a, None, w, None
        dq_a, dq_w = a.float(), w.float()
    elif mode == 1024:
        aq, asc = orc.quant_block_1x128(a)
        wq, wsc = orc.quant_block_128x128(w)
        dq_a, dq_w = aq.float() * orc._expand(asc, n, K), wq.float() * orc._expand(wsc, wrows, K)
    elif mode == 512:
        aq, asc = orc.quant_rowwise(a)
        wq, wsc = orc.quant_rowwise(w)
        dq_a, dq_w = aq.float() * asc, wq.float() * wsc
    else:
        aq, asc = orc.quant_tensor(a)
        wq, wsc = orc.quant_tensor(w, per_expert=True)
        dq_a, dq_w = aq.float() * asc, wq.float() * wsc.view(-1, 1, 1)
    ref = torch.cat([dq_a[offsets[e]:offsets[e + 1]] @ dq_w[e].t() for e in range(E)])
    dev = lambda t: None if t is None else t.to(DEV).contiguous()
    if gated:
        gt, vl = ref.to(torch.bfloat16).chunk(2, dim=-1)
        act = torch.nn.functional.silu(gt) * vl
        if mode == 1024:
            out = torch.zeros(n, N, dtype=torch.float8_e4m3fn, device=DEV)
            osc = torch.zeros(n, (N + 127) // 128, dtype=torch.float32, device=DEV)
            ops.grouped_gemm(dev(aq), dev(asc), dev(wq), dev(wsc), off_d, mt, N, mode, True, out, out_scale=osc)
            got = out.cpu().float() * orc._expand(osc.cpu(), n, N)
            rq, rs = orc.quant_block_1x128(act)
            want = rq.float() * orc._expand(rs, n, N)
        else:
            out = torch.zeros(n, N, dtype=torch.bfloat16, device=DEV)
            amax = torch.zeros(n if mode == 512 else 1, dtype=torch.float32, device=DEV)
            ops.grouped_gemm(dev(aq), dev(asc), dev(wq), dev(wsc), off_d, mt, N, mode, True, out, amax=amax)
            got, want = out.cpu().float(), act.float()
            if mode == 512:
                torch.testing.assert_close(amax.cpu(), act.float().abs().amax(dim=1), rtol=1e-2, atol=1e-6)
            if mode == 256:
                torch.testing.assert_close(amax.cpu(), act.float().abs().amax().view(1), rtol=1e-2, atol=1e-6)
    else:
        out = torch.zeros(n, N, dtype=torch.bfloat16, device=DEV)
        ops.grouped_gemm(dev(aq), dev(asc), dev(wq), dev(wsc), off_d, mt, N, mode, False, out)
        got, want = out.cpu().float(), ref
    assert ops.device_status() == 0
    # one e4m3 step of the re-quantised output at the largest magnitude is 1/16 of it: the layer tolerance applies
    assert orc.cosine(got, want) >= 0.9999 and orc.max_rel_err(got, want) <= REL_MAX


def test_profiler_sees_the_kernel_names_the_reference_script_filters_on(ops, workspace):
    """test/torch_test.py:180-205 times the layer by summing profiler rows whose kernel name contains
    "GemmUniversal" (bf16, block) or "GemmGrouped" (channel); test/bench.py:149-168 does the matching."""
    a, b, b1, _, m_indices = make_inputs(3, 64, 256, 128, 4, 2, 1.0, 0.05)
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        run_layer(a, b, b1, m_indices, 0, workspace)
        run_layer(a, b, b1, m_indices, 512, workspace)
        torch.cuda.synchronize()
    names = [e.key for e in prof.key_averages()]
    gemm = [n for n in names if "GemmUniversal" in n and "GemmGrouped" in n]
    assert gemm, names


@pytest.mark.parametrize("counts,N,K", [(RAGGED, 384, 640), (LARGE, 384, 640), (MANY, 1280, 256)],
                         ids=["ragged-narrow", "pairs", "many-wide"])
@pytest.mark.parametrize("mode", [0, 512, 1024])
def test_grouped_gemm_row_addresses_equal_scatter_map(ops, mode, counts, N, K):
    """dqmoe_grouped_gemm_rows (stage 2 storing each row to an explicit address, the path the
    expert-parallel layer uses to write into peer memory) against the same GEMM with a scatter map."""
    import ctypes
    from dqmoe_b200 import _lib
    E, n = len(counts), sum(counts)
    g = torch.Generator().manual_seed(mode + N)
    a = torch.randn(n, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, N, K, generator=g) * 0.05).to(torch.bfloat16)
    offsets = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32).to(DEV)
    mt = ops.mtile_prefix(offsets)
    if mode == 0:
        aq, asc, wq, wsc = a, None, w, None
    elif mode == 1024:
        aq, asc = orc.quant_block_1x128(a)
        wq, wsc = orc.quant_block_128x128(w)
    else:
        aq, asc = orc.quant_rowwise(a)
        wq, wsc = orc.quant_rowwise(w)
    dev = lambda t: None if t is None else t.to(DEV).contiguous()
    aq, asc, wq, wsc = dev(aq), dev(asc), dev(wq), dev(wsc)
    perm = torch.randperm(n, generator=g).to(torch.int32).to(DEV)
    perm[5] = -1  # a row without a destination
    want = torch.zeros(n, N, dtype=torch.bfloat16, device=DEV)
    ops.grouped_gemm(aq, asc, wq, wsc, offsets, mt, N, mode, False, want, dest_to_src=perm)
    got = torch.zeros(n, N, dtype=torch.bfloat16, device=DEV)
    row_dst = torch.where(perm >= 0, got.data_ptr() + perm.to(torch.int64) * (N * 2), torch.zeros((), dtype=torch.int64, device=DEV))
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    lib = _lib.load()
    _lib.check(lib.dqmoe_grouped_gemm_rows(p(aq), p(asc), p(wq), p(wsc), p(offsets), p(mt), n, N, K, E, mode,
                                           p(row_dst), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    assert ops.device_status() == 0
    assert torch.equal(got, want)


@pytest.mark.parametrize("mode,scoring", [(0, "softmax"), (1024, "softmax"), (1024, "sigmoid"), (512, "softmax"),
                                          (256, "sigmoid")])
def test_moe_block_router_to_weighted_output(ops, mode, scoring):
    """dqmoe_moe_block (router, activation quantisation, layer, weighted combine) against the oracle's moe_block."""
    E, T, H, I, k = 16, 200, 512, 256, 4
    a, b, b1, _, _ = make_inputs(31, T, H, I, E, k, 1.0, 0.05)
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(5))
    if mode == 0:
        ref = orc.moe_block(a, logits, b, b1, k, scoring, 0)
        out = ops.moe_block(a.to(DEV), logits.to(DEV), b.to(DEV), None, b1.to(DEV), None, k, scoring, 0)
    else:
        qs = orc.quantize_inputs(a, b, b1, mode)
        ref = orc.moe_block(a, logits, b, b1, k, scoring, mode, quantized=qs)
        out = ops.moe_block(a.to(DEV), logits.to(DEV), qs[2].to(DEV), qs[3].to(DEV).contiguous().view(E, -1)
                            if mode == 512 else qs[3].to(DEV).contiguous(), qs[4].to(DEV),
                            qs[5].to(DEV).contiguous().view(E, -1) if mode == 512 else qs[5].to(DEV).contiguous(),
                            k, scoring, mode)
    assert ops.device_status() == 0
    assert_close(out, ref)


@pytest.mark.parametrize("E,T,H,I,k", [(8, 64, 1024, 2048, 2), (8, 300, 512, 384, 3), (4, 2000, 512, 256, 1), (3, 5, 192, 160, 2)])
def test_layer_fp16_operands(ops, workspace, E, T, H, I, k):
    """dqmoe_moe_forward_f16: fp16 activations, weights and output against the oracle's layer run on fp16
    tensors (torch_moe_grouped of test/util.py:71-92 is dtype-generic). Includes the 2000-row-per-expert case
    that takes the CTA-pair tiles and a ragged one."""
    a, b, b1, _, m_indices = make_inputs(23, T, H, I, E, k, 1.0, 0.05)
    a, b, b1 = a.half(), b.half(), b1.half()
    ref = orc.moe_layer_bf16(a, b, b1, m_indices, E)
    assert ref.dtype == torch.float16
    d = torch.zeros(T, k, H, dtype=torch.float16, device=DEV)
    ops.moe_forward_f16(a.to(DEV), b.to(DEV), b1.to(DEV), d, m_indices.to(DEV), workspace)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(d, ref)
    # fp16 has three more mantissa bits than bf16: the result must be closer to the oracle than a bf16 run is
    assert orc.max_rel_err(d.cpu(), ref) < 5e-3


@pytest.mark.parametrize("mode,n_shared", [(0, 1), (1024, 1), (1024, 2)])
def test_moe_block_with_shared_experts(ops, mode, n_shared):
    """dqmoe_moe_block_shared: the last n_shared experts of the weight tensors see every token with weight 1
    (DeepSeek-style shared experts); checked against the oracle's moe_block with the same slots appended."""
    E, T, H, I, k = 16, 150, 512, 256, 4
    a, b, b1, _, _ = make_inputs(41, T, H, I, E + n_shared, k, 1.0, 0.05)
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(6))
    if mode == 0:
        ref = orc.moe_block(a, logits, b, b1, k, "sigmoid", 0, n_shared=n_shared)
        out = ops.moe_block(a.to(DEV), logits.to(DEV), b.to(DEV), None, b1.to(DEV), None, k, "sigmoid", 0,
                            n_shared=n_shared)
    else:
        qs = orc.quantize_inputs(a, b, b1, 1024)
        ref = orc.moe_block(a, logits, b, b1, k, "sigmoid", 1024, quantized=qs, n_shared=n_shared)
        out = ops.moe_block(a.to(DEV), logits.to(DEV), qs[2].to(DEV), qs[3].to(DEV).contiguous(), qs[4].to(DEV),
                            qs[5].to(DEV).contiguous(), k, "sigmoid", 1024, n_shared=n_shared)
    assert ops.device_status() == 0
    assert_close(out, ref)
    # without the shared slots the result differs: the shared experts really contributed
    plain = orc.moe_block(a, logits, b[:E], b1[:E], k, "sigmoid", 0)
    assert (ref.float() - plain.float()).abs().max() > 0


@pytest.mark.parametrize("mode", [0, 256, 1024])
def test_layer_replays_from_a_cuda_graph(ops, workspace, mode):
    """The layer enqueues kernels only (no host synchronisation, no allocation), so after one warm-up
    call it can be captured into a CUDA graph and replayed on new inputs (decode loops do this)."""
    E, T, H, I, k = 8, 16, 512, 256, 2
    a, b, b1, _, m_indices = make_inputs(9, T, H, I, E, k, 1.0, 0.05)
    a2, _, _, _, m2 = make_inputs(10, T, H, I, E, k, 1.0, 0.05)
    if mode == 0:
        q = [a.to(DEV), None, b.to(DEV), None, b1.to(DEV), None]
        q2 = [a2.to(DEV), None]
        ref2 = orc.moe_layer_bf16(a2, b, b1, m2, E)
    else:
        qs = orc.quantize_inputs(a, b, b1, mode)
        q = [t.to(DEV).contiguous() for t in qs]
        qs2 = orc.quantize_inputs(a2, b, b1, mode)
        q2 = [qs2[0].to(DEV), qs2[1].to(DEV).contiguous()]
        ref2 = orc.moe_layer_fp8(*qs2, m2, E, mode)
    idx = m_indices.to(DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ops.moe_forward(*q, d, idx, workspace, mode)  # warm-up: one-time host set-up happens here
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            ops.moe_forward(*q, d, idx, workspace, mode)
    # new inputs written into the captured buffers, then replay
    q[0].copy_(q2[0])
    if q2[1] is not None:
        q[1].copy_(q2[1])
    idx.copy_(m2.to(DEV))
    d.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert_close(d, ref2)


@pytest.mark.parametrize("mode,E,T,H,I,k", [(0, 2, 3, 4104, 2056, 2), (0, 3, 4, 1048, 520, 2), (256, 2, 4, 4112, 8208, 2),
                                            (256, 3, 1, 1040, 528, 3)])
def test_decode_path_ragged_sizes(ops, workspace, mode, E, T, H, I, k):
    """Up to 8 expanded rows take the weight-streaming path: rows longer than one 4 KB ring segment with a short last
    segment, a last pass of fewer than 8 / 16 columns (bf16 sizes that are 8 mod 16), several slots on one expert, a
    dropped slot."""
    a, b, b1, _, m_indices = make_inputs(19, T, H, I, E, k, 1.0, 0.05)
    if T > 1:
        m_indices[1, 0] = -1
    d, ref = run_layer(a, b, b1, m_indices, mode, workspace)
    assert ops.device_status() == 0
    assert_close(d, ref)
    if T > 1:
        assert torch.count_nonzero(d[1, 0]) == 0
