"""Expert biases and the fp32 (TF32) instantiation of the layer against the oracle, through the torch front
end and through the plugin-shaped entry points (the bias inputs and the FLOAT type of test/trt_test.py:82-89,
:121, :140-150; csrc/moe_kernels.h:72-78)."""
import pytest
import torch

from helpers import make_inputs
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, REL_MAX = 0.999, 2e-2          # the layer tolerance: cosine and max|x - ref| / max|ref|
COS_MIN_TF32, REL_MAX_TF32 = 0.99999, 5e-3  # fp32 operands read as TF32 (10-bit mantissa) against an fp32 reference


@pytest.fixture(scope="module")
def ops():
    from dqmoe_b200 import ops as _ops
    return _ops


def _biases(seed, E, H, I):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(E, 2 * I, generator=g) * 0.5, torch.randn(E, H, generator=g) * 0.5


@pytest.mark.parametrize("mode", [0, 256, 512, 1024])
@pytest.mark.parametrize("E,T,H,I,k", [(8, 96, 512, 384, 2), (4, 700, 384, 640, 2), (3, 5, 192, 160, 2)])
def test_layer_with_biases_matches_oracle(ops, mode, E, T, H, I, k):
    a, b, b1, _, idx = make_inputs(31, T, H, I, E, k, 1.0, 0.05)
    bias1, bias2 = _biases(5, E, H, I)
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, mode) + 256, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    if mode == 0:
        ref = orc.moe_layer_bf16(a, b, b1, idx, E, bias1, bias2)
        plain = orc.moe_layer_bf16(a, b, b1, idx, E)
        ops.moe_forward(a.to(DEV), None, b.to(DEV), None, b1.to(DEV), None, d, idx.to(DEV), ws, 0,
                        bias1=bias1.to(DEV), bias2=bias2.to(DEV))
    else:
        q = orc.quantize_inputs(a, b, b1, mode)
        ref = orc.moe_layer_fp8(*q, idx, E, mode, bias1=bias1, bias2=bias2)
        plain = orc.moe_layer_fp8(*q, idx, E, mode)
        qd = [t.to(DEV).contiguous() for t in q]
        ops.moe_forward(*qd, d, idx.to(DEV), ws, mode, bias1=bias1.to(DEV), bias2=bias2.to(DEV))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = d.cpu()
    assert orc.cosine(got, ref) >= COS_MIN and orc.max_rel_err(got, ref) <= REL_MAX
    assert orc.cosine(got, plain) < 0.99  # the biases are large enough to matter


def test_only_one_bias_given(ops):
    E, T, H, I, k = 4, 64, 256, 256, 2
    a, b, b1, _, idx = make_inputs(33, T, H, I, E, k, 1.0, 0.05)
    _, bias2 = _biases(6, E, H, I)
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, 0) + 256, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward(a.to(DEV), None, b.to(DEV), None, b1.to(DEV), None, d, idx.to(DEV), ws, 0, bias2=bias2.to(DEV))
    ref = orc.moe_layer_bf16(a, b, b1, idx, E, None, bias2)
    assert orc.cosine(d.cpu(), ref) >= COS_MIN and orc.max_rel_err(d.cpu(), ref) <= REL_MAX


@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("E,T,H,I,k", [(8, 96, 512, 384, 2), (4, 700, 384, 640, 2), (3, 5, 192, 160, 2), (1, 1, 16, 16, 1),
                                       (4, 1300, 1000, 520, 3)])
def test_layer_fp32_operands(ops, E, T, H, I, k, with_bias):
    a, b, b1, _, idx = make_inputs(41, T, H, I, E, k, 1.0, 0.05)
    a, b, b1 = a.float(), b.float(), b1.float()
    g = torch.Generator().manual_seed(3)  # give the operands mantissa bits beyond bf16 and TF32
    a = a + torch.randn(a.shape, generator=g) * 1e-3
    b = b + torch.randn(b.shape, generator=g) * 1e-4
    b1 = b1 + torch.randn(b1.shape, generator=g) * 1e-4
    bias1, bias2 = _biases(7, E, H, I) if with_bias else (None, None)
    ref = orc.moe_layer_bf16(a, b, b1, idx, E, bias1, bias2)
    assert ref.dtype == torch.float32
    ws = torch.empty(ops.moe_workspace_bytes_f32(T, H, I, E, k) + 256, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.float32, device=DEV)
    ops.moe_forward_f32(a.to(DEV), b.to(DEV), b1.to(DEV), d, idx.to(DEV), ws,
                        None if bias1 is None else bias1.to(DEV), None if bias2 is None else bias2.to(DEV))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = d.cpu()
    assert orc.cosine(got, ref) >= COS_MIN_TF32, orc.cosine(got, ref)
    assert orc.max_rel_err(got, ref) <= REL_MAX_TF32, orc.max_rel_err(got, ref)


def test_plugin_bias_inputs_and_float_type():
    from dqmoe_b200 import ops, plugin
    E, T, H, I, k = 8, 96, 512, 384, 2
    a, b, b1, _, idx = make_inputs(17, T, H, I, E, k, 1.0, 0.05)
    bias1, bias2 = _biases(8, E, H, I)
    # channel FP8 with biases, HALF output (the FP8 engine of test/trt_test.py:56-150 with use_bias = 1)
    q = orc.quantize_inputs(a, b, b1, 512)
    ref = orc.moe_layer_fp8(*q, idx, E, 512, bias1=bias1, bias2=bias2)
    aq, as_, bq, bs, b1q, b1s = [t.to(DEV).contiguous() for t in q]
    p = plugin.MoePlugin(E, k, H, I, max_num_tokens=128, use_bias=1, type=plugin.DT_FP8, output_type=plugin.DT_HALF,
                         quant_mode=512)
    out = p.enqueue([aq, bq, b1q, idx.to(DEV), bias1.to(DEV), bias2.to(DEV), as_, bs, b1s])
    torch.cuda.synchronize()
    assert out.dtype == torch.float16 and ops.device_status() == 0
    assert orc.cosine(out.float().cpu(), ref) >= COS_MIN and orc.max_rel_err(out.float().cpu(), ref) <= REL_MAX
    # FLOAT operands and output, with and without biases
    af, bf, b1f = a.float(), b.float(), b1.float()
    for use_bias in (0, 1):
        pf = plugin.MoePlugin(E, k, H, I, max_num_tokens=128, use_bias=use_bias, type=plugin.DT_FLOAT,
                              output_type=plugin.DT_FLOAT, quant_mode=0)
        out = pf.enqueue([af.to(DEV), bf.to(DEV), b1f.to(DEV), idx.to(DEV), bias1.to(DEV), bias2.to(DEV)])
        torch.cuda.synchronize()
        ref = orc.moe_layer_bf16(af, bf, b1f, idx, E, *((bias1, bias2) if use_bias else (None, None)))
        assert out.dtype == torch.float32 and ops.device_status() == 0
        assert orc.cosine(out.cpu(), ref) >= COS_MIN_TF32 and orc.max_rel_err(out.cpu(), ref) <= REL_MAX_TF32
    # half operands with biases
    ph = plugin.MoePlugin(E, k, H, I, max_num_tokens=128, use_bias=1, type=plugin.DT_HALF, output_type=plugin.DT_HALF,
                          quant_mode=0)
    out = ph.enqueue([a.half().to(DEV), b.half().to(DEV), b1.half().to(DEV), idx.to(DEV), bias1.to(DEV), bias2.to(DEV)])
    ref = orc.moe_layer_bf16(a.half(), b.half(), b1.half(), idx, E, bias1, bias2)
    assert orc.cosine(out.cpu(), ref) >= COS_MIN and orc.max_rel_err(out.cpu(), ref) <= REL_MAX


def test_route_topk_with_masked_logits_selects_each_expert_once(ops):
    """Rows with fewer than k logits above -inf: the masked experts fill the last slots in id order,
    every expert at most once (the oracle's stable sort gives the same)."""
    T, E, k = 64, 40, 4
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(T, E, generator=g)
    logits[::2] = float("-inf")
    logits[::2, 7] = 0.25            # one finite logit in every second row
    logits[1::4, 3:] = float("-inf")  # three finite logits
    idx, w = ops.route_topk(logits.to(DEV), k, "softmax")
    ref_idx, ref_w = orc.route_topk(logits, k, "softmax")
    assert torch.equal(idx.cpu(), ref_idx)
    assert all(len(set(row.tolist())) == k for row in idx.cpu())
    assert torch.allclose(w.cpu(), ref_w, atol=1e-6)


def test_scale_tensors_are_validated(ops):
    E, T, H, I, k = 4, 32, 256, 256, 2
    a, b, b1, _, idx = make_inputs(35, T, H, I, E, k, 1.0, 0.05)
    q = [t.to(DEV).contiguous() for t in orc.quantize_inputs(a, b, b1, 1024)]
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, 1024) + 256, dtype=torch.uint8, device=DEV)
    d = torch.zeros(T, k, H, dtype=torch.bfloat16, device=DEV)
    short = torch.ones(T, 1, device=DEV)  # a per-token scale passed in block mode
    with pytest.raises(RuntimeError, match="a_scale is a contiguous torch.float32 CUDA tensor of 64 elements"):
        ops.moe_forward(q[0], short, q[2], q[3], q[4], q[5], d, idx.to(DEV), ws, 1024)
    with pytest.raises(RuntimeError, match="b1_scale"):
        ops.moe_forward(q[0], q[1], q[2], q[3], q[4], q[5].double(), d, idx.to(DEV), ws, 1024)
    with pytest.raises(RuntimeError, match="bias1"):
        ops.moe_forward(*q, d, idx.to(DEV), ws, 1024, bias1=torch.zeros(E, I, device=DEV))
