"""The plugin-shaped front end (dqmoe_plugin_*) against the oracle, with the plugin's input order
and output types of the reference's TensorRT test (test/trt_test.py:97-150, 505-560)."""
import pytest
import torch

from helpers import make_inputs
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, REL_MAX = 0.999, 2e-2  # the layer tolerance: cosine and max|x - ref| / max|ref|


def _inputs(mode, a, b, b1, idx):
    bias = None  # bias1 / bias2 are never read (use_bias = 0)
    if mode == 0:
        return [a.to(DEV), b.to(DEV), b1.to(DEV), idx.to(DEV), bias, bias], orc.moe_layer_bf16(a, b, b1, idx, b.shape[0])
    q = orc.quantize_inputs(a, b, b1, mode)
    ref = orc.moe_layer_fp8(*q, idx, b.shape[0], mode)
    aq, as_, bq, bs, b1q, b1s = [t.to(DEV).contiguous() for t in q]
    return [aq, bq, b1q, idx.to(DEV), bias, bias, as_, bs, b1s], ref


@pytest.mark.parametrize("mode,out_type", [(512, 1), (1024, 1), (1024, 7), (256, 0), (0, 7), (0, 1)])
def test_plugin_enqueue_matches_oracle(mode, out_type):
    from dqmoe_b200 import ops, plugin
    E, T, H, I, k = 8, 96, 512, 384, 2
    a, b, b1, _, idx = make_inputs(17, T, H, I, E, k, 1.0, 0.05)
    p = plugin.MoePlugin(E, k, H, I, max_num_tokens=128, type=plugin.DT_FP8 if mode else plugin.DT_BF16,
                         output_type=out_type, quant_mode=mode)
    inputs, ref = _inputs(mode, a, b, b1, idx)
    out = p.enqueue(inputs)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert out.dtype == {0: torch.float32, 1: torch.float16, 7: torch.bfloat16}[out_type]
    assert out.shape == (T, k, H)
    got = out.float().cpu()
    assert orc.cosine(got, ref) >= COS_MIN
    assert orc.max_rel_err(got, ref) <= REL_MAX
    # HALF / FLOAT outputs are exact conversions of the layer's bf16 result
    if out_type != 7:
        direct = plugin.MoePlugin(E, k, H, I, 128, type=p.fields["type"], output_type=plugin.DT_BF16, quant_mode=mode)
        assert torch.equal(direct.enqueue(inputs).float(), out.float())


def test_plugin_half_operands():
    """The fp16 engine of test/trt_test.py:386-455: HALF inputs, HALF output, quant_mode 0."""
    from dqmoe_b200 import ops, plugin
    E, T, H, I, k = 8, 96, 512, 384, 2
    a, b, b1, _, idx = make_inputs(19, T, H, I, E, k, 1.0, 0.05)
    a, b, b1 = a.half(), b.half(), b1.half()
    p = plugin.MoePlugin(E, k, H, I, max_num_tokens=128, type=plugin.DT_HALF, output_type=plugin.DT_HALF, quant_mode=0)
    out = p.enqueue([a.to(DEV), b.to(DEV), b1.to(DEV), idx.to(DEV), None, None])
    torch.cuda.synchronize()
    assert ops.device_status() == 0 and out.dtype == torch.float16
    ref = orc.moe_layer_bf16(a, b, b1, idx, E)
    assert orc.cosine(out.cpu(), ref) >= COS_MIN and orc.max_rel_err(out.cpu(), ref) <= REL_MAX


def test_plugin_rejects_too_many_tokens():
    from dqmoe_b200 import plugin
    p = plugin.MoePlugin(8, 2, 512, 384, max_num_tokens=16, type=plugin.DT_BF16, quant_mode=0)
    x = torch.zeros(32, 512, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="exceeds max_num_tokens"):
        p.enqueue([x, x, x, x, None, None], workspace=torch.empty(4096, dtype=torch.uint8, device=DEV))
