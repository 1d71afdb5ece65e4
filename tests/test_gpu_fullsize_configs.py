"""Parity at the full size of the other benchmark configurations, where the CPU oracle cannot run the whole batch
in seconds: the DeepSeek-V3-shape block-FP8 layer (E=256, top-8, sigmoid scores), the Qwen-MoE-shape channel-FP8
layer with Zipf-skewed routing (E=128, top-8), the Mixtral-shape decode sweep (T in {1, 16, 64, 256}, bf16 and
per-tensor FP8) and the two large shapes of the reference's own driver (test/torch_test.py:22-23).

Every output row of the bf16, channel and block layers depends only on its own token and expert, so a sample of
tokens is checked against the oracle at full H and I (with the sample's experts only, renumbered), and the same
sample run as a small batch must reproduce the full batch's rows bit for bit. The per-tensor mode shares one scale
of the intermediate between all rows, so its decode shapes are checked whole."""
import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, REL_MAX = 0.999, 2e-2  # the layer tolerance: cosine and max|x - ref| / max|ref|


@pytest.fixture(scope="module")
def ops():
    from dqmoe_b200 import ops as _ops
    return _ops


def _weights(ops, E, H, I, mode, std, seed, chunk=16):
    """Seeded expert weights, generated and quantised on the device in chunks of experts."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    parts = []
    for e0 in range(0, E, chunk):
        n = min(chunk, E - e0)
        b = (torch.randn(n, 2 * I, H, generator=g, device=DEV) * std).to(torch.bfloat16)
        b1 = (torch.randn(n, H, I, generator=g, device=DEV) * std).to(torch.bfloat16)
        if mode == 1024:
            parts.append((*ops.per_block_cast_to_fp8(b), *ops.per_block_cast_to_fp8(b1)))
        elif mode == 512:
            bq, bs = ops.per_channel_cast_to_fp8(b)
            b1q, b1s = ops.per_channel_cast_to_fp8(b1)
            parts.append((bq, bs.view(n, -1), b1q, b1s.view(n, -1)))
        elif mode == 256:
            parts.append((*ops.per_tensor_cast_to_fp8(b, per_expert=True), *ops.per_tensor_cast_to_fp8(b1, per_expert=True)))
        else:
            parts.append((b, None, b1, None))
        del b, b1
    return tuple(None if parts[0][i] is None else torch.cat([p[i] for p in parts]) for i in range(4))


def _activations(ops, x, mode):
    if mode == 1024:
        return ops.per_token_block_cast_to_fp8(x)
    if mode == 512:
        q, s = ops.per_token_cast_to_fp8(x)
        return q, s.view(-1)
    if mode == 256:
        return ops.per_tensor_cast_to_fp8(x)
    return x, None


def _layer(ops, aq, as_, w, idx, mode, k, H, I, E):
    T = aq.shape[0]
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, mode) + 256, dtype=torch.uint8, device=DEV)
    d = torch.empty(T, k, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward(aq, as_, w[0], w[1], w[2], w[3], d, idx, ws, mode)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return d


def _oracle_rows(aq, as_, w, idx, rows, mode):
    """The oracle on the tokens `rows`, with only the experts those tokens use (renumbered densely)."""
    sub_idx = idx[rows]
    used, inverse = torch.unique(sub_idx, return_inverse=True)
    sel = used.long()
    remap = inverse.to(torch.int32).cpu()
    cpu = lambda t: None if t is None else t.cpu()
    a_s = None if as_ is None else (as_ if mode == 256 else as_[rows])
    if mode == 0:
        return orc.moe_layer_bf16(cpu(aq[rows]), cpu(w[0][sel]), cpu(w[2][sel]), remap, used.numel())
    return orc.moe_layer_fp8(cpu(aq[rows]), cpu(a_s), cpu(w[0][sel]), cpu(w[1][sel]), cpu(w[2][sel]), cpu(w[3][sel]), remap,
                             used.numel(), mode)


def _check_sampled(ops, T, H, I, E, k, mode, scoring, std_w, std_a, seed, sample, zipf=False):
    g = torch.Generator(device=DEV).manual_seed(seed)
    x = (torch.randn(T, H, generator=g, device=DEV) * std_a).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=DEV)
    if zipf:  # a per-expert bias that skews the loads like Zipf(1.1)
        perm = torch.randperm(E, generator=g, device=DEV)
        logits = logits + (-1.1 * torch.log(torch.arange(1, E + 1, device=DEV, dtype=torch.float32)))[perm]
    idx, _ = ops.route_topk(logits, k, scoring)
    w = _weights(ops, E, H, I, mode, std_w, seed + 1)
    aq, as_ = _activations(ops, x, mode)
    d = _layer(ops, aq, as_, w, idx, mode, k, H, I, E)
    assert torch.isfinite(d.float()).all()
    assert (d.float().abs().amax(dim=2) > 0).all()  # every slot of every token written
    # a small batch of spread-out tokens reproduces the full batch's rows bit for bit
    rows = torch.arange(3, T, max(T // 257, 1), device=DEV)[:257]
    small = _layer(ops, aq[rows].contiguous(), None if as_ is None else as_[rows].contiguous(), w, idx[rows].contiguous(),
                   mode, k, H, I, E)
    assert torch.equal(small, d[rows])
    # a sample against the oracle at full H and I
    srows = torch.arange(1, T, max(T // sample, 1), device=DEV)[:sample]
    ref = _oracle_rows(aq, as_, w, idx, srows, mode)
    got = d[srows].cpu()
    assert orc.cosine(got, ref) >= COS_MIN, orc.cosine(got, ref)
    assert orc.max_rel_err(got, ref) <= REL_MAX, orc.max_rel_err(got, ref)
    if zipf:
        counts = torch.bincount(idx.flatten().long(), minlength=E)
        assert counts.max() > 8 * max(int(counts.min()), 1)  # the routing really is skewed


def test_deepseek_v3_shape_block_fp8_full_size(ops):
    """T=8192, H=7168, I=2048, E=256, top-8 of sigmoid scores, 1x128 / 128x128 block FP8."""
    _check_sampled(ops, 8192, 7168, 2048, 256, 8, 1024, "sigmoid", 0.02, 1.0, 31, sample=6)


def test_qwen_moe_shape_channel_fp8_zipf_full_size(ops):
    """T=16384, H=2048, I=768, E=128, top-8, per-token / per-channel FP8, Zipf(1.1)-skewed expert loads."""
    _check_sampled(ops, 16384, 2048, 768, 128, 8, 512, "softmax", 0.02, 1.0, 41, sample=12, zipf=True)


@pytest.mark.parametrize("E,T,H,I,k", [(64, 16384, 2880, 2880, 3), (4, 35456, 7168, 4096, 1)])
def test_reference_driver_large_shapes_bf16(ops, E, T, H, I, k):
    """The two large shapes of the reference's driver with its N(0, 0.05) inputs (test/torch_test.py:19-25, 60-76)."""
    _check_sampled(ops, T, H, I, E, k, 0, "softmax", 0.05, 0.05, 51, sample=8)


@pytest.fixture(scope="module")
def mixtral_weights(ops):
    H, I, E = 4096, 14336, 8
    g = torch.Generator(device=DEV).manual_seed(61)
    b = (torch.randn(E, 2 * I, H, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    b1 = (torch.randn(E, H, I, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    bq, bs = ops.per_tensor_cast_to_fp8(b, per_expert=True)
    b1q, b1s = ops.per_tensor_cast_to_fp8(b1, per_expert=True)
    return {0: (b, None, b1, None), 256: (bq, bs, b1q, b1s)}


@pytest.mark.parametrize("mode", [0, 256])
@pytest.mark.parametrize("T", [1, 4, 16, 64, 256])
def test_decode_sweep_shapes_full_size(ops, mixtral_weights, T, mode):
    """Mixtral shape (H=4096, I=14336, E=8, top-2) at the decode sweep's token counts; T <= 4 takes the GEMV path.
    bf16 rows are independent, so a sample of tokens goes to the oracle; the per-tensor mode shares one scale of the
    intermediate between all rows and is checked whole."""
    H, I, E, k = 4096, 14336, 8, 2
    w = mixtral_weights[mode]
    g = torch.Generator(device=DEV).manual_seed(70 + T)
    x = torch.randn(T, H, generator=g, device=DEV).to(torch.bfloat16)
    idx, _ = ops.route_topk(torch.randn(T, E, generator=g, device=DEV), k, "softmax")
    aq, as_ = _activations(ops, x, mode)
    d = _layer(ops, aq, as_, w, idx, mode, k, H, I, E)
    assert torch.isfinite(d.float()).all() and (d.float().abs().amax(dim=2) > 0).all()
    rows = torch.arange(0, T, max(T // 6, 1), device=DEV)[:6] if mode == 0 else torch.arange(T, device=DEV)
    ref = _oracle_rows(aq, as_, w, idx, rows, mode)
    got = d[rows].cpu()
    assert orc.cosine(got, ref) >= COS_MIN, orc.cosine(got, ref)
    assert orc.max_rel_err(got, ref) <= REL_MAX, orc.max_rel_err(got, ref)
