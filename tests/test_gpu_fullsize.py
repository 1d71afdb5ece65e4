"""Parity at the full size of the headline configuration (Mixtral-shape prefill: T=4096, H=4096, I=14336, E=8,
top-2, 1x128 / 128x128 block FP8), where the CPU oracle cannot run the whole batch in seconds:
size-independent properties of the layer (every output row depends only on its own token and expert) tie the
full batch bit-exactly to a small subset, and the subset is checked against the oracle at full H and I."""
import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, REL_MAX = 0.999, 2e-2  # the layer tolerance: cosine and max|x - ref| / max|ref|
T, H, I, E, K = 4096, 4096, 14336, 8, 2


@pytest.fixture(scope="module")
def problem():
    from dqmoe_b200 import ops
    g = torch.Generator(device=DEV).manual_seed(2024)
    x = torch.randn(T, H, generator=g, device=DEV).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=DEV)
    idx, _ = ops.route_topk(logits, K, "softmax")
    b = (torch.randn(E, 2 * I, H, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    bq, bs = ops.per_block_cast_to_fp8(b)
    del b
    b1 = (torch.randn(E, H, I, generator=g, device=DEV) * 0.02).to(torch.bfloat16)
    b1q, b1s = ops.per_block_cast_to_fp8(b1)
    del b1
    aq, as_ = ops.per_token_block_cast_to_fp8(x)
    ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, K, 1024), dtype=torch.uint8, device=DEV)
    d = torch.empty(T, K, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward(aq, as_, bq, bs, b1q, b1s, d, idx, ws, 1024)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return dict(ops=ops, aq=aq, as_=as_, bq=bq, bs=bs, b1q=b1q, b1s=b1s, idx=idx, ws=ws, d=d)


def _run(p, rows):
    """The layer on a subset / reordering of the tokens (rows: index tensor on the device)."""
    ops = p["ops"]
    aq, as_, idx = p["aq"][rows].contiguous(), p["as_"][rows].contiguous(), p["idx"][rows].contiguous()
    out = torch.empty(rows.numel(), K, H, dtype=torch.bfloat16, device=DEV)
    ops.moe_forward(aq, as_, p["bq"], p["bs"], p["b1q"], p["b1s"], out, idx, p["ws"], 1024)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return out


def test_full_size_token_permutation_is_bit_exact(problem):
    perm = torch.randperm(T, generator=torch.Generator().manual_seed(1)).to(DEV)
    out = _run(problem, perm)
    assert torch.equal(out, problem["d"][perm])


def test_full_size_rows_equal_the_rows_of_a_small_batch(problem):
    rows = torch.arange(0, T, 13, device=DEV)[:300]  # 300 tokens spread over the batch: ragged expert counts
    out = _run(problem, rows)
    assert torch.equal(out, problem["d"][rows])


def test_full_size_sample_matches_the_oracle(problem):
    rows = torch.arange(5, T, 127, device=DEV)[:32]
    p = problem
    ref = orc.moe_layer_fp8(p["aq"][rows].cpu(), p["as_"][rows].cpu(), p["bq"].cpu(), p["bs"].cpu(), p["b1q"].cpu(),
                            p["b1s"].cpu(), p["idx"][rows].cpu(), E, 1024)
    got = p["d"][rows].cpu()
    assert orc.cosine(got, ref) >= COS_MIN
    assert orc.max_rel_err(got, ref) <= REL_MAX


def test_full_size_output_is_finite_and_every_slot_written(problem):
    d = problem["d"]
    assert torch.isfinite(d.float()).all()
    assert (d.float().abs().amax(dim=2) > 0).all()  # no slot of any token left untouched
