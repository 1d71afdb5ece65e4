"""Host-side logic of the expert-parallel layer on CPU: two gloo ranks, the compute steps
replaced by the CPU oracle (test infrastructure), the plumbing (count exchange, split sizes,
variable-size all-to-all, regrouping, combine) is the package's own code."""
import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleBackend:
    """CPU stand-in for dqmoe_b200.ep.CudaBackend, built from oracle/ functions."""

    def __init__(self):
        from oracle import moe_oracle as orc
        self.orc = orc

    def route_sort(self, ids, E):
        return self.orc.route_sort(ids, E)

    def permute(self, a, dest_to_src, k, scale=None):
        rows = self.orc.permute_rows(a, dest_to_src, k)
        if scale is None:
            return rows
        return rows, self.orc.permute_rows(scale, dest_to_src, k)

    def segment_ids(self, counts, values, n):
        out = torch.repeat_interleave(values.long(), counts.long()).to(torch.int32)
        assert out.numel() == n
        return out

    def experts(self, rows, row_scale, ids, weights_q, E_local, mode, out):
        b, bs, b1, b1s = weights_q
        idx = ids.view(-1, 1)
        if mode == 0:
            d = self.orc.moe_layer_bf16(rows, b, b1, idx, E_local)
        else:
            sc = row_scale if mode == 1024 else row_scale.view(-1)
            d = self.orc.moe_layer_fp8(rows, sc, b, bs, b1, b1s, idx, E_local, mode)
        out.copy_(d[:, 0])

    def finalize_scatter(self, rows, dest_to_src, d):
        d.view(-1, d.shape[-1])[dest_to_src.long()] = rows

    def finalize_weighted(self, d, weights):
        return self.orc.finalize_weighted(d, weights)


def _worker(rank, world, init_file, mode, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from dqmoe_b200 import ep
    from helpers import make_inputs
    from oracle import moe_oracle as orc
    torch.set_num_threads(2)
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    try:
        E, T, H, I, k = 4, 24, 256, 128, 2
        # the model (weights) is global; each rank has its own tokens and routing
        _, b, b1, _, _ = make_inputs(100, T, H, I, E, k, 1.0, 0.05)
        a, _, _, _, m_indices = make_inputs(200 + rank, T, H, I, E, k, 1.0, 0.05)
        if rank == 1:
            m_indices[3, 0] = -1  # a dropped row on one rank only
        weights = torch.rand(T, k)
        lo, hi = ep.expert_range(rank, world, E)
        if mode == 0:
            wq_all = (b, None, b1, None)
            aq, asc = a, None
            ref = orc.moe_layer_bf16(a, b, b1, m_indices, E)
        else:
            _, _, bq, bs, b1q, b1s = orc.quantize_inputs(a, b, b1, mode)
            aq, asc = orc.quant_block_1x128(a) if mode == 1024 else orc.quant_rowwise(a)
            wq_all = (bq, bs, b1q, b1s)
            ref = orc.moe_layer_fp8(aq, asc if mode == 1024 else asc.view(-1), bq, bs, b1q, b1s, m_indices, E, mode)
        wq = tuple(None if t is None else t[lo:hi].contiguous() for t in wq_all)
        layer = ep.ExpertParallelLayer(E, k, mode, wq, OracleBackend())
        d = layer.forward(aq, asc, m_indices)
        out = layer.forward(aq, asc, m_indices, weights)
        cos, rel = orc.cosine(d, ref), orc.max_rel_err(d, ref)
        wref = orc.finalize_weighted(ref, weights)
        ok = cos > 0.9999 and rel < 1e-2 and orc.cosine(out, wref) > 0.9999
        dropped_zero = bool(torch.count_nonzero(d[3, 0]) == 0) if rank == 1 else True
        # count exchange: what this rank receives equals what the others counted for its experts
        counts, _, _, _ = orc.route_sort(m_indices, E)
        recv = layer.exchange_counts(counts)
        gathered = [torch.empty_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts)
        want = torch.stack([g[lo:hi] for g in gathered])
        results[rank] = (ok, cos, rel, dropped_zero, bool(torch.equal(recv, want)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", [0, 512, 1024])
def test_expert_parallel_two_ranks_matches_single_process_oracle(mode):
    world = 2
    with tempfile.TemporaryDirectory() as tmp:
        mgr = mp.Manager()
        results = mgr.dict()
        mp.spawn(_worker, args=(world, os.path.join(tmp, "init"), mode, results), nprocs=world, join=True)
        for rank in range(world):
            ok, cos, rel, dropped_zero, counts_ok = results[rank]
            assert ok, (rank, cos, rel)
            assert dropped_zero and counts_ok


def test_expert_range_and_splits():
    from dqmoe_b200 import ep
    assert ep.expert_range(0, 4, 256) == (0, 64) and ep.expert_range(3, 4, 256) == (192, 256)
    with pytest.raises(RuntimeError, match="E % world == 0"):
        ep.expert_range(0, 3, 8)
    counts = torch.tensor([1, 2, 3, 4, 5, 6], dtype=torch.int32)
    assert ep.send_splits(counts, 3) == [3, 7, 11]


def _mismatch_worker(rank, world, init_file, results):
    sys.path.insert(0, ROOT)
    from dqmoe_b200 import ep
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    try:
        try:
            ep.ExpertParallelLayer(4 if rank == 0 else 8, 2, 0, (None, None, None, None), OracleBackend())
            results[rank] = "no error"
        except RuntimeError as e:
            results[rank] = str(e)
    finally:
        dist.destroy_process_group()


def test_ranks_built_with_different_expert_counts_raise_on_every_rank():
    with tempfile.TemporaryDirectory() as tmp:
        results = mp.Manager().dict()
        mp.spawn(_mismatch_worker, args=(2, os.path.join(tmp, "init"), results), nprocs=2, join=True)
        for rank in range(2):
            assert "all ranks built the layer with the same sizes" in results[rank], results[rank]
            assert "'E': (4, 8)" in results[rank]


def _leaving_worker(rank, world, init_file, results):
    """Rank 1 leaves between two steps (no call in flight); rank 0's next step must end with an error,
    not hang: the process group carries a short timeout."""
    import datetime
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from dqmoe_b200 import ep
    from helpers import make_inputs
    torch.set_num_threads(2)
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    E, T, H, I, k = 4, 16, 128, 128, 2
    _, b, b1, _, _ = make_inputs(100, T, H, I, E, k, 1.0, 0.05)
    a, _, _, _, m_indices = make_inputs(200 + rank, T, H, I, E, k, 1.0, 0.05)
    lo, hi = ep.expert_range(rank, world, E)
    layer = ep.ExpertParallelLayer(E, k, 0, (b[lo:hi].contiguous(), None, b1[lo:hi].contiguous(), None), OracleBackend())
    layer.forward(a, None, m_indices)  # step 1: both ranks
    if rank == 1:
        results[rank] = "left after step 1"
        dist.destroy_process_group()
        return
    try:
        layer.forward(a, None, m_indices)  # step 2: the peer is gone
        results[rank] = "no error"
    except RuntimeError as e:
        results[rank] = "error: " + str(e)[:200]
    try:
        dist.destroy_process_group()
    except Exception:
        pass


def test_a_rank_leaving_between_steps_ends_the_next_step_with_an_error():
    with tempfile.TemporaryDirectory() as tmp:
        results = mp.Manager().dict()
        mp.spawn(_leaving_worker, args=(2, os.path.join(tmp, "init"), results), nprocs=2, join=True)
        assert results[1] == "left after step 1"
        assert results[0].startswith("error: "), results[0]


def test_send_splits_that_do_not_match_the_rows_raise():
    """A split-size list that does not add up to the rows sent is refused on the host, before any exchange."""
    from dqmoe_b200 import ep
    layer = object.__new__(ep.ExpertParallelLayer)
    layer.group = None
    x = torch.zeros(10, 4)
    with pytest.raises(RuntimeError, match="split sizes"):
        ep.ExpertParallelLayer.all_to_all_rows(layer, x, 10, [4, 4], [5, 5])
