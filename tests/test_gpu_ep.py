"""Expert-parallel layer on real GPUs (needs >= 2 devices; skipped otherwise): NCCL all-to-all
dispatch/combine with the CUDA kernels, checked against the single-GPU layer holding all experts."""
import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, init_file, mode, impl, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from dqmoe_b200 import ep, ops
    from helpers import make_inputs
    from oracle import moe_oracle as orc
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=dev)
    try:
        E, T, H, I, k = 8, 300, 512, 384, 2
        _, b, b1, _, _ = make_inputs(100, T, H, I, E, k, 1.0, 0.05)       # the model, same on every rank
        a, _, _, _, m_indices = make_inputs(200 + rank, T, H, I, E, k, 1.0, 0.05)
        if rank == world - 1:
            m_indices[3, 0] = -1
        weights = torch.rand(T, k)
        lo, hi = ep.expert_range(rank, world, E)
        if mode == 0:
            full = (b.to(dev), None, b1.to(dev), None)
            aq, asc = a.to(dev), None
        elif mode == 1024:
            full = (*ops.per_block_cast_to_fp8(b.to(dev)), *ops.per_block_cast_to_fp8(b1.to(dev)))
            aq, asc = ops.per_token_block_cast_to_fp8(a.to(dev))
        elif mode == 2048:
            full = (*ops.mx_cast_weights_to_fp8(b.to(dev)), *ops.mx_cast_weights_to_fp8(b1.to(dev)))
            aq, asc = ops.mx_cast_to_fp8(a.to(dev))
        else:
            bq, bs = ops.per_channel_cast_to_fp8(b.to(dev))
            b1q, b1s = ops.per_channel_cast_to_fp8(b1.to(dev))
            full = (bq, bs.view(E, -1), b1q, b1s.view(E, -1))
            aq, asc = ops.per_token_cast_to_fp8(a.to(dev))
            asc = asc.view(-1)
        # single-GPU reference on this rank: all experts local
        ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, mode), dtype=torch.uint8, device=dev)
        ref = torch.zeros(T, k, H, dtype=torch.bfloat16, device=dev)
        idx = m_indices.to(dev)
        ops.moe_forward(aq, asc, full[0], full[1], full[2], full[3], ref, idx, ws, mode)
        if mode == 2048:  # tiled scale bytes: an expert's 128-row blocks are contiguous, so a range of experts is a byte range
            per_b, per_b1 = full[1].numel() // E, full[3].numel() // E
            shard = (full[0][lo:hi].contiguous(), full[1][lo * per_b:hi * per_b].contiguous(), full[2][lo:hi].contiguous(),
                     full[3][lo * per_b1:hi * per_b1].contiguous())
        else:
            shard = tuple(None if t is None else t[lo:hi].contiguous() for t in full)
        if impl == "peer":  # exchange through peer-mapped memory, three calls in a row (flag epochs)
            layer = ep.PeerExpertParallelLayer(T, H, I, E, k, mode, shard, ops)
            layer.forward(aq, asc, idx, zero_dropped=True)
            d = layer.forward(aq, asc, idx, zero_dropped=True).clone()
            out = layer.forward(aq, asc, idx, weights.to(dev), zero_dropped=True)
        else:
            layer = ep.ExpertParallelLayer(E, k, mode, shard, ep.CudaBackend(ops))
            d = layer.forward(aq, asc, idx)
            out = layer.forward(aq, asc, idx, weights.to(dev))
        torch.cuda.synchronize()
        status = ops.device_status()
        same = bool(torch.equal(d, ref))  # same kernels, same per-row arithmetic: bit-identical
        wref = ops.finalize_weighted(ref, weights.to(dev))
        results[rank] = (status, same, orc.cosine(d.cpu(), ref.cpu()), bool(torch.equal(out, wref)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
@pytest.mark.parametrize("mode,impl", [(0, "nccl"), (512, "nccl"), (1024, "nccl"), (0, "peer"), (512, "peer"), (1024, "peer"),
                                       (2048, "peer")])
def test_expert_parallel_matches_single_gpu(mode, impl, world):
    """world = 1 runs the whole exchange (count matrix, plan, dispatch, row-address epilogue, flags) on one
    GPU, so the kernels of csrc/ep.cu are exercised where only one device is available."""
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    with tempfile.TemporaryDirectory() as tmp:
        results = mp.Manager().dict()
        mp.spawn(_worker, args=(world, os.path.join(tmp, "init"), mode, impl, results), nprocs=world, join=True)
        for rank in range(world):
            status, same, cos, wsame = results[rank]
            assert status == 0
            assert cos >= 0.9999, (rank, cos)
            assert same and wsame, (rank, cos)


def _failure_worker(rank, world, init_file, results):
    """Failure paths of the peer exchange on one GPU, none of which faults or hangs it: a receive buffer that is
    too small (status 202, nothing moved), flag waits that run out after a millisecond (201, 211), and a clean
    call on the same context afterwards."""
    import ctypes
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from dqmoe_b200 import _lib, ep, ops
    from helpers import make_inputs
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=dev)
    try:
        lib = _lib.load()
        E, T, H, I, k = 8, 300, 512, 384, 2
        a, b, b1, _, m_indices = make_inputs(300, T, H, I, E, k, 1.0, 0.05)
        full = (b.to(dev), None, b1.to(dev), None)
        aq, idx = a.to(dev), m_indices.to(dev)
        ws = torch.empty(ops.moe_workspace_bytes(T, H, I, E, k, 0), dtype=torch.uint8, device=dev)
        ref = torch.zeros(T, k, H, dtype=torch.bfloat16, device=dev)
        ops.moe_forward(aq, None, full[0], None, full[2], None, ref, idx, ws, 0)
        out = {}
        # 1. capacity smaller than the rows received: every rank sends and computes nothing, status 202
        small = ep.PeerExpertParallelLayer(T, H, I, E, k, 0, full, ops, capacity_rows=128)
        d = small.forward(aq, None, idx, zero_dropped=True)
        torch.cuda.synchronize()
        out["overflow_untouched"] = bool(torch.count_nonzero(d) == 0)
        try:
            small.check_status()
            out["overflow_raises"] = False
        except RuntimeError as e:
            out["overflow_raises"] = "202" in str(e) and "capacity_rows=128" in str(e)
        out["status_cleared"] = ops.device_status() == 0
        # the same layer object keeps working for a routing that fits: all rows to one slot of one expert pair
        few = idx.clone()
        few[64:] = -1
        d = small.forward(aq, None, few, zero_dropped=True)
        torch.cuda.synchronize()
        out["fits_after_overflow"] = ops.device_status() == 0 and bool(torch.equal(d[:64], ref[:64])) and \
            bool(torch.count_nonzero(d[64:]) == 0)
        # 2. waits that run out: a flag nobody sets, limit of about one millisecond
        _lib.check(lib.dqmoe_ep_set_wait_limit(2_000_000))
        layer = ep.PeerExpertParallelLayer(T, H, I, E, k, 0, full, ops)
        vp = ctypes.c_void_p
        stream = vp(torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(lib.dqmoe_ep_wait(vp(layer.local["flags"]), 1, world, 987654, stream))
        out["wait_status"] = ops.device_status()
        _lib.check(lib.dqmoe_ep_wait(vp(layer.local["flags"]), 2, world, 987654, stream))
        out["wait2_status"] = ops.device_status()
        _lib.check(lib.dqmoe_ep_plan(vp(layer.local["cnt"]), vp(layer.local["flags"]), E, rank, world, 987654, layer.cap,
                                     vp(layer.send_base.data_ptr()), vp(layer.rx_offsets.data_ptr()),
                                     vp(layer.rx_mtiles.data_ptr()), stream))
        out["plan_status"] = ops.device_status()
        out["plan_void"] = int(layer.send_base[E].item()) == 1 and int(layer.rx_offsets[-1].item()) == 0
        _lib.check(lib.dqmoe_ep_set_wait_limit(0))
        # 3. the context is intact: a normal call is bit-identical to the single-GPU layer
        d = layer.forward(aq, None, idx, zero_dropped=True)
        torch.cuda.synchronize()
        out["clean_after"] = ops.device_status() == 0 and bool(torch.equal(d, ref))
        results[rank] = out
    finally:
        dist.destroy_process_group()


def test_peer_exchange_failure_paths_report_status_and_leave_the_context_usable():
    with tempfile.TemporaryDirectory() as tmp:
        results = mp.Manager().dict()
        mp.spawn(_failure_worker, args=(1, os.path.join(tmp, "init"), results), nprocs=1, join=True)
        r = results[0]
        assert r["overflow_untouched"] and r["overflow_raises"] and r["status_cleared"], r
        assert r["fits_after_overflow"], r
        assert r["wait_status"] == 211 and r["wait2_status"] == 212 and r["plan_status"] == 201 and r["plan_void"], r
        assert r["clean_after"], r
