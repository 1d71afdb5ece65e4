"""Expert-parallel MoE layer over the GPUs of one node.

Rank r owns experts [r*E/W, (r+1)*E/W) (weights sharded, never moved); every rank
keeps its own tokens (data parallel). One layer call is

  1. expert sort of the local rows by global expert id  -> rows grouped by
     destination rank, then by expert (experts are partitioned contiguously);
  2. all-to-all of the per-(rank, expert) row counts;
  3. dispatch: variable-size all-to-all of the packed rows (+ their scales);
  4. regroup the received rows by local expert, grouped fc1 -> SwiGLU -> fc2 on the
     local experts, results written back in receive order;
  5. combine: the reverse all-to-all; scatter to d[T, k, H] (and weighted combine).

The reference has no distributed code at all (device 0 is hard-coded,
csrc/moe_kernels.h:633); this is the expert-parallel extension of its layer
(m_grouped_moe_nt_contiguous, csrc/pybind11_register.h:99-151). The collectives
are torch.distributed calls (NCCL on GPUs); received rows always land in this
GPU's memory before a kernel touches them. All compute goes through a `backend`
object: `CudaBackend` below (libdqmoe_b200.so) is the only one the package has.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def expert_range(rank: int, world: int, E: int) -> Tuple[int, int]:
    """Experts owned by `rank`: a contiguous block of E / world."""
    if E % world != 0:
        raise RuntimeError(f"[ASSERT FAILED] ep.py  Condition: E % world == 0  Info: E={E} world={world}")
    per = E // world
    return rank * per, (rank + 1) * per


def send_splits(counts: torch.Tensor, world: int) -> List[int]:
    """Rows going to each rank, from the per-expert counts [E] of the local sort."""
    return counts.view(world, -1).sum(dim=1).tolist()


class CudaBackend:
    """The kernels of libdqmoe_b200.so behind the small interface the EP layer needs."""

    def __init__(self, ops):
        self.ops = ops

    def route_sort(self, ids, E):
        return self.ops.route_sort(ids, E)

    def permute(self, a, dest_to_src, k, scale=None):
        return self.ops.moe_permute(a, dest_to_src, k, scale)

    def segment_ids(self, counts, values, n):
        return self.ops.segment_ids(counts, values, n)

    def experts(self, rows, row_scale, ids, weights_q, E_local, mode, out):
        """Grouped fc1 -> SwiGLU -> fc2 of `rows` (expert id per row in `ids`) into out[rows, H]."""
        b, bs, b1, b1s = weights_q
        n = rows.shape[0]
        H = rows.shape[1]
        I = b1.shape[2]
        ws = torch.empty(max(self.ops.moe_workspace_bytes(n, H, I, E_local, 1, mode), 256), dtype=torch.uint8,
                         device=rows.device)
        # the layer with k = 1: row i is "token" i with the single expert ids[i]
        self.ops.moe_forward(rows, row_scale, b, bs, b1, b1s, out.view(n, 1, H), ids.view(n, 1), ws, mode)

    def finalize_scatter(self, rows, dest_to_src, d):
        self.ops.finalize_scatter(rows, dest_to_src, d)

    def finalize_weighted(self, d, weights):
        return self.ops.finalize_weighted(d, weights)


def check_same_config(group, **config) -> None:
    """Every rank must have built its layer with the same sizes: a rank with another E or k would send
    counts and rows the others lay out differently. One small all_gather at construction; raises on every
    rank when the values differ."""
    names = sorted(config)
    mine = torch.tensor([int(config[n]) for n in names], dtype=torch.int64)
    backend = dist.get_backend(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    mine = mine.to(dev)
    everyone = [torch.empty_like(mine) for _ in range(dist.get_world_size(group))]
    dist.all_gather(everyone, mine, group=group)
    for r, other in enumerate(everyone):
        if not torch.equal(other, everyone[0]):
            diff = {n: (int(everyone[0][i]), int(other[i])) for i, n in enumerate(names) if other[i] != everyone[0][i]}
            raise RuntimeError(f"[ASSERT FAILED] ep.py  Condition: all ranks built the layer with the same sizes  "
                               f"Info: rank {r} differs from rank 0 in {diff}")


class ExpertParallelLayer:
    """One expert-parallel MoE layer; `weights_q` holds this rank's experts only."""

    def __init__(self, E: int, k: int, mode: int, weights_q, backend, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E, self.k, self.mode = E, k, mode
        check_same_config(group, E=E, k=k, mode=mode)
        self.lo, self.hi = expert_range(self.rank, self.world, E)
        self.E_local = self.hi - self.lo
        self.weights_q = weights_q
        self.backend = backend

    # ------------------------------------------------------------------ plumbing

    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """counts [E] (rows per global expert on this rank) -> recv_counts [W, E_local]
        (rows arriving from each rank for each local expert)."""
        W = self.world
        send = counts.view(W, self.E_local).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv

    def all_to_all_rows(self, x: torch.Tensor, out_rows: int, in_splits, out_splits) -> torch.Tensor:
        """Variable-size all-to-all over the leading (row) dimension; bytes are moved as uint8."""
        if sum(in_splits) != x.shape[0] or sum(out_splits) != out_rows or min(list(in_splits) + list(out_splits) + [0]) < 0:
            raise RuntimeError(f"[ASSERT FAILED] ep.py  Condition: split sizes add up to the rows exchanged  "
                               f"Info: sending {x.shape[0]} rows as {list(in_splits)}, receiving {out_rows} as {list(out_splits)}")
        flat = x.reshape(x.shape[0], -1)
        as_bytes = flat.view(torch.uint8) if flat.dtype != torch.uint8 else flat
        out = torch.empty((out_rows, as_bytes.shape[1]), dtype=torch.uint8, device=x.device)
        dist.all_to_all_single(out, as_bytes, output_split_sizes=out_splits, input_split_sizes=in_splits,
                               group=self.group)
        return out.view(x.dtype).view((out_rows,) + tuple(x.shape[1:]))

    # ------------------------------------------------------------------ layer

    def forward(self, a: torch.Tensor, a_scale: Optional[torch.Tensor], m_indices: torch.Tensor,
                route_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        """a [T, H] (e4m3 or bf16) with its scales, m_indices [T, k] global expert ids.
        Returns d [T, k, H] bf16, or the weighted combine [T, H] when route_weights is given."""
        be, k, W = self.backend, self.k, self.world
        T, H = a.shape
        n = T * k
        if a_scale is not None and self.mode == 256:
            raise RuntimeError("[ASSERT FAILED] ep.py  Condition: mode != FP8_TENSOR  "
                               "Info: a per-tensor scale differs per rank; use channel or block mode with EP")
        # 1. local sort by global expert id: rows for rank 0's experts first, then rank 1's, ...
        counts, offsets, d2s, _ = be.route_sort(m_indices, self.E)
        # 2. counts to the owners; split sizes must reach the host (one small synchronising copy)
        recv_counts = self.exchange_counts(counts)
        splits = torch.stack([counts.view(W, -1).sum(dim=1), recv_counts.sum(dim=1)]).cpu()  # the one host sync
        in_splits, out_splits = splits[0].tolist(), splits[1].tolist()
        n_recv = int(sum(out_splits))
        kept = int(sum(in_splits))
        # 3. dispatch: gather the kept rows (expert-sorted = destination-sorted) and send them
        if a_scale is not None:
            sc = a_scale.view(T, -1)
            rows, row_scale = be.permute(a, d2s[:kept], k, sc)
            recv_scale = self.all_to_all_rows(row_scale, n_recv, in_splits, out_splits)
        else:
            rows, recv_scale = be.permute(a, d2s[:kept], k), None
        recv_rows = self.all_to_all_rows(rows, n_recv, in_splits, out_splits)
        # 4. expert id of every received row: segments (src rank, local expert) of recv_counts
        local_ids = torch.arange(self.E_local, dtype=torch.int32, device=a.device).repeat(W)
        ids = be.segment_ids(recv_counts.reshape(-1), local_ids, n_recv)
        out_rows = torch.empty((n_recv, H), dtype=torch.bfloat16, device=a.device)
        if n_recv > 0:
            be.experts(recv_rows, recv_scale, ids, self.weights_q, self.E_local, self.mode, out_rows)
        # 5. combine: rows travel back in the same order, then scatter to slot order
        back = self.all_to_all_rows(out_rows, kept, out_splits, in_splits)
        d = torch.zeros((T, k, H), dtype=torch.bfloat16, device=a.device) if kept < n else \
            torch.empty((T, k, H), dtype=torch.bfloat16, device=a.device)
        if kept > 0:
            be.finalize_scatter(back, d2s[:kept], d)
        if route_weights is None:
            return d
        return be.finalize_weighted(d, route_weights)


class PeerExpertParallelLayer:
    """Expert-parallel layer whose exchange runs over peer-mapped memory instead of collectives.

    Same partitioning as ExpertParallelLayer. Every rank allocates one symmetric buffer
    (torch.distributed._symmetric_memory: the same allocation mapped into every rank of the node)
    holding the count matrix, flags, the receive buffers and the output d[T, k, H]. A call then is
    a fixed sequence of kernels on one stream with no host synchronisation and no collective:
    sort -> publish counts + plan (one launch) -> dispatch (rows written straight into the owners' receive
    buffers, already grouped by expert) -> wait -> grouped fc1 -> grouped fc2 whose epilogue stores
    every result row directly into its home rank's d (NVLink stores) -> signal -> wait.
    bf16, block FP8, MXFP8 and channel FP8 modes (MXFP8: a_scale is the row-major UE8M0 bytes [T, H/32], the weight
    scales are tiled by row index over this rank's experts; the received scale rows are tiled locally before fc1;
    channel mode adds the per-row re-quantisation pass between
    the GEMMs, bounded by the received row count read on the device). The returned tensor aliases
    the symmetric output buffer and is overwritten by a later call: by the next one with out_buffers = 1,
    by the one after it with out_buffers = 2 (calls then alternate between two output buffers, so a caller
    can still be copying call i's result while call i + 1 runs).
    """

    def __init__(self, T: int, H: int, I: int, E: int, k: int, mode: int, weights_q, ops, group=None,
                 capacity_rows: Optional[int] = None, capacity_factor: float = 2.0, out_buffers: int = 1):
        import ctypes
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads/stores only
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        if mode not in (0, 512, 1024, 2048):
            raise RuntimeError("[ASSERT FAILED] ep.py  Condition: mode in (0, 512, 1024, 2048)  Info: peer exchange supports bf16, channel, block FP8 and MXFP8")
        if mode == 2048 and (H % 128 or I % 128):
            raise RuntimeError("[ASSERT FAILED] ep.py  Condition: H % 128 == 0 and I % 128 == 0 in the MXFP8 mode")
        self.ops, self.lib, self.check, self.ct = ops, _lib.load(), _lib.check, ctypes
        self.group = group if group is not None else dist.group.WORLD
        self.W, self.me = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.W > 8:
            raise RuntimeError("[ASSERT FAILED] ep.py  Condition: world <= 8")
        self.T, self.H, self.I, self.E, self.k, self.mode = T, H, I, E, k, mode
        check_same_config(self.group, T=T, H=H, I=I, E=E, k=k, mode=mode,
                          capacity_rows=-1 if capacity_rows is None else capacity_rows,
                          capacity_factor_x1000=int(capacity_factor * 1000))
        self.lo, self.hi = expert_range(self.me, self.W, E)
        self.El = self.hi - self.lo
        self.weights_q = weights_q
        self.esz = 1 if mode else 2
        self.n = T * k
        # Rows this rank can receive in one call. Balanced routing sends about n = T*k rows to every rank;
        # the default leaves room for `capacity_factor` times that (never more than the worst case W*n).
        # The plan kernel compares every rank's incoming rows with the capacity: on overflow the call moves
        # and computes nothing on any rank and the device status word reads 202 (see check_status()).
        worst = self.W * self.n
        if capacity_rows is None:
            capacity_rows = min(worst, int(capacity_factor * self.n + 127) // 128 * 128)
        if capacity_rows < 0:
            raise RuntimeError("[ASSERT FAILED] ep.py  Condition: capacity_rows >= 0")
        self.cap = min(capacity_rows, worst)
        # fp32 words of scale that travel with a row: block mode one per 128 columns; MXFP8 H/32 bytes = H/128 words
        self.scale_cols = (H + 127) // 128 if mode in (1024, 2048) else (1 if mode == 512 else 0)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev

        def up(x):
            return (x + 255) // 256 * 256
        off, self.off = 0, {}
        if out_buffers not in (1, 2):
            raise RuntimeError("[ASSERT FAILED] ep.py  Condition: out_buffers in (1, 2)")
        self.out_buffers = out_buffers
        for name, nbytes in (("cnt", self.W * E * 4), ("flags", 3 * 8 * 4), ("rx_rows", self.cap * H * self.esz),
                             ("rx_scale", self.cap * max(self.scale_cols, 1) * 4), ("rx_home", self.cap * 4),
                             ("d_out", self.n * H * 2), ("d_out1", self.n * H * 2 if out_buffers == 2 else 0)):
            self.off[name] = off
            off += up(nbytes)
        self.sym = symm_mem.empty(off, dtype=torch.uint8, device=dev)
        self.sym.zero_()
        self.handle = symm_mem.rendezvous(self.sym, self.group)
        bases = [int(p) for p in self.handle.buffer_ptrs]
        self._ptr_arrays = {}
        for name in self.off:
            arr = (ctypes.c_void_p * self.W)(*[b + self.off[name] for b in bases])
            self._ptr_arrays[name] = arr
        self.local = {name: self.sym.data_ptr() + o for name, o in self.off.items()}
        self.send_base = torch.zeros(E + 1, dtype=torch.int32, device=dev)  # [E] = plan void (see dqmoe_ep_plan)
        self.rx_offsets = torch.zeros(self.El + 1, dtype=torch.int32, device=dev)
        self.rx_mtiles = torch.zeros(self.El + 1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.row_dst = torch.zeros(self.cap, dtype=torch.int64, device=dev)
        self.act = torch.empty(self.cap * I * self.esz, dtype=torch.uint8, device=dev)
        self.act_scale = torch.empty(self.cap * ((I + 127) // 128), dtype=torch.float32, device=dev)
        if mode == 2048:  # scale bytes in the tiled layout of this rank's receive buffer (see dqmoe_mx_tile_scales)
            self.rx_sf_tiled = torch.zeros(int(self.lib.dqmoe_mx_tiled_scale_bytes(self.cap, self.El, H)), dtype=torch.uint8,
                                           device=dev)
            self.act_sf_tiled = torch.zeros(int(self.lib.dqmoe_mx_tiled_scale_bytes(self.cap, self.El, I)), dtype=torch.uint8,
                                            device=dev)
        if mode == 512:  # stage 1 writes bf16 and collects the row amax; a second pass quantises
            self.act_bf16 = torch.empty(self.cap * I, dtype=torch.bfloat16, device=dev)
            self.amax = torch.zeros(self.cap, dtype=torch.float32, device=dev)
        self.d_outs = [self.sym[self.off[nm]:self.off[nm] + self.n * H * 2].view(torch.bfloat16).view(T, k, H)
                       for nm in (("d_out", "d_out1") if out_buffers == 2 else ("d_out",))]
        self.d_out = self.d_outs[0]
        self.epoch = 0
        torch.cuda.synchronize()
        dist.barrier(self.group)  # every rank's flags are zero before anyone publishes

    def check_status(self) -> None:
        """Synchronise and raise if a kernel of an earlier call gave up: forward() enqueues without a host
        synchronisation, so a caller that must know whether an output is complete calls this after it.
        202 = a rank's receive buffer (capacity_rows) was too small for the routing of that call; 201 / 211 /
        212 = a peer never arrived at the count exchange / the dispatch / the combine."""
        code = self.ops.device_status()
        if code != 0:
            raise RuntimeError(f"[ASSERT FAILED] ep.py  Condition: device_status() == 0  Info: status {code}"
                               + (f": more than capacity_rows={self.cap} rows for one rank" if code == 202 else ""))

    def forward(self, a: torch.Tensor, a_scale: Optional[torch.Tensor], m_indices: torch.Tensor,
                route_weights: Optional[torch.Tensor] = None, zero_dropped: bool = False,
                timeline: Optional[list] = None) -> torch.Tensor:
        """timeline: a list that receives (phase name, CUDA event recorded after the phase's launches) pairs,
        for measuring where a call's time goes; None records nothing."""
        ct, lib, ops = self.ct, self.lib, self.ops
        W, me, E, El, H, I, k = self.W, self.me, self.E, self.El, self.H, self.I, self.k
        if tuple(a.shape) != (self.T, H) or tuple(m_indices.shape) != (self.T, k):
            raise RuntimeError("[ASSERT FAILED] ep.py  Condition: a is [T, H] and m_indices is [T, k] of the sizes given at construction")
        self.epoch += 1
        ep_ = self.epoch
        cur = torch.cuda.current_stream(self.dev)
        stream = ct.c_void_p(cur.cuda_stream)
        P = self._ptr_arrays
        vp = ct.c_void_p
        out_name = "d_out1" if (self.out_buffers == 2 and ep_ % 2 == 0) else "d_out"
        d_out = self.d_outs[1] if out_name == "d_out1" else self.d_outs[0]

        def mark(name):
            if timeline is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(cur)
                timeline.append((name, ev))
        mark("start")
        if zero_dropped:
            d_out.zero_()
        counts, offsets, d2s, _ = ops.route_sort(m_indices, E)
        mark("sort")
        self.check(lib.dqmoe_ep_publish_plan(vp(counts.data_ptr()), E, me, W, P["cnt"], P["flags"], ep_, self.cap,
                                             vp(self.send_base.data_ptr()), vp(self.rx_offsets.data_ptr()),
                                             vp(self.rx_mtiles.data_ptr()), stream))
        mark("plan")
        sc_ptr = vp(a_scale.data_ptr()) if self.scale_cols else None
        self.check(lib.dqmoe_ep_dispatch(vp(a.data_ptr()), sc_ptr, H * self.esz, self.scale_cols, k, self.n,
                                         vp(offsets.data_ptr()), vp(d2s.data_ptr()), vp(self.send_base.data_ptr()),
                                         E, me, W, P["rx_rows"], P["rx_scale"], P["rx_home"], P["flags"],
                                         vp(self.done.data_ptr()), ep_, stream))
        mark("dispatch")
        self.check(lib.dqmoe_ep_wait_row_ptrs(vp(self.local["flags"]), ep_, vp(self.local["rx_home"]),
                                              vp(self.rx_offsets.data_ptr()), El, P[out_name], W, H * 2, self.cap,
                                              vp(self.row_dst.data_ptr()), stream))
        mark("wait_rows+row_ptrs")
        b, bs, b1, b1s = self.weights_q
        sp = lambda t: None if t is None else vp(t.data_ptr())
        rx_scale = vp(self.local["rx_scale"]) if self.scale_cols else None
        if self.mode == 2048:
            # received scale rows (row-major, in receive order) -> tiled by this rank's tiles; then the two MXFP8 GEMMs
            self.check(lib.dqmoe_mx_tile_scales(rx_scale, self.cap, H, None, 1, vp(self.rx_offsets.data_ptr()),
                                                vp(self.rx_mtiles.data_ptr()), El, vp(self.rx_sf_tiled.data_ptr()), stream))
            self.check(lib.dqmoe_grouped_gemm_mx(vp(self.local["rx_rows"]), vp(self.rx_sf_tiled.data_ptr()), vp(b.data_ptr()),
                                                 sp(bs), vp(self.rx_offsets.data_ptr()), vp(self.rx_mtiles.data_ptr()),
                                                 self.cap, I, H, El, 1, vp(self.act.data_ptr()),
                                                 vp(self.act_sf_tiled.data_ptr()), None, stream))
            mark("fc1")
            self.check(lib.dqmoe_grouped_gemm_mx_rows(vp(self.act.data_ptr()), vp(self.act_sf_tiled.data_ptr()),
                                                      vp(b1.data_ptr()), sp(b1s), vp(self.rx_offsets.data_ptr()),
                                                      vp(self.rx_mtiles.data_ptr()), self.cap, H, I, El,
                                                      vp(self.row_dst.data_ptr()), stream))
        elif self.mode == 512:
            self.amax.zero_()
            self.check(lib.dqmoe_grouped_gemm(vp(self.local["rx_rows"]), rx_scale, vp(b.data_ptr()), sp(bs),
                                              vp(self.rx_offsets.data_ptr()), vp(self.rx_mtiles.data_ptr()), self.cap, I,
                                              H, El, self.mode, 1, vp(self.act_bf16.data_ptr()), None,
                                              vp(self.amax.data_ptr()), None, stream))
            n_rx = vp(self.rx_offsets.data_ptr() + 4 * El)  # rows received, on the device
            self.check(lib.dqmoe_requant_from_amax_dev(vp(self.act_bf16.data_ptr()), self.cap, I, vp(self.amax.data_ptr()),
                                                       1, vp(self.act.data_ptr()), vp(self.act_scale.data_ptr()), n_rx,
                                                       stream))
        else:
            self.check(lib.dqmoe_grouped_gemm(vp(self.local["rx_rows"]), rx_scale, vp(b.data_ptr()), sp(bs),
                                              vp(self.rx_offsets.data_ptr()), vp(self.rx_mtiles.data_ptr()), self.cap, I,
                                              H, El, self.mode, 1, vp(self.act.data_ptr()), vp(self.act_scale.data_ptr()),
                                              None, None, stream))
        if self.mode != 2048:
            mark("fc1")
            self.check(lib.dqmoe_grouped_gemm_rows(vp(self.act.data_ptr()), vp(self.act_scale.data_ptr()) if self.mode else None,
                                                   vp(b1.data_ptr()), sp(b1s), vp(self.rx_offsets.data_ptr()),
                                                   vp(self.rx_mtiles.data_ptr()), self.cap, H, I, El, self.mode,
                                                   vp(self.row_dst.data_ptr()), stream))
        mark("fc2")
        self.check(lib.dqmoe_ep_signal_wait(P["flags"], 2, me, W, ep_, stream))
        mark("wait_results")
        if route_weights is None:
            return d_out
        return ops.finalize_weighted(d_out, route_weights)
