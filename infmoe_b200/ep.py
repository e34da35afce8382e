"""Expert-parallel MoE layer over torch.distributed (one process per GPU, NCCL over NVLink).

The reference is single-GPU (device 0 is hard-wired, plugin/MoELayerPlugin.cc:319); this module adds the
sharding its path allows.  Tokens are data-parallel (rank r owns a contiguous block of rows; the global
token index is rank-major), experts are sharded in contiguous blocks of E/R per rank.  Per layer pass:

  1. local routing over all E centroids            (infmoe_route)
  2. local dispatch metadata, rows grouped by expert and therefore by owner rank (infmoe_expert_count / _scatter)
  3. all-to-all of the per-expert counts, then of the rows themselves
  4. the owner runs its experts on the received rows (infmoe_layer_expert_forward; rows keep their order)
  5. all-to-all back, local combine into token order  (infmoe_expert_gather / _mix_gather)

Only steps 3 and 5 communicate.  Received rows land in this GPU's own memory before any kernel touches them.
The compute steps go through a small `stages` object so that the exchange logic can be exercised on CPU ranks
(gloo) with a stand-in; the default stages call the C ABI on the current CUDA device.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import capi
from .plugin import MoELayer


def expert_range(expert_count: int, world: int, rank: int):
    """Contiguous block of experts owned by `rank` (E must divide evenly)."""
    if expert_count % world:
        raise ValueError(f"expert_count {expert_count} is not divisible by the number of ranks {world}")
    per = expert_count // world
    return rank * per, (rank + 1) * per


class CudaStages:
    """The per-rank compute steps through the C ABI on the current CUDA device."""

    def __init__(self, local_layer: MoELayer, centroids: np.ndarray, gating_ln: Optional[np.ndarray], variant: str):
        self.layer = local_layer
        self.variant = variant
        self.centroids = torch.from_numpy(np.ascontiguousarray(centroids, np.float32)).cuda()
        self.gating_ln = None
        if variant == "cpm_2":
            self.gating_ln = torch.from_numpy(np.ascontiguousarray(gating_ln, np.float32)).cuda()
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    @staticmethod
    def _stream():
        return torch.cuda.current_stream().cuda_stream

    def route(self, x):
        T, D = x.shape
        E = self.centroids.shape[0]
        gate = torch.empty(T, dtype=torch.int32, device=x.device)
        score = torch.empty(T, dtype=torch.float32, device=x.device)
        ln = self.gating_ln.data_ptr() if self.gating_ln is not None else None
        capi.check(capi.lib().infmoe_route(x.data_ptr(), self.centroids.data_ptr(), ln, T, D, E, gate.data_ptr(),
                                           score.data_ptr(), self.status.data_ptr(), self._stream()))
        return gate, score

    def dispatch(self, gate, E):
        T = gate.shape[0]
        pos = torch.empty(max(T, 1), dtype=torch.int32, device=gate.device)
        count = torch.empty(E, dtype=torch.int32, device=gate.device)
        offset = torch.empty(E + 1, dtype=torch.int32, device=gate.device)
        capi.check(capi.lib().infmoe_expert_count(T, E, gate.data_ptr(), pos.data_ptr(), count.data_ptr(),
                                                  offset.data_ptr(), self.status.data_ptr(), self._stream()))
        return count, pos[:T]

    def scatter(self, x, score, pos):
        T, D = x.shape
        routed = torch.empty_like(x)
        rscore = torch.empty_like(score)
        capi.check(capi.lib().infmoe_expert_scatter(T, D, x.data_ptr(), score.data_ptr(), pos.data_ptr(),
                                                    routed.data_ptr(), rscore.data_ptr(), self._stream()))
        return routed, rscore

    def experts(self, rows, expert_of_row):
        return self.layer.expert_forward(rows, expert_of_row)

    def experts_to(self, rows, expert_of_row, row_dst, row_score=None):
        self.layer.expert_forward_scatter(rows, expert_of_row, row_dst, row_score)

    def combine(self, post, routed, rscore, pos):
        T, D = post.shape
        out = torch.empty_like(post)
        if self.variant == "base_layer":
            capi.check(capi.lib().infmoe_expert_mix_gather(T, D, pos.data_ptr(), routed.data_ptr(), post.data_ptr(),
                                                           rscore.data_ptr(), out.data_ptr(), self._stream()))
        else:
            capi.check(capi.lib().infmoe_expert_gather(T, D, post.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                                       self._stream()))
        return out

    def check(self):
        st = int(self.status.item())
        if st:
            self.status.zero_()
            raise capi.InfMoEError(3, f"routing/dispatch raised device status 0x{st:x}")
        self.layer.sync_status(self._stream())


class PeerOutput:
    """The output buffer of every rank, mapped into this process (CUDA IPC over NVLink peer access).

    Each rank allocates [rows][D] floats with cudaMalloc (an IPC handle needs the base of an allocation, which a
    block of the caching allocator is not), publishes the handle, and opens the handles of the others.  `base[r]`
    is the address of rank r's buffer as seen from here; `tensor` is this rank's own buffer.
    """

    def __init__(self, rows: int, D: int, group=None):
        from cuda.bindings import runtime as rt
        self._rt = rt
        self.rows, self.D = rows, D
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        err, ptr = rt.cudaMalloc(max(rows, 1) * D * 4)
        self._check(err, "cudaMalloc")
        self._own = int(ptr)
        err, handle = rt.cudaIpcGetMemHandle(self._own)
        self._check(err, "cudaIpcGetMemHandle")
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle.reserved), group=group)
        self.base, self._opened = [], []
        for r, raw in enumerate(handles):
            if r == rank:
                self.base.append(self._own)
                continue
            h = rt.cudaIpcMemHandle_t()
            h.reserved = raw
            err, p = rt.cudaIpcOpenMemHandle(h, rt.cudaIpcMemLazyEnablePeerAccess)
            self._check(err, f"cudaIpcOpenMemHandle (rank {r})")
            self.base.append(int(p))
            self._opened.append(int(p))

        class _View:   # minimal CUDA array interface over the raw allocation
            __cuda_array_interface__ = {"shape": (max(rows, 1), D), "typestr": "<f4", "data": (self._own, False),
                                        "version": 2}

        self.tensor = torch.as_tensor(_View(), device=torch.device("cuda", torch.cuda.current_device()))[:rows]
        self.base_dev = torch.tensor(self.base, dtype=torch.int64, device=self.tensor.device)

    @staticmethod
    def _check(err, what):
        if int(err) != 0:
            raise RuntimeError(f"{what} failed with CUDA error {int(err)}")

    def close(self):
        """Every rank must have finished writing (a barrier) before anybody calls this."""
        rt = self._rt
        for p in self._opened:
            rt.cudaIpcCloseMemHandle(p)
        self._opened = []
        if self._own:
            self.tensor = None
            rt.cudaFree(self._own)
            self._own = 0


class ExpertParallelMoE:
    """forward(x_local) -> out_local for one MoE layer sharded over the ranks of `group`."""

    def __init__(self, stages, expert_count: int, group=None, peer_output: bool = False):
        """peer_output: the owner of an expert writes each result row straight into the output buffer of the rank
        the token came from (peer stores from the GEMM epilogue) instead of sending rows back through a second
        all-to-all; needs CUDA ranks with peer access and stages that offer `experts_to`."""
        self.stages = stages
        self.group = group
        self.peer_output = peer_output
        self._peer = None
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.expert_count = expert_count
        self.e_lo, self.e_hi = expert_range(expert_count, self.world, self.rank)
        self.last = {}

    def _all_to_all(self, send, out_splits: List[int], in_splits: List[int]):
        out = send.new_empty((sum(out_splits),) + tuple(send.shape[1:]))
        if self.world == 1:
            out.copy_(send)
            return out
        dist.all_to_all_single(out, send, output_split_sizes=out_splits, input_split_sizes=in_splits, group=self.group)
        return out

    PHASES = ("local_route_dispatch_scatter", "counts_exchange", "rows_out", "experts", "rows_back", "combine")

    def close(self):
        if self._peer is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self._peer.close()
            self._peer = None

    def set_timing(self, enable: bool) -> None:
        """Record CUDA events between the phases of forward(); read them with phase_ms()."""
        self._timing = [] if enable else None

    def phase_ms(self):
        """Average device milliseconds per phase over the timed calls -> dict (empty when timing is off)."""
        calls = getattr(self, "_timing", None) or []
        if not calls:
            return {}
        torch.cuda.synchronize()
        tot = [0.0] * len(self.PHASES)
        for ev in calls:
            for i in range(len(self.PHASES)):
                tot[i] += ev[i].elapsed_time(ev[i + 1])
        return {name: t / len(calls) for name, t in zip(self.PHASES, tot)}

    def _experts_to_peers(self, x, received, expert_of_row, pos, rscore, send_rows, recv_rows, mark):
        """The return path without a second row exchange: the token index of every row (and, for the base_layer
        mix, its score) travels with it; the owner turns them into addresses inside the source rank's output
        buffer and the GEMM epilogue stores the rows there; one small collective orders the stores before the
        buffers are read."""
        T, D = x.shape
        if self._peer is None or self._peer.rows != T or self._peer.D != D:
            if self._peer is not None:
                self.close()
            self._peer = PeerOutput(T, D, self.group)
        peer = self._peer
        home = self._all_to_all(pos.to(torch.int32).contiguous(), recv_rows, send_rows)   # token index at the source
        src = torch.repeat_interleave(torch.arange(self.world), torch.tensor(recv_rows)).to(x.device, non_blocking=True)
        dst = peer.base_dev[src] + home.to(torch.int64) * (D * 4)
        scores = None
        if self.stages.variant == "base_layer":
            scores = self._all_to_all(rscore.contiguous(), recv_rows, send_rows)
        self.stages.experts_to(received, expert_of_row, dst.contiguous(), scores)
        mark()
        # every rank's stores are complete, and visible, before any rank reads its buffer
        flag = torch.zeros(1, device=x.device)
        dist.all_reduce(flag, group=self.group)
        mark()
        out = peer.tensor.clone()
        mark()
        return out

    def forward(self, x):
        R, E = self.world, self.expert_count
        per = E // R
        marks = []

        def mark():
            if getattr(self, "_timing", None) is not None and x.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append(ev)

        mark()
        gate, score = self.stages.route(x)
        count, pos = self.stages.dispatch(gate, E)
        routed, rscore = self.stages.scatter(x, score, pos)
        mark()
        # counts: what every rank sends to every expert.  recv_counts[src][e_local]
        send_counts = count.view(R, per)
        recv_counts = torch.empty_like(send_counts)
        if R == 1:
            recv_counts.copy_(send_counts)
        else:
            dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=self.group)
        # the one host synchronisation of the pass: the split sizes of the row exchange
        both = torch.stack((send_counts, recv_counts)).cpu()
        send_rows = both[0].sum(dim=1).tolist()
        recv_mat = both[1]
        recv_rows = recv_mat.sum(dim=1).tolist()
        mark()
        received = self._all_to_all(routed, recv_rows, send_rows)
        mark()
        # expert of every received row: rows arrive grouped by (source rank, local expert)
        local_ids = torch.arange(per, dtype=torch.int32).repeat(R)
        expert_of_row = torch.repeat_interleave(local_ids, recv_mat.reshape(-1).to(torch.int64)).to(
            x.device, non_blocking=True)
        if self.peer_output and R > 1:
            out = self._experts_to_peers(x, received, expert_of_row.contiguous(), pos, rscore, send_rows, recv_rows,
                                         mark)
        else:
            processed = self.stages.experts(received, expert_of_row.contiguous())
            mark()
            post = self._all_to_all(processed, send_rows, recv_rows)
            mark()
            out = self.stages.combine(post, routed, rscore, pos)
            mark()
        if marks:
            self._timing.append(marks)
        self.last = {"gate": gate, "score": score, "pos": pos, "count": count, "recv_counts": recv_mat}
        return out
