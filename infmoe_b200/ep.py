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


class ExpertParallelMoE:
    """forward(x_local) -> out_local for one MoE layer sharded over the ranks of `group`."""

    def __init__(self, stages, expert_count: int, group=None):
        self.stages = stages
        self.group = group
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
