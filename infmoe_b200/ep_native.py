"""ctypes wrapper of the expert-parallel entry points of the C ABI (infmoe_ep_*).

One `NativeExpertParallel` object is one rank's share of a MoE layer whose experts are sharded over the GPUs of a
node: routing, the row exchange over NVLink peer memory, the local experts and the return of the results all happen
inside the library, stream ordered and without host synchronisation.  This module only moves pointers.

    uid = unique_id() on rank 0, handed to the other ranks by any host channel (torch.distributed, a file, MPI ...)
    ep = NativeExpertParallel.create(local_layer, centroids, ln, variant, rank, world, uid, max_tokens)
    out = ep.forward(x_local)          # CUDA tensor [tokens][D]; a view of the library's output buffer

`create_loopback` builds all ranks inside one process on one GPU (tests, single-GPU emulation).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np

from . import capi
from .plugin import MoELayer, _fptr

PHASES = ("route_dispatch_send", "wait_rows", "experts", "wait_results", "copy_out")


def unique_id() -> bytes:
    buf = ctypes.create_string_buffer(capi.EP_ID_BYTES)
    capi.check(capi.lib().infmoe_ep_unique_id(buf))
    return buf.raw


def _config(local: MoELayer, centroids: np.ndarray, ln: Optional[np.ndarray], variant: str, rank: int, world: int,
            uid: Optional[bytes], max_tokens: int, keep: list) -> capi.EpConfig:
    cent = np.ascontiguousarray(centroids, dtype=np.float32)
    lnw = np.ascontiguousarray(ln, dtype=np.float32) if ln is not None and variant == "cpm_2" else None
    idbuf = ctypes.create_string_buffer(uid, capi.EP_ID_BYTES) if uid is not None else None
    keep += [cent, lnw, idbuf]
    return capi.EpConfig(rank, world, ctypes.cast(idbuf, ctypes.c_void_p) if idbuf is not None else None,
                         cent.shape[0], cent.shape[1], local.hidden_size, int(max_tokens), _fptr(cent), _fptr(lnw),
                         variant.encode("utf-8"), local._h)


class NativeExpertParallel:
    def __init__(self, handle: int, local: MoELayer, rank: int, world: int, D: int, max_tokens: int):
        self._h = ctypes.c_void_p(handle)
        self.local = local          # borrowed by the library: keep it alive
        self.rank, self.world, self.D, self.max_tokens = rank, world, D, max_tokens
        self._group: List["NativeExpertParallel"] = [self]

    # -- construction ---------------------------------------------------------------------------
    @classmethod
    def create(cls, local: MoELayer, centroids: np.ndarray, ln: Optional[np.ndarray], variant: str, rank: int,
               world: int, uid: Optional[bytes], max_tokens: int) -> "NativeExpertParallel":
        """Collective over all ranks (NCCL communicator + CUDA IPC mappings); uses the current CUDA device."""
        keep: list = []
        cfg = _config(local, centroids, ln, variant, rank, world, uid, max_tokens, keep)
        h = ctypes.c_void_p()
        capi.check(capi.lib().infmoe_ep_create(ctypes.byref(cfg), ctypes.byref(h)))
        return cls(h.value, local, rank, world, cfg.embedding_size, max_tokens)

    @classmethod
    def create_loopback(cls, locals_: Sequence[MoELayer], centroids: np.ndarray, ln: Optional[np.ndarray],
                        variant: str, max_tokens: int) -> List["NativeExpertParallel"]:
        """All ranks in this process on the current device; drive them with `loopback_forward`."""
        world = len(locals_)
        keep: list = []
        cfgs = (capi.EpConfig * world)(*[_config(l, centroids, ln, variant, r, world, None, max_tokens, keep)
                                         for r, l in enumerate(locals_)])
        hs = (ctypes.c_void_p * world)()
        capi.check(capi.lib().infmoe_ep_create_loopback(cfgs, world, hs))
        eps = [cls(hs[r], locals_[r], r, world, cfgs[r].embedding_size, max_tokens) for r in range(world)]
        for e in eps:
            e._group = eps
        return eps

    # -- the pass -------------------------------------------------------------------------------
    def output_view(self, tokens: int):
        """The library's output buffer of this rank as a CUDA tensor [tokens][D] (no copy)."""
        import torch

        p = ctypes.c_void_p()
        capi.check(capi.lib().infmoe_ep_output(self._h, ctypes.byref(p)))

        class _View:
            __cuda_array_interface__ = {"shape": (max(int(tokens), 1), self.D), "typestr": "<f4",
                                        "data": (p.value, False), "version": 2}

        return torch.as_tensor(_View(), device=torch.device("cuda", torch.cuda.current_device()))[:tokens]

    def forward(self, x, out=None, stream: Optional[int] = None):
        """x: contiguous float32 CUDA tensor [tokens][D].  Returns `out` if given, else a view of the library's
        output buffer (valid until the next forward)."""
        import torch

        if not (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()):
            raise ValueError("x must be a contiguous float32 CUDA tensor")
        T = x.shape[0]
        s = torch.cuda.current_stream(x.device).cuda_stream if stream is None else stream
        capi.check(capi.lib().infmoe_ep_forward(self._h, x.data_ptr(), out.data_ptr() if out is not None else None, T, s))
        return out if out is not None else self.output_view(T)

    def forward_host_ptr(self, h_in: int, h_out: int, tokens: int) -> None:
        capi.check(capi.lib().infmoe_ep_forward_host(self._h, h_in, h_out, int(tokens)))

    def submit_host_ptr(self, h_in: int, h_out: int, tokens: int) -> None:
        """Enqueues a step with host buffers and returns; at most two steps in flight (see wait_host)."""
        capi.check(capi.lib().infmoe_ep_submit_host(self._h, h_in, h_out, int(tokens)))

    def wait_host(self) -> None:
        """Blocks until the oldest submitted step's result is in its output buffer; raises on its status."""
        capi.check(capi.lib().infmoe_ep_wait_host(self._h))

    def sync_status(self, stream: Optional[int] = None) -> None:
        import torch

        s = torch.cuda.current_stream().cuda_stream if stream is None else stream
        capi.check(capi.lib().infmoe_ep_sync_status(self._h, s))

    def last_routing(self):
        ptrs = [ctypes.c_void_p() for _ in range(5)]
        capi.check(capi.lib().infmoe_ep_last_routing(self._h, *[ctypes.byref(p) for p in ptrs]))
        return tuple(p.value for p in ptrs)

    def received(self):
        """(region_count ptr, expert_of_slot ptr, home_of_slot ptr, region_size)."""
        a, b, c = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        n = ctypes.c_int64()
        capi.check(capi.lib().infmoe_ep_received(self._h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), ctypes.byref(n)))
        return a.value, b.value, c.value, int(n.value)

    def set_profiling(self, enable: bool) -> None:
        capi.check(capi.lib().infmoe_ep_set_profiling(self._h, 1 if enable else 0))

    def phase_ms(self):
        ms = (ctypes.c_float * 5)()
        n = ctypes.c_int32()
        capi.check(capi.lib().infmoe_ep_phase_ms(self._h, ms, ctypes.byref(n)))
        return dict(zip(PHASES, [float(v) for v in ms])), int(n.value)

    def destroy(self) -> None:
        if self._h:
            capi.lib().infmoe_ep_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def loopback_forward(eps: Sequence[NativeExpertParallel], xs, stream: Optional[int] = None):
    """One pass of all loopback ranks on one stream: begin everywhere, experts everywhere, end everywhere.
    xs[r]: rank r's rows (CUDA tensor).  Returns the ranks' outputs (views of the library's buffers)."""
    import torch

    s = torch.cuda.current_stream().cuda_stream if stream is None else stream
    lib = capi.lib()
    for ep, x in zip(eps, xs):
        capi.check(lib.infmoe_ep_forward_begin(ep._h, x.data_ptr(), x.shape[0], s))
    for ep in eps:
        capi.check(lib.infmoe_ep_forward_experts(ep._h, s))
    for ep in eps:
        capi.check(lib.infmoe_ep_forward_end(ep._h, None, s))
    return [ep.output_view(x.shape[0]) for ep, x in zip(eps, xs)]
