"""Helpers shared by the GPU parity tests: device buffers through torch, calls through the C ABI."""
import ctypes

import numpy as np
import torch

from infmoe_b200 import capi


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def stream():
    return torch.cuda.current_stream().cuda_stream


def route(x, c, ln=None):
    T, D = x.shape
    E = c.shape[0]
    dx, dc = dev(x), dev(c)
    dl = dev(ln) if ln is not None else None
    gate = torch.full((T,), -7, dtype=torch.int32, device="cuda")
    score = torch.zeros(T, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.check(capi.lib().infmoe_route(dx.data_ptr(), dc.data_ptr(), dl.data_ptr() if dl is not None else None, T, D,
                                       E, gate.data_ptr(), score.data_ptr(), status.data_ptr(), stream()))
    torch.cuda.synchronize()
    return gate.cpu().numpy(), score.cpu().numpy(), int(status.item())


def expert_count(gate, E):
    T = gate.shape[0]
    dg = dev(gate)
    pos = torch.full((max(T, 1),), -1, dtype=torch.int32, device="cuda")
    count = torch.full((E,), -1, dtype=torch.int32, device="cuda")
    offset = torch.full((E + 1,), -1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.check(capi.lib().infmoe_expert_count(T, E, dg.data_ptr(), pos.data_ptr(), count.data_ptr(),
                                              offset.data_ptr(), status.data_ptr(), stream()))
    torch.cuda.synchronize()
    return count.cpu().numpy(), offset.cpu().numpy(), pos.cpu().numpy()[:T], int(status.item())


def t5ff_run(x, ln, wi0, wi1, wo):
    n, D = x.shape
    F = wi0.shape[0]
    need = ctypes.c_size_t()
    capi.check(capi.lib().infmoe_t5ff_workspace_bytes(n, D, F, ctypes.byref(need)))
    ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    dx, dl, d0, d1, do = dev(x), dev(ln), dev(wi0), dev(wi1), dev(wo)
    y = torch.empty_like(dx)
    capi.check(capi.lib().infmoe_t5ff_run(n, D, F, dl.data_ptr(), d0.data_ptr(), d1.data_ptr(), do.data_ptr(),
                                          dx.data_ptr(), y.data_ptr(), ws.data_ptr(), need.value, stream()))
    torch.cuda.synchronize()
    return y.cpu().numpy()


from infmoe_b200.devmem import read_device  # noqa: E402,F401
