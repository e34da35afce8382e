"""numpy front-end of the CPU oracle (oracle.c).  TEST INFRASTRUCTURE ONLY.

Nothing in the product imports this module: only the tests, the smoke check
and the benchmark's CPU-baseline leg do.  Every function takes and returns
C-contiguous numpy arrays and forwards to the C restatement, which cites the
reference file:line each step follows.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

VARIANTS = {"default": 0, "cpm_2": 1, "base_layer": 2}

_c_f = ctypes.POINTER(ctypes.c_float)
_c_d = ctypes.POINTER(ctypes.c_double)
_c_i = ctypes.POINTER(ctypes.c_int32)
_c_fpp = ctypes.POINTER(_c_f)


def build(force: bool = False) -> str:
    """Compile liboracle.so with gcc if it is missing or older than oracle.c."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _f(a):
    return a.ctypes.data_as(_c_f) if a is not None else None


def _d(a):
    return a.ctypes.data_as(_c_d) if a is not None else None


def _i(a):
    return a.ctypes.data_as(_c_i) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _check(rc, what):
    if rc == 1:
        raise FloatingPointError(f"{what}: a token selected no expert (NaN scores)")
    if rc != 0:
        raise RuntimeError(f"{what}: oracle error {rc}")


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(ctypes.c_int(int(n)))


def layernorm(x, gamma):
    x, gamma = _f32(x), _f32(gamma)
    n, D = x.reshape(-1, x.shape[-1]).shape
    out = np.empty_like(x)
    lib().oracle_layernorm(_f(x), _f(gamma), ctypes.c_int64(n), ctypes.c_int(D), _f(out))
    return out


def layernorm_reference_order(x, gamma):
    x, gamma = _f32(x), _f32(gamma)
    n, D = x.reshape(-1, x.shape[-1]).shape
    out = np.empty_like(x)
    lib().oracle_layernorm_reference_order(_f(x), _f(gamma), ctypes.c_int64(n), ctypes.c_int(D), _f(out))
    return out


def route(x, centroids, gamma=None, want_aff=False):
    """-> gate int32[T], score f32[T] (and aff f32[T][E])."""
    x, centroids = _f32(x), _f32(centroids)
    T, D = x.shape
    E = centroids.shape[0]
    assert centroids.shape == (E, D)
    g = _f32(gamma) if gamma is not None else None
    gate = np.empty(T, np.int32)
    score = np.empty(T, np.float32)
    aff = np.empty((T, E), np.float32) if want_aff else None
    rc = lib().oracle_route(_f(x), _f(centroids), _f(g), ctypes.c_int64(T), ctypes.c_int(D), ctypes.c_int(E),
                            _i(gate), _f(score), _f(aff))
    _check(rc, "route")
    return (gate, score, aff) if want_aff else (gate, score)


def select_top1(aff):
    aff = _f32(aff)
    T, E = aff.shape
    gate = np.empty(T, np.int32)
    score = np.empty(T, np.float32)
    rc = lib().oracle_select_top1(_f(aff), ctypes.c_int64(T), ctypes.c_int(E), _i(gate), _f(score))
    _check(rc, "select_top1")
    return gate, score


def route_f64(x, centroids, gamma=None):
    x, centroids = _f32(x), _f32(centroids)
    T, D = x.shape
    E = centroids.shape[0]
    g = _f32(gamma) if gamma is not None else None
    gate = np.empty(T, np.int32)
    top1 = np.empty(T, np.float64)
    top2 = np.empty(T, np.float64)
    lib().oracle_route_f64(_f(x), _f(centroids), _f(g), ctypes.c_int64(T), ctypes.c_int(D), ctypes.c_int(E),
                           _i(gate), _d(top1), _d(top2))
    return gate, top1, top2


def dispatch(gate, E):
    """-> count int32[E], offset int32[E+1], pos int32[T]."""
    gate = np.ascontiguousarray(gate, np.int32)
    T = gate.shape[0]
    count = np.zeros(E, np.int32)
    offset = np.zeros(E + 1, np.int32)
    pos = np.empty(T, np.int32)
    rc = lib().oracle_dispatch(_i(gate), ctypes.c_int64(T), ctypes.c_int(E), _i(count), _i(offset), _i(pos))
    _check(rc, "dispatch")
    return count, offset, pos


def scatter(x, score, pos):
    x, score = _f32(x), _f32(score)
    pos = np.ascontiguousarray(pos, np.int32)
    T, D = x.shape
    routed = np.empty_like(x)
    rscore = np.empty(T, np.float32)
    lib().oracle_scatter(_f(x), _f(score), _i(pos), ctypes.c_int64(T), ctypes.c_int(D), _f(routed), _f(rscore))
    return routed, rscore


def gather(rows, pos):
    rows = _f32(rows)
    pos = np.ascontiguousarray(pos, np.int32)
    T, D = rows.shape
    out = np.empty_like(rows)
    lib().oracle_gather(_f(rows), _i(pos), ctypes.c_int64(T), ctypes.c_int(D), _f(out))
    return out


def mix_gather(post, routed, rscore, pos):
    post, routed, rscore = _f32(post), _f32(routed), _f32(rscore)
    pos = np.ascontiguousarray(pos, np.int32)
    T, D = post.shape
    out = np.empty_like(post)
    lib().oracle_mix_gather(_f(post), _f(routed), _f(rscore), _i(pos), ctypes.c_int64(T), ctypes.c_int(D), _f(out))
    return out


def gelu_dot(a, b):
    a = _f32(a)
    b = _f32(b).copy()
    lib().oracle_gelu_dot(_f(a), _f(b), ctypes.c_int64(a.size))
    return b


def sgemm_nt(A, B, C=None):
    """C (+)= A @ B.T in FP32; A [M][K], B [N][K]."""
    A, B = _f32(A), _f32(B)
    M, K = A.shape
    N = B.shape[0]
    acc = C is not None
    out = _f32(C).copy() if acc else np.empty((M, N), np.float32)
    lib().oracle_sgemm_nt(ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), _f(A), _f(B), _f(out),
                          ctypes.c_int(1 if acc else 0))
    return out


def expert_ffn_f32(x, ln_w, wi0, wi1, wo):
    x, ln_w, wi0, wi1, wo = map(_f32, (x, ln_w, wi0, wi1, wo))
    n, D = x.shape
    F = wi0.shape[0]
    assert wi0.shape == (F, D) and wi1.shape == (F, D) and wo.shape == (D, F)
    y = np.empty_like(x)
    rc = lib().oracle_expert_ffn_f32(_f(x), ctypes.c_int64(n), ctypes.c_int(D), ctypes.c_int(F), _f(ln_w), _f(wi0),
                                     _f(wi1), _f(wo), _f(y))
    _check(rc, "expert_ffn_f32")
    return y


def expert_ffn_f64(x, ln_w, wi0, wi1, wo):
    x, ln_w, wi0, wi1, wo = map(_f32, (x, ln_w, wi0, wi1, wo))
    n, D = x.shape
    F = wi0.shape[0]
    y = np.empty((n, D), np.float64)
    rc = lib().oracle_expert_ffn_f64(_f(x), ctypes.c_int64(n), ctypes.c_int(D), ctypes.c_int(F), _f(ln_w), _f(wi0),
                                     _f(wi1), _f(wo), _d(y))
    _check(rc, "expert_ffn_f64")
    return y


def _ptr_array(arrs):
    keep = [(_f32(a) if a is not None else None) for a in arrs]
    arr_t = _c_f * len(keep)
    ptrs = arr_t(*[(_f(a) if a is not None else ctypes.cast(None, _c_f)) for a in keep])
    return keep, ptrs


def layer_forward_f32(x, variant, centroids, gating_ln_w, experts, literal_gather=False):
    """experts: list of E tuples (ln_w, wi0, wi1, wo) or None for experts known to be empty.

    -> dict(out, gate, score, count, offset, pos)"""
    x, centroids = _f32(x), _f32(centroids)
    T, D = x.shape
    E = centroids.shape[0]
    F = next(e[1].shape[0] for e in experts if e is not None)
    g = _f32(gating_ln_w) if gating_ln_w is not None else None
    cols = [[(e[i] if e is not None else None) for e in experts] for i in range(4)]
    keeps, ptrs = zip(*[_ptr_array(c) for c in cols])
    out = np.empty_like(x)
    gate = np.empty(T, np.int32)
    score = np.empty(T, np.float32)
    count = np.empty(E, np.int32)
    offset = np.empty(E + 1, np.int32)
    pos = np.empty(T, np.int32)
    rc = lib().oracle_layer_forward_f32(_f(x), ctypes.c_int64(T), ctypes.c_int(D), ctypes.c_int(F), ctypes.c_int(E),
                                        ctypes.c_int(VARIANTS[variant]), _f(centroids), _f(g), ptrs[0], ptrs[1],
                                        ptrs[2], ptrs[3], ctypes.c_int(1 if literal_gather else 0), _f(out),
                                        _i(gate), _f(score), _i(count), _i(offset), _i(pos))
    _check(rc, "layer_forward_f32")
    del keeps
    return dict(out=out, gate=gate, score=score, count=count, offset=offset, pos=pos)


def layer_forward_f64(x, variant, gate, score, experts):
    """FP64-accumulated layer output for a GIVEN routing decision (gate, score)."""
    x = _f32(x)
    T, D = x.shape
    E = len(experts)
    F = next(e[1].shape[0] for e in experts if e is not None)
    gate = np.ascontiguousarray(gate, np.int32)
    score = _f32(score)
    cols = [[(e[i] if e is not None else None) for e in experts] for i in range(4)]
    keeps, ptrs = zip(*[_ptr_array(c) for c in cols])
    out = np.empty((T, D), np.float64)
    rc = lib().oracle_layer_forward_f64(_f(x), ctypes.c_int64(T), ctypes.c_int(D), ctypes.c_int(F), ctypes.c_int(E),
                                        ctypes.c_int(VARIANTS[variant]), _i(gate), _f(score), ptrs[0], ptrs[1],
                                        ptrs[2], ptrs[3], _d(out))
    _check(rc, "layer_forward_f64")
    del keeps
    return out


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    den = np.linalg.norm(b.ravel())
    return float(np.linalg.norm((a - b).ravel()) / (den if den > 0 else 1.0))
