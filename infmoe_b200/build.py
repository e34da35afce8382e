"""Builds the native libraries in-tree with nvcc for sm_100a.

    python -m infmoe_b200.build          # libinfmoe_b200.so (+ libtrtmoelayer.so)

nvcc cross-compiles without a GPU.  Objects are cached under infmoe_b200/build/
and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libinfmoe_b200.so")
PLUGIN_LIB = os.path.join(PKG, "libtrtmoelayer.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH + ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden",
                     "-I", os.path.join(ROOT, "include"), "-I", CSRC]

CORE_SOURCES = ["route.cu", "dispatch.cu", "rows.cu", "ffn_simt.cu", "ffn_umma.cu", "layer.cu", "ep.cu", "npz.cc"]
PLUGIN_SOURCES = ["plugin/MoELayerPlugin.cc", "plugin/MoELayerPluginCreator.cc", "plugin/host_driver.cc"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "nvcc"
    for p in (cand, "/usr/local/cuda/bin/nvcc"):
        try:
            subprocess.run([p, "--version"], check=True, capture_output=True)
            return p
        except (OSError, subprocess.CalledProcessError):
            continue
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _headers():
    hs = []
    for d, _, files in os.walk(CSRC):
        hs += [os.path.join(d, f) for f in files if f.endswith((".h", ".cuh", ".hh"))]
    hs.append(os.path.join(ROOT, "include", "infmoe_c.h"))
    return hs


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _compile(nvcc: str, src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, src.replace("/", "_") + ".o")
    path = os.path.join(CSRC, src)
    if _stale(obj, [path] + _headers()):
        cmd = [nvcc] + NVCC_FLAGS + (["-x", "cu"] if src.endswith(".cc") else []) + ["-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def _link(nvcc: str, objs, out: str, extra, verbose: bool) -> None:
    if _stale(out, objs):
        cmd = [nvcc] + ARCH + ["-shared", "-o", out] + objs + extra
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed for {out}:\n{r.stdout}\n{r.stderr}")


def build(verbose: bool = False) -> str:
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=8) as ex:
        core = list(ex.map(lambda s: _compile(nvcc, s, verbose), CORE_SOURCES))
        plugin_srcs = [s for s in PLUGIN_SOURCES if os.path.exists(os.path.join(CSRC, s))]
        plug = list(ex.map(lambda s: _compile(nvcc, s, verbose), plugin_srcs))
    _link(nvcc, core, LIB, ["-lz", "-ldl"], verbose)
    if plug:
        _link(nvcc, plug, PLUGIN_LIB, ["-L", PKG, "-linfmoe_b200", "-Xlinker", "-rpath,$ORIGIN"], verbose)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-q" not in sys.argv))
