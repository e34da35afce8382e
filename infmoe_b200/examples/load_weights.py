"""Times the expert-weight loader: npz file -> page-locked host memory (infmoe_layer_initialize).

    python -m infmoe_b200.examples.load_weights [--experts 8] [--d-model 2048] [--d-ff 8192] [--compressed]

Writes a weight file in the reference's key layout to a temporary directory, loads it with 1 and with 8 reader
threads (INFMOE_LOAD_THREADS is read once per process, so each setting runs in a child process), and prints one
JSON line with the file size, the GB/s of each setting and, for comparison, the rate at which the same file is
read sequentially into ordinary memory.  The file has just been written, so it is served from the page cache:
the figures are the loader's own ceiling (parsing, copying or inflating, page-locked destination), not a disk's.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _child(path, E, D, F):
    from infmoe_b200 import MoELayer

    cent = np.zeros((E, D), np.float32)
    layer = MoELayer.create(E, D, F, 2, cent, path, "T5_FF", "default", None)
    t0 = time.perf_counter()
    layer.initialize()
    dt = time.perf_counter() - t0
    layer.terminate()
    print(json.dumps({"seconds": dt}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-ff", type=int, default=8192)
    ap.add_argument("--compressed", action="store_true")
    ap.add_argument("--child", default=None)
    args = ap.parse_args()
    E, D, F = args.experts, args.d_model, args.d_ff
    if args.child:
        _child(args.child, E, D, F)
        return
    from infmoe_b200 import synth

    w = synth.scaled(synth.WORKLOADS["cpm2"], expert_count=E, embedding_size=D, hidden_size=F, batch=1, seq_len=1)
    with tempfile.TemporaryDirectory() as tmp:
        path = synth.write_npz(w, os.path.join(tmp, "experts.npz"), compressed=args.compressed)
        size = os.path.getsize(path)
        payload = 4 * E * (3 * D * F + D)
        t0 = time.perf_counter()
        with open(path, "rb") as f:
            while f.read(64 << 20):
                pass
        raw = size / (time.perf_counter() - t0) / 1e9
        res = {"file_bytes": size, "payload_bytes": payload, "compressed": args.compressed,
               "sequential_read_gbs": raw, "note": "file served from the page cache"}
        for threads in (1, 8):
            env = dict(os.environ, INFMOE_LOAD_THREADS=str(threads))
            out = subprocess.run([sys.executable, "-m", "infmoe_b200.examples.load_weights", "--child", path,
                                  "--experts", str(E), "--d-model", str(D), "--d-ff", str(F)], env=env, cwd=ROOT,
                                 capture_output=True, text=True, check=True).stdout.strip().splitlines()[-1]
            sec = json.loads(out)["seconds"]
            res[f"threads_{threads}"] = {"seconds": sec, "payload_gbs": payload / sec / 1e9}
    print(json.dumps(res))


if __name__ == "__main__":
    main()
