#!/usr/bin/env python3
"""N MoE layers stacked back to back, as the reference's demo does through TensorRT
(python/examples/stacked_moe.py:12-62: same plugin instance added `moe_layers` times to one
network, random input, one timed inference).

Here the layers are enqueued directly on one CUDA stream through the C ABI: layer l reads the
output of layer l-1, nothing synchronises with the host between layers, and the device status
is read once at the end.  Weights come from an npz file in the reference's format, written by
`MoELayerConfig.generate_random_weight_file` (python/infmoe/config.py:47-66).

    python -m infmoe_b200.examples.stacked_moe --layers 3
    python -m infmoe_b200.examples.stacked_moe --layers 3 --expert-count 20 --embedding-size 4096 \
        --hidden-size 16384 --seq-len 512 --batch 80 --max-concurrency 4      # the reference demo's sizes
"""
from __future__ import annotations

import argparse
import os
import tempfile
import time

import numpy as np


def run_stacked_moe(moe_layers: int, expert_count: int, embedding_size: int, hidden_size: int, seq_len: int,
                    batch: int, max_concurrency: int, moe_variant: str, weight_file: str | None, resident: int,
                    repeats: int, return_output: bool = False) -> dict:
    import torch

    from infmoe_b200 import MoELayerConfig, MoELayerPlugin

    config = MoELayerConfig(seq_len=seq_len, expert_count=expert_count, embedding_size=embedding_size,
                            hidden_size=hidden_size, max_concurrency=max_concurrency, moe_variant=moe_variant,
                            sublayer_type="T5_FF", max_batch_size=batch, expert_centroids=None,
                            layernorm_weight=None, weight_file_path=None)
    config.generate_random_centroids(seed=1)
    if moe_variant == "cpm_2":
        config.generate_random_layernorm_weight(seed=2)
    path = weight_file or os.path.join(tempfile.gettempdir(), "moe_weight.npz")
    config.generate_random_weight_file(path, overwrite=weight_file is None, seed=3)
    print(repr(config))

    # one plugin, `moe_layers` clones sharing its weights (MoELayerPlugin.cc:83-108)
    first = MoELayerPlugin(config).create_plugin()
    first.initialize()
    first.set_residency(resident)
    layers = [first] + [first.clone() for _ in range(moe_layers - 1)]

    tokens = batch * seq_len
    dev = torch.device("cuda", torch.cuda.current_device())
    x = torch.from_numpy(np.random.default_rng(4).random((batch, seq_len, embedding_size), dtype=np.float32)).to(dev)
    bufs = [torch.empty_like(x), torch.empty_like(x)]
    workspace = torch.empty(max(l.get_workspace_size(tokens) for l in layers), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def inference():
        src = x
        for i, layer in enumerate(layers):
            dst = bufs[i & 1]
            layer.enqueue(src.data_ptr(), dst.data_ptr(), workspace.data_ptr(), workspace.numel(), tokens, stream)
            src = dst
        return src

    out = inference()                      # first pass also loads what is loaded lazily
    layers[-1].sync_status(stream)
    torch.cuda.synchronize(dev)
    start = time.time()
    for _ in range(repeats):
        out = inference()
    for layer in layers:
        layer.sync_status(stream)          # device-side findings of every layer (bad routing, a wait that ran out)
    torch.cuda.synchronize(dev)
    elapsed = (time.time() - start) / repeats
    print("Inference has cost", elapsed, "seconds")
    print("Output shape", tuple(out.shape))
    result = {"seconds": elapsed, "tokens_per_s": tokens * moe_layers / elapsed, "shape": tuple(out.shape),
              "finite": bool(torch.isfinite(out).all().item()), "weight_file": config.weight_file_path,
              "centroids": config.expert_centroids, "layernorm_weight": config.layernorm_weight}
    if return_output:
        result["input"] = x.cpu().numpy()
        result["output"] = out.cpu().numpy()
    for layer in layers[1:]:
        layer.terminate()
    first.terminate()
    return result


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--expert-count", type=int, default=8)
    ap.add_argument("--embedding-size", type=int, default=1024)
    ap.add_argument("--hidden-size", type=int, default=4096)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--max-concurrency", type=int, default=4)
    ap.add_argument("--moe-variant", default="cpm_2", choices=["cpm_2", "base_layer", "default"])
    ap.add_argument("--weight-file", default=None, help="existing npz in the reference's format (default: generate)")
    ap.add_argument("--resident", type=int, default=-1, help="-1 automatic, 0 stream experts per call, 1 keep on device")
    ap.add_argument("--repeats", type=int, default=3)
    a = ap.parse_args()
    r = run_stacked_moe(a.layers, a.expert_count, a.embedding_size, a.hidden_size, a.seq_len, a.batch,
                        a.max_concurrency, a.moe_variant, a.weight_file, a.resident, a.repeats)
    print({k: r[k] for k in ("seconds", "tokens_per_s", "shape", "finite")})


if __name__ == "__main__":
    main()
