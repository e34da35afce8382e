"""Seeded synthetic workloads for the MoE layer (there is no dataset on this path).

The five named configurations are the ones the benchmark and the parity tests
run.  Small tensors (input, centroids, LayerNorm weights) come from numpy's
Philox generator keyed by (seed, tensor id), so every tensor can be regenerated
independently.  Expert matrices come either from numpy (small cases, and the
npz fixtures) or, for the multi-gigabyte cases, from a seeded torch CUDA
generator directly in device memory (one seed per expert, so a single expert
can be regenerated or copied back for the checker).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict, Optional, Tuple

import numpy as np

# tensor ids for the Philox key
_ID_X, _ID_CENTROIDS, _ID_GATING_LN, _ID_ZIPF_PERM, _ID_EXPERT0 = 0, 1, 2, 3, 16


@dataclass(frozen=True)
class Workload:
    name: str
    variant: str              # "default" | "cpm_2" | "base_layer"
    expert_count: int
    embedding_size: int       # d_model
    hidden_size: int          # d_ff
    batch: int
    seq_len: int
    max_concurrency: int = 2
    seed: int = 1234
    zipf_s: float = 0.0       # > 0: skewed routing (a few experts take most tokens)
    streamed: bool = False    # experts streamed from pinned host memory instead of resident

    @property
    def tokens(self) -> int:
        return self.batch * self.seq_len

    @property
    def shape(self) -> Tuple[int, int, int]:
        return (self.batch, self.seq_len, self.embedding_size)

    def ffn_flops(self, tokens: Optional[int] = None) -> float:
        """Useful flops of the three expert GEMMs: 6 * T * D * F."""
        t = self.tokens if tokens is None else tokens
        return 6.0 * t * self.embedding_size * self.hidden_size

    def expert_bytes(self) -> int:
        return 4 * (3 * self.embedding_size * self.hidden_size + self.embedding_size)


WORKLOADS: Dict[str, Workload] = {
    # correctness anchor, runs anywhere
    "tiny_default": Workload("tiny_default", "default", 4, 64, 256, 2, 16, seed=1234),
    # the configuration the headline metric is quoted on
    "cpm2": Workload("cpm2", "cpm_2", 32, 4096, 10240, 8, 512, seed=1235),
    # same per-tile shapes as cpm2 (d_model, tokens per expert) with a quarter of the experts and half the
    # d_ff: small enough (2 GB of weights, still far beyond L2) to capture under a profiler
    "cpm2_profile": Workload("cpm2_profile", "cpm_2", 8, 4096, 5120, 2, 512, seed=1235),
    # the row-wise kernels (routing, dispatch, scatter + LayerNorm) at exactly the shapes of cpm2 -- same tokens,
    # d_model and expert count -- with a d_ff of 512, so that the whole layer holds 0.8 GB: for profiler captures
    "cpm2_rows_profile": Workload("cpm2_rows_profile", "cpm_2", 32, 4096, 512, 8, 512, seed=1235),
    # skewed routing, stresses the grouped GEMM's load balance
    "base_layer_zipf": Workload("base_layer_zipf", "base_layer", 64, 1024, 4096, 16, 1024, seed=1236, zipf_s=1.1),
    # expert-parallel case (sharded over 2/4/8 GPUs)
    "ep_cpm2": Workload("ep_cpm2", "cpm_2", 128, 4096, 10240, 128, 512, seed=1237),
    # decode regime with streamed experts
    "offload_t1": Workload("offload_t1", "cpm_2", 32, 4096, 10240, 1, 1, seed=1238, streamed=True),
    "offload_t8": Workload("offload_t8", "cpm_2", 32, 4096, 10240, 1, 8, seed=1238, streamed=True),
    "offload_t64": Workload("offload_t64", "cpm_2", 32, 4096, 10240, 1, 64, seed=1238, streamed=True),
}


def scaled(w: Workload, **kw) -> Workload:
    """A smaller/larger variant of a named workload (same distributions)."""
    return replace(w, **kw)


def _rng(seed: int, tensor_id: int, sub: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[(seed << 20) ^ tensor_id, sub]))


def gen_inputs(w: Workload):
    """-> x f32[T][D] ~ N(0,1), centroids f32[E][D] ~ N(0, 0.02), gating LayerNorm weight f32[D] (cpm_2) or None."""
    T, D, E = w.tokens, w.embedding_size, w.expert_count
    x = _rng(w.seed, _ID_X).standard_normal((T, D), dtype=np.float32)
    cent = (_rng(w.seed, _ID_CENTROIDS).standard_normal((E, D), dtype=np.float32) * np.float32(0.02))
    ln = None
    if w.variant == "cpm_2":
        ln = (1.0 + 0.01 * _rng(w.seed, _ID_GATING_LN).standard_normal(D, dtype=np.float32)).astype(np.float32)
    if w.zipf_s > 0:
        # The reference has no gate bias, so the skew goes through the data: feature 0 is a
        # constant 1 and centroid column 0 carries tau * ln p_e with p_e ~ rank^-s.
        ranks = _rng(w.seed, _ID_ZIPF_PERM).permutation(E) + 1
        p = ranks.astype(np.float64) ** (-w.zipf_s)
        p /= p.sum()
        score_std = 0.02 * np.sqrt(D - 1)             # std of the unbiased part of a score
        tau = np.sqrt(6.0) / np.pi * score_std         # Gumbel scale with that std
        x[:, 0] = 1.0
        cent[:, 0] = (tau * np.log(p)).astype(np.float32)
    return x, cent, ln


def gen_expert_numpy(w: Workload, e: int):
    """One expert's weights on the host: ln 1+N(0,0.01), wi ~ N(0, 1/sqrt(D)), wo ~ N(0, 1/sqrt(F))."""
    D, F = w.embedding_size, w.hidden_size
    r = _rng(w.seed, _ID_EXPERT0, e)
    ln = (1.0 + 0.01 * r.standard_normal(D, dtype=np.float32)).astype(np.float32)
    wi0 = r.standard_normal((F, D), dtype=np.float32) * np.float32(1.0 / np.sqrt(D))
    wi1 = r.standard_normal((F, D), dtype=np.float32) * np.float32(1.0 / np.sqrt(D))
    wo = r.standard_normal((D, F), dtype=np.float32) * np.float32(1.0 / np.sqrt(F))
    return ln, wi0, wi1, wo


def gen_expert_torch(w: Workload, e: int, device):
    """Same distributions, generated in device memory (seeded per expert)."""
    import torch

    D, F = w.embedding_size, w.hidden_size
    g = torch.Generator(device=device)
    g.manual_seed((w.seed << 20) + e)
    ln = 1.0 + 0.01 * torch.randn(D, generator=g, device=device, dtype=torch.float32)
    wi0 = torch.randn(F, D, generator=g, device=device, dtype=torch.float32) * (1.0 / np.sqrt(D))
    wi1 = torch.randn(F, D, generator=g, device=device, dtype=torch.float32) * (1.0 / np.sqrt(D))
    wo = torch.randn(D, F, generator=g, device=device, dtype=torch.float32) * (1.0 / np.sqrt(F))
    return ln, wi0, wi1, wo


def write_npz(w: Workload, path: str, compressed: bool = False) -> str:
    """Writes the expert weight file in the reference's key layout (C-contiguous arrays)."""
    arrays = {}
    for e in range(w.expert_count):
        ln, wi0, wi1, wo = gen_expert_numpy(w, e)
        arrays[f"{e}/layer_norm_weight"] = ln
        arrays[f"{e}/wi_0_weight"] = wi0
        arrays[f"{e}/wi_1_weight"] = wi1
        arrays[f"{e}/wo_weight"] = wo
    (np.savez_compressed if compressed else np.savez)(path, **arrays)
    return path if path.endswith(".npz") else path + ".npz"
