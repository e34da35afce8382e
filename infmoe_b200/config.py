"""MoELayerConfig: same dataclass as the reference's python/infmoe/config.py:9-54
(eleven fields and three generate_* helpers with the same names).

Two deliberate differences from the reference helper:
  * generate_random_weight_file writes `wo_weight` C-contiguous.  The reference
    saves a transposed view (config.py:52), which numpy stores with
    fortran_order=True and the reference's C++ reader then misreads;
  * a `seed` argument (default None = unseeded, like the reference) makes the
    helpers reproducible.
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from typing import Optional

import numpy as np


@dataclass
class MoELayerConfig:
    r"""
    Configuration for MoE layer
    """

    seq_len: int
    expert_count: int
    embedding_size: int
    hidden_size: int
    max_concurrency: int
    moe_variant: str
    sublayer_type: str
    max_batch_size: int
    expert_centroids: Optional[np.ndarray]
    layernorm_weight: Optional[np.ndarray]
    weight_file_path: str

    def generate_random_centroids(self, seed: Optional[int] = None) -> None:
        rng = np.random.default_rng(seed)
        self.expert_centroids = rng.random((self.expert_count, self.embedding_size), dtype=np.float32)

    def generate_random_layernorm_weight(self, seed: Optional[int] = None) -> None:
        rng = np.random.default_rng(seed)
        self.layernorm_weight = rng.random(self.embedding_size, dtype=np.float32)

    def generate_random_weight_file(self, weight_path: str, overwrite: bool, seed: Optional[int] = None):
        if os.path.isfile(weight_path):
            if overwrite:
                os.remove(weight_path)
            else:
                print(f'WARNING: weight file to generate exists: {weight_path}', file=sys.stderr)
                self.weight_file_path = weight_path
                return
        rng = np.random.default_rng(seed)
        weights = {}
        # like the reference, one random matrix is shared by all experts (config.py:45-53)
        layer_norm_weight = rng.random(self.embedding_size, dtype=np.float32)
        w_weight = rng.random((self.hidden_size, self.embedding_size), dtype=np.float32)
        wo = np.ascontiguousarray(w_weight.transpose())
        for i in range(self.expert_count):
            weights[f'{i}/layer_norm_weight'] = layer_norm_weight
            weights[f'{i}/wi_0_weight'] = w_weight
            weights[f'{i}/wi_1_weight'] = w_weight
            weights[f'{i}/wo_weight'] = wo
        np.savez(weight_path, **weights)
        self.weight_file_path = weight_path if weight_path.endswith('.npz') else weight_path + '.npz'
