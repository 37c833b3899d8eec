"""Seeded synthetic KV tensors with the value distribution of the benchmark
configs: x = z * s, z ~ N(0,1), s per (layer, head, channel) ~ lognormal(0, 0.5)."""
import numpy as np


def synthetic_kv(n_vectors: int, dim: int, seed: int = 0, groups: int = 8) -> np.ndarray:
    rng = np.random.default_rng(seed)
    scale = rng.lognormal(0.0, 0.5, size=(groups, dim)).astype(np.float32)
    z = rng.standard_normal((n_vectors, dim)).astype(np.float32)
    g = np.arange(n_vectors) % groups
    return (z * scale[g]).astype(np.float32)
