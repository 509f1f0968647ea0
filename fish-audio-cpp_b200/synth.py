"""Seeded synthetic workloads with the value distributions the headline configurations name.

Activations: fp16 N(0,1) with 0.5 % of the K channels (chosen once per case, shared by all
tokens) scaled x20. Weights: int8 uniform integers in [-127, 127], row-major [N, K]. Weight
scales: fp16 uniform in [1e-3, 5e-3], one per (row, K-group). numpy only, so the same arrays
feed the CPU oracle and (after upload) the CUDA library.
"""
from __future__ import annotations

import numpy as np

# The slow-AR projections: name -> (K, N). gate_up is the two 9728-row matrices, packed; gate is one of them
# alone (w1 as the reference runs it, src/engine/dual_ar_engine.cc:640-644): the single-GEMM headline case.
PROJECTIONS = {"qkv": (2560, 6144), "o": (4096, 2560), "gate_up": (2560, 19456), "down": (9728, 2560),
               "gate": (2560, 9728)}
# The four projections of a layer (the decode sweep and the prefill cases run over these).
LAYER_PROJECTIONS = ("qkv", "o", "gate_up", "down")


def num_groups(K: int, g: int) -> int:
    g = K if g <= 0 or g > K else g
    return (K + g - 1) // g


def activations(rng: np.random.Generator, M: int, K: int, outlier_frac: float = 0.005,
                outlier_gain: float = 20.0) -> np.ndarray:
    x = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    n_out = max(1, int(round(outlier_frac * K)))
    idx = rng.choice(K, size=n_out, replace=False)
    x[:, idx] = (x[:, idx].astype(np.float32) * outlier_gain).astype(np.float16)
    return x


def weights(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    return rng.integers(-127, 128, size=(N, K), dtype=np.int8)


def weight_scales(rng: np.random.Generator, N: int, G: int) -> np.ndarray:
    s = rng.uniform(1e-3, 5e-3, size=(N, G)).astype(np.float16)
    return s if G > 1 else s.reshape(N)


def linear_case(seed: int, M: int, N: int, K: int, g: int):
    """(X fp16 [M,K], W int8 [N,K], ws fp16 [N,G] or [N]) for one seeded case."""
    rng = np.random.default_rng(seed)
    return activations(rng, M, K), weights(rng, N, K), weight_scales(rng, N, num_groups(K, g))
