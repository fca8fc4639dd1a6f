"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations: weights ~ N(0, 0.02) quantized by the oracle's restatement of the
reference quantizers, activations ~ N(0, 1)."""
import numpy as np

import orc


def weights(ty, n, k, seed=0, period=None):
    """uint8 [n, row_size].  With `period`, only that many distinct rows are quantized and
    the matrix repeats them (full-size matrices whose outputs must then repeat too)."""
    rows = n if period is None else min(period, n)
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    q = orc.quantize_rows(ty, w)
    if rows < n:
        reps = (n + rows - 1) // rows
        q = np.tile(q, (reps, 1))[:n]
    return np.ascontiguousarray(q)


def activations(m, k, seed=1):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((m, k)).astype(np.float32)
