"""Shared helpers of the test-suite: seeded synthetic data with the shapes and value distributions of
the benchmark configurations (anisotropic Gaussian rows, L2-normalised; clustered low-dim rows)."""
import numpy as np


def anisotropic(n: int, dim: int, seed: int, offset: int = 0) -> np.ndarray:
    """Rows N(0,1) * s with s = exp(0.5*N(0,1)) drawn once per dimension from `seed`, then L2-normalised.
    `offset` selects a different row stream (queries) under the same per-dimension scale."""
    s = np.exp(0.5 * np.random.default_rng(seed).standard_normal(dim))
    x = np.random.default_rng(seed * 7919 + 13 + offset).standard_normal((n, dim)) * s
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    return np.ascontiguousarray(x, dtype=np.float32)


def clustered(n: int, dim: int, seed: int, n_clusters: int = 1000, sigma: float = 0.3, offset: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    centres = rng.standard_normal((n_clusters, dim))
    r2 = np.random.default_rng(seed * 31 + 7 + offset)
    x = centres[r2.integers(0, n_clusters, n)] + sigma * r2.standard_normal((n, dim))
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    return np.ascontiguousarray(x, dtype=np.float32)


def assert_topk_equal(scores, slots, ref_scores, ref_slots, rel=1e-4):
    """Identical id lists except for ties inside `rel`; scores within `rel` relative."""
    assert scores.shape == ref_scores.shape and slots.shape == ref_slots.shape
    denom = np.maximum(np.abs(ref_scores), 1e-30)
    assert np.all(np.abs(scores - ref_scores) <= rel * denom + 1e-30), "scores differ beyond tolerance"
    bad = np.argwhere(slots != ref_slots)
    for q, j in bad:
        # an id mismatch is acceptable only where the reference scores tie within tolerance
        s = ref_scores[q, j]
        assert abs(scores[q, j] - s) <= rel * max(abs(s), 1e-30), f"query {q} rank {j}: ids differ without a tie"
