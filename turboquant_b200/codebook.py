"""Lloyd-Max code books for one coordinate of a random unit vector.

After the random rotation a coordinate of a unit vector in R^d has density
f(x) = Gamma(d/2) / (sqrt(pi) Gamma((d-1)/2)) * (1 - x^2)^((d-3)/2) on [-1, 1].
The code book for b bits is the 2^b-level scalar quantiser that minimises the
mean squared error under f (reference codebook.py:68-143).

The JSON files under codebooks/ were produced by the reference's solver
(codebooks/make_codebooks.py) and are what the kernels use, so both sides of
a parity test see the same constants to the bit.  `compute_lloyd_max_codebook`
is this package's own solver for other (d, bits).
"""

from __future__ import annotations

import json
import math
import os

import numpy as np
import torch

_CODEBOOK_DIR = os.path.join(os.path.dirname(__file__), "codebooks")
_CACHE: dict[tuple[int, int], dict] = {}


def _log_norm_const(d: int) -> float:
    return math.lgamma(d / 2.0) - 0.5 * math.log(math.pi) - math.lgamma((d - 1) / 2.0)


def beta_pdf(x, d: int):
    """Density of one coordinate of a uniform point on the sphere S^(d-1)."""
    if d < 3:
        raise ValueError("need d >= 3")
    x = np.clip(np.asarray(x, dtype=np.float64), -1 + 1e-15, 1 - 1e-15)
    return np.exp(_log_norm_const(d) + 0.5 * (d - 3) * np.log1p(-x * x))


def compute_lloyd_max_codebook(d: int, bits: int, max_iter: int = 200, tol: float = 1e-12) -> dict:
    """Lloyd-Max iteration on a fine grid (composite Simpson weights).

    Returns the same dictionary keys as the reference: centroids, boundaries
    (with the outer edges -1 and 1), mse_per_coord, mse_total, d, bits.
    """
    n = 2 ** bits
    m = 400_001                                     # odd number of grid points
    half_width = min(1.0, 12.0 / math.sqrt(d))      # the density is negligible outside
    xs = np.linspace(-half_width, half_width, m)
    w = np.ones(m)
    w[1:-1:2] = 4.0
    w[2:-1:2] = 2.0
    w *= (xs[1] - xs[0]) / 3.0
    pw = beta_pdf(xs, d) * w
    cdf = np.cumsum(pw)
    cdf /= cdf[-1]
    centroids = np.array([xs[min(np.searchsorted(cdf, (i + 0.5) / n), m - 1)] for i in range(n)])
    prev = float("inf")
    cost = prev
    for _ in range(max_iter):
        edges = np.concatenate([[-1.0], 0.5 * (centroids[:-1] + centroids[1:]), [1.0]])
        cell = np.clip(np.searchsorted(edges, xs, side="right") - 1, 0, n - 1)
        mass = np.bincount(cell, weights=pw, minlength=n)
        mom = np.bincount(cell, weights=pw * xs, minlength=n)
        centroids = np.where(mass > 1e-30, mom / np.maximum(mass, 1e-300), 0.5 * (edges[:-1] + edges[1:]))
        cost = float(np.sum(pw * (xs - centroids[cell]) ** 2))
        if abs(prev - cost) < tol:
            break
        prev = cost
    edges = np.concatenate([[-1.0], 0.5 * (centroids[:-1] + centroids[1:]), [1.0]])
    return {"centroids": centroids.tolist(), "boundaries": edges.tolist(), "mse_per_coord": cost,
            "mse_total": cost * d, "d": d, "bits": bits}


def get_codebook(d: int, bits: int) -> dict:
    """Code book for (d, bits): shipped JSON if present, else solved (not written to disk)."""
    key = (d, bits)
    if key not in _CACHE:
        path = os.path.join(_CODEBOOK_DIR, f"codebook_d{d}_b{bits}.json")
        if os.path.exists(path):
            with open(path) as fh:
                _CACHE[key] = json.load(fh)
        else:
            _CACHE[key] = compute_lloyd_max_codebook(d, bits)
    return _CACHE[key]


def get_codebook_tensors(d: int, bits: int, device, dtype: torch.dtype = torch.float32):
    """(centroids (2^b,), boundaries (2^b+1,)) as tensors (reference codebook.py:176-181)."""
    cb = get_codebook(d, bits)
    return (torch.tensor(cb["centroids"], device=device, dtype=dtype),
            torch.tensor(cb["boundaries"], device=device, dtype=dtype))
