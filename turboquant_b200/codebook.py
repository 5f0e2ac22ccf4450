"""Lloyd-Max code books for one coordinate of a random unit vector.

After the random rotation a coordinate of a unit vector in R^d has density
f(x) = Gamma(d/2) / (sqrt(pi) Gamma((d-1)/2)) * (1 - x^2)^((d-3)/2) on [-1, 1].
The code book for b bits is the 2^b-level scalar quantiser that minimises the
mean squared error under f (reference codebook.py:68-143).

The JSON files under codebooks/ were produced by the reference's solver
(codebooks/make_codebooks.py) and are what the kernels use, so both sides of
a parity test see the same constants to the bit.  `compute_lloyd_max_codebook`
is this package's own solver for other (d, bits); it reproduces the shipped
files (tests/test_host_logic_cpu.py).
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
    """Lloyd-Max iteration with closed-form cell integrals.

    Under f, mass, first and second moment of a cell have closed forms: the
    CDF and the truncated second moment are regularised incomplete beta
    functions of x^2, and x f(x) has the antiderivative
    -c (1 - x^2)^((d-1)/2) / (d - 1).  The iteration itself follows the
    reference (codebook.py:68-143): centroids start at the quantile midpoints
    of a 10000-point cumulative sum, every step moves them to the conditional
    means of the cells between their midpoints, and it stops when the cost
    changes by less than `tol`.  Starting point and stopping rule are part of
    the result (the cost is flat around the optimum), so with them this solver
    reproduces the shipped JSON files to ~1e-13.

    Returns the same dictionary keys as the reference: centroids, boundaries
    (with the outer edges -1 and 1), mse_per_coord, mse_total, d, bits.
    """
    from scipy import special          # the reference's solver needs scipy too (setup.py:16)
    if d < 3 or bits < 1:
        raise ValueError("need d >= 3 and bits >= 1")
    n = 2 ** bits
    a = (d - 1) / 2.0
    log_c = _log_norm_const(d)

    def cdf(x):
        return 0.5 + 0.5 * np.sign(x) * special.betainc(0.5, a, np.minimum(x * x, 1.0))

    def first_moment(x):               # antiderivative of x f(x)
        with np.errstate(divide="ignore"):
            return -np.exp(log_c + a * np.log1p(-np.minimum(x * x, 1.0))) / (d - 1)

    def second_moment(x):              # integral of t^2 f(t) over [-1, x]; E[x^2] = 1/d
        return (0.5 + 0.5 * np.sign(x) * special.betainc(1.5, a, np.minimum(x * x, 1.0))) / d

    def edges_of(c):
        return np.concatenate([[-1.0], 0.5 * (c[:-1] + c[1:]), [1.0]])

    grid = np.linspace(-1 + 1e-10, 1 - 1e-10, 10000)
    cum = np.cumsum(beta_pdf(grid, d)) * (grid[1] - grid[0])
    cum /= cum[-1]
    centroids = np.array([grid[min(int(np.searchsorted(cum, (i + 0.5) / n)), len(grid) - 1)] for i in range(n)])
    prev = float("inf")
    cost = prev
    for _ in range(max_iter):
        e = edges_of(centroids)
        mass, mom = np.diff(cdf(e)), np.diff(first_moment(e))
        centroids = np.where(mass < 1e-30, 0.5 * (e[:-1] + e[1:]), mom / np.maximum(mass, 1e-300))
        e = edges_of(centroids)
        cost = float(np.sum(np.diff(second_moment(e)) - 2.0 * centroids * np.diff(first_moment(e))
                            + centroids * centroids * np.diff(cdf(e))))
        if abs(prev - cost) < tol:
            break
        prev = cost
    return {"centroids": centroids.tolist(), "boundaries": edges_of(centroids).tolist(), "mse_per_coord": cost,
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


def main(argv=None) -> None:
    """`python -m turboquant_b200.codebook D BITS [OUT.json]`: solve a code book for another head
    dimension (e.g. 576 for an MLA latent of 512 + 64) and print it or write it as JSON."""
    import sys
    args = list(sys.argv[1:] if argv is None else argv)
    if len(args) not in (2, 3):
        raise SystemExit("usage: python -m turboquant_b200.codebook D BITS [OUT.json]")
    book = compute_lloyd_max_codebook(int(args[0]), int(args[1]))
    text = json.dumps(book, indent=2)
    if len(args) == 3:
        with open(args[2], "w") as fh:
            fh.write(text)
    else:
        print(text)


if __name__ == "__main__":
    main()
