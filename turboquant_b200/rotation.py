"""Per-layer random matrices: the rotation Pi and the QJL projection S.

Same construction and seeding as the reference (rotation.py:17-56) so that a
layer's constants are identical on both sides: both are drawn on a seeded CPU
generator, Pi is the Q factor of a Gaussian matrix with the signs of diag(R)
folded in, S is plain Gaussian.
"""

from __future__ import annotations

import torch


def generate_rotation_matrix(d: int, device, dtype: torch.dtype = torch.float32, seed: int = 42) -> torch.Tensor:
    """Random orthogonal (d, d) matrix, reproducible from `seed`."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    q, r = torch.linalg.qr(torch.randn(d, d, generator=gen, dtype=torch.float32))
    q = q * torch.sign(torch.diag(r)).unsqueeze(0)
    return q.to(device=device, dtype=dtype)


def generate_qjl_matrix(d: int, device, dtype: torch.dtype = torch.float32, seed: int = 12345) -> torch.Tensor:
    """(d, d) matrix of i.i.d. N(0, 1) entries, reproducible from `seed`."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    return torch.randn(d, d, generator=gen, dtype=torch.float32).to(device=device, dtype=dtype)


def rotate_forward(x: torch.Tensor, Pi: torch.Tensor) -> torch.Tensor:
    """y = x @ Pi^T."""
    return torch.matmul(x, Pi.T)


def rotate_backward(y: torch.Tensor, Pi: torch.Tensor) -> torch.Tensor:
    """x = y @ Pi."""
    return torch.matmul(y, Pi)
