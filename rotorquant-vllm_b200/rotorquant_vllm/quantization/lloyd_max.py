"""Lloyd-Max scalar codebooks for the coordinates of a randomly rotated unit vector.

A coordinate of a rotated ``d``-dimensional unit vector has density
``Gamma(d/2) / (sqrt(pi) Gamma((d-1)/2)) (1 - x^2)^((d-3)/2)`` on ``[-1, 1]``,
which for ``d >= 64`` is very close to ``N(0, 1/d)``.  The codebook is the fixed
point of the Lloyd-Max iteration (boundaries = midpoints of neighbouring
centroids, centroids = conditional means), evaluated with
``scipy.integrate.quad`` on the host.

Mirrors src/rotorquant_vllm/quantization/lloyd_max.py of the reference
(``solve_lloyd_max`` :32-86, ``compute_expected_distortion`` :89-104,
``LloydMaxCodebook`` :107-124): same start point, same integration limits,
same stopping rule, so the fp32 centroids and boundaries come out bit for bit
the same -- including the 3-bit middle boundary, which is integration noise of
order -1e-17 rather than an exact zero, and decides how exact zeros are coded.
"""

from __future__ import annotations

import math

import torch
from scipy import integrate

_SPAN_SIGMAS = 3.5      # centroids start uniformly inside +-3.5 sigma
_OUTER_FACTOR = 3       # outermost cells integrate out to +-3 * 3.5 sigma
_MIN_MASS = 1e-15       # a cell with less probability keeps its centroid


def beta_pdf(x: float, d: int) -> float:
    """Exact density of one coordinate of a random point on the unit sphere in ``d`` dimensions."""
    if abs(x) >= 1.0:
        return 0.0
    coeff = math.gamma(d / 2) / (math.sqrt(math.pi) * math.gamma((d - 1) / 2))
    return coeff * (1 - x * x) ** ((d - 3) / 2)


def gaussian_approx_pdf(x: float, d: int) -> float:
    """``N(0, 1/d)`` density."""
    sigma2 = 1.0 / d
    return (1.0 / math.sqrt(2 * math.pi * sigma2)) * math.exp(-x * x / (2 * sigma2))


def _density(d: int, use_exact: bool):
    if use_exact:
        return lambda x: beta_pdf(x, d)
    return lambda x: gaussian_approx_pdf(x, d)


def _cell_edges(boundaries: list[float], lo: float, hi: float) -> list[float]:
    return [lo * _OUTER_FACTOR, *boundaries, hi * _OUTER_FACTOR]


def _midpoints(centroids: list[float]) -> list[float]:
    return [(left + right) / 2.0 for left, right in zip(centroids[:-1], centroids[1:])]


def solve_lloyd_max(d: int, bits: int, use_exact: bool = False, max_iter: int = 200,
                    tol: float = 1e-10):
    """Centroids (``2**bits``) and boundaries (``2**bits - 1``) as sorted fp32 tensors."""
    levels = 2 ** bits
    pdf = _density(d, use_exact)
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -_SPAN_SIGMAS * sigma, _SPAN_SIGMAS * sigma
    centroids = [lo + (hi - lo) * (i + 0.5) / levels for i in range(levels)]

    def first_moment(x):
        return x * pdf(x)

    for _ in range(max_iter):
        edges = _cell_edges(_midpoints(centroids), lo, hi)
        updated = []
        for i, (a, b) in enumerate(zip(edges[:-1], edges[1:])):
            moment, _ = integrate.quad(first_moment, a, b)
            mass, _ = integrate.quad(pdf, a, b)
            updated.append(moment / mass if mass > _MIN_MASS else centroids[i])
        shift = max(abs(n - o) for n, o in zip(updated, centroids))
        centroids = updated
        if shift < tol:
            break

    return (torch.tensor(centroids, dtype=torch.float32),
            torch.tensor(_midpoints(centroids), dtype=torch.float32))


def compute_expected_distortion(d: int, bits: int, centroids: torch.Tensor,
                                boundaries: torch.Tensor, use_exact: bool = False) -> float:
    """Expected squared error per coordinate of the given codebook."""
    pdf = _density(d, use_exact)
    sigma = 1.0 / math.sqrt(d)
    edges = _cell_edges(boundaries.tolist(), -_SPAN_SIGMAS * sigma, _SPAN_SIGMAS * sigma)
    total = 0.0
    for i, (a, b) in enumerate(zip(edges[:-1], edges[1:])):
        c = centroids[i].item()
        part, _ = integrate.quad(lambda x: (x - c) ** 2 * pdf(x), a, b)
        total += part
    return total


class LloydMaxCodebook:
    """Codebook for dimension ``d`` and ``bits`` bits per coordinate."""

    def __init__(self, d: int, bits: int, use_exact: bool = False):
        self.d = d
        self.bits = bits
        self.n_levels = 2 ** bits
        self.centroids, self.boundaries = solve_lloyd_max(d, bits, use_exact)
        self.distortion = compute_expected_distortion(d, bits, self.centroids, self.boundaries,
                                                      use_exact)

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        """Index of the nearest centroid of every value."""
        c = self.centroids.to(x.device)
        return (x.unsqueeze(-1) - c).abs().argmin(dim=-1)

    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        """Centroid value of every index."""
        return self.centroids.to(indices.device)[indices]

    def __repr__(self) -> str:
        return (f"LloydMaxCodebook(d={self.d}, bits={self.bits}, levels={self.n_levels}, "
                f"distortion_per_coord={self.distortion:.6f})")
