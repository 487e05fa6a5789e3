"""Real-basis Clebsch-Gordan (Wigner 3j) tensors and their sparse term lists.

Numerical conventions follow the reference (``src/lunatp/utils/cg.py:102-180``, which follows e3nn 0.6):

* SU(2) coefficients ``<j1 m1 j2 m2 | j3 m3>`` in the Condon-Shortley phase convention;
* real spherical basis obtained with the unitary ``Q_l`` whose rows are complex ``m = -l..l`` and whose columns
  are the real components, including the global phase ``(-i)^l``;
* the real tensor is divided by its Frobenius norm, so ``sum(C**2) == 1``;
* ``cg_terms`` keeps entries with ``|c * path_weight| > 1e-12`` in ``(i, j, k)`` lexicographic order
  (``src/lunatp/utils/cg.py:31-41``).

The SU(2) part here is Racah's closed form evaluated in exact rational arithmetic, so coefficients are correct to
the last bit of the final square root for any degree.
"""

from __future__ import annotations

from fractions import Fraction
from functools import lru_cache
from math import factorial, sqrt

import numpy as np

CG_COEFFICIENT_THRESHOLD = 1.0e-12


def _su2_coefficient(j1: int, m1: int, j2: int, m2: int, j3: int, m3: int) -> float:
    """Racah's formula for integer spins; returns 0 outside the selection rules."""
    if m3 != m1 + m2 or not abs(j1 - j2) <= j3 <= j1 + j2:
        return 0.0
    if abs(m1) > j1 or abs(m2) > j2 or abs(m3) > j3:
        return 0.0
    f = factorial
    triangle = Fraction(
        (2 * j3 + 1) * f(j3 + j1 - j2) * f(j3 - j1 + j2) * f(j1 + j2 - j3),
        f(j1 + j2 + j3 + 1),
    )
    magnetic = f(j3 + m3) * f(j3 - m3) * f(j1 - m1) * f(j1 + m1) * f(j2 - m2) * f(j2 + m2)
    series = Fraction(0)
    k_lo = max(0, j2 - j3 - m1, j1 - j3 + m2)
    k_hi = min(j1 + j2 - j3, j1 - m1, j2 + m2)
    for k in range(k_lo, k_hi + 1):
        denominator = (
            f(k) * f(j1 + j2 - j3 - k) * f(j1 - m1 - k) * f(j2 + m2 - k)
            * f(j3 - j2 + m1 + k) * f(j3 - j1 - m2 + k)
        )
        series += Fraction((-1) ** k, denominator)
    squared = triangle * magnetic * series * series
    value = sqrt(float(squared.numerator) / float(squared.denominator)) if squared else 0.0
    return value if series >= 0 else -value


@lru_cache(maxsize=None)
def su2_clebsch_gordan(j1: int, j2: int, j3: int) -> np.ndarray:
    """Dense ``[2j1+1, 2j2+1, 2j3+1]`` table indexed by ``(j1+m1, j2+m2, j3+m3)``."""
    table = np.zeros((2 * j1 + 1, 2 * j2 + 1, 2 * j3 + 1), dtype=np.float64)
    for m1 in range(-j1, j1 + 1):
        for m2 in range(-j2, j2 + 1):
            m3 = m1 + m2
            if abs(m3) <= j3:
                table[j1 + m1, j2 + m2, j3 + m3] = _su2_coefficient(j1, m1, j2, m2, j3, m3)
    table.setflags(write=False)
    return table


@lru_cache(maxsize=None)
def real_to_complex_basis(l: int) -> np.ndarray:
    """Unitary ``Q`` with ``Y_complex = Q @ Y_real`` in the reference's ordering and phase."""
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    inv_sqrt2 = 1.0 / sqrt(2.0)
    for m in range(1, l + 1):
        sign = (-1.0) ** m
        # negative m row
        q[l - m, l + m] = inv_sqrt2
        q[l - m, l - m] = -1j * inv_sqrt2
        # positive m row
        q[l + m, l + m] = sign * inv_sqrt2
        q[l + m, l - m] = 1j * sign * inv_sqrt2
    q[l, l] = 1.0
    q = ((-1j) ** l) * q
    q.setflags(write=False)
    return q


@lru_cache(maxsize=None)
def _wigner_3j_cached(l1: int, l2: int, l3: int) -> np.ndarray:
    q1, q2, q3 = real_to_complex_basis(l1), real_to_complex_basis(l2), real_to_complex_basis(l3)
    su2 = su2_clebsch_gordan(l1, l2, l3).astype(np.complex128)
    real = np.einsum("ai,bj,ck,abc->ijk", q1, q2, np.conj(q3), su2)
    if not np.all(np.abs(real.imag) < 1e-5):
        raise ArithmeticError(f"real-basis coupling ({l1},{l2},{l3}) has an imaginary part")
    real = np.ascontiguousarray(real.real)
    real /= np.linalg.norm(real)
    real.setflags(write=False)
    return real


def wigner_3j(l1: int, l2: int, l3: int) -> np.ndarray:
    """Real-basis coupling tensor ``[2l1+1, 2l2+1, 2l3+1]`` in float64 (read-only array)."""
    for degree in (l1, l2, l3):
        if not isinstance(degree, int) or degree < 0:
            raise ValueError("degrees must be nonnegative integers")
    if not abs(l2 - l3) <= l1 <= l2 + l3:
        raise ValueError(f"({l1},{l2},{l3}) violates the triangle inequality")
    return _wigner_3j_cached(l1, l2, l3)


def cg_terms(l1: int, l2: int, l3: int, path_weight: float) -> list[tuple[int, int, int, float]]:
    """Sparse ``(i, j, k, coefficient * path_weight)`` list in lexicographic order."""
    tensor = wigner_3j(l1, l2, l3)
    terms = []
    for i in range(tensor.shape[0]):
        for j in range(tensor.shape[1]):
            for k in range(tensor.shape[2]):
                value = float(tensor[i, j, k]) * path_weight
                if abs(value) > CG_COEFFICIENT_THRESHOLD:
                    terms.append((i, j, k, value))
    return terms


__all__ = ["wigner_3j", "cg_terms", "su2_clebsch_gordan", "real_to_complex_basis", "CG_COEFFICIENT_THRESHOLD"]
