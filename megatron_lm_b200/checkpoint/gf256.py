"""GF(2^8) arithmetic and erasure-code generator matrices.

Field: polynomial x^8 + x^4 + x^3 + x^2 + 1 (0x11d), generator alpha = 2.  A code with k data
and m parity members has an m x k coefficient matrix G; parity_i = XOR_j G[i][j] * data_j.
``m <= 2`` uses the Vandermonde rows G[0][j] = 1, G[1][j] = alpha^j (the classic P/Q pair,
MDS for k <= 255); larger m uses a Cauchy matrix, which is MDS by construction.  Decoding inverts
the k x k matrix formed by the surviving rows of [I; G] by Gaussian elimination in the field.
"""
from __future__ import annotations

from functools import lru_cache
from typing import List, Sequence, Tuple

import numpy as np

POLY = 0x11D


@lru_cache(maxsize=None)
def tables() -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """(exp[512], log[256], mul[256, 256]) as uint8 / int arrays."""
    exp = np.zeros(512, dtype=np.int32)
    log = np.zeros(256, dtype=np.int32)
    x = 1
    for i in range(255):
        exp[i] = x
        log[x] = i
        x <<= 1
        if x & 0x100:
            x ^= POLY
    exp[255:510] = exp[0:255]
    a = np.arange(256)
    mul = np.zeros((256, 256), dtype=np.uint8)
    nz = a[1:]
    mul[1:, 1:] = exp[(log[nz][:, None] + log[nz][None, :]) % 255].astype(np.uint8)
    return exp, log, mul


def gf_mul(a: int, b: int) -> int:
    return int(tables()[2][a, b])


def gf_inv(a: int) -> int:
    if a == 0:
        raise ZeroDivisionError("0 has no inverse in GF(256)")
    exp, log, _ = tables()
    return int(exp[(255 - log[a]) % 255])


def gf_pow(a: int, n: int) -> int:
    if n == 0:
        return 1
    if a == 0:
        return 0
    exp, log, _ = tables()
    return int(exp[(log[a] * n) % 255])


def generator_matrix(k: int, m: int) -> np.ndarray:
    if not (1 <= k and 1 <= m and k + m <= 255):
        raise ValueError("need 1 <= k, 1 <= m, k + m <= 255")
    G = np.zeros((m, k), dtype=np.uint8)
    if m <= 2:
        G[0, :] = 1
        if m == 2:
            G[1, :] = [gf_pow(2, j) for j in range(k)]
        return G
    xs = list(range(k, k + m))          # Cauchy: 1 / (x_i + y_j) with disjoint x, y
    ys = list(range(k))
    for i, x in enumerate(xs):
        for j, y in enumerate(ys):
            G[i, j] = gf_inv(x ^ y)
    return G


def gf_matinv(A: np.ndarray) -> np.ndarray:
    n = A.shape[0]
    _, _, mul = tables()
    M = np.concatenate([A.astype(np.uint8), np.eye(n, dtype=np.uint8)], axis=1)
    for c in range(n):
        piv = next((r for r in range(c, n) if M[r, c] != 0), None)
        if piv is None:
            raise np.linalg.LinAlgError("singular matrix over GF(256)")
        if piv != c:
            M[[c, piv]] = M[[piv, c]]
        M[c] = mul[gf_inv(int(M[c, c]))][M[c]]
        for r in range(n):
            if r != c and M[r, c] != 0:
                M[r] ^= mul[int(M[r, c])][M[c]]
    return M[:, n:].copy()


def decode_matrix(k: int, m: int, present: Sequence[int], wanted: Sequence[int]) -> Tuple[np.ndarray, List[int]]:
    """Rows that rebuild the members ``wanted`` (indices 0..k-1 data, k..k+m-1 parity) from
    the first k members of ``present``.  Returns (matrix [len(wanted), k], members used)."""
    present = [p for p in present]
    if len(present) < k:
        raise ValueError(f"{len(present)} members survive, {k} needed")
    use = present[:k]
    full = np.concatenate([np.eye(k, dtype=np.uint8), generator_matrix(k, m)], axis=0)
    inv = gf_matinv(full[use])                       # data = inv @ members[use]
    _, _, mul = tables()
    rows = []
    for w in wanted:
        coeff = full[w]                              # member w = coeff @ data = (coeff @ inv) @ members[use]
        row = np.zeros(k, dtype=np.uint8)
        for t in range(k):
            if coeff[t]:
                row ^= mul[int(coeff[t])][inv[t]]
        rows.append(row)
    return np.stack(rows), use


def apply_matrix_numpy(M: np.ndarray, members: Sequence[np.ndarray]) -> List[np.ndarray]:
    """out_i = XOR_j M[i][j] * members[j] on uint8 arrays (table lookups; the CPU oracle)."""
    _, _, mul = tables()
    outs = []
    for i in range(M.shape[0]):
        acc = np.zeros_like(members[0])
        for j, d in enumerate(members):
            c = int(M[i, j])
            if c == 0:
                continue
            acc ^= d if c == 1 else mul[c][d]
        outs.append(acc)
    return outs
