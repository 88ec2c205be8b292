"""Seeded synthetic inputs: random-walk C-alpha chains and the wavelength schedule.

CPU only; used by the benchmark and, through ``oracle/chains.py``, by the tests.  These generators stand in for
the PDB-derived coordinates the reference trains on (``utils/train_utils/data_utils.py:302-303``
names the datasets; none is shipped with this repository).

Chain model: ``r_0 = 0``; the first unit step is uniform on the sphere; for every
later step the virtual bond angle between ``(r_{t-1} - r_t)`` and
``(r_{t+1} - r_t)`` is uniform in [90, 120] degrees, the azimuth about the previous
step is uniform in [0, 2 pi), and every step is 3.8 Angstrom long.

Wavelength schedule (benchmark inputs): ``lambda_i = lo + (hi - lo) * (b**(2 i / d) - 1) / (b - 1)``
for ``i = 0 .. d/2 - 1``; wavenumber ``k_i = 2 pi / lambda_i``.  The reference's module
(``utils/model_utils/wf_embedding/wf_embedding.py:30-31``) uses exponents ``i / (K - 1)``
instead; that variant lives in the product's ``WaveFunctionEmbedding`` module.
"""
import math

import numpy as np

STEP = 3.8  # Angstrom between consecutive C-alpha atoms


def random_walk_chain(length, rng):
    """One chain, ``[length, 3]`` float64.  ``rng`` is a ``numpy.random.Generator``."""
    r = np.zeros((max(length, 1), 3), dtype=np.float64)
    u = rng.normal(size=3)
    u /= np.linalg.norm(u)
    if length > 1:
        r[1] = r[0] + STEP * u
    if length > 2:
        phi = np.deg2rad(rng.uniform(90.0, 120.0, size=length - 2))
        psi = rng.uniform(0.0, 2.0 * math.pi, size=length - 2)
        for t in range(2, length):
            # orthonormal frame (u, e1, e2)
            a = np.array([1.0, 0.0, 0.0]) if abs(u[0]) < 0.9 else np.array([0.0, 1.0, 0.0])
            e1 = np.cross(u, a)
            e1 /= np.linalg.norm(e1)
            e2 = np.cross(u, e1)
            c = -math.cos(phi[t - 2])  # u_t . u_{t-1} in [0, 0.5]
            s = math.sqrt(max(0.0, 1.0 - c * c))
            u = c * u + s * (math.cos(psi[t - 2]) * e1 + math.sin(psi[t - 2]) * e2)
            u /= np.linalg.norm(u)
            r[t] = r[t - 1] + STEP * u
    return r[:length]


def chain_batch(lengths, n_pad, seed):
    """Padded batch.  Returns ``coords [Z, n_pad, 3] float32`` (padding rows are 0, the
    reference's batch convention, ``utils/train_utils/data_utils.py:233-237``) and
    ``mask [Z, n_pad] bool`` with True = padded."""
    rng = np.random.default_rng(seed)
    z = len(lengths)
    coords = np.zeros((z, n_pad, 3), dtype=np.float32)
    mask = np.ones((z, n_pad), dtype=bool)
    for b, length in enumerate(lengths):
        coords[b, :length] = random_walk_chain(int(length), rng).astype(np.float32)
        mask[b, :length] = False
    return coords, mask


def draw_lengths(z, lo, hi, seed):
    """``z`` lengths uniform in ``[lo, hi]`` inclusive."""
    rng = np.random.default_rng(seed)
    return rng.integers(lo, hi + 1, size=z).astype(np.int64)


def wavenumbers(d_model=512, lam_min=3.7, lam_max=20.0, base=20.0):
    """Benchmark wavenumber schedule, ``[d_model // 2] float32``."""
    i = np.arange(d_model // 2, dtype=np.float64)
    lam = lam_min + (lam_max - lam_min) * (base ** (2.0 * i / d_model) - 1.0) / (base - 1.0)
    return (2.0 * math.pi / lam).astype(np.float32)


def sigmas(heads=8, lo=3.0, hi=15.0):
    """Per-head RBF spreads, linearly spaced, float32."""
    return np.linspace(lo, hi, heads, dtype=np.float64).astype(np.float32)
