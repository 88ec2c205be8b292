"""CPU oracle for the isotropic Wavefunction Embedding (test infrastructure).

Restates the reference's dense PyTorch formulation, ``wf_embedding_torch`` in
``tests/wf_embed/wf_embed.py:91-129``, with the observer axis processed in chunks so
that long sequences fit in host memory (the unchunked intermediate is
``Z*N*N*K*4`` bytes).  The reference sums over its axis 1; because distances and the
pair mask are symmetric this equals summing over the source axis, which is what the
chunked form does (sources stay on axis 1, observers move to axis 2).

Pinned against the reference function itself: ``tests/golden/make_golden.py`` extracts
``wf_embedding_torch`` from the reference tree, runs it on seeded inputs and stores the
outputs; ``tests/test_oracle_we.py`` checks this restatement reproduces them bit for bit.
The reference function ignores ``dropout_p``; the reference *kernel* does not.  Its index-hash dropout
(``isotropic/cuda/wf_embedding_kernel.cu:27-46,227-232``) is restated in ``dropout_keep`` and applied when
``dropout_p > 0``.  That part is parity unpinned: the reference holds no test or vector for it, and its kernel
cannot run where this oracle is built.
"""
import numpy as np
import torch


def _magnitudes(dists, pair_mask, mag_type):
    # tests/wf_embed/wf_embed.py:108-116
    if mag_type == 0:
        return torch.where(pair_mask, torch.zeros_like(dists), torch.ones_like(dists))
    if mag_type == 1:
        return 1 / torch.where(pair_mask, float("inf"), dists)
    if mag_type == 2:
        # the dense reference leaves padded pairs unmasked here (wf_embed.py:114); the
        # reference kernel masks them (wf_embedding_kernel.cu:201,220-221) and that is
        # what is restated.  On unpadded input the two agree (1/log2(0) = -0).
        return torch.where(pair_mask, torch.zeros_like(dists), 1 / torch.log2(dists))
    if mag_type == 3:
        return 1 / torch.where(pair_mask, float("inf"), torch.sqrt(dists))
    raise ValueError(f"magnitude_type must be 0..3, not {mag_type}")


def dropout_hash(z, i, j, k, seed):
    """``hash5`` of the reference kernel (``wf_embedding_kernel.cu:27-40``) for index arrays ``z, i, j, k``
    (broadcastable): the seed xor-ed with one multiply-add term per index, then a multiply/xor-shift finaliser,
    all in wrapping 32-bit arithmetic."""
    u = lambda a: np.asarray(a).astype(np.uint32)
    c = np.uint32
    with np.errstate(over="ignore"):
        h = c(seed) ^ (u(z) * c(0x85ebca6b) + c(0x9e3779b9))
        h = h ^ (u(i) * c(0xc2b2ae35) + c(0x165667b1))
        h = h ^ (u(j) * c(0x27d4eb2f) + c(0xd6e8feb8))
        h = h ^ (u(k) * c(0x85ebca6b) + c(0x1b873593))
        h = (h ^ (h >> c(16))) * c(0x85ebca6b)
        h = h ^ (h >> c(13))
        h = (h ^ (h >> c(16))) * c(0xc2b2ae35)
        h = h ^ (h >> c(16))
    return h


def dropout_keep(z, i, j, k, seed, dropout_p):
    """Keep mask of the reference kernel's dropout (``wf_embedding_kernel.cu:42-46``): the hash is mapped to [0, 1]
    with a float division by ``float(UINT32_MAX)`` (which is 2^32 in fp32) and values >= p are kept."""
    normalized = dropout_hash(z, i, j, k, seed).astype(np.float32) / np.float32(4294967295.0)
    return normalized >= np.float32(dropout_p)


def wf_embedding_ref(coords, wavenumbers, mag_type=1, mask=None, rows=None, chunk=128,
                     dtype=None, return_sums=False, dropout_p=0.0, seed=0):
    """Features ``[Z, R, 2K]`` for observer rows ``rows = (begin, end)`` (default: all).

    coords ``[Z, N, 3]``, wavenumbers ``[K]``, mask ``[Z, N]`` bool with True = padded.
    ``dtype`` (default: that of ``coords``) selects fp32 (the reference's arithmetic) or
    fp64 (a tight truth for error budgets).  With ``return_sums`` also returns the two
    per-row sums the reference kernel stores for its backward,
    ``sum_j mag*r*cos(k r)`` and ``sum_j mag*r*sin(k r)``
    (``isotropic/cuda/wf_embedding_kernel.cu:237-238``), each ``[Z, R, K]``.
    With ``dropout_p > 0`` single evaluations are dropped and the kept ones scaled by ``1/(1-p)``, in the
    features and in the stored sums, as the reference kernel does (``:227-238``).
    """
    dtype = dtype or coords.dtype
    coords = coords.to(dtype)
    wavenumbers = wavenumbers.to(dtype)
    z, n, _ = coords.shape
    k = wavenumbers.shape[0]
    mask = mask if mask is not None else torch.zeros(z, n, dtype=torch.bool)
    r0, r1 = rows if rows is not None else (0, n)
    out = torch.empty(z, r1 - r0, 2 * k, dtype=dtype)
    cs = torch.empty(z, r1 - r0, k, dtype=dtype) if return_sums else None
    sn = torch.empty(z, r1 - r0, k, dtype=dtype) if return_sums else None
    for i0 in range(r0, r1, chunk):
        i1 = min(i0 + chunk, r1)
        # [Z, N(source), C(observer)]                          wf_embed.py:100
        dists = torch.sqrt(torch.sum((coords[:, :, None, :] - coords[:, None, i0:i1, :]) ** 2, dim=3))
        phases = dists[:, :, :, None] * wavenumbers[None, None, None, :]  # :103
        pair_mask = mask[:, :, None] | mask[:, None, i0:i1] | (dists == 0)  # :106
        mags = _magnitudes(dists, pair_mask, mag_type)[:, :, :, None]
        cosp, sinp = torch.cos(phases), torch.sin(phases)
        if dropout_p != 0.0:
            keep = dropout_keep(np.arange(z)[:, None, None, None], np.arange(i0, i1)[None, None, :, None],
                                np.arange(n)[None, :, None, None], np.arange(k)[None, None, None, :], seed, dropout_p)
            keep = torch.from_numpy(keep).to(dtype) / (1 - dropout_p)
            cosp, sinp = cosp * keep, sinp * keep
        real = mags * cosp  # :119
        imag = mags * sinp  # :120
        feats = torch.stack([real.sum(dim=1), imag.sum(dim=1)], dim=-1)  # :123-127
        out[:, i0 - r0:i1 - r0] = feats.view(z, i1 - i0, 2 * k)
        if return_sums:
            valid = (~pair_mask)[:, :, :, None].to(dtype)
            if mag_type == 1:
                w = valid  # mag * r == 1 on valid pairs
            else:
                w = torch.where(pair_mask[:, :, :, None], torch.zeros_like(mags), mags * dists[:, :, :, None])
            cs[:, i0 - r0:i1 - r0] = (w * cosp).sum(dim=1)
            sn[:, i0 - r0:i1 - r0] = (w * sinp).sum(dim=1)
    if return_sums:
        return out, cs, sn
    return out


def dk_analytic(d_out, cos_sums, sin_sums):
    """Wavenumber gradient from the stored sums,
    ``isotropic/cuda/wf_embedding.py:72-81``: ``sum_{z,n} dO_im * cos_sums - dO_re * sin_sums``."""
    return ((d_out[:, :, 1::2] * cos_sums) - (d_out[:, :, 0::2] * sin_sums)).sum(dim=(0, 1))


def dk_autograd(coords, wavenumbers, d_out, mag_type=1, mask=None, dtype=torch.float64, chunk=64, dropout_p=0.0, seed=0):
    """Wavenumber gradient by autograd through the dense formulation (the reference test's
    own check, ``tests/wf_embed/wf_embed.py:60-74``), accumulated over observer chunks."""
    wn = wavenumbers.detach().to(dtype).clone().requires_grad_(True)
    n = coords.shape[1]
    for i0 in range(0, n, chunk):
        i1 = min(i0 + chunk, n)
        out = wf_embedding_ref(coords, wn, mag_type, mask, rows=(i0, i1), chunk=chunk, dtype=dtype,
                               dropout_p=dropout_p, seed=seed)
        (out * d_out[:, i0:i1].to(dtype)).sum().backward()
    return wn.grad


def rel_l2(truth, test):
    """The reference's error metric, ``utils/test_utils.py:10-11``: ``|A-B|_2 / |A|_2``."""
    truth = truth.double()
    return float(torch.norm(truth - test.double()) / torch.norm(truth))
