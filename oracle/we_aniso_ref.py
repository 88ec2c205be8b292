"""CPU oracle for the anisotropic Wavefunction Embedding with per-wavenumber C-beta scaling
(test infrastructure).

Restates the reference's dense PyTorch formulation ``wf_embedding_torch`` in
``tests/wf_embed/wf_embed_aniso_learnCB_learnK.py:116-166``, observer-chunked: for observer i, source j,
``R = A_i - A_j``, ``r = |R|``, the phase of wavenumber k is ``k * (r - s_k * (R/r . B_j))`` with ``B_j`` the
(unit) C-beta direction of the source and ``s_k`` its learnable per-wavenumber magnitude; features are
``sum_j cos(phase)/r`` and ``sum_j sin(phase)/r`` interleaved; pairs with r == 0 or a padded token are excluded.

Pinned against the reference function by ``tests/golden/we_aniso_reference.npz`` (outputs and the autograd
gradients w.r.t. ``cb_magnitudes`` and ``wavenumbers``).  ``partials`` returns what the reference kernel stores for
its O(N) backward (``anisotropic/cb_scaling/learnable_wavenumbers/cuda/wf_embedding.py:42-79``): the derivatives of
every output element w.r.t. ``s_k`` and ``k``.
"""
import torch


def wf_embedding_aniso_ref(coords_a, coords_b, cb_magnitudes, wavenumbers, mask=None, rows=None, chunk=64, dtype=None,
                           partials=False):
    """Features ``[Z, R, 2K]`` for observer rows ``rows`` (default all).  With ``partials`` also returns
    ``d_cb`` and ``d_k``, each ``[Z, R, 2K]``."""
    dtype = dtype or coords_a.dtype
    A, B = coords_a.to(dtype), coords_b.to(dtype)
    s, kk = cb_magnitudes.to(dtype), wavenumbers.to(dtype)
    z, n, _ = A.shape
    nk = kk.shape[0]
    mask = mask if mask is not None else torch.zeros(z, n, dtype=torch.bool)
    r0, r1 = rows if rows is not None else (0, n)
    out = torch.empty(z, r1 - r0, 2 * nk, dtype=dtype)
    dcb = torch.empty_like(out) if partials else None
    dk = torch.empty_like(out) if partials else None
    for i0 in range(r0, r1, chunk):
        i1 = min(i0 + chunk, r1)
        R = A[:, i0:i1, None, :] - A[:, None, :, :]  # [Z, C(observer), N(source), 3]      :125
        R_norm = torch.linalg.vector_norm(R, dim=3, keepdim=True)  # :128
        R_unit = R / torch.where(R_norm == 0, float("inf"), R_norm)  # :129
        cb = B[:, :, None, :] * s[None, None, :, None]  # [Z, N, K, 3]                      :139
        dists_b = torch.sum(R_unit[:, :, :, None, :] * cb[:, None, :, :, :], dim=4)  # [Z, C, N, K]   :141
        dists_ab = R_norm - dists_b  # :143
        phases = dists_ab * kk[None, None, None, :]  # :146
        pm = mask[:, i0:i1, None, None] | mask[:, None, :, None] | (R_norm == 0)  # :149
        mags = 1 / torch.where(pm, float("inf"), R_norm)  # :152
        cosp, sinp = torch.cos(phases), torch.sin(phases)
        real, imag = mags * cosp, mags * sinp  # :155-156
        out[:, i0 - r0:i1 - r0] = torch.stack([real.sum(dim=2), imag.sum(dim=2)], dim=-1).view(z, i1 - i0, 2 * nk)  # :159-163
        if partials:
            b_unit = torch.sum(R_unit[:, :, :, None, :] * B[:, None, :, None, :], dim=4)  # R/r . B_j, [Z,C,N,1]
            kb = kk[None, None, None, :] * b_unit  # d phase / d s_k = -k b
            d_re_s, d_im_s = mags * sinp * kb, -mags * cosp * kb
            d_re_k, d_im_k = -mags * sinp * dists_ab, mags * cosp * dists_ab
            dcb[:, i0 - r0:i1 - r0] = torch.stack([d_re_s.sum(dim=2), d_im_s.sum(dim=2)], dim=-1).view(z, i1 - i0, 2 * nk)
            dk[:, i0 - r0:i1 - r0] = torch.stack([d_re_k.sum(dim=2), d_im_k.sum(dim=2)], dim=-1).view(z, i1 - i0, 2 * nk)
    if partials:
        return out, dcb, dk
    return out


def grads_from_partials(d_out, d_cb, d_k):
    """The reference's backward (``.../learnable_wavenumbers/cuda/wf_embedding.py:66-79``): multiply the stored partials
    with dO, sum over batch and rows, add the real and imaginary halves.  Returns ``(d_cb_magnitudes [K], d_wavenumbers [K])``."""
    a = (d_out * d_cb).sum(dim=(0, 1))
    b = (d_out * d_k).sum(dim=(0, 1))
    return a[::2] + a[1::2], b[::2] + b[1::2]
