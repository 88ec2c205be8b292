"""``WaveFunctionEmbedding`` module, isotropic branch.

Mirrors ``utils/model_utils/wf_embedding/wf_embedding.py:24-49`` of the reference: same
constructor arguments, same parameter names (``wavenumbers`` holds log-wavenumbers,
``aa_magnitudes``), same wavelength schedule (``logspace(0, 1, K, base)``, i.e. exponents
``i / (K - 1)``), same ``forward(coords_alpha, coords_beta, key_padding_mask)`` signature, so a
reference checkpoint loads.  Both branches of the reference are provided: the isotropic kernel and the
anisotropic one with per-wavenumber C-beta scaling (``wf_embedding_learnCB``, the reference's default).
``get_CaCb_coords`` (``:48-49``, the first call of ``FeaturizeProtein.forward``, ``utils/model_utils/gnn/gnn.py:44``)
builds the C-alpha positions and virtual C-beta directions the anisotropic branch takes.
"""
import torch
import torch.nn as nn

from proteusai_b200.utils.model_utils.wf_embedding.anisotropic.cb_scaling.learnable_wavenumbers.cuda.wf_embedding import (
    wf_embedding as wf_embedding_learnCB)
from proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding import wf_embedding as wf_embedding_iso


class WaveFunctionEmbedding(nn.Module):

    def __init__(self, d_wf=512, min_wl=4.0, max_wl=35.0, base_wl=20.0, anisotropic=True, learn_wl=False, learn_aa=False):
        super(WaveFunctionEmbedding, self).__init__()
        wl = min_wl + (max_wl - min_wl) * ((torch.logspace(0, 1, d_wf // 2, base_wl) - 1) / (base_wl - 1))
        wn = torch.log(torch.pi * 2 / wl)
        self.wavenumbers = nn.Parameter(wn, requires_grad=learn_wl)  # log of the wavenumbers
        self.aa_magnitudes = nn.Parameter(torch.ones(d_wf // 2), requires_grad=learn_aa)
        self.aniso = anisotropic

    def get_wavenumbers(self):
        return torch.exp(self.wavenumbers)

    def forward(self, coords_alpha, coords_beta=None, key_padding_mask=None):
        if self.aniso:
            return wf_embedding_learnCB(coords_alpha, coords_beta, self.aa_magnitudes, self.get_wavenumbers(), mask=key_padding_mask)
        return wf_embedding_iso(coords_alpha, self.get_wavenumbers(), magnitude_type=1, dropout_p=0.0, mask=key_padding_mask)

    def get_CaCb_coords(self, coords, chain_idxs=None, norm=False):
        """``(C-alpha [Z,N,3], virtual C-beta relative to C-alpha [Z,N,3])``.

        Backbone input ``[Z,N,3(N,CA,C),3]`` (what the model passes): the ideal-geometry construction from the two bond
        vectors and their cross product with ProteinMPNN's coefficients, as ``get_Cb_from_BB``
        (``utils/model_utils/base_modules/Cb_utils.py:97-116``); padded residues (all zeros) give a zero C-beta;
        ``norm=True`` scales to unit vectors.  C-alpha-only input ``[Z,N,3]`` with ``chain_idxs`` is passed on to the
        reference's own ``get_coords`` when the reference tree is importable (it is not restated here)."""
        if coords.dim() == 4:
            n, ca, c = coords[:, :, 0, :], coords[:, :, 1, :], coords[:, :, 2, :]
            b1, b2 = ca - n, c - ca
            b3 = torch.linalg.cross(b1, b2, dim=2)
            cb = -0.58273431 * b2 + 0.56802827 * b1 - 0.54067466 * b3
            if norm:
                cb = cb * (1 / torch.linalg.vector_norm(cb, dim=2, keepdim=True).clamp(1e-6))
            return ca, cb
        if coords.dim() == 3:
            try:
                from utils.model_utils.base_modules.Cb_utils import get_coords
            except ImportError as exc:
                raise NotImplementedError(
                    "C-alpha-only input needs the reference's utils.model_utils.base_modules.Cb_utils on sys.path; "
                    "backbone input [Z,N,3,3] is handled here") from exc
            return get_coords(coords, chain_idxs, norm)
        raise ValueError(f"invalid input size for coordinates, expected (batch,N,3) for Ca only model or (batch,N,3,3) "
                         f"for backbone model, but got {coords.shape=}")
