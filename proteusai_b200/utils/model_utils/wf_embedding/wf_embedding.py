"""``WaveFunctionEmbedding`` module, isotropic branch.

Mirrors ``utils/model_utils/wf_embedding/wf_embedding.py:24-49`` of the reference: same
constructor arguments, same parameter names (``wavenumbers`` holds log-wavenumbers,
``aa_magnitudes``), same wavelength schedule (``logspace(0, 1, K, base)``, i.e. exponents
``i / (K - 1)``), same ``forward(coords_alpha, coords_beta, key_padding_mask)`` signature, so a
reference checkpoint loads.  Both branches of the reference are provided: the isotropic kernel and the
anisotropic one with per-wavenumber C-beta scaling (``wf_embedding_learnCB``, the reference's default).
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
