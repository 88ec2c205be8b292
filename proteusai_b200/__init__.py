"""proteusai_b200: B200 (sm_100a) kernels for proteusAI's Wavefunction Embedding and Geometric
Attention behind the reference's own Python call signatures.

``install_dropin()`` registers the modules of this package under the import paths the reference
uses (``utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding``, the anisotropic
``...anisotropic.cb_scaling.learnable_wavenumbers.cuda.wf_embedding`` and ``utils.model_utils.attn.geometric_attn``), so reference code importing those names gets the B200
implementation without being edited.
"""
import importlib
import sys

__version__ = "0.1.0"

_DROPIN = {
    "utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding":
        "proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding",
    "utils.model_utils.wf_embedding.anisotropic.cb_scaling.learnable_wavenumbers.cuda.wf_embedding":
        "proteusai_b200.utils.model_utils.wf_embedding.anisotropic.cb_scaling.learnable_wavenumbers.cuda.wf_embedding",
    "utils.model_utils.attn.geometric_attn":
        "proteusai_b200.utils.model_utils.attn.geometric_attn",
}


def install_dropin(force=False):
    """Alias this package's modules to the reference's import paths (only those leaf modules;
    parent packages of the reference, if importable, are left alone)."""
    done = []
    for ref_name, ours in _DROPIN.items():
        if ref_name in sys.modules and not force:
            continue
        try:
            mod = importlib.import_module(ours)
        except ModuleNotFoundError:
            continue
        sys.modules[ref_name] = mod
        done.append(ref_name)
    return done
