"""proteusai_b200: B200 (sm_100a) kernels for proteusAI's Wavefunction Embedding and Geometric
Attention behind the reference's own Python call signatures.

``install_dropin()`` registers the modules of this package under the import paths of the reference's
kernel-backed LEAF modules, so that the reference's own, unedited code (``proteusAI.py``, ``learn_seqs.py``,
``utils/model_utils/gnn/gnn.py``, ``utils/model_utils/wf_embedding/wf_embedding.py``) imports and runs with the B200
kernels underneath:

* ``utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding``                                   isotropic WE
* ``utils.model_utils.wf_embedding.anisotropic.cb_scaling.learnable_wavenumbers.cuda.wf_embedding`` the variant the model
  calls by default
* ``utils.model_utils.attn.geometric_attn``                                                         geometric attention
* the two per-amino-acid variants that ``wf_embedding/wf_embedding.py:16-17`` imports but the model never calls
  (``anisotropic.aa_scaling.learnable_aa.learnable_wavenumber`` and ``anisotropic.aa_scaling.static_aa``) resolve to
  placeholder modules whose ``wf_embedding`` raises: they exist so that the import succeeds without the reference's
  unbuilt CUDA extensions.
"""
import importlib
import sys
import types

__version__ = "0.2.0"

_DROPIN = {
    "utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding":
        "proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding",
    "utils.model_utils.wf_embedding.anisotropic.cb_scaling.learnable_wavenumbers.cuda.wf_embedding":
        "proteusai_b200.utils.model_utils.wf_embedding.anisotropic.cb_scaling.learnable_wavenumbers.cuda.wf_embedding",
    "utils.model_utils.attn.geometric_attn":
        "proteusai_b200.utils.model_utils.attn.geometric_attn",
}

# imported by the reference's WaveFunctionEmbedding module, never called by the model: placeholders
_NOT_BUILT = (
    "utils.model_utils.wf_embedding.anisotropic.aa_scaling.learnable_aa.learnable_wavenumber.cuda.wf_embedding",
    "utils.model_utils.wf_embedding.anisotropic.aa_scaling.static_aa.cuda.wf_embedding",
)


def _placeholder(ref_name):
    mod = types.ModuleType(ref_name, "placeholder installed by proteusai_b200.install_dropin(): variant not built for B200")

    def wf_embedding(*args, **kwargs):
        raise RuntimeError(
            f"{ref_name}.wf_embedding: this per-amino-acid anisotropic variant is not built for B200; the variants that are "
            "built are the isotropic one and cb_scaling/learnable_wavenumbers (what WaveFunctionEmbedding calls)")

    mod.wf_embedding = wf_embedding
    mod.__proteus_b200_placeholder__ = True
    return mod


def install_dropin(force=False):
    """Alias this package's modules to the reference's import paths (only the leaf modules listed in the module
    docstring; the reference's own packages and modules above them are left alone and keep working).  Call it before
    the reference's modules are imported.  Returns the names it installed."""
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
    for ref_name in _NOT_BUILT:
        if ref_name in sys.modules and not force:
            continue
        sys.modules[ref_name] = _placeholder(ref_name)
        done.append(ref_name)
    return done
