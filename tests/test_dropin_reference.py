"""The drop-in against the reference's own, unedited source tree.

These tests need a checkout of jaimec00/proteusAI; its path comes from the environment variable
``PROTEUS_REFERENCE_ROOT`` (they are skipped when it is unset, e.g. on a machine that only has this repository).
They run in a child interpreter so that the aliased modules do not leak into the other tests."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("PROTEUS_REFERENCE_ROOT")
needs_reference = pytest.mark.skipif(not REF or not os.path.isfile(os.path.join(REF or "", "proteusAI.py")),
                                     reason="PROTEUS_REFERENCE_ROOT does not name a proteusAI checkout")


def _run(code):
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, REF]))
    res = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], capture_output=True, text=True, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout + res.stderr
    return res.stdout


@needs_reference
def test_reference_model_imports_and_builds_on_the_b200_leaves():
    out = _run("""
        import sys
        import proteusai_b200
        installed = proteusai_b200.install_dropin()
        assert len(installed) == 5, installed
        import proteusAI                                   # the reference's model file, unedited
        import utils.model_utils.wf_embedding.wf_embedding as ref_we
        import proteusai_b200.utils.model_utils.wf_embedding.isotropic.cuda.wf_embedding as ours_iso
        import proteusai_b200.utils.model_utils.wf_embedding.anisotropic.cb_scaling.learnable_wavenumbers.cuda.wf_embedding as ours_cb
        assert ref_we.__file__.startswith(sys.argv[1] if len(sys.argv) > 1 else ""), ref_we.__file__
        assert ref_we.wf_embedding_iso is ours_iso.wf_embedding          # wf_embedding/wf_embedding.py:15
        assert ref_we.wf_embedding_learnCB is ours_cb.wf_embedding       # :18, what the model calls
        model = proteusAI.proteusAI()
        fe = model.featurizer.wf_embedding
        assert type(fe).__module__ == "utils.model_utils.wf_embedding.wf_embedding"
        assert fe.forward.__globals__["wf_embedding_learnCB"] is ours_cb.wf_embedding
        try:
            ref_we.wf_embedding_staticAA()
        except RuntimeError as exc:
            assert "not built" in str(exc)
        else:
            raise AssertionError("placeholder did not raise")
        from utils.model_utils.attn.geometric_attn import geometric_attn
        import proteusai_b200.utils.model_utils.attn.geometric_attn as ours_ga
        assert geometric_attn is ours_ga.geometric_attn
        print("ok", sum(p.numel() for p in model.parameters()))
    """)
    assert out.startswith("ok")


@needs_reference
def test_virtual_cbeta_matches_the_reference_function():
    _run("""
        import torch
        from utils.model_utils.base_modules.Cb_utils import get_coords
        from proteusai_b200.utils.model_utils.wf_embedding.wf_embedding import WaveFunctionEmbedding
        g = torch.Generator().manual_seed(0)
        bb = torch.randn(2, 50, 3, 3, generator=g) * 3
        bb[1, 40:] = 0                                     # padding
        m = WaveFunctionEmbedding(d_wf=32)
        for norm in (False, True):
            ca, cb = m.get_CaCb_coords(bb, None, norm)
            ca_r, cb_r = get_coords(bb, None, norm)
            assert torch.equal(ca, ca_r) and torch.equal(cb, cb_r), norm
    """)


@needs_reference
@pytest.mark.gpu
def test_reference_featurizer_forward_runs_on_the_b200_kernels():
    """FeaturizeProtein.forward of the reference (gnn.py:41-63): virtual C-beta, the anisotropic WE on the B200 kernel,
    the reference's own neighbour search and edge features; node features against the CPU oracle of the same WE."""
    _run("""
        import torch
        import proteusai_b200
        proteusai_b200.install_dropin()
        import proteusAI
        from oracle.we_aniso_ref import wf_embedding_aniso_ref
        from oracle import chains
        torch.manual_seed(0)
        model = proteusAI.proteusAI().cuda().eval()
        z, n = 2, 96
        ca, mask = chains.chain_batch([96, 60], n, seed=4)
        ca, mask = torch.from_numpy(ca), torch.from_numpy(mask)
        g = torch.Generator().manual_seed(1)
        bb = ca[:, :, None, :] + torch.randn(z, n, 3, 3, generator=g) * torch.tensor([1.0, 0.0, 1.0])[None, None, :, None]
        bb[mask] = 0
        labels = torch.randint(0, 20, (z, n), generator=g)
        with torch.no_grad():
            V, E, K, S, edge_mask, ar = model.featurizer(bb.cuda(), labels.cuda(), None, node_mask=mask.cuda())
            fe = model.featurizer
            ca_d, cb_d = fe.wf_embedding.get_CaCb_coords(bb.cuda(), None, norm=False)
            wf = fe.wf_embedding(ca_d, cb_d, key_padding_mask=mask.cuda())
        ref = wf_embedding_aniso_ref(ca_d.cpu(), cb_d.cpu(), fe.wf_embedding.aa_magnitudes.detach().cpu(),
                                     fe.wf_embedding.get_wavenumbers().detach().cpu(), mask)
        ref = ref[0] if isinstance(ref, tuple) else ref
        err = (torch.linalg.vector_norm(ref - wf.cpu()) / torch.linalg.vector_norm(ref)).item()
        assert err < 1e-4, err
        assert V.shape == (z, n, 128) and E.shape[:3] == (z, n, 30) and torch.isfinite(V).all()
        print("ok", err)
    """)
