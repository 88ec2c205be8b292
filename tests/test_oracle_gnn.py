"""The neighbour / edge-feature oracle against the reference's own methods (golden vectors) and against itself."""
import os

import numpy as np
import torch

from oracle import chains
from oracle.gnn_ref import edge_rbf_ref, get_neighbors_ref


def _cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "gnn_reference.npz"))
    for name in sorted({k.split(".")[0] for k in g.files}):
        yield name, {k.split(".", 1)[1]: torch.from_numpy(np.asarray(g[k])) for k in g.files if k.startswith(name + ".")}


def test_golden_bit_exact(golden_dir):
    torch.set_num_threads(1)
    n = 0
    for name, t in _cases(golden_dir):
        atoms, mask, k = t["atoms"], t["mask"], int(t["k"])
        idx, edge_mask = get_neighbors_ref(atoms[:, :, 1], mask, k)
        assert torch.equal(idx, t["idx"]) and torch.equal(edge_mask, t["edge_mask"]), name
        if "feats" in t:
            feats = edge_rbf_ref(atoms, idx, t["centers"], float(t["spread"]))
            assert torch.equal(feats, t["feats"]), name
        n += 1
    assert n == 3


def test_neighbour_semantics():
    c, m = chains.chain_batch([60, 25], 60, seed=9)
    c[~m] += np.array([7.25, -4.5, 2.75], dtype=np.float32)  # off the origin, where the padding sits
    ca, mask = torch.from_numpy(c), torch.from_numpy(m)
    idx, em = get_neighbors_ref(ca, mask, 12)
    node = torch.arange(60).view(1, -1, 1)
    assert torch.all(idx[1, 25:] == node[0, 25:]) and not em[1, 25:].any()      # masked nodes: themselves, no edges
    assert torch.all(idx[~em] == node.expand_as(idx)[~em])                        # dropped edges point home
    d = torch.linalg.vector_norm(ca[:, :, None] - torch.gather(ca[:, None].expand(-1, 60, -1, -1), 2,
                                                              idx[..., None].expand(-1, -1, -1, 3)), dim=3)
    assert torch.all(d[em] < 12) and torch.all(d[em] > 0)
    both = em[0, :, 1:] & em[0, :, :-1]
    assert torch.all(d[0, :, 1:][both] >= d[0, :, :-1][both] - 1e-5)              # ascending (3.8 A bonds tie up to rounding)
    assert not mask[1][idx[1][em[1]]].any()                                        # no kept edge reaches a masked node
