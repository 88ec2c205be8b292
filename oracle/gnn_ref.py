"""CPU oracle for the neighbour graph and the radial-basis edge features (test infrastructure).

Restates two methods of the reference's ``FeaturizeProtein`` (``utils/model_utils/gnn/gnn.py``):
``get_neighbors`` (``:97-117``) and the tensor part of ``get_edges`` (``:119-131``, up to the ``view`` that flattens
the features; the LayerNorm and the projection that follow are PyTorch modules).

Pinned against the reference methods themselves: ``tests/golden/make_golden.py`` cuts them out of the reference
file, runs them on seeded inputs and stores the outputs (``gnn_reference.npz``); ``tests/test_oracle_gnn.py`` checks
this restatement against them bit for bit.
"""
import torch


def get_neighbors_ref(ca, node_mask, k, max_dist=12.0):
    """ca ``[Z,N,3]``, node_mask ``[Z,N]`` bool (True = masked).  Returns ``(idx [Z,N,K] int64, edge_mask [Z,N,K] bool)``.

    The reference writes ``torch.where(dists==0 | node_mask.unsqueeze(2), inf, dists)`` (``gnn.py:104``).  Python binds
    ``|`` tighter than ``==``, so this compares the distances with the mask *as a number*: rows of unmasked nodes lose
    their zero distances (the node itself, coincident points), rows of masked nodes lose distances equal to 1.  Masked
    nodes are therefore NOT removed from the candidates; their edges are dropped afterwards by the edge mask."""
    z, n, _ = ca.shape
    dists = torch.sqrt(torch.sum((ca.unsqueeze(1) - ca.unsqueeze(2)) ** 2, dim=3))  # :103
    excluded = dists == node_mask.unsqueeze(2).to(dists.dtype)                        # :104, as evaluated
    dists = torch.where(excluded, float("inf"), dists)
    topk = dists.topk(k, dim=2, largest=False)                                        # :107
    node_idxs = torch.arange(n).view(1, -1, 1)
    edge_mask = ~(node_mask.unsqueeze(2) | torch.gather(node_mask.unsqueeze(2).expand(-1, -1, k), 1, topk.indices))  # :111
    edge_mask = edge_mask & (topk.values != 0) & (topk.values < max_dist)             # :112
    return torch.where(edge_mask, topk.indices, node_idxs), edge_mask                 # :113


def edge_rbf_ref(atoms, idx, centers, spread):
    """atoms ``[Z,N,A,3]``, idx ``[Z,N,K]`` → ``[Z,N,K,A*A*R]`` (``gnn.py:119-131``)."""
    z, n, a, s = atoms.shape
    k = idx.shape[2]
    ck = torch.gather(atoms.unsqueeze(2).expand(-1, -1, k, -1, -1), 1,
                      idx.unsqueeze(3).unsqueeze(4).expand(-1, -1, -1, a, s))          # :125
    dists = torch.sqrt(torch.sum((atoms.unsqueeze(2).unsqueeze(4) - ck.unsqueeze(3)) ** 2, dim=5))  # :128
    rbfs = torch.exp(-((dists.unsqueeze(5) - centers.view(1, 1, 1, 1, 1, -1)) ** 2) / (spread ** 2))  # :131
    return rbfs.view(z, n, k, -1)
