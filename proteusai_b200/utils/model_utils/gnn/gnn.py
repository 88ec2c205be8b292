"""Neighbour graph and radial-basis edge features of the reference's ``FeaturizeProtein``
(``utils/model_utils/gnn/gnn.py:23-137``) over the B200 kernels.

``EdgeFeaturizer`` carries the graph part of that module under the same method and attribute names —
``get_neighbors(Ca, node_mask)`` (``:97-117``) and ``get_edges(C, K)`` (``:119-137``) with ``edge_norm``, ``edge_proj``,
``rbf_centers`` and ``spread`` — so its state dict keys match the reference's.  The reference builds an ``N x N``
distance matrix, calls ``torch.topk`` and broadcasts a ``[Z,N,K,4,4,R]`` tensor; here one kernel streams the
coordinates and keeps the K nearest per node, a second writes the feature rows.  Node features, sequence features
and the autoregressive mask of ``FeaturizeProtein.forward`` are not part of this class.
"""
import torch
import torch.nn as nn

from proteusai_b200 import _lib


def knn_neighbors(Ca, node_mask, k, max_dist=12.0):
    """``(idx [Z,N,K] int64, edge_mask [Z,N,K] bool)`` for C-alpha coordinates ``[Z,N,3]`` and ``node_mask [Z,N]``
    (True = masked, or None).  Neighbours come in ascending order of distance; dropped edges point back at the node."""
    if not Ca.is_cuda:
        raise RuntimeError("knn_neighbors needs CUDA tensors: there is no CPU path")
    z, n, s = Ca.shape
    assert s == 3 and n >= k
    ca = Ca.detach().to(torch.float32).contiguous()
    valid = None if node_mask is None else (~node_mask.bool()).contiguous().view(torch.uint8)
    idx = torch.empty(z, n, k, dtype=torch.int64, device=Ca.device)
    edge_mask = torch.empty(z, n, k, dtype=torch.bool, device=Ca.device)
    with torch.cuda.device(Ca.device):
        _lib.check(_lib.lib().pai_knn_neighbors(_lib.ptr(ca), _lib.ptr(valid), _lib.ptr(idx), _lib.ptr(edge_mask), z, n, k,
                                                float(max_dist), _lib.current_stream()), "pai_knn_neighbors")
    return idx, edge_mask


def edge_rbf(C, K, rbf_centers, spread, norm=None):
    """``[Z,N,K,A*A*R]`` radial-basis features of the distances between the ``A`` atoms of every node ``C [Z,N,A,3]``
    and the atoms of its neighbours ``K [Z,N,K]``.  ``norm`` (an ``nn.LayerNorm`` over the features, fp32, A = 4 and
    R = 16) is applied inside the kernel, before the features are written."""
    if not C.is_cuda:
        raise RuntimeError("edge_rbf needs CUDA tensors: there is no CPU path")
    z, n, a, s = C.shape
    assert s == 3 and K.shape[:2] == (z, n)
    k = K.shape[2]
    atoms = C.detach().to(torch.float32).contiguous()
    idx = K.to(torch.int64).contiguous()
    centers = rbf_centers.detach().to(torch.float32).contiguous()
    r = centers.numel()
    out = torch.empty(z, n, k, a * a * r, dtype=torch.float32, device=C.device)
    gamma = beta = None
    eps = 0.0
    if norm is not None:
        gamma = norm.weight.detach().to(torch.float32).contiguous()
        beta = norm.bias.detach().to(torch.float32).contiguous()
        eps = norm.eps
    with torch.cuda.device(C.device):
        _lib.check(_lib.lib().pai_edge_rbf(_lib.ptr(atoms), _lib.ptr(idx), _lib.ptr(centers), float(spread), _lib.ptr(gamma),
                                           _lib.ptr(beta), float(eps), _lib.ptr(out), z, n, k, a, r, _lib.current_stream()),
                   "pai_edge_rbf")
    return out


class EdgeFeaturizer(nn.Module):

    def __init__(self, K=30, De=128, min_rbf=2.0, max_rbf=22.0, num_rbfs=16):
        super().__init__()
        self.K = K
        self.edge_norm = nn.LayerNorm(int(num_rbfs * 4 * 4))
        self.edge_proj = nn.Linear(int(num_rbfs * 4 * 4), De)
        self.register_buffer("rbf_centers", torch.linspace(min_rbf, max_rbf, int(num_rbfs)))
        self.spread = (max_rbf - min_rbf) / num_rbfs

    def get_neighbors(self, Ca, node_mask=None):
        dimZ, dimN, dimS = Ca.shape
        assert dimN >= self.K
        return knn_neighbors(Ca, node_mask, self.K)

    def get_edges(self, C, K):
        # without gradients to record, the LayerNorm runs inside the feature kernel (4 x 4 x 16 features, fp32 parameters)
        fused = (not (torch.is_grad_enabled() and any(p.requires_grad for p in self.edge_norm.parameters()))
                 and C.shape[2] == 4 and self.rbf_centers.numel() == 16 and self.edge_norm.weight.dtype == torch.float32)
        if fused:
            return self.edge_proj(edge_rbf(C, K, self.rbf_centers, self.spread, norm=self.edge_norm))
        E = edge_rbf(C, K, self.rbf_centers, self.spread)  # Z x N x K x (4*4*num_rbfs)
        return self.edge_proj(self.edge_norm(E))           # Z x N x K x De

    def forward(self, C, node_mask=None):
        """C ``[Z,N,4,3]`` (N, C-alpha, C, C-beta).  Returns ``(E [Z,N,K,De], K [Z,N,K], edge_mask [Z,N,K])``."""
        K, edge_mask = self.get_neighbors(C[:, :, 1, :], node_mask)
        return self.get_edges(C, K), K, edge_mask
