"""Generate the golden vectors under tests/golden/ from the reference's own functions.

Run once in a container where the reference tree is mounted:

    python tests/golden/make_golden.py /path/to/reference

The reference's test modules cannot be imported (they import a CUDA extension that is
not built and a module path that no longer exists), so the two pure-PyTorch functions
are cut out of their files by AST and executed as they stand:

* ``wf_embedding_torch``  from ``tests/wf_embed/wf_embed.py``
* ``torch_attn``          from ``tests/attn/geo_attn.py``
* ``wf_embedding_torch``  (anisotropic, C-beta scaling) from ``tests/wf_embed/wf_embed_aniso_learnCB_learnK.py``
* ``FeaturizeProtein.get_neighbors`` / ``get_edges`` from ``utils/model_utils/gnn/gnn.py`` (a second argument ``gnn``
  regenerates only their file)

Inputs are seeded; inputs and the reference's outputs (and gradients obtained by
autograd through the reference functions, as the reference's tests do) are stored in
``.npz`` files which the CPU tests compare the oracle against, and the GPU tests compare
the CUDA path against.
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import chains  # noqa: E402


def extract(path, name):
    src = open(path).read()
    tree = ast.parse(src)
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            ns = {"torch": torch, "math": __import__("math")}
            exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), ns)
            return ns[name]
    raise KeyError(name)


def extract_method(path, cls, name):
    """A method of a class in the reference file, as a plain function taking ``self`` first."""
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.ClassDef) and node.name == cls:
            for item in node.body:
                if isinstance(item, ast.FunctionDef) and item.name == name:
                    ns = {"torch": torch}
                    exec(compile(ast.Module(body=[item], type_ignores=[]), path, "exec"), ns)
                    return ns[name]
    raise KeyError(f"{cls}.{name}")


def backbone_atoms(ca, rng):
    """Four atoms per node (N, C-alpha, C, C-beta) at bonded distances around the C-alpha trace."""
    z, n, _ = ca.shape
    off = rng.normal(size=(z, n, 4, 3))
    off /= np.linalg.norm(off, axis=3, keepdims=True)
    off *= np.array([1.46, 0.0, 1.52, 1.53])[None, None, :, None]
    return (ca[:, :, None, :] + off).astype(np.float32)


def gnn_golden(ref_root):
    """Neighbour graph and edge features from the reference's own FeaturizeProtein methods (gnn.py:97-131)."""
    from types import SimpleNamespace
    path = os.path.join(ref_root, "utils/model_utils/gnn/gnn.py")
    get_neighbors = extract_method(path, "FeaturizeProtein", "get_neighbors")
    get_edges = extract_method(path, "FeaturizeProtein", "get_edges")
    min_rbf, max_rbf, num_rbfs = 2.0, 22.0, 16          # the reference's defaults (gnn.py:24)
    blob = {}
    rng = np.random.default_rng(20240606)
    for name, lengths, n, k in (("padded_k30", [48, 20], 48, 30), ("short_k8", [40, 9], 40, 8), ("k40", [90], 90, 40)):
        c, m = chains.chain_batch(lengths, n, seed=23)
        # Chains start at the origin, which is also where padding sits: move the real nodes away, otherwise the first node
        # of a chain ties exactly with every padded node and torch.topk's unspecified tie order decides the outputs.
        c[~m] += np.array([7.25, -4.5, 2.75], dtype=np.float32)
        if name == "short_k8":
            c[0, 5] = c[0, 4]  # a coincident pair
        atoms = backbone_atoms(c, rng)
        me = SimpleNamespace(K=k, rbf_centers=torch.linspace(min_rbf, max_rbf, num_rbfs), spread=(max_rbf - min_rbf) / num_rbfs,
                             edge_norm=lambda t: t, edge_proj=lambda t: t)  # the two modules after the features: identity here
        ca, mask = torch.from_numpy(atoms[:, :, 1].copy()), torch.from_numpy(m)
        idx, edge_mask = get_neighbors(me, ca, node_mask=mask)
        feats = get_edges(me, torch.from_numpy(atoms), idx)
        blob.update({f"{name}.atoms": atoms, f"{name}.mask": m, f"{name}.k": np.int64(k), f"{name}.idx": idx.numpy(),
                     f"{name}.edge_mask": edge_mask.numpy(), f"{name}.centers": me.rbf_centers.numpy(),
                     f"{name}.spread": np.float64(me.spread)})
        if name != "k40":  # (the feature tensor is large: kept for two cases)
            blob[f"{name}.feats"] = feats.numpy()
    np.savez_compressed(os.path.join(HERE, "gnn_reference.npz"), **blob)


def we_cases():
    g = torch.Generator().manual_seed(20240601)
    cases = {}
    # the reference test's own input style: coords = max_wl * randn, wavenumbers = randn
    z, n, k = 2, 96, 16
    coords = 20 * torch.randn((z, n, 3), generator=g)
    wn = torch.randn((k,), generator=g)
    mask = torch.zeros(z, n, dtype=torch.bool)
    mask[0, 70:] = True
    mask[1, 5] = True
    mask[1, 40:44] = True
    coords[1, 11] = coords[1, 10]  # coincident pair (d == 0 is excluded)
    for mt in (0, 1, 3):
        cases[f"randn_m{mt}"] = (coords, wn, mt, mask)
    cases["randn_m2_nomask"] = (coords, wn.abs() + 0.1, 2, torch.zeros(z, n, dtype=torch.bool))
    # chain-style inputs with the benchmark wavelength schedule
    c, m = chains.chain_batch([160, 97], 160, seed=7)
    cases["chain_m1"] = (torch.from_numpy(c), torch.from_numpy(chains.wavenumbers(64)), 1, torch.from_numpy(m))
    return cases


def attn_cases():
    g = torch.Generator().manual_seed(20240602)
    cases = {}
    z, h, n, d = 2, 3, 48, 16
    q, k, v = (torch.randn((z, h, n, d), generator=g) for _ in range(3))
    # the reference test's own input style: collinear coords, spreads 3, betas 1, no padding
    coords = 50 * torch.randn((z, n, 1), generator=g).expand(z, n, 3).contiguous()
    spreads = torch.full((h,), 3.0)
    betas = torch.full((h,), 1.0)
    nomask = torch.zeros(z, n, dtype=torch.bool)
    cases["collinear"] = (q, k, v, coords, spreads, betas, nomask, 0.0, 1.0)
    c, m = chains.chain_batch([48, 29], 48, seed=11)
    cases["chain_padded"] = (q, k, v, torch.from_numpy(c), torch.tensor([3.0, 8.0, 15.0]),
                             torch.tensor([0.5, 1.0, 2.0]), torch.from_numpy(m), 0.001, 0.99)
    return cases


def attn_d64_cases():
    """Head dimension 64 (what the CUDA kernel supports), inputs exactly representable in bf16 so that the kernel and
    the reference function see identical values.  One case in the reference test's own style (collinear coordinates,
    spreads 3, betas 1, no padding, window [0, 1]); one on a padded random-walk chain with the module's defaults
    (min_rbf 0.001, max_rbf 1.0)."""
    g = torch.Generator().manual_seed(20240603)
    bf = lambda t: t.to(torch.bfloat16).float()
    cases = {}
    z, h, n, d = 1, 2, 144, 64
    q, k, v = (bf(torch.randn((z, h, n, d), generator=g)) for _ in range(3))
    coords = 50 * torch.randn((z, n, 1), generator=g).expand(z, n, 3).contiguous()
    cases["d64_collinear"] = (q, k, v, coords, torch.full((h,), 3.0), torch.full((h,), 1.0),
                              torch.zeros(z, n, dtype=torch.bool), 0.0, 1.0)
    c, m = chains.chain_batch([120], n, seed=13)
    cases["d64_chain_padded"] = (q, k, v, torch.from_numpy(c), torch.tensor([4.0, 12.0]), torch.tensor([0.7, 1.5]),
                                 torch.from_numpy(m), 0.001, 1.0)
    return cases


def main(ref_root, only=None):
    torch.set_num_threads(1)
    if only == "gnn":
        gnn_golden(ref_root)
        print("wrote gnn_reference.npz")
        return
    wf_embedding_torch = extract(os.path.join(ref_root, "tests/wf_embed/wf_embed.py"), "wf_embedding_torch")
    torch_attn = extract(os.path.join(ref_root, "tests/attn/geo_attn.py"), "torch_attn")
    torch.set_num_threads(1)  # reductions stay in one fixed order

    blob = {}
    for name, (coords, wn, mt, mask) in we_cases().items():
        wn_g = wn.clone().requires_grad_(True)
        out = wf_embedding_torch(coords, wn_g, mt, 0.0, mask)
        out.sum().backward()  # the reference test's backward check, wf_embed.py:60-68
        blob.update({f"{name}.coords": coords.numpy(), f"{name}.wn": wn.numpy(), f"{name}.mag": np.int64(mt),
                     f"{name}.mask": mask.numpy(), f"{name}.out": out.detach().numpy(),
                     f"{name}.dk_sum": wn_g.grad.numpy()})
    np.savez_compressed(os.path.join(HERE, "we_reference.npz"), **blob)

    blob = {}
    for name, (q, k, v, coords, spreads, betas, mask, lo, hi) in attn_cases().items():
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v, spreads, betas)]
        out = torch_attn(leaves[0], leaves[1], leaves[2], coords, leaves[3], leaves[4], mask, lo, hi)
        valid_rows = (~mask)[:, None, :, None].expand_as(out)
        out[valid_rows].sum().backward()
        blob.update({f"{name}.q": q.numpy(), f"{name}.k": k.numpy(), f"{name}.v": v.numpy(),
                     f"{name}.coords": coords.numpy(), f"{name}.spreads": spreads.numpy(),
                     f"{name}.betas": betas.numpy(), f"{name}.mask": mask.numpy(),
                     f"{name}.min_rbf": np.float64(lo), f"{name}.max_rbf": np.float64(hi),
                     f"{name}.out": out.detach().numpy()})
        for nm, t in zip(("dq", "dk", "dv", "dspreads", "dbetas"), leaves):
            blob[f"{name}.{nm}"] = t.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "geoattn_reference.npz"), **blob)

    blob = {}
    g = torch.Generator().manual_seed(20240604)
    for name, (q, k, v, coords, spreads, betas, mask, lo, hi) in attn_d64_cases().items():
        # The dense reference gives NaN rows for padded queries, which poison dK and dV of the whole sample.  The
        # reference function therefore runs, unmodified, on the valid prefix only (no mask needed); the stored
        # inputs keep the padded length, so a kernel under test must also get the masking right.
        nv = int((~mask[0]).sum())
        assert not mask[0, :nv].any() and mask[0, nv:].all() and q.shape[0] == 1
        leaves = [t.clone().requires_grad_(True) for t in (q[:, :, :nv], k[:, :, :nv], v[:, :, :nv], spreads, betas)]
        out = torch_attn(leaves[0], leaves[1], leaves[2], coords[:, :nv], leaves[3], leaves[4],
                         torch.zeros(1, nv, dtype=torch.bool), lo, hi)  # (mask=None trips a dtype bug in the reference)
        d_out = torch.randn(q.shape, generator=g).to(torch.bfloat16).float()
        out.mul(d_out[:, :, :nv]).sum().backward()
        blob[f"{name}.n_valid"] = np.int64(nv)
        to16 = lambda t: t.to(torch.bfloat16).view(torch.int16).numpy()  # bf16 bit patterns
        blob.update({f"{name}.q": to16(q), f"{name}.k": to16(k), f"{name}.v": to16(v), f"{name}.d_out": to16(d_out),
                     f"{name}.coords": coords.numpy(), f"{name}.spreads": spreads.numpy(), f"{name}.betas": betas.numpy(),
                     f"{name}.mask": mask.numpy(), f"{name}.min_rbf": np.float64(lo), f"{name}.max_rbf": np.float64(hi),
                     f"{name}.out": out.detach().numpy().astype(np.float32)})
        for nm, t in zip(("dq", "dk", "dv", "dspreads", "dbetas"), leaves):
            blob[f"{name}.{nm}"] = t.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "geoattn_reference_d64.npz"), **blob)

    # anisotropic WE with per-wavenumber C-beta scaling: outputs and autograd gradients of the reference function
    aniso_torch = extract(os.path.join(ref_root, "tests/wf_embed/wf_embed_aniso_learnCB_learnK.py"), "wf_embedding_torch")
    g = torch.Generator().manual_seed(20240605)
    blob = {}
    z, n, k = 2, 80, 12
    cases = {}
    # the reference test's own input style: A = max_wl * rand, B = normalised randn, cb = rand, wavenumbers = randn
    a = 20 * torch.rand((z, n, 3), generator=g)
    b = torch.randn((z, n, 3), generator=g)
    b = b / torch.linalg.vector_norm(b, dim=2, keepdim=True)
    a[1, 8] = a[1, 7]  # a coincident pair
    cases["rand"] = (a, b, torch.rand((k,), generator=g), torch.randn((k,), generator=g), torch.zeros(z, n, dtype=torch.bool))
    c, m = chains.chain_batch([80, 51], 80, seed=17)
    cases["chain_padded"] = (torch.from_numpy(c), b, torch.rand((k,), generator=g) * 2, torch.from_numpy(chains.wavenumbers(2 * k)),
                             torch.from_numpy(m))
    for name, (ca, cbv, cbm, wn, mask) in cases.items():
        cbm_g, wn_g = cbm.clone().requires_grad_(True), wn.clone().requires_grad_(True)
        out = aniso_torch(ca, cbv, cbm_g, wn_g, mask)
        d_out = torch.randn(out.shape, generator=g)
        (out * d_out).sum().backward()
        blob.update({f"{name}.coords_a": ca.numpy(), f"{name}.coords_b": cbv.numpy(), f"{name}.cb": cbm.numpy(), f"{name}.wn": wn.numpy(),
                     f"{name}.mask": mask.numpy(), f"{name}.d_out": d_out.numpy(), f"{name}.out": out.detach().numpy(),
                     f"{name}.d_cb": cbm_g.grad.numpy(), f"{name}.d_wn": wn_g.grad.numpy()})
    np.savez_compressed(os.path.join(HERE, "we_aniso_reference.npz"), **blob)
    gnn_golden(ref_root)
    print("wrote", sorted(os.listdir(HERE)))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference [gnn]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else None)
