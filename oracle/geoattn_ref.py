"""CPU oracle for the Geometric Attention (test infrastructure).

Restates, line by line, the reference's dense PyTorch formulation ``torch_attn`` in
``tests/attn/geo_attn.py:172-212``.  Two logit forms share every other line:

``variant="beta_abs"``      the form the reference tree implements and tests,
                            ``S + beta * Rn * |S|`` with ``Rn = 2 (R - min_rbf) / (max_rbf - min_rbf) - 1``
                            and pairs with ``R`` outside ``[min_rbf, max_rbf]`` masked out
                            (``tests/attn/geo_attn.py:204-207``,
                            ``old/old_scripts/attn/geometric_attn.py:196-201``).
                            Pinned bit for bit against the reference function by the
                            committed golden vectors.
``variant="one_plus_rbf"``  the form the reference README states (``README.md:40``),
                            ``S * (1 + R)`` with ``R = exp(-d^2 / (2 sigma_h^2))``, a pair valid iff
                            query and key are both unpadded.  Differs from the pinned form
                            in the one logit line; parity unpinned by the reference's own
                            tests for that line (no reference code evaluates it).

Rows of padded queries are set to 0 afterwards, which is what the reference kernel
stores for them (``geometric_attn.py:233``); the dense softmax alone gives NaN there.
"""
import torch


def geoattn_ref(Q, K, V, coords, spreads, betas=None, mask=None, min_rbf=0.0, max_rbf=1.0,
                variant="one_plus_rbf", zero_padded_rows=True):
    """Q, K, V ``[Z, H, N, d]``; coords ``[Z, N, 3]``; spreads/betas ``[H]``; mask ``[Z, N]``
    bool, True = padded.  Computes in the dtype of Q.  Returns O ``[Z, H, N, d]``."""
    batch, nheads, n, d_k = Q.shape
    mask = torch.zeros(batch, n, dtype=torch.bool) if mask is None else mask
    coords = coords.to(Q.dtype)
    spreads = spreads.to(Q.dtype)
    S = torch.matmul(Q, K.transpose(2, 3)) / (d_k ** 0.5)  # geo_attn.py:194
    dists = torch.sqrt(torch.sum((coords[:, :, None, :] - coords[:, None, :, :]) ** 2, axis=3))[:, None, :, :]  # :196
    rbfs = torch.exp(-(dists ** 2) / (2 * (spreads[None, :, None, None] ** 2)))  # :202
    attn_mask = mask[:, None, :, None] | mask[:, None, None, :]  # :204 (first two terms)
    if variant == "beta_abs":
        b = betas.to(Q.dtype)[None, :, None, None]
        attn_mask = attn_mask | (rbfs < min_rbf) | (rbfs > max_rbf)  # :204
        rbfs = (2 * (rbfs - min_rbf) / (max_rbf - min_rbf)) - 1  # :205
        S = torch.where(attn_mask, -float("inf"), S + b * rbfs * torch.abs(S))  # :207
    elif variant == "one_plus_rbf":
        S = torch.where(attn_mask, -float("inf"), S * (1 + rbfs))
    else:
        raise ValueError(variant)
    P = torch.softmax(S, dim=-1)  # :208
    if zero_padded_rows:
        # a row with every key masked: softmax gives NaN, the kernel stores 0
        dead = torch.all(attn_mask, dim=-1, keepdim=True)
        P = torch.where(dead, torch.zeros_like(P), P)
    return torch.matmul(P, V)  # :210


def geoattn_grads_autograd(Q, K, V, coords, spreads, dO, mask=None, variant="one_plus_rbf",
                           betas=None, min_rbf=0.0, max_rbf=1.0, dtype=torch.float32):
    """O and (dQ, dK, dV, d_spreads[, d_betas]) by autograd through :func:`geoattn_ref`."""
    leaves = [t.detach().to(dtype).clone().requires_grad_(True) for t in (Q, K, V, spreads)]
    b = None
    if variant == "beta_abs":
        b = betas.detach().to(dtype).clone().requires_grad_(True)
    O = geoattn_ref(leaves[0], leaves[1], leaves[2], coords, leaves[3], b, mask, min_rbf, max_rbf, variant)
    O.backward(dO.to(dtype))
    grads = [t.grad if t.grad is not None else torch.zeros_like(t) for t in leaves]
    if b is not None:
        grads.append(b.grad)
    return O.detach(), grads


def geoattn_grads_closed_form(Q, K, V, coords, spreads, dO, mask=None, dtype=torch.float64):
    """Closed-form gradients of the ``one_plus_rbf`` form, the formulas the kernel evaluates
    (``old/old_scripts/attn/geometric_attn.py:463-504`` with ``SR = S (1 + R)``):
    ``dV = P^T dO``, ``dP = dO V^T``, ``D = rowsum(O * dO)``, ``dSR = P * (dP - D)``,
    ``dS = dSR (1 + R)``, ``dQ = dS K scale``, ``dK = dS^T Q scale``,
    ``dsigma_h = sum dSR * S * R * d^2 / sigma_h^3``.  Returns (O, L, dQ, dK, dV, dsigma)."""
    Q, K, V, dO = (t.to(dtype) for t in (Q, K, V, dO))
    coords, spreads = coords.to(dtype), spreads.to(dtype)
    z, h, n, d = Q.shape
    mask = torch.zeros(z, n, dtype=torch.bool) if mask is None else mask
    scale = 1.0 / d ** 0.5
    S = torch.matmul(Q, K.transpose(2, 3)) * scale
    d2 = torch.sum((coords[:, :, None, :] - coords[:, None, :, :]) ** 2, dim=3)[:, None]
    R = torch.exp(-d2 / (2 * spreads[None, :, None, None] ** 2))
    pm = mask[:, None, :, None] | mask[:, None, None, :]
    SR = torch.where(pm, -float("inf"), S * (1 + R))
    L = torch.logsumexp(SR, dim=-1)  # -inf on dead rows
    P = torch.where(pm, torch.zeros_like(SR), torch.exp(SR - torch.where(torch.isinf(L), torch.zeros_like(L), L)[..., None]))
    O = torch.matmul(P, V)
    dO = torch.where(mask[:, None, :, None], torch.zeros_like(dO), dO)
    dV = torch.matmul(P.transpose(2, 3), dO)
    dP = torch.matmul(dO, V.transpose(2, 3))
    D = torch.sum(O * dO, dim=-1, keepdim=True)
    dSR = P * (dP - D)
    dS = dSR * (1 + R)
    dQ = torch.matmul(dS, K) * scale
    dK = torch.matmul(dS.transpose(2, 3), Q) * scale
    dsig = torch.sum(dSR * S * R * d2 / spreads[None, :, None, None] ** 3, dim=(0, 2, 3))
    return O, L, dQ, dK, dV, dsig
