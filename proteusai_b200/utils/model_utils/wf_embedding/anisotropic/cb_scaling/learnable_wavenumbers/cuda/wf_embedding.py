"""Anisotropic Wavefunction Embedding with per-wavenumber C-beta scaling: the reference's Python surface over the
B200 kernel.

Same names, argument order and gradient tuple as
``utils/model_utils/wf_embedding/anisotropic/cb_scaling/learnable_wavenumbers/cuda/wf_embedding.py:16-79`` of the
reference: ``wf_embedding(coordsA, coordsB, cb_magnitudes, wavenumbers, mask=None)`` returns ``[Z, N, 2K]``; the backward
returns gradients for ``cb_magnitudes`` and ``wavenumbers`` only.  ``mask=None`` means "no padding" (the reference
crashes on it); padding travels as an explicit validity array instead of the x == 12345 sentinel; the backward
reduction is one fused kernel pair instead of PyTorch elementwise products and sums.
"""
import torch

from proteusai_b200 import _lib


def wf_embedding(coordsA, coordsB, cb_magnitudes, wavenumbers, mask=None):
    return _wf_embedding.apply(coordsA, coordsB, cb_magnitudes, wavenumbers, mask)


def we_aniso_forward_rows(coordsA, coordsB, cb_magnitudes, wavenumbers, mask=None, row_begin=0, row_end=None):
    """Forward on observer rows ``[row_begin, row_end)``; returns ``(out, d_cb, d_k)``, each ``[Z, N, 2K]`` fp32
    (only the rows of the range are written)."""
    if not coordsA.is_cuda:
        raise RuntimeError("wf_embedding needs CUDA tensors: there is no CPU path")
    batch, n, space = coordsA.shape
    assert space == 3 and coordsB.shape == coordsA.shape
    row_end = n if row_end is None else row_end
    a = coordsA.transpose(1, 2).to(torch.float32).contiguous()
    b = coordsB.transpose(1, 2).to(torch.float32).contiguous()
    cb = cb_magnitudes.detach().to(torch.float32).contiguous()
    wn = wavenumbers.detach().to(torch.float32).contiguous()
    k = wn.shape[0]
    assert cb.shape[0] == k
    valid = None if mask is None else (~mask.bool()).contiguous().view(torch.uint8)  # a bool is one byte, 0 or 1
    dev = coordsA.device
    out, d_cb, d_k = (torch.empty(batch, n, 2 * k, dtype=torch.float32, device=dev) for _ in range(3))
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().pai_we_aniso_fwd(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(valid), _lib.ptr(cb), _lib.ptr(wn), _lib.ptr(out), _lib.ptr(d_cb), _lib.ptr(d_k),
            batch, n, k, row_begin, row_end, _lib.current_stream()), "pai_we_aniso_fwd")
    return out, d_cb, d_k


def we_aniso_backward(d_out, d_cb, d_k, row_begin=0, row_end=None):
    """``(grad_cb_magnitudes [K], grad_wavenumbers [K])`` from the stored partials over rows ``[row_begin, row_end)``."""
    batch, n, d_model = d_cb.shape
    k = d_model // 2
    row_end = n if row_end is None else row_end
    d_out = d_out.to(torch.float32).contiguous()
    dev = d_out.device
    g_cb, g_k = torch.empty(k, dtype=torch.float32, device=dev), torch.empty(k, dtype=torch.float32, device=dev)
    lib = _lib.lib()
    ws_bytes = lib.pai_we_aniso_bwd_workspace_bytes(batch, n, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.pai_we_aniso_bwd(
            _lib.ptr(d_out), _lib.ptr(d_cb), _lib.ptr(d_k), _lib.ptr(g_cb), _lib.ptr(g_k), _lib.ptr(ws), ws_bytes,
            batch, n, k, row_begin, row_end, _lib.current_stream()), "pai_we_aniso_bwd")
    return g_cb, g_k


class _wf_embedding(torch.autograd.Function):

    @staticmethod
    def forward(ctx, coordsA, coordsB, cb_magnitudes, wavenumbers, mask):
        out, d_cb, d_k = we_aniso_forward_rows(coordsA, coordsB, cb_magnitudes, wavenumbers, mask)
        ctx.save_for_backward(d_cb, d_k)
        ctx.dtypes = (cb_magnitudes.dtype, wavenumbers.dtype)
        return out.to(coordsA.dtype)

    @staticmethod
    def backward(ctx, dO):
        d_cb, d_k = ctx.saved_tensors
        g_cb, g_k = we_aniso_backward(dO, d_cb, d_k)
        return None, None, g_cb.to(ctx.dtypes[0]), g_k.to(ctx.dtypes[1]), None
