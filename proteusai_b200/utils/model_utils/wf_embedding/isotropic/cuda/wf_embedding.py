"""Isotropic Wavefunction Embedding: the reference's Python surface over the B200 kernels.

Same names, argument order and return values as
``utils/model_utils/wf_embedding/isotropic/cuda/wf_embedding.py:18-83`` of the reference:
``wf_embedding(coords, wavenumbers, magnitude_type=1, dropout_p=0.0, mask=None)`` and the
``_wf_embedding`` autograd Function whose backward returns a gradient for the wavenumbers only.
Differences, all supersets: ``mask=None`` means "no padding" (the reference crashes on it);
padding travels as an explicit validity array instead of the x == 12345 sentinel; the backward
reduction is one fused kernel instead of three elementwise PyTorch kernels and a sum.
Dropout (``dropout_p > 0``) follows the reference kernel's index hash.
"""
import numpy as np
import torch

from proteusai_b200 import _lib


def wf_embedding(coords, wavenumbers, magnitude_type=1, dropout_p=0.0, mask=None):
    return _wf_embedding.apply(coords, wavenumbers, magnitude_type, dropout_p, mask)


def we_forward_rows(coords, wavenumbers, magnitude_type=1, mask=None, row_begin=0, row_end=None,
                    out=None, cos_sums=None, sin_sums=None, dropout_p=0.0, seed=0, reproducible=False):
    """Run the forward kernel on observer rows ``[row_begin, row_end)`` of every batch element.

    Returns ``(out [Z,N,2K], cos_sums [Z,N,K], sin_sums [Z,N,K])``; only the rows of the range are
    written (the other rows of freshly allocated buffers are left uninitialised).  This is the
    multi-GPU building block: every rank holds all coordinates and computes its own rows.
    With ``dropout_p > 0`` evaluations are dropped by the reference kernel's index hash under ``seed``
    (the pattern does not depend on the row range, so all ranks of a sharded call pass the same seed).
    ``reproducible=True`` asks for sums that are bit-identical from launch to launch (``PAI_WE_REPRODUCIBLE``
    of the C ABI): by default partial sums are added in arrival order and the last bit can differ.
    """
    assert magnitude_type in [0, 1, 2, 3]  # mag=1, 1/|R|, 1/log2(|R|), 1/sqrt(|R|)
    if not coords.is_cuda:
        raise RuntimeError("wf_embedding needs CUDA tensors: there is no CPU path")
    batch, n, space = coords.shape
    assert space == 3
    row_end = n if row_end is None else row_end
    # [Z,3,N] fp32 planes, as the reference lays them out for its kernel (wf_embedding.py:32)
    planes = coords.transpose(1, 2).to(torch.float32).contiguous()
    wn = wavenumbers.detach().to(torch.float32).contiguous()
    k = wn.shape[0]
    valid = None if mask is None else (~mask.bool()).contiguous().view(torch.uint8)  # a bool is one byte, 0 or 1
    dev = coords.device
    if out is None:
        out = torch.empty(batch, n, 2 * k, dtype=torch.float32, device=dev)
    if cos_sums is None:
        cos_sums = torch.empty(batch, n, k, dtype=torch.float32, device=dev)
    if sin_sums is None:
        sin_sums = torch.empty(batch, n, k, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().pai_we_fwd(
            _lib.ptr(planes), _lib.ptr(valid), _lib.ptr(wn), _lib.ptr(out), _lib.ptr(cos_sums), _lib.ptr(sin_sums),
            batch, n, k, row_begin, row_end, magnitude_type, float(dropout_p), int(seed) & 0xFFFFFFFF,
            _lib.WE_REPRODUCIBLE if reproducible else 0, _lib.current_stream()), "pai_we_fwd")
    return out, cos_sums, sin_sums


def we_backward_dk(d_out, cos_sums, sin_sums, row_begin=0, row_end=None):
    """``dk [K]`` from the stored sums over rows ``[row_begin, row_end)`` (fused reduction kernel)."""
    batch, n, k = cos_sums.shape
    row_end = n if row_end is None else row_end
    d_out = d_out.to(torch.float32).contiguous()
    dev = d_out.device
    dk = torch.empty(k, dtype=torch.float32, device=dev)
    lib = _lib.lib()
    ws_bytes = lib.pai_we_bwd_dk_workspace_bytes(batch, n, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.pai_we_bwd_dk(
            _lib.ptr(d_out), _lib.ptr(cos_sums), _lib.ptr(sin_sums), _lib.ptr(dk), _lib.ptr(ws), ws_bytes,
            batch, n, k, row_begin, row_end, _lib.current_stream()), "pai_we_bwd_dk")
    return dk


class _wf_embedding(torch.autograd.Function):

    @staticmethod
    def forward(ctx, coords, wavenumbers, magnitude_type, dropout_p, mask):
        # a fresh 32-bit seed per call, drawn as the reference draws it (wf_embedding.py:48-49)
        seed = int(np.random.default_rng().integers(0, 2**32, dtype=np.uint32)) if dropout_p != 0.0 else 0
        out, cos_sums, sin_sums = we_forward_rows(coords, wavenumbers, magnitude_type, mask, dropout_p=dropout_p, seed=seed)
        ctx.save_for_backward(cos_sums, sin_sums)
        ctx.wn_dtype = wavenumbers.dtype
        return out

    @staticmethod
    def backward(ctx, dO):
        # padded rows hold zeros in both sums, so they drop out without the mask
        cos_sums, sin_sums = ctx.saved_tensors
        dk = we_backward_dk(dO, cos_sums, sin_sums)
        return None, dk.to(ctx.wn_dtype), None, None, None
