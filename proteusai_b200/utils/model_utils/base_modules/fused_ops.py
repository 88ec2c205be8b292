"""Fused bf16 row operations of the encoder block (inference): ``LayerNorm(x + y)`` in one pass and the erf GELU.

The reference runs these as PyTorch operators (``old/old_scripts/encoder.py:30-39``,
``utils/model_utils/base_modules/base_modules.py:46-52``); here they are single HBM-bound kernels behind
``pai_add_layernorm_bf16`` / ``pai_gelu_bf16``.  They have no backward: the modules use them only when no gradient is
being recorded and fall back to the PyTorch operators otherwise.
"""
import torch

from proteusai_b200 import _lib


def usable(*tensors):
    """The fused kernels apply to bf16 CUDA tensors when autograd is not recording."""
    if torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
        return False
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors)


def add_layernorm(x, y, weight, bias, eps):
    """``LayerNorm(x + y)`` over the last axis (``y`` may be ``None``); ``weight``/``bias`` bf16 or fp32."""
    d = x.shape[-1]
    x = x.contiguous()
    y = None if y is None else y.contiguous()
    fp32 = weight.dtype == torch.float32
    if weight.dtype != bias.dtype or weight.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("LayerNorm weight and bias must both be bf16 or both fp32")
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().pai_add_layernorm_bf16(
            _lib.ptr(x), _lib.ptr(y), _lib.ptr(weight.detach().contiguous()), _lib.ptr(bias.detach().contiguous()), int(fp32),
            _lib.ptr(out), x.numel() // d, d, float(eps), _lib.current_stream()), "pai_add_layernorm_bf16")
    return out


def gelu(x, inplace=False):
    """Erf GELU of a bf16 tensor whose element count is a multiple of 8."""
    x = x.contiguous()
    out = x if inplace else torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().pai_gelu_bf16(_lib.ptr(x), _lib.ptr(out), x.numel(), _lib.current_stream()), "pai_gelu_bf16")
    return out
