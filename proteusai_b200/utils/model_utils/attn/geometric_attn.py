"""Geometric attention: the reference's Python surface over the B200 tcgen05 kernels.

Same names, argument order and gradient tuple as ``old/old_scripts/attn/geometric_attn.py:545-660``
(imported by the reference as ``utils.model_utils.attn.geometric_attn``):
``geometric_attn(Q, K, V, coords, spreads, betas, mask=None, min_rbf=0.0, max_rbf=1.0)`` returns
``[Z, H, N, d]``; the backward returns ``(dQ, dK, dV, None, d_spreads, d_betas, None, None, None)``.

Two logit forms are available, chosen per call (``form=`` of ``geometric_attn``, ``logit_form=`` of ``GeoAttention``)
or, when a call does not say, by the module default (``set_logit_form``):

``"one_plus_rbf"`` (default)  the form the reference's README states, ``S * (1 + exp(-d^2 / (2 sigma_h^2)))``, a pair
                              valid iff both tokens are unpadded; ``betas``, ``min_rbf`` and ``max_rbf`` stay in the
                              signature for compatibility and do not enter; ``d_betas`` is ``None``.  A call that
                              hands this form trainable ``betas`` or a window other than ``[0, 1]`` gets a warning:
                              a model trained with the reference tree's kernel needs ``"beta_abs"``.
``"beta_abs"``                the form the reference tree's Triton kernel and its test implement,
                              ``S + beta * Rn * |S|`` with ``Rn = 2 (R - min_rbf) / (max_rbf - min_rbf) - 1`` and pairs with
                              ``R`` outside ``[min_rbf, max_rbf]`` masked out (``geometric_attn.py:193-201``); ``d_betas``
                              is returned.

Products are bf16 x bf16 with fp32 accumulation (the reference casts to fp16); outputs and gradients come
back in the dtype of ``Q``.  Heads of up to 64 dimensions are supported (narrower ones run zero-padded to 64).
"""
import ctypes
import os
import warnings
from collections import OrderedDict

import torch

from proteusai_b200 import _lib

_FORMS = {"one_plus_rbf": 0, "beta_abs": 1}
_KERNEL_D = 64  # head dimension the kernels are built for; narrower heads are zero-padded by geometric_attn
_logit_form = os.environ.get("PROTEUS_GEOATTN_FORM", "one_plus_rbf")


def set_logit_form(name):
    """Select the logit form used by ``geometric_attn`` from now on; returns the previous one."""
    global _logit_form
    if name not in _FORMS:
        raise ValueError(f"logit form must be one of {sorted(_FORMS)}, not {name!r}")
    prev, _logit_form = _logit_form, name
    return prev


def get_logit_form():
    return _logit_form


_check_spreads = True


class spreads_known_positive:
    """Context in which ``geometric_attn`` skips its ``spreads > 0`` assertion.  The assertion copies a flag from the
    device and so stalls the host once per call; a caller whose spreads are positive by construction (``GeoAttention``:
    ``min_spread + exp(w)``) wraps its call in this to keep the launch queue running ahead of the GPU."""

    def __enter__(self):
        global _check_spreads
        self.prev, _check_spreads = _check_spreads, False

    def __exit__(self, *exc):
        global _check_spreads
        _check_spreads = self.prev


def geometric_attn(Q, K, V, coords, spreads, betas=None, mask=None, min_rbf=0.00, max_rbf=1.00, form=None):
    """wrapper so that the Function can be called with keyword arguments.  ``form``: ``"one_plus_rbf"``, ``"beta_abs"``
    or ``None`` for the module default (see the module docstring); the other arguments are the reference's."""
    if form is None:
        return _geometric_attn.apply(Q, K, V, coords, spreads, betas, mask, min_rbf, max_rbf)
    return _geometric_attn.apply(Q, K, V, coords, spreads, betas, mask, min_rbf, max_rbf, form)


_warned_ignored = False


def _warn_ignored_once(betas, min_rbf, max_rbf):
    """The ``one_plus_rbf`` form has no beta and no RBF window: say so once if the caller seems to rely on them."""
    global _warned_ignored
    if _warned_ignored:
        return
    what = []
    if betas is not None and betas.requires_grad:
        what.append("trainable betas (they receive no gradient)")
    if float(min_rbf) != 0.0 or float(max_rbf) != 1.0:
        what.append(f"the RBF window [{min_rbf}, {max_rbf}]")
    if what:
        _warned_ignored = True
        warnings.warn("geometric_attn: the 'one_plus_rbf' logit form ignores " + " and ".join(what) +
                      "; pass form='beta_abs' (or set_logit_form('beta_abs')) for the reference tree's S + beta*Rn*|S| form",
                      stacklevel=3)


class GeoPlan:
    """Per-mask data shared by every attention call of a batch: the validity bytes the kernels read and the
    batch plan (non-empty 128-token tiles per sample, samples longest first) made by ``pai_geoattn_plan``."""

    __slots__ = ("mask", "version", "valid", "plan", "schedules")

    def __init__(self, mask):
        self.mask, self.version = mask, mask._version
        batch, n = mask.shape
        self.valid = (~mask.bool()).contiguous().view(torch.uint8)  # a bool is one byte, 0 or 1
        lib = _lib.lib()
        nbytes = lib.pai_geoattn_plan_bytes(batch, n)
        self.plan = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device=mask.device)
        with torch.cuda.device(mask.device):
            _lib.check(lib.pai_geoattn_plan(_lib.ptr(self.valid), batch, n, _lib.ptr(self.plan), nbytes, _lib.current_stream()),
                       "pai_geoattn_plan")
        self.schedules = {}

    def schedule(self, nheads, backward):
        """``(tensor, bins)``: the balanced assignment of this plan's work items to persistent CTAs for ``nheads`` heads
        (``pai_geoattn_schedule``), made on first use; two CTAs per SM for the forward, one for the backward."""
        key = (int(nheads), bool(backward))
        hit = self.schedules.get(key)
        if hit is None:
            batch, n = self.mask.shape
            sms = torch.cuda.get_device_properties(self.plan.device).multi_processor_count
            bins = min(sms * (1 if backward else 2), 1024)
            if batch * nheads * ((n + 127) // 128) > 8 * bins:
                # many items per CTA slot: one CTA per item, issued longest first, balances by itself
                hit = self.schedules[key] = (None, 0)
                return hit
            lib = _lib.lib()
            nbytes = lib.pai_geoattn_schedule_bytes(batch, n, nheads, bins)
            sched = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device=self.plan.device)
            with torch.cuda.device(self.plan.device):
                _lib.check(lib.pai_geoattn_schedule(_lib.ptr(self.plan), batch, n, nheads, bins, 1 if backward else 0, _lib.ptr(sched),
                                                    nbytes, _lib.current_stream()), "pai_geoattn_schedule")
            hit = self.schedules[key] = (sched, bins)
        return hit


_plans = OrderedDict()  # (data_ptr, shape, device) -> GeoPlan; the entry keeps its mask alive, so the address cannot be reused
_PLAN_CACHE = 8


def geoattn_plan(mask):
    """The ``GeoPlan`` of a key-padding mask ``[Z,N]`` (True = padded), or ``None`` for ``mask=None``.  Plans are cached
    by mask tensor (address and version counter), so the layers of a model, and forward and backward, share one:
    the mask is inverted and scanned once per batch, not once per call."""
    if mask is None:
        return None
    if not mask.is_cuda:
        raise RuntimeError("geometric_attn needs CUDA tensors: there is no CPU path")
    key = (mask.data_ptr(), tuple(mask.shape), mask.dtype, mask.device)
    hit = _plans.get(key)
    if hit is not None and hit.mask is mask and hit.version == mask._version:
        _plans.move_to_end(key)
        return hit
    plan = GeoPlan(mask)
    _plans[key] = plan
    _plans.move_to_end(key)
    while len(_plans) > _PLAN_CACHE:
        _plans.popitem(last=False)
    return plan


def _strided_ok(t):
    """True when the kernel can read/write ``t`` ``[Z,H,N,d]`` in place: d contiguous, rows on 16-byte boundaries."""
    return t.stride(3) == 1 and all(t.size(a) == 1 or (t.stride(a) % 8 == 0 and t.stride(a) >= t.size(3)) for a in range(3))


def _strides3(t):
    return (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def geoattn_forward(Q, K, V, coords, spreads, mask=None, zh_begin=0, zh_end=None, out=None, lse=None,
                    betas=None, min_rbf=0.0, max_rbf=1.0, form="one_plus_rbf", out_layout="zhnd", scale=None,
                    q_begin=0, q_end=None):
    """Forward on the (batch, head) pairs ``[zh_begin, zh_end)`` and the query rows ``[q_begin, q_end)`` (``q_begin`` a
    multiple of 128, ``q_end`` a multiple of 128 or N).  Q, K, V are bf16 ``[Z,H,N,d]``, read in place through
    their strides when ``d`` is contiguous and the other strides are multiples of 8 elements (for instance the permuted
    views of a fused projection output ``[Z,N,3,H,d]``), copied otherwise.  Returns ``(O bf16 [Z,H,N,d], L fp32 [Z,H,N])``;
    only the pairs and rows of the ranges are written.  ``out_layout="znhd"`` allocates O as ``[Z,N,H,d]`` in memory and
    returns its ``[Z,H,N,d]`` view, so that ``O.permute(0, 2, 1, 3).reshape(Z, N, H*d)`` is free.  ``scale`` is the
    softmax scale (default ``1/sqrt(d)``)."""
    if not Q.is_cuda:
        raise RuntimeError("geometric_attn needs CUDA tensors: there is no CPU path")
    batch, nheads, n, d_k = Q.shape
    Q, K, V = (t if _strided_ok(t) else t.contiguous() for t in (Q, K, V))
    zh_end = batch * nheads if zh_end is None else zh_end
    q_end = n if q_end is None else q_end
    dev = Q.device
    coords = coords.to(torch.float32).contiguous()
    sigma = spreads.detach().to(torch.float32).contiguous()
    gp = geoattn_plan(mask)
    # the whole problem in one call: use the balanced schedule of persistent CTAs
    whole = gp is not None and zh_begin == 0 and zh_end == batch * nheads and q_begin == 0 and q_end == n
    sched, bins = gp.schedule(nheads, False) if whole else (None, 0)
    beta = None if betas is None else betas.detach().to(torch.float32).contiguous()
    if out is None:
        if out_layout == "znhd":
            out = torch.empty(batch, n, nheads, d_k, dtype=torch.bfloat16, device=dev).permute(0, 2, 1, 3)
        else:
            out = torch.empty(batch, nheads, n, d_k, dtype=torch.bfloat16, device=dev)
    elif not _strided_ok(out):
        raise ValueError("out must have a contiguous last axis and strides that are multiples of 8 elements")
    if lse is None:
        lse = torch.empty(batch, nheads, n, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().pai_geoattn_fwd_strided(
            _lib.ptr(Q), _strides3(Q), _lib.ptr(K), _strides3(K), _lib.ptr(V), _strides3(V), _lib.ptr(coords), _lib.ptr(sigma),
            _lib.ptr(beta), _lib.ptr(gp.valid) if gp else None, _lib.ptr(gp.plan) if gp else None, _lib.ptr(sched), bins, _lib.ptr(out),
            _strides3(out),
            _lib.ptr(lse), batch, nheads, n, d_k, float(scale) if scale is not None else 1.0 / (d_k ** 0.5), float(min_rbf),
            float(max_rbf), _FORMS[form], zh_begin, zh_end, q_begin, q_end, _lib.current_stream()), "pai_geoattn_fwd_strided")
    return out, lse


def geoattn_backward(Q, K, V, O, dO, lse, coords, spreads, mask=None, zh_begin=0, zh_end=None,
                     betas=None, min_rbf=0.0, max_rbf=1.0, form="one_plus_rbf", scale=None, q_begin=0, q_end=None):
    """Gradients on the (batch, head) pairs ``[zh_begin, zh_end)``.  Q, K, V, O, dO bf16 contiguous.
    Returns fp32 ``(dQ, dK, dV [Z,H,N,d], d_spreads [H])`` and, for the ``beta_abs`` form, ``d_betas [H]`` as a fifth
    element; only the pairs of the range are written.  With a query range ``[q_begin, q_end)`` only those query rows
    contribute: their dQ rows are written and dK, dV, d_spreads, d_betas are partial sums to be added over the shards."""
    batch, nheads, n, d_k = Q.shape
    zh_end = batch * nheads if zh_end is None else zh_end
    q_end = n if q_end is None else q_end
    dev = Q.device
    coords = coords.to(torch.float32).contiguous()
    sigma = spreads.detach().to(torch.float32).contiguous()
    gp = geoattn_plan(mask)
    whole = gp is not None and zh_begin == 0 and zh_end == batch * nheads and q_begin == 0 and q_end == n
    sched, bins = gp.schedule(nheads, True) if whole else (None, 0)
    dq, dk, dv = (torch.empty(batch, nheads, n, d_k, dtype=torch.float32, device=dev) for _ in range(3))
    dsig = torch.empty(nheads, dtype=torch.float32, device=dev)
    beta = None if betas is None else betas.detach().to(torch.float32).contiguous()
    dbeta = torch.empty(nheads, dtype=torch.float32, device=dev) if form == "beta_abs" else None
    lib = _lib.lib()
    ws_bytes = lib.pai_geoattn_bwd_workspace_bytes(batch, nheads, n, d_k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.pai_geoattn_bwd(
            _lib.ptr(Q), _lib.ptr(K), _lib.ptr(V), _lib.ptr(O), _lib.ptr(dO), _lib.ptr(lse), _lib.ptr(coords),
            _lib.ptr(sigma), _lib.ptr(beta), _lib.ptr(gp.valid) if gp else None, _lib.ptr(gp.plan) if gp else None, _lib.ptr(sched), bins,
            _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(dsig), _lib.ptr(dbeta), _lib.ptr(ws), ws_bytes, batch, nheads, n, d_k,
            float(scale) if scale is not None else 1.0 / (d_k ** 0.5), float(min_rbf), float(max_rbf), _FORMS[form], zh_begin,
            zh_end, q_begin, q_end, _lib.current_stream()), "pai_geoattn_bwd")
    if form == "beta_abs":
        return dq, dk, dv, dsig, dbeta
    return dq, dk, dv, dsig


class _geometric_attn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, Q, K, V, coords, spreads, betas, mask, min_rbf, max_rbf, form=None):
        # (the reference's nine arguments; the optional tenth selects the logit form for this call)
        ctx.n_inputs = 9 if form is None else 10
        assert Q.shape == K.shape == V.shape, f"Q, K, and V projection shapes must match, but got {Q.shape=}, {K.shape=}, {V.shape=}"
        batch, nheads, N, d_k = Q.shape
        assert coords.dim() == 3 and coords.size(2) == 3, f"coordinates must be of shape (batch, N, 3), not {coords.shape}"
        assert spreads.size(0) == nheads, f"number of spreads per batch must be equal to nheads, not {spreads.size(0)=} and {nheads=}"
        if _check_spreads:  # reads the device back (a host synchronisation), as the reference's assert does
            assert torch.all(spreads > 0), f"spreads must be a tensor of positive, non-zero floats, not {spreads}"
        # Without a backward to prepare for, Q, K, V are read through their strides (no copies) and O is laid out
        # [Z,N,H,d] in memory, which is what the head concatenation that follows wants; the backward kernels read
        # contiguous [Z,H,N,d] tensors, so with gradients everything is made contiguous here once.
        needs_bwd = any(ctx.needs_input_grad)
        if d_k > _KERNEL_D:
            raise RuntimeError(f"geometric_attn: head dimension {d_k} is not supported by the B200 kernel (at most {_KERNEL_D})")
        scale = 1.0 / (d_k ** 0.5)
        if d_k < _KERNEL_D:
            # The kernel is built for heads of 64.  Narrower heads (the reference's own test uses 32) run zero-padded:
            # zeros add nothing to Q K^T, the extra columns of V give zero columns of O, and the softmax scale stays
            # that of the true width.  The padded columns are cut off again below (and from the gradients).
            pad = lambda t: torch.nn.functional.pad(t.to(torch.bfloat16), (0, _KERNEL_D - d_k))
            qb, kb, vb = pad(Q), pad(K), pad(V)
        elif needs_bwd:
            qb, kb, vb = (t.to(torch.bfloat16).contiguous() for t in (Q, K, V))
        else:
            qb, kb, vb = (t.to(torch.bfloat16) for t in (Q, K, V))
        form = _logit_form if form is None else form
        if form not in _FORMS:
            raise ValueError(f"logit form must be one of {sorted(_FORMS)}, not {form!r}")
        if form == "beta_abs" and betas is None:
            raise ValueError("the beta_abs logit form needs betas")
        if form == "one_plus_rbf":
            _warn_ignored_once(betas, min_rbf, max_rbf)
        out, lse = geoattn_forward(qb, kb, vb, coords, spreads, mask, betas=betas, min_rbf=min_rbf, max_rbf=max_rbf, form=form,
                                   out_layout="zhnd" if needs_bwd else "znhd", scale=scale)
        ctx.save_for_backward(qb, kb, vb, out, lse, coords, spreads, mask if mask is not None else torch.empty(0),
                              betas if betas is not None else torch.empty(0))
        ctx.has_mask = mask is not None
        ctx.form, ctx.min_rbf, ctx.max_rbf = form, min_rbf, max_rbf
        ctx.in_dtype = Q.dtype
        ctx.spread_dtype = spreads.dtype
        ctx.d_k, ctx.scale = d_k, scale
        return out[..., :d_k].to(Q.dtype)

    @staticmethod
    def backward(ctx, dO):
        qb, kb, vb, out, lse, coords, spreads, mask, betas = ctx.saved_tensors
        mask = mask if ctx.has_mask else None
        dt = ctx.in_dtype
        d_k = ctx.d_k
        if d_k < _KERNEL_D:
            dO = torch.nn.functional.pad(dO, (0, _KERNEL_D - d_k))
        tail = (None,) * (ctx.n_inputs - 6)  # mask, min_rbf, max_rbf (and the form, when it was passed)
        if ctx.form == "beta_abs":
            dq, dk, dv, dsig, dbeta = geoattn_backward(qb, kb, vb, out, dO.to(torch.bfloat16).contiguous(), lse, coords, spreads,
                                                       mask, betas=betas, min_rbf=ctx.min_rbf, max_rbf=ctx.max_rbf, form=ctx.form,
                                                       scale=ctx.scale)
            return (dq[..., :d_k].to(dt), dk[..., :d_k].to(dt), dv[..., :d_k].to(dt), None, dsig.to(ctx.spread_dtype),
                    dbeta.to(betas.dtype)) + tail
        dq, dk, dv, dsig = geoattn_backward(qb, kb, vb, out, dO.to(torch.bfloat16).contiguous(), lse, coords, spreads, mask,
                                            scale=ctx.scale)
        return (dq[..., :d_k].to(dt), dk[..., :d_k].to(dt), dv[..., :d_k].to(dt), None, dsig.to(ctx.spread_dtype), None) + tail
