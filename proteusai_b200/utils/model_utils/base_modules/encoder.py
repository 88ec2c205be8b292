"""``GeoAttention`` and ``Encoder`` modules over the B200 geometric-attention kernel, and the small
encoder-only model used as the end-to-end inference configuration.

``GeoAttention`` keeps the reference's constructor, parameter names and semantics
(``old/old_scripts/encoder.py:43-121``): per-head projection weights ``q_proj/k_proj/v_proj [H, d_model, d_k]``
with biases ``[H, d_k]``, ``spreads = min_spread + exp(spread_weights)``, ``betas = exp(beta_weights)``,
heads concatenated d_k-major / head-minor before the bias-free ``out_proj``.  The projections run as one GEMM
over all heads (and over Q, K, V together for self-attention) instead of the reference's per-head broadcast
matmul, which copies the input once per head.  ``logit_form`` (an addition to the reference's constructor) selects
the attention logit form for this module: ``"one_plus_rbf"`` (``S (1 + R)``; ``beta_weights``, ``min_rbf`` and ``max_rbf``
are then unused), ``"beta_abs"`` (the reference tree's ``S + beta Rn |S|`` with the RBF window, what a checkpoint trained
with the reference's own kernel expects), or ``None`` for the default of ``geometric_attn``.

``Encoder`` is the reference's post-norm block (``old/old_scripts/encoder.py:8-41``): ``LN(x + drop(attn))``
then ``LN(x + drop(ffn))``, each one fused kernel in bf16 inference.  The reference's ``forward`` passes ``coords_beta`` positionally into a
``GeoAttention.forward`` that has no such parameter (a TypeError there); here it is accepted and unused.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from proteusai_b200.utils.model_utils.attn import geometric_attn as _ga
from proteusai_b200.utils.model_utils.attn.geometric_attn import geometric_attn, spreads_known_positive
from proteusai_b200.utils.model_utils.base_modules import fused_ops
from proteusai_b200.utils.model_utils.base_modules.base_modules import MLP
from proteusai_b200.utils.model_utils.wf_embedding.wf_embedding import WaveFunctionEmbedding


class GeoAttention(nn.Module):

    def __init__(self, d_model=512, heads=8, min_spread=2.0, min_rbf=0.001, max_rbf=1.00, learn_spreads=True, logit_form=None):
        super().__init__()
        if logit_form is not None and logit_form not in ("one_plus_rbf", "beta_abs"):
            raise ValueError(f"logit_form must be 'one_plus_rbf', 'beta_abs' or None, not {logit_form!r}")
        self.logit_form = logit_form
        self._packed = {}  # inference-time cache of the fused projection weights (see _packed_weights)
        if d_model % heads != 0:
            raise ValueError(f"number of dimensions ({d_model}) must be divisible by number of attention heads ({heads})")
        self.heads, self.d_model, self.d_k = heads, d_model, d_model // heads
        self.spread_weights = nn.Parameter(torch.zeros(heads), requires_grad=learn_spreads)
        self.beta_weights = nn.Parameter(torch.zeros(heads))
        self.min_spread, self.min_rbf, self.max_rbf = min_spread, min_rbf, max_rbf
        bound = (6 / (self.d_k + d_model)) ** 0.5  # Xavier-uniform
        for name in ("q", "k", "v"):
            setattr(self, f"{name}_proj", nn.Parameter((torch.rand(heads, d_model, self.d_k) * 2 - 1) * bound))
            setattr(self, f"{name}_bias", nn.Parameter(torch.zeros(heads, self.d_k)))
        self.out_proj = nn.Linear(d_model, d_model, bias=False)

    def _cached(self, name, param, build):
        """``build()`` with gradients recorded; without, its value is kept until the parameter changes (version counter)."""
        if torch.is_grad_enabled() and param.requires_grad:
            return build()
        stamp = (param.data_ptr(), param._version)
        hit = self._packed.get(name)
        if hit is None or hit[0] != stamp:
            hit = (stamp, build())
            self._packed[name] = hit
        return hit[1]

    def get_spreads(self):
        return self._cached("spreads", self.spread_weights, lambda: self.min_spread + torch.exp(self.spread_weights))

    def get_betas(self):
        return self._cached("betas", self.beta_weights, lambda: torch.exp(self.beta_weights))

    def _packed_weights(self, names, dtype):
        """``[D, S*H*dk]`` weight and ``[S*H*dk]`` bias of the fused projection for the weight sets ``names`` (``"q"``,
        ``"k"``, ``"v"``), in ``dtype``.  Without gradient recording the packed tensors are kept and reused until a
        parameter changes (its version counter moves), so a forward does no concatenation or cast; with gradients they
        are rebuilt every call so that autograd sees the parameters."""
        ws = [getattr(self, f"{n}_proj") for n in names]
        bs = [getattr(self, f"{n}_bias") for n in names]
        build = lambda: (
            torch.cat([w.permute(1, 0, 2).reshape(self.d_model, self.heads * self.d_k) for w in ws], dim=1).to(dtype).contiguous(),
            torch.cat([b.reshape(self.heads * self.d_k) for b in bs]).to(dtype).contiguous())
        if torch.is_grad_enabled() and any(t.requires_grad for t in ws + bs):
            return build()
        key = ("proj", names, dtype, ws[0].device)
        stamp = tuple((t.data_ptr(), t._version) for t in ws + bs)
        hit = self._packed.get(key)
        if hit is None or hit[0] != stamp:
            hit = (stamp, build())
            self._packed[key] = hit
        return hit[1]

    def _out_weight(self, dtype):
        """``out_proj.weight`` with its input columns reordered from the reference's d_k-major / head-minor feature order
        (feature dd*H + h) to heads kept whole (feature h*d_k + dd), cached like the projection weights."""
        w = self.out_proj.weight
        build = lambda: w.view(self.d_model, self.d_k, self.heads).transpose(1, 2).reshape(self.d_model, self.d_model).to(dtype).contiguous()
        if torch.is_grad_enabled() and w.requires_grad:
            return build()
        key = ("out", dtype, w.device)
        stamp = (w.data_ptr(), w._version)
        hit = self._packed.get(key)
        if hit is None or hit[0] != stamp:
            hit = (stamp, build())
            self._packed[key] = hit
        return hit[1]

    def _project(self, x, names):
        """Per-head projections ``x W_h + b_h`` for one or several weight sets as ONE GEMM:
        ``[Z*N, D] x [D, S*H*dk]`` (the reference's broadcast ``matmul(x.unsqueeze(1), W.unsqueeze(0))`` materialises
        ``x`` once per head).  Returns a list of ``[Z, H, N, dk]`` views."""
        z, n, d = x.shape
        w2, b2 = self._packed_weights(names, x.dtype)
        y = torch.addmm(b2, x.reshape(z * n, d), w2).view(z, n, len(names), self.heads, self.d_k)
        return [y[:, :, i].permute(0, 2, 1, 3) for i in range(len(names))]

    def forward(self, q, k, v, coords, mask=None, flash=True):
        assert q.shape == k.shape == v.shape and q.dim() == 3 and q.shape[2] == self.d_model
        batch, n, _ = q.shape
        if q is k and k is v:  # self-attention: one fused GEMM for Q, K and V
            Q, K, V = self._project(q, ("q", "k", "v"))
        else:
            (Q,), (K,), (V,) = (self._project(x, (nm,)) for x, nm in ((q, "q"), (k, "k"), (v, "v")))
        form = self.logit_form if self.logit_form is not None else _ga.get_logit_form()
        with spreads_known_positive():  # min_spread + exp(w) > 0: no need to read it back from the device
            if form == "one_plus_rbf":  # no beta, no window in this form: hand it neither
                out = geometric_attn(Q, K, V, coords, self.get_spreads(), None, mask=mask, form=form)
            else:
                out = geometric_attn(Q, K, V, coords, self.get_spreads(), self.get_betas(), mask=mask,
                                     min_rbf=self.min_rbf, max_rbf=self.max_rbf, form=form)  # [Z,H,N,dk]
        # The reference concatenates the heads d_k-major / head-minor (feature dd*H + h) before out_proj.  The same
        # product with the heads kept whole (feature h*d_k + dd) and the columns of the weight reordered to match:
        # the activation view below is free when the kernel wrote O as [Z,N,H,d_k] (inference), the weight is small.
        return F.linear(out.permute(0, 2, 1, 3).reshape(batch, n, self.d_model), self._out_weight(out.dtype))


class Encoder(nn.Module):

    def __init__(self, d_model=512, heads=8, min_spread=2.0, min_rbf=0.001, d_hidden=2048, hidden_layers=0,
                 dropout=0.10, learn_spreads=True, logit_form=None):
        super().__init__()
        self.attn = GeoAttention(d_model=d_model, heads=heads, min_spread=min_spread, min_rbf=min_rbf, learn_spreads=learn_spreads,
                                 logit_form=logit_form)
        self.attn_norm = nn.LayerNorm(d_model)
        self.ffn = MLP(d_in=d_model, d_out=d_model, d_hidden=d_hidden, hidden_layers=hidden_layers, dropout=dropout)
        self.ffn_norm = nn.LayerNorm(d_model)
        self.dropout = nn.Dropout(dropout)

    def _add_norm(self, x, y, norm):
        """``norm(x + dropout(y))``: one fused pass for bf16 inference, the PyTorch operators otherwise."""
        drop_off = not self.training or self.dropout.p == 0.0
        if drop_off and x.shape[-1] % 8 == 0 and x.shape[-1] <= 4096 and fused_ops.usable(x, y, norm.weight, norm.bias):
            return fused_ops.add_layernorm(x, y, norm.weight, norm.bias, norm.eps)
        return norm(x + self.dropout(y))

    def forward(self, q, k, v, coords, coords_beta=None, mask=None):
        q = self._add_norm(q, self.attn(q, k, v, coords, mask=mask), self.attn_norm)
        return self._add_norm(q, self.ffn(q), self.ffn_norm)


class ProteusEncoderModel(nn.Module):
    """Token embedding (vocabulary 33) added to the wavefunction embedding, ``layers`` post-norm encoder
    blocks with geometric attention, a linear head to 20 amino-acid logits (the model of the reference
    README, ``README.md:38,48``, from the modules above)."""

    def __init__(self, d_model=512, heads=8, layers=4, d_hidden=2048, vocab=33, n_out=20, sigma_lo=3.0, sigma_hi=15.0,
                 min_wl=3.7, max_wl=20.0, base_wl=20.0):
        super().__init__()
        self.embed = nn.Embedding(vocab, d_model)
        self.wf_embedding = WaveFunctionEmbedding(d_wf=d_model, min_wl=min_wl, max_wl=max_wl, base_wl=base_wl, anisotropic=False)
        self.encoders = nn.ModuleList(Encoder(d_model=d_model, heads=heads, d_hidden=d_hidden, dropout=0.0) for _ in range(layers))
        self.head = nn.Linear(d_model, n_out)
        # spreads linearly spaced in [sigma_lo, sigma_hi]: spread = min_spread + exp(w)
        sig = torch.linspace(sigma_lo, sigma_hi, heads)
        for enc in self.encoders:
            enc.attn.spread_weights.data = torch.log(sig - enc.attn.min_spread)

    def to_compute_dtype_(self, dtype=torch.bfloat16):
        """Cast the GEMM / LayerNorm weights to ``dtype`` for inference, keeping in fp32 what the kernels read as fp32
        and what loses too much in 8 mantissa bits: the wavenumbers (phases reach hundreds of radians) and the spreads."""
        self.to(dtype)
        self.wf_embedding.float()
        for enc in self.encoders:
            enc.attn.spread_weights.data = enc.attn.spread_weights.data.float()
            enc.attn.beta_weights.data = enc.attn.beta_weights.data.float()
        return self

    def forward(self, tokens, coords, mask=None):
        wf = self.wf_embedding(coords, None, key_padding_mask=mask)  # fp32 [Z,N,d_model]
        x = self.embed(tokens) + wf.to(self.embed.weight.dtype)
        for enc in self.encoders:
            x = enc(x, x, x, coords, mask=mask)
        return self.head(x)
