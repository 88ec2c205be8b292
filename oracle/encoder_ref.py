"""CPU oracle for the encoder model (test infrastructure): the arithmetic of ``ProteusEncoderModel`` -- token embedding
plus wavefunction embedding, post-norm encoder layers of geometric attention and a GELU feed-forward block, linear head
(the reference's modules ``old/old_scripts/encoder.py:8-121`` and ``utils/model_utils/base_modules/base_modules.py:6-52``
composed as the reference README describes, ``README.md:38,48``) -- evaluated in fp32 on the CPU with the oracles of
both kernels in place of the kernels.  The per-head projections follow the reference's broadcast matmul
(``encoder.py:106-108``), the head concatenation its d_k-major / head-minor order (``:114-115``)."""
import torch

from oracle.geoattn_ref import geoattn_ref
from oracle.we_ref import wf_embedding_ref


def encoder_forward_ref(model, tokens, coords, mask, act=None):
    """The model's arithmetic in fp32 on the CPU with the oracle in place of both kernels.  ``act`` rounds an
    activation where the GPU path stores one (identity by default; bf16 rounding to follow the bf16 inference path
    operator by operator, so that what is compared is the kernels, not the storage format)."""
    m = model
    act = act or (lambda t: t)
    wn = m.wf_embedding.get_wavenumbers().detach().float().cpu()
    x = act(act(m.embed.weight.detach().float().cpu()[tokens]) + act(wf_embedding_ref(coords, wn, 1, mask)))
    for enc in m.encoders:
        a = enc.attn
        z, n, _ = x.shape
        proj = lambda w, b: torch.matmul(x.unsqueeze(1), w.detach().float().cpu().unsqueeze(0)) + b.detach().float().cpu()[None, :, None, :]
        q, k, v = proj(a.q_proj, a.q_bias), proj(a.k_proj, a.k_bias), proj(a.v_proj, a.v_bias)
        q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))  # the kernel's input rounding
        o = act(geoattn_ref(q, k, v, coords, a.get_spreads().detach().float().cpu(), mask=mask))
        o = act(o.permute(0, 2, 3, 1).reshape(z, n, a.d_model) @ a.out_proj.weight.detach().float().cpu().T)
        ln = lambda mod, t: act(torch.nn.functional.layer_norm(t, (t.shape[-1],), mod.weight.detach().float().cpu(), mod.bias.detach().float().cpu()))
        x = ln(enc.attn_norm, x + o)
        f = enc.ffn
        h = act(torch.nn.functional.gelu(act(x @ f.in_proj.weight.detach().float().cpu().T + f.in_proj.bias.detach().float().cpu())))
        x = ln(enc.ffn_norm, x + act(h @ f.out_proj.weight.detach().float().cpu().T + f.out_proj.bias.detach().float().cpu()))
    return act(x @ m.head.weight.detach().float().cpu().T + m.head.bias.detach().float().cpu())
