"""GeoAttention / Encoder / encoder model on the GPU against the same modules evaluated with the CPU oracles."""
import pytest
import torch

from oracle import chains
from oracle.geoattn_ref import geoattn_ref
from oracle.we_ref import wf_embedding_ref

pytestmark = pytest.mark.gpu


def _reference_forward(model, tokens, coords, mask):
    """The model's arithmetic in fp32 on the CPU with the oracle in place of both kernels."""
    m = model
    wn = m.wf_embedding.get_wavenumbers().detach().float().cpu()
    x = m.embed.weight.detach().float().cpu()[tokens] + wf_embedding_ref(coords, wn, 1, mask)
    for enc in m.encoders:
        a = enc.attn
        z, n, _ = x.shape
        proj = lambda w, b: torch.matmul(x.unsqueeze(1), w.detach().float().cpu().unsqueeze(0)) + b.detach().float().cpu()[None, :, None, :]
        q, k, v = proj(a.q_proj, a.q_bias), proj(a.k_proj, a.k_bias), proj(a.v_proj, a.v_bias)
        q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))  # the kernel's input rounding
        o = geoattn_ref(q, k, v, coords, a.get_spreads().detach().float().cpu(), mask=mask)
        o = o.permute(0, 2, 3, 1).reshape(z, n, a.d_model) @ a.out_proj.weight.detach().float().cpu().T
        ln = lambda mod, t: torch.nn.functional.layer_norm(t, (t.shape[-1],), mod.weight.detach().float().cpu(), mod.bias.detach().float().cpu())
        x = ln(enc.attn_norm, x + o)
        f = enc.ffn
        h = torch.nn.functional.gelu(x @ f.in_proj.weight.detach().float().cpu().T + f.in_proj.bias.detach().float().cpu())
        x = ln(enc.ffn_norm, x + h @ f.out_proj.weight.detach().float().cpu().T + f.out_proj.bias.detach().float().cpu())
    return x @ m.head.weight.detach().float().cpu().T + m.head.bias.detach().float().cpu()


def test_geoattention_module_head_layout_and_grads():
    from proteusai_b200.utils.model_utils.base_modules.encoder import GeoAttention
    torch.manual_seed(0)
    mod = GeoAttention(d_model=128, heads=2).cuda()
    assert set(dict(mod.named_parameters())) == {"spread_weights", "beta_weights", "q_proj", "k_proj", "v_proj", "q_bias", "k_bias",
                                                  "v_bias", "out_proj.weight"}
    c, m = chains.chain_batch([150, 90], 150, seed=2)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    x = torch.randn(2, 150, 128)
    out = mod(x.cuda(), x.cuda(), x.cuda(), c.cuda(), mask=m.cuda())
    proj = lambda w, b: torch.matmul(x.unsqueeze(1), w.detach().cpu().unsqueeze(0)) + b.detach().cpu()[None, :, None, :]
    q, k, v = (proj(getattr(mod, f"{n}_proj"), getattr(mod, f"{n}_bias")).to(torch.bfloat16).float() for n in "qkv")
    ref = geoattn_ref(q, k, v, c, mod.get_spreads().detach().cpu(), mask=m)
    ref = ref.permute(0, 2, 3, 1).reshape(2, 150, 128) @ mod.out_proj.weight.detach().cpu().T
    assert (out.detach().cpu() - ref).abs().max().item() < 2e-2
    out.square().sum().backward()
    for name, prm in mod.named_parameters():
        if name != "beta_weights":
            assert prm.grad is not None and torch.isfinite(prm.grad).all(), name


def test_encoder_model_inference_matches_oracle_composition():
    from proteusai_b200.utils.model_utils.base_modules.encoder import ProteusEncoderModel
    torch.manual_seed(1)
    model = ProteusEncoderModel(d_model=128, heads=2, layers=2, d_hidden=256).cuda().eval()
    lengths = [200, 64, 131]
    c, m = chains.chain_batch(lengths, 200, seed=3)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    tokens = torch.randint(0, 33, (3, 200), generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        logits = model(tokens.cuda(), c.cuda(), m.cuda()).float().cpu()
        ref = _reference_forward(model, tokens, c, m)
    valid = ~m
    assert (logits[valid] - ref[valid]).abs().max().item() < 5e-2
    agree = (logits[valid].argmax(-1) == ref[valid].argmax(-1)).float().mean().item()
    assert agree >= 0.99
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        lb = model(tokens.cuda(), c.cuda(), m.cuda()).float().cpu()
    assert (lb[valid].argmax(-1) == ref[valid].argmax(-1)).float().mean().item() >= 0.9
