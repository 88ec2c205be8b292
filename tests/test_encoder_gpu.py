"""GeoAttention / Encoder / encoder model on the GPU against the same modules evaluated with the CPU oracles."""
import pytest
import torch

from oracle import chains
from oracle.encoder_ref import encoder_forward_ref as _reference_forward
from oracle.geoattn_ref import geoattn_ref

pytestmark = pytest.mark.gpu


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


def test_encoder_model_bf16_inference_uses_fused_ops_and_matches_oracle_composition():
    """The bf16 inference configuration: strided Q/K/V straight from the fused projection, O written head-major,
    LayerNorm(x + y) and GELU as fused kernels.  Compared with the fp32 oracle composition of the same weights."""
    from proteusai_b200.utils.model_utils.base_modules.encoder import ProteusEncoderModel
    torch.manual_seed(5)
    model = ProteusEncoderModel(d_model=128, heads=2, layers=2, d_hidden=256).cuda().eval()
    lengths = [200, 64, 131]
    c, m = chains.chain_batch(lengths, 200, seed=6)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    tokens = torch.randint(0, 33, (3, 200), generator=torch.Generator().manual_seed(7))
    with torch.no_grad():
        ref = _reference_forward(model, tokens, c, m)
        model.to_compute_dtype_(torch.bfloat16)
        logits = model(tokens.cuda(), c.cuda(), m.cuda()).float().cpu()
    valid = ~m
    err = (logits[valid] - ref[valid]).abs().max().item()
    agree = (logits[valid].argmax(-1) == ref[valid].argmax(-1)).float().mean().item()
    assert err < 1e-1 and agree >= 0.95, (err, agree)


def test_config5_shape_bf16_matches_oracle_composition():
    """The encoder at the configuration the benchmark times: d_model 512, 8 heads, 4 layers, FFN 2048, bf16, chains padded
    to N = 1024 (five chains with lengths from 64 to 1024 keep the CPU oracle to seconds).  The oracle composes the CPU
    restatements of both kernels with fp32 arithmetic on the bf16 weights, rounding activations to bf16 where the GPU
    path stores them.  Bar: logits within 5e-2, and the same arg-max on at least 99 % of the valid tokens whose oracle top-2 gap
    is wider than that tolerance can close (0.1), 98 % over all valid tokens."""
    from proteusai_b200.utils.model_utils.base_modules.encoder import ProteusEncoderModel
    torch.manual_seed(1005)
    model = ProteusEncoderModel(d_model=512, heads=8, layers=4, d_hidden=2048).cuda().eval().to_compute_dtype_(torch.bfloat16)
    lengths = [1024, 700, 333, 129, 64]
    n = 1024
    c, m = chains.chain_batch(lengths, n, seed=1005)
    c, m = torch.from_numpy(c), torch.from_numpy(m)
    tokens = torch.randint(0, 33, (len(lengths), n), generator=torch.Generator().manual_seed(1005))
    with torch.no_grad():
        logits = model(tokens.cuda(), c.cuda(), m.cuda()).float().cpu()
        ref = _reference_forward(model, tokens, c, m, act=lambda t: t.to(torch.bfloat16).float())
    from proteusai_b200 import _lib
    _lib.device_status()
    valid = ~m
    lg, rf = logits[valid], ref[valid]
    err = (lg - rf).abs().max().item()
    same = lg.argmax(-1) == rf.argmax(-1)
    top2 = rf.topk(2, dim=-1).values
    gap = top2[:, 0] - top2[:, 1]                      # how decided the oracle's own arg-max is
    decided = gap > 2 * 5e-2                           # two logits each within the 5e-2 bar cannot swap across a larger gap
    agree, agree_decided = same.float().mean().item(), same[decided].float().mean().item()
    print(f"config-5 shape: logits max-abs {err:.3e}, arg-max agreement {agree:.4f} on {int(valid.sum())} tokens, "
          f"{agree_decided:.4f} on the {int(decided.sum())} whose top-2 gap exceeds 0.1")
    # 99 % of the tokens wherever the oracle's decision is wider than the logit tolerance allows to flip (all of them, in
    # fact); over all tokens, near-ties included, random-init logits leave about 1 % undecided at bf16 precision
    assert err < 5e-2 and agree_decided >= 0.99 and agree >= 0.98, (err, agree, agree_decided)


@pytest.mark.parametrize("d", [8, 128, 512, 520, 1024, 4096])
def test_add_layernorm_kernel(d):
    from proteusai_b200.utils.model_utils.base_modules import fused_ops
    g = torch.Generator().manual_seed(d)
    rows = 37
    x = torch.randn(rows, d, generator=g).to(torch.bfloat16)
    y = (3 * torch.randn(rows, d, generator=g) + 1).to(torch.bfloat16)
    w = torch.randn(d, generator=g)
    b = torch.randn(d, generator=g)
    ref = torch.nn.functional.layer_norm(x.float() + y.float(), (d,), w, b, 1e-5)
    out = fused_ops.add_layernorm(x.cuda(), y.cuda(), w.cuda(), b.cuda(), 1e-5)
    assert out.dtype == torch.bfloat16
    assert (out.float().cpu() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()
    wb, bb = w.to(torch.bfloat16), b.to(torch.bfloat16)
    ref = torch.nn.functional.layer_norm(x.float(), (d,), wb.float(), bb.float(), 1e-5)
    out = fused_ops.add_layernorm(x.cuda(), None, wb.cuda(), bb.cuda(), 1e-5)
    assert (out.float().cpu() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()


def test_gelu_kernel():
    from proteusai_b200.utils.model_utils.base_modules import fused_ops
    x = torch.cat([torch.linspace(-12, 12, 4001), torch.randn(4096 - 4001 + 8 * 100, generator=torch.Generator().manual_seed(0))])
    x = x[: (x.numel() // 8) * 8].to(torch.bfloat16)
    ref = torch.nn.functional.gelu(x.double())
    out = fused_ops.gelu(x.cuda()).float().cpu().double()
    assert ((out - ref).abs() <= 2 ** -8 * ref.abs() + 1e-7).all()
    y = x.cuda().clone()
    assert fused_ops.gelu(y, inplace=True).data_ptr() == y.data_ptr()
    assert torch.equal(y.float().cpu().double(), out)
