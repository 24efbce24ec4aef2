"""Wan DiT on CPU (fp32): parity with the reference's serial model, state-dict round trip."""
import importlib.util
from types import SimpleNamespace

import pytest
import torch

from conftest import reference_file
from teletron_b200.models import WanModel, wan_config


def _load_reference_wan():
    path = reference_file("teletron/models/wan/wan_model.py")
    if path is None:
        pytest.skip("reference tree not available")
    spec = importlib.util.spec_from_file_location("ref_wan_model", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.FLASH_ATTN_3_AVAILABLE = mod.FLASH_ATTN_2_AVAILABLE = mod.SAGE_ATTN_AVAILABLE = False
    return mod


def _inputs(i2v=False):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 16, 3, 16, 16, generator=g)
    ctx = torch.randn(1, 512 if i2v else 32, 64, generator=g)
    t = torch.tensor([412.0])
    kw = {}
    if i2v:
        kw = dict(clip_feature=torch.randn(1, 257, 1280, generator=g), y=torch.randn(1, 20, 3, 16, 16, generator=g))
    return x, t, ctx, kw


@pytest.mark.parametrize("i2v", [False, True])
def test_matches_reference_forward_and_grads(i2v):
    ref = _load_reference_wan()
    P = ref.WanParams
    P.in_channels, P.ffn_dim, P.text_dim, P.freq_dim = (36 if i2v else 16), 512, 64, 64
    P.has_image_input = i2v
    torch.manual_seed(1)
    rm = ref.WanModel(SimpleNamespace(hidden_size=128, num_attention_heads=4, num_layers=2)).float()
    cfg = wan_config("wan-tiny", in_dim=36 if i2v else 16, has_image_input=i2v)
    m = WanModel(cfg)
    missing, unexpected = m.load_state_dict(rm.state_dict(), strict=True)
    assert not missing and not unexpected
    x, t, ctx, kw = _inputs(i2v)
    out_ref = rm(x, t, ctx, **kw)
    out = m(x, t, ctx, **kw)
    assert out.shape == out_ref.shape
    assert (out - out_ref).abs().max().item() < 2e-4 * max(1.0, out_ref.abs().max().item())
    out_ref.square().mean().backward()
    out.square().mean().backward()
    ref_grads = dict(rm.named_parameters())
    sd_grads = {}
    for n, p in m.named_parameters():
        sd_grads[n] = p.grad
    # fused projections: compare slice by slice
    for n, p in ref_grads.items():
        if n in sd_grads:
            g = sd_grads[n]
        else:
            base, leaf, kind = n.rsplit(".", 2)
            fused = {"q": ("qkv", 0), "k": ("qkv", 1), "v": ("qkv", 2)} if base.endswith("self_attn") else \
                {"k": ("kv", 0), "v": ("kv", 1), "k_img": ("kv_img", 0), "v_img": ("kv_img", 1)}
            attr, idx = fused[leaf]
            full = sd_grads[f"{base}.{attr}.{kind}"]
            g = full[idx * 128:(idx + 1) * 128]
        assert p.grad is not None and g is not None, n
        denom = p.grad.norm() + g.norm() + 1e-12
        assert (0.5 * (p.grad - g).norm() / denom).item() < 1e-4, n


def test_state_dict_round_trip_has_reference_keys():
    m = WanModel(wan_config("wan-tiny"))
    sd = m.state_dict()
    for k in ("blocks.0.self_attn.q.weight", "blocks.1.cross_attn.v.bias", "blocks.0.modulation",
              "head.head.weight", "head.modulation", "patch_embedding.weight", "time_projection.1.weight",
              "blocks.0.norm3.weight", "blocks.0.ffn.2.bias", "text_embedding.0.weight"):
        assert k in sd, k
    assert not any("qkv" in k or ".kv." in k for k in sd)
    m2 = WanModel(wan_config("wan-tiny"))
    m2.load_state_dict(sd)
    for (n1, p1), (n2, p2) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(p1, p2), n1
