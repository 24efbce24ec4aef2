"""CPU tests: VAE (causality, shapes, tiling), text / image encoders, the wan_encoder bundle, weight
converter and model-shape detection, and the sampling pipeline end to end on tiny models."""
from argparse import Namespace

import pytest
import torch

from teletron_b200.infer import HunyuanVideoPipeline, WanVideoPipeline
from teletron_b200.models import WanModel, get_encoder, wan_config
from teletron_b200.models.convert import (convert_wan_state_dict, detect_wan_config, from_diffusers,
                                          hash_state_dict_keys)
from teletron_b200.models.encoders import UMT5Encoder, WanImageEncoder, WanVideoVAE, encode_prompt
from teletron_b200.models.encoders.wan_encoder import HashTokenizer
from teletron_b200.models.hunyuan import HunyuanVideoModel, hunyuan_config


def test_vae_shapes_causality_and_tiling():
    torch.manual_seed(0)
    vae = WanVideoVAE(dim=16)
    v = torch.rand(3, 13, 32, 48) * 2 - 1
    z = vae.encode([v])
    assert z.shape == (1, 16, 4, 4, 6)                      # 1 + (13-1)/4 frames, /8 spatially
    z_prefix = vae.encode([v[:, :5]])
    assert torch.allclose(z_prefix, z[:, :, :2], atol=1e-5)  # causal in time: a prefix encodes to a prefix
    rec = vae.decode(z)
    assert rec.shape == (1, 3, 13, 32, 48) and rec.abs().max() <= 1.0
    rec_prefix = vae.decode(z[:, :, :2])
    assert torch.allclose(rec_prefix, rec[:, :, :5], atol=1e-5)
    zt = vae.encode([v], tiled=True, tile_size=(4, 6), tile_stride=(4, 6))   # one tile covers everything
    assert torch.allclose(zt, z, atol=1e-5)
    rt = vae.decode(z, tiled=True, tile_size=(3, 4), tile_stride=(2, 3))
    assert rt.shape == rec.shape and torch.isfinite(rt).all()


def test_text_and_image_encoders():
    torch.manual_seed(0)
    t5 = UMT5Encoder(vocab=500, dim=64, dim_attn=64, dim_ffn=128, num_heads=4, num_layers=2)
    ids = torch.randint(2, 500, (2, 12))
    mask = torch.ones(2, 12, dtype=torch.long)
    mask[0, 7:] = 0
    out = encode_prompt(t5, ids, mask)
    assert out.shape == (2, 12, 64) and out[0, 7:].abs().max() == 0 and out[1].abs().sum() > 0
    # padding must not influence valid positions
    ids2 = ids.clone()
    ids2[0, 7:] = 3
    assert torch.allclose(encode_prompt(t5, ids2, mask)[0, :7], out[0, :7], atol=1e-5)
    # relative position buckets: symmetric offsets land in different halves, far offsets saturate
    pe = t5.blocks[0].pos_embedding
    b = pe._bucket(torch.tensor([[-200, -1, 0, 1, 200]]))
    assert b[0, 2] == 0 and b[0, 0] == 15 and b[0, 4] == 31 and b[0, 1] != b[0, 3]
    clip = WanImageEncoder(dim=64, layers=3, heads=4)
    assert clip.encode_image(torch.rand(2, 3, 50, 70) * 2 - 1).shape == (2, 257, 64)


def test_wan_encoder_bundle_schema():
    for task, n in (("t2v", 4), ("i2v", 4)):
        enc = get_encoder("wan_encoder", device=torch.device("cpu"), small=True, dtype=torch.float32, text_len=16,
                          args=Namespace(task_type=task, consumer_models_num=2))
        enc.setup()
        tensors, hdr = enc.encode(dict(prompts="a red fox runs", images=torch.rand(9, 3, 32, 32) * 2 - 1))
        assert enc.get_output_schema() == ["context", "clip_feature", "image_emb_y", "latents", "noise"]
        ctx, clip, y, lat, noise = tensors
        assert ctx.shape == (1, 16, 64) and lat.shape == (1, 16, 3, 4, 4) and noise.shape == lat.shape
        if task == "i2v":
            assert clip.shape == (1, 257, 64) and y.shape == (1, 20, 3, 4, 4)
            assert y[0, :4, 0].min() == 1 and y[0, :4, 1:].max() == 0
        else:
            assert clip.numel() == 0 and y.numel() == 0


def _to_diffusers_names(sd):
    inv = {}
    for k, v in sd.items():
        n = k
        n = n.replace(".self_attn.q.", ".attn1.to_q.").replace(".self_attn.k.", ".attn1.to_k.")
        n = n.replace(".self_attn.v.", ".attn1.to_v.").replace(".self_attn.o.", ".attn1.to_out.0.")
        n = n.replace(".self_attn.norm_", ".attn1.norm_")
        n = n.replace(".cross_attn.q.", ".attn2.to_q.").replace(".cross_attn.k.", ".attn2.to_k.")
        n = n.replace(".cross_attn.v.", ".attn2.to_v.").replace(".cross_attn.o.", ".attn2.to_out.0.")
        n = n.replace(".cross_attn.norm_", ".attn2.norm_")
        n = n.replace(".ffn.0.", ".ffn.net.0.proj.").replace(".ffn.2.", ".ffn.net.2.")
        n = n.replace(".norm3.", ".norm2.")
        if n.endswith(".modulation") and n.startswith("blocks."):
            n = n.replace(".modulation", ".scale_shift_table")
        n = n.replace("text_embedding.0.", "condition_embedder.text_embedder.linear_1.")
        n = n.replace("text_embedding.2.", "condition_embedder.text_embedder.linear_2.")
        n = n.replace("time_embedding.0.", "condition_embedder.time_embedder.linear_1.")
        n = n.replace("time_embedding.2.", "condition_embedder.time_embedder.linear_2.")
        n = n.replace("time_projection.1.", "condition_embedder.time_proj.")
        n = "scale_shift_table" if n == "head.modulation" else n
        n = n.replace("head.head.", "proj_out.")
        inv[n] = v
    return inv


def test_converter_round_trip_and_detection():
    m = WanModel(wan_config("wan-tiny", dim=256, num_heads=2))
    sd = m.state_dict()
    diff = _to_diffusers_names(sd)
    assert "blocks.0.attn1.to_q.weight" in diff and "condition_embedder.time_proj.bias" in diff
    back, cfg = convert_wan_state_dict(diff)
    assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) for k in sd)
    assert (cfg.dim, cfg.num_heads, cfg.num_layers, cfg.ffn_dim, cfg.in_dim, cfg.has_image_input) == (256, 2, 2, 512, 16, False)
    pref, cfg2 = convert_wan_state_dict({"model.diffusion_model." + k: v for k, v in sd.items()})
    assert set(pref) == set(sd) and cfg2.dim == 256
    assert hash_state_dict_keys(sd) == hash_state_dict_keys(dict(reversed(list(sd.items()))))
    m2 = WanModel(detect_wan_config(sd))
    m2.load_state_dict(back)


def test_pipelines_run_end_to_end():
    torch.manual_seed(0)
    dit = WanModel(wan_config("wan-tiny", in_dim=36, has_image_input=True, text_dim=64)).eval()
    t5 = UMT5Encoder(vocab=512, dim=64, dim_attn=64, dim_ffn=128, num_heads=4, num_layers=1)
    pipe = WanVideoPipeline.from_modules(dit, WanVideoVAE(dim=16), t5, WanImageEncoder(dim=1280, layers=1, heads=16),
                                         HashTokenizer(512, 512), device="cpu", torch_dtype=torch.float32)
    frames = pipe("a cat", negative_prompt="blurry", input_image=torch.rand(3, 64, 64) * 2 - 1, height=70, width=64,
                  num_frames=10, num_inference_steps=2, seed=0, tiled=False, output_type="tensor")
    assert frames.shape == (3, 13, 64, 64)                  # frames rounded to 4k+1, H to a multiple of 16
    again = pipe("a cat", negative_prompt="blurry", input_image=torch.rand(3, 64, 64) * 2 - 1, height=70, width=64,
                 num_frames=10, num_inference_steps=2, seed=0, tiled=False, output_type="latent")
    assert again.shape == (1, 16, 4, 8, 8)
    hy = HunyuanVideoModel(hunyuan_config("hunyuan-tiny", hidden_size=64, num_attention_heads=4,
                                          attention_head_dim=16, rope_axes_dim=(4, 6, 6))).eval()
    hp = HunyuanVideoPipeline(hy, None, device="cpu", torch_dtype=torch.float32)
    lat = hp(torch.randn(1, 8, 64), torch.ones(1, 8, dtype=torch.long), torch.randn(1, 32), height=32, width=32,
             num_frames=5, num_inference_steps=2, seed=1)
    assert lat.shape == (1, 16, 2, 4, 4) and torch.isfinite(lat).all()


def test_model_manager_loads_shards_detects_type_and_merges_lora(tmp_path):
    from teletron_b200.models import WanModel, wan_config
    from teletron_b200.models.model_manager import ModelManager, is_lora_state_dict, merge_lora

    torch.manual_seed(0)
    cfg = wan_config("wan-tiny", dim=256, num_heads=2, ffn_dim=512, text_dim=64, freq_dim=64, num_layers=2)
    src = WanModel(cfg)
    sd = {k: v.detach().clone() for k, v in src.state_dict().items()}
    keys = sorted(sd)
    folder = tmp_path / "dit"
    folder.mkdir()
    torch.save({k: sd[k] for k in keys[: len(keys) // 2]}, folder / "part-00001.pth")       # two shards
    torch.save({"state_dict": {k: sd[k] for k in keys[len(keys) // 2:]}}, folder / "part-00002.pth")
    mm = ModelManager(torch_dtype=torch.float32, device="cpu")
    model = mm.load_model(str(folder))
    assert mm.fetch_model("wan_video_dit") is model and mm.fetch_model("wan_video_vae") is None
    with pytest.raises(KeyError):
        mm.fetch_model("wan_video_vae", require=True)
    got = model.state_dict()
    assert all(torch.equal(got[k], sd[k]) for k in sd)
    assert (model.cfg.dim, model.cfg.num_layers, model.cfg.ffn_dim) == (256, 2, 512)

    # a rank-4 adapter on two projections, PEFT naming with a prefix and kohya naming with alpha
    down1, up1 = torch.randn(4, 256) * 0.1, torch.randn(256, 4) * 0.1
    down2, up2 = torch.randn(4, 256) * 0.1, torch.randn(512, 4) * 0.1
    lora = {"base_model.model.blocks.0.self_attn.q.lora_A.weight": down1,
            "base_model.model.blocks.0.self_attn.q.lora_B.weight": up1,
            "blocks.1.ffn.0.lora_down.weight": down2, "blocks.1.ffn.0.lora_up.weight": up2,
            "blocks.1.ffn.0.alpha": torch.tensor(2.0)}
    assert is_lora_state_dict(lora) and not is_lora_state_dict(sd)
    kind, names = mm.load_lora(state_dict=lora, lora_alpha=0.5)
    assert kind == "wan_video_dit" and sorted(names) == ["blocks.0.self_attn.q.weight", "blocks.1.ffn.0.weight"]
    got = model.state_dict()
    assert torch.allclose(got["blocks.0.self_attn.q.weight"], sd["blocks.0.self_attn.q.weight"] + 0.5 * up1 @ down1,
                          atol=1e-6)
    assert torch.allclose(got["blocks.1.ffn.0.weight"], sd["blocks.1.ffn.0.weight"] + 0.5 * (2.0 / 4) * up2 @ down2,
                          atol=1e-6)
    assert torch.equal(got["blocks.1.self_attn.q.weight"], sd["blocks.1.self_attn.q.weight"])
    with pytest.raises(ValueError):
        merge_lora(model, {"nowhere.lora_A.weight": down1, "nowhere.lora_B.weight": up1})
    with pytest.raises(ValueError):
        mm.load_lora(state_dict=sd)
    assert mm.to("cpu") is mm


def test_convert_cli_writes_a_checkpoint_the_trainer_loads(tmp_path, capsys):
    from teletron_b200.models.convert import main as convert_main
    from teletron_b200.train import Trainer, parse_args

    torch.manual_seed(3)
    cfg = wan_config("wan-tiny")
    src = WanModel(cfg)
    sd = {k: v.detach().clone() for k, v in src.state_dict().items()}
    torch.save({"model.diffusion_model." + k: v for k, v in sd.items()}, tmp_path / "community.pth")
    out = tmp_path / "ckpt"
    assert convert_main(["--input", str(tmp_path / "community.pth"), "--output", str(out), "--dtype", "fp32"]) == 0
    assert f"dim {cfg.dim}, {cfg.num_layers} layers" in capsys.readouterr().out
    assert (out / "latest_checkpointed_iteration.txt").read_text() == "release"
    a = parse_args(argv=("--model ParallelWanModel --model-preset wan-tiny --train-iters 1 --micro-batch-size 1 "
                         f"--synthetic-latents --num-frames 5 --video-resolution 64 64 --pretrained-checkpoint {out}").split())
    a.text_dim, a.text_len = 64, 16
    t = Trainer(a, build_data=False)
    got = t.model.state_dict()
    assert a.iteration == 0 and all(torch.equal(got[k].float(), sd[k]) for k in sd)


def test_generation_example_runs_on_tiny_models(tmp_path):
    import importlib.util
    from pathlib import Path

    from teletron_b200.utils.video_io import read_video_frames

    path = Path(__file__).resolve().parents[1] / "examples" / "wan" / "generate_wan.py"
    spec = importlib.util.spec_from_file_location("generate_wan", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = tmp_path / "smoke.avi"
    assert mod.main(["--tiny", "--device", "cpu", "--height", "64", "--width", "64", "--frames", "9", "--steps", "2",
                     "--out", str(out)]) == 0
    assert read_video_frames(str(out)).shape == (9, 64, 64, 3)
    # image-to-video: the first frame comes from the clip just written
    out2 = tmp_path / "smoke_i2v.avi"
    assert mod.main(["--tiny", "--device", "cpu", "--height", "64", "--width", "64", "--frames", "5", "--steps", "1",
                     "--image", str(out), "--out", str(out2)]) == 0
    assert read_video_frames(str(out2)).shape[0] == 5


def test_hunyuan_pipeline_cfg_and_image_to_video():
    torch.manual_seed(0)
    kw = dict(hidden_size=64, num_attention_heads=4, attention_head_dim=16, rope_axes_dim=(4, 6, 6))
    text, mask, pooled = torch.randn(1, 8, 64), torch.ones(1, 8, dtype=torch.long), torch.randn(1, 32)
    ntext, npooled = torch.randn(1, 8, 64), torch.randn(1, 32)
    hp = HunyuanVideoPipeline(HunyuanVideoModel(hunyuan_config("hunyuan-tiny", **kw)).eval(), None, device="cpu",
                              torch_dtype=torch.float32)
    common = dict(height=32, width=32, num_frames=5, num_inference_steps=2, seed=1)
    base = hp(text, mask, pooled, **common)
    same = hp(text, mask, pooled, negative_prompt_embeds=ntext, negative_prompt_mask=mask,
              negative_pooled_embeds=npooled, cfg_scale=1.0, **common)
    cfg = hp(text, mask, pooled, negative_prompt_embeds=ntext, negative_prompt_mask=mask,
             negative_pooled_embeds=npooled, cfg_scale=4.0, **common)
    assert torch.equal(base, same) and not torch.allclose(base, cfg) and torch.isfinite(cfg).all()
    with pytest.raises(ValueError):
        hp(text, mask, pooled, negative_prompt_embeds=ntext, cfg_scale=2.0, **common)
    # image-to-video: 33 input channels, the first-frame latent changes the sample
    i2v = HunyuanVideoPipeline(HunyuanVideoModel(hunyuan_config("hunyuan-tiny", in_channels=33, **kw)).eval(), None,
                               device="cpu", torch_dtype=torch.float32)
    free = i2v(text, mask, pooled, **common)
    cond = i2v(text, mask, pooled, first_frame_latent=torch.randn(1, 16, 1, 4, 4), **common)
    assert free.shape == cond.shape == (1, 16, 2, 4, 4) and not torch.allclose(free, cond)


def test_step_cache_skips_dit_calls_only_above_zero_threshold():
    from teletron_b200.infer.wan_pipeline import StepCache

    torch.manual_seed(0)
    dit = WanModel(wan_config("wan-tiny", text_dim=64)).eval()
    t5 = UMT5Encoder(vocab=512, dim=64, dim_attn=64, dim_ffn=128, num_heads=4, num_layers=1)
    pipe = WanVideoPipeline.from_modules(dit, WanVideoVAE(dim=16), t5, None, HashTokenizer(512, 512), device="cpu",
                                         torch_dtype=torch.float32)
    calls = []
    dit.register_forward_hook(lambda m, a, o: calls.append(1))
    kw = dict(negative_prompt="blurry", height=64, width=64, num_frames=5, num_inference_steps=6, seed=0,
              tiled=False, output_type="latent")
    plain = pipe("a cat", **kw)
    n_plain = len(calls)
    assert n_plain == 12                                            # 6 steps x 2 guidance branches
    calls.clear()
    exact = pipe("a cat", tea_cache_l1_thresh=0.0, **kw)            # threshold 0: every step computes
    assert len(calls) == 12 and torch.equal(exact, plain)
    calls.clear()
    fast = pipe("a cat", tea_cache_l1_thresh=1e9, **kw)             # huge threshold: only first and last steps compute
    assert len(calls) == 4 and [c.skipped for c in pipe.last_step_caches] == [4, 4]
    assert fast.shape == plain.shape and torch.isfinite(fast).all() and not torch.equal(fast, plain)
    c = StepCache(4, 0.5, coefficients=[2.0, 0.0])                  # rescale d -> 2 d
    m = torch.ones(1, 6, 8)
    assert c.should_skip(m) is False
    c.last_out = torch.zeros(1)
    assert c.should_skip(m * 1.1) is True                           # 2 * 0.1 = 0.2 < 0.5
    assert c.should_skip(m * 1.1 * 1.2) is False                    # + 2 * 0.2 = 0.6 >= 0.5


def test_encoder_checkpoints_load_from_their_published_key_spelling(tmp_path):
    """The CLIP and VAE files store ``visual.*`` / ``encoder.*`` (plus an unused text tower); the modules keep them
    under ``model.``.  Both loaders must rename, and must refuse a file that leaves tensors unset."""
    from teletron_b200.models.model_manager import ModelManager, align_checkpoint_keys

    torch.manual_seed(0)
    clip = WanImageEncoder(dim=64, layers=2, heads=4)
    published = {k[len("model."):]: v.clone() for k, v in clip.state_dict().items()}
    published["textual.embedding.weight"] = torch.zeros(3, 3)
    published["log_scale"] = torch.zeros(())
    fresh = WanImageEncoder(dim=64, layers=2, heads=4)
    aligned = align_checkpoint_keys(fresh, published)
    assert set(aligned) == set(fresh.state_dict()) and not any(k.startswith("model.textual") for k in aligned)
    fresh.load_state_dict(aligned)
    assert all(torch.equal(a, b) for a, b in zip(fresh.state_dict().values(), clip.state_dict().values()))
    # the encoder bundle's loader: same renaming, and a loud error for an incomplete file
    enc = get_encoder("wan_encoder", device="cpu", args=Namespace(task_type="i2v", consumer_models_num=1,
                                                                 encoder_model_path=str(tmp_path),
                                                                 encoder_tokenizer_path=None), small=True)
    vae = WanVideoVAE(dim=16)
    torch.save({k[len("model."):]: v for k, v in vae.state_dict().items() if k.startswith("model.")},
               tmp_path / "Wan2.1_VAE.pth")
    target = WanVideoVAE(dim=16)
    assert enc._load(target, "Wan2.1_VAE.pth")
    assert torch.equal(target.state_dict()["model.encoder.conv1.weight"], vae.state_dict()["model.encoder.conv1.weight"])
    broken = {k: v for k, v in list(published.items())[:5]}
    torch.save(broken, tmp_path / "models_clip_open-clip-xlm-roberta-large-vit-huge-14.pth")
    with pytest.raises(RuntimeError, match="are not in the file"):
        enc._load(WanImageEncoder(dim=64, layers=2, heads=4), "models_clip_open-clip-xlm-roberta-large-vit-huge-14.pth")
    assert not enc._load(target, "absent.pth")


def test_model_manager_loads_a_published_style_vae_file(tmp_path):
    """Full-size VAE built on the meta device, weights from a file with the published key spelling, constants
    re-created: the loaded model encodes exactly like the source."""
    from teletron_b200.models.model_manager import ModelManager

    torch.manual_seed(0)
    vae = WanVideoVAE()
    path = tmp_path / "Wan2.1_VAE.pth"
    torch.save({k[len("model."):]: v for k, v in vae.state_dict().items()}, path)
    mm = ModelManager(torch_dtype=torch.float32, device="cpu")
    loaded = mm.load_model(str(path))
    assert mm.fetch_model("wan_video_vae") is loaded and not any(b.is_meta for b in loaded.buffers())
    x = torch.randn(3, 5, 32, 32)
    assert torch.equal(loaded.encode([x], device="cpu"), vae.encode([x], device="cpu"))


# ------------------------------------------------------------------------------ parity with the reference's encoder files
def _load_reference_module(rel, name, stubs=None):
    """Load one file of the reference by path (its package imports Megatron on import, its files mostly do not)."""
    import importlib.util
    import sys
    import types

    import pytest
    from conftest import reference_file

    path = reference_file(rel)
    if path is None:
        pytest.skip("reference tree not available")
    added = []
    for mod_name, attrs in (stubs or {}).items():
        parts = mod_name.split(".")
        for i in range(1, len(parts) + 1):
            n = ".".join(parts[:i])
            if n not in sys.modules:
                sys.modules[n] = types.ModuleType(n)
                added.append(n)
        for k, v in attrs.items():
            setattr(sys.modules[mod_name], k, v)
    try:
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for n in added:
            sys.modules.pop(n, None)
    return mod


def test_vae_matches_the_reference_file_whole_clip_and_chunked():
    """Same state dict in the reference's VideoVAE_ (which walks the clip in chunks with its per-layer cache) and
    here: encode and decode agree for the whole-clip pass and for the chunked pass, which also agree with each other."""
    from teletron_b200.models.encoders.wan_vae import WanVideoVAE

    ref = _load_reference_module("teletron/models/wan/encoder/wan_video_vae.py", "ref_wan_vae")
    torch.manual_seed(0)
    vae = WanVideoVAE(dim=8).float()
    for p in vae.model.parameters():
        torch.nn.init.normal_(p, std=0.15)
    rv = ref.VideoVAE_(dim=8, z_dim=16).float().eval()
    missing, unexpected = rv.load_state_dict(vae.model.state_dict(), strict=True)
    assert not missing and not unexpected
    x = torch.rand(1, 3, 17, 32, 48) * 2 - 1
    scale = [vae.mean, vae.inv_std]
    with torch.no_grad():
        z_ref = rv.encode(x, scale)
        v_ref = rv.decode(z_ref, scale).clamp_(-1, 1)
    z_whole = vae.encode([x[0]], chunk_frames=0)
    z_chunk = vae.encode([x[0]], chunk_frames=4)
    z_chunk8 = vae.encode([x[0]], chunk_frames=8)
    tol = 1e-5 * max(1.0, float(z_ref.abs().max()))
    assert z_whole.shape == z_ref.shape == (1, 16, 5, 4, 6)
    assert float((z_whole - z_ref).abs().max()) < tol and float((z_chunk - z_ref).abs().max()) < tol
    assert float((z_chunk8 - z_whole).abs().max()) < tol
    v_whole = vae.decode(z_ref, chunk_frames=0)
    v_chunk = vae.decode(z_ref, chunk_frames=1)
    v_chunk2 = vae.decode(z_ref, chunk_frames=2)
    assert v_whole.shape == v_ref.shape == (1, 3, 17, 32, 48)
    assert float((v_whole - v_ref).abs().max()) < 1e-4 and float((v_chunk - v_ref).abs().max()) < 1e-4
    assert float((v_chunk2 - v_whole).abs().max()) < 1e-4
    # long clips switch to chunks by themselves
    assert vae._chunk(81, None, 4) == 4 and vae._chunk(17, None, 4) == 0 and vae._chunk(81, 0, 4) == 0


def test_umt5_encoder_matches_the_reference_file():
    from teletron_b200.models.encoders.umt5 import UMT5Encoder

    ref = _load_reference_module("teletron/models/wan/encoder/wan_video_text_encoder.py", "ref_wan_t5")
    torch.manual_seed(0)
    kw = dict(vocab=200, dim=64, dim_attn=64, dim_ffn=160, num_heads=4, num_layers=3, num_buckets=32, shared_pos=False)
    rm = ref.WanTextEncoder(dropout=0.0, **kw).float().eval()
    m = UMT5Encoder(**kw).float().eval()
    missing, unexpected = m.load_state_dict(rm.state_dict(), strict=True)
    assert not missing and not unexpected
    ids = torch.randint(0, 200, (2, 24))
    mask = torch.ones(2, 24, dtype=torch.long)
    mask[0, 17:] = 0
    mask[1, 9:] = 0
    with torch.no_grad():
        a, b = rm(ids, mask), m(ids, mask)
    assert a.shape == b.shape == (2, 24, 64)
    assert float((a - b).abs().max()) < 1e-4 * max(1.0, float(a.abs().max()))


def test_clip_vision_tower_matches_the_reference_file():
    """The reference's ViT (open-CLIP ViT-H/14 layout: pre-norm, GELU MLP, class token) with the same weights: the
    tokens after the second-to-last block are the i2v conditioning features."""
    import torch.nn.functional as F
    from einops import rearrange

    from teletron_b200.models.encoders.clip_vit import VisionTransformer

    def flash_attention(q, k, v, num_heads, compatibility_mode=False):   # what wan_model.py does in that mode
        q, k, v = (rearrange(t, "b s (n d) -> b n s d", n=num_heads) for t in (q, k, v))
        return rearrange(F.scaled_dot_product_attention(q, k, v), "b n s d -> b s (n d)")

    ref = _load_reference_module("teletron/models/wan/encoder/wan_video_image_encoder.py", "ref_wan_clip",
                                 stubs={"teletron.models.wan.wan_model": {"flash_attention": flash_attention}})
    torch.manual_seed(0)
    rm = ref.VisionTransformer(image_size=56, patch_size=14, dim=64, mlp_ratio=4, out_dim=32, num_heads=4, num_layers=4,
                               pool_type="token", pre_norm=True, post_norm=False, activation="gelu").float().eval()
    m = VisionTransformer(image_size=56, patch=14, dim=64, heads=4, layers=4, mlp_ratio=4, out_dim=32).float().eval()
    missing, unexpected = m.load_state_dict(rm.state_dict(), strict=True)
    assert not missing and not unexpected
    x = torch.randn(2, 3, 56, 56)
    with torch.no_grad():
        a, b = rm(x, use_31_block=True), m(x, use_31_block=True)
    assert a.shape == b.shape == (2, 17, 64)
    assert float((a - b).abs().max()) < 1e-4 * max(1.0, float(a.abs().max()))
