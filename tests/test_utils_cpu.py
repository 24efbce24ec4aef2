"""Utility modules on CPU: video reading / writing round trip through whichever backend is installed,
frame sampling, time windows."""
import numpy as np
import pytest
import torch

from teletron_b200.utils import video_io


def _have_writer():
    try:
        import imageio  # noqa: F401
        return True
    except ImportError:
        pass
    try:
        import cv2  # noqa: F401
        return True
    except ImportError:
        return False


def _clip(T=12, H=48, W=64):
    t = np.arange(T, dtype=np.float32)[:, None, None]
    y = np.arange(H, dtype=np.float32)[None, :, None]
    x = np.arange(W, dtype=np.float32)[None, None, :]
    r = (x * 3 + t * 10) % 256
    g = (y * 4 + t * 5) % 256
    b = np.full((T, H, W), 128.0, dtype=np.float32)
    return np.stack([np.broadcast_to(c, (T, H, W)) for c in (r, g, b)], axis=-1).astype(np.uint8)


@pytest.mark.skipif(not _have_writer(), reason="no video writer backend installed")
def test_video_round_trip_sampling_and_time_window(tmp_path):
    clip = _clip()
    path = str(tmp_path / "clip.avi")
    video_io.save_video(list(clip), path, fps=8)
    fr = video_io.read_video_frames(path)
    assert fr.shape == (12, 48, 64, 3) and fr.dtype == torch.uint8
    # lossy codec: compare smooth statistics, frame by frame
    err = (fr.float() - torch.from_numpy(clip).float()).abs().mean().item()
    assert err < 12.0, err
    assert abs(video_io.get_fps(path) - 8.0) < 1e-3
    sub = video_io.read_video_frames(path, num_frames=3, stride=4, start=1)      # frames 1, 5, 9
    assert sub.shape[0] == 3 and torch.equal(sub[1], fr[5])
    picked = video_io.sample_video(path, [0, 7, 3])
    assert picked.shape == (3, 48, 64, 3) and np.array_equal(picked[1], fr[7].numpy())
    assert np.array_equal(video_io.sample_video(fr, [2, 2]), fr[[2, 2]].numpy())
    frames, info = video_io.read_video(path, backend=None, start_sec=0.5, end_sec=1.0)   # frames 4..8 at 8 fps
    assert frames.shape == (5, 3, 48, 64) and abs(info["video_fps"] - 8.0) < 1e-3
    assert torch.equal(frames[0], fr[4].permute(2, 0, 1))
    thwc, _ = video_io.read_video(path, backend=None, output_format="thwc")
    assert thwc.shape == (12, 48, 64, 3)
    pil = video_io.load_video(path)
    assert len(pil) == 12
    x = video_io.frames_to_tensor(fr)
    assert x.shape == (12, 3, 48, 64) and -1.0 <= float(x.min()) and float(x.max()) <= 1.0


def test_video_io_argument_errors(tmp_path):
    with pytest.raises(FileNotFoundError):
        video_io.open_frames(str(tmp_path / "missing.mp4"))
    p = tmp_path / "x.avi"
    p.write_bytes(b"")
    with pytest.raises(ValueError):
        video_io.open_frames(str(p), backend="vlc")
    with pytest.raises(ValueError):
        video_io.read_video(str(p), output_format="CTHW")
    with pytest.raises(ValueError):
        video_io.read_video(str(p), start_sec=2.0, end_sec=1.0)


CAPTIONS = [
    "Visit https://example.com/cat.png NOW!!! @bob  a <person> walks -- “quoted” 192.168.1.1 #12 #123456 1920x1080",
    "this-is-my-cute-cat_video_file.mp4 page 12 click for details... jc6640 6640vc231 free shipping worldwide",
    "一只猫 a cat   sitting &amp; &quot;smiling&quot; ‘single’ — dash",
    "'quoted whole'", "Hello_World, it's (fine) [ok] {yes} | no * star", "  A%20url+encoded caption\\nnext line ",
    "download free wallpaper 1024×768 j2d1a2a3 : spaced ,comma", ".hidden", "-leading dash and trailing:",
]


def test_clean_prompt_matches_the_reference_rules():
    """Same output as the reference's function on a spread of captions (its ``ftfy`` import is stubbed with
    an identity repair, which is also what this package does when ftfy is missing)."""
    import importlib.util
    import sys
    import types

    from conftest import reference_file
    from teletron_b200.utils import prompt as P

    ref_path = reference_file("teletron/utils/prompt.py")
    if ref_path is None:
        pytest.skip("reference tree not available")
    had = "ftfy" in sys.modules
    try:
        import ftfy  # noqa: F401
    except ImportError:
        sys.modules["ftfy"] = types.SimpleNamespace(fix_text=lambda t: t)
    try:
        spec = importlib.util.spec_from_file_location("ref_prompt", ref_path)
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
        for c in CAPTIONS:
            assert P.clean_prompt(c) == ref.clean_prompt(c), c
    finally:
        if not had:
            sys.modules.pop("ftfy", None)
    assert P.clean_prompt("一只猫 cat", keep_cjk=True) == "一只猫 cat" and P.clean_prompt("一只猫 cat") == "cat"


def test_prompt_clean_modes_and_long_prompt_chunks():
    import types

    from teletron_b200.utils import prompt as P

    assert P.canonicalize("Hello_World!! It's <|x|> ok", "<|x|>") == "hello world its <|x|> ok"
    assert P.apply_clean_mode("  A  &amp;amp; B ", "lower") == "a & b"
    assert P.apply_clean_mode("  A   B ", "whitespace") == "A B" and P.apply_clean_mode(" x ", None) == " x "
    with pytest.raises(ValueError):
        P.apply_clean_mode("x", "shout")

    class Tok:                                              # the slice of the HF tokenizer API that is used
        model_max_length = 4

        def __call__(self, text, return_tensors="pt", padding=None, max_length=None, truncation=False):
            ids = [3 + len(w) for w in text.split()]
            if padding == "max_length":
                ids = (ids + [0] * max_length)[:max_length]
            return types.SimpleNamespace(input_ids=torch.tensor([ids]))

    ids = P.tokenize_long_prompt(Tok(), "a bb ccc dddd eeeee ffffff")
    assert ids.shape == (2, 4) and ids.tolist() == [[4, 5, 6, 7], [8, 9, 0, 0]]
    assert Tok.model_max_length == 4


def test_activation_memory_fit_and_max_frames():
    from teletron_b200.utils.flops import fit_activation_memory, max_trainable_frames

    static, per_tok = fit_activation_memory([(1000, 12.0), (3000, 16.0), (2000, 14.0)])
    assert abs(static - 10.0) < 1e-9 and abs(per_tok - 0.002) < 1e-12
    with pytest.raises(ValueError):
        fit_activation_memory([(1000, 12.0)])
    with pytest.raises(ValueError):
        fit_activation_memory([(1000, 12.0), (1000, 13.0)])
    # 64 x 64 video: 16 tokens per latent frame; room = 100 - 8 - 10 = 82 GiB -> 41,000 tokens -> 2,562 latent frames
    assert max_trainable_frames(100.0, 10.0, 0.002, 64, 64) == (2562 - 1) * 4 + 1
    assert max_trainable_frames(100.0, 10.0, 0.002, 64, 64, cp=2) == (5125 - 1) * 4 + 1
    assert max_trainable_frames(15.0, 10.0, 0.002, 64, 64) == 0


def test_megatron_tokenizer_types(tmp_path):
    from argparse import Namespace

    import sentencepiece as spm

    from teletron_b200.utils.tokenizer import build_tokenizer

    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n".join(["a cat sits on the mat", "the dog runs in the park", "video of a sunny beach",
                                 "a person walks the dog on the beach"] * 20))
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(tmp_path / "sp"), vocab_size=60,
                                   model_type="bpe", pad_id=3)
    model = str(tmp_path / "sp.model")
    a = Namespace(tokenizer_type="SentencePieceTokenizer", tokenizer_model=model, vocab_extra_ids=2,
                  make_vocab_size_divisible_by=16, tensor_model_parallel_size=2)
    tok = build_tokenizer(a)
    assert tok.vocab_size == 60 + 4 + 2                        # <CLS> <SEP> <EOD> <MASK> + two sentinels; pad/bos/eos exist
    assert a.padded_vocab_size == 96 and a.padded_vocab_size % 32 == 0
    ids = tok.tokenize("a cat <SEP> the dog <extra_id_1>")
    assert tok.sep in ids and ids[-1] == tok.vocab["<extra_id_1>"]
    assert tok.detokenize(ids) == "a cat <SEP> the dog <extra_id_1>"
    assert len({tok.cls, tok.sep, tok.eod, tok.mask, tok.pad, tok.bos, tok.eos}) == 7
    gpt = build_tokenizer(Namespace(tokenizer_type="GPTSentencePieceTokenizer", tokenizer_model=model))
    assert gpt.vocab_size == 60 and gpt.eod == gpt.eos and gpt.detokenize(gpt.tokenize("the park")) == "the park"
    ll = build_tokenizer(Namespace(tokenizer_type="Llama2Tokenizer", tokenizer_model=model))
    plain = ll.tokenize("a cat", bos=False)
    assert ll.tokenize("a cat") == [ll.bos] + plain and ll.tokenize("a cat", bos=False, eos=True) == plain + [ll.eos]

    vocab = tmp_path / "vocab.txt"
    vocab.write_text("\n".join(["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "the", "cat", "sat", "##s", "dog"]))
    bert = build_tokenizer(Namespace(tokenizer_type="BertWordPieceLowerCase", vocab_file=str(vocab),
                                     make_vocab_size_divisible_by=8))
    assert bert.tokenize("The cats sat") == [5, 6, 8, 7] and (bert.cls, bert.sep, bert.pad, bert.mask) == (2, 3, 0, 4)
    assert bert.eod == 3 and bert.vocab_size == 10

    null = build_tokenizer(Namespace(tokenizer_type="NullTokenizer", vocab_size=100))
    assert null.tokenize("3 14 15") == [3, 14, 15] and null.eod == 100
    with pytest.raises(NotImplementedError):
        build_tokenizer(Namespace(tokenizer_type="Klingon"))


def test_planner_reproduces_the_measured_configurations(capsys):
    from teletron_b200.models import wan_config
    from teletron_b200.utils.flops import activation_gib_per_token, plan
    from teletron_b200.utils.plan import main as plan_main

    # the calibration point: Wan2.1-1.3B, full recompute, 197 KiB per token
    assert abs(activation_gib_per_token(1536, 30, True) * 2 ** 20 - 197.5) < 3.0
    r = plan(wan_config("wan2.1-1.3b-t2v"), 1.42e9, 720, 1280, 161, tflops_per_gpu=1000.0)
    assert r["tokens"] == 147_600 and abs(r["static_gib"] + r["activation_gib"] - 51.7) < 2.0   # measured 51.73 GiB
    assert r["fits"] and 800 < r["max_frames"] < 900 and 17.0 < r["seconds_per_sample"] < 23.0  # measured 21.9 s
    big = plan(wan_config("wan2.1-14b-i2v"), 16.4e9, 720, 1280, 81, gpus=8, cp=8)
    assert big["fits"] and 3.5 < big["seconds_per_sample"] < 5.0                                 # measured 4.36 s
    assert not plan(wan_config("wan2.1-14b-i2v"), 16.4e9, 720, 1280, 81, gpus=1)["fits"]
    assert plan_main(["--model", "wan-tiny", "--height", "64", "--width", "64", "--frames", "5"]) == 0
    assert "tokens per sample" in capsys.readouterr().out


@pytest.mark.skipif(not _have_writer(), reason="no video writer backend installed")
def test_video_folder_dataset_feeds_the_encoders(tmp_path):
    import json

    from teletron_b200.data import build_dataset
    from teletron_b200.data.synthetic_encoder import SyntheticWanEncoder
    from teletron_b200.data.video_folder import resize_center_crop

    root = tmp_path / "data"
    (root / "clips").mkdir(parents=True)
    video_io.save_video(list(_clip(T=12, H=48, W=64)), str(root / "clips" / "a.avi"), fps=8)
    video_io.save_video(list(_clip(T=3, H=40, W=40)), str(root / "clips" / "b.avi"), fps=8)        # shorter than asked
    with open(root / "metadata.jsonl", "w") as f:
        f.write(json.dumps({"video": "clips/a.avi", "caption": "A CAT  @bob on   a mat"}) + "\n")
        f.write(json.dumps({"video": "clips/b.avi", "caption": "dog"}) + "\n")
    ds = build_dataset("VideoFolderDataset", data_path=[str(root)], num_frames=5, height=32, width=32, frame_stride=2)
    assert len(ds) == 2
    it = ds[0]
    assert it["images"].shape == (5, 3, 32, 32) and it["raw_first_image"].shape == (3, 32, 32) and it["index"] == 0
    assert -1.0 <= float(it["images"].min()) and float(it["images"].max()) <= 1.0
    assert it["prompts"] == "a cat on a mat"
    short = ds[1]
    assert short["images"].shape == (5, 3, 32, 32) and torch.equal(short["images"][3], short["images"][4])
    x = resize_center_crop(torch.zeros(2, 3, 48, 64), 32, 32)
    assert x.shape == (2, 3, 32, 32)
    enc = SyntheticWanEncoder(device="cpu", text_len=8, text_dim=16)
    tensors, _ = enc.encode(it)
    assert tensors[3].shape == (1, 16, 2, 4, 4)                                    # latents of a 5 x 32 x 32 clip
    # captions from sidecar files when there is no metadata file
    side = tmp_path / "side"
    side.mkdir()
    video_io.save_video(list(_clip(T=5, H=32, W=32)), str(side / "c.avi"), fps=8)
    (side / "c.txt").write_text("a red car\n")
    ds2 = build_dataset("VideoFolderDataset", data_path=str(side), num_frames=5, height=32, width=32)
    assert ds2[0]["prompts"] == "a red car"
    with pytest.raises(ValueError):
        build_dataset("VideoFolderDataset", data_path=None)


def test_registry_surface():
    from teletron_b200.data import build_dataset
    from teletron_b200.models.registry import MODELS, Registry

    reg = Registry("thing")

    @reg.register("named")
    class A:
        def __init__(self, x=1, y=2):
            self.x, self.y = x, y

    @reg.register
    class B(A):
        pass

    reg.register_module(A, "alias")
    assert len(reg) == 3 and "B" in reg and reg.get_module("alias") is A and set(reg.list_modules()) == {"named", "B", "alias"}
    assert reg.build("named", 5).x == 5
    obj = reg.build({"type": "B", "x": 7, "y": 8}, y=9)
    assert isinstance(obj, B) and (obj.x, obj.y) == (7, 9)
    with pytest.raises(KeyError):
        reg.register_module(B, "named")                       # a different class under a taken name
    with pytest.raises(KeyError):
        reg.build({"x": 1})
    reg.unregister("alias")
    assert "alias" not in reg and "thing" in repr(reg)
    with pytest.raises(KeyError):
        reg.unregister("alias")
    assert "ParallelWanModel" in MODELS and "ParallelHunyuanVideoModel" in MODELS
    ds = build_dataset({"type": "FakeDataset", "num_frames": 5, "height": 16, "width": 16, "length": 3})
    assert len(ds) == 3 and ds[0]["images"].shape == (5, 3, 16, 16)


def test_config_dictionary(tmp_path):
    from teletron_b200.utils.config import Config, load_config

    c = Config(model=dict(dim=128, patch=(1, 2, 2), blocks=[dict(kind="dual"), dict(kind="single")]), lr=1e-4)
    assert c.model.dim == 128 and c.model.blocks[1].kind == "single" and c.model.patch == (1, 2, 2)
    c.update(model=dict(dim=256), seed=3)
    assert c.model.dim == 256 and c.model.patch == (1, 2, 2) and c.seed == 3        # nested merge keeps siblings
    c.update(model={"__force__": True, "dim": 64})
    assert c.model.to_dict() == {"dim": 64}                                             # forced replacement
    assert c.setdefault("lr", 5.0) == 1e-4 and c.setdefault("wd", 0.1) == 0.1 and c.wd == 0.1
    d = c.copy()
    d.model.dim = 1
    assert c.model.dim == 64
    with pytest.raises(AttributeError):
        c.missing
    del c.wd
    assert "wd" not in c and "Config:" in str(c)
    c.sizes = (3, (4, 5))
    for name in ("cfg.json", "cfg.yaml", "cfg.pkl"):
        path = tmp_path / "sub" / name
        c.save(str(path))
        back = Config.load(str(path))
        assert back.to_dict() == c.to_dict() and back.sizes == (3, (4, 5)), name
    (tmp_path / "folder").mkdir()
    c.save(str(tmp_path / "folder" / "config.json"))
    assert load_config(str(tmp_path / "folder")).lr == 1e-4 and load_config({"a": {"b": 1}}).a.b == 1
    assert load_config(c) is c
    extra = tmp_path / "extra.yaml"
    extra.write_text("model:\n  dim: 512\nnew: yes\n")
    c.merge_from_file(str(extra))
    assert c.model.dim == 512 and c.new is True
    with pytest.raises(ValueError):
        Config.load(str(tmp_path / "conf.py"))


def test_status_word_values_are_described():
    from teletron_b200.ops._lib import describe_status

    assert describe_status(0) == "ok"
    assert describe_status(0x503) == "a peer barrier waiting for rank 3 ran out of its time budget"
    assert "MMA-issuing warp" in describe_status(0x202) and "wait #2" in describe_status(0x202)
    assert "misaligned" in describe_status(0x600) and describe_status(0x7ff).startswith("unknown status")


def test_epilogue_staging_swizzle_is_a_conflict_free_bijection():
    """Index arithmetic of ``stage_put`` / ``stage_flush`` (csrc/tt_common.cuh), restated on the host: a warp parks
    32 rows of CH 16-byte chunks (row = lane) and reads them back with CH lanes per row.  Every (row, chunk) must land
    in a slot of its own, the reader must find what the writer put there, and neither side may have two lanes of a
    quarter warp (the unit in which 16-byte shared-memory accesses are served) in the same 16-byte bank group."""
    for CH in (8, 16):
        put = lambda lane, chunk: lane * CH * 16 + ((chunk ^ (lane & (CH - 1))) << 4)
        slots = {put(l, c) for l in range(32) for c in range(CH)}
        assert len(slots) == 32 * CH and max(slots) == 32 * CH * 16 - 16
        # writer: one instruction = 32 lanes, same chunk index; served quarter warp by quarter warp
        for c in range(CH):
            for q in range(4):
                banks = {(put(l, c) % 128) // 16 for l in range(q * 8, q * 8 + 8)}
                assert len(banks) == 8
        # reader: lane -> (row = i * (32 // CH) + lane // CH, chunk = lane % CH); it reads the slot of (row, chunk)
        rpi = 32 // CH
        seen = set()
        for i in range(32 // rpi):
            addr = []
            for lane in range(32):
                row, chunk = i * rpi + lane // CH, lane % CH
                addr.append(row * CH * 16 + ((chunk ^ (row & (CH - 1))) << 4))
                assert addr[-1] == put(row, chunk)
                seen.add((row, chunk))
            for q in range(4):
                assert len({(a % 128) // 16 for a in addr[q * 8:q * 8 + 8]}) == 8
        assert len(seen) == 32 * CH
