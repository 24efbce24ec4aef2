"""Sample a video with the Wan2.1 pipeline: text-to-video, or image-to-video when ``--image`` is given.

    python examples/wan/generate_wan.py --dit <dit file(s)> --text-encoder models_t5_umt5-xxl-enc-bf16.pth \
        --vae Wan2.1_VAE.pth --tokenizer <umt5 tokenizer folder> --prompt "a cat on a skateboard" --out cat.mp4
    python examples/wan/generate_wan.py --tiny --device cpu --out smoke.avi      # random tiny models, plumbing check

Checkpoints go through ``ModelManager`` (type detection, diffusers / community / native naming, sharded files); LoRA
adapter files given with ``--lora`` are folded into the DiT before sampling.
"""
import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

from teletron_b200.infer import WanVideoPipeline  # noqa: E402
from teletron_b200.models.model_manager import ModelManager  # noqa: E402
from teletron_b200.utils.video_io import read_video_frames, save_video  # noqa: E402


def tiny_pipeline(device, dtype, i2v: bool):
    from teletron_b200.models import WanModel, wan_config
    from teletron_b200.models.encoders import UMT5Encoder, WanImageEncoder, WanVideoVAE
    from teletron_b200.models.encoders.wan_encoder import HashTokenizer

    torch.manual_seed(0)
    dit = WanModel(wan_config("wan-tiny", text_dim=64, **(dict(in_dim=36, has_image_input=True) if i2v else {}))).eval()
    t5 = UMT5Encoder(vocab=512, dim=64, dim_attn=64, dim_ffn=128, num_heads=4, num_layers=1)
    clip = WanImageEncoder(dim=1280, layers=1, heads=16) if i2v else None
    return WanVideoPipeline.from_modules(dit.to(device, dtype), WanVideoVAE(dim=16).to(device, dtype), t5.to(device, dtype),
                                         clip.to(device, dtype) if clip is not None else None, HashTokenizer(512, 512),
                                         device=device, torch_dtype=dtype)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dit", nargs="+", default=None)
    ap.add_argument("--text-encoder", default=None)
    ap.add_argument("--image-encoder", default=None)
    ap.add_argument("--vae", default=None)
    ap.add_argument("--tokenizer", default=None, help="Hugging Face tokenizer folder of the umT5 text encoder")
    ap.add_argument("--lora", nargs="*", default=[])
    ap.add_argument("--lora-alpha", type=float, default=1.0)
    ap.add_argument("--prompt", default="a corgi running on a beach at sunset")
    ap.add_argument("--negative-prompt", default="")
    ap.add_argument("--image", default=None, help="first frame (image file or video whose first frame is taken)")
    ap.add_argument("--height", type=int, default=480)
    ap.add_argument("--width", type=int, default=832)
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--cfg-scale", type=float, default=5.0)
    ap.add_argument("--shift", type=float, default=5.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--fps", type=int, default=16)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--offload", action="store_true", help="keep only the running stage's model on the GPU")
    ap.add_argument("--tiny", action="store_true", help="random tiny models instead of checkpoints")
    ap.add_argument("--out", default="sample.mp4")
    a = ap.parse_args(argv)

    dtype = torch.float32 if a.device == "cpu" else torch.bfloat16
    image = None
    if a.image:
        if a.image.lower().endswith((".png", ".jpg", ".jpeg", ".bmp", ".webp")):
            from PIL import Image

            image = Image.open(a.image).convert("RGB")
        else:
            image = read_video_frames(a.image, num_frames=1)[0]
    if a.tiny:
        pipe = tiny_pipeline(a.device, dtype, i2v=image is not None)
    else:
        if not (a.dit and a.text_encoder and a.vae and a.tokenizer):
            ap.error("--dit, --text-encoder, --vae and --tokenizer are required (or --tiny)")
        from teletron_b200.models.encoders.wan_encoder import HFTokenizer

        mm = ModelManager(torch_dtype=dtype, device="cpu" if a.offload else a.device)
        mm.load_model(a.dit if len(a.dit) > 1 else a.dit[0])
        for p in (a.text_encoder, a.vae, a.image_encoder):
            if p:
                mm.load_model(p)
        for p in a.lora:
            kind, names = mm.load_lora(p, lora_alpha=a.lora_alpha, kind="wan_video_dit")
            print(f"merged {len(names)} adapter matrices from {p} into {kind}")
        pipe = WanVideoPipeline.from_model_manager(mm, device=a.device, torch_dtype=dtype,
                                                   tokenizer=HFTokenizer(a.tokenizer, 512))
        if a.offload:
            pipe.enable_cpu_offload()
    frames = pipe(a.prompt, negative_prompt=a.negative_prompt, input_image=image, height=a.height, width=a.width,
                  num_frames=a.frames, cfg_scale=a.cfg_scale, num_inference_steps=a.steps, sigma_shift=a.shift,
                  seed=a.seed, tiled=not a.tiny)
    save_video(frames, a.out, fps=a.fps)
    print(f"wrote {len(frames)} frames to {a.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
