"""``wan_encoder``: the encoder bundle an encoder rank runs for Wan training — umT5 text encoder, CLIP
ViT-H image encoder and the video VAE — turning a raw sample (prompt, video frames, first frame)
into ``[context, clip_feature, image_emb_y, latents(, noise)]`` (teletron/models/wan/encoder/
wan_encoder.py:14-102, wan_encoder_utils.py:22-60,91-144,168-227).

  context       [1, 512, 4096]  prompt embedding, zero past the prompt length
  clip_feature  [1, 257, 1280]  CLIP tokens of the first frame (i2v; empty for t2v)
  image_emb_y   [1, 20, f, h, w] 4-channel first-frame mask + VAE latent of [first frame, zeros...]
  latents       [1, 16, f, h, w] VAE latent of the clip
  noise         same shape as latents, only with several timestep-expert replicas so that all
                replicas of a DP rank see the same noise

Weights are loaded from ``--encoder-model-path`` when it holds the usual files
(``models_t5_umt5-xxl-enc-bf16.pth``, ``models_clip_open-clip-xlm-roberta-large-vit-huge-14.pth``,
``Wan2.1_VAE.pth``); without a path the models are random-initialised at full size (benchmarks,
tests).  Tokenisation uses the HuggingFace tokenizer at ``--encoder-tokenizer-path`` when given,
else a deterministic hashing tokenizer.
"""
from __future__ import annotations

import os
import zlib
from typing import List

import torch

from ...data.base_encoder import BaseEncoder
from ...utils.prompt import apply_clean_mode
from ..registry import ENCODERS
from .clip_vit import WanImageEncoder
from .umt5 import UMT5Encoder, encode_prompt
from .wan_vae import WanVideoVAE

T5_FILE = "models_t5_umt5-xxl-enc-bf16.pth"
CLIP_FILE = "models_clip_open-clip-xlm-roberta-large-vit-huge-14.pth"
VAE_FILE = "Wan2.1_VAE.pth"


class HashTokenizer:
    """Whitespace tokens hashed into the vocabulary; stands in when no tokenizer files exist."""

    def __init__(self, vocab: int, seq_len: int):
        self.vocab, self.seq_len = vocab, seq_len

    def __call__(self, texts: List[str]):
        ids = torch.zeros(len(texts), self.seq_len, dtype=torch.long)
        mask = torch.zeros(len(texts), self.seq_len, dtype=torch.long)
        for i, t in enumerate(texts):
            words = apply_clean_mode(t, "whitespace").split()[: self.seq_len - 1]
            toks = [2 + zlib.crc32(w.encode()) % (self.vocab - 2) for w in words] + [1]
            ids[i, :len(toks)] = torch.tensor(toks)
            mask[i, :len(toks)] = 1
        return ids, mask


class HFTokenizer:
    """Hugging Face tokenizer with the prompter's text cleaning in front (``clean``: None, "whitespace", "lower"
    or "canonicalize"; the Wan prompter uses "whitespace", teletron/models/wan/encoder/wan_prompter.py:38-97)."""

    def __init__(self, path: str, seq_len: int, clean: str = "whitespace"):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path)
        self.seq_len, self.clean = seq_len, clean

    def __call__(self, texts):
        texts = [apply_clean_mode(t, self.clean) for t in ([texts] if isinstance(texts, str) else texts)]
        out = self.tok(texts, return_tensors="pt", padding="max_length", truncation=True, max_length=self.seq_len,
                       add_special_tokens=True)
        return out.input_ids, out.attention_mask


@ENCODERS.register("wan_encoder")
class WanVideoEncoder(BaseEncoder):
    def __init__(self, device=None, args=None, dtype=torch.bfloat16, text_len=512, small: bool = False, **kw):
        super().__init__(device, **kw)
        named = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
                 "fp32": torch.float32, "float32": torch.float32}
        enc_dtype = getattr(args, "encoder_dtype", None)     # --encoder-dtype (teletron/core/distributed/base_encoder.py:25)
        if enc_dtype is not None:
            if enc_dtype not in named:
                raise ValueError(f"unknown --encoder-dtype {enc_dtype!r}")
            dtype = named[enc_dtype]
        self.args, self.dtype, self.text_len, self.small = args, dtype, text_len, small
        self.vae_kw = dict(tiled=bool(getattr(args, "vae_tiled", False)),
                           tile_size=tuple(getattr(args, "vae_tile_size", (34, 34))),
                           tile_stride=tuple(getattr(args, "vae_tile_stride", (18, 16))))
        self.i2v = getattr(args, "task_type", None) == "i2v"
        self.with_noise = getattr(args, "consumer_models_num", 1) > 1
        self.model_path = getattr(args, "encoder_model_path", None)
        self.tokenizer_path = getattr(args, "encoder_tokenizer_path", None)
        self.seq = 0

    def get_output_schema(self):
        return ["context", "clip_feature", "image_emb_y", "latents"] + (["noise"] if self.with_noise else [])

    def _load(self, module, filename):
        if self.model_path and os.path.exists(os.path.join(self.model_path, filename)):
            from ..model_manager import align_checkpoint_keys

            path = os.path.join(self.model_path, filename)
            sd = torch.load(path, map_location="cpu", weights_only=True)
            sd = align_checkpoint_keys(module, sd.get("model_state", sd))
            missing, _ = module.load_state_dict(sd, strict=False)
            missing = [k for k in missing if k.split(".")[-1] not in ("mean", "std", "inv_std")]
            if missing:        # a half-loaded encoder would train the DiT on noise features without any other sign
                raise RuntimeError(f"{path}: {len(missing)} tensors of {type(module).__name__} are not in the file, "
                                   f"e.g. {missing[:3]}")
            return True
        return False

    def setup(self):
        dev = self.device
        if self.small:   # test-sized models with the real structure
            self.t5 = UMT5Encoder(vocab=4096, dim=64, dim_attn=64, dim_ffn=128, num_heads=4, num_layers=2)
            self.clip = WanImageEncoder(dim=64, layers=3, heads=4)
            self.vae = WanVideoVAE(dim=16)
        else:
            with torch.device("meta"):
                t5, clip, vae = UMT5Encoder(), WanImageEncoder(), WanVideoVAE()
            self.t5, self.clip, self.vae = (m.to_empty(device=dev) for m in (t5, clip, vae))
            for m in (self.t5, self.clip, self.vae):
                for p in m.parameters():
                    torch.nn.init.normal_(p, std=0.02)
            self.vae.reset_constants(dev)        # buffers built on the meta device hold no values
            self.clip.reset_constants(dev)
        self._load(self.t5, T5_FILE)
        self._load(self.clip, CLIP_FILE)
        self._load(self.vae, VAE_FILE)
        self.t5 = self.t5.to(device=dev, dtype=self.dtype).eval().requires_grad_(False)
        self.clip = self.clip.to(device=dev, dtype=self.dtype).eval().requires_grad_(False)
        self.vae = self.vae.to(device=dev, dtype=self.dtype).eval().requires_grad_(False)
        vocab = self.t5.token_embedding.num_embeddings
        self.tokenizer = (HFTokenizer(self.tokenizer_path, self.text_len) if self.tokenizer_path
                          else HashTokenizer(vocab, self.text_len))

    @torch.no_grad()
    def encode(self, raw_batch):
        dev, dt = self.device, self.dtype
        prompt = raw_batch["prompts"]
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        ids, mask = self.tokenizer(prompts)
        context = encode_prompt(self.t5, ids.to(dev), mask.to(dev))                      # [B, L, d]
        video = raw_batch["images"]
        if video.dim() == 4:
            video = video.unsqueeze(0)
        video = video.to(dev, dt).clamp(-1, 1).permute(0, 2, 1, 3, 4)                     # [B, 3, T, H, W]
        latents = self.vae.encode(list(video), device=dev, **self.vae_kw)                 # [B, 16, f, h, w]
        B, _, f, h, w = latents.shape
        if self.i2v:
            first = video[:, :, 0]
            clip = self.clip.encode_image(first)
            cond = torch.cat([video[:, :, :1], torch.zeros_like(video[:, :, 1:])], dim=2)
            y = self.vae.encode(list(cond), device=dev, **self.vae_kw)
            msk = torch.zeros(B, 4, f, h, w, device=dev, dtype=dt)
            msk[:, :, 0] = 1
            y = torch.cat([msk, y], dim=1)
        else:
            clip = torch.zeros(B, 0, 1280, device=dev, dtype=dt)
            y = torch.zeros(B, 0, f, h, w, device=dev, dtype=dt)
        tensors = [context.to(dt), clip.to(dt), y.to(dt), latents.to(dt)]
        if self.with_noise:
            tensors.append(torch.randn_like(latents))
        hdr = self._get_tensors_size(tensors, self.seq)
        self.seq += 1
        return tensors, hdr
