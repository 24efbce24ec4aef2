"""Wan2.1 video VAE: causal 3-D convolutional auto-encoder, 16 latent channels, 8x spatial and
4x temporal compression (1 + 4k frames -> 1 + k latent frames).

Architecture and parameter names follow the reference VAE (teletron/models/wan/encoder/
wan_video_vae.py:34-598) so its checkpoints load: ``encoder.conv1``, ``encoder.downsamples.N``
(residual blocks, ``Resample`` with ``resample.1`` / ``time_conv``), ``encoder.middle``, ``encoder.head``,
``conv1`` / ``conv2`` 1x1x1 convolutions, and the mirrored decoder.  Two ways to run it, the same function:
  * one pass over the whole clip (short clips: the 96-channel full-resolution activations of the first stage cost
    about 0.19 GB per 480P frame in bf16);
  * in temporal chunks, as the reference does (wan_video_vae.py:121-173, 215-221, 526-576): the encoder takes the
    first frame, then ``chunk_frames`` (4) frames at a time, the decoder one latent frame at a time, and every
    causal convolution keeps the last frames of its input as the history of the next chunk (``StreamState``), so
    activation memory does not grow with the clip length.
Temporal resampling:
  * down-sampling keeps the first frame and applies the stride-2, kernel-3 ``time_conv`` to the sequence without
    padding (across chunks: the last frame of the previous chunk is the first input of the next);
  * up-sampling keeps the first frame and, for the following frames, applies the causal ``time_conv`` with a zero
    history and interleaves its two channel halves in time.
Latents are normalised with the published per-channel mean / std.  ``tiled`` decoding / encoding
splits H x W into overlapping tiles blended with linear feathering.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

LATENT_MEAN = [-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508,
               0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497, 0.2503, -0.2921]
LATENT_STD = [2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743,
              3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251, 1.9160]


class StreamState(dict):
    """Per-layer history of a clip that is fed chunk by chunk: causal convolutions store the last frames of their
    input here (keyed by the module), resampling layers whether they have seen the first frame."""


_STREAM = None  # the StreamState of the chunked pass in progress (None: whole-clip pass)


class _streaming:
    def __init__(self, state: StreamState):
        self.state = state

    def __enter__(self):
        global _STREAM
        self.prev, _STREAM = _STREAM, self.state
        return self.state

    def __exit__(self, *exc):
        global _STREAM
        _STREAM = self.prev
        return False


class CausalConv3d(nn.Conv3d):
    """Conv3d that pads only the past along time (2 * pad_t frames in front, none behind).  In a chunked pass the
    "past" of a chunk is the tail of the previous chunk's input instead of zeros."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._pad = (self.padding[2], self.padding[2], self.padding[1], self.padding[1], 2 * self.padding[0], 0)
        self.padding = (0, 0, 0)

    def forward(self, x):
        tpad = self._pad[4]
        if _STREAM is None or tpad == 0:
            return super().forward(F.pad(x, self._pad))
        hist = _STREAM.get(self)
        if hist is None:
            hist = x.new_zeros(x.shape[0], x.shape[1], tpad, x.shape[3], x.shape[4])
        xin = torch.cat([hist, x], dim=2)
        _STREAM[self] = xin[:, :, -tpad:].clone()
        return super().forward(F.pad(xin, self._pad[:4] + (0, 0)))


class RMS_norm(nn.Module):
    def __init__(self, dim, channel_first=True, images=True, bias=False):
        super().__init__()
        extra = (1, 1) if images else (1, 1, 1)
        shape = (dim, *extra) if channel_first else (dim,)
        self.channel_first = channel_first
        self.scale = dim ** 0.5
        self.gamma = nn.Parameter(torch.ones(shape))
        self.bias = nn.Parameter(torch.zeros(shape)) if bias else 0.0

    def forward(self, x):
        return F.normalize(x, dim=(1 if self.channel_first else -1)) * self.scale * self.gamma + self.bias


def _per_frame(fn, x):
    b, c, t, h, w = x.shape
    y = fn(x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w))
    return y.reshape(b, t, *y.shape[1:]).permute(0, 2, 1, 3, 4)


class Resample(nn.Module):
    def __init__(self, dim, mode):
        super().__init__()
        assert mode in ("none", "upsample2d", "upsample3d", "downsample2d", "downsample3d")
        self.dim, self.mode = dim, mode
        if mode.startswith("upsample"):
            self.resample = nn.Sequential(nn.Upsample(scale_factor=(2.0, 2.0), mode="nearest-exact"),
                                          nn.Conv2d(dim, dim // 2, 3, padding=1))
            if mode == "upsample3d":
                self.time_conv = CausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0))
        elif mode.startswith("downsample"):
            self.resample = nn.Sequential(nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=(2, 2)))
            if mode == "downsample3d":
                self.time_conv = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0))
        else:
            self.resample = nn.Identity()

    def forward(self, x):
        b, c, t, h, w = x.shape
        st = _STREAM
        first = st is None or ("seen", self) not in st       # this call holds the clip's first frame
        if st is not None:
            st[("seen", self)] = True
        if self.mode == "upsample3d":
            keep = 1 if first else 0                          # the clip's first frame is not doubled
            if t > keep:
                rest = self.time_conv(x[:, :, keep:])         # zero history for the first frame that goes through
                rest = rest.reshape(b, 2, c, t - keep, h, w)
                rest = torch.stack((rest[:, 0], rest[:, 1]), dim=3).reshape(b, c, 2 * (t - keep), h, w)
                x = torch.cat([x[:, :, :keep], rest], dim=2)
        if self.mode != "none":
            x = _per_frame(lambda y: self.resample(y.float()).to(y.dtype) if isinstance(self.resample[0], nn.Upsample)
                           else self.resample(y), x)
        if self.mode == "downsample3d":
            if st is None:
                if x.shape[2] > 1:
                    x = torch.cat([x[:, :, :1], nn.Conv3d.forward(self.time_conv, x)], dim=2)  # no padding, stride 2
            else:
                # the stride-2 windows continue across chunks: the previous chunk's last frame opens this chunk's
                # first window, so a chunk after the first has to bring an even number of frames
                last = x[:, :, -1:].clone()
                if first:
                    if x.shape[2] > 1:
                        assert (x.shape[2] - 1) % 2 == 0, "the first chunk takes 1 + 2k frames"
                        x = torch.cat([x[:, :, :1], nn.Conv3d.forward(self.time_conv, x)], dim=2)
                else:
                    assert x.shape[2] % 2 == 0, "chunks after the first take an even number of frames per stage"
                    x = nn.Conv3d.forward(self.time_conv, torch.cat([st[("last", self)], x], dim=2))
                st[("last", self)] = last
        return x


class ResidualBlock(nn.Module):
    def __init__(self, in_dim, out_dim, dropout=0.0):
        super().__init__()
        self.residual = nn.Sequential(RMS_norm(in_dim, images=False), nn.SiLU(), CausalConv3d(in_dim, out_dim, 3, padding=1),
                                      RMS_norm(out_dim, images=False), nn.SiLU(), nn.Dropout(dropout),
                                      CausalConv3d(out_dim, out_dim, 3, padding=1))
        self.shortcut = CausalConv3d(in_dim, out_dim, 1) if in_dim != out_dim else nn.Identity()

    def forward(self, x):
        return self.residual(x) + self.shortcut(x)


class AttentionBlock(nn.Module):
    """Single-head self-attention over the pixels of each frame."""

    def __init__(self, dim):
        super().__init__()
        self.norm = RMS_norm(dim)
        self.to_qkv = nn.Conv2d(dim, dim * 3, 1)
        self.proj = nn.Conv2d(dim, dim, 1)
        nn.init.zeros_(self.proj.weight)

    def forward(self, x):
        def one(y):
            n, c, h, w = y.shape
            q, k, v = self.to_qkv(self.norm(y)).reshape(n, 1, c * 3, h * w).permute(0, 1, 3, 2).chunk(3, dim=-1)
            o = F.scaled_dot_product_attention(q, k, v)
            return self.proj(o.squeeze(1).permute(0, 2, 1).reshape(n, c, h, w))

        return x + _per_frame(one, x)


class Encoder3d(nn.Module):
    def __init__(self, dim=96, z_dim=32, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_downsample=(False, True, True), dropout=0.0):
        super().__init__()
        dims = [dim * u for u in [1] + list(dim_mult)]
        scale = 1.0
        self.conv1 = CausalConv3d(3, dims[0], 3, padding=1)
        layers = []
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            for _ in range(num_res_blocks):
                layers.append(ResidualBlock(a, b, dropout))
                if scale in attn_scales:
                    layers.append(AttentionBlock(b))
                a = b
            if i != len(dim_mult) - 1:
                layers.append(Resample(b, "downsample3d" if temperal_downsample[i] else "downsample2d"))
                scale /= 2.0
        self.downsamples = nn.Sequential(*layers)
        self.middle = nn.Sequential(ResidualBlock(b, b, dropout), AttentionBlock(b), ResidualBlock(b, b, dropout))
        self.head = nn.Sequential(RMS_norm(b, images=False), nn.SiLU(), CausalConv3d(b, z_dim, 3, padding=1))

    def forward(self, x):
        return self.head(self.middle(self.downsamples(self.conv1(x))))


class Decoder3d(nn.Module):
    def __init__(self, dim=96, z_dim=16, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_upsample=(True, True, False), dropout=0.0):
        super().__init__()
        dims = [dim * u for u in [dim_mult[-1]] + list(dim_mult[::-1])]
        scale = 1.0 / 2 ** (len(dim_mult) - 2)
        self.conv1 = CausalConv3d(z_dim, dims[0], 3, padding=1)
        self.middle = nn.Sequential(ResidualBlock(dims[0], dims[0], dropout), AttentionBlock(dims[0]),
                                    ResidualBlock(dims[0], dims[0], dropout))
        layers = []
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            if i in (1, 2, 3):
                a = a // 2
            for _ in range(num_res_blocks + 1):
                layers.append(ResidualBlock(a, b, dropout))
                if scale in attn_scales:
                    layers.append(AttentionBlock(b))
                a = b
            if i != len(dim_mult) - 1:
                layers.append(Resample(b, "upsample3d" if temperal_upsample[i] else "upsample2d"))
                scale *= 2.0
        self.upsamples = nn.Sequential(*layers)
        self.head = nn.Sequential(RMS_norm(b, images=False), nn.SiLU(), CausalConv3d(b, 3, 3, padding=1))

    def forward(self, z):
        return self.head(self.upsamples(self.middle(self.conv1(z))))


class VideoVAE_(nn.Module):
    def __init__(self, dim=96, z_dim=16, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_downsample=(False, True, True), dropout=0.0):
        super().__init__()
        self.z_dim = z_dim
        self.encoder = Encoder3d(dim, z_dim * 2, dim_mult, num_res_blocks, attn_scales, temperal_downsample, dropout)
        self.conv1 = CausalConv3d(z_dim * 2, z_dim * 2, 1)
        self.conv2 = CausalConv3d(z_dim, z_dim, 1)
        self.decoder = Decoder3d(dim, z_dim, dim_mult, num_res_blocks, attn_scales, temperal_downsample[::-1], dropout)

    def encode(self, x, scale, chunk_frames: int = 0):
        """``chunk_frames`` > 0: the first frame, then that many frames at a time (a multiple of 4), with the
        convolutions' history carried between chunks."""
        if chunk_frames and x.shape[2] > 1:
            assert chunk_frames % 4 == 0 and (x.shape[2] - 1) % 4 == 0, "chunks of 4k frames after the first frame"
            outs = []
            with _streaming(StreamState()):
                outs.append(self.encoder(x[:, :, :1]))
                for t0 in range(1, x.shape[2], chunk_frames):
                    outs.append(self.encoder(x[:, :, t0:t0 + chunk_frames]))
            h = torch.cat(outs, dim=2)
        else:
            h = self.encoder(x)
        mu, _logvar = self.conv1(h).chunk(2, dim=1)
        mean, inv_std = scale
        return (mu - mean.view(1, -1, 1, 1, 1)) * inv_std.view(1, -1, 1, 1, 1)

    def decode(self, z, scale, chunk_frames: int = 0):
        """``chunk_frames`` > 0: that many latent frames at a time (the reference decodes one by one)."""
        mean, inv_std = scale
        z = z / inv_std.view(1, -1, 1, 1, 1) + mean.view(1, -1, 1, 1, 1)
        x = self.conv2(z)
        if chunk_frames and x.shape[2] > 1:
            outs = []
            with _streaming(StreamState()):
                for t0 in range(0, x.shape[2], chunk_frames):
                    outs.append(self.decoder(x[:, :, t0:t0 + chunk_frames]).clamp_(-1, 1))
            return torch.cat(outs, dim=2)
        return self.decoder(x).clamp_(-1, 1)


class WanVideoVAE(nn.Module):
    """encode([C,T,H,W] clips in [-1,1]) -> [16, 1+(T-1)/4, H/8, W/8]; decode is the inverse."""

    upsampling_factor = 8

    def __init__(self, z_dim=16, dim=96):
        super().__init__()
        self.register_buffer("mean", torch.tensor(LATENT_MEAN[:z_dim]), persistent=False)
        self.register_buffer("inv_std", 1.0 / torch.tensor(LATENT_STD[:z_dim]), persistent=False)
        self.model = VideoVAE_(dim=dim, z_dim=z_dim).eval().requires_grad_(False)
        self.z_dim = z_dim

    def reset_constants(self, device=None):
        """(Re)create the latent normalisation constants, e.g. after building the module on the meta device:
        they are not part of any checkpoint."""
        dev = device if device is not None else next(self.model.parameters()).device
        self.mean = torch.tensor(LATENT_MEAN[:self.z_dim], device=dev)
        self.inv_std = 1.0 / torch.tensor(LATENT_STD[:self.z_dim], device=dev)

    def _scale(self, ref):
        return self.mean.to(ref), self.inv_std.to(ref)

    @staticmethod
    def _feather(n, overlap, lead, trail, device):
        w = torch.ones(n, device=device)
        if overlap > 0:
            ramp = (torch.arange(overlap, device=device) + 1) / overlap
            if lead:
                w[:overlap] = ramp
            if trail:
                w[-overlap:] = ramp.flip(0)
        return w

    def _tiled(self, fn, x, tile, stride, out_scale, out_channels):
        """Run ``fn`` on overlapping H x W tiles of x [1,C,T,H,W] and blend with linear feathering."""
        _, _, T, H, W = x.shape
        th, tw = tile
        sh, sw = stride
        probe = None
        acc = wsum = None
        hs = list(range(0, max(H - th, 0) + 1, sh)) or [0]
        ws = list(range(0, max(W - tw, 0) + 1, sw)) or [0]
        if hs[-1] + th < H:
            hs.append(H - th)
        if ws[-1] + tw < W:
            ws.append(W - tw)
        for h0 in hs:
            for w0 in ws:
                out = fn(x[:, :, :, h0:h0 + th, w0:w0 + tw])
                if acc is None:
                    To = out.shape[2]
                    Ho, Wo = int(H * out_scale), int(W * out_scale)
                    acc = torch.zeros(1, out_channels, To, Ho, Wo, device=x.device, dtype=torch.float32)
                    wsum = torch.zeros(1, 1, 1, Ho, Wo, device=x.device, dtype=torch.float32)
                oh, ow = out.shape[3], out.shape[4]
                ov_h, ov_w = int((th - sh) * out_scale), int((tw - sw) * out_scale)
                mh = self._feather(oh, ov_h, h0 > 0, h0 + th < H, x.device)
                mw = self._feather(ow, ov_w, w0 > 0, w0 + tw < W, x.device)
                m = (mh[:, None] * mw[None, :]).view(1, 1, 1, oh, ow)
                y0, x0 = int(h0 * out_scale), int(w0 * out_scale)
                acc[:, :, :, y0:y0 + oh, x0:x0 + ow] += out.float() * m
                wsum[:, :, :, y0:y0 + oh, x0:x0 + ow] += m
        return (acc / wsum.clamp_min(1e-6)).to(x.dtype)

    # frames per chunk: None = decide by clip length (whole clip up to `whole_clip_frames` frames, chunked beyond),
    # 0 = always the whole clip, n = chunks of n frames (encoder; multiple of 4) / n latent frames (decoder)
    whole_clip_frames = 33

    def _chunk(self, frames: int, chunk_frames, default: int) -> int:
        if chunk_frames is None:
            return default if frames > self.whole_clip_frames else 0
        return int(chunk_frames)

    @torch.no_grad()
    def encode(self, videos, device=None, tiled=False, tile_size=(34, 34), tile_stride=(18, 16), chunk_frames=None):
        outs = []
        for v in videos:
            x = v.unsqueeze(0).to(device or v.device)
            scale = self._scale(x)
            ck = self._chunk(x.shape[2], chunk_frames, 4)
            if tiled:
                tile = (tile_size[0] * 8, tile_size[1] * 8)
                stride = (tile_stride[0] * 8, tile_stride[1] * 8)
                z = self._tiled(lambda t: self.model.encode(t, scale, ck), x, tile, stride, 1 / 8, self.z_dim)
            else:
                z = self.model.encode(x, scale, ck)
            outs.append(z.squeeze(0))
        return torch.stack(outs)

    @torch.no_grad()
    def decode(self, latents, device=None, tiled=False, tile_size=(34, 34), tile_stride=(18, 16), chunk_frames=None):
        outs = []
        for z in latents:
            z = z.unsqueeze(0).to(device or z.device)
            scale = self._scale(z)
            ck = self._chunk(4 * (z.shape[2] - 1) + 1, chunk_frames, 1)
            if tiled:
                v = self._tiled(lambda t: self.model.decode(t, scale, ck), z, tile_size, tile_stride, 8, 3)
            else:
                v = self.model.decode(z, scale, ck)
            outs.append(v.squeeze(0))
        return torch.stack(outs)
