"""Wan2.1 video VAE: causal 3-D convolutional auto-encoder, 16 latent channels, 8x spatial and
4x temporal compression (1 + 4k frames -> 1 + k latent frames).

Architecture and parameter names follow the reference VAE (teletron/models/wan/encoder/
wan_video_vae.py:34-598) so its checkpoints load: ``encoder.conv1``, ``encoder.downsamples.N``
(residual blocks, ``Resample`` with ``resample.1`` / ``time_conv``), ``encoder.middle``, ``encoder.head``,
``conv1`` / ``conv2`` 1x1x1 convolutions, and the mirrored decoder.  The reference walks the clip in
temporal chunks with a per-layer feature cache to save memory; with causal convolutions that is the
same function as one pass over the whole clip, which is what this implementation does (180 GB
of HBM make the cache unnecessary):
  * temporal down-sampling keeps the first frame and applies the stride-2, kernel-3 ``time_conv``
    to the whole sequence without padding;
  * temporal up-sampling keeps the first frame and, for the following frames, applies the causal
    ``time_conv`` with a zero history and interleaves its two channel halves in time.
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


class CausalConv3d(nn.Conv3d):
    """Conv3d that pads only the past along time (2 * pad_t frames in front, none behind)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._pad = (self.padding[2], self.padding[2], self.padding[1], self.padding[1], 2 * self.padding[0], 0)
        self.padding = (0, 0, 0)

    def forward(self, x):
        return super().forward(F.pad(x, self._pad))


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
        if self.mode == "upsample3d" and t > 1:
            rest = self.time_conv(x[:, :, 1:])                      # zero history for the frames after the first
            rest = rest.reshape(b, 2, c, t - 1, h, w)
            rest = torch.stack((rest[:, 0], rest[:, 1]), dim=3).reshape(b, c, 2 * (t - 1), h, w)
            x = torch.cat([x[:, :, :1], rest], dim=2)
        if self.mode != "none":
            x = _per_frame(lambda y: self.resample(y.float()).to(y.dtype) if isinstance(self.resample[0], nn.Upsample)
                           else self.resample(y), x)
        if self.mode == "downsample3d" and x.shape[2] > 1:
            x = torch.cat([x[:, :, :1], nn.Conv3d.forward(self.time_conv, x)], dim=2)  # no padding, stride 2
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

    def encode(self, x, scale):
        mu, _logvar = self.conv1(self.encoder(x)).chunk(2, dim=1)
        mean, inv_std = scale
        return (mu - mean.view(1, -1, 1, 1, 1)) * inv_std.view(1, -1, 1, 1, 1)

    def decode(self, z, scale):
        mean, inv_std = scale
        z = z / inv_std.view(1, -1, 1, 1, 1) + mean.view(1, -1, 1, 1, 1)
        return self.decoder(self.conv2(z)).clamp_(-1, 1)


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

    @torch.no_grad()
    def encode(self, videos, device=None, tiled=False, tile_size=(34, 34), tile_stride=(18, 16)):
        outs = []
        for v in videos:
            x = v.unsqueeze(0).to(device or v.device)
            scale = self._scale(x)
            if tiled:
                tile = (tile_size[0] * 8, tile_size[1] * 8)
                stride = (tile_stride[0] * 8, tile_stride[1] * 8)
                z = self._tiled(lambda t: self.model.encode(t, scale), x, tile, stride, 1 / 8, self.z_dim)
            else:
                z = self.model.encode(x, scale)
            outs.append(z.squeeze(0))
        return torch.stack(outs)

    @torch.no_grad()
    def decode(self, latents, device=None, tiled=False, tile_size=(34, 34), tile_stride=(18, 16)):
        outs = []
        for z in latents:
            z = z.unsqueeze(0).to(device or z.device)
            scale = self._scale(z)
            if tiled:
                v = self._tiled(lambda t: self.model.decode(t, scale), z, tile_size, tile_stride, 8, 3)
            else:
                v = self.model.decode(z, scale)
            outs.append(v.squeeze(0))
        return torch.stack(outs)
