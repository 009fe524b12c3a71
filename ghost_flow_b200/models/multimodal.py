"""CLIP, diffusion (DDPM + UNet) and NeRF.

* CLIP (ghostflow-nn/src/clip.rs:17-678): ``CLIPConfig.vit_b_32 / vit_b_16 / vit_l_14``, vision and text towers,
  ``encode_image / encode_text / forward / zero_shot_classify / image_to_text_retrieval / text_to_image_retrieval``;
  logits = cosine similarity * exp(logit_scale), logit_scale initialised to ln(1/0.07) (clip.rs:520-546).
* Diffusion (ghostflow-nn/src/diffusion.rs:18-527): ``DiffusionConfig.stable_diffusion / ddpm / tiny``,
  ``BetaSchedule``, ``NoiseScheduler.add_noise / predict_x0``, ``ResidualBlock``, ``UNet``, ``DDPM.forward / sample``.
* NeRF (ghostflow-nn/src/nerf.rs:16-594): ``NeRFConfig.default / tiny / large``, ``PositionalEncoder``, ``NeRFMLP``,
  ``RaySampler``, ``VolumeRenderer.render_rays``, ``NeRF.render``. Positional encoding and the volume-rendering
  compositor run as CUDA kernels on GPU tensors (``ops.render``), with the PyTorch formulas below as the CPU
  path and test oracle. The fine pass samples from the coarse weights (the reference re-uses uniform samples,
  nerf.rs:462-469).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from ..nn.conv import Conv2d
from ..nn.layers import Embedding, GroupNorm, LayerNorm, Linear
from ..nn.module import Module, ModuleList, Parameter
from ..nn.transformer import TransformerEncoderLayer


# =========================================================================== CLIP
@dataclass
class CLIPVisionConfig:
    """Vision tower parameters (ghostflow-nn/src/clip.rs:28-44)."""
    image_size: int = 224
    patch_size: int = 16
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    mlp_ratio: int = 4


@dataclass
class CLIPTextConfig:
    """Text tower parameters (ghostflow-nn/src/clip.rs:45-62)."""
    vocab_size: int = 49408
    hidden_size: int = 512
    num_layers: int = 12
    num_heads: int = 8
    max_position_embeddings: int = 77


@dataclass
class CLIPConfig:
    embed_dim: int = 512
    logit_scale_init: float = 2.6592
    image_size: int = 224
    patch_size: int = 16
    vision_width: int = 768
    vision_layers: int = 12
    vision_heads: int = 12
    vocab_size: int = 49408
    text_width: int = 512
    text_layers: int = 12
    text_heads: int = 8
    max_text_len: int = 77

    @classmethod
    def from_towers(cls, vision: "CLIPVisionConfig", text: "CLIPTextConfig", embed_dim: int = 512):
        """The flat configuration of this package from the reference's two tower records."""
        return cls(embed_dim=embed_dim, image_size=vision.image_size, patch_size=vision.patch_size,
                   vision_width=vision.hidden_size, vision_layers=vision.num_layers, vision_heads=vision.num_heads,
                   vocab_size=text.vocab_size, text_width=text.hidden_size, text_layers=text.num_layers,
                   text_heads=text.num_heads, max_text_len=text.max_position_embeddings)

    @property
    def vision_config(self) -> "CLIPVisionConfig":
        return CLIPVisionConfig(self.image_size, self.patch_size, self.vision_width, self.vision_layers,
                                self.vision_heads, 4)

    @property
    def text_config(self) -> "CLIPTextConfig":
        return CLIPTextConfig(self.vocab_size, self.text_width, self.text_layers, self.text_heads, self.max_text_len)

    @classmethod
    def vit_b_32(cls): return cls(patch_size=32)
    @classmethod
    def vit_b_16(cls): return cls()
    @classmethod
    def vit_l_14(cls): return cls(embed_dim=768, patch_size=14, vision_width=1024, vision_layers=24, vision_heads=16,
                                  text_width=768, text_heads=12)
    @classmethod
    def tiny(cls): return cls(embed_dim=32, image_size=32, patch_size=8, vision_width=64, vision_layers=2,
                              vision_heads=2, vocab_size=100, text_width=48, text_layers=2, text_heads=2,
                              max_text_len=16)


class MLP(Module):
    """The feed-forward block of a CLIP layer (ghostflow-nn/src/clip.rs:400-430): Linear, QuickGELU-free GELU, Linear."""

    def __init__(self, width: int, hidden: int):
        super().__init__()
        self.fc1, self.fc2 = Linear(width, hidden), Linear(hidden, width)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x)))


class CLIPTextLayer(TransformerEncoderLayer):
    """One pre-norm, causally masked layer of the text tower (ghostflow-nn/src/clip.rs:300-350)."""

    def __init__(self, c: "CLIPConfig"):
        super().__init__(c.text_width, c.text_heads, 4 * c.text_width, 0.0, True, causal=True)


class CLIPVisionEncoder(Module):
    def __init__(self, c: CLIPConfig):
        super().__init__()
        self.patch = c.patch_size
        n = (c.image_size // c.patch_size) ** 2
        self.proj = Linear(3 * c.patch_size ** 2, c.vision_width, bias=False)
        self.cls = Parameter(torch.zeros(1, 1, c.vision_width))
        self.pos = Parameter(torch.randn(1, n + 1, c.vision_width) * 0.02)
        self.pre = LayerNorm(c.vision_width)
        self.layers = ModuleList([TransformerEncoderLayer(c.vision_width, c.vision_heads, 4 * c.vision_width, 0.0, True)
                                  for _ in range(c.vision_layers)])
        self.post = LayerNorm(c.vision_width)
        self.out = Linear(c.vision_width, c.embed_dim, bias=False)

    def forward(self, img):
        x = self.proj(F.unfold(img, self.patch, stride=self.patch).transpose(1, 2))
        x = self.pre(torch.cat((self.cls.to(x.dtype).expand(x.shape[0], -1, -1), x), 1) + self.pos.to(x.dtype))
        for l in self.layers:
            x = l(x)
        return self.out(self.post(x[:, 0]))


class CLIPTextEncoder(Module):
    def __init__(self, c: CLIPConfig):
        super().__init__()
        self.tok = Embedding(c.vocab_size, c.text_width)
        self.pos = Parameter(torch.randn(1, c.max_text_len, c.text_width) * 0.01)
        self.layers = ModuleList([CLIPTextLayer(c) for _ in range(c.text_layers)])
        self.norm = LayerNorm(c.text_width)
        self.out = Linear(c.text_width, c.embed_dim, bias=False)

    def forward(self, ids):
        x = self.tok(ids) + self.pos[:, :ids.shape[1]].to(self.tok.weight.dtype)
        for l in self.layers:
            x = l(x)
        x = self.norm(x)
        eot = ids.argmax(-1)   # the end-of-text token has the highest id
        return self.out(x[torch.arange(x.shape[0], device=x.device), eot])


class CLIP(Module):
    def __init__(self, config: CLIPConfig | None = None):
        super().__init__()
        self.config = c = config or CLIPConfig()
        self.vision = CLIPVisionEncoder(c)
        self.text = CLIPTextEncoder(c)
        self.logit_scale = Parameter(torch.tensor(c.logit_scale_init))

    def encode_image(self, img):
        return F.normalize(self.vision(img).float(), dim=-1)

    def encode_text(self, ids):
        return F.normalize(self.text(ids).float(), dim=-1)

    def forward(self, img, ids):
        """(logits_per_image, logits_per_text)."""
        i, t = self.encode_image(img), self.encode_text(ids)
        logits = self.logit_scale.exp() * i @ t.t()
        return logits, logits.t()

    def contrastive_loss(self, img, ids):
        li, lt = self.forward(img, ids)
        tgt = torch.arange(li.shape[0], device=li.device)
        return 0.5 * (F.cross_entropy(li, tgt) + F.cross_entropy(lt, tgt))

    @torch.no_grad()
    def zero_shot_classify(self, img, class_token_ids):
        return torch.softmax(self.forward(img, class_token_ids)[0], -1)

    @torch.no_grad()
    def image_to_text_retrieval(self, img, ids, k: int = 1):
        return self.forward(img, ids)[0].topk(min(k, ids.shape[0]), -1).indices

    @torch.no_grad()
    def text_to_image_retrieval(self, ids, img, k: int = 1):
        return self.forward(img, ids)[1].topk(min(k, img.shape[0]), -1).indices


# =========================================================================== diffusion
class BetaSchedule(enum.Enum):
    Linear = "linear"
    Cosine = "cosine"
    ScaledLinear = "scaled_linear"


@dataclass
class DiffusionConfig:
    image_size: int = 256
    in_channels: int = 3
    model_channels: int = 128
    num_res_blocks: int = 2
    channel_mult: tuple = (1, 2, 4, 8)
    num_heads: int = 8
    num_timesteps: int = 1000
    beta_schedule: BetaSchedule = BetaSchedule.Linear
    beta_start: float = 1e-4
    beta_end: float = 0.02

    @classmethod
    def stable_diffusion(cls): return cls(512, 4, 320, 2, (1, 2, 4, 4), 8, 1000, BetaSchedule.ScaledLinear,
                                          0.00085, 0.012)
    @classmethod
    def ddpm(cls): return cls(channel_mult=(1, 1, 2, 2, 4, 4), num_heads=4)
    @classmethod
    def tiny(cls): return cls(32, 3, 64, 1, (1, 2), 2, 100)


class NoiseScheduler:
    def __init__(self, config: DiffusionConfig | None = None):
        c = config or DiffusionConfig()
        T = c.num_timesteps
        if c.beta_schedule == BetaSchedule.Linear:
            betas = torch.linspace(c.beta_start, c.beta_end, T, dtype=torch.float64)
        elif c.beta_schedule == BetaSchedule.ScaledLinear:
            betas = torch.linspace(c.beta_start ** 0.5, c.beta_end ** 0.5, T, dtype=torch.float64) ** 2
        else:
            s = 0.008
            t = torch.arange(T + 1, dtype=torch.float64) / T
            ac = torch.cos((t + s) / (1 + s) * math.pi / 2) ** 2
            betas = (1 - ac[1:] / ac[:-1]).clamp(max=0.999)
        self.betas = betas.float()
        self.alphas = 1.0 - self.betas
        self.alphas_cumprod = torch.cumprod(self.alphas, 0)
        self.num_timesteps = T

    def _gather(self, v, t, x):
        return v.to(x.device)[t].view(-1, *[1] * (x.dim() - 1)).to(x.dtype)

    def add_noise(self, x0, noise, t):
        """``sqrt(abar_t) x0 + sqrt(1 - abar_t) noise``."""
        ab = self._gather(self.alphas_cumprod, t, x0)
        return ab.sqrt() * x0 + (1 - ab).sqrt() * noise

    def predict_x0(self, xt, noise_pred, t):
        ab = self._gather(self.alphas_cumprod, t, xt)
        return (xt - (1 - ab).sqrt() * noise_pred) / ab.sqrt()

    def step(self, xt, noise_pred, t: int, generator=None):
        """One ancestral DDPM step x_t -> x_{t-1}."""
        b, a, ab = self.betas[t], self.alphas[t], self.alphas_cumprod[t]
        mean = (xt - b / (1 - ab).sqrt() * noise_pred) / a.sqrt()
        if t == 0:
            return mean
        ab_prev = self.alphas_cumprod[t - 1]
        var = b * (1 - ab_prev) / (1 - ab)
        z = torch.randn(xt.shape, generator=generator, device=xt.device if generator is None else "cpu").to(xt.device, xt.dtype)
        return mean + var.sqrt() * z


def _timestep_embedding(t, dim):
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    a = t.float()[:, None] * freqs[None]
    return torch.cat((a.sin(), a.cos()), -1)


class ResidualBlock(Module):
    def __init__(self, cin, cout, temb_dim):
        super().__init__()
        self.n1 = GroupNorm(min(32, cin), cin)
        self.c1 = Conv2d(cin, cout, 3, 1, 1)
        self.t = Linear(temb_dim, cout)
        self.n2 = GroupNorm(min(32, cout), cout)
        self.c2 = Conv2d(cout, cout, 3, 1, 1)
        self.skip = Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x, temb):
        h = self.c1(F.silu(self.n1(x)))
        h = h + self.t(F.silu(temb))[:, :, None, None]
        h = self.c2(F.silu(self.n2(h)))
        return h + (self.skip(x) if self.skip is not None else x)


class _AttnBlock(Module):
    def __init__(self, ch, heads):
        super().__init__()
        self.norm = GroupNorm(min(32, ch), ch)
        self.qkv = Conv2d(ch, 3 * ch, 1)
        self.proj = Conv2d(ch, ch, 1)
        self.heads = heads

    def forward(self, x):
        B, C, H, W = x.shape
        q, k, v = self.qkv(self.norm(x)).view(B, 3, self.heads, C // self.heads, H * W).unbind(1)
        a = torch.softmax(q.transpose(-1, -2) @ k / math.sqrt(C // self.heads), -1)
        return x + self.proj((v @ a.transpose(-1, -2)).reshape(B, C, H, W))


class UNet(Module):
    def __init__(self, config: DiffusionConfig | None = None):
        super().__init__()
        self.config = c = config or DiffusionConfig()
        ch = c.model_channels
        self.temb_dim = 4 * ch
        self.time = torch.nn.Sequential(torch.nn.Linear(ch, self.temb_dim), torch.nn.SiLU(),
                                        torch.nn.Linear(self.temb_dim, self.temb_dim))
        self.inp = Conv2d(c.in_channels, ch, 3, 1, 1)
        self.down = ModuleList()
        chans, cur = [ch], ch
        for li, m in enumerate(c.channel_mult):
            for _ in range(c.num_res_blocks):
                self.down.append(ResidualBlock(cur, ch * m, self.temb_dim))
                cur = ch * m
                chans.append(cur)
            if li + 1 < len(c.channel_mult):
                self.down.append(Conv2d(cur, cur, 3, 2, 1))
                chans.append(cur)
        self.mid1 = ResidualBlock(cur, cur, self.temb_dim)
        self.mid_attn = _AttnBlock(cur, c.num_heads)
        self.mid2 = ResidualBlock(cur, cur, self.temb_dim)
        self.up = ModuleList()
        for li, m in reversed(list(enumerate(c.channel_mult))):
            for _ in range(c.num_res_blocks + 1):
                self.up.append(ResidualBlock(cur + chans.pop(), ch * m, self.temb_dim))
                cur = ch * m
            if li > 0:
                self.up.append(torch.nn.Upsample(scale_factor=2, mode="nearest"))
        self.out_norm = GroupNorm(min(32, cur), cur)
        self.out = Conv2d(cur, c.in_channels, 3, 1, 1)

    def forward(self, x, t):
        temb = self.time(_timestep_embedding(t, self.config.model_channels).to(x.dtype))
        h = self.inp(x)
        hs = [h]
        for m in self.down:
            h = m(h, temb) if isinstance(m, ResidualBlock) else m(h)
            hs.append(h)
        h = self.mid2(self.mid_attn(self.mid1(h, temb)), temb)
        for m in self.up:
            if isinstance(m, ResidualBlock):
                h = m(torch.cat((h, hs.pop()), 1), temb)
            else:
                h = m(h)
        return self.out(F.silu(self.out_norm(h)))


class DDPM(Module):
    def __init__(self, config: DiffusionConfig | None = None):
        super().__init__()
        self.config = config or DiffusionConfig()
        self.unet = UNet(self.config)
        self.scheduler = NoiseScheduler(self.config)

    def forward(self, x0, generator=None):
        """Training loss: MSE between the true and the predicted noise at a random timestep."""
        B = x0.shape[0]
        t = torch.randint(0, self.scheduler.num_timesteps, (B,), generator=generator).to(x0.device)
        noise = torch.randn(x0.shape, generator=generator).to(x0.device, x0.dtype)
        return F.mse_loss(self.unet(self.scheduler.add_noise(x0, noise, t), t), noise)

    @torch.no_grad()
    def sample(self, shape, num_steps: int | None = None, generator=None, device=None):
        x = torch.randn(shape, generator=generator).to(device or next(self.parameters()).device)
        T = self.scheduler.num_timesteps
        steps = list(range(T - 1, -1, -1)) if num_steps is None else \
            torch.linspace(T - 1, 0, num_steps).long().tolist()
        for t in steps:
            tt = torch.full((shape[0],), t, device=x.device, dtype=torch.long)
            x = self.scheduler.step(x, self.unet(x, tt), t, generator)
        return x


# =========================================================================== NeRF
@dataclass
class NeRFConfig:
    num_coarse_samples: int = 64
    num_fine_samples: int = 128
    num_freq_bands: int = 10
    num_dir_freq_bands: int = 4
    hidden_dim: int = 256
    num_layers: int = 8
    skip_layer: int = 4
    use_view_dirs: bool = True
    near: float = 2.0
    far: float = 6.0

    @classmethod
    def default(cls): return cls()
    @classmethod
    def tiny(cls): return cls(32, 64, 6, 4, 128, 4, 2)
    @classmethod
    def large(cls): return cls(128, 256, 15, 6, 512, 10, 5)


class PositionalEncoder(Module):
    """``[x, sin(2^k x), cos(2^k x)]`` for k < num_freqs (ghostflow-nn/src/nerf.rs:111-147)."""

    def __init__(self, num_freqs: int, include_input: bool = True):
        super().__init__()
        self.num_freqs, self.include_input = num_freqs, include_input

    def out_dim(self, d):
        return d * (2 * self.num_freqs + (1 if self.include_input else 0))

    def forward(self, x):
        from ..ops import render

        return render.positional_encoding(x, self.num_freqs, self.include_input)


class NeRFMLP(Module):
    def __init__(self, c: NeRFConfig):
        super().__init__()
        self.c = c
        self.pe, self.de = PositionalEncoder(c.num_freq_bands), PositionalEncoder(c.num_dir_freq_bands)
        din = self.pe.out_dim(3)
        self.layers = ModuleList()
        for i in range(c.num_layers):
            self.layers.append(Linear(din if i == 0 else c.hidden_dim + (din if i == c.skip_layer else 0), c.hidden_dim))
        self.sigma = Linear(c.hidden_dim, 1)
        if c.use_view_dirs:
            self.feat = Linear(c.hidden_dim, c.hidden_dim)
            self.rgb1 = Linear(c.hidden_dim + self.de.out_dim(3), c.hidden_dim // 2)
            self.rgb2 = Linear(c.hidden_dim // 2, 3)
        else:
            self.rgb2 = Linear(c.hidden_dim, 3)

    def forward(self, pts, dirs=None):
        """pts ``[..., 3]`` (and unit view directions) -> (rgb in [0,1], sigma >= 0)."""
        e = self.pe(pts)
        h = e
        for i, l in enumerate(self.layers):
            if i == self.c.skip_layer and i > 0:
                h = torch.cat((h, e), -1)
            h = torch.relu(l(h))
        sigma = torch.relu(self.sigma(h)).squeeze(-1)
        if self.c.use_view_dirs and dirs is not None:
            h = torch.relu(self.rgb1(torch.cat((self.feat(h), self.de(dirs)), -1)))
        return torch.sigmoid(self.rgb2(h)), sigma


class RaySampler:
    def __init__(self, near: float, far: float):
        self.near, self.far = near, far

    def sample_uniform(self, n_rays: int, n_samples: int, perturb: bool = False, generator=None, device=None):
        """Depths ``[n_rays, n_samples]``, stratified when ``perturb``."""
        t = torch.linspace(0, 1, n_samples, device=device)
        z = (self.near * (1 - t) + self.far * t).expand(n_rays, n_samples).clone()
        if perturb:
            mid = 0.5 * (z[:, 1:] + z[:, :-1])
            lo = torch.cat((z[:, :1], mid), -1)
            hi = torch.cat((mid, z[:, -1:]), -1)
            z = lo + (hi - lo) * torch.rand(z.shape, generator=generator).to(z.device)
        return z

    @staticmethod
    def sample_pdf(bins, weights, n_samples: int, generator=None):
        """Inverse-transform sampling of depths from piecewise-constant ``weights`` over ``bins``."""
        w = weights + 1e-5
        cdf = torch.cumsum(w / w.sum(-1, keepdim=True), -1)
        cdf = torch.cat((torch.zeros_like(cdf[:, :1]), cdf), -1)
        u = torch.rand(cdf.shape[0], n_samples, generator=generator).to(cdf.device) if generator is not None else \
            torch.linspace(0, 1, n_samples, device=cdf.device).expand(cdf.shape[0], n_samples).contiguous()
        idx = torch.searchsorted(cdf, u, right=True).clamp(1, cdf.shape[-1] - 1)
        c0, c1 = cdf.gather(1, idx - 1), cdf.gather(1, idx)
        b0, b1 = bins.gather(1, (idx - 1).clamp(max=bins.shape[1] - 1)), bins.gather(1, idx.clamp(max=bins.shape[1] - 1))
        return b0 + (u - c0) / (c1 - c0).clamp(min=1e-5) * (b1 - b0)


class VolumeRenderer:
    """``C = sum_i T_i (1 - exp(-sigma_i delta_i)) c_i``, ``T_i = prod_{j<i} exp(-sigma_j delta_j)``
    (ghostflow-nn/src/nerf.rs:353-408)."""

    def __init__(self, white_background: bool = False):
        self.white_background = white_background

    def render_rays(self, rgb, sigma, z_vals, ray_norm=None):
        """rgb ``[R, S, 3]``, sigma ``[R, S]``, z_vals ``[R, S]`` -> (color ``[R,3]``, depth, acc, weights)."""
        from ..ops import render

        return render.volume_render(rgb, sigma, z_vals, ray_norm, self.white_background)


class NeRF(Module):
    def __init__(self, config: NeRFConfig | None = None):
        super().__init__()
        self.config = c = config or NeRFConfig()
        self.coarse = NeRFMLP(c)
        self.fine = NeRFMLP(c) if c.num_fine_samples > 0 else None
        self.sampler = RaySampler(c.near, c.far)
        self.renderer = VolumeRenderer()

    def _run(self, mlp, o, d, z):
        pts = o[:, None, :] + d[:, None, :] * z[..., None]
        dirs = F.normalize(d, dim=-1)[:, None, :].expand_as(pts)
        rgb, sigma = mlp(pts, dirs)
        return self.renderer.render_rays(rgb.float(), sigma.float(), z, d.norm(dim=-1))

    def render(self, rays_o, rays_d, perturb: bool = False, generator=None):
        """Headless render: rays ``[R, 3]`` -> dict(color, depth, acc [, coarse_color])."""
        c = self.config
        z = self.sampler.sample_uniform(rays_o.shape[0], c.num_coarse_samples, perturb, generator, rays_o.device)
        color, depth, acc, w = self._run(self.coarse, rays_o, rays_d, z)
        out = {"color": color, "depth": depth, "acc": acc}
        if self.fine is not None:
            mid = 0.5 * (z[:, 1:] + z[:, :-1])
            zf = RaySampler.sample_pdf(mid, w[:, 1:-1].detach(), c.num_fine_samples, generator)
            z2, _ = torch.sort(torch.cat((z, zf), -1), -1)
            cf, df, af, _ = self._run(self.fine, rays_o, rays_d, z2)
            out = {"color": cf, "depth": df, "acc": af, "coarse_color": color}
        return out

    forward = render
