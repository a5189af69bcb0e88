"""Self-contained diffusion-transformer denoisers that exercise the projection routing.

The reference drives its operator from diffusers models (`sdacc/diffusion_research/models/`:
`dit_xl.py:5-15`, `sigma.py:73-86`, `sd3.py:52-65` list the routed projection groups: fused self
Q|K|V, cross-attention Q and fused K|V, FFN-in, FFN-out; attention cores and attention output
projections stay BF16).  diffusers and checkpoints are not available offline, so these are
random-initialised transformers of the same shapes whose routed projections go through
`routing.ProjectionState`, and whose protected parts are plain BF16 torch modules.  They exist to
measure a full denoise step with the sparse operator against the same step with dense BF16
projections; they are not image generators of any quality.
"""
import math
from dataclasses import dataclass, replace

import torch
from torch import nn
from torch.nn import functional as F

from .backend import Prologue
from .routing import ProjectionState, OrdinaryProxy, pack_members


@dataclass(frozen=True)
class Spec:
    name: str
    family: str            # "dit" | "pixart" | "mmdit"
    blocks: int
    hidden: int
    heads: int
    mlp: int
    grid: int              # patch tokens per side
    patch: int = 2
    latent_channels: int = 4
    out_channels: int = 4
    text_tokens: int = 0
    text_dim: int = 0
    pooled_dim: int = 0
    classes: int = 0
    mode: int = 4
    steps: int = 50
    sampler: str = "ddim"
    guidance: float = 4.0

    @property
    def tokens(self):
        return self.grid * self.grid


SPECS = {
    # DiT-XL/2 at 512x512: latent 4x64x64, learned sigma (8 output channels), 50 DDIM steps, 2:4
    "dit-xl-512": Spec("dit-xl-512", "dit", 28, 1152, 16, 4608, 32, out_channels=8, classes=1000,
                       mode=4, steps=50, sampler="ddim", guidance=4.0),
    # PixArt-Sigma at 1024x1024: latent 4x128x128, 300 text tokens of dim 4096, 20 DPM-Solver++ steps, 6:8
    "pixart-sigma-1024": Spec("pixart-sigma-1024", "pixart", 28, 1152, 16, 4608, 64, out_channels=8,
                              text_tokens=300, text_dim=4096, mode=8, steps=20, sampler="dpmpp2m", guidance=4.5),
    # SD3.5-Large-style MMDiT at 512x512: 16-channel latent 64x64, 333 text tokens, pooled 2048, 25 FlowMatch steps, 4:6
    "sd35-large-512": Spec("sd35-large-512", "mmdit", 38, 2432, 38, 9728, 32, latent_channels=16, out_channels=16,
                           text_tokens=333, text_dim=4096, pooled_dim=2048, mode=6, steps=25,
                           sampler="flowmatch", guidance=4.5),
}


def tiny(spec, blocks=2, hidden=128, heads=4, mlp=256, grid=4, text_tokens=None, text_dim=64, pooled_dim=None):
    """Small instance of the same family for CPU tests."""
    return replace(spec, blocks=blocks, hidden=hidden, heads=heads, mlp=mlp, grid=grid,
                   text_tokens=(min(spec.text_tokens, 7) if text_tokens is None else text_tokens),
                   text_dim=text_dim if spec.text_dim else 0,
                   pooled_dim=(32 if spec.pooled_dim else 0) if pooled_dim is None else pooled_dim,
                   classes=min(spec.classes, 10))


# ------------------------------------------------------------------------------------------------
# building blocks
# ------------------------------------------------------------------------------------------------

def sincos_embedding(positions, dim, max_period=10000.0):
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=positions.device) / half)
    args = positions.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def grid_embedding(grid, dim):
    ys, xs = torch.meshgrid(torch.arange(grid), torch.arange(grid), indexing="ij")
    return torch.cat([sincos_embedding(ys.reshape(-1), dim // 2), sincos_embedding(xs.reshape(-1), dim // 2)], dim=-1)


def gate(x, g, y):
    """x + g[b] * y with g BF16 [batch, hidden]."""
    return torch.addcmul(x, g[:, None], y)


def norm_modulate(shift, scale):
    """LayerNorm (no affine, eps 1e-6) followed by x * (1 + scale[b]) + shift[b], as a prologue of
    the projection that consumes it; shift / scale are BF16 [batch, hidden] (views are fine)."""
    return Prologue.norm_modulate(shift, scale, 1e-6)


class TimestepEmbedder(nn.Module):
    def __init__(self, hidden, extra=0):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(256, hidden), nn.Linear(hidden, hidden)
        self.pooled = nn.Sequential(nn.Linear(extra, hidden), nn.SiLU(), nn.Linear(hidden, hidden)) if extra else None

    def forward(self, t, pooled=None):
        emb = self.fc2(F.silu(self.fc1(sincos_embedding(t, 256).to(self.fc1.weight.dtype))))
        return emb if self.pooled is None else emb + self.pooled(pooled)


class RoutedAttention(nn.Module):
    """Attention whose Q|K|V members (or Q and K|V for cross-attention) are routed; the core
    (scaled_dot_product_attention) and the output projection are protected BF16."""

    def __init__(self, hidden, heads, cross=False, qk_norm=False, out_proj=True):
        super().__init__()
        self.heads, self.cross = heads, cross
        self.to_q, self.to_k, self.to_v = (nn.Linear(hidden, hidden) for _ in range(3))
        self.to_out = nn.Linear(hidden, hidden) if out_proj else None
        self.norm_q = nn.RMSNorm(hidden // heads, eps=1e-6) if qk_norm else None
        self.norm_k = nn.RMSNorm(hidden // heads, eps=1e-6) if qk_norm else None
        self.states = None

    def groups(self):
        if self.cross:
            return [("cross-Q", [self.to_q]), ("cross-KV", [self.to_k, self.to_v])]
        return [("QKV", [self.to_q, self.to_k, self.to_v])]

    def heads_view(self, x):
        return x.reshape(x.shape[0], x.shape[1], self.heads, -1).transpose(1, 2)

    def qkv(self, x, context=None, prologue=None):
        if self.cross:
            (q,), (k, v) = self.states[0].members_output(x, prologue), self.states[1].members_output(context)
        else:
            q, k, v = self.states[0].members_output(x, prologue)
        q, k, v = self.heads_view(q), self.heads_view(k), self.heads_view(v)
        if self.norm_q is not None:
            q, k = self.norm_q(q), self.norm_k(k)
        return q, k, v

    def finish(self, attended):
        merged = attended.transpose(1, 2).reshape(attended.shape[0], attended.shape[2], -1)
        return merged if self.to_out is None else self.to_out(merged)

    def forward(self, x, context=None, prologue=None):
        q, k, v = self.qkv(x, context, prologue)
        return self.finish(F.scaled_dot_product_attention(q, k, v))


class RoutedFeedForward(nn.Module):
    def __init__(self, hidden, mlp):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(hidden, mlp), nn.Linear(mlp, hidden)

    def groups(self):
        return [("FFN-in", [self.fc1]), ("FFN-out", [self.fc2])]

    def install(self, states):
        self.fc1, self.fc2 = OrdinaryProxy(states[0]), OrdinaryProxy(states[1])

    def forward(self, x, prologue=None, gated_residual=None):
        """fc2(gelu(fc1(prologue(x)))); with gated_residual = (residual, gate) the block's
        residual + gate * (...) is part of the second projection.  The GELU is its prologue."""
        return self.fc2(self.fc1(x, prologue), Prologue.gelu(), gated_residual)


class DiTBlock(nn.Module):
    """adaLN-Zero block: conditioning vector -> six modulation vectors per block."""

    def __init__(self, spec):
        super().__init__()
        h = spec.hidden
        self.attn, self.ff = RoutedAttention(h, spec.heads), RoutedFeedForward(h, spec.mlp)
        self.adaln = nn.Linear(h, 6 * h)

    def forward(self, x, c, context=None):
        s1, c1, g1, s2, c2, g2 = self.adaln(F.silu(c)).chunk(6, dim=-1)
        x = gate(x, g1, self.attn(x, prologue=norm_modulate(s1, c1)))
        return self.ff(x, norm_modulate(s2, c2), gated_residual=(x, g2))


class PixArtBlock(nn.Module):
    """adaLN-single block with cross-attention to the projected text tokens."""

    def __init__(self, spec):
        super().__init__()
        h = spec.hidden
        self.attn = RoutedAttention(h, spec.heads)
        self.cross = RoutedAttention(h, spec.heads, cross=True)
        self.ff = RoutedFeedForward(h, spec.mlp)
        self.table = nn.Parameter(torch.randn(6, h) / math.sqrt(h))

    def forward(self, x, c6, context):
        s1, c1, g1, s2, c2, g2 = (self.table[None] + c6.reshape(c6.shape[0], 6, -1)).unbind(1)
        x = gate(x, g1, self.attn(x, prologue=norm_modulate(s1, c1)))
        x = x + self.cross(x, context)
        return self.ff(x, norm_modulate(s2, c2), gated_residual=(x, g2))


class JointBlock(nn.Module):
    """MMDiT block: image and text streams with their own QKV / FFN, one joint attention."""

    def __init__(self, spec, last):
        super().__init__()
        h = spec.hidden
        self.last = last
        self.attn = RoutedAttention(h, spec.heads, qk_norm=True)
        self.attn_text = RoutedAttention(h, spec.heads, qk_norm=True, out_proj=not last)
        self.ff = RoutedFeedForward(h, spec.mlp)
        self.ff_text = None if last else RoutedFeedForward(h, spec.mlp)
        self.adaln = nn.Linear(h, 6 * h)
        self.adaln_text = nn.Linear(h, (2 if last else 6) * h)

    def forward(self, x, text, c):
        act = F.silu(c)
        s1, c1, g1, s2, c2, g2 = self.adaln(act).chunk(6, dim=-1)
        mod_text = self.adaln_text(act).chunk(2 if self.last else 6, dim=-1)
        q, k, v = self.attn.qkv(x, prologue=norm_modulate(s1, c1))
        tq, tk, tv = self.attn_text.qkv(text, prologue=norm_modulate(mod_text[0], mod_text[1]))
        joint = F.scaled_dot_product_attention(torch.cat([q, tq], 2), torch.cat([k, tk], 2), torch.cat([v, tv], 2))
        tokens = x.shape[1]
        x = gate(x, g1, self.attn.finish(joint[:, :, :tokens]))
        x = self.ff(x, norm_modulate(s2, c2), gated_residual=(x, g2))
        if self.last:
            return x, text
        text = gate(text, mod_text[2], self.attn_text.finish(joint[:, :, tokens:]))
        text = self.ff_text(text, norm_modulate(mod_text[3], mod_text[4]), gated_residual=(text, mod_text[5]))
        return x, text


# ------------------------------------------------------------------------------------------------
# the denoiser
# ------------------------------------------------------------------------------------------------

class Denoiser(nn.Module):
    """forward(latent [B,C,H,W], t [B], cond) -> model output [B,out_channels,H,W].

    cond: class ids [B] (dit) | text [B,T,text_dim] (pixart) | (text, pooled [B,pooled_dim]) (mmdit).
    """

    def __init__(self, spec):
        super().__init__()
        self.spec = spec
        h, p = spec.hidden, spec.patch
        self.embed = nn.Linear(spec.latent_channels * p * p, h)
        self.register_buffer("pos", grid_embedding(spec.grid, h), persistent=False)
        self.time = TimestepEmbedder(h, spec.pooled_dim)
        if spec.family == "dit":
            self.classes = nn.Embedding(spec.classes + 1, h)
            self.blocks = nn.ModuleList(DiTBlock(spec) for _ in range(spec.blocks))
        elif spec.family == "pixart":
            self.caption = nn.Sequential(nn.Linear(spec.text_dim, h), nn.GELU(approximate="tanh"), nn.Linear(h, h))
            self.adaln_single = nn.Linear(h, 6 * h)
            self.blocks = nn.ModuleList(PixArtBlock(spec) for _ in range(spec.blocks))
        elif spec.family == "mmdit":
            self.context = nn.Linear(spec.text_dim, h)
            self.blocks = nn.ModuleList(JointBlock(spec, i == spec.blocks - 1) for i in range(spec.blocks))
        else:
            raise ValueError("unknown denoiser family")
        self.final_adaln = nn.Linear(h, 2 * h)
        self.final = nn.Linear(h, p * p * spec.out_channels)
        self.states, self.units = [], []
        self._install()

    # -- routing -------------------------------------------------------------------------------

    def _routed(self, block):
        parts = [block.attn]
        if hasattr(block, "cross"):
            parts.append(block.cross)
        parts.append(block.ff)
        if hasattr(block, "attn_text"):
            parts += [block.attn_text] + ([block.ff_text] if block.ff_text is not None else [])
        return parts

    def _install(self):
        """One ProjectionState per routed group, in the order the reference inventories them."""
        spec = self.spec
        image_rows, text_rows = 2 * spec.tokens, 2 * spec.text_tokens
        for index, block in enumerate(self.blocks):
            for part in self._routed(block):
                text_side = part is getattr(block, "attn_text", None) or part is getattr(block, "ff_text", None)
                states = []
                for role, members in part.groups():
                    state = ProjectionState(members, {})
                    rows = text_rows if (text_side or role == "cross-KV") else image_rows
                    self.units.append(dict(unit=len(self.units), block=index, module=("text." if text_side else "") + role,
                                           m=rows, k=members[0].in_features, n=sum(m.out_features for m in members)))
                    states.append(state)
                    self.states.append(state)
                if isinstance(part, RoutedFeedForward):
                    part.install(states)
                else:
                    part.states = states

    def pack(self, mode=None, packer=pack_members, only_profitable=True):
        """Prune + quantise + pack the routed groups for `mode` (default: the spec's).  With
        `only_profitable` the groups that `profile.selectable` rejects for their (M, K, N) get no
        operator and stay dense under `select` (the reference keeps such shapes dense too)."""
        from .profile import selectable
        mode = self.spec.mode if mode is None else mode
        for state, unit in zip(self.states, self.units):
            if only_profitable and not selectable(mode, unit["m"], unit["k"], unit["n"]):
                continue
            state.ops[mode] = packer(state.members, mode)
        return mode

    def select(self, mode):
        """Route every group that has an operator for `mode` through it; the others run dense."""
        for state in self.states:
            state.select(mode if mode in state.ops else 0)

    def sparse_units(self, mode):
        return sum(1 for state in self.states if mode in state.ops)

    def fuse_neighbours(self, enabled=True):
        """Run LayerNorm + modulation and GELU inside the sparse front-end kernels (no effect on
        the dense path, which keeps them as separate PyTorch operators)."""
        for state in self.states:
            state.fuse = bool(enabled)

    # -- forward -------------------------------------------------------------------------------

    def patchify(self, latent):
        b, c, hh, ww = latent.shape
        p = self.spec.patch
        x = latent.reshape(b, c, hh // p, p, ww // p, p).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(b, (hh // p) * (ww // p), c * p * p)

    def unpatchify(self, x):
        b, g, p, c = x.shape[0], self.spec.grid, self.spec.patch, self.spec.out_channels
        return x.reshape(b, g, g, c, p, p).permute(0, 3, 1, 4, 2, 5).reshape(b, c, g * p, g * p)

    def forward(self, latent, t, cond):
        spec = self.spec
        x = self.embed(self.patchify(latent)) + self.pos.to(latent.dtype)
        if spec.family == "dit":
            c = self.time(t) + self.classes(cond)
            for block in self.blocks:
                x = block(x, c)
        elif spec.family == "pixart":
            c = self.time(t)
            c6, context = self.adaln_single(F.silu(c)), self.caption(cond)
            for block in self.blocks:
                x = block(x, c6, context)
        else:
            text, pooled = cond
            c, text = self.time(t, pooled), self.context(text)
            for block in self.blocks:
                x, text = block(x, text, c)
        shift, scale = self.final_adaln(F.silu(c)).chunk(2, dim=-1)
        return self.unpatchify(self.final(norm_modulate(shift, scale).torch_reference(x)))


# ------------------------------------------------------------------------------------------------
# samplers: per-step coefficient tables (host) + one device update, classifier-free guidance
# ------------------------------------------------------------------------------------------------

def _alphas_cumprod(train_steps=1000, beta_start=1e-4, beta_end=0.02):
    betas = torch.linspace(beta_start, beta_end, train_steps, dtype=torch.float64)
    return torch.cumprod(1 - betas, 0)


def sampler_table(spec):
    """(timesteps [S], coefficients [S,4]) such that each update is
    x <- a*x + b*out + c*previous_x0 (ddim / flowmatch use c = 0; d is the x0-mixing weight)."""
    steps = spec.steps
    if spec.sampler == "flowmatch":
        shift = 3.0
        sig = torch.linspace(1.0, 1.0 / steps, steps, dtype=torch.float64)
        sig = torch.cat([shift * sig / (1 + (shift - 1) * sig), torch.zeros(1, dtype=torch.float64)])
        coef = torch.stack([torch.ones(steps, dtype=torch.float64), sig[1:] - sig[:-1],
                            torch.zeros(steps, dtype=torch.float64), torch.zeros(steps, dtype=torch.float64)], 1)
        return (1000 * sig[:-1]).float(), coef.float()
    ac = _alphas_cumprod()
    ts = torch.linspace(999, 0, steps + 1, dtype=torch.float64).round().long()
    a_t, a_n = ac[ts[:-1]], torch.cat([ac[ts[1:-1]], torch.ones(1, dtype=torch.float64)])
    if spec.sampler == "ddim":
        # x0 = (x - sqrt(1-a_t) eps)/sqrt(a_t);  x' = sqrt(a_n) x0 + sqrt(1-a_n) eps
        ratio = (a_n / a_t).sqrt()
        coef = torch.stack([ratio, (1 - a_n).sqrt() - ratio * (1 - a_t).sqrt(),
                            torch.zeros_like(ratio), torch.zeros_like(ratio)], 1)
        return ts[:-1].float(), coef.float()
    if spec.sampler == "dpmpp2m":
        # data-prediction multistep: x' = (s_n/s_t) x - alpha_n (e^{-h} - 1) D,  D = (1+1/(2r)) x0 - 1/(2r) x0_prev
        alpha, sigma = a_t.sqrt(), (1 - a_t).sqrt()
        alpha_n, sigma_n = a_n.sqrt(), (1 - a_n).clamp_min(1e-10).sqrt()
        lam, lam_n = torch.log(alpha / sigma), torch.log(alpha_n / sigma_n)
        h = lam_n - lam
        gain = -alpha_n * torch.expm1(-h)
        r = torch.ones_like(h)
        r[1:] = h[:-1] / h[1:]
        w_prev = torch.where(torch.arange(steps) == 0, torch.zeros_like(h), 1 / (2 * r))
        w_prev[-1] = 0.0                                  # first-order final step
        # x0 = (x - sigma eps)/alpha folded into a, b:  x' = a x + b eps + c x0_prev, d = 1/alpha for x0 bookkeeping
        w_cur = 1 + w_prev
        a = sigma_n / sigma + gain * w_cur / alpha
        b = -gain * w_cur * sigma / alpha
        c = -gain * w_prev
        return ts[:-1].float(), torch.stack([a, b, c, sigma / alpha], 1).float()
    raise ValueError("unknown sampler")


class DenoiseLoop:
    """One image (CFG batch of 2 = conditional + unconditional) per call of `run`.

    A step = one model forward on the CFG batch, guidance, and the sampler update.  With
    `graph=True` the step is captured once in a CUDA graph; the per-step timestep and coefficients
    are small device tensors refreshed before each replay.
    """

    def __init__(self, model, dtype=torch.bfloat16, graph=False, images=1):
        self.model, self.spec, self.dtype, self.images = model, model.spec, dtype, images
        device = next(model.parameters()).device
        spec = self.spec
        side = spec.grid * spec.patch
        ts, coef = sampler_table(spec)
        self.ts, self.coefs = ts.to(device), coef.to(device)
        self.t = torch.zeros(2 * images, device=device)
        self.coef = torch.zeros(4, device=device)
        self.x = torch.zeros(images, spec.latent_channels, side, side, device=device, dtype=torch.float32)
        self.prev_x0 = torch.zeros_like(self.x)
        self.cond = None
        self.graph = None
        self.use_graph = graph

    def conditioning(self, seed=0):
        """Synthetic conditioning for the CFG pair: [conditional..., unconditional...]."""
        spec, device, n = self.spec, self.x.device, self.images
        gen = torch.Generator(device="cpu").manual_seed(seed)
        if spec.family == "dit":
            ids = torch.randint(0, spec.classes, (n,), generator=gen)
            return torch.cat([ids, torch.full((n,), spec.classes)]).to(device)
        text = torch.randn(n, spec.text_tokens, spec.text_dim, generator=gen)
        text = torch.cat([text, torch.zeros_like(text)]).to(device, self.dtype)
        if spec.family == "pixart":
            return text
        pooled = torch.randn(n, spec.pooled_dim, generator=gen)
        return text, torch.cat([pooled, torch.zeros_like(pooled)]).to(device, self.dtype)

    def step(self):
        spec = self.spec
        out = self.model(torch.cat([self.x, self.x]).to(self.dtype), self.t, self.cond).float()
        out = out[:, :spec.latent_channels]
        cond, uncond = out.chunk(2)
        guided = torch.lerp(uncond, cond, spec.guidance)
        a, b, c, d = self.coef.unbind()
        if spec.sampler == "dpmpp2m":
            # d = sigma/alpha with alpha^2 + sigma^2 = 1, so x0 = x/alpha - d*eps = x*sqrt(1+d^2) - d*eps
            x0 = self.x * torch.sqrt(1 + d * d) - d * guided
            new = a * self.x + b * guided + c * self.prev_x0
            self.prev_x0.copy_(x0)
        else:
            new = a * self.x + b * guided
        self.x.copy_(new)

    def _launch(self):
        if not self.use_graph:
            return self.step()
        if self.graph is None:
            side = torch.cuda.Stream(self.x.device)
            side.wait_stream(torch.cuda.current_stream())
            keep = (self.x.clone(), self.prev_x0.clone())
            with torch.cuda.stream(side), torch.no_grad():
                self.step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.x.copy_(keep[0])
            self.prev_x0.copy_(keep[1])
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph), torch.no_grad():
                self.step()
            self.x.copy_(keep[0])
            self.prev_x0.copy_(keep[1])
        self.graph.replay()

    def inputs(self, seed=0):
        """(initial latent noise, conditioning) for `run`, drawn on the host from `seed` and moved to
        the device: callers that time the loop draw them beforehand and pass them to `run`."""
        gen = torch.Generator(device="cpu").manual_seed(seed)
        return torch.randn(self.x.shape, generator=gen).to(self.x.device), self.conditioning(seed)

    @torch.no_grad()
    def run(self, seed=0, steps=None, inputs=None):
        """Full sampling loop from seeded noise (or from `inputs` = what `inputs(seed)` returned);
        returns the final latent (fp32)."""
        noise, cond = self.inputs(seed) if inputs is None else inputs
        self.x.copy_(noise)
        self.prev_x0.zero_()
        if self.cond is None:
            self.cond = cond
        elif isinstance(cond, tuple):
            for dst, src in zip(self.cond, cond):
                dst.copy_(src)
        else:
            self.cond.copy_(cond)
        for i in range(self.spec.steps if steps is None else steps):
            self.t.copy_(self.ts[i].expand_as(self.t))
            self.coef.copy_(self.coefs[i])
            self._launch()
        return self.x.clone()


def images_for_rank(total, rank, world):
    """Data-parallel split of a batch of images: rank r takes images r, r+world, ... (no exchange)."""
    return list(range(rank, total, world))


def build(name, device="cuda", dtype=torch.bfloat16, seed=0, **overrides):
    spec = replace(SPECS[name], **overrides) if overrides else SPECS[name]
    torch.manual_seed(seed)
    with torch.device(device):
        model = Denoiser(spec)
    for p in model.parameters():
        if p.ndim == 2:
            p.data.normal_(0, 0.02)
    return model.to(dtype).eval()
