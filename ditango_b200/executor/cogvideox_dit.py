"""Random-init CogVideoX-5B-shaped DiT driven by the sequence-parallel attention path.

A plain-PyTorch restatement of the reference's CogVideoX fork -- block structure of
executor/cogvideox/cogvideox_transformer_3d.py:139-190 (LayerNormZero modulation, joint text+video
attention, GELU-tanh feed-forward), model forward :447-543 (embed, shard tokens and rotary tables
over the sequence-parallel group with zero-padded uneven shards, blocks, gather, final norm / proj,
unpatchify), attention adapter executor/cogvideox/attention_processor.py:31-86 (use-ditango) and
baseline/ulysses.py:32-136 (use-ulysses), denoising loop pipeline_cogvideox.py:608-656 (in-batch
classifier-free guidance).  diffusers is not required.  Weights are random: this module exists to
measure per-step latency and exposed communication of the two attention modes inside a whole
denoising loop; projections and feed-forward are library GEMMs, the attention is this package's.
"""
import math
from dataclasses import dataclass
from typing import Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..baseline.ulysses import heads_to_sequence, sequence_to_heads
from ..core.attention import proAttention
from ..utils import remove_padding_after_gather, split_tensor_uneven, update_timestep
from .. import ops as _engine


@dataclass
class DiTConfig:
    num_layers: int = 42
    num_heads: int = 48
    head_dim: int = 64
    in_channels: int = 16
    patch_size: int = 2
    text_dim: int = 4096
    time_dim: int = 512
    frames: int = 13
    height: int = 60
    width: int = 90
    text_len: int = 226

    @property
    def dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def video_tokens(self) -> int:
        return self.frames * (self.height // self.patch_size) * (self.width // self.patch_size)


def rotary_tables(cfg: DiTConfig, device, dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """3-D rotary tables [video_tokens, head_dim]: head_dim split 1/4 : 3/8 : 3/8 over (t, h, w)."""
    d_t = cfg.head_dim // 4
    d_h = d_w = (cfg.head_dim - d_t) // 2
    gh, gw = cfg.height // cfg.patch_size, cfg.width // cfg.patch_size

    def axis(n, d):
        freqs = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        ang = torch.outer(torch.arange(n, dtype=torch.float32), freqs)
        return ang.repeat_interleave(2, dim=1)                       # [n, d]
    t = axis(cfg.frames, d_t)[:, None, None, :].expand(cfg.frames, gh, gw, d_t)
    h = axis(gh, d_h)[None, :, None, :].expand(cfg.frames, gh, gw, d_h)
    w = axis(gw, d_w)[None, None, :, :].expand(cfg.frames, gh, gw, d_w)
    ang = torch.cat([t, h, w], dim=-1).reshape(-1, cfg.head_dim)
    return ang.cos().to(device=device, dtype=dtype), ang.sin().to(device=device, dtype=dtype)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, S, H, D] with interleaved (real, imaginary) channel pairs; cos/sin [S, D]."""
    xr, xi = x.float().unflatten(-1, (-1, 2)).unbind(-1)
    rot = torch.stack([-xi, xr], dim=-1).flatten(-2)
    return (x.float() * cos[None, :, None, :] + rot * sin[None, :, None, :]).to(x.dtype)


class LayerNormZero(nn.Module):
    def __init__(self, time_dim: int, dim: int):
        super().__init__()
        self.linear = nn.Linear(time_dim, 6 * dim)
        self.norm = nn.LayerNorm(dim, eps=1e-5)

    def forward(self, h, enc, temb):
        shift, scale, gate, e_shift, e_scale, e_gate = self.linear(F.silu(temb)).chunk(6, dim=1)
        h = self.norm(h) * (1 + scale)[:, None] + shift[:, None]
        enc = self.norm(enc) * (1 + e_scale)[:, None] + e_shift[:, None]
        return h, enc, gate[:, None], e_gate[:, None]


class DiTBlock(nn.Module):
    def __init__(self, cfg: DiTConfig, layer_id: int, group, mode: str):
        super().__init__()
        dim = cfg.dim
        self.cfg, self.mode, self.group = cfg, mode, group
        self.norm1 = LayerNormZero(cfg.time_dim, dim)
        self.to_q, self.to_k, self.to_v = (nn.Linear(dim, dim) for _ in range(3))
        self.norm_q = nn.LayerNorm(cfg.head_dim, eps=1e-6)
        self.norm_k = nn.LayerNorm(cfg.head_dim, eps=1e-6)
        self.to_out = nn.Linear(dim, dim)
        self.norm2 = LayerNormZero(cfg.time_dim, dim)
        self.ff_in = nn.Linear(dim, 4 * dim)
        self.ff_out = nn.Linear(4 * dim, dim)
        self.attention = proAttention(layer_id, group) if mode != "ulysses" else None

    def _attend(self, h, enc, rope):
        cfg = self.cfg
        B, text_len = h.shape[0], enc.shape[1]
        H, D = cfg.num_heads, cfg.head_dim
        if self.mode == "ulysses":
            # project the local shards, exchange heads for sequence per stream, then text before video
            def proj(x):
                return [f(x).view(B, x.shape[1], H, D) for f in (self.to_q, self.to_k, self.to_v)]
            q, k, v = heads_to_sequence(proj(h), self.group)
            eq, ek, ev = heads_to_sequence(proj(enc), self.group)
            text_all = eq.shape[1]
            q, k, v = (torch.cat([a, b], dim=1) for a, b in ((eq, q), (ek, k), (ev, v)))
            q, k = self.norm_q(q), self.norm_k(k)
            cos, sin = rope                                          # unsharded (padded) tables
            q = torch.cat([q[:, :text_all], apply_rotary(q[:, text_all:], cos, sin)], dim=1)
            k = torch.cat([k[:, :text_all], apply_rotary(k[:, text_all:], cos, sin)], dim=1)
            out, _ = _engine.flash_partial(q.contiguous(), k.contiguous(), v.contiguous(), out_dtype=torch.bfloat16,
                                           softmax_scale=1.0 / math.sqrt(D))
            o_enc = sequence_to_heads(out[:, :text_all].contiguous(), self.group).flatten(2).to(h.dtype)
            o_vid = sequence_to_heads(out[:, text_all:].contiguous(), self.group).flatten(2).to(h.dtype)
            return self.to_out(o_vid), self.to_out(o_enc)
        x = torch.cat([enc, h], dim=1)
        q, k, v = (f(x).view(B, -1, H, D) for f in (self.to_q, self.to_k, self.to_v))
        q, k = self.norm_q(q), self.norm_k(k)
        cos, sin = rope                                              # this rank's slice of the tables
        q = torch.cat([q[:, :text_len], apply_rotary(q[:, text_len:], cos, sin)], dim=1)
        k = torch.cat([k[:, :text_len], apply_rotary(k[:, text_len:], cos, sin)], dim=1)
        out = self.attention.attn(q.contiguous(), k.contiguous(), v.contiguous())
        out = self.to_out(out.to(x.dtype).flatten(2))
        return out[:, text_len:], out[:, :text_len]

    def forward(self, h, enc, temb, rope):
        text_len = enc.shape[1]
        nh, nenc, gate, e_gate = self.norm1(h, enc, temb)
        a_h, a_enc = self._attend(nh, nenc, rope)
        h = h + gate * a_h
        enc = enc + e_gate * a_enc
        nh, nenc, gate, e_gate = self.norm2(h, enc, temb)
        ff = self.ff_out(F.gelu(self.ff_in(torch.cat([nenc, nh], dim=1)), approximate="tanh"))
        return h + gate * ff[:, text_len:], enc + e_gate * ff[:, :text_len]


class CogVideoXDiT(nn.Module):
    """mode: 'ditango' / 'ring' (proAttention; the stride schedule decides reuse) or 'ulysses'."""

    def __init__(self, cfg: DiTConfig, group, mode: str = "ditango"):
        super().__init__()
        self.cfg, self.group, self.mode = cfg, group, mode
        p = cfg.patch_size
        self.patch_embed = nn.Linear(cfg.in_channels * p * p, cfg.dim)
        self.text_proj = nn.Linear(cfg.text_dim, cfg.dim)
        self.time_embed = nn.Sequential(nn.Linear(cfg.dim, cfg.time_dim), nn.SiLU(), nn.Linear(cfg.time_dim, cfg.time_dim))
        self.blocks = nn.ModuleList(DiTBlock(cfg, i, group, mode) for i in range(cfg.num_layers))
        self.norm_final = nn.LayerNorm(cfg.dim, eps=1e-5)
        self.norm_out = nn.LayerNorm(cfg.dim, eps=1e-5, elementwise_affine=False)
        self.out_mod = nn.Linear(cfg.time_dim, 2 * cfg.dim)
        self.proj_out = nn.Linear(cfg.dim, cfg.in_channels * p * p)
        self._rope = None

    def _timestep_embedding(self, t: torch.Tensor) -> torch.Tensor:
        half = self.cfg.dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
        ang = t.float()[:, None] * freqs[None]
        return torch.cat([ang.cos(), ang.sin()], dim=-1)

    def forward(self, latents: torch.Tensor, text: torch.Tensor, timestep: torch.Tensor) -> torch.Tensor:
        """latents [B, F, C, H, W], text [B, text_len, text_dim], timestep [B] -> noise prediction like latents."""
        cfg, p = self.cfg, self.cfg.patch_size
        B, Fr, C, Hh, Ww = latents.shape
        dtype = self.patch_embed.weight.dtype
        temb = self.time_embed(self._timestep_embedding(timestep).to(dtype))
        x = latents.reshape(B, Fr, C, Hh // p, p, Ww // p, p).permute(0, 1, 3, 5, 2, 4, 6).flatten(4).flatten(1, 3)
        h = self.patch_embed(x.to(dtype))
        enc = self.text_proj(text.to(dtype))
        N, r = self.group.world_size, self.group.rank_in_group
        if self._rope is None:
            self._rope = rotary_tables(cfg, latents.device)
        cos, sin = self._rope
        if N > 1:
            h = split_tensor_uneven(h, N, dim=1, tensor_name="hidden")[r]
            enc = split_tensor_uneven(enc, N, dim=1, tensor_name="encoder_hidden")[r]
            if self.mode == "ulysses":
                # full tables in the gathered order: every rank's shard keeps its zero padding
                cos = torch.cat(split_tensor_uneven(cos, N, dim=0), dim=0)
                sin = torch.cat(split_tensor_uneven(sin, N, dim=0), dim=0)
            else:
                cos, sin = split_tensor_uneven(cos, N, dim=0)[r], split_tensor_uneven(sin, N, dim=0)[r]
        for blk in self.blocks:
            h, enc = blk(h, enc, temb, (cos, sin))
        if N > 1:
            h = remove_padding_after_gather(self.group.all_gather(h.contiguous(), dim=1), "hidden")
            enc = remove_padding_after_gather(self.group.all_gather(enc.contiguous(), dim=1), "encoder_hidden")
        text_len = enc.shape[1]
        h = self.norm_final(torch.cat([enc, h], dim=1))[:, text_len:]
        shift, scale = self.out_mod(F.silu(temb)).chunk(2, dim=1)
        h = self.proj_out(self.norm_out(h) * (1 + scale)[:, None] + shift[:, None])
        out = h.reshape(B, Fr, Hh // p, Ww // p, -1, p, p).permute(0, 1, 4, 2, 5, 3, 6).flatten(5, 6).flatten(3, 4)
        return out


@torch.no_grad()
def denoise(model: CogVideoXDiT, latents: torch.Tensor, text_cond: torch.Tensor, text_uncond: torch.Tensor,
            num_steps: int, guidance_scale: float = 6.0, first_step: int = 0, on_step=None) -> torch.Tensor:
    """Denoising loop with in-batch classifier-free guidance and a plain Euler update (the scheduler is
    not part of the attention path).  Sets the global step index before every model call."""
    text = torch.cat([text_uncond, text_cond], dim=0)
    for i in range(first_step, first_step + num_steps):
        update_timestep(i)
        t = torch.full((2 * latents.shape[0],), 1000.0 * (1.0 - i / max(1, first_step + num_steps)), device=latents.device)
        noise = model(torch.cat([latents, latents], dim=0), text, t).float()
        n_uncond, n_text = noise.chunk(2)
        noise = n_uncond + guidance_scale * (n_text - n_uncond)
        latents = (latents.float() - noise / (first_step + num_steps)).to(latents.dtype)
        if on_step is not None:
            on_step(i)
    return latents
