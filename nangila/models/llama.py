"""Llama-style decoder (RMSNorm, rotary position embedding, SwiGLU MLP, untied head, no biases), the
model of the fully-sharded benchmark: 24 layers, d_model 2048, 16 heads, SwiGLU 5632, vocabulary
32000, sequence 2048 (about 1.3 B parameters).

The reference's FSDP examples wrap Hugging Face Llama checkpoints (examples/train_fsdp_llm.py); here
the architecture is defined directly and initialised randomly. Each :class:`DecoderBlock` is the unit
``fully_shard`` wraps.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    n_layer: int = 24
    n_head: int = 16
    n_kv_head: int = 16
    d_model: int = 2048
    d_mlp: int = 5632
    vocab_size: int = 32000
    max_seq: int = 2048
    rope_theta: float = 10000.0
    eps: float = 1e-5

    @staticmethod
    def llama_1_3b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def tiny() -> "LlamaConfig":
        return LlamaConfig(n_layer=2, n_head=4, n_kv_head=2, d_model=128, d_mlp=352, vocab_size=1024, max_seq=128)


class RMSNorm(nn.Module):
    def __init__(self, d: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, (x.size(-1),), self.weight, self.eps)


def rope_table(seq: int, head_dim: int, theta: float, device) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return torch.stack((ang.cos(), ang.sin()), dim=-1)  # [seq, head_dim / 2, 2]


def apply_rope(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x: [b, t, h, d]; rotates consecutive (even, odd) pairs."""
    b, t, h, d = x.shape
    xf = x.float().view(b, t, h, d // 2, 2)
    cos, sin = table[:t, None, :, 0], table[:t, None, :, 1]
    out = torch.stack((xf[..., 0] * cos - xf[..., 1] * sin, xf[..., 0] * sin + xf[..., 1] * cos), dim=-1)
    return out.view(b, t, h, d).to(x.dtype)


class DecoderBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.h, self.kv = cfg.n_head, cfg.n_kv_head
        self.hd = cfg.d_model // cfg.n_head
        self.norm1 = RMSNorm(cfg.d_model, cfg.eps)
        self.wq = nn.Linear(cfg.d_model, self.h * self.hd, bias=False)
        self.wk = nn.Linear(cfg.d_model, self.kv * self.hd, bias=False)
        self.wv = nn.Linear(cfg.d_model, self.kv * self.hd, bias=False)
        self.wo = nn.Linear(self.h * self.hd, cfg.d_model, bias=False)
        self.norm2 = RMSNorm(cfg.d_model, cfg.eps)
        self.gate = nn.Linear(cfg.d_model, cfg.d_mlp, bias=False)
        self.up = nn.Linear(cfg.d_model, cfg.d_mlp, bias=False)
        self.down = nn.Linear(cfg.d_mlp, cfg.d_model, bias=False)

    def forward(self, x: torch.Tensor, rope: torch.Tensor) -> torch.Tensor:
        b, t, _ = x.shape
        y = self.norm1(x)
        q = apply_rope(self.wq(y).view(b, t, self.h, self.hd), rope).transpose(1, 2)
        k = apply_rope(self.wk(y).view(b, t, self.kv, self.hd), rope).transpose(1, 2)
        v = self.wv(y).view(b, t, self.kv, self.hd).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.kv != self.h)
        x = x + self.wo(a.transpose(1, 2).reshape(b, t, self.h * self.hd))
        y = self.norm2(x)
        return x + self.down(F.silu(self.gate(y)) * self.up(y))


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.blocks = nn.ModuleList([DecoderBlock(cfg) for _ in range(cfg.n_layer)])
        self.norm = RMSNorm(cfg.d_model, cfg.eps)
        self.head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
        self._rope: torch.Tensor | None = None

    def forward(self, idx: torch.Tensor, targets: torch.Tensor | None = None):
        t = idx.size(1)
        if self._rope is None or self._rope.device != idx.device or self._rope.size(0) < t:
            self._rope = rope_table(max(t, self.cfg.max_seq), self.cfg.d_model // self.cfg.n_head, self.cfg.rope_theta, idx.device)
        x = self.embed(idx)
        for blk in self.blocks:
            x = blk(x, self._rope)
        logits = self.head(self.norm(x))
        if targets is None:
            return logits
        from ..ops.fused_ce import fused_cross_entropy  # fused kernels for bf16 logits on a GPU, PyTorch's path otherwise

        return fused_cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1))

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())
