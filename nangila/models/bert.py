"""BERT encoder with a masked-language-model head, the model of the DGC benchmark
(BERT-large: 24 layers, d_model 1024, 16 heads, MLP 4096, vocabulary 30522, sequence 512).

Post-LayerNorm encoder blocks, learned position and segment embeddings, GELU MLP, and the MLM head
(dense + GELU + LayerNorm, decoder tied to the token embedding). The reference ships no model; its
examples train Hugging Face models through DDP (examples/train_llm.py:230-332).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class BertConfig:
    n_layer: int = 24
    n_head: int = 16
    d_model: int = 1024
    d_mlp: int = 4096
    vocab_size: int = 30522
    padded_vocab: int = 30592  # multiple of 128
    max_pos: int = 512
    type_vocab: int = 2
    mask_token: int = 103
    mask_prob: float = 0.15

    @staticmethod
    def large() -> "BertConfig":
        return BertConfig()

    @staticmethod
    def base() -> "BertConfig":
        return BertConfig(n_layer=12, n_head=12, d_model=768, d_mlp=3072)

    @staticmethod
    def tiny() -> "BertConfig":
        return BertConfig(n_layer=2, n_head=4, d_model=128, d_mlp=512, vocab_size=1000, padded_vocab=1024, max_pos=64,
                          mask_token=3)


class EncoderBlock(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.n_head = cfg.n_head
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln1 = nn.LayerNorm(cfg.d_model, eps=1e-12)
        self.fc = nn.Linear(cfg.d_model, cfg.d_mlp)
        self.out = nn.Linear(cfg.d_mlp, cfg.d_model)
        self.ln2 = nn.LayerNorm(cfg.d_model, eps=1e-12)

    def forward(self, x: torch.Tensor, attn_mask: torch.Tensor | None) -> torch.Tensor:
        b, t, c = x.shape
        q, k, v = self.qkv(x).view(b, t, 3, self.n_head, c // self.n_head).unbind(dim=2)
        y = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=attn_mask)
        x = self.ln1(x + self.proj(y.transpose(1, 2).reshape(b, t, c)))
        return self.ln2(x + self.out(F.gelu(self.fc(x))))


class BertMLM(nn.Module):
    def __init__(self, cfg: BertConfig):
        super().__init__()
        self.cfg = cfg
        self.tok = nn.Embedding(cfg.padded_vocab, cfg.d_model)
        self.pos = nn.Embedding(cfg.max_pos, cfg.d_model)
        self.seg = nn.Embedding(cfg.type_vocab, cfg.d_model)
        self.ln_emb = nn.LayerNorm(cfg.d_model, eps=1e-12)
        self.blocks = nn.ModuleList([EncoderBlock(cfg) for _ in range(cfg.n_layer)])
        self.head_dense = nn.Linear(cfg.d_model, cfg.d_model)
        self.head_ln = nn.LayerNorm(cfg.d_model, eps=1e-12)
        self.head_bias = nn.Parameter(torch.zeros(cfg.padded_vocab))
        self.apply(self._init)

    @staticmethod
    def _init(m: nn.Module) -> None:
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def encode(self, ids: torch.Tensor, segments: torch.Tensor | None = None,
               padding_mask: torch.Tensor | None = None) -> torch.Tensor:
        b, t = ids.shape
        x = self.tok(ids) + self.pos(torch.arange(t, device=ids.device))
        x = x + self.seg(segments if segments is not None else torch.zeros_like(ids))
        x = self.ln_emb(x)
        mask = None if padding_mask is None else padding_mask[:, None, None, :].to(torch.bool)
        for blk in self.blocks:
            x = blk(x, mask)
        return x

    def forward(self, ids: torch.Tensor, labels: torch.Tensor | None = None, segments: torch.Tensor | None = None,
                padding_mask: torch.Tensor | None = None):
        """``labels`` holds the original token at masked positions and -100 elsewhere; returns the MLM
        loss (or the logits when ``labels`` is None)."""
        x = self.encode(ids, segments, padding_mask)
        if labels is not None:
            # only masked positions reach the vocabulary GEMM (15 % of the tokens)
            sel = labels.reshape(-1) != -100
            x = x.reshape(-1, x.size(-1))[sel]
            tgt = labels.reshape(-1)[sel]
        h = self.head_ln(F.gelu(self.head_dense(x)))
        logits = F.linear(h, self.tok.weight, self.head_bias)
        if labels is None:
            return logits
        from ..ops.fused_ce import fused_cross_entropy  # fused kernels for bf16 logits on a GPU, PyTorch's path otherwise

        return fused_cross_entropy(logits, tgt, self.cfg.vocab_size)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())


def mask_tokens(ids: torch.Tensor, cfg: BertConfig, generator: torch.Generator | None = None):
    """BERT's corruption: 15 % of the positions are selected; of those 80 % become [MASK], 10 % a random
    token, 10 % stay. Returns (corrupted ids, labels with -100 at unselected positions)."""
    r = torch.rand(ids.shape, device=ids.device, generator=generator)
    sel = r < cfg.mask_prob
    labels = torch.where(sel, ids, torch.full_like(ids, -100))
    r2 = torch.rand(ids.shape, device=ids.device, generator=generator)
    out = ids.clone()
    out[sel & (r2 < 0.8)] = cfg.mask_token
    rnd = torch.randint(0, cfg.vocab_size, ids.shape, device=ids.device, generator=generator)
    swap = sel & (r2 >= 0.8) & (r2 < 0.9)
    out[swap] = rnd[swap]
    return out, labels
