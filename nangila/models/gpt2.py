"""GPT-2 (decoder-only transformer with learned positions, pre-LayerNorm, GELU MLP, tied
embeddings) for the DDP throughput benchmark and the loss-parity tests.

The reference ships no model; its examples train Hugging Face causal LMs through DDP
(examples/train_llm.py:230-332). This definition is the "GPT-2 small" of the headline benchmark:
12 layers, d_model 768, 12 heads, MLP 3072, vocabulary 50257, context 1024.

GEMMs go to cuBLAS through ``torch.nn.functional.linear`` and attention to the fused
``scaled_dot_product_attention`` kernel; the loss over the padded vocabulary is this framework's fused
cross-entropy kernel pair (``nangila/ops/fused_ce.py``); the gradient exchange is what this framework replaces.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import fused_grads as FG


@dataclass
class GPT2Config:
    n_layer: int = 12
    n_head: int = 12
    d_model: int = 768
    d_mlp: int = 3072
    vocab_size: int = 50257
    n_ctx: int = 1024
    padded_vocab: int = 50304  # multiple of 128: keeps the LM-head GEMM on aligned tiles

    @staticmethod
    def small() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(n_layer=2, n_head=4, d_model=128, d_mlp=512, vocab_size=1000, n_ctx=128, padded_vocab=1024)


class Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.n_head = cfg.n_head
        self.ln1 = nn.LayerNorm(cfg.d_model)
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln2 = nn.LayerNorm(cfg.d_model)
        self.fc = nn.Linear(cfg.d_model, cfg.d_mlp)
        self.out = nn.Linear(cfg.d_mlp, cfg.d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # same modules and parameters as plain nn.Linear / nn.LayerNorm calls; with NANGILA_FUSED_GRADS=1 the bias and
        # LayerNorm parameter gradients of bf16 CUDA tensors come from the column-sum kernel (nangila/ops/fused_grads.py)
        b, t, c = x.shape
        qkv = FG.linear(FG.layer_norm(x, self.ln1), self.qkv).view(b, t, 3, self.n_head, c // self.n_head)
        q, k, v = qkv.unbind(dim=2)
        y = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + FG.linear(y.transpose(1, 2).reshape(b, t, c), self.proj)
        x = x + FG.linear(F.gelu(FG.linear(FG.layer_norm(x, self.ln2), self.fc), approximate="tanh"), self.out)
        return x


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.padded_vocab, cfg.d_model)
        self.wpe = nn.Embedding(cfg.n_ctx, cfg.d_model)
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(cfg.n_layer)])
        self.ln_f = nn.LayerNorm(cfg.d_model)
        self.apply(self._init)
        for blk in self.blocks:  # GPT-2's scaled init of the residual projections
            for lin in (blk.proj, blk.out):
                nn.init.normal_(lin.weight, std=0.02 / math.sqrt(2 * cfg.n_layer))

    @staticmethod
    def _init(m: nn.Module) -> None:
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, std=0.02)

    def forward(self, idx: torch.Tensor, targets: torch.Tensor | None = None):
        b, t = idx.shape
        pos = torch.arange(t, device=idx.device)
        x = self.wte(idx) + self.wpe(pos)
        for blk in self.blocks:
            x = blk(x)
        x = FG.layer_norm(x, self.ln_f)
        logits = F.linear(x, self.wte.weight)  # tied head over the padded vocabulary
        if targets is None:
            return logits
        # the padded columns are excluded from the softmax, so the model has exactly `vocab_size` classes;
        # bf16 logits on a GPU take the fused kernel pair (no fp32 copy of the logits), the rest PyTorch's path
        from ..ops.fused_ce import fused_cross_entropy

        return fused_cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1), self.cfg.vocab_size)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())
