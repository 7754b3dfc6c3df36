"""GPT-2 (decoder-only transformer) for the bf16 data-parallel configuration: 24 layers,
d_model 1024, 16 heads, FFN 4096, vocabulary 50257, sequence 1024 ("medium"). Plain torch.nn on
cuBLAS and the fused attention of `scaled_dot_product_attention`; the library under test is the
bucketed bf16 gradient reduction with the AdamW update fused behind it."""
from __future__ import annotations

import dataclasses

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclasses.dataclass
class GPT2Config:
    n_layer: int = 24
    d_model: int = 1024
    n_head: int = 16
    d_ff: int = 4096
    vocab: int = 50257
    seq_len: int = 1024


class Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.ln1 = nn.LayerNorm(cfg.d_model)
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln2 = nn.LayerNorm(cfg.d_model)
        self.fc1 = nn.Linear(cfg.d_model, cfg.d_ff)
        self.fc2 = nn.Linear(cfg.d_ff, cfg.d_model)
        self.n_head = cfg.n_head

    def forward(self, x):
        b, t, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, t, 3, self.n_head, d // self.n_head).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, t, d))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config = GPT2Config()):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab, cfg.d_model)
        self.wpe = nn.Embedding(cfg.seq_len, cfg.d_model)
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = nn.LayerNorm(cfg.d_model)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, idx):
        b, t = idx.shape
        x = self.wte(idx) + self.wpe(torch.arange(t, device=idx.device))
        for blk in self.blocks:
            x = blk(x)
        return F.linear(self.ln_f(x), self.wte.weight)   # tied output embedding

    def loss(self, idx):
        logits = self.forward(idx[:, :-1])
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), idx[:, 1:].reshape(-1))


def synthetic_batch(cfg: GPT2Config, batch: int, device, generator=None, pin: bool = False):
    idx = torch.randint(0, cfg.vocab, (batch, cfg.seq_len + 1), generator=generator)
    return (idx.pin_memory(),) if pin else (idx.to(device),)
