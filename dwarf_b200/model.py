"""condM-shaped hybrid language model used by the end-to-end training benchmark.

Mirrors the shape of the reference's CondMTransformer (train/train_2048_condU.py:320-365:
token + position embedding, N blocks, final norm, tied lm_head) with DSQG attention in all
layers but one and full causal softmax attention in the remaining one
(train/train_2048_condM_layer_ablation.py:214-286).  Per the benchmark specification the
norms are RMSNorm and the FFN is GELU; weights are N(0, 0.02).  This is a benchmark
vehicle for the DSQG op, not a re-implementation of the reference's training scripts.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .modules import DSQGAttentionQW
from .ops import OFFSETS_43


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


class FFN(nn.Module):
    def __init__(self, dim, hidden):
        super().__init__()
        self.fc1 = nn.Linear(dim, hidden)
        self.fc2 = nn.Linear(hidden, dim)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x)))


class FullCausalAttention(nn.Module):
    """The one full-attention layer (F.scaled_dot_product_attention, as in the reference)."""

    def __init__(self, dim, heads):
        super().__init__()
        self.heads = heads
        self.qkv_proj = nn.Linear(dim, 3 * dim)
        self.out_proj = nn.Linear(dim, dim)

    def forward(self, x):
        B, N, D = x.shape
        q, k, v = (t.view(B, N, self.heads, D // self.heads).transpose(1, 2) for t in self.qkv_proj(x).split(D, -1))
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.out_proj(o.transpose(1, 2).reshape(B, N, D))


class Block(nn.Module):
    def __init__(self, dim, heads, ffn, seq_len, full_attention, offsets):
        super().__init__()
        self.norm1, self.norm2 = RMSNorm(dim), RMSNorm(dim)
        self.attn = FullCausalAttention(dim, heads) if full_attention else \
            DSQGAttentionQW(dim, heads, seq_len=seq_len, dropout=0.0, offsets=offsets)
        self.ffn = FFN(dim, ffn)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.ffn(self.norm2(x))


class CondMLM(nn.Module):
    def __init__(self, vocab=32000, dim=256, heads=8, layers=6, ffn=1024, seq_len=2048,
                 full_attention_layer=5, offsets=OFFSETS_43):
        super().__init__()
        self.embedding = nn.Embedding(vocab, dim)
        self.pos_embed = nn.Embedding(seq_len, dim)
        self.blocks = nn.ModuleList(Block(dim, heads, ffn, seq_len, i == full_attention_layer, offsets)
                                    for i in range(layers))
        self.norm = RMSNorm(dim)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, 0.0, 0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    def forward(self, ids):
        B, N = ids.shape
        x = self.embedding(ids) + self.pos_embed(torch.arange(N, device=ids.device))[None]
        for blk in self.blocks:
            x = blk(x)
        return F.linear(self.norm(x), self.embedding.weight)       # tied lm_head
