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

from .modules import DSQGAttentionN_Fused, DSQGAttentionQW
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

    def attend(self, x):
        B, N, D = x.shape
        q, k, v = (t.view(B, N, self.heads, D // self.heads).transpose(1, 2) for t in self.qkv_proj(x).split(D, -1))
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.out_proj(o.transpose(1, 2).reshape(B, N, D)), k, v

    def forward(self, x):
        return self.attend(x)[0]

    def decode(self, x, k_cache, v_cache, t):
        """x [S,D]: token at position t; k_cache, v_cache [S,H,T,HD] hold positions < t and
        receive this token's k, v (this layer's cache grows with the sequence)."""
        S, D = x.shape
        q, k, v = (u.view(S, self.heads, 1, D // self.heads) for u in self.qkv_proj(x).split(D, -1))
        k_cache[:, :, t:t + 1] = k
        v_cache[:, :, t:t + 1] = v
        o = F.scaled_dot_product_attention(q.to(k_cache.dtype), k_cache[:, :, :t + 1], v_cache[:, :, :t + 1])
        return self.out_proj(o.reshape(S, D).to(x.dtype))


class Block(nn.Module):
    def __init__(self, dim, heads, ffn, seq_len, full_attention, offsets, attention="condM"):
        super().__init__()
        self.norm1, self.norm2 = RMSNorm(dim), RMSNorm(dim)
        dsqg_cls = {"condM": DSQGAttentionN_Fused, "condU": DSQGAttentionQW}[attention]
        self.attn = FullCausalAttention(dim, heads) if full_attention else \
            dsqg_cls(dim, heads, seq_len=seq_len, dropout=0.0, offsets=offsets)
        self.ffn = FFN(dim, ffn)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.ffn(self.norm2(x))

    def forward_kv(self, x):
        y, k, v = self.attn.attend(self.norm1(x))
        x = x + y
        return x + self.ffn(self.norm2(x)), k, v


class CondMLM(nn.Module):
    """attention = "condM": DSQG layers with the position bias only (the reference's condM,
    kernels/dsqg_attention_v2.py:434-477) -- the shape the end-to-end benchmark configuration names;
    "condU": with scale_embed and the per-head gain (train/train_2048_condU.py:116-205)."""

    def __init__(self, vocab=32000, dim=256, heads=8, layers=6, ffn=1024, seq_len=2048,
                 full_attention_layer=5, offsets=OFFSETS_43, attention="condM"):
        super().__init__()
        self.embedding = nn.Embedding(vocab, dim)
        self.pos_embed = nn.Embedding(seq_len, dim)
        self.blocks = nn.ModuleList(Block(dim, heads, ffn, seq_len, i == full_attention_layer, offsets, attention)
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

    # ---- incremental decoding over the O(1) DSQG rings -------------------------------------
    # The reference's generate() re-runs the model on the whole prefix for every new token
    # (train/train_2048_condU.py:463-487) and describes the cache only in prose (README.md:175-179):
    # a DSQG layer needs the last max(offset)+1 keys/values, the one full-attention layer keeps all.

    @torch.no_grad()
    def prefill(self, ids, max_len=None):
        """Runs the prompt ids [S,N] through the model, fills the decode caches from the k, v every
        layer computed and returns (logits of the last position [S,vocab], state)."""
        from .decode import DSQGRingCache
        S, N = ids.shape
        max_len = self.pos_embed.num_embeddings if max_len is None else max_len
        dsqg_blocks = [i for i, b in enumerate(self.blocks) if not isinstance(b.attn, FullCausalAttention)]
        first = self.blocks[dsqg_blocks[0]].attn
        cache = DSQGRingCache(len(dsqg_blocks), S, first.num_heads, first.head_dim, first._offsets,
                              dtype=torch.bfloat16, device=ids.device)
        state = {"cache": cache, "ring_of": {b: i for i, b in enumerate(dsqg_blocks)}, "t": N, "full": {}}
        x = self.embedding(ids) + self.pos_embed(torch.arange(N, device=ids.device))[None]
        for i, blk in enumerate(self.blocks):
            x, k, v = blk.forward_kv(x)
            if i in state["ring_of"]:
                cache.prefill(state["ring_of"][i], k, v)
            else:
                kc = torch.zeros(S, k.shape[1], max_len, k.shape[3], dtype=k.dtype, device=k.device)
                vc = torch.zeros_like(kc)
                kc[:, :, :N] = k
                vc[:, :, :N] = v
                state["full"][i] = (kc, vc)
        return F.linear(self.norm(x[:, -1]), self.embedding.weight), state

    @torch.no_grad()
    def decode_token(self, ids_t, state):
        """ids_t [S]: the token at position state["t"] of every sequence -> logits [S,vocab]."""
        t = state["t"]
        if t >= self.pos_embed.num_embeddings:
            raise ValueError("decode_token: position beyond the model's seq_len")
        cache = state["cache"]
        cache.advance()
        x = self.embedding(ids_t) + self.pos_embed.weight[t]
        for i, blk in enumerate(self.blocks):
            h = blk.norm1(x)
            if i in state["ring_of"]:
                # the kernel ahead of the step is this layer's projection, never a writer of the rings
                # or the write head, so the overlapped launch is allowed
                x = x + blk.attn.decode(h, cache, state["ring_of"][i], overlap=True)
            else:
                x = x + blk.attn.decode(h, *state["full"][i], t)
            x = x + blk.ffn(blk.norm2(x))
        state["t"] = t + 1
        return F.linear(self.norm(x), self.embedding.weight)

    @torch.no_grad()
    def generate(self, ids, max_new_tokens, temperature=0.0, generator=None):
        """Greedy (temperature 0) or sampled continuation of ids [S,N]: one prefill, then one
        decode_token per new token.  Returns [S, N + max_new_tokens]."""
        logits, state = self.prefill(ids, max_len=ids.shape[1] + max_new_tokens)
        out = [ids]
        for step in range(max_new_tokens):
            if temperature > 0:
                nxt = torch.multinomial(torch.softmax(logits.float() / temperature, -1), 1, generator=generator)[:, 0]
            else:
                nxt = logits.argmax(-1)
            out.append(nxt[:, None])
            if step + 1 < max_new_tokens:
                logits = self.decode_token(nxt, state)
        return torch.cat(out, 1)
