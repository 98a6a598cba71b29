"""Drop-in operator functions and attention modules with the DWARF reference's names.

* ``dsqg_attention_v2(q, k, v, pos_bias)``               kernels/dsqg_attention_v2.py:417-427
* ``dsqg_attention_v3(q, k, v, pos_bias, scale_embed)``  kernels/dsqg_attention_v3.py:445-456
* ``DSQGAttentionN_Fused``                               kernels/dsqg_attention_v2.py:434-477
* ``DSQGAttentionV3``                                    kernels/dsqg_attention_v3.py:463-536
* ``DSQGAttentionQW`` (V3 + per-head ``if_gain``)        train/train_2048_condU.py:116-205

Parameter names and shapes (``qkv_proj``, ``out_proj``, ``gate_proj``, ``pos_bias [J,H]``,
``scale_embed [J,HD]``, ``if_gain [H]``) match the reference so its state dicts load.
Unlike the reference, any ascending offset set is accepted and the ``if_gain`` multiply is
fused into the kernel epilogue.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn as nn

from .ops import (ALL_OFFSETS, InjectKVFunction, causal_mean, dsqg_attention, dsqg_attention_packed,
                  packed_path_available)


def dsqg_attention_v2(q, k, v, pos_bias, offsets: Sequence[int] = ALL_OFFSETS):
    """condM op.  q, k, v [B,H,N,HD] (non-bf16 inputs are computed in bf16 and the result is
    cast back, as in the reference); pos_bias [J,H] fp32."""
    orig = q.dtype
    if orig != torch.bfloat16:
        q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    out = dsqg_attention(q, k, v, pos_bias, None, None, offsets)
    return out if orig == torch.bfloat16 else out.to(orig)


def dsqg_attention_v3(q, k, v, pos_bias, scale_embed, offsets: Sequence[int] = ALL_OFFSETS):
    """condU op: adds the Q-weighted scale term q.scale_embed[j]/sqrt(HD) to every score."""
    orig = q.dtype
    if orig != torch.bfloat16:
        q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    out = dsqg_attention(q, k, v, pos_bias, None, scale_embed, offsets)
    return out if orig == torch.bfloat16 else out.to(orig)


def _log_linear_bias(offsets, num_heads):
    # pos_bias[j,h] = -log(1+delta_j) * alpha_h  (kernels/dsqg_attention_v2.py:454-456)
    alphas = torch.linspace(0.2, 2.0, num_heads)
    logs = torch.tensor([math.log(1.0 + d) for d in offsets], dtype=torch.float32)
    return -logs[:, None] * alphas[None, :]


class _DSQGAttentionBase(nn.Module):
    """qkv projection -> DSQG op -> sigmoid gate -> output projection."""

    def __init__(self, embedding_dim, num_heads, seq_len=2048, offsets=None, dropout=0.1,
                 gate_bias=2.0, with_scale_embed=False, with_if_gain=False, offsets_in_state_dict=True):
        super().__init__()
        if embedding_dim % num_heads:
            raise ValueError("embedding_dim must be divisible by num_heads")
        self.embedding_dim, self.num_heads = embedding_dim, num_heads
        self.head_dim = embedding_dim // num_heads
        self.seq_len = seq_len
        offsets = list(ALL_OFFSETS if offsets is None else offsets)
        # the kernel-file modules of the reference keep `offsets` in their state dict
        # (kernels/dsqg_attention_v2.py:448, kernels/dsqg_attention_v3.py:488); its condU script module does not
        self.register_buffer("offsets", torch.tensor(offsets, dtype=torch.long), persistent=offsets_in_state_dict)
        self._offsets = tuple(offsets)
        self.n_offsets = len(offsets)
        self.qkv_proj = nn.Linear(embedding_dim, 3 * embedding_dim, bias=True)
        self.out_proj = nn.Linear(embedding_dim, embedding_dim, bias=True)
        self.gate_proj = nn.Linear(embedding_dim, embedding_dim, bias=True)
        nn.init.constant_(self.gate_proj.bias, gate_bias)
        self.pos_bias = nn.Parameter(_log_linear_bias(offsets, num_heads))
        if with_scale_embed:
            self.scale_embed = nn.Parameter(torch.zeros(self.n_offsets, self.head_dim))
        if with_if_gain:
            self.if_gain = nn.Parameter(torch.ones(num_heads))
        self.dropout = nn.Dropout(dropout)
        self._packed = None            # decided on first use: can the copy-free path take this layer?

    def _project_heads(self, x):
        """x [B,N,D] -> q, k, v [B,H,N,HD] contiguous."""
        B, N, D = x.shape
        H, HD = self.num_heads, self.head_dim
        return tuple(t.view(B, N, H, HD).permute(0, 2, 1, 3).contiguous()
                     for t in self.qkv_proj(x).split(D, dim=-1))

    def _packed_ok(self, qkv):
        """The copy-free path applies to bf16 activations (autocast) and head widths / offset sets
        the tensor-core kernels take (with scale_embed: head widths up to 64)."""
        if qkv.dtype != torch.bfloat16 or not qkv.is_cuda:
            return False
        if self._packed is None:
            self._packed = packed_path_available(self.head_dim, self._offsets, hasattr(self, "scale_embed"))
        return self._packed

    def attend(self, x, kv_inject=None):
        """The layer's output together with the k, v [B,H,N,HD] bf16 the op saw (what a decode
        cache has to be filled with)."""
        B, N, D = x.shape
        qkv = self.qkv_proj(x)
        if self._packed_ok(qkv):
            # q, k, v are read in place from the projection output, the result comes back
            # token-major and already gated: none of the reference's permute copies
            # (train/train_2048_condU.py:171-175,189-191) is made
            H, HD = self.num_heads, self.head_dim
            qkv = qkv.contiguous()
            if kv_inject is not None:
                # Huygens K/V injection (train_2048_condU.py:178-181) as two in-place adds on the key and
                # value thirds of the projection output; the deltas arrive [B,H,N,HD] (permuted views of
                # token-major projections cost nothing to bring back)
                if qkv._is_view():          # an in-place autograd function needs a tensor that owns its history
                    qkv = qkv.clone()
                qkv = InjectKVFunction.apply(qkv, kv_inject[0].permute(0, 2, 1, 3).reshape(B, N, D),
                                             kv_inject[1].permute(0, 2, 1, 3).reshape(B, N, D))
            qkv5 = qkv.view(B, N, 3, H, HD)
            gate = self.gate_proj(x)
            y = dsqg_attention_packed(qkv5, self.pos_bias, getattr(self, "if_gain", None),
                                      gate.to(torch.bfloat16), self._offsets, getattr(self, "scale_embed", None))
            return (self.dropout(self.out_proj(y)), qkv5[:, :, 1].permute(0, 2, 1, 3), qkv5[:, :, 2].permute(0, 2, 1, 3))
        H, HD = self.num_heads, self.head_dim
        q, k, v = (t.view(B, N, H, HD).permute(0, 2, 1, 3).contiguous() for t in qkv.split(D, dim=-1))
        if kv_inject is not None:          # Huygens K/V injection, train_2048_condU.py:178-181
            k = k + kv_inject[0]
            v = v + kv_inject[1]
        orig = q.dtype
        if orig != torch.bfloat16:
            q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
        out = dsqg_attention(q, k, v, self.pos_bias, getattr(self, "if_gain", None),
                             getattr(self, "scale_embed", None), self._offsets)
        out = out if orig == torch.bfloat16 else out.to(orig)
        flat = out.permute(0, 2, 1, 3).reshape(B, N, D)
        return self.dropout(self.out_proj(flat * torch.sigmoid(self.gate_proj(x)))), k, v

    def forward(self, x, kv_inject=None):
        return self.attend(x, kv_inject)[0]

    def decode(self, x, cache, layer, overlap=False):
        """One new token per sequence: x [S,D] -> [S,D], reading the previous tokens' k, v from
        ring `layer` of `cache` (a DSQGRingCache whose `advance()` ran for this token) and storing
        this token's there.  The reference has no such path: its generate() re-runs the whole
        prefix (train/train_2048_condU.py:463-487)."""
        S, D = x.shape
        H, HD = self.num_heads, self.head_dim
        q, k, v = (t.reshape(S, H, HD).to(cache.k.dtype).contiguous() for t in self.qkv_proj(x).split(D, dim=-1))
        out = cache.step(layer, q, k, v, self.pos_bias, getattr(self, "if_gain", None),
                         getattr(self, "scale_embed", None), overlap=overlap)
        flat = out.reshape(S, D).to(x.dtype)
        return self.out_proj(flat * torch.sigmoid(self.gate_proj(x)))

    def attn_summary(self):
        with torch.no_grad():
            pb = self.pos_bias.detach().float().cpu()
            info = {"pos_bias_abs_mean": pb.abs().mean().item(),
                    "pos_bias_abs_max": pb.abs().max().item(),
                    "pos_bias_mean_per_head": pb.mean(0).tolist()}
            if hasattr(self, "scale_embed"):
                se = self.scale_embed.detach().float().cpu()
                info["scale_embed_abs_mean"] = se.abs().mean().item()
                info["scale_embed_abs_max"] = se.abs().max().item()
            if hasattr(self, "if_gain"):
                info["if_gain"] = self.if_gain.detach().float().cpu().tolist()
        return info


class DSQGAttentionN_Fused(_DSQGAttentionBase):
    """condM attention (pos_bias only; gate bias 2.0)."""

    def __init__(self, embedding_dim, num_heads, seq_len=2048, offsets=None, dropout=0.1):
        super().__init__(embedding_dim, num_heads, seq_len, offsets, dropout, gate_bias=2.0)

    def forward(self, x):                      # the reference signature has no kv_inject here
        return super().forward(x)


class DSQGAttentionV3(_DSQGAttentionBase):
    """condU attention: pos_bias + scale_embed (zero-init), gate bias 0."""

    def __init__(self, embedding_dim, num_heads, seq_len=2048, offsets=None, dropout=0.1):
        super().__init__(embedding_dim, num_heads, seq_len, offsets, dropout, gate_bias=0.0,
                         with_scale_embed=True)


class DSQGAttentionQW(_DSQGAttentionBase):
    """condU attention with the per-head IF gain; the gain multiply runs inside the kernel.
    As in the reference script (train/train_2048_condU.py:139-166) the state dict holds no
    `offsets` entry, so its checkpoints load with strict=True."""

    def __init__(self, embedding_dim, num_heads, seq_len=2048, dropout=0.1, offsets=None):
        super().__init__(embedding_dim, num_heads, seq_len, offsets, dropout, gate_bias=0.0,
                         with_scale_embed=True, with_if_gain=True, offsets_in_state_dict=False)


class InterferenceInjection(nn.Module):
    """The K/V deltas of the condU "interference" block (train/train_2048_condU.py:277-295): a
    gated causal running mean of the normalised block input, projected to key and value space.
    Parameter names match the reference block (`inter_norm`, `inter_gate`, `inter_k_proj`,
    `inter_v_proj`).  forward(x [B,N,D]) returns (k_delta, v_delta), each [B,H,N,HD], ready for
    `DSQGAttentionQW.forward(x, kv_inject=...)`; the pooling runs as one scan kernel."""

    def __init__(self, embedding_dim, num_heads):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, embedding_dim // num_heads
        self.inter_norm = nn.LayerNorm(embedding_dim)
        self.inter_gate = nn.Linear(embedding_dim, embedding_dim)
        self.inter_k_proj = nn.Linear(embedding_dim, embedding_dim)
        self.inter_v_proj = nn.Linear(embedding_dim, embedding_dim)

    def forward(self, x):
        xi = self.inter_norm(x)
        B, N, D = xi.shape
        H, HD = self.num_heads, self.head_dim
        pool = causal_mean(xi)                                  # xi.cumsum(dim=1) / counts
        inter = torch.sigmoid(self.inter_gate(xi)) * pool
        k_delta = self.inter_k_proj(inter).view(B, N, H, HD).permute(0, 2, 1, 3)
        v_delta = self.inter_v_proj(inter).view(B, N, H, HD).permute(0, 2, 1, 3)
        return k_delta, v_delta
