"""Single-token DSQG decode over per-layer circular K/V ring buffers.

The DWARF reference has no decode path (README.md:175-179 describes the O(1) cache in
prose; its generate() re-runs the whole prefix, train/train_2048_condU.py:463-487).
This module provides that cache: a ring of R = max(offsets)+1 slots per (sequence, head),
a write head per sequence, and one kernel launch per layer per token.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib
from .ops import OFFSETS_43, _dtype_code, _f32c, _ptr


def dsqg_decode_step(q, k_new, v_new, k_ring, v_ring, head, pos_bias, head_gain=None,
                     scale_embed=None, offsets: Sequence[int] = OFFSETS_43, fill=None, out=None, overlap=False):
    """One decode step for one layer.

    q, k_new, v_new [S,H,D]; k_ring, v_ring [S,H,R,D] (updated in place at slot head[s]);
    head int32 [S] on the device; fill int32 [S] (valid tokens incl. the new one) or None
    for a full ring.  Returns out [S,H,D].

    overlap=True launches the kernel so that its ring gather runs while the kernel ahead of it
    in the stream is still finishing (`dsqg_decode_overlapped`): allowed only when that kernel
    writes none of this call's head, fill, k_ring, v_ring.
    """
    lib = _lib.load()
    off, J = _lib.offsets_array(offsets)
    S, H, R, D = k_ring.shape
    for name, t in (("q", q), ("k_new", k_new), ("v_new", v_new)):
        if tuple(t.shape) != (S, H, D) or t.dtype != k_ring.dtype or not t.is_contiguous():
            raise ValueError(f"dsqg_decode: {name} must be contiguous [{S},{H},{D}] {k_ring.dtype}")
    if v_ring.shape != k_ring.shape or not (k_ring.is_contiguous() and v_ring.is_contiguous()):
        raise ValueError("dsqg_decode: k_ring and v_ring must be contiguous [S,H,R,D]")
    if head.dtype != torch.int32 or tuple(head.shape) != (S,):
        raise ValueError("dsqg_decode: head must be int32 [S]")
    if fill is not None and (fill.dtype != torch.int32 or tuple(fill.shape) != (S,)):
        raise ValueError("dsqg_decode: fill must be int32 [S]")
    if tuple(pos_bias.shape) != (J, H):
        raise ValueError(f"dsqg_decode: pos_bias must be [{J},{H}]")
    pb, hg, se = _f32c(pos_bias), _f32c(head_gain), _f32c(scale_embed)
    if out is None:
        out = torch.empty_like(q)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        entry = lib.dsqg_decode_overlapped if overlap else lib.dsqg_decode
        _lib.check(entry(q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
                         k_ring.data_ptr(), v_ring.data_ptr(), head.data_ptr(), _ptr(fill),
                         pb.data_ptr(), _ptr(se), _ptr(hg), off, J, R,
                         out.data_ptr(), S, H, D, _dtype_code(q), stream), "dsqg_decode")
    return out


def dsqg_decode_step_kv(q, k_new, v_new, kv_ring, head, pos_bias, head_gain=None, scale_embed=None,
                        offsets: Sequence[int] = OFFSETS_43, fill=None, out=None, overlap=False):
    """dsqg_decode_step over one ring that holds key and value of a slot side by side:
    kv_ring [S,H,R,2,D] (updated in place).  A tap is one contiguous read of 2*D elements."""
    lib = _lib.load()
    off, J = _lib.offsets_array(offsets)
    S, H, R, two, D = kv_ring.shape
    if two != 2 or not kv_ring.is_contiguous():
        raise ValueError("dsqg_decode_kv: kv_ring must be contiguous [S,H,R,2,D]")
    for name, t in (("q", q), ("k_new", k_new), ("v_new", v_new)):
        if tuple(t.shape) != (S, H, D) or t.dtype != kv_ring.dtype or not t.is_contiguous():
            raise ValueError(f"dsqg_decode_kv: {name} must be contiguous [{S},{H},{D}] {kv_ring.dtype}")
    if head.dtype != torch.int32 or tuple(head.shape) != (S,):
        raise ValueError("dsqg_decode_kv: head must be int32 [S]")
    if fill is not None and (fill.dtype != torch.int32 or tuple(fill.shape) != (S,)):
        raise ValueError("dsqg_decode_kv: fill must be int32 [S]")
    if tuple(pos_bias.shape) != (J, H):
        raise ValueError(f"dsqg_decode_kv: pos_bias must be [{J},{H}]")
    pb, hg, se = _f32c(pos_bias), _f32c(head_gain), _f32c(scale_embed)
    if out is None:
        out = torch.empty_like(q)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        _lib.check(lib.dsqg_decode_kv(q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), kv_ring.data_ptr(),
                                      head.data_ptr(), _ptr(fill), pb.data_ptr(), _ptr(se), _ptr(hg), off, J, R,
                                      out.data_ptr(), S, H, D, _dtype_code(q), stream, int(overlap)), "dsqg_decode_kv")
    return out


class DSQGRingCache:
    """K/V rings for L layers, one shared write head per sequence.  interleaved=True (default) keeps
    key and value of a slot side by side in one tensor kv [L,S,H,R,2,D] (a tap is one contiguous
    read; `k` and `v` are strided views of it); interleaved=False keeps two tensors k, v [L,S,H,R,D]."""

    def __init__(self, layers, sequences, heads, head_dim, offsets: Sequence[int] = OFFSETS_43,
                 dtype=torch.bfloat16, device="cuda", interleaved=True):
        self.offsets = tuple(int(o) for o in offsets)
        self.R = max(self.offsets) + 1
        self.interleaved = interleaved
        if interleaved:
            self.kv = torch.zeros(layers, sequences, heads, self.R, 2, head_dim, dtype=dtype, device=device)
            self.k, self.v = self.kv[..., 0, :], self.kv[..., 1, :]
        else:
            self.kv = None
            self.k = torch.zeros(layers, sequences, heads, self.R, head_dim, dtype=dtype, device=device)
            self.v = torch.zeros_like(self.k)
        self.head = torch.full((sequences,), -1, dtype=torch.int32, device=device)
        self.fill = torch.zeros(sequences, dtype=torch.int32, device=device)

    def prefill(self, layer, k, v):
        """Load the rings of `layer` from a prefix in training layout: k, v [S,H,N,D].  Sets head
        and fill for the whole cache (call it with the same N for every layer)."""
        lib = _lib.load()
        S, H, N, D = k.shape
        if tuple(self.k[layer].shape) != (S, H, self.R, D) or k.dtype != self.k.dtype or v.shape != k.shape:
            raise ValueError("dsqg ring prefill: k, v must be [S,H,N,D] matching the cache")
        k, v = k.contiguous(), v.contiguous()
        with torch.cuda.device(k.device):
            stream = torch.cuda.current_stream(k.device).cuda_stream
            if self.interleaved:
                _lib.check(lib.dsqg_ring_prefill_kv(k.data_ptr(), v.data_ptr(), self.kv[layer].data_ptr(),
                                                    self.head.data_ptr(), self.fill.data_ptr(),
                                                    S, H, N, D, self.R, _dtype_code(k), stream), "dsqg_ring_prefill_kv")
                return
            _lib.check(lib.dsqg_ring_prefill(k.data_ptr(), v.data_ptr(), self.k[layer].data_ptr(),
                                             self.v[layer].data_ptr(), self.head.data_ptr(), self.fill.data_ptr(),
                                             S, H, N, D, self.R, _dtype_code(k), stream), "dsqg_ring_prefill")

    def advance(self):
        """Move every write head to the next slot; call once per token before the layers run."""
        self.head = torch.remainder(self.head + 1, self.R).to(torch.int32)
        self.fill = torch.clamp(self.fill + 1, max=self.R).to(torch.int32)

    def step(self, layer, q, k_new, v_new, pos_bias, head_gain=None, scale_embed=None, out=None, overlap=False):
        """Decode step of `layer`.  overlap=True is safe from the second layer of a token on (the
        kernel ahead is then another layer's step or a projection, never `advance`/`prefill`)."""
        if self.interleaved:
            return dsqg_decode_step_kv(q, k_new, v_new, self.kv[layer], self.head, pos_bias,
                                       head_gain, scale_embed, self.offsets, self.fill, out, overlap)
        return dsqg_decode_step(q, k_new, v_new, self.k[layer], self.v[layer], self.head, pos_bias,
                                head_gain, scale_embed, self.offsets, self.fill, out, overlap)
