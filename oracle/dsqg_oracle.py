"""CPU oracle for DSQG attention -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

This file restates, in plain PyTorch on the CPU, the algorithm of the DWARF
reference's pure-PyTorch DSQG path.  It exists only so that the CUDA kernels of
``dwarf_b200`` can be checked against the reference's arithmetic.  Nothing in
the ``dwarf_b200`` package imports it; only the test-suite, the smoke check and
the CPU-baseline leg of the benchmark do.

Reference functions followed (paths relative to the DWARF repository):

* ``kernels/dsqg_attention_v2.py:484-497``  ``_reference``      (condM op)
* ``kernels/dsqg_attention_v3.py:543-561``  ``_reference_v3``   (condU op,
  adds the Q-weighted ``scale_embed`` term)
* ``train/train_2048_condU.py:187``         per-head ``if_gain`` on the output
* ``train/train_2048_condM_layer_ablation.py:106-130`` the same math written
  with shifted copies of K and V (second, independent statement)

The reference hard-codes its 44-offset set and the padding 1536.  The only
generalisation made here is that the offset list is an argument and the padding
is ``max(offsets)``; for the 44-offset set the result is bit-identical to the
reference functions (pinned by ``tests/golden/make_golden.py``, which imports
the reference itself, and by ``tests/test_oracle_golden.py``).

Parity status: PINNED against outputs of the reference's own functions
(committed under ``tests/golden/``).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

# Offset sets (reference: kernels/dsqg_attention_v3.py:47-49).
SPARSE_TAPS = [48, 64, 96, 128, 192, 256, 384, 512, 768, 1024, 1536]
OFFSETS_44 = list(range(33)) + SPARSE_TAPS            # what the reference code uses
OFFSETS_43 = list(range(32)) + SPARSE_TAPS            # dense 0..31 (benchmark configs)
OFFSETS_45 = OFFSETS_43 + [2048, 3072]                # N=4096 configuration


def index_mask_oracle(N: int, offsets: Sequence[int]):
    """Integer part of the op: source row ``n - delta_j`` and validity ``n >= delta_j``.

    Follows the gather index / mask of ``kernels/dsqg_attention_v2.py:491,495``.
    Returns ``(src [N,J] int64, valid [N,J] bool)``; ``src`` is -1 where invalid.
    """
    off = torch.tensor(list(offsets), dtype=torch.long)
    ni = torch.arange(N, dtype=torch.long)
    src = ni[:, None] - off[None, :]
    valid = src >= 0
    return torch.where(valid, src, torch.full_like(src, -1)), valid


def dsqg_reference(q, k, v, pos_bias, scale_embed=None, head_gain=None,
                   offsets: Sequence[int] = OFFSETS_44, compute_dtype=torch.float32):
    """Pure-PyTorch DSQG forward, line for line ``_reference_v3`` with an offsets argument.

    q, k, v      [B,H,N,HD]; pos_bias [J,H]; scale_embed [J,HD] or None;
    head_gain    [H] or None (multiplies the output, train_2048_condU.py:187).
    Differentiable through autograd; the autograd gradient is the gradient oracle
    (as in kernels/dsqg_attention_v2.py:526-528).
    Returns the output in ``compute_dtype`` (the reference's final ``.to(q.dtype)``
    is left to the caller so that fp32 results can be compared before rounding).
    """
    B, H, N, HD = q.shape
    sc = HD ** -0.5
    off = torch.tensor(list(offsets), device=q.device, dtype=torch.long)
    pad = int(max(offsets)) if len(offsets) else 0
    qf = q.to(compute_dtype)
    kp = F.pad(k.to(compute_dtype), (0, 0, pad, 0))
    vp = F.pad(v.to(compute_dtype), (0, 0, pad, 0))
    ni = torch.arange(N, device=q.device)
    gi = pad - off[None, :] + ni[:, None]
    Ka = kp[:, :, gi, :]
    Va = vp[:, :, gi, :]
    s = (qf.unsqueeze(3) * Ka).sum(-1) * sc
    s = s + pos_bias.to(compute_dtype).T[None, :, None, :]
    if scale_embed is not None:
        q_dyn = (qf.unsqueeze(3) * scale_embed.to(compute_dtype)[None, None, :, :]).sum(-1) * sc
        s = s + q_dyn
    s = s.masked_fill((ni[:, None] < off[None, :]).unsqueeze(0).unsqueeze(0), float('-inf'))
    a = F.softmax(s, dim=-1)
    out = (a.unsqueeze(-1) * Va).sum(3)
    if head_gain is not None:
        out = out * head_gain.to(compute_dtype).view(1, H, 1, 1)
    return out


def dsqg_reference_chunked(q, k, v, pos_bias, scale_embed=None, head_gain=None,
                           offsets: Sequence[int] = OFFSETS_44, chunk: int = 2,
                           compute_dtype=torch.float32):
    """Forward only, batch processed in chunks so the [B,H,N,J,HD] gathers fit in RAM."""
    outs = []
    with torch.no_grad():
        for b0 in range(0, q.shape[0], chunk):
            sl = slice(b0, b0 + chunk)
            outs.append(dsqg_reference(q[sl], k[sl], v[sl], pos_bias, scale_embed, head_gain,
                                       offsets, compute_dtype))
    return torch.cat(outs, 0)


def dsqg_reference_grads(q, k, v, pos_bias, dout, scale_embed=None, head_gain=None,
                         offsets: Sequence[int] = OFFSETS_44, chunk: int = 2,
                         compute_dtype=torch.float32):
    """Forward + autograd backward of ``dsqg_reference`` with upstream gradient ``dout``.

    Returns a dict with out, dq, dk, dv, dpb and (when given) dse, dgain, all in
    ``compute_dtype``.  Processed in batch chunks; parameter gradients are summed.
    """
    res = {"out": [], "dq": [], "dk": [], "dv": []}
    dpb = torch.zeros_like(pos_bias, dtype=compute_dtype)
    dse = None if scale_embed is None else torch.zeros_like(scale_embed, dtype=compute_dtype)
    dg = None if head_gain is None else torch.zeros_like(head_gain, dtype=compute_dtype)
    for b0 in range(0, q.shape[0], chunk):
        sl = slice(b0, b0 + chunk)
        qc, kc, vc = (t[sl].detach().to(compute_dtype).requires_grad_(True) for t in (q, k, v))
        pb = pos_bias.detach().to(compute_dtype).requires_grad_(True)
        se = None if scale_embed is None else scale_embed.detach().to(compute_dtype).requires_grad_(True)
        g = None if head_gain is None else head_gain.detach().to(compute_dtype).requires_grad_(True)
        o = dsqg_reference(qc, kc, vc, pb, se, g, offsets, compute_dtype)
        o.backward(dout[sl].to(compute_dtype))
        res["out"].append(o.detach()); res["dq"].append(qc.grad)
        res["dk"].append(kc.grad); res["dv"].append(vc.grad)
        dpb += pb.grad
        if se is not None: dse += se.grad
        if g is not None: dg += g.grad
    out = {name: torch.cat(parts, 0) for name, parts in res.items()}
    out["dpb"] = dpb
    if dse is not None: out["dse"] = dse
    if dg is not None: out["dgain"] = dg
    return out


def pos_bias_init(offsets: Sequence[int], num_heads: int):
    """``pos_bias[j,h] = -log(1+delta_j) * alpha_h``, alpha = linspace(0.2, 2.0, H).

    Follows kernels/dsqg_attention_v2.py:454-456.
    """
    alphas = torch.linspace(0.2, 2.0, num_heads)
    delta_vals = torch.tensor([math.log(1.0 + d) for d in offsets], dtype=torch.float32)
    return -delta_vals.unsqueeze(1) * alphas.unsqueeze(0)


def linearise_ring(ring, head, fill=None):
    """Ring buffer [S,H,R,D] with per-sequence write head -> time-ordered [S,H,L,D].

    The slot ``head[s]`` holds the newest token (position t); slot ``head-1`` the
    one before, and so on, wrapping modulo R.  ``fill[s]`` (default R) is the number
    of valid tokens including the newest.  All sequences must share the same fill
    for a rectangular result.
    """
    S, H, R, D = ring.shape
    L = R if fill is None else int(fill[0])
    if fill is not None:
        assert all(int(f) == L for f in fill)
    idx = (head.view(S, 1).long() - torch.arange(L - 1, -1, -1).view(1, L)) % R   # [S,L]
    idx = idx.view(S, 1, L, 1).expand(S, H, L, D)
    return torch.gather(ring, 2, idx)


def decode_reference(q, k_new, v_new, k_ring, v_ring, head, pos_bias, head_gain=None,
                     offsets: Sequence[int] = OFFSETS_43, fill=None, scale_embed=None,
                     compute_dtype=torch.float32):
    """Single-token decode oracle.

    The reference has no decode code (README.md:175-179 is prose), so the step is
    *defined* through the full-sequence reference: write k_new, v_new into slot
    ``head[s]`` of each ring, linearise the ring into a length-L sequence (L = fill,
    newest token last), run ``dsqg_reference`` with q placed in the last row and
    take that row.  Returns (out [S,H,D], k_ring', v_ring').
    """
    S, H, R, D = k_ring.shape
    k_ring = k_ring.clone(); v_ring = v_ring.clone()
    ar = torch.arange(S)
    k_ring[ar, :, head.long(), :] = k_new.to(k_ring.dtype)
    v_ring[ar, :, head.long(), :] = v_new.to(v_ring.dtype)
    kl = linearise_ring(k_ring, head, fill)
    vl = linearise_ring(v_ring, head, fill)
    L = kl.shape[2]
    qs = torch.zeros(S, H, L, D, dtype=compute_dtype)
    qs[:, :, -1, :] = q.to(compute_dtype)
    out = dsqg_reference(qs, kl, vl, pos_bias, scale_embed, head_gain, offsets, compute_dtype)
    return out[:, :, -1, :], k_ring, v_ring


def decode_reference_direct(q, k_new, v_new, k_ring, v_ring, head, pos_bias, head_gain=None,
                            offsets: Sequence[int] = OFFSETS_43, fill=None, scale_embed=None,
                            compute_dtype=torch.float32):
    """Same result as ``decode_reference`` without building the whole sequence.

    Only the newest row is evaluated: tap j reads ring slot ``(head - delta_j) mod R``
    and is valid iff ``delta_j < fill``.  ``fill`` may differ per sequence here.
    Checked equal to ``decode_reference`` in tests/test_oracle_golden.py; used where the
    full-sequence form would need too much memory.
    """
    S, H, R, D = k_ring.shape
    k_ring = k_ring.clone(); v_ring = v_ring.clone()
    ar = torch.arange(S)
    k_ring[ar, :, head.long(), :] = k_new.to(k_ring.dtype)
    v_ring[ar, :, head.long(), :] = v_new.to(v_ring.dtype)
    off = torch.tensor(list(offsets), dtype=torch.long)
    J = off.numel()
    slot = (head.view(S, 1).long() - off.view(1, J)) % R                      # [S,J]
    fl = torch.full((S,), R, dtype=torch.long) if fill is None else torch.as_tensor(fill).long()
    valid = off.view(1, J) < fl.view(S, 1)                                     # [S,J]
    idx = slot.view(S, 1, J, 1).expand(S, H, J, D)
    Ka = torch.gather(k_ring, 2, idx).to(compute_dtype)
    Va = torch.gather(v_ring, 2, idx).to(compute_dtype)
    qf = q.to(compute_dtype)
    sc = D ** -0.5
    s = (qf.unsqueeze(2) * Ka).sum(-1) * sc + pos_bias.to(compute_dtype).T[None]
    if scale_embed is not None:
        s = s + (qf.unsqueeze(2) * scale_embed.to(compute_dtype)[None, None]).sum(-1) * sc
    s = s.masked_fill(~valid.view(S, 1, J), float('-inf'))
    a = F.softmax(s, dim=-1)
    out = (a.unsqueeze(-1) * Va).sum(2)
    if head_gain is not None:
        out = out * head_gain.to(compute_dtype).view(1, H, 1)
    return out, k_ring, v_ring
