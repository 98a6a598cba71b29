"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (no dataset stands behind the DSQG op benchmarks; these are fully synthetic).

Everything is drawn from a CPU ``torch.Generator`` in fp32 and then cast / moved, so the
same seed yields the same values for the CUDA path and for a CPU checker.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch

from .ops import ALL_OFFSETS, OFFSETS_43, OFFSETS_45


_TENSOR_SALT = {"q": 1, "k": 2, "v": 3, "dout": 4}


@dataclass
class OpConfig:
    name: str
    B: int
    H: int
    N: int
    D: int
    dtype: torch.dtype
    offsets: Tuple[int, ...]
    qkv_scale: float = 0.5
    bias_noise: float = 0.05
    random_gain: bool = True
    seed: int = 1234


#: The DSQG op configurations of the benchmark specification.
OP_CONFIGS = {
    "cfg0": OpConfig("cfg0 fwd fp32 B2 H8 N2048 D32 J43", 2, 8, 2048, 32, torch.float32, OFFSETS_43,
                     qkv_scale=1.0, bias_noise=0.0, random_gain=False, seed=100),
    "cfg1": OpConfig("cfg1 fwd+bwd bf16 B32 H8 N2048 D32 J43", 32, 8, 2048, 32, torch.bfloat16,
                     OFFSETS_43, seed=101),
    "cfg2": OpConfig("cfg2 fwd+bwd bf16 B16 H12 N2048 D64 J43", 16, 12, 2048, 64, torch.bfloat16,
                     OFFSETS_43, seed=102),
    "cfg2_4k": OpConfig("cfg2 fwd+bwd bf16 B16 H12 N4096 D64 J45", 16, 12, 4096, 64, torch.bfloat16,
                        OFFSETS_45, seed=103),
}


def log_linear_pos_bias(offsets, H):
    """pos_bias[j,h] = -alpha_h * log(1+delta_j), alpha = linspace(0.2, 2.0, H)."""
    alphas = torch.linspace(0.2, 2.0, H)
    logs = torch.tensor([math.log(1.0 + d) for d in offsets], dtype=torch.float32)
    return -logs[:, None] * alphas[None, :]


def make_op_inputs(cfg: OpConfig, device="cpu", B: Optional[int] = None, with_dout: bool = True):
    """Returns dict(q, k, v, dout, pos_bias, head_gain, offsets).  ``B`` overrides the batch
    (for bounded CPU samples and for sharding); the values of the first B batches are
    the same as in the full problem."""
    g = torch.Generator(device="cpu").manual_seed(cfg.seed)
    J = len(cfg.offsets)
    pb = log_linear_pos_bias(cfg.offsets, cfg.H)
    if cfg.bias_noise:
        pb = pb + torch.randn(J, cfg.H, generator=g) * cfg.bias_noise
    gain = (torch.rand(cfg.H, generator=g) * 0.4 + 0.8) if cfg.random_gain else None
    nb = cfg.B if B is None else B
    shape = (nb, cfg.H, cfg.N, cfg.D)
    res = {"pos_bias": pb.to(device), "head_gain": None if gain is None else gain.to(device),
           "offsets": cfg.offsets}
    names = ("q", "k", "v") + (("dout",) if with_dout else ())
    for nm in names:
        sc = 1.0 if nm == "dout" else cfg.qkv_scale
        # per-tensor, per-batch generators: batch b of tensor nm never depends on nb
        parts = []
        for b in range(nb):
            gb = torch.Generator(device="cpu").manual_seed(cfg.seed * 1000003 + _TENSOR_SALT[nm] * 7919 + b)
            parts.append(torch.randn(shape[1:], generator=gb) * sc)
        res[nm] = torch.stack(parts).to(cfg.dtype).to(device)
    return res


@dataclass
class DecodeConfig:
    name: str = "cfg3 decode bf16 S256 H12 D64 R1537 L10 J43"
    S: int = 256
    H: int = 12
    D: int = 64
    layers: int = 10
    dtype: torch.dtype = torch.bfloat16
    offsets: Tuple[int, ...] = OFFSETS_43
    seed: int = 104

    @property
    def R(self):
        return max(self.offsets) + 1


def make_decode_inputs(cfg: DecodeConfig, device="cpu", S: Optional[int] = None, layers: Optional[int] = None,
                       rings_on=None):
    """Fully populated rings ~ N(0,1), a random write head per sequence, new q,k,v ~ N(0,1).
    rings_on: a CUDA device on which the two ring tensors are drawn directly (seeded generator of
    that device) instead of on the host; everything else stays on `device`."""
    g = torch.Generator(device="cpu").manual_seed(cfg.seed)
    S = cfg.S if S is None else S
    L = cfg.layers if layers is None else layers
    J = len(cfg.offsets)
    pb = log_linear_pos_bias(cfg.offsets, cfg.H) + torch.randn(J, cfg.H, generator=g) * 0.05
    gain = torch.rand(cfg.H, generator=g) * 0.4 + 0.8
    head = torch.randint(0, cfg.R, (S,), generator=g, dtype=torch.int32)
    mk = lambda *shape: torch.randn(*shape, generator=g).to(cfg.dtype).to(device)
    if rings_on == "meta":            # the caller draws the rings itself
        ring = lambda: None
    elif rings_on is not None:
        gd = torch.Generator(device=rings_on).manual_seed(cfg.seed + 1)
        ring = lambda: torch.randn(L, S, cfg.H, cfg.R, cfg.D, generator=gd, device=rings_on, dtype=cfg.dtype)
    else:
        ring = lambda: mk(L, S, cfg.H, cfg.R, cfg.D)
    return {"k_ring": ring(), "v_ring": ring(),
            "q": mk(L, S, cfg.H, cfg.D), "k_new": mk(L, S, cfg.H, cfg.D), "v_new": mk(L, S, cfg.H, cfg.D),
            "head": head.to(device), "pos_bias": pb.to(device), "head_gain": gain.to(device),
            "offsets": cfg.offsets}
