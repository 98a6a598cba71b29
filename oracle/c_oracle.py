"""ctypes binding of oracle/dsqg_oracle.c (double-accumulating loop-nest oracle).

TEST INFRASTRUCTURE, NOT PRODUCT CODE: only tests/, the smoke check and the
benchmark's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libdsqg_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with gcc (``make -C oracle``)."""
    src = os.path.join(_HERE, "dsqg_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libdsqg_oracle.so"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _f32(t):
    return None if t is None else np.ascontiguousarray(t.detach().cpu().float().numpy())


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def fwd(q, k, v, pos_bias, scale_embed=None, head_gain=None, offsets=()):
    """Forward with double accumulation.  Returns (out fp32 [B,H,N,D], lse fp32 [B,H,N])."""
    B, H, N, D = q.shape
    qa, ka, va, pb, se, g = map(_f32, (q, k, v, pos_bias, scale_embed, head_gain))
    off = np.asarray(list(offsets), dtype=np.int32)
    out = np.empty((B, H, N, D), np.float32)
    lse = np.empty((B, H, N), np.float32)
    rc = lib().dsqg_oracle_fwd(_p(qa), _p(ka), _p(va), _p(pb), _p(se), _p(g), _p(off),
                               len(off), B, H, N, D, _p(out), _p(lse))
    assert rc == 0
    return torch.from_numpy(out), torch.from_numpy(lse)


def bwd(q, k, v, pos_bias, dout, scale_embed=None, head_gain=None, offsets=()):
    """Backward with double accumulation.  Returns dict dq, dk, dv, dpb[, dse][, dgain]."""
    B, H, N, D = q.shape
    qa, ka, va, pb, se, g, do = map(_f32, (q, k, v, pos_bias, scale_embed, head_gain, dout))
    off = np.asarray(list(offsets), dtype=np.int32)
    dq = np.empty((B, H, N, D), np.float32); dk = np.empty_like(dq); dv = np.empty_like(dq)
    dpb = np.empty((len(off), H), np.float32)
    dse = None if se is None else np.empty((len(off), D), np.float32)
    dg = None if g is None else np.empty((H,), np.float32)
    rc = lib().dsqg_oracle_bwd(_p(qa), _p(ka), _p(va), _p(pb), _p(se), _p(g), _p(off),
                               len(off), B, H, N, D, _p(do), _p(dq), _p(dk), _p(dv),
                               _p(dpb), _p(dse), _p(dg))
    assert rc == 0
    res = {"dq": torch.from_numpy(dq), "dk": torch.from_numpy(dk), "dv": torch.from_numpy(dv),
           "dpb": torch.from_numpy(dpb)}
    if dse is not None: res["dse"] = torch.from_numpy(dse)
    if dg is not None: res["dgain"] = torch.from_numpy(dg)
    return res
