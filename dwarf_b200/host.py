"""Forward+backward steps whose tensors live in pinned HOST memory.

A caller that keeps activations on the host (an offloading trainer, a plugin host that owns
no device memory) pays one upload of (q, k, v, dout) and one download of (out, dq, dk, dv)
per step.  `DSQGHostPipeline` overlaps them with the kernels: an upload stream, a compute
stream and a download stream work on `depth` rotating sets of device buffers, so that while
step i runs on the SMs the copy engines upload step i+1 and download step i-1 (PCIe is full
duplex).  All arithmetic happens in libdsqg_b200.so through the C ABI (dsqg_fwd, dsqg_bwd);
there is no autograd graph and no per-step allocation.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib
from .ops import _dtype_code


class DSQGHostPipeline:
    """pipe = DSQGHostPipeline((B,H,N,D), torch.bfloat16, offsets, device); pipe.submit(...) per step.

    `submit` returns at once; results are complete after `synchronize()` (or after a later
    `submit` has reused the same slot, i.e. `depth` steps later).  Host tensors must be pinned
    and contiguous.  Parameter gradients (dpos_bias [J,H], dhead_gain [H]) of every step are
    downloaded into the host tensors given to `submit` when those are not None.
    """

    def __init__(self, shape: Sequence[int], dtype: torch.dtype, offsets: Sequence[int], device, depth: int = 2,
                 scale_embed: bool = False):
        if depth < 1:
            raise ValueError("dsqg host pipeline: depth must be >= 1")
        self.lib = _lib.load()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("dsqg host pipeline: needs a CUDA device (there is no CPU path)")
        self.B, self.H, self.N, self.D = (int(x) for x in shape)
        self.dtype = dtype
        self.off, self.J = _lib.offsets_array(offsets)
        self.depth = depth
        self.with_se = bool(scale_embed)
        B, H, N, D, J = self.B, self.H, self.N, self.D, self.J
        with torch.cuda.device(self.device):
            self.up, self.run, self.down = (torch.cuda.Stream(self.device) for _ in range(3))
            nbytes = self.lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, int(self.with_se))
            self.slots = []
            for _ in range(depth):
                t = lambda: torch.empty(B, H, N, D, dtype=dtype, device=self.device)
                self.slots.append({
                    "q": t(), "k": t(), "v": t(), "dout": t(), "out": t(), "dq": t(), "dk": t(), "dv": t(),
                    "lse": torch.empty(B, H, N, device=self.device),
                    "dpb": torch.empty(J, H, device=self.device), "dg": torch.empty(H, device=self.device),
                    "dse": torch.empty(J, D, device=self.device) if self.with_se else None,
                    "scratch": torch.empty(nbytes, dtype=torch.uint8, device=self.device), "nbytes": nbytes,
                    "uploaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "free": torch.cuda.Event(),
                })
        self.step = 0
        self._dt = _dtype_code(self.slots[0]["q"])

    def _check_host(self, name, t):
        if t.device.type != "cpu" or not t.is_pinned() or not t.is_contiguous():
            raise ValueError(f"dsqg host pipeline: {name} must be a contiguous pinned host tensor")
        if tuple(t.shape) != (self.B, self.H, self.N, self.D) or t.dtype != self.dtype:
            raise ValueError(f"dsqg host pipeline: {name} must be {(self.B, self.H, self.N, self.D)} {self.dtype}")

    def submit(self, q, k, v, dout, pos_bias, head_gain, out, dq, dk, dv,
               dpos_bias: Optional[torch.Tensor] = None, dhead_gain: Optional[torch.Tensor] = None,
               scale_embed: Optional[torch.Tensor] = None, dscale_embed: Optional[torch.Tensor] = None):
        """q, k, v, dout (inputs) and out, dq, dk, dv (results): pinned host [B,H,N,D];
        pos_bias [J,H], head_gain [H] (or None) and scale_embed [J,D] (only for a pipeline built with
        scale_embed=True): fp32 DEVICE tensors, read when the step runs."""
        if (scale_embed is not None) != self.with_se:
            raise ValueError("dsqg host pipeline: scale_embed must be given exactly when the pipeline was built with scale_embed=True")
        if scale_embed is not None and (tuple(scale_embed.shape) != (self.J, self.D) or scale_embed.dtype != torch.float32
                                        or not scale_embed.is_cuda):
            raise ValueError(f"dsqg host pipeline: scale_embed must be a float32 device tensor [{self.J},{self.D}]")
        for name, t in (("q", q), ("k", k), ("v", v), ("dout", dout), ("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
            self._check_host(name, t)
        if tuple(pos_bias.shape) != (self.J, self.H) or pos_bias.dtype != torch.float32 or not pos_bias.is_cuda:
            raise ValueError(f"dsqg host pipeline: pos_bias must be a float32 device tensor [{self.J},{self.H}]")
        s = self.slots[self.step % self.depth]
        first_use = self.step < self.depth
        self.step += 1
        lib, B, H, N, D, J = self.lib, self.B, self.H, self.N, self.D, self.J
        with torch.cuda.device(self.device):
            with torch.cuda.stream(self.up):
                if not first_use:
                    self.up.wait_event(s["free"])            # the slot's previous results have left the device
                for name, t in (("q", q), ("k", k), ("v", v), ("dout", dout)):
                    s[name].copy_(t, non_blocking=True)
                s["uploaded"].record(self.up)
            with torch.cuda.stream(self.run):
                self.run.wait_event(s["uploaded"])
                sp = self.run.cuda_stream
                hg = None if head_gain is None else head_gain.data_ptr()
                sep = None if scale_embed is None else scale_embed.data_ptr()
                _lib.check(lib.dsqg_fwd(s["q"].data_ptr(), s["k"].data_ptr(), s["v"].data_ptr(), pos_bias.data_ptr(),
                                        sep, hg, self.off, J, s["out"].data_ptr(), s["lse"].data_ptr(),
                                        B, H, N, D, self._dt, sp), "dsqg_fwd")
                _lib.check(lib.dsqg_bwd(s["q"].data_ptr(), s["k"].data_ptr(), s["v"].data_ptr(), pos_bias.data_ptr(),
                                        sep, hg, self.off, J, s["out"].data_ptr(), s["lse"].data_ptr(),
                                        s["dout"].data_ptr(), s["dq"].data_ptr(), s["dk"].data_ptr(), s["dv"].data_ptr(),
                                        s["dpb"].data_ptr(), None if scale_embed is None else s["dse"].data_ptr(),
                                        None if head_gain is None else s["dg"].data_ptr(),
                                        s["scratch"].data_ptr(), s["nbytes"], B, H, N, D, self._dt, sp), "dsqg_bwd")
                s["computed"].record(self.run)
            with torch.cuda.stream(self.down):
                self.down.wait_event(s["computed"])
                for name, t in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
                    t.copy_(s[name], non_blocking=True)
                if dpos_bias is not None:
                    dpos_bias.copy_(s["dpb"], non_blocking=True)
                if dhead_gain is not None and head_gain is not None:
                    dhead_gain.copy_(s["dg"], non_blocking=True)
                if dscale_embed is not None and scale_embed is not None:
                    dscale_embed.copy_(s["dse"], non_blocking=True)
                s["free"].record(self.down)

    def join(self, stream: Optional[torch.cuda.Stream] = None):
        """Make `stream` (default: the current stream) wait for everything submitted so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s in self.slots[:min(self.step, self.depth)]:
            stream.wait_event(s["free"])

    def synchronize(self):
        for st in (self.up, self.run, self.down):
            st.synchronize()
