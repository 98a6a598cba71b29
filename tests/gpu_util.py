"""Helpers for the GPU parity tests: run the CUDA op (through the ctypes C-ABI binding) and
compare with the CPU oracles."""
import torch

import dwarf_b200
from oracle import c_oracle as C
from oracle import dsqg_oracle as O

BF16_ABS_TOL = 2e-2        # absolute tolerance for bf16 outputs and gradients (benchmark spec)
BF16_ULP = 2.0 ** -8       # one bf16 rounding step relative to the value (output rounding)
PARAM_REL_TOL_BF16 = 2e-2  # dpos_bias / dscale_embed / dhead_gain in the bf16 path: sums over all rows of
                           # terms that carry delta = sum_d dout*out with the bf16-rounded saved output
                           # (as in the reference kernels, kernels/dsqg_attention_v3.py:170-191)
FP32_REL_TOL = 1e-5        # ||x-ref||_inf / ||ref||_inf for the fp32 instantiation


def _inside_poison(t, dev, dtype, poison):
    """A device copy of t that sits in the middle of a larger buffer filled with `poison`."""
    pad = 8192
    buf = torch.full((t.numel() + 2 * pad,), poison, dtype=dtype, device=dev)
    view = buf[pad:pad + t.numel()].view(t.shape)
    view.copy_(t)
    return view.detach()


def cuda_fwd_bwd(q, k, v, pos_bias, dout=None, scale_embed=None, head_gain=None, offsets=None,
                 dtype=torch.bfloat16, poison=float("nan")):
    """Run forward (+ backward when dout is given) on cuda:0.  Inputs are CPU tensors.
    poison: value the memory before and after q, k, v and dout is filled with (NaN by default, so
    every parity test also checks that nothing outside the tensors reaches a result); None puts
    the tensors in ordinary allocations."""
    dev = torch.device("cuda", 0)
    put = (lambda t: t.to(dev, dtype)) if poison is None else (lambda t: _inside_poison(t, dev, dtype, poison))
    qd, kd, vd = (put(t).requires_grad_(dout is not None) for t in (q, k, v))
    pb = pos_bias.to(dev).float().requires_grad_(dout is not None)
    se = None if scale_embed is None else scale_embed.to(dev).float().requires_grad_(dout is not None)
    hg = None if head_gain is None else head_gain.to(dev).float().requires_grad_(dout is not None)
    out = dwarf_b200.dsqg_attention(qd, kd, vd, pb, hg, se, offsets)
    res = {"out": out.detach().float().cpu()}
    if dout is not None:
        out.backward(put(dout))
        res.update(dq=qd.grad.float().cpu(), dk=kd.grad.float().cpu(), dv=vd.grad.float().cpu(),
                   dpb=pb.grad.cpu())
        if se is not None: res["dse"] = se.grad.cpu()
        if hg is not None: res["dgain"] = hg.grad.cpu()
    return res


def oracle_fwd_bwd(q, k, v, pos_bias, dout=None, scale_embed=None, head_gain=None, offsets=None):
    """Double-accumulating C oracle on the same (fp32-valued) inputs."""
    out, lse = C.fwd(q, k, v, pos_bias, scale_embed, head_gain, offsets)
    res = {"out": out, "lse": lse}
    if dout is not None:
        res.update(C.bwd(q, k, v, pos_bias, dout, scale_embed, head_gain, offsets))
    return res


def assert_bf16_close(x, ref, name):
    err = (x.double() - ref.double()).abs()
    tol = BF16_ABS_TOL + BF16_ULP * ref.double().abs()
    bad = err > tol
    assert not bool(bad.any()), (f"{name}: max abs err {err.max().item():.4g} "
                                 f"(|ref|max {ref.abs().max().item():.4g}), {int(bad.sum())} elements out of tolerance")


def assert_param_grad_close(x, ref, name, rel, abs_floor=1e-2):
    """max |x - ref| <= rel * max|ref| + abs_floor (the floor covers gradients that are exactly
    zero in the reference, e.g. a single-tap softmax)."""
    err = (x.double() - ref.double()).abs().max().item()
    bound = rel * ref.double().abs().max().item() + abs_floor
    assert err <= bound, f"{name}: max abs err {err:.3g} > {bound:.3g} (|ref|max {ref.abs().max().item():.3g})"


def rel_inf(x, ref):
    return ((x.double() - ref.double()).abs().max() / ref.double().abs().max().clamp_min(1e-30)).item()
