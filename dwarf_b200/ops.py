"""DSQG attention as a torch.autograd.Function over the native C ABI.

Mirrors the operator layer of the DWARF reference:
``_DSQGFn`` / ``_DSQGFnV3`` (kernels/dsqg_attention_v2.py:337-414,
kernels/dsqg_attention_v3.py:359-442) and their functional wrappers
(:417-427, :445-456).  PyTorch is used for device memory and streams only; all
arithmetic happens in libdsqg_b200.so.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from . import _lib

SPARSE_TAPS = (48, 64, 96, 128, 192, 256, 384, 512, 768, 1024, 1536)
#: The reference's 44-offset set (kernels/dsqg_attention_v3.py:47-49): dense 0..32 + 11 taps.
ALL_OFFSETS = tuple(range(33)) + SPARSE_TAPS
#: Dense 0..31 + the same 11 taps: the 43-offset set the benchmark configurations name.
OFFSETS_43 = tuple(range(32)) + SPARSE_TAPS
#: 43-set extended for N = 4096.
OFFSETS_45 = OFFSETS_43 + (2048, 3072)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.DSQG_DTYPE_BF16
    if t.dtype == torch.float32:
        return _lib.DSQG_DTYPE_F32
    raise TypeError(f"dsqg: q/k/v must be bfloat16 or float32, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _check_inputs(q, k, v, pos_bias, head_gain, scale_embed, J):
    if not q.is_cuda:
        raise RuntimeError("dsqg: tensors must live on a CUDA device (there is no CPU path)")
    if q.dim() != 4:
        raise ValueError(f"dsqg: q must be [B,H,N,HD], got {tuple(q.shape)}")
    B, H, N, D = q.shape
    for name, t in (("k", k), ("v", v)):
        if t.shape != q.shape or t.dtype != q.dtype or t.device != q.device:
            raise ValueError(f"dsqg: {name} must match q in shape, dtype and device")
    if tuple(pos_bias.shape) != (J, H):
        raise ValueError(f"dsqg: pos_bias must be [{J},{H}], got {tuple(pos_bias.shape)}")
    if scale_embed is not None and tuple(scale_embed.shape) != (J, D):
        raise ValueError(f"dsqg: scale_embed must be [{J},{D}], got {tuple(scale_embed.shape)}")
    if head_gain is not None and tuple(head_gain.shape) != (H,):
        raise ValueError(f"dsqg: head_gain must be [{H}], got {tuple(head_gain.shape)}")


def _padded_head_dim(q, off, J, has_scale_embed):
    """Head dimension the kernels are called with.  The bf16 tensor-core kernels exist for
    D in {32, 64, 96, 128}; another bf16 head dimension (80 in the reference's 85M condM model,
    train/train_2048_85m_condM.py:67-69; 48) is zero-padded up to the next of those when the
    tensor-core kernels take the padded problem, with the scale 1/sqrt(D) of the true width passed
    explicitly: several times faster than the CUDA-core kernels on the odd width.  The reference
    pads to a power of two inside its kernels (kernels/dsqg_attention_v2.py:344).  fp32 tensors
    are never padded."""
    D = q.shape[-1]
    if q.dtype != torch.bfloat16 or D % 32 == 0 or D > 128 or D % 8 != 0:
        return D
    Dp = (D + 31) // 32 * 32
    lib = _lib.load()
    return Dp if lib.dsqg_tensor_core_path(_lib.DSQG_DTYPE_BF16, Dp, off, J, int(has_scale_embed)) else D


def _f32c(t):
    return None if t is None else t.detach().to(torch.float32).contiguous()


class DSQGFunction(torch.autograd.Function):
    """out = DSQG(q, k, v; pos_bias, head_gain, scale_embed, offsets) with autograd.

    Saves (q, k, v, pos_bias, head_gain, scale_embed, out, lse) like the reference
    (kernels/dsqg_attention_v3.py:384) and returns gradients for the six tensors.
    """

    @staticmethod
    def forward(ctx, q, k, v, pos_bias, head_gain, scale_embed, offsets):
        lib = _lib.load()
        off, J = _lib.offsets_array(offsets)
        _check_inputs(q, k, v, pos_bias, head_gain, scale_embed, J)
        pb, hg, se = _f32c(pos_bias), _f32c(head_gain), _f32c(scale_embed)
        B, H, N, D = q.shape
        Dp = _padded_head_dim(q, off, J, scale_embed is not None)
        if Dp != D:                              # zero columns change no score and give zero outputs
            q, k, v = (F.pad(t, (0, Dp - D)) for t in (q, k, v))
            se = None if se is None else F.pad(se, (0, Dp - D))
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out = torch.empty_like(q)
        lse = torch.empty(B, H, N, device=q.device, dtype=torch.float32)
        with torch.cuda.device(q.device):
            stream = torch.cuda.current_stream(q.device).cuda_stream
            _lib.check(lib.dsqg_fwd_scaled(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), _ptr(se),
                                           _ptr(hg), off, J, out.data_ptr(), lse.data_ptr(),
                                           B, H, N, Dp, _dtype_code(q), stream, D ** -0.5), "dsqg_fwd")
        ctx.save_for_backward(q, k, v, pb, hg, se, out, lse)
        ctx.offsets = tuple(offsets)
        ctx.head_dim = D
        ctx.param_dtypes = (pos_bias.dtype, None if head_gain is None else head_gain.dtype,
                            None if scale_embed is None else scale_embed.dtype)
        return out if Dp == D else out[..., :D].contiguous()

    @staticmethod
    def backward(ctx, dout):
        lib = _lib.load()
        q, k, v, pb, hg, se, out, lse = ctx.saved_tensors
        off, J = _lib.offsets_array(ctx.offsets)
        B, H, N, Dp = q.shape
        D = ctx.head_dim
        if dout.dtype != q.dtype:
            dout = dout.to(q.dtype)
        if Dp != D:
            dout = F.pad(dout, (0, Dp - D))
        dout = dout.contiguous()                      # kernels/dsqg_attention_v3.py:394
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dpb = torch.empty_like(pb)
        dse = None if se is None else torch.empty_like(se)
        dhg = None if hg is None else torch.empty_like(hg)
        nbytes = lib.dsqg_bwd_scratch_bytes(J, B, H, N, Dp, int(se is not None))
        scratch = torch.empty(nbytes, device=q.device, dtype=torch.uint8)
        with torch.cuda.device(q.device):
            stream = torch.cuda.current_stream(q.device).cuda_stream
            _lib.check(lib.dsqg_bwd_scaled(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), _ptr(se),
                                           _ptr(hg), off, J, out.data_ptr(), lse.data_ptr(), dout.data_ptr(),
                                           dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                           dpb.data_ptr(), _ptr(dse), _ptr(dhg),
                                           scratch.data_ptr(), nbytes, B, H, N, Dp, _dtype_code(q), stream,
                                           D ** -0.5), "dsqg_bwd")
        if Dp != D:
            dq, dk, dv = (t[..., :D].contiguous() for t in (dq, dk, dv))
            dse = None if dse is None else dse[:, :D].contiguous()
        pb_dt, hg_dt, se_dt = ctx.param_dtypes
        return (dq, dk, dv, dpb.to(pb_dt),
                None if dhg is None else dhg.to(hg_dt),
                None if dse is None else dse.to(se_dt), None)


class CausalMeanFunction(torch.autograd.Function):
    """pool[b,n,:] = mean(x[b,0..n,:]) with autograd (the backward is the kernel's reverse mode)."""

    @staticmethod
    def forward(ctx, x):
        if not x.is_cuda or x.dim() != 3 or x.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("causal_mean: x must be a CUDA [B,N,D] tensor in bfloat16 or float32")
        x = x.contiguous()
        ctx.meta = tuple(x.shape)
        return CausalMeanFunction._run(x, 0)

    @staticmethod
    def backward(ctx, dout):
        return CausalMeanFunction._run(dout.contiguous(), 1)

    @staticmethod
    def _run(x, reverse):
        lib = _lib.load()
        B, N, D = x.shape
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            stream = torch.cuda.current_stream(x.device).cuda_stream
            _lib.check(lib.dsqg_causal_mean(x.data_ptr(), out.data_ptr(), B, N, D, _dtype_code(x), reverse, stream),
                       "dsqg_causal_mean")
        return out


def causal_mean(x):
    """Causal running mean over the sequence dimension of x [B,N,D] (bf16 or fp32; other dtypes are
    computed in fp32 and cast back): the pooling of the reference's interference block,
    `x.cumsum(dim=1) / counts` (train/train_2048_condU.py:289-292), as one kernel."""
    if x.dtype in (torch.bfloat16, torch.float32):
        return CausalMeanFunction.apply(x)
    return CausalMeanFunction.apply(x.float()).to(x.dtype)


class DSQGPackedFunction(torch.autograd.Function):
    """DSQG on the un-permuted output of a fused qkv projection, with a token-major result.

    qkv [B,N,3,H,HD] bf16 (a view of the [B,N,3*H*HD] projection output; q, k, v are read in place
    through strides), gate [B,N,H*HD] bf16 or None -> y [B,N,H*HD] = DSQG(q,k,v) (* sigmoid(gate)).
    Replaces the three `.permute(0,2,1,3).contiguous()` copies, the output permute and the gate
    multiply of the reference's attention modules (train/train_2048_condU.py:171-175,189-191) and
    their autograd backward; the gradient comes back as one dqkv tensor in the layout of qkv."""

    @staticmethod
    def forward(ctx, qkv, gate, pos_bias, head_gain, offsets, scale_embed=None):
        lib = _lib.load()
        off, J = _lib.offsets_array(offsets)
        B, N, three, H, D = qkv.shape
        if three != 3 or qkv.dtype != torch.bfloat16 or not qkv.is_contiguous():
            raise ValueError("dsqg packed: qkv must be a contiguous bf16 [B,N,3,H,HD] tensor")
        if gate is not None and (gate.dtype != torch.bfloat16 or tuple(gate.shape) != (B, N, H * D)):
            raise ValueError("dsqg packed: gate must be bf16 [B,N,H*HD]")
        gate = None if gate is None else gate.contiguous()
        pb, hg = _f32c(pos_bias), _f32c(head_gain)
        if tuple(pb.shape) != (J, H):
            raise ValueError(f"dsqg: pos_bias must be [{J},{H}], got {tuple(pb.shape)}")
        se = _f32c(scale_embed)
        if se is not None and tuple(se.shape) != (J, D):
            raise ValueError(f"dsqg: scale_embed must be [{J},{D}], got {tuple(se.shape)}")
        y = torch.empty(B, N, H * D, device=qkv.device, dtype=qkv.dtype)
        lse = torch.empty(B, H, N, device=qkv.device, dtype=torch.float32)
        st_in = _lib.Strides(N * 3 * H * D, D, 3 * H * D)
        st_out = _lib.Strides(N * H * D, D, H * D)
        p0, esz = qkv.data_ptr(), qkv.element_size()
        with torch.cuda.device(qkv.device):
            stream = torch.cuda.current_stream(qkv.device).cuda_stream
            if se is None:
                _lib.check(lib.dsqg_fwd_strided(p0, p0 + H * D * esz, p0 + 2 * H * D * esz, st_in, pb.data_ptr(),
                                                _ptr(hg), off, J, y.data_ptr(), st_out, _ptr(gate), lse.data_ptr(),
                                                B, H, N, D, _lib.DSQG_DTYPE_BF16, stream, 0.0), "dsqg_fwd_strided")
            else:
                _lib.check(lib.dsqg_fwd_strided_se(p0, p0 + H * D * esz, p0 + 2 * H * D * esz, st_in, pb.data_ptr(),
                                                   se.data_ptr(), _ptr(hg), off, J, y.data_ptr(), st_out, _ptr(gate),
                                                   lse.data_ptr(), B, H, N, D, _lib.DSQG_DTYPE_BF16, stream, 0.0),
                           "dsqg_fwd_strided_se")
        ctx.save_for_backward(qkv, gate, pb, hg, y, lse, se)
        ctx.offsets = tuple(offsets)
        ctx.param_dtypes = (pos_bias.dtype, None if head_gain is None else head_gain.dtype,
                            None if scale_embed is None else scale_embed.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.load()
        qkv, gate, pb, hg, y, lse, se = ctx.saved_tensors
        off, J = _lib.offsets_array(ctx.offsets)
        B, N, _, H, D = qkv.shape
        dy = dy.to(qkv.dtype).contiguous()
        st_in = _lib.Strides(N * 3 * H * D, D, 3 * H * D)
        st_out = _lib.Strides(N * H * D, D, H * D)
        dqkv = torch.empty_like(qkv)
        dpb = torch.empty_like(pb)
        dhg = None if hg is None else torch.empty_like(hg)
        dse = None if se is None else torch.empty_like(se)
        nbytes = lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, 0 if se is None else 1)
        scratch = torch.empty(nbytes, device=qkv.device, dtype=torch.uint8)
        p0, g0, esz = qkv.data_ptr(), dqkv.data_ptr(), qkv.element_size()
        with torch.cuda.device(qkv.device):
            stream = torch.cuda.current_stream(qkv.device).cuda_stream
            dgate, dout, delta = None, dy, None
            if gate is not None:
                dout, dgate = torch.empty_like(y), torch.empty_like(gate)
                delta = torch.empty(B, H, N, device=qkv.device, dtype=torch.float32)
                _lib.check(lib.dsqg_gate_bwd(dy.data_ptr(), y.data_ptr(), gate.data_ptr(), st_out, dout.data_ptr(),
                                             dgate.data_ptr(), delta.data_ptr(), B, H, N, D, stream), "dsqg_gate_bwd")
            if se is None:
                _lib.check(lib.dsqg_bwd_strided(p0, p0 + H * D * esz, p0 + 2 * H * D * esz, st_in, pb.data_ptr(),
                                                _ptr(hg), off, J, y.data_ptr(), lse.data_ptr(), dout.data_ptr(), st_out,
                                                _ptr(delta), g0, g0 + H * D * esz, g0 + 2 * H * D * esz, dpb.data_ptr(),
                                                _ptr(dhg), scratch.data_ptr(), nbytes, B, H, N, D,
                                                _lib.DSQG_DTYPE_BF16, stream, 0.0), "dsqg_bwd_strided")
            else:
                _lib.check(lib.dsqg_bwd_strided_se(p0, p0 + H * D * esz, p0 + 2 * H * D * esz, st_in, pb.data_ptr(),
                                                   se.data_ptr(), _ptr(hg), off, J, y.data_ptr(), lse.data_ptr(),
                                                   dout.data_ptr(), st_out, _ptr(delta), g0, g0 + H * D * esz,
                                                   g0 + 2 * H * D * esz, dpb.data_ptr(), dse.data_ptr(), _ptr(dhg),
                                                   scratch.data_ptr(), nbytes, B, H, N, D, _lib.DSQG_DTYPE_BF16,
                                                   stream, 0.0), "dsqg_bwd_strided_se")
        pb_dt, hg_dt, se_dt = ctx.param_dtypes
        return (dqkv, dgate, dpb.to(pb_dt), None if dhg is None else dhg.to(hg_dt), None,
                None if dse is None else dse.to(se_dt))


class InjectKVFunction(torch.autograd.Function):
    """k += k_delta; v += v_delta (train/train_2048_condU.py:178-181) applied IN PLACE to the key
    and value thirds of a fused projection output qkv [B,N,3*D] (a non-leaf tensor that is not a
    view, e.g. what nn.Linear returned), so the packed operator can go on reading q, k, v in place.
    k_delta, v_delta: [B,N,D] token-major.  Backward: the deltas' gradients are the key and value
    thirds of qkv's gradient (views, no copy)."""

    @staticmethod
    def forward(ctx, qkv, k_delta, v_delta):
        B, N, D3 = qkv.shape
        if D3 % 3 or tuple(k_delta.shape) != (B, N, D3 // 3) or tuple(v_delta.shape) != (B, N, D3 // 3):
            raise ValueError("dsqg inject: qkv must be [B,N,3*D] and the deltas [B,N,D]")
        thirds = qkv.view(B, N, 3, D3 // 3)
        thirds[:, :, 1].add_(k_delta)
        thirds[:, :, 2].add_(v_delta)
        ctx.mark_dirty(qkv)
        ctx.delta_dtypes = (k_delta.dtype, v_delta.dtype)
        return qkv

    @staticmethod
    def backward(ctx, g):
        B, N, D3 = g.shape
        thirds = g.view(B, N, 3, D3 // 3) if g.is_contiguous() else g.reshape(B, N, 3, D3 // 3)
        kdt, vdt = ctx.delta_dtypes
        return g, thirds[:, :, 1].to(kdt), thirds[:, :, 2].to(vdt)


def packed_path_available(head_dim: int, offsets: Sequence[int], scale_embed: bool = False) -> bool:
    """True when dsqg_attention_packed can take this head width and offset set (the bf16 tensor-core
    kernels; with scale_embed head widths up to 64); otherwise callers use dsqg_attention on
    permuted copies."""
    off, J = _lib.offsets_array(offsets)
    return bool(_lib.load().dsqg_tensor_core_path(_lib.DSQG_DTYPE_BF16, int(head_dim), off, J, 1 if scale_embed else 0))


def dsqg_attention_packed(qkv, pos_bias, head_gain=None, gate=None, offsets: Sequence[int] = ALL_OFFSETS,
                          scale_embed=None):
    """DSQG straight on the fused projection output.  qkv: [B,N,3,H,HD] bf16 contiguous; gate: None
    or [B,N,H*HD] bf16 (pre-sigmoid); scale_embed: None or [J,HD] (the reference's v3 op).  Returns
    [B,N,H*HD] bf16, already multiplied by sigmoid(gate) when a gate is given."""
    return DSQGPackedFunction.apply(qkv, gate, pos_bias, head_gain, tuple(int(o) for o in offsets), scale_embed)


def dsqg_attention(q, k, v, pos_bias, head_gain=None, scale_embed=None,
                   offsets: Sequence[int] = ALL_OFFSETS):
    """General DSQG entry: any ascending offset set, optional per-head output gain and
    Q-weighted scale embedding.  q, k, v: [B,H,N,HD] bf16 (fast path) or fp32; fp16 inputs
    are computed in bf16 as the reference does (kernels/dsqg_attention_v3.py:452-456) and
    the result is returned in the caller's dtype."""
    orig_dtype = q.dtype
    if orig_dtype not in (torch.bfloat16, torch.float32):
        q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    out = DSQGFunction.apply(q, k, v, pos_bias, head_gain, scale_embed, tuple(int(o) for o in offsets))
    return out if out.dtype == orig_dtype else out.to(orig_dtype)


def dsqg_forward_lse(q, k, v, pos_bias, head_gain=None, scale_embed=None,
                     offsets: Sequence[int] = ALL_OFFSETS):
    """Forward without autograd; returns (out, lse).  lse is the natural-log softmax
    denominator per row, the tensor the reference saves for backward."""
    lib = _lib.load()
    off, J = _lib.offsets_array(offsets)
    _check_inputs(q, k, v, pos_bias, head_gain, scale_embed, J)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    pb, hg, se = _f32c(pos_bias), _f32c(head_gain), _f32c(scale_embed)
    B, H, N, D = q.shape
    out = torch.empty_like(q)
    lse = torch.empty(B, H, N, device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        _lib.check(lib.dsqg_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), _ptr(se),
                                _ptr(hg), off, J, out.data_ptr(), lse.data_ptr(),
                                B, H, N, D, _dtype_code(q), stream), "dsqg_fwd")
    return out, lse
