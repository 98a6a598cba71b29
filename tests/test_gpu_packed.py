"""GPU tests of the copy-free layout path (dsqg_fwd_strided / dsqg_bwd_strided / dsqg_gate_bwd through
DSQGPackedFunction): q, k, v read in place from a fused qkv projection output [B,N,3,H,HD], result
token-major [B,N,H*HD], sigmoid gate folded into the epilogue.  The check is the chain the reference
runs -- permute copies, op, permute, gate multiply (train/train_2048_condU.py:171-175,184-191) --
evaluated with the C oracle in fp32."""
import pytest
import torch

import dwarf_b200
from dwarf_b200 import synth
from oracle import dsqg_oracle as O
from tests.gpu_util import (PARAM_REL_TOL_BF16, assert_bf16_close, assert_param_grad_close, oracle_fwd_bwd)

pytestmark = pytest.mark.gpu


def _case(B, N, H, D, offsets, seed):
    g = torch.Generator().manual_seed(seed)
    qkv = (torch.randn(B, N, 3, H, D, generator=g) * 0.5).bfloat16()
    gate = torch.randn(B, N, H * D, generator=g).bfloat16()
    dy = torch.randn(B, N, H * D, generator=g).bfloat16()
    pb = synth.log_linear_pos_bias(offsets, H) + torch.randn(len(offsets), H, generator=g) * 0.05
    gain = torch.rand(H, generator=g) * 0.4 + 0.8
    return qkv, gate, dy, pb, gain


def _reference(qkv, gate, dy, pb, gain, offsets):
    """permute -> oracle op -> permute -> * sigmoid(gate), and the gradients of that chain."""
    B, N, _, H, D = qkv.shape
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3).float().contiguous() for i in range(3))
    tok = lambda t: t.permute(0, 2, 1, 3).reshape(B, N, H * D)            # [B,H,N,D] -> [B,N,H*D]
    heads = lambda t: t.view(B, N, H, D).permute(0, 2, 1, 3).contiguous()
    fwd = oracle_fwd_bwd(q, k, v, pb, None, None, gain, offsets)
    o = tok(fwd["out"])
    if gate is None:
        y, dout, dgate = o, dy.float(), None
    else:
        s = torch.sigmoid(gate.float())
        y, dout = o * s, dy.float() * s
        dgate = dy.float() * o * s * (1 - s)
    bwd = oracle_fwd_bwd(q, k, v, pb, heads(dout), None, gain, offsets)
    dqkv = torch.stack([bwd[nm].permute(0, 2, 1, 3) for nm in ("dq", "dk", "dv")], dim=2)   # [B,N,3,H,D]
    return y, dqkv, dgate, bwd["dpb"], bwd["dgain"]


@pytest.mark.parametrize("shape", [(2, 300, 4, 32), (1, 2047, 8, 32), (2, 130, 3, 64), (1, 70, 2, 128), (1, 1, 2, 32)])
@pytest.mark.parametrize("offsets", [O.OFFSETS_43, O.OFFSETS_44], ids=["J43", "J44"])
@pytest.mark.parametrize("with_gate", [True, False])
def test_packed_qkv_token_major_out_and_gate_fold_vs_oracle_chain(shape, offsets, with_gate):
    B, N, H, D = shape
    qkv, gate, dy, pb, gain = _case(B, N, H, D, offsets, 11 + N + D)
    if not with_gate:
        gate = None
    y_ref, dqkv_ref, dgate_ref, dpb_ref, dgain_ref = _reference(qkv, gate, dy, pb, gain, offsets)
    dev = torch.device("cuda", 0)
    assert dwarf_b200.packed_path_available(D, offsets)
    qkv_d = qkv.to(dev).requires_grad_(True)
    gate_d = None if gate is None else gate.to(dev).requires_grad_(True)
    pb_d, gain_d = pb.to(dev).requires_grad_(True), gain.to(dev).requires_grad_(True)
    y = dwarf_b200.dsqg_attention_packed(qkv_d, pb_d, gain_d, gate_d, offsets)
    assert y.shape == (B, N, H * D) and y.dtype == torch.bfloat16
    y.backward(dy.to(dev))
    assert_bf16_close(y.detach().float().cpu(), y_ref, "y")
    assert_bf16_close(qkv_d.grad.float().cpu(), dqkv_ref, "dqkv")
    if with_gate:
        assert_bf16_close(gate_d.grad.float().cpu(), dgate_ref, "dgate")
    assert_param_grad_close(pb_d.grad.cpu(), dpb_ref, "dpb", PARAM_REL_TOL_BF16)
    assert_param_grad_close(gain_d.grad.cpu(), dgain_ref, "dgain", PARAM_REL_TOL_BF16)


def test_packed_path_equals_copy_path_bitwise_without_gate():
    """Same kernels, same arithmetic, other addresses: without the gate the strided entries must give
    exactly the bits of the contiguous entries on permuted copies."""
    dev = torch.device("cuda", 0)
    B, N, H, D = 2, 777, 4, 32
    qkv, _, dy, pb, gain = _case(B, N, H, D, O.OFFSETS_43, 5)
    qkv_d = qkv.to(dev).requires_grad_(True)
    pb_d, gain_d = pb.to(dev).requires_grad_(True), gain.to(dev).requires_grad_(True)
    y = dwarf_b200.dsqg_attention_packed(qkv_d, pb_d, gain_d, None, O.OFFSETS_43)
    y.backward(dy.to(dev))
    q, k, v = (qkv.to(dev)[:, :, i].permute(0, 2, 1, 3).contiguous().requires_grad_(True) for i in range(3))
    pb2, gain2 = pb.to(dev).requires_grad_(True), gain.to(dev).requires_grad_(True)
    o = dwarf_b200.dsqg_attention(q, k, v, pb2, gain2, None, O.OFFSETS_43)
    o.backward(dy.to(dev).view(B, N, H, D).permute(0, 2, 1, 3).contiguous())
    assert torch.equal(y.detach(), o.detach().permute(0, 2, 1, 3).reshape(B, N, H * D))
    for i, t in enumerate((q, k, v)):
        assert torch.equal(qkv_d.grad[:, :, i], t.grad.permute(0, 2, 1, 3))
    assert torch.equal(pb_d.grad, pb2.grad) and torch.equal(gain_d.grad, gain2.grad)


def test_module_takes_the_packed_path_under_autocast_and_matches_the_copy_path():
    dev = torch.device("cuda", 0)
    torch.manual_seed(2)
    m = dwarf_b200.DSQGAttentionN_Fused(256, 8, dropout=0.0, offsets=O.OFFSETS_43).to(dev)
    x = torch.randn(2, 200, 256, device=dev, requires_grad=True)

    def run(packed):
        m._packed = packed
        for p in m.parameters():
            p.grad = None
        x.grad = None
        with torch.amp.autocast("cuda", dtype=torch.bfloat16):
            y = m(x)
        y.float().sum().backward()
        return y.detach().float(), x.grad.clone(), m.pos_bias.grad.clone(), m.gate_proj.weight.grad.clone()

    a, b = run(None), run(False)
    assert m._packed is False
    m._packed = None
    for nm, u, w in zip(("y", "dx", "dpos_bias", "dgate_w"), a, b):
        scale = w.abs().max().item() + 1e-6
        assert (u - w).abs().max().item() <= 2e-2 * max(1.0, scale), nm
    # fp32 activations (no autocast) keep the copy path; so do layers with scale_embed on head widths above 64
    assert not m._packed_ok(torch.zeros(1, device=dev))
    assert dwarf_b200.DSQGAttentionV3(64, 2).to(dev)._packed_ok(torch.zeros(1, device=dev, dtype=torch.bfloat16))
    assert not dwarf_b200.DSQGAttentionV3(256, 2).to(dev)._packed_ok(torch.zeros(1, device=dev, dtype=torch.bfloat16))


@pytest.mark.parametrize("shape", [(2, 300, 4, 32), (1, 1500, 3, 64), (1, 1, 2, 32)])
@pytest.mark.parametrize("offsets", [O.OFFSETS_43, O.OFFSETS_44], ids=["J43", "J44"])
@pytest.mark.parametrize("with_gate", [True, False])
def test_packed_path_with_scale_embed_vs_oracle_chain(shape, offsets, with_gate):
    """The reference's v3 op (q-weighted scale selection) on the packed layout: the chain of
    train/train_2048_condU.py:171-175,184-191 with the oracle in fp32."""
    B, N, H, D = shape
    qkv, gate, dy, pb, gain = _case(B, N, H, D, offsets, 31 + N + D)
    g = torch.Generator().manual_seed(99)
    se = torch.randn(len(offsets), D, generator=g) * 0.3
    if not with_gate:
        gate = None
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3).float().contiguous() for i in range(3))
    tok = lambda t: t.permute(0, 2, 1, 3).reshape(B, N, H * D)
    heads = lambda t: t.view(B, N, H, D).permute(0, 2, 1, 3).contiguous()
    o = tok(oracle_fwd_bwd(q, k, v, pb, None, se, gain, offsets)["out"])
    if gate is None:
        y_ref, dout, dgate_ref = o, dy.float(), None
    else:
        sg = torch.sigmoid(gate.float())
        y_ref, dout, dgate_ref = o * sg, dy.float() * sg, dy.float() * o * sg * (1 - sg)
    bwd = oracle_fwd_bwd(q, k, v, pb, heads(dout), se, gain, offsets)
    dqkv_ref = torch.stack([bwd[nm].permute(0, 2, 1, 3) for nm in ("dq", "dk", "dv")], dim=2)
    dev = torch.device("cuda", 0)
    assert dwarf_b200.packed_path_available(D, offsets, scale_embed=True)
    qkv_d = qkv.to(dev).requires_grad_(True)
    gate_d = None if gate is None else gate.to(dev).requires_grad_(True)
    pb_d, gain_d, se_d = (t.to(dev).requires_grad_(True) for t in (pb, gain, se))
    y = dwarf_b200.dsqg_attention_packed(qkv_d, pb_d, gain_d, gate_d, offsets, scale_embed=se_d)
    y.backward(dy.to(dev))
    assert_bf16_close(y.detach().float().cpu(), y_ref, "y")
    assert_bf16_close(qkv_d.grad.float().cpu(), dqkv_ref, "dqkv")
    if with_gate:
        assert_bf16_close(gate_d.grad.float().cpu(), dgate_ref, "dgate")
    assert_param_grad_close(pb_d.grad.cpu(), bwd["dpb"], "dpb", PARAM_REL_TOL_BF16)
    assert_param_grad_close(gain_d.grad.cpu(), bwd["dgain"], "dgain", PARAM_REL_TOL_BF16)
    assert_param_grad_close(se_d.grad.cpu(), bwd["dse"], "dse", PARAM_REL_TOL_BF16)


def test_packed_path_with_scale_embed_equals_copy_path_bitwise():
    dev = torch.device("cuda", 0)
    B, N, H, D = 2, 777, 4, 32
    qkv, _, dy, pb, gain = _case(B, N, H, D, O.OFFSETS_43, 6)
    se = torch.randn(43, D, generator=torch.Generator().manual_seed(3)) * 0.3
    leaf = lambda t: t.to(dev).requires_grad_(True)
    qkv_d, pb_d, gain_d, se_d = leaf(qkv), leaf(pb), leaf(gain), leaf(se)
    y = dwarf_b200.dsqg_attention_packed(qkv_d, pb_d, gain_d, None, O.OFFSETS_43, scale_embed=se_d)
    y.backward(dy.to(dev))
    q, k, v = (qkv.to(dev)[:, :, i].permute(0, 2, 1, 3).contiguous().requires_grad_(True) for i in range(3))
    pb2, gain2, se2 = leaf(pb), leaf(gain), leaf(se)
    o = dwarf_b200.dsqg_attention(q, k, v, pb2, gain2, se2, O.OFFSETS_43)
    o.backward(dy.to(dev).view(B, N, H, D).permute(0, 2, 1, 3).contiguous())
    assert torch.equal(y.detach(), o.detach().permute(0, 2, 1, 3).reshape(B, N, H * D))
    for i, t in enumerate((q, k, v)):
        assert torch.equal(qkv_d.grad[:, :, i], t.grad.permute(0, 2, 1, 3))
    assert torch.equal(pb_d.grad, pb2.grad) and torch.equal(gain_d.grad, gain2.grad) and torch.equal(se_d.grad, se2.grad)


def test_condu_layer_with_kv_injection_takes_the_packed_path_and_matches_the_copy_path():
    """DSQGAttentionQW (scale_embed, if_gain) with kv_inject under autocast: the injection becomes two
    in-place adds on the projection output (train/train_2048_condU.py:178-181); output and every
    gradient, the deltas' included, agree with the copy path."""
    dev = torch.device("cuda", 0)
    torch.manual_seed(4)
    m = dwarf_b200.DSQGAttentionQW(256, 8, dropout=0.0, offsets=O.OFFSETS_44).to(dev)
    with torch.no_grad():
        m.scale_embed.normal_(0, 0.2)
        m.if_gain.uniform_(0.8, 1.2)
    B, N = 2, 333
    x = torch.randn(B, N, 256, device=dev, requires_grad=True)
    kd = (torch.randn(B, 8, N, 32, device=dev) * 0.3).requires_grad_(True)
    vd = (torch.randn(B, 8, N, 32, device=dev) * 0.3).requires_grad_(True)

    def run(packed):
        m._packed = packed
        for p in list(m.parameters()) + [x, kd, vd]:
            p.grad = None
        with torch.amp.autocast("cuda", dtype=torch.bfloat16):
            y = m(x, kv_inject=(kd.bfloat16(), vd.bfloat16()))
        (y.float() * torch.linspace(-1, 1, 256, device=dev)).sum().backward()
        return (y.detach().float(), x.grad.clone(), kd.grad.clone(), vd.grad.clone(), m.scale_embed.grad.clone(),
                m.pos_bias.grad.clone(), m.if_gain.grad.clone())

    a, b = run(None), run(False)
    assert m._packed is False
    m._packed = None
    for nm, u, w in zip(("y", "dx", "dk_delta", "dv_delta", "dscale_embed", "dpos_bias", "dif_gain"), a, b):
        scale = w.abs().max().item() + 1e-6
        assert (u - w).abs().max().item() <= 2e-2 * max(1.0, scale), nm
    # the key/value tensors handed to a decode cache are the injected ones
    with torch.no_grad(), torch.amp.autocast("cuda", dtype=torch.bfloat16):
        _, k_seen, _ = m.attend(x, kv_inject=(kd.bfloat16(), vd.bfloat16()))
        qkv = m.qkv_proj(x).view(B, N, 3, 8, 32)
        want = (qkv[:, :, 1].permute(0, 2, 1, 3) + kd.bfloat16())
    assert torch.equal(k_seen, want)


def test_strided_entries_refuse_what_they_cannot_take():
    from dwarf_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    x = torch.zeros(4096, device=dev, dtype=torch.bfloat16)
    p = x.data_ptr()
    off, J = _lib.offsets_array(O.OFFSETS_43)
    ok = _lib.Strides(3 * 2 * 32 * 16, 32, 3 * 2 * 32)
    odd = _lib.Strides(3 * 2 * 32 * 16, 32, 3 * 2 * 32 + 4)
    f32 = torch.zeros(64, device=dev).data_ptr()
    args = lambda st, D, dt: (p, p, p, st, f32, None, off, J, p, st, None, f32, 1, 2, 16, D, dt, None, 0.0)
    assert lib.dsqg_fwd_strided(*args(odd, 32, 0)) == -5             # strides must be multiples of 8 elements
    assert lib.dsqg_fwd_strided(*args(ok, 80, 0)) == -8              # no tensor-core kernel for this width
    assert lib.dsqg_fwd_strided(*args(ok, 32, 1)) == -8              # fp32
    assert not dwarf_b200.packed_path_available(80, O.OFFSETS_43)


# ------------------------------------------------------------------ causal mean (interference pooling)
@pytest.mark.parametrize("shape", [(2, 2048, 256), (3, 777, 64), (1, 1, 8), (2, 33, 40), (1, 4096, 768)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_causal_mean_forward_and_backward_vs_float64(shape, dtype):
    """out[n] = mean(x[0..n]) and its adjoint against float64 numpy (the reference computes
    `xi.cumsum(dim=1) / counts`, train/train_2048_condU.py:289-292)."""
    import numpy as np
    B, N, D = shape
    g = torch.Generator().manual_seed(N + D)
    x = torch.randn(B, N, D, generator=g).to(dtype)
    dy = torch.randn(B, N, D, generator=g).to(dtype)
    counts = np.arange(1, N + 1, dtype=np.float64)[None, :, None]
    ref = np.cumsum(x.double().numpy(), axis=1) / counts
    ref_dx = np.flip(np.cumsum(np.flip(dy.double().numpy() / counts, axis=1), axis=1), axis=1)
    xd = x.to("cuda:0").requires_grad_(True)
    y = dwarf_b200.causal_mean(xd)
    y.backward(dy.to("cuda:0"))
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -8
    for got, want, nm in ((y.detach(), ref, "out"), (xd.grad, ref_dx, "dx")):
        err = np.abs(got.double().cpu().numpy() - want)
        assert (err <= tol * (np.abs(want) + 1.0)).all(), (nm, err.max())
    # fp16 activations (the reference's autocast default) go through fp32
    assert dwarf_b200.causal_mean(x.half().to("cuda:0")).dtype == torch.float16


def test_interference_injection_feeds_kv_inject_like_the_reference_block():
    """The reference's interference block (train/train_2048_condU.py:283-297) written with PyTorch's
    cumsum against InterferenceInjection + DSQGAttentionQW(kv_inject=...): same output, same gradient."""
    dev = torch.device("cuda", 0)
    torch.manual_seed(4)
    E, H, N = 64, 2, 150
    inj = dwarf_b200.InterferenceInjection(E, H).to(dev)
    attn = dwarf_b200.DSQGAttentionQW(E, H, dropout=0.0).to(dev)
    x = torch.randn(2, N, E, device=dev, requires_grad=True)

    def reference_deltas(x):
        xi = inj.inter_norm(x)
        counts = torch.arange(1, N + 1, device=dev, dtype=xi.dtype).view(1, N, 1)
        pool = xi.cumsum(dim=1) / counts
        inter = torch.sigmoid(inj.inter_gate(xi)) * pool
        f = lambda t: t.view(2, N, H, E // H).permute(0, 2, 1, 3).contiguous()
        return f(inj.inter_k_proj(inter)), f(inj.inter_v_proj(inter))

    ya = attn(x, kv_inject=inj(x)); ya.sum().backward(); ga = x.grad.clone(); x.grad = None
    yb = attn(x, kv_inject=reference_deltas(x)); yb.sum().backward(); gb = x.grad.clone()
    assert (ya - yb).abs().max().item() < 2e-2 and (ga - gb).abs().max().item() < 2e-2 * max(1.0, gb.abs().max().item())


def test_strided_entries_take_any_row_layouts_not_only_the_packed_one():
    """q, k, v as three separate token-major tensors [B,N,H,D] and a head-major result [B,H,N,D]
    (different strides for inputs and output), straight through the C ABI: bitwise the contiguous kernels."""
    from dwarf_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, N, H, D = 2, 257, 3, 64
    offsets = O.OFFSETS_44
    g = torch.Generator().manual_seed(21)
    q, k, v = ((torch.randn(B, N, H, D, generator=g) * 0.5).bfloat16().to(dev) for _ in range(3))      # token-major
    dout = torch.randn(B, H, N, D, generator=g).bfloat16().to(dev)                                      # head-major
    pb = (synth.log_linear_pos_bias(offsets, H)).to(dev)
    off, J = _lib.offsets_array(offsets)
    st = torch.cuda.current_stream().cuda_stream
    tok, head = _lib.Strides(N * H * D, D, H * D), _lib.Strides(H * N * D, N * D, D)
    out = torch.empty(B, H, N, D, device=dev, dtype=torch.bfloat16); lse = torch.empty(B, H, N, device=dev)
    _lib.check(lib.dsqg_fwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), tok, pb.data_ptr(), None, off, J,
                                    out.data_ptr(), head, None, lse.data_ptr(), B, H, N, D, 0, st, 0.0), "fwd")
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    dpb = torch.empty(J, H, device=dev)
    nbytes = lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, 0)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    _lib.check(lib.dsqg_bwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), tok, pb.data_ptr(), None, off, J,
                                    out.data_ptr(), lse.data_ptr(), dout.data_ptr(), head, None,
                                    dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dpb.data_ptr(), None,
                                    scratch.data_ptr(), nbytes, B, H, N, D, 0, st, 0.0), "bwd")
    qc, kc, vc = (t.permute(0, 2, 1, 3).contiguous().requires_grad_(True) for t in (q, k, v))
    pb2 = pb.clone().requires_grad_(True)
    ref = dwarf_b200.dsqg_attention(qc, kc, vc, pb2, None, None, offsets)
    ref.backward(dout)
    assert torch.equal(out, ref.detach())
    for got, want in ((dq, qc.grad), (dk, kc.grad), (dv, vc.grad)):
        assert torch.equal(got, want.permute(0, 2, 1, 3))
    assert torch.equal(dpb, pb2.grad)
