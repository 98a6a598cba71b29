"""GPU tests of the forward whose dense window runs on tcgen05 tensor cores with accumulators in tensor
memory (kernel path 4, csrc/dsqg_umma.cu): offset sets without sparse taps, bf16, D = 32 or 64.  Checked against
the C oracle (reference math: kernels/dsqg_attention_v3.py:60-163 without scale_embed) and against the
default kernels; offset sets the path does not take must give the bits of the default kernels."""
import pytest
import torch

import dwarf_b200
from dwarf_b200 import _lib, synth
from oracle import dsqg_oracle as O
from tests.gpu_util import assert_bf16_close, oracle_fwd_bwd

pytestmark = pytest.mark.gpu


def bf16_valued(*shape, scale=1.0, gen=None):
    """fp32 tensor whose values are exactly representable in bf16."""
    return (torch.randn(*shape, generator=gen) * scale).bfloat16().float()

DENSE_SETS = {"0..32": tuple(range(33)), "0..15": tuple(range(16)), "1..20": tuple(range(1, 21)), "0": (0,),
              "5..32": tuple(range(5, 33))}


def _forward(path, q, k, v, pb, gain, offsets):
    lib = _lib.load()
    assert lib.dsqg_set_kernel_path(path) == 0
    try:
        B, H, N, D = q.shape
        out = torch.full_like(q, float("nan"))
        lse = torch.full((B, H, N), float("nan"), device=q.device)
        off, J = _lib.offsets_array(offsets)
        _lib.check(lib.dsqg_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), None,
                                None if gain is None else gain.data_ptr(), off, J, out.data_ptr(), lse.data_ptr(),
                                B, H, N, D, _lib.DSQG_DTYPE_BF16, torch.cuda.current_stream().cuda_stream), "dsqg_fwd")
        torch.cuda.synchronize()
    finally:
        lib.dsqg_set_kernel_path(0)
    assert lib.dsqg_device_error(1) == 0, "a bounded device-side wait gave up"
    return out, lse


@pytest.mark.parametrize("shape", [(1, 2, 256, 32), (2, 3, 1000, 32), (1, 1, 1, 32), (2, 2, 127, 32), (1, 3, 129, 32),
                                   (3, 8, 2048, 32), (40, 8, 640, 32),
                                   (1, 2, 256, 64), (2, 3, 1000, 64), (1, 1, 1, 64), (1, 3, 129, 64), (20, 12, 640, 64)])
@pytest.mark.parametrize("name", list(DENSE_SETS))
def test_dense_window_forward_on_tcgen05_vs_oracle_and_default_kernels(shape, name):
    B, H, N, D = shape
    offsets = DENSE_SETS[name]
    g = torch.Generator().manual_seed(7 + N + len(offsets))
    q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
    pb = synth.log_linear_pos_bias(offsets, H) + torch.randn(len(offsets), H, generator=g) * 0.05
    gain = torch.rand(H, generator=g) * 0.4 + 0.8
    ref = oracle_fwd_bwd(q, k, v, pb, None, None, gain, offsets)
    dev = torch.device("cuda", 0)
    args = [t.bfloat16().to(dev) for t in (q, k, v)] + [pb.to(dev), gain.to(dev)]
    out4, lse4 = _forward(4, *args, offsets)
    out2, lse2 = _forward(2, *args, offsets)
    assert not torch.isnan(out4).any()
    assert_bf16_close(out4.float().cpu(), ref["out"], "out")
    # rows without a valid tap (offset sets that do not start at 0): zero output, -inf lse, as the default kernels
    empty = torch.isinf(lse2)
    assert torch.equal(torch.isinf(lse4), empty)
    assert torch.equal(out4[empty], out2[empty])
    assert (lse4[~empty] - lse2[~empty]).abs().max().item() <= 2e-3 if (~empty).any() else True
    assert (out4.float() - out2.float()).abs().max().item() <= 2e-2


def test_backward_after_the_tcgen05_forward_matches_the_oracle():
    """The autograd backward consumes the out and lse the tcgen05 forward saved."""
    lib = _lib.load()
    B, H, N, D = 2, 4, 700, 32
    offsets = DENSE_SETS["0..32"]
    g = torch.Generator().manual_seed(3)
    q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
    dout = bf16_valued(B, H, N, D, gen=g)
    pb = synth.log_linear_pos_bias(offsets, H)
    ref = oracle_fwd_bwd(q, k, v, pb, dout, None, None, offsets)
    dev = torch.device("cuda", 0)
    qd, kd, vd = (t.bfloat16().to(dev).requires_grad_(True) for t in (q, k, v))
    pbd = pb.to(dev).requires_grad_(True)
    lib.dsqg_set_kernel_path(4)
    try:
        out = dwarf_b200.dsqg_attention(qd, kd, vd, pbd, None, None, offsets)
        out.backward(dout.bfloat16().to(dev))
        torch.cuda.synchronize()
    finally:
        lib.dsqg_set_kernel_path(0)
    assert lib.dsqg_device_error(1) == 0
    for nm, t in (("dq", qd), ("dk", kd), ("dv", vd)):
        assert_bf16_close(t.grad.float().cpu(), ref[nm], nm)


@pytest.mark.parametrize("shape", [(1, 2, 256, 32), (2, 3, 1000, 32), (1, 1, 1, 32), (2, 2, 127, 32), (1, 3, 129, 32),
                                   (2, 8, 2048, 32), (1, 2, 1700, 32), (20, 8, 640, 32)])
@pytest.mark.parametrize("offsets", [O.OFFSETS_43, O.OFFSETS_44, tuple(range(1, 30)) + (40, 77, 1500),
                                     tuple(range(32)) + tuple(range(40, 40 + 16 * 24, 24))],
                         ids=["J43", "J44", "odd", "16-sparse"])
def test_forward_with_sparse_taps_on_the_tcgen05_path_vs_oracle(shape, offsets):
    """Offset sets with sparse taps at D = 32: dense window on tcgen05, sparse taps by the softmax warps."""
    B, H, N, D = shape
    g = torch.Generator().manual_seed(17 + N + len(offsets))
    q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
    pb = synth.log_linear_pos_bias(offsets, H) + torch.randn(len(offsets), H, generator=g) * 0.05
    gain = torch.rand(H, generator=g) * 0.4 + 0.8
    ref = oracle_fwd_bwd(q, k, v, pb, None, None, gain, offsets)
    dev = torch.device("cuda", 0)
    args = [t.bfloat16().to(dev) for t in (q, k, v)] + [pb.to(dev), gain.to(dev)]
    out4, lse4 = _forward(4, *args, offsets)
    out2, lse2 = _forward(2, *args, offsets)
    assert not torch.isnan(out4).any()
    assert_bf16_close(out4.float().cpu(), ref["out"], "out")
    if N >= 1000:       # other arithmetic than the default kernels: equal bits would mean the path was not taken
        assert not torch.equal(out4, out2)
    empty = torch.isinf(lse2)
    assert torch.equal(torch.isinf(lse4), empty)
    if (~empty).any():
        assert (lse4[~empty] - lse2[~empty]).abs().max().item() <= 2e-3
        assert (lse4[~empty].cpu() - ref["lse"][~empty.cpu()]).abs().max().item() <= 2e-3


def test_large_sparse_scores_move_the_running_maximum():
    """A sparse tap far above the dense window's maximum (rescale path of the online softmax)."""
    B, H, N, D = 1, 2, 1600, 32
    offsets = O.OFFSETS_43
    g = torch.Generator().manual_seed(23)
    q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
    pb = synth.log_linear_pos_bias(offsets, H)
    pb[40] += 60.0                                   # offset 768 dominates wherever it is valid
    pb[35] += 25.0
    ref = oracle_fwd_bwd(q, k, v, pb, None, None, None, offsets)
    dev = torch.device("cuda", 0)
    args = [t.bfloat16().to(dev) for t in (q, k, v)] + [pb.to(dev), None]
    out4, lse4 = _forward(4, *args, offsets)
    assert_bf16_close(out4.float().cpu(), ref["out"], "out")
    assert (lse4.cpu() - ref["lse"]).abs().max().item() <= 2e-3 * max(1.0, ref["lse"].abs().max().item())


def test_what_the_path_does_not_take_falls_through_to_the_default_kernels():
    """D = 64 with sparse taps, dense windows wider than 32: the bits of the automatic choice."""
    dev = torch.device("cuda", 0)
    for (B, H, N, D), offsets in (((1, 2, 1700, 64), O.OFFSETS_43), ((1, 2, 300, 32), tuple(range(41)) + (128,))):
        g = torch.Generator().manual_seed(5)
        q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
        pb = synth.log_linear_pos_bias(offsets, H)
        args = [t.bfloat16().to(dev) for t in (q, k, v)] + [pb.to(dev), None]
        out4, lse4 = _forward(4, *args, offsets)
        out0, lse0 = _forward(0, *args, offsets)
        assert torch.equal(out4, out0) and torch.equal(lse4, lse0)


def test_the_automatic_choice_takes_the_tcgen05_forward_where_it_measures_faster():
    """D = 64, no sparse taps, at least 296 tiles of 128 rows: the bits of kernel path 4, not of the
    register-fed kernel; a smaller problem of the same kind stays on the register-fed kernel."""
    dev = torch.device("cuda", 0)
    offsets = DENSE_SETS["0..32"]
    for (B, H, N, D), uses_tcgen05 in (((5, 12, 640, 64), True), ((4, 12, 640, 64), False)):
        g = torch.Generator().manual_seed(9)
        q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
        pb = synth.log_linear_pos_bias(offsets, H)
        args = [t.bfloat16().to(dev) for t in (q, k, v)] + [pb.to(dev), None]
        out0, _ = _forward(0, *args, offsets)
        out2, _ = _forward(2, *args, offsets)
        out4, _ = _forward(4, *args, offsets)
        assert not torch.equal(out2, out4), "the two kernels round differently somewhere in a problem of this size"
        assert torch.equal(out0, out4 if uses_tcgen05 else out2), (B, H, N, D)
