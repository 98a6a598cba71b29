"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracles
and the committed golden vectors of the reference.  Run with `pytest -m gpu` on a B200."""
import ctypes

import pytest
import torch

import dwarf_b200
from dwarf_b200 import _lib, synth
from oracle import dsqg_oracle as O
from tests.gpu_util import (BF16_ABS_TOL, FP32_REL_TOL, PARAM_REL_TOL_BF16, assert_bf16_close, assert_param_grad_close,
                            cuda_fwd_bwd, oracle_fwd_bwd, rel_inf)
from tests.helpers import GOLDEN_FN_CASES, GOLDEN_MODULE_CASES, load_case

pytestmark = pytest.mark.gpu


def bf16_valued(*shape, scale=1.0, gen=None):
    return (torch.randn(*shape, generator=gen) * scale).to(torch.bfloat16).float()


# ------------------------------------------------------------------ golden vectors
@pytest.mark.parametrize("name", GOLDEN_FN_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_golden_function_cases(golden, name, dtype):
    c = load_case(golden, name)
    if dtype == torch.bfloat16 and not c["bf16"]:
        pytest.skip("fp32-valued inputs are not representable in bf16")
    r = cuda_fwd_bwd(c["q"], c["k"], c["v"], c["pos_bias"], c["dout"], c.get("scale_embed"), None,
                     c["offsets"], dtype)
    names = ["out", "dq", "dk", "dv"]
    if dtype == torch.float32:
        for nm in names:
            assert rel_inf(r[nm], c[nm]) < FP32_REL_TOL, (nm, rel_inf(r[nm], c[nm]))
        assert_param_grad_close(r["dpb"], c["dpb"], "dpb", 5e-5)
        if "dse" in c: assert_param_grad_close(r["dse"], c["dse"], "dse", 5e-5)
    else:
        for nm in names:
            assert_bf16_close(r[nm], c[nm], nm)
        assert_param_grad_close(r["dpb"], c["dpb"], "dpb", PARAM_REL_TOL_BF16)
        if "dse" in c: assert_param_grad_close(r["dse"], c["dse"], "dse", PARAM_REL_TOL_BF16)


@pytest.mark.parametrize("name", GOLDEN_MODULE_CASES)
def test_golden_other_offset_sets_fp32(golden, name):
    c = load_case(golden, name)
    r = cuda_fwd_bwd(c["q"], c["k"], c["v"], c["pos_bias"], offsets=c["offsets"], dtype=torch.float32)
    assert rel_inf(r["out"], c["out"]) < FP32_REL_TOL


# ------------------------------------------------------------------ seeded shapes vs oracle
# the reference's own self-test shapes (kernels/dsqg_attention_v2.py:508-513), trimmed in B
REF_SHAPES = [(1, 8, 64, 32), (2, 8, 512, 32), (2, 8, 2047, 32), (1, 4, 2047, 80), (2, 3, 300, 64),
              (1, 2, 1700, 128), (1, 1, 1, 32), (1, 2, 33, 16)]


@pytest.fixture(params=["auto", "generic", "mma", "tma", "tcgen05"])
def kernel_path(request):
    """Runs a test with the automatic kernel choice, with the generic CUDA-core kernels forced, with
    the tensor-core kernels, with the forward that stages V through the copy engine, and with the
    tcgen05 forward (which takes dense-only offset sets and hands every other set to the tensor-core
    kernels); no bounded wait may have given up."""
    lib = _lib.load()
    lib.dsqg_set_kernel_path({"auto": 0, "generic": 1, "mma": 2, "tma": 3, "tcgen05": 4}[request.param])
    yield request.param
    lib.dsqg_set_kernel_path(0)
    assert lib.dsqg_device_error(1) == 0, "a bounded device-side wait gave up"


@pytest.mark.parametrize("shape", REF_SHAPES)
@pytest.mark.parametrize("offsets", [O.OFFSETS_44, O.OFFSETS_43, O.OFFSETS_45,
                                     tuple(range(41)) + (128, 384, 1536), tuple(range(2, 60)) + (64, 1000)],
                         ids=["J44", "J43", "J45", "d41", "odd"])
def test_bf16_forward_backward_vs_oracle(shape, offsets, kernel_path):
    B, H, N, D = shape
    g = torch.Generator().manual_seed(42 + N + D)
    q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
    dout = bf16_valued(B, H, N, D, gen=g)
    pb = synth.log_linear_pos_bias(offsets, H) + torch.randn(len(offsets), H, generator=g) * 0.05
    gain = torch.rand(H, generator=g) * 0.4 + 0.8
    ref = oracle_fwd_bwd(q, k, v, pb, dout, None, gain, offsets)
    r = cuda_fwd_bwd(q, k, v, pb, dout, None, gain, offsets, torch.bfloat16)
    for nm in ("out", "dq", "dk", "dv"):
        assert_bf16_close(r[nm], ref[nm], nm)
    assert_param_grad_close(r["dpb"], ref["dpb"], "dpb", PARAM_REL_TOL_BF16)
    assert_param_grad_close(r["dgain"], ref["dgain"], "dgain", PARAM_REL_TOL_BF16)


@pytest.mark.parametrize("poison", [float("nan"), float("inf"), -3.0e38])
@pytest.mark.parametrize("shape", [(3, 2, 9, 32), (3, 2, 33, 32), (2, 2, 70, 32), (2, 3, 45, 64), (1, 2, 2047, 32), (1, 2, 41, 96)])
@pytest.mark.parametrize("with_se", [False, True])
def test_memory_around_the_tensors_is_never_used(shape, poison, with_se, kernel_path):
    """q, k, v and dout sit inside buffers of NaN / Inf / huge values: a tile that reaches past row
    N-1 of the last (b,h) must not let what lies behind the tensor into any result.  The offset
    set has small sparse taps (5, 6 after a dense run 0..3), which pair the missing rows of such a
    tile with key rows past the end inside the same 8-row group as existing ones."""
    B, H, N, D = shape
    offsets = (0, 1, 2, 3, 5, 6, 64, 150)
    g = torch.Generator().manual_seed(7 + N + D)
    q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
    dout = bf16_valued(B, H, N, D, gen=g)
    pb = torch.randn(len(offsets), H, generator=g) * 0.5
    gain = torch.rand(H, generator=g) * 0.4 + 0.8
    se = torch.randn(len(offsets), D, generator=g) * 0.05 if with_se else None
    ref = oracle_fwd_bwd(q, k, v, pb, dout, se, gain, offsets)
    r = cuda_fwd_bwd(q, k, v, pb, dout, se, gain, offsets, torch.bfloat16, poison=poison)
    for nm in ("out", "dq", "dk", "dv"):
        assert_bf16_close(r[nm], ref[nm], nm)
    assert_param_grad_close(r["dpb"], ref["dpb"], "dpb", PARAM_REL_TOL_BF16)
    assert_param_grad_close(r["dgain"], ref["dgain"], "dgain", PARAM_REL_TOL_BF16)
    if with_se:
        assert_param_grad_close(r["dse"], ref["dse"], "dse", PARAM_REL_TOL_BF16)


@pytest.mark.parametrize("shape", [(2, 3, 700, 80), (1, 2, 300, 48), (1, 2, 90, 80), (1, 1, 2047, 80)])
@pytest.mark.parametrize("offsets", [O.OFFSETS_43, O.OFFSETS_44, tuple(range(41)) + (128, 384, 1536)],
                         ids=["J43", "J44", "d41"])
def test_bf16_odd_head_widths_run_zero_padded_on_the_tensor_core_kernels(shape, offsets):
    """HD = 80 (the reference's 85M condM model) and 48: the operator pads the head dimension with
    zero columns to 96 / 64 when the tensor-core kernels take the padded problem and passes the
    true 1/sqrt(HD); results and gradients have the caller's width and match the oracle."""
    B, H, N, D = shape
    lib = _lib.load()
    off, J = _lib.offsets_array(offsets)
    padded = (D + 31) // 32 * 32
    assert lib.dsqg_tensor_core_path(0, D, off, J, 0) == 0
    takes_padded = lib.dsqg_tensor_core_path(0, padded, off, J, 0) == 1
    assert takes_padded == (padded == 64 or offsets[32] != 32 or offsets[33] != 33)   # wide heads: dense window up to 32
    g = torch.Generator().manual_seed(5 + N + D)
    q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
    dout = bf16_valued(B, H, N, D, gen=g)
    pb = synth.log_linear_pos_bias(offsets, H) + torch.randn(len(offsets), H, generator=g) * 0.05
    gain = torch.rand(H, generator=g) * 0.4 + 0.8
    ref = oracle_fwd_bwd(q, k, v, pb, dout, None, gain, offsets)
    r = cuda_fwd_bwd(q, k, v, pb, dout, None, gain, offsets, torch.bfloat16)
    for nm in ("out", "dq", "dk", "dv"):
        assert r[nm].shape == (B, H, N, D)
        assert_bf16_close(r[nm], ref[nm], nm)
    assert_param_grad_close(r["dpb"], ref["dpb"], "dpb", PARAM_REL_TOL_BF16)
    assert_param_grad_close(r["dgain"], ref["dgain"], "dgain", PARAM_REL_TOL_BF16)


@pytest.mark.parametrize("shape", [(1, 2, 333, 96), (2, 2, 1700, 128), (1, 3, 40, 128)])
@pytest.mark.parametrize("path", ["auto", "generic"])
def test_bf16_wide_heads_vs_oracle(shape, path):
    """D = 96 and 128: tensor-core kernels for the 32-wide dense window, generic kernels forced
    as the cross-check."""
    lib = _lib.load()
    lib.dsqg_set_kernel_path(1 if path == "generic" else 0)
    try:
        B, H, N, D = shape
        g = torch.Generator().manual_seed(7 + N + D)
        q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
        dout = bf16_valued(B, H, N, D, gen=g)
        pb = synth.log_linear_pos_bias(O.OFFSETS_43, H) + torch.randn(43, H, generator=g) * 0.05
        gain = torch.rand(H, generator=g) * 0.4 + 0.8
        ref = oracle_fwd_bwd(q, k, v, pb, dout, None, gain, O.OFFSETS_43)
        r = cuda_fwd_bwd(q, k, v, pb, dout, None, gain, O.OFFSETS_43, torch.bfloat16)
        for nm in ("out", "dq", "dk", "dv"):
            assert_bf16_close(r[nm], ref[nm], nm)
        assert_param_grad_close(r["dpb"], ref["dpb"], "dpb", PARAM_REL_TOL_BF16)
        assert_param_grad_close(r["dgain"], ref["dgain"], "dgain", PARAM_REL_TOL_BF16)
    finally:
        lib.dsqg_set_kernel_path(0)


@pytest.mark.parametrize("shape", [(1, 4, 64, 32), (2, 2, 1600, 32), (1, 3, 200, 64), (1, 2, 100, 80),
                                   (1, 2, 576, 32), (1, 2, 2047, 64), (1, 1, 1, 32), (2, 1, 17, 64)])
def test_bf16_scale_embed_and_gain_vs_oracle(shape):
    B, H, N, D = shape
    g = torch.Generator().manual_seed(7 + N)
    q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
    dout = bf16_valued(B, H, N, D, gen=g)
    pb = torch.randn(44, H, generator=g) * 0.5
    se = torch.randn(44, D, generator=g) * 0.05
    gain = torch.rand(H, generator=g) + 0.5
    ref = oracle_fwd_bwd(q, k, v, pb, dout, se, gain, O.OFFSETS_44)
    r = cuda_fwd_bwd(q, k, v, pb, dout, se, gain, O.OFFSETS_44, torch.bfloat16)
    for nm in ("out", "dq", "dk", "dv"):
        assert_bf16_close(r[nm], ref[nm], nm)
    for nm in ("dpb", "dse", "dgain"):
        assert_param_grad_close(r[nm], ref[nm], nm, PARAM_REL_TOL_BF16)


@pytest.mark.parametrize("shape", [(1, 8, 64, 32), (2, 4, 777, 32), (1, 2, 1600, 64), (1, 1, 90, 80)])
def test_fp32_forward_backward_vs_oracle_1e5(shape):
    B, H, N, D = shape
    g = torch.Generator().manual_seed(11 + N)
    q, k, v, dout = (torch.randn(B, H, N, D, generator=g) for _ in range(4))
    pb = synth.log_linear_pos_bias(O.OFFSETS_43, H)
    se = torch.randn(43, D, generator=g) * 0.05
    gain = torch.rand(H, generator=g) + 0.5
    ref = oracle_fwd_bwd(q, k, v, pb, dout, se, gain, O.OFFSETS_43)
    r = cuda_fwd_bwd(q, k, v, pb, dout, se, gain, O.OFFSETS_43, torch.float32)
    for nm in ("out", "dq", "dk", "dv"):
        assert rel_inf(r[nm], ref[nm]) < FP32_REL_TOL, (nm, rel_inf(r[nm], ref[nm]))
    for nm in ("dpb", "dse", "dgain"):
        assert_param_grad_close(r[nm], ref[nm], nm, 5e-5)


def test_config0_fp32_forward_gate():
    """Benchmark configuration 0 (B2 H8 N2048 D32 fp32, 43 offsets) against the PyTorch
    restatement of the reference: <= 1e-5 relative."""
    cfg = synth.OP_CONFIGS["cfg0"]
    x = synth.make_op_inputs(cfg, with_dout=False)
    ref = O.dsqg_reference_chunked(x["q"], x["k"], x["v"], x["pos_bias"], None, None, cfg.offsets, chunk=1)
    r = cuda_fwd_bwd(x["q"], x["k"], x["v"], x["pos_bias"], offsets=cfg.offsets, dtype=torch.float32)
    assert rel_inf(r["out"], ref) < FP32_REL_TOL


# ------------------------------------------------------------------ identities and edge cases
def test_v3_with_zero_scale_embed_equals_v2():
    # kernels/dsqg_attention_v3.py:612-628
    torch.manual_seed(7)
    dev = "cuda:0"
    q, k, v = (torch.randn(2, 8, 128, 32, device=dev, dtype=torch.bfloat16) * 0.1 for _ in range(3))
    pb = torch.randn(44, 8, device=dev) * 0.5
    a = dwarf_b200.dsqg_attention_v2(q, k, v, pb)
    b = dwarf_b200.dsqg_attention_v3(q, k, v, pb, torch.zeros(44, 32, device=dev))
    assert (a.float() - b.float()).abs().max().item() < 1e-3


def test_softmax_weights_sum_to_one_and_gain_scales_output():
    dev = "cuda:0"
    g = torch.Generator().manual_seed(3)
    B, H, N, D = 2, 8, 2048, 32
    q, k = (bf16_valued(B, H, N, D, scale=0.5, gen=g).to(dev, torch.bfloat16) for _ in range(2))
    v = torch.ones(B, H, N, D, device=dev, dtype=torch.bfloat16)
    pb = synth.log_linear_pos_bias(O.OFFSETS_43, H).to(dev)
    gain = torch.tensor([0.5, 1.0, 2.0, 4.0, 0.25, 1.0, 1.0, 8.0], device=dev)
    out = dwarf_b200.dsqg_attention(q, k, v, pb, gain, None, O.OFFSETS_43).float()
    assert (out - gain.view(1, H, 1, 1)).abs().max().item() <= 2e-2 * 8


def test_offset_set_without_zero_gives_zero_rows_and_finite_grads():
    dev = "cuda:0"
    offsets = (1, 2, 3, 8)
    g = torch.Generator().manual_seed(5)
    B, H, N, D = 1, 2, 40, 32
    q, k, v = (bf16_valued(B, H, N, D, gen=g) for _ in range(3))
    dout = bf16_valued(B, H, N, D, gen=g)
    pb = torch.randn(4, H, generator=g)
    ref = oracle_fwd_bwd(q, k, v, pb, dout, None, None, offsets)
    for dtype in (torch.bfloat16, torch.float32):
        r = cuda_fwd_bwd(q, k, v, pb, dout, None, None, offsets, dtype)
        assert torch.all(r["out"][:, :, 0] == 0)
        for nm in ("out", "dq", "dk", "dv"):
            assert torch.isfinite(r[nm]).all()
            assert_bf16_close(r[nm], ref[nm], nm)
    out, lse = dwarf_b200.dsqg_forward_lse(q.to(dev, torch.bfloat16), k.to(dev, torch.bfloat16),
                                           v.to(dev, torch.bfloat16), pb.to(dev), offsets=offsets)
    assert torch.all(lse[:, :, 0] == float("-inf")) and torch.isfinite(lse[:, :, 1:]).all()


def test_lse_matches_oracle():
    g = torch.Generator().manual_seed(8)
    B, H, N, D = 1, 4, 1600, 32
    q, k, v = (bf16_valued(B, H, N, D, scale=0.5, gen=g) for _ in range(3))
    pb = torch.randn(44, H, generator=g) * 0.5
    ref = oracle_fwd_bwd(q, k, v, pb, None, None, None, O.OFFSETS_44)
    dev = "cuda:0"
    for dtype, tol in ((torch.bfloat16, 2e-3), (torch.float32, 2e-5)):
        _, lse = dwarf_b200.dsqg_forward_lse(q.to(dev, dtype), k.to(dev, dtype), v.to(dev, dtype),
                                             pb.to(dev), offsets=O.OFFSETS_44)
        assert (lse.cpu() - ref["lse"]).abs().max().item() < tol


def test_causality_on_gpu():
    # perturb position 10: rows < 10 must not change (train_2048_condM_layer_ablation.py:410-426)
    dev = "cuda:0"
    torch.manual_seed(1)
    q, k, v = (torch.randn(1, 8, 64, 32, device=dev, dtype=torch.bfloat16) for _ in range(3))
    pb = torch.randn(44, 8, device=dev)
    a = dwarf_b200.dsqg_attention_v2(q, k, v, pb)
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 10] += 1; v2[:, :, 10] -= 1
    b = dwarf_b200.dsqg_attention_v2(q, k2, v2, pb)
    assert torch.equal(a[:, :, :10], b[:, :, :10]) and not torch.equal(a[:, :, 10:], b[:, :, 10:])


def test_bitwise_determinism_and_no_unwritten_rows():
    """No atomics anywhere: two runs are bit-identical.  Outputs are poison-filled before the
    launch (direct C-ABI call) so that an unwritten row would show up as NaN."""
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(9)
    B, H, N, D = 3, 8, 2047, 32
    mk = lambda: bf16_valued(B, H, N, D, scale=0.5, gen=g).to(dev, torch.bfloat16)
    q, k, v, dout = mk(), mk(), mk(), mk()
    pb = (torch.randn(43, H, generator=g) * 0.5).to(dev)
    se = (torch.randn(43, D, generator=g) * 0.05).to(dev)
    gain = (torch.rand(H, generator=g) + 0.5).to(dev)
    off, J = _lib.offsets_array(O.OFFSETS_43)
    stream = torch.cuda.current_stream().cuda_stream

    def run():
        nan = float("nan")
        out = torch.full_like(q, nan); lse = torch.full((B, H, N), nan, device=dev)
        dq, dk, dv = (torch.full_like(q, nan) for _ in range(3))
        dpb = torch.full((J, H), nan, device=dev); dse = torch.full((J, D), nan, device=dev)
        dg = torch.full((H,), nan, device=dev)
        nbytes = lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, 1)
        scratch = torch.full((nbytes // 4,), nan, device=dev)
        _lib.check(lib.dsqg_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), se.data_ptr(),
                                gain.data_ptr(), off, J, out.data_ptr(), lse.data_ptr(), B, H, N, D, 0, stream), "fwd")
        _lib.check(lib.dsqg_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), se.data_ptr(),
                                gain.data_ptr(), off, J, out.data_ptr(), lse.data_ptr(), dout.data_ptr(),
                                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dpb.data_ptr(), dse.data_ptr(),
                                dg.data_ptr(), scratch.data_ptr(), nbytes, B, H, N, D, 0, stream), "bwd")
        torch.cuda.synchronize()
        return out, lse, dq, dk, dv, dpb, dse, dg

    a, b = run(), run()
    for x, y in zip(a, b):
        assert torch.isfinite(x.float()).all()
        assert torch.equal(x, y)


@pytest.mark.parametrize("with_se", [False, True])
@pytest.mark.parametrize("shape", [(3, 8, 2047, 32), (2, 3, 700, 64), (1, 2, 40, 32)])
def test_fused_parameter_reduction_equals_staged_backward_bitwise(shape, with_se):
    """Tensor-core path: one dsqg_bwd call lets the first CTAs of the dK/dV kernel finish dpos_bias
    and dhead_gain; running the three stages as separate calls uses the stand-alone reduction
    kernel.  Same additions in the same order: every output is bit-identical, none unwritten."""
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(sum(shape))
    B, H, N, D = shape
    mk = lambda: bf16_valued(B, H, N, D, scale=0.5, gen=g).to(dev, torch.bfloat16)
    q, k, v, dout = mk(), mk(), mk(), mk()
    pb = (torch.randn(43, H, generator=g) * 0.5).to(dev)
    gain = (torch.rand(H, generator=g) + 0.5).to(dev)
    se = (torch.randn(43, D, generator=g) * 0.05).to(dev) if with_se else None
    sep = se.data_ptr() if with_se else None
    off, J = _lib.offsets_array(O.OFFSETS_43)
    stream = torch.cuda.current_stream().cuda_stream
    out = torch.empty_like(q); lse = torch.empty(B, H, N, device=dev)
    _lib.check(lib.dsqg_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), sep, gain.data_ptr(),
                            off, J, out.data_ptr(), lse.data_ptr(), B, H, N, D, 0, stream), "fwd")

    def run(stage_list):
        nan = float("nan")
        dq, dk, dv = (torch.full_like(q, nan) for _ in range(3))
        dpb = torch.full((J, H), nan, device=dev); dg = torch.full((H,), nan, device=dev)
        dse = torch.full((J, D), nan, device=dev)
        nbytes = lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, int(with_se))
        scratch = torch.full((nbytes // 4,), nan, device=dev)
        for st in stage_list:
            _lib.check(lib.dsqg_bwd_stages(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), sep,
                                           gain.data_ptr(), off, J, out.data_ptr(), lse.data_ptr(), dout.data_ptr(),
                                           dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dpb.data_ptr(),
                                           dse.data_ptr() if with_se else None,
                                           dg.data_ptr(), scratch.data_ptr(), nbytes, B, H, N, D, 0, stream, st), "bwd")
        torch.cuda.synchronize()
        return (dq, dk, dv, dpb, dg) + ((dse,) if with_se else ())

    fused, staged = run([7]), run([1, 2, 4])
    for x, y in zip(fused, staged):
        assert torch.isfinite(x.float()).all()
        assert torch.equal(x, y)


def test_non_default_stream_and_checkpoint_and_autocast():
    dev = torch.device("cuda", 0)
    m = dwarf_b200.DSQGAttentionQW(256, 8, dropout=0.0).to(dev)
    with torch.no_grad():
        m.scale_embed.normal_(0, 0.05); m.if_gain.uniform_(0.8, 1.2)
    x = torch.randn(2, 256, 256, device=dev, requires_grad=True)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.amp.autocast("cuda", dtype=torch.bfloat16):
            y = torch.utils.checkpoint.checkpoint(m, x, use_reentrant=False)
        y.float().sum().backward()
    s.synchronize()
    assert torch.isfinite(x.grad).all() and torch.isfinite(m.pos_bias.grad).all()
    assert torch.isfinite(m.if_gain.grad).all() and m.scale_embed.grad.abs().sum() > 0
    # fp16 autocast (the reference's default, train_2048_condU.py:582): computed in bf16, returned fp16
    q = torch.randn(1, 8, 64, 32, device=dev, dtype=torch.float16)
    out = dwarf_b200.dsqg_attention_v2(q, q, q, m.pos_bias.detach())
    assert out.dtype == torch.float16


def test_module_matches_reference_module_math():
    """DSQGAttentionN_Fused on the GPU against the same module math evaluated with the oracle."""
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    m = dwarf_b200.DSQGAttentionN_Fused(64, 2, dropout=0.0, offsets=O.OFFSETS_43).eval()
    x = torch.randn(1, 100, 64)
    with torch.no_grad():
        qkv = m.qkv_proj(x)
        q, k, v = (t.view(1, 100, 2, 32).permute(0, 2, 1, 3).bfloat16().float() for t in qkv.split(64, -1))
        o = O.dsqg_reference(q, k, v, m.pos_bias, None, None, O.OFFSETS_43)
        ref = m.out_proj(o.permute(0, 2, 1, 3).reshape(1, 100, 64) * torch.sigmoid(m.gate_proj(x)))
        got = m.to(dev)(x.to(dev)).cpu()
    assert (got - ref).abs().max().item() < 2e-2


def test_gpu_argument_errors_raise_with_status():
    dev = torch.device("cuda", 0)
    q = torch.zeros(1, 2, 16, 32, device=dev, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        dwarf_b200.dsqg_attention(q, q, q, torch.zeros(43, 2, device=dev))          # J mismatch
    with pytest.raises(dwarf_b200.DSQGError) as e:
        dwarf_b200.dsqg_attention(q, q, q, torch.zeros(3, 2, device=dev), offsets=(0, 2, 1))
    assert e.value.status == -3
    q12 = torch.zeros(1, 2, 16, 12, device=dev, dtype=torch.bfloat16)
    with pytest.raises(dwarf_b200.DSQGError) as e:
        dwarf_b200.dsqg_attention(q12, q12, q12, torch.zeros(44, 2, device=dev))
    assert e.value.status == -2
    # the context is still usable afterwards
    out = dwarf_b200.dsqg_attention(q, q, q, torch.zeros(44, 2, device=dev))
    assert torch.isfinite(out.float()).all()


# ------------------------------------------------------------------ full benchmark sizes
# Tensors that meet the benchmark's plain bound (|x - ref| <= 2e-2, no term relative to the value) on the
# whole batch.  dv at cfg1 is the one exception: its largest values are near 4.5, where one bf16 rounding
# step of the stored result is 0.031, and its largest error is 0.0215; it keeps the bound that adds the
# rounding of the stored value (2e-2 + 2^-8 |ref|).
PLAIN_2E2 = {"cfg1": ("out", "dq", "dk"), "cfg2": ("out", "dq", "dk", "dv"), "cfg2_4k": ("out", "dq", "dk", "dv")}


@pytest.mark.parametrize("cfg_name", ["cfg1", "cfg2", "cfg2_4k"])
def test_full_size_configs_vs_c_oracle_whole_batch(cfg_name, record_property):
    """Full benchmark shape on the GPU against the (threaded, double-accumulating) C oracle on every
    batch entry: out, dq, dk, dv element-wise, dpos_bias and dhead_gain (sums over all B*N rows of a
    head) to 1 % of their largest entry.  The largest absolute error of every tensor is printed and
    recorded."""
    cfg = synth.OP_CONFIGS[cfg_name]
    x = synth.make_op_inputs(cfg)
    r = cuda_fwd_bwd(x["q"], x["k"], x["v"], x["pos_bias"], x["dout"], None, x["head_gain"],
                     cfg.offsets, cfg.dtype)
    f = lambda t: t.float()
    ref = oracle_fwd_bwd(f(x["q"]), f(x["k"]), f(x["v"]), x["pos_bias"], f(x["dout"]), None,
                         x["head_gain"], cfg.offsets)
    for nm in ("out", "dq", "dk", "dv", "dpb", "dgain"):
        err = (r[nm].double() - ref[nm].double()).abs().max().item()
        record_property(f"{cfg_name}_{nm}_max_abs_err", err)
        print(f"{cfg_name} {nm}: max abs err {err:.4g} (|ref| max {ref[nm].abs().max().item():.4g})")
    for nm in ("out", "dq", "dk", "dv"):
        assert torch.isfinite(r[nm]).all()
        if nm in PLAIN_2E2[cfg_name]:
            err = (r[nm].double() - ref[nm].double()).abs().max().item()
            assert err <= BF16_ABS_TOL, f"{nm}: max abs err {err:.4g} > {BF16_ABS_TOL}"
        else:
            assert_bf16_close(r[nm], ref[nm], nm)
    assert_param_grad_close(r["dpb"], ref["dpb"], "dpb", 1e-2, abs_floor=0.0)
    assert_param_grad_close(r["dgain"], ref["dgain"], "dgain", 1e-3, abs_floor=0.0)
    # row 0 of every (b,h) attends only to itself: out[0] = gain * v[0]
    want = x["v"][:, :, 0].float() * x["head_gain"].view(1, cfg.H, 1)
    assert (r["out"][:, :, 0] - want).abs().max().item() <= BF16_ABS_TOL


# ------------------------------------------------------------------ gather index and causal mask, read directly
@pytest.mark.parametrize("offsets", [O.OFFSETS_43, O.OFFSETS_44, O.OFFSETS_45], ids=["J43", "J44", "J45"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("coding", ["mod", "div"])
def test_gather_index_and_mask_are_exact(offsets, dtype, coding):
    """q = 0 and pos_bias = 0 make every valid tap of a row weigh 1/count.  With V rows one-hot in
    `n mod 128` (first pass) and in `n div 128` (second pass; D = 128) the output row n is a histogram of
    the value rows the kernel gathered: it must be non-zero exactly at the codes of the rows n - delta_j
    with n - delta_j >= 0 (the gather index and mask of kernels/dsqg_attention_v2.py:491,495), exactly zero
    elsewhere, and multiplicity / count where it is non-zero."""
    B, H, N, D = 1, 2, 1800, 128
    n = torch.arange(N)
    code = (n % 128) if coding == "mod" else (n // 128)
    v = torch.zeros(B, H, N, D)
    v[:, :, n, code] = 1.0
    q = torch.zeros(B, H, N, D)
    k = (torch.randn(B, H, N, D, generator=torch.Generator().manual_seed(1)) * 0.5).bfloat16().float()   # irrelevant: q = 0
    pb = torch.zeros(len(offsets), H)
    r = cuda_fwd_bwd(q, k, v, pb, None, None, None, offsets, dtype)["out"]
    off = torch.tensor(offsets)
    src = n[:, None] - off[None, :]                          # [N, J] gathered row index
    valid = src >= 0
    hist = torch.zeros(N, D)
    rows = n[:, None].expand_as(src)[valid]
    hist.index_put_((rows, code[src[valid]]), torch.ones(int(valid.sum())), accumulate=True)
    count = valid.sum(1).float()
    want = hist / count[:, None]
    for h in range(H):
        got = r[0, h]
        assert torch.equal(got != 0, hist != 0), "the set of gathered rows differs from {n - delta_j >= 0}"
        tol = 1e-6 if dtype == torch.float32 else 2.0 ** -7          # one rounding step of the stored bf16 value
        assert ((got - want).abs() <= tol * want).all()


def test_module_kv_inject_matches_oracle():
    """K/V injection hook of the condU attention (train/train_2048_condU.py:178-181): k += k_delta,
    v += v_delta before the op.  Module output and the gradients that reach the injected tensors
    against the same module math evaluated with the oracle."""
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    E, Hh, N = 64, 2, 90
    m = dwarf_b200.DSQGAttentionQW(E, Hh, dropout=0.0, offsets=O.OFFSETS_43).eval()
    with torch.no_grad():
        m.scale_embed.normal_(0, 0.05); m.if_gain.uniform_(0.8, 1.2)
    x = torch.randn(1, N, E)
    kd = (torch.randn(1, Hh, N, E // Hh) * 0.3).requires_grad_(True)
    vd = (torch.randn(1, Hh, N, E // Hh) * 0.3).requires_grad_(True)
    # oracle side: same projections, injection, bf16 rounding of q, k, v as the module does
    qkv = m.qkv_proj(x)
    q, k, v = (t.view(1, N, Hh, E // Hh).permute(0, 2, 1, 3) for t in qkv.split(E, -1))
    rnd = lambda t: t + (t.bfloat16().float() - t).detach()          # value rounding, identity gradient
    o = O.dsqg_reference(rnd(q), rnd(k + kd), rnd(v + vd), m.pos_bias, m.scale_embed, m.if_gain, O.OFFSETS_43)
    ref = m.out_proj(o.permute(0, 2, 1, 3).reshape(1, N, E) * torch.sigmoid(m.gate_proj(x)))
    ref.sum().backward()
    ref_gk, ref_gv = kd.grad.clone(), vd.grad.clone()
    md = m.to(dev)
    kd2 = kd.detach().to(dev).requires_grad_(True)
    vd2 = vd.detach().to(dev).requires_grad_(True)
    got = md(x.to(dev), kv_inject=(kd2, vd2))
    got.sum().backward()
    assert (got.detach().cpu() - ref.detach()).abs().max().item() < 2e-2
    assert (kd2.grad.cpu() - ref_gk).abs().max().item() < 2e-2
    assert (vd2.grad.cpu() - ref_gv).abs().max().item() < 2e-2
    without = md(x.to(dev))
    assert (without - got).abs().max().item() > 1e-3             # the injection is not a no-op


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier nothing signals runs out after its cycle limit: the kernel returns, the
    error word names the wait site, reading with reset clears it, and the context stays usable."""
    lib = _lib.load()
    assert lib.dsqg_device_error(1) >= 0
    assert lib.dsqg_device_error(0) == 0
    _lib.check(lib.dsqg_test_wait_timeout(20000, torch.cuda.current_stream().cuda_stream), "wait")
    torch.cuda.synchronize()
    assert lib.dsqg_device_error(0) == 0x7e57
    assert lib.dsqg_device_error(1) == 0x7e57
    assert lib.dsqg_device_error(0) == 0
    assert lib.dsqg_test_wait_timeout(0, None) == -8
    q = torch.zeros(1, 2, 16, 32, device="cuda:0", dtype=torch.bfloat16)
    assert torch.isfinite(dwarf_b200.dsqg_attention(q, q, q, torch.zeros(44, 2, device="cuda:0")).float()).all()
