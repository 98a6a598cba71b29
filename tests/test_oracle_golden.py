"""CPU tests: the oracles against the golden vectors generated from the reference itself,
and the oracles against each other.  No GPU, no reference checkout needed."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as C
from oracle import dsqg_oracle as O
from tests.helpers import (GOLDEN_FN_CASES, GOLDEN_MODULE_CASES, load_case, max_abs, rel_inf)


@pytest.mark.parametrize("name", GOLDEN_FN_CASES)
def test_torch_oracle_matches_reference_outputs(golden, name):
    c = load_case(golden, name)
    r = O.dsqg_reference_grads(c["q"], c["k"], c["v"], c["pos_bias"], c["dout"], c.get("scale_embed"),
                               None, c["offsets"], chunk=8)
    # same torch build as the generator: forward, dq and the parameter gradients are bit-exact
    assert torch.equal(r["out"], c["out"])
    assert torch.equal(r["dq"], c["dq"])
    assert torch.equal(r["dpb"], c["dpb"])
    if "dse" in c:
        assert torch.equal(r["dse"], c["dse"])
    # dk/dv: scatter-add backward, summation order not fixed even inside the reference
    assert rel_inf(r["dk"], c["dk"]) < 2e-6 and rel_inf(r["dv"], c["dv"]) < 2e-6


@pytest.mark.parametrize("name", GOLDEN_MODULE_CASES)
def test_torch_oracle_matches_reference_module_other_offset_sets(golden, name):
    c = load_case(golden, name)
    out = O.dsqg_reference(c["q"], c["k"], c["v"], c["pos_bias"], None, None, c["offsets"])
    assert max_abs(out, c["out"]) < 2e-6
    assert len(c["offsets"]) in (43, 45)


@pytest.mark.parametrize("name", GOLDEN_FN_CASES)
def test_c_oracle_matches_reference_outputs(golden, name):
    c = load_case(golden, name)
    out, lse = C.fwd(c["q"], c["k"], c["v"], c["pos_bias"], c.get("scale_embed"), None, c["offsets"])
    assert rel_inf(out, c["out"]) < 5e-6          # double accumulation vs the reference's fp32
    g = C.bwd(c["q"], c["k"], c["v"], c["pos_bias"], c["dout"], c.get("scale_embed"), None, c["offsets"])
    for nm in ("dq", "dk", "dv", "dpb") + (("dse",) if "dse" in c else ()):
        assert rel_inf(g[nm], c[nm]) < 2e-5, nm
    assert torch.isfinite(lse).all()


@pytest.mark.parametrize("name", GOLDEN_MODULE_CASES)
def test_c_oracle_other_offset_sets(golden, name):
    c = load_case(golden, name)
    out, _ = C.fwd(c["q"], c["k"], c["v"], c["pos_bias"], None, None, c["offsets"])
    assert rel_inf(out, c["out"]) < 5e-6


def test_offset_sets():
    assert len(O.OFFSETS_44) == 44 and len(O.OFFSETS_43) == 43 and len(O.OFFSETS_45) == 45
    assert O.OFFSETS_44[:33] == list(range(33)) and O.OFFSETS_43[:32] == list(range(32))
    assert O.OFFSETS_44[33:] == O.SPARSE_TAPS == O.OFFSETS_43[32:]


def test_index_mask_oracle_is_exact():
    N = 70
    src, valid = O.index_mask_oracle(N, O.OFFSETS_44)
    for n in (0, 1, 31, 32, 33, 47, 48, 63, 64, 69):
        for j, d in enumerate(O.OFFSETS_44):
            assert bool(valid[n, j]) == (n - d >= 0)
            assert int(src[n, j]) == (n - d if n >= d else -1)
    assert int(valid.sum()) == sum(max(0, N - d) for d in O.OFFSETS_44)


def test_gain_and_scale_embed_semantics():
    torch.manual_seed(0)
    B, H, N, D = 1, 3, 130, 16
    q, k, v = (torch.randn(B, H, N, D) for _ in range(3))
    pb = torch.randn(44, H) * 0.5
    g = torch.tensor([0.5, 1.0, 2.0])
    base = O.dsqg_reference(q, k, v, pb, None, None, O.OFFSETS_44)
    gained = O.dsqg_reference(q, k, v, pb, None, g, O.OFFSETS_44)
    assert torch.allclose(gained, base * g.view(1, H, 1, 1))
    # V3 with a zero scale_embed is V2 (reference test kernels/dsqg_attention_v3.py:612-628)
    z = O.dsqg_reference(q, k, v, pb, torch.zeros(44, D), None, O.OFFSETS_44)
    assert torch.equal(z, base)
    # softmax weights sum to one: constant V gives constant output (tools/check_kernel.py:470-526)
    ones = O.dsqg_reference(q, k, torch.ones_like(v), pb, None, None, O.OFFSETS_44)
    assert torch.allclose(ones, torch.ones_like(ones), atol=1e-6)


def test_causality_of_oracle():
    # perturbing position p must not change rows < p (train_2048_condM_layer_ablation.py:410-426)
    torch.manual_seed(1)
    B, H, N, D = 1, 2, 64, 8
    q, k, v = (torch.randn(B, H, N, D) for _ in range(3))
    pb = torch.randn(43, H)
    a = O.dsqg_reference(q, k, v, pb, None, None, O.OFFSETS_43)
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 10] += 1.0; v2[:, :, 10] -= 1.0
    b = O.dsqg_reference(q, k2, v2, pb, None, None, O.OFFSETS_43)
    assert torch.equal(a[:, :, :10], b[:, :, :10]) and not torch.equal(a[:, :, 10:], b[:, :, 10:])


def test_c_and_torch_oracles_agree_with_gain_in_double():
    torch.manual_seed(2)
    B, H, N, D = 2, 2, 100, 24
    q, k, v, do = (torch.randn(B, H, N, D) for _ in range(4))
    pb = torch.randn(43, H) * 0.5; se = torch.randn(43, D) * 0.05; g = torch.rand(H) + 0.5
    r = O.dsqg_reference_grads(q, k, v, pb, do, se, g, O.OFFSETS_43, compute_dtype=torch.float64)
    out, _ = C.fwd(q, k, v, pb, se, g, O.OFFSETS_43)
    assert rel_inf(out, r["out"]) < 1e-6
    c = C.bwd(q, k, v, pb, do, se, g, O.OFFSETS_43)
    for nm in c:
        assert rel_inf(c[nm], r[nm]) < 1e-6, nm


def test_fully_masked_rows_in_c_oracle():
    # offset sets without delta = 0: row 0 has no valid tap -> out = 0, lse = -inf
    q, k, v = (torch.randn(1, 1, 8, 8) for _ in range(3))
    out, lse = C.fwd(q, k, v, torch.zeros(3, 1), None, None, [1, 2, 4])
    assert torch.all(out[0, 0, 0] == 0) and lse[0, 0, 0] == float("-inf")
    assert torch.isfinite(lse[0, 0, 1:]).all()


def test_decode_oracles_agree():
    torch.manual_seed(3)
    S, H, D = 3, 2, 8
    offsets = [0, 1, 2, 3, 6, 9]
    R = 10
    kr, vr = torch.randn(S, H, R, D), torch.randn(S, H, R, D)
    q, kn, vn = (torch.randn(S, H, D) for _ in range(3))
    pb = torch.randn(len(offsets), H); g = torch.rand(H) + 0.5
    for head_val in range(R):
        head = torch.full((S,), head_val, dtype=torch.int32)
        a, ka, va = O.decode_reference(q, kn, vn, kr, vr, head, pb, g, offsets)
        b, kb, vb = O.decode_reference_direct(q, kn, vn, kr, vr, head, pb, g, offsets)
        assert torch.allclose(a, b, atol=1e-6) and torch.equal(ka, kb) and torch.equal(va, vb)
        assert torch.equal(ka[:, :, head_val], kn)
    # partially filled ring: taps with delta >= fill are masked
    head = torch.tensor([4, 4, 4], dtype=torch.int32); fill = torch.tensor([5, 5, 5], dtype=torch.int32)
    a, _, _ = O.decode_reference(q, kn, vn, kr, vr, head, pb, g, offsets, fill=fill)
    b, _, _ = O.decode_reference_direct(q, kn, vn, kr, vr, head, pb, g, offsets, fill=fill)
    assert torch.allclose(a, b, atol=1e-6)
