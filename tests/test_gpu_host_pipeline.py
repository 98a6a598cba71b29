"""GPU tests of DSQGHostPipeline: pinned host tensors in, pinned host tensors out, the copies of
neighbouring steps overlapping the kernels.  Every step must give exactly what the autograd
operator gives for the same inputs (same kernels, same order of operations: bit-exact)."""
import pytest
import torch

import dwarf_b200

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("with_se", [False, True])
@pytest.mark.parametrize("depth", [1, 2, 3])
def test_pipeline_steps_equal_the_autograd_operator(depth, with_se):
    g = torch.Generator().manual_seed(depth)
    B, H, N, D = 2, 4, 300, 32
    offsets = tuple(range(9)) + (16, 48, 128)
    pb = torch.randn(len(offsets), H, generator=g).to(DEV)
    gain = (torch.rand(H, generator=g) + 0.5).to(DEV)
    se = (torch.randn(len(offsets), D, generator=g) * 0.05).to(DEV) if with_se else None
    pipe = dwarf_b200.DSQGHostPipeline((B, H, N, D), torch.bfloat16, offsets, DEV, depth=depth, scale_embed=with_se)
    steps = 5
    pin = lambda: torch.empty(B, H, N, D, dtype=torch.bfloat16).pin_memory()
    ins = [[(torch.randn(B, H, N, D, generator=g) * 0.5).to(torch.bfloat16).pin_memory() for _ in range(4)] for _ in range(steps)]
    outs = [[pin() for _ in range(4)] for _ in range(steps)]
    dpb = [torch.empty(len(offsets), H).pin_memory() for _ in range(steps)]
    dg = [torch.empty(H).pin_memory() for _ in range(steps)]
    dse = [torch.empty(len(offsets), D).pin_memory() for _ in range(steps)]
    for i in range(steps):
        pipe.submit(*ins[i], pb, gain, *outs[i], dpos_bias=dpb[i], dhead_gain=dg[i], scale_embed=se,
                    dscale_embed=dse[i] if with_se else None)
    pipe.synchronize()
    for i in range(steps):
        q, k, v = (t.to(DEV).requires_grad_(True) for t in ins[i][:3])
        pbp, gp = pb.clone().requires_grad_(True), gain.clone().requires_grad_(True)
        sep = se.clone().requires_grad_(True) if with_se else None
        o = dwarf_b200.dsqg_attention(q, k, v, pbp, gp, sep, offsets)
        o.backward(ins[i][3].to(DEV))
        for got, ref in zip(outs[i], (o.detach(), q.grad, k.grad, v.grad)):
            assert torch.equal(got, ref.cpu())
        assert torch.equal(dpb[i], pbp.grad.cpu()) and torch.equal(dg[i], gp.grad.cpu())
        if with_se:
            assert torch.equal(dse[i], sep.grad.cpu())


def test_pipeline_rejects_pageable_host_tensors():
    B, H, N, D = 1, 2, 64, 32
    offsets = (0, 1, 2)
    pipe = dwarf_b200.DSQGHostPipeline((B, H, N, D), torch.bfloat16, offsets, DEV)
    pinned = [torch.zeros(B, H, N, D, dtype=torch.bfloat16).pin_memory() for _ in range(8)]
    pb = torch.zeros(len(offsets), H, device=DEV)
    bad = list(pinned); bad[1] = torch.zeros(B, H, N, D, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        pipe.submit(*bad[:4], pb, None, *bad[4:])
    pipe.submit(*pinned[:4], pb, None, *pinned[4:])          # without head_gain
    pipe.synchronize()
    assert torch.equal(pinned[4], torch.zeros_like(pinned[4]))
