"""GPU test of dsqg_bwd_static, the backward entry point for callers that cannot allocate
device memory (fixed-arena servers, plugin hosts that own no allocator): its scratch is an
array built into the library instead of a buffer the caller passes.

The file sorts last on purpose, so a run that stops at the first failure has already gone
through every other test.  The test calls the entry point through the C ABI twice in a row
(the array keeps the previous call's contents) and expects exactly the results of dsqg_bwd
with a caller-allocated scratch: the kernels and their fixed-order reductions are the same,
so the comparison is bitwise.
"""
import pytest
import torch

from dwarf_b200 import _lib

pytestmark = pytest.mark.gpu

OFFSETS = tuple(range(32)) + (48, 64, 96, 128, 192, 256, 384, 512, 768, 1024, 1536)


def _problem(B, H, N, D, seed, dev):
    g = torch.Generator().manual_seed(seed)
    mk = lambda s=0.5: (torch.randn(B, H, N, D, generator=g) * s).to(torch.bfloat16).to(dev)
    q, k, v, dout = mk(), mk(), mk(), mk(1.0)
    J = len(OFFSETS)
    pb = (torch.randn(J, H, generator=g) * 0.5).to(dev)
    gain = (torch.rand(H, generator=g) * 0.4 + 0.8).to(dev)
    return q, k, v, dout, pb, gain


def _forward(lib, q, k, v, pb, gain, off, J, shape, stream, se=None):
    B, H, N, D = shape
    out = torch.empty_like(q)
    lse = torch.empty(B, H, N, device=q.device)
    _lib.check(lib.dsqg_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(),
                            None if se is None else se.data_ptr(), gain.data_ptr(),
                            off, J, out.data_ptr(), lse.data_ptr(), B, H, N, D, 0, stream), "dsqg_fwd")
    return out, lse


def _backward(lib, static, q, k, v, pb, gain, off, J, out, lse, dout, shape, stream, se=None, outputs=None):
    """One backward call; `outputs` (optional) are result tensors allocated by an earlier call, so that
    this call makes no allocation of its own on the test's side either."""
    B, H, N, D = shape
    nan = float("nan")
    if outputs is None:
        dq, dk, dv = (torch.full_like(q, nan) for _ in range(3))
        dpb = torch.full((J, H), nan, device=q.device)
        dg = torch.full((H,), nan, device=q.device)
        dse = None if se is None else torch.full((J, D), nan, device=q.device)
    else:
        dq, dk, dv, dpb, dg, dse = outputs
    common = (q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), None if se is None else se.data_ptr(),
              gain.data_ptr(), off, J, out.data_ptr(), lse.data_ptr(), dout.data_ptr(), dq.data_ptr(),
              dk.data_ptr(), dv.data_ptr(), dpb.data_ptr(), None if dse is None else dse.data_ptr(), dg.data_ptr())
    if static:
        _lib.check(lib.dsqg_bwd_static(*common, B, H, N, D, 0, stream), "dsqg_bwd_static")
    else:
        nbytes = lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, int(se is not None))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        _lib.check(lib.dsqg_bwd(*common, scratch.data_ptr(), nbytes, B, H, N, D, 0, stream), "dsqg_bwd")
    torch.cuda.synchronize()
    return dq, dk, dv, dpb, dg, dse


def test_static_scratch_backward_matches_regular_backward_twice_in_a_row():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    off, J = _lib.offsets_array(OFFSETS)
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second call finds the first one's leftovers
    for shape, seed in (((2, 8, 2047, 32), 1), ((3, 4, 1600, 64), 2)):
        q, k, v, dout, pb, gain = _problem(*shape, seed, dev)
        out, lse = _forward(lib, q, k, v, pb, gain, off, J, shape, stream)
        want = _backward(lib, False, q, k, v, pb, gain, off, J, out, lse, dout, shape, stream)
        for attempt in range(2):
            got = _backward(lib, True, q, k, v, pb, gain, off, J, out, lse, dout, shape, stream)
            for name, a, b in zip(("dq", "dk", "dv", "dpos_bias", "dhead_gain"), got, want):
                assert torch.isfinite(a.float()).all(), (name, attempt)
                assert torch.equal(a, b), (name, attempt, (a.float() - b.float()).abs().max().item())


def test_static_scratch_backward_with_scale_embed_and_without_any_allocation():
    """The scale_embed carve-up is the one that needs the most of the built-in array (per-row table,
    per-tile partials, prepared tables): a small case of it, twice in a row, bitwise against dsqg_bwd.
    The second call reuses the first call's result tensors, so nothing at all is allocated around it:
    the device's free memory must read the same before and after."""
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    off, J = _lib.offsets_array(OFFSETS)
    stream = torch.cuda.current_stream().cuda_stream
    shape = (1, 4, 600, 32)
    B, H, N, D = shape
    assert 0 < lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, 1) <= _lib.DSQG_STATIC_SCRATCH_BYTES
    q, k, v, dout, pb, gain = _problem(*shape, 5, dev)
    se = (torch.randn(J, D, generator=torch.Generator().manual_seed(6)) * 0.05).to(dev)
    out, lse = _forward(lib, q, k, v, pb, gain, off, J, shape, stream, se)
    want = _backward(lib, False, q, k, v, pb, gain, off, J, out, lse, dout, shape, stream, se)
    got = _backward(lib, True, q, k, v, pb, gain, off, J, out, lse, dout, shape, stream, se)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    again = _backward(lib, True, q, k, v, pb, gain, off, J, out, lse, dout, shape, stream, se, outputs=got)
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before, "dsqg_bwd_static changed the amount of free device memory"
    for name, a, b in zip(("dq", "dk", "dv", "dpos_bias", "dhead_gain", "dscale_embed"), again, want):
        assert torch.isfinite(a.float()).all(), name
        assert torch.equal(a, b), (name, (a.float() - b.float()).abs().max().item())


def test_static_scratch_limit_is_enforced_before_any_launch():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    off, J = _lib.offsets_array(OFFSETS)
    B, H, N, D = 64, 8, 4096, 32                      # needs > 8 MiB of scratch
    assert lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, 0) > _lib.DSQG_STATIC_SCRATCH_BYTES
    x = torch.zeros(16, device=dev)                   # never dereferenced: the call is refused on the host
    p = x.data_ptr()
    rc = lib.dsqg_bwd_static(p, p, p, p, None, None, off, J, p, p, p, p, p, p, p, None, None, B, H, N, D, 0, None)
    assert rc == -9
    assert b"DSQG_STATIC_SCRATCH_BYTES" in lib.dsqg_status_str(rc)
    # argument errors are still reported as such
    assert lib.dsqg_bwd_static(None, p, p, p, None, None, off, J, p, p, p, p, p, p, p, None, None, 1, 1, 16, 32, 0, None) == -1
