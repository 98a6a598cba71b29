"""GPU tests of the ring-buffer decode kernel against the decode oracle (which is defined as
the last row of the full-sequence reference on the time-ordered ring)."""
import pytest
import torch

import dwarf_b200
from dwarf_b200 import synth
from oracle import dsqg_oracle as O
from tests.gpu_util import assert_bf16_close, rel_inf

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


LAYOUT = "separate"


@pytest.fixture(autouse=True, params=["separate", "interleaved"])
def ring_layout(request):
    """Every test runs over two rings [S,H,R,D] (dsqg_decode) and over one ring that holds key and value
    of a slot side by side, [S,H,R,2,D] (dsqg_decode_kv)."""
    global LAYOUT
    LAYOUT = request.param
    yield request.param
    LAYOUT = "separate"


def run_cuda(q, kn, vn, kr, vr, head, pb, gain, offsets, fill=None, se=None, dtype=torch.bfloat16):
    to = lambda t: t.to(DEV, dtype).contiguous()
    args = (head.to(DEV), pb.to(DEV), None if gain is None else gain.to(DEV), None if se is None else se.to(DEV),
            offsets, None if fill is None else fill.to(DEV))
    if LAYOUT == "interleaved":
        kv = torch.stack([to(kr), to(vr)], dim=-2).contiguous()
        out = dwarf_b200.dsqg_decode_step_kv(to(q), to(kn), to(vn), kv, *args)
        return out.float().cpu(), kv[..., 0, :].float().cpu(), kv[..., 1, :].float().cpu()
    krd, vrd = to(kr), to(vr)
    out = dwarf_b200.dsqg_decode_step(to(q), to(kn), to(vn), krd, vrd, *args)
    return out.float().cpu(), krd.float().cpu(), vrd.float().cpu()


def bf16v(*shape, gen=None):
    return torch.randn(*shape, generator=gen).to(torch.bfloat16).float()


def test_every_head_position_small_ring_matches_full_sequence_oracle():
    g = torch.Generator().manual_seed(0)
    offsets = (0, 1, 2, 3, 6, 9, 12)
    R, S, H, D = 13, 13, 3, 32
    kr, vr = bf16v(S, H, R, D, gen=g), bf16v(S, H, R, D, gen=g)
    q, kn, vn = (bf16v(S, H, D, gen=g) for _ in range(3))
    pb = torch.randn(len(offsets), H, generator=g); gain = torch.rand(H, generator=g) + 0.5
    head = torch.arange(S, dtype=torch.int32)             # one sequence per head position 0..R-1
    out, k2, v2 = run_cuda(q, kn, vn, kr, vr, head, pb, gain, offsets)
    for s in range(S):     # full-sequence definition, one sequence at a time (fill may differ)
        ref, kref, vref = O.decode_reference(q[s:s + 1], kn[s:s + 1], vn[s:s + 1], kr[s:s + 1], vr[s:s + 1],
                                             head[s:s + 1], pb, gain, offsets)
        assert_bf16_close(out[s:s + 1], ref, f"out[s={s}]")
        assert torch.equal(k2[s:s + 1], kref) and torch.equal(v2[s:s + 1], vref)   # ring update is exact


@pytest.mark.parametrize("D", [32, 64, 80, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_full_ring_1537_slots_43_taps(D, dtype):
    g = torch.Generator().manual_seed(D)
    S, H, R = 5, 4, 1537
    kr, vr = bf16v(S, H, R, D, gen=g), bf16v(S, H, R, D, gen=g)
    q, kn, vn = (bf16v(S, H, D, gen=g) for _ in range(3))
    pb = synth.log_linear_pos_bias(O.OFFSETS_43, H); gain = torch.rand(H, generator=g) + 0.5
    se = torch.randn(43, D, generator=g) * 0.05
    head = torch.tensor([0, 1, 31, 1535, 1536], dtype=torch.int32)      # wrap-around cases
    out, k2, v2 = run_cuda(q, kn, vn, kr, vr, head, pb, gain, O.OFFSETS_43, se=se, dtype=dtype)
    ref, kref, vref = O.decode_reference_direct(q, kn, vn, kr, vr, head, pb, gain, O.OFFSETS_43, scale_embed=se)
    if dtype == torch.float32:
        assert rel_inf(out, ref) < 1e-5
    else:
        assert_bf16_close(out, ref, "out")
    assert torch.equal(k2, kref) and torch.equal(v2, vref)


def test_partially_filled_ring_masks_taps():
    g = torch.Generator().manual_seed(4)
    S, H, D, R = 6, 2, 64, 1537
    kr, vr = bf16v(S, H, R, D, gen=g), bf16v(S, H, R, D, gen=g)
    q, kn, vn = (bf16v(S, H, D, gen=g) for _ in range(3))
    pb = synth.log_linear_pos_bias(O.OFFSETS_43, H)
    head = torch.tensor([0, 4, 40, 100, 700, 1536], dtype=torch.int32)
    fill = torch.tensor([1, 5, 41, 101, 701, 1537], dtype=torch.int32)
    out, _, _ = run_cuda(q, kn, vn, kr, vr, head, pb, None, O.OFFSETS_43, fill=fill)
    ref, _, _ = O.decode_reference_direct(q, kn, vn, kr, vr, head, pb, None, O.OFFSETS_43, fill=fill)
    assert_bf16_close(out, ref, "out")
    assert_bf16_close(out[0], vn[0], "first token attends to itself only")
    # the full-sequence definition agrees for one of the partial fills
    ref_full, _, _ = O.decode_reference(q[2:3], kn[2:3], vn[2:3], kr[2:3], vr[2:3], head[2:3], pb, None,
                                        O.OFFSETS_43, fill=fill[2:3])
    assert_bf16_close(out[2:3], ref_full, "out vs full-sequence oracle")


def test_decode_reproduces_training_forward_token_by_token():
    """Feeding a sequence through the ring cache one token at a time gives the rows of the
    full-sequence forward kernel."""
    g = torch.Generator().manual_seed(6)
    S, H, D, N = 2, 4, 32, 70
    offsets = tuple(range(8)) + (16, 32, 48)
    q, k, v = (bf16v(S, H, N, D, gen=g).to(DEV, torch.bfloat16) for _ in range(3))
    pb = torch.randn(len(offsets), H, generator=g).to(DEV)
    gain = (torch.rand(H, generator=g) + 0.5).to(DEV)
    full = dwarf_b200.dsqg_attention(q, k, v, pb, gain, None, offsets).float()
    cache = dwarf_b200.DSQGRingCache(1, S, H, D, offsets, interleaved=LAYOUT == "interleaved")
    assert cache.R == 49
    for t in range(N):
        cache.advance()
        o = cache.step(0, q[:, :, t].contiguous(), k[:, :, t].contiguous(), v[:, :, t].contiguous(), pb, gain)
        assert (o.float() - full[:, :, t]).abs().max().item() <= 2e-2, t


@pytest.mark.parametrize("N", [5, 49, 50, 120])
def test_prefill_then_decode_continues_the_sequence(N):
    """Rings filled from a training-layout prefix of N tokens, then token N decoded: must equal
    row N of the full-sequence forward over N+1 tokens (prefix shorter, equal and longer than R)."""
    g = torch.Generator().manual_seed(N)
    S, H, D = 3, 2, 64
    offsets = tuple(range(8)) + (16, 32, 48)
    q, k, v = (bf16v(S, H, N + 1, D, gen=g).to(DEV, torch.bfloat16) for _ in range(3))
    pb = torch.randn(len(offsets), H, generator=g).to(DEV)
    full = dwarf_b200.dsqg_attention(q, k, v, pb, None, None, offsets).float()
    cache = dwarf_b200.DSQGRingCache(1, S, H, D, offsets, interleaved=LAYOUT == "interleaved")
    cache.prefill(0, k[:, :, :N].contiguous(), v[:, :, :N].contiguous())
    assert int(cache.head[0]) == (N - 1) % cache.R and int(cache.fill[0]) == min(N, cache.R)
    cache.advance()
    o = cache.step(0, q[:, :, N].contiguous(), k[:, :, N].contiguous(), v[:, :, N].contiguous(), pb)
    assert (o.float() - full[:, :, N]).abs().max().item() <= 2e-2


def test_benchmark_shape_runs_and_matches_on_a_sample():
    cfg = synth.DecodeConfig()
    x = synth.make_decode_inputs(cfg, device="cpu", layers=1)
    to = lambda t: t.to(DEV)
    kr, vr = to(x["k_ring"][0]), to(x["v_ring"][0])
    out = dwarf_b200.dsqg_decode_step(to(x["q"][0]), to(x["k_new"][0]), to(x["v_new"][0]), kr, vr, to(x["head"]),
                                      to(x["pos_bias"]), to(x["head_gain"]), None, cfg.offsets)
    sl = slice(0, 16)
    f = lambda t: t[0][sl].float()
    ref, kref, _ = O.decode_reference_direct(f(x["q"]), f(x["k_new"]), f(x["v_new"]), f(x["k_ring"]), f(x["v_ring"]),
                                             x["head"][sl], x["pos_bias"], x["head_gain"], cfg.offsets)
    assert_bf16_close(out[sl].float().cpu(), ref, "out")
    assert torch.equal(kr[sl].float().cpu(), kref)


@pytest.mark.parametrize("D,J", [(64, 43), (32, 43), (64, 45), (128, 43)])
def test_overlapped_launch_equals_plain_launch_over_a_stack_of_layers(D, J):
    """dsqg_decode_overlapped over several layers back to back (each layer its own rings, one shared
    write head), eagerly and replayed from a CUDA graph, gives bit-identical outputs and rings."""
    g = torch.Generator().manual_seed(100 + D + J)
    offsets = O.OFFSETS_43 if J == 43 else tuple(O.OFFSETS_43) + (2048, 3072)
    L, S, H, R = 4, 24, 4, max(offsets) + 1
    to = lambda t: t.to(torch.bfloat16).to(DEV)
    kr0, vr0 = to(torch.randn(L, S, H, R, D, generator=g)), to(torch.randn(L, S, H, R, D, generator=g))
    q, kn, vn = (to(torch.randn(L, S, H, D, generator=g)) for _ in range(3))
    head = torch.randint(0, R, (S,), generator=g, dtype=torch.int32).to(DEV)
    fill = torch.randint(1, R + 1, (S,), generator=g, dtype=torch.int32).to(DEV)
    pb = synth.log_linear_pos_bias(offsets, H).to(DEV)

    def run(overlap, kr, vr, out):
        if LAYOUT == "interleaved":       # one ring per layer; the results are copied back into kr, vr for the comparison
            kv = torch.stack([kr, vr], dim=-2).contiguous()
            for l in range(L):
                dwarf_b200.dsqg_decode_step_kv(q[l], kn[l], vn[l], kv[l], head, pb, None, None, offsets,
                                               fill, out[l], overlap=overlap)
            kr.copy_(kv[..., 0, :]); vr.copy_(kv[..., 1, :])
            return
        for l in range(L):
            dwarf_b200.dsqg_decode_step(q[l], kn[l], vn[l], kr[l], vr[l], head, pb, None, None, offsets,
                                        fill, out[l], overlap=overlap)

    kr_a, vr_a, out_a = kr0.clone(), vr0.clone(), torch.empty_like(q)
    run(False, kr_a, vr_a, out_a)
    kr_b, vr_b, out_b = kr0.clone(), vr0.clone(), torch.full_like(q, float("nan"))
    run(True, kr_b, vr_b, out_b)
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b) and torch.equal(kr_a, kr_b) and torch.equal(vr_a, vr_b)

    kr_c, vr_c, out_c = kr0.clone(), vr0.clone(), torch.full_like(q, float("nan"))
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            run(True, kr_c, vr_c, out_c)
    torch.cuda.current_stream().wait_stream(side)
    kr_c.copy_(kr0); vr_c.copy_(vr0)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_c) and torch.equal(kr_a, kr_c) and torch.equal(vr_a, vr_c)
