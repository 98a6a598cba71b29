"""CPU tests of the host-side logic: drop-in module surface, synthetic inputs, sharding
and the 2-rank (gloo) plumbing used by the multi-GPU benchmark."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import dwarf_b200
from dwarf_b200 import dist as ddist
from dwarf_b200 import synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_offset_sets_match_reference_definition():
    assert dwarf_b200.ALL_OFFSETS == tuple(range(33)) + (48, 64, 96, 128, 192, 256, 384, 512, 768, 1024, 1536)
    assert len(dwarf_b200.OFFSETS_43) == 43 and dwarf_b200.OFFSETS_43[31] == 31
    assert dwarf_b200.OFFSETS_45[-2:] == (2048, 3072)


def test_module_surface_matches_reference_names():
    m = dwarf_b200.DSQGAttentionN_Fused(256, 8)
    assert set(dict(m.named_parameters())) == {
        "pos_bias", "qkv_proj.weight", "qkv_proj.bias", "out_proj.weight", "out_proj.bias",
        "gate_proj.weight", "gate_proj.bias"}
    assert tuple(m.pos_bias.shape) == (44, 8) and m.offsets.dtype == torch.long
    assert float(m.gate_proj.bias[0]) == 2.0
    # pos_bias[j,h] = -log(1+delta_j) * alpha_h
    assert torch.allclose(m.pos_bias[1], -torch.log(torch.tensor(2.0)) * torch.linspace(0.2, 2.0, 8))
    m3 = dwarf_b200.DSQGAttentionV3(256, 8)
    assert tuple(m3.scale_embed.shape) == (44, 32) and float(m3.scale_embed.abs().sum()) == 0.0
    qw = dwarf_b200.DSQGAttentionQW(256, 8)
    assert tuple(qw.if_gain.shape) == (8,) and set(qw.attn_summary()) >= {"if_gain", "scale_embed_abs_max"}
    assert set(m.attn_summary()) == {"pos_bias_abs_mean", "pos_bias_abs_max", "pos_bias_mean_per_head"}
    m43 = dwarf_b200.DSQGAttentionN_Fused(64, 2, offsets=dwarf_b200.OFFSETS_43)
    assert tuple(m43.pos_bias.shape) == (43, 2)


def test_reference_shaped_state_dicts_load_strictly():
    """Key sets of the reference's modules: kernels/dsqg_attention_v2.py:434-456 (N_Fused),
    kernels/dsqg_attention_v3.py:463-500 (V3), train/train_2048_condU.py:139-166 (QW: no `offsets`)."""
    E, H, J = 64, 2, 44
    lin = lambda name, o, i: {f"{name}.weight": torch.zeros(o, i), f"{name}.bias": torch.zeros(o)}
    common = {**lin("qkv_proj", 3 * E, E), **lin("out_proj", E, E), **lin("gate_proj", E, E),
              "pos_bias": torch.zeros(J, H)}
    offs = {"offsets": torch.tensor(dwarf_b200.ALL_OFFSETS, dtype=torch.long)}
    se = {"scale_embed": torch.zeros(J, E // H)}
    cases = [(dwarf_b200.DSQGAttentionN_Fused, {**common, **offs}),
             (dwarf_b200.DSQGAttentionV3, {**common, **offs, **se}),
             (dwarf_b200.DSQGAttentionQW, {**common, **se, "if_gain": torch.ones(H)})]
    for cls, sd in cases:
        m = cls(E, H)
        assert set(m.state_dict()) == set(sd), cls.__name__
        m.load_state_dict(sd, strict=True)
        assert m.offsets.tolist() == list(dwarf_b200.ALL_OFFSETS)


def test_compat_shims_export_reference_names():
    sys.path.insert(0, os.path.join(ROOT, "dwarf_b200", "compat"))
    try:
        import dsqg_attention_v2 as s2
        import dsqg_attention_v3 as s3
    finally:
        sys.path.pop(0)
    assert len(s2.ALL_OFFSETS) == 44 and callable(s2.dsqg_attention_v2) and s2.DSQGAttentionN_Fused
    assert callable(s3.dsqg_attention_v3) and s3.DSQGAttentionV3


def test_host_pipeline_needs_a_cuda_device():
    with pytest.raises(RuntimeError):
        dwarf_b200.DSQGHostPipeline((1, 2, 64, 32), torch.bfloat16, (0, 1, 2), "cpu")
    with pytest.raises(ValueError):
        dwarf_b200.DSQGHostPipeline((1, 2, 64, 32), torch.bfloat16, (0, 1, 2), "cuda:0", depth=0)


def test_synthetic_inputs_are_seeded_and_prefix_stable():
    cfg = synth.OP_CONFIGS["cfg1"]
    a = synth.make_op_inputs(cfg, B=2)
    b = synth.make_op_inputs(cfg, B=1)
    assert torch.equal(a["q"][:1], b["q"]) and torch.equal(a["dout"][:1], b["dout"])
    assert a["q"].dtype == torch.bfloat16 and tuple(a["pos_bias"].shape) == (43, 8)
    assert 0.8 <= float(a["head_gain"].min()) and float(a["head_gain"].max()) <= 1.2
    assert abs(float(a["q"].float().std()) - 0.5) < 0.01
    c0 = synth.make_op_inputs(synth.OP_CONFIGS["cfg0"], B=1, with_dout=False)
    assert c0["q"].dtype == torch.float32 and c0["head_gain"] is None and "dout" not in c0


def test_shard_range_partitions_exactly():
    for total in (1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            pieces = [ddist.shard_range(total, r, world) for r in range(world)]
            assert pieces[0][0] == 0 and pieces[-1][1] == total
            assert all(pieces[i][1] == pieces[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in pieces]
            assert max(sizes) - min(sizes) <= 1


def _gloo_worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    r, lr, w = ddist.init_process_group("gloo")
    b, e = ddist.shard_range(32, r, w)
    ddist.barrier()
    slow = ddist.max_over_ranks(10.0 + r)          # the timing rule: MAX over ranks
    units = ddist.sum_over_ranks(e - b)
    q.put((r, b, e, slow, units))
    dist.destroy_process_group()


def test_two_rank_gloo_sharding_and_timing_reduction():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    res = sorted(q.get(timeout=120) for _ in range(2))
    [p.join(60) for p in procs]
    assert [p.exitcode for p in procs] == [0, 0]
    assert res[0][1:3] == (0, 16) and res[1][1:3] == (16, 32)
    assert all(r[3] == 11.0 and r[4] == 32.0 for r in res)


def test_odd_head_widths_are_padded_only_when_the_tensor_core_kernels_take_them():
    """Host-side choice of the head dimension the kernels are called with (no device access)."""
    from dwarf_b200 import _lib, ops
    off43, J43 = _lib.offsets_array(ops.OFFSETS_43)
    wide = tuple(range(41)) + (128, 384, 1536)
    offw, Jw = _lib.offsets_array(wide)
    q = lambda D, dt=torch.bfloat16: torch.zeros(1, 1, 4, D, dtype=dt)
    assert ops._padded_head_dim(q(80), off43, J43, False) == 96
    assert ops._padded_head_dim(q(48), off43, J43, False) == 64
    assert ops._padded_head_dim(q(48), off43, J43, True) == 64       # scale_embed runs on the 64-wide kernels
    assert ops._padded_head_dim(q(80), off43, J43, True) == 80       # but not on the 96-wide ones
    assert ops._padded_head_dim(q(80), offw, Jw, False) == 80        # dense window wider than 32
    assert ops._padded_head_dim(q(80, torch.float32), off43, J43, False) == 80
    for D in (32, 64, 96, 128):
        assert ops._padded_head_dim(q(D), off43, J43, False) == D
