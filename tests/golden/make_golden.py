"""Generate golden vectors for DSQG attention from the DWARF reference itself.

Run once, in a container that has the reference checkout (it does not travel to
the GPU machines):

    python tests/golden/make_golden.py --reference /path/to/DWARF

It imports the reference's own functions, unmodified:

* ``kernels/dsqg_attention_v2.py``  ``_reference``      (condM op, 44 offsets)
* ``kernels/dsqg_attention_v3.py``  ``_reference_v3``   (condU op, 44 offsets)
* ``train/train_2048_condM_layer_ablation.py`` ``DSQGAttentionN`` (takes an
  ``offsets`` argument; used for the 43- and 45-offset sets)

runs them on seeded inputs, takes gradients with autograd (the reference's own
gradient oracle, ``kernels/dsqg_attention_v2.py:526-528``) and stores inputs and
outputs in ``tests/golden/dsqg_golden.npz``.  Inputs that the reference would feed
in bf16 are stored as bf16 bit patterns (uint16); outputs are fp32.

While generating, the CPU oracle in ``oracle/dsqg_oracle.py`` is checked to be
bit-identical to the reference on every case for out, dq, dpos_bias and dscale_embed,
and equal to 2e-6 relative for dk, dv (the reference's own scatter-add backward is not
run-to-run deterministic at that level).
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def bf16_bits(t):
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16).copy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a DWARF checkout")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "kernels"))
    sys.path.insert(0, os.path.join(args.reference, "train"))
    sys.path.insert(0, ROOT)
    import dsqg_attention_v2 as ref_v2
    import dsqg_attention_v3 as ref_v3
    import train_2048_condM_layer_ablation as ref_la
    from oracle import dsqg_oracle as O

    assert list(ref_v3.ALL_OFFSETS) == O.OFFSETS_44 == list(ref_v2.ALL_OFFSETS)
    store = {}

    def run_fn(name, fn, shape, seed, use_se, bf16_inputs=True, qscale=0.1):
        """The reference's own test recipe (kernels/dsqg_attention_v3.py:579-601)."""
        B, H, N, HD = shape
        torch.manual_seed(seed)
        mk = (lambda: (torch.randn(B, H, N, HD) * qscale).to(torch.bfloat16).float()) \
            if bf16_inputs else (lambda: torch.randn(B, H, N, HD) * qscale)
        q, k, v = mk(), mk(), mk()
        pb = torch.randn(44, H) * 0.5
        se = torch.randn(44, HD) * 0.05 if use_se else None
        dout = torch.randn(B, H, N, HD)
        if bf16_inputs:
            dout = dout.to(torch.bfloat16).float()
        qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
        pbr = pb.clone().requires_grad_(True)
        ser = None if se is None else se.clone().requires_grad_(True)
        out = fn(qr, kr, vr, pbr, ser) if use_se else fn(qr, kr, vr, pbr)
        out.backward(dout)
        # oracle port must be bit-identical to the reference function
        po = O.dsqg_reference_grads(q, k, v, pb, dout, se, None, O.OFFSETS_44, chunk=B)
        assert torch.equal(po["out"], out.detach()), name
        assert torch.equal(po["dq"], qr.grad) and torch.equal(po["dpb"], pbr.grad), name
        # dK/dV come from a scatter-add (index_put backward) whose summation order varies
        # from run to run on CPU threads: the reference differs from itself by ~1e-7 there.
        for nm, ref_g in (("dk", kr.grad), ("dv", vr.grad)):
            assert (po[nm] - ref_g).abs().max() <= 2e-6 * max(1.0, ref_g.abs().max().item()), name
        if use_se:
            assert torch.equal(po["dse"], ser.grad), name
        enc = bf16_bits if bf16_inputs else (lambda t: t.numpy().copy())
        store[f"{name}/shape"] = np.array(shape, np.int64)
        store[f"{name}/offsets"] = np.array(O.OFFSETS_44, np.int32)
        store[f"{name}/bf16_inputs"] = np.array(int(bf16_inputs))
        for nm, t in (("q", q), ("k", k), ("v", v), ("dout", dout)):
            store[f"{name}/{nm}"] = enc(t)
        store[f"{name}/pos_bias"] = pb.numpy().copy()
        if use_se:
            store[f"{name}/scale_embed"] = se.numpy().copy()
            store[f"{name}/dse"] = ser.grad.numpy().copy()
        store[f"{name}/out"] = out.detach().numpy().copy()
        store[f"{name}/dq"] = qr.grad.numpy().copy()
        store[f"{name}/dk"] = kr.grad.numpy().copy()
        store[f"{name}/dv"] = vr.grad.numpy().copy()
        store[f"{name}/dpb"] = pbr.grad.numpy().copy()
        print(f"{name}: shape={shape} |out|max={out.abs().max():.4f}")

    # the reference's own self-test shapes, shrunk in B/H to keep the file small
    run_fn("v2_tiny", ref_v2._reference, (1, 2, 64, 32), 42, False)
    run_fn("v3_tiny", ref_v3._reference_v3, (1, 2, 64, 32), 42, True)
    run_fn("v3_alltaps_d8", ref_v3._reference_v3, (1, 1, 1552, 8), 43, True, qscale=1.0)
    run_fn("v3_d64", ref_v3._reference_v3, (1, 2, 96, 64), 44, True, qscale=0.5)
    run_fn("v2_hd80", ref_v2._reference, (1, 1, 80, 80), 45, False)
    run_fn("v2_fp32", ref_v2._reference, (1, 1, 160, 32), 46, False, bf16_inputs=False, qscale=1.0)

    # Other offset sets through the reference's own module (it accepts `offsets`).
    def run_module(name, offsets, H, HD, N, seed):
        torch.manual_seed(seed)
        D = H * HD
        mod = ref_la.DSQGAttentionN(D, H, seq_len=N, offsets=list(offsets), dropout=0.0)
        mod.eval()
        with torch.no_grad():
            mod.qkv_proj.weight.copy_(torch.randn(3 * D, D) * (D ** -0.5))
            mod.qkv_proj.bias.zero_()
            mod.gate_proj.weight.zero_(); mod.gate_proj.bias.zero_()   # gate = sigmoid(0) = 0.5
            mod.pos_bias.add_(torch.randn_like(mod.pos_bias) * 0.05)
        x = torch.randn(1, N, D)
        grabbed = {}
        hook = mod.out_proj.register_forward_pre_hook(lambda m, inp: grabbed.__setitem__("x", inp[0]))
        mod(x)
        hook.remove()
        gathered = grabbed["x"].detach() * 2.0      # undo the exact 0.5 gate
        out_ref = gathered.view(1, N, H, HD).permute(0, 2, 1, 3).contiguous()
        with torch.no_grad():
            qkv = mod.qkv_proj(x)
            q, k, v = (t.view(1, N, H, HD).permute(0, 2, 1, 3).contiguous() for t in qkv.split(D, dim=-1))
        pb = mod.pos_bias.detach().clone()
        po = O.dsqg_reference(q, k, v, pb, None, None, list(offsets))
        err = (po - out_ref).abs().max().item()
        assert err < 2e-6, (name, err)   # shifted-copy form sums in the same order; tiny fp slack
        store[f"{name}/shape"] = np.array((1, H, N, HD), np.int64)
        store[f"{name}/offsets"] = np.array(list(offsets), np.int32)
        store[f"{name}/bf16_inputs"] = np.array(0)
        for nm, t in (("q", q), ("k", k), ("v", v)):
            store[f"{name}/{nm}"] = t.numpy().copy()
        store[f"{name}/pos_bias"] = pb.numpy().copy()
        store[f"{name}/out"] = out_ref.numpy().copy()
        print(f"{name}: J={len(offsets)} N={N} oracle-vs-module max err {err:.2e}")

    run_module("la43", O.OFFSETS_43, 1, 8, 1600, 47)
    run_module("la45", O.OFFSETS_45, 1, 8, 3104, 48)

    path = os.path.join(HERE, "dsqg_golden.npz")
    np.savez_compressed(path, **store)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
