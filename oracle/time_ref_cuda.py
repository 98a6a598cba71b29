"""Times the reference's hand-written CUDA DSQG extension (built by oracle/build_ref_cuda.py into
oracle/_ref/) on the current GPU beside this library on the same shape and offsets, and checks
that both agree.  Measurement infrastructure; prints one JSON line.

    python oracle/time_ref_cuda.py [B H N]        # head width 32, the reference kernel's d50 offsets

The reference kernel only exists for its 44-tap set 0..40, 128, 384, 1536 and head widths 32 / 48
(kernels/dsqg_cuda/dsqg_cuda_kernel.cu:19-22,510); that is the shape both sides run.
"""
import importlib.util
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
D50 = tuple(range(41)) + (128, 384, 1536)


def load_ref():
    path = os.path.join(HERE, "_ref", "dsqg_cuda_ref.so")
    spec = importlib.util.spec_from_file_location("dsqg_cuda_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def timed(fn, n=30, warm=5):
    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3


def main():
    import dwarf_b200
    from dwarf_b200 import _lib
    B, H, N = (int(a) for a in sys.argv[1:4]) if len(sys.argv) >= 4 else (32, 8, 2048)
    D, J = 32, len(D50)
    dev = torch.device("cuda", 0)
    ref = load_ref()
    g = torch.Generator().manual_seed(0)
    q, k, v = ((torch.randn(B, H, N, D, generator=g) * 0.5).bfloat16().to(dev) for _ in range(3))
    dout = torch.randn(B, H, N, D, generator=g).bfloat16().to(dev)
    pb = (torch.randn(J, H, generator=g) * 0.5).to(dev)
    se = (torch.randn(J, D, generator=g) * 0.05).to(dev)
    lib = _lib.load()
    off, _ = _lib.offsets_array(D50)
    out = torch.empty_like(q); lse = torch.empty(B, H, N, device=dev)
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    dpb = torch.empty(J, H, device=dev); dse = torch.empty(J, D, device=dev)
    nbytes = lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, 1)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    st = None                                   # legacy default stream: what the reference kernel launches on

    def ours_fwd():
        _lib.check(lib.dsqg_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), se.data_ptr(), None, off, J,
                                out.data_ptr(), lse.data_ptr(), B, H, N, D, 0, st), "fwd")

    def ours_bwd():
        _lib.check(lib.dsqg_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), pb.data_ptr(), se.data_ptr(), None, off, J,
                                out.data_ptr(), lse.data_ptr(), dout.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                dv.data_ptr(), dpb.data_ptr(), dse.data_ptr(), None, scratch.data_ptr(), nbytes,
                                B, H, N, D, 0, st), "bwd")

    with torch.cuda.stream(torch.cuda.default_stream()):
        ro, rl = ref.forward(q, k, v, pb, se)
        rg = ref.backward(q, k, v, pb, se, ro, rl, dout)
        ours_fwd(); ours_bwd()
        torch.cuda.synchronize()
        agree = {"out": (out.float() - ro.float()).abs().max().item(),
                 "dq": (dq.float() - rg[0].float()).abs().max().item(),
                 "dk": (dk.float() - rg[1].float()).abs().max().item(),
                 "dv": (dv.float() - rg[2].float()).abs().max().item(),
                 "dpb_rel": ((dpb - rg[3]).abs().max() / rg[3].abs().max()).item(),
                 "dse_rel": ((dse - rg[4]).abs().max() / rg[4].abs().max()).item()}
        res = {"shape": [B, H, N, D], "offsets": "0..40,128,384,1536 (J=44), with scale_embed",
               "reference_cuda_us": {"fwd": timed(lambda: ref.forward(q, k, v, pb, se)),
                                     "bwd": timed(lambda: ref.backward(q, k, v, pb, se, ro, rl, dout))},
               "this_library_us": {"fwd": timed(ours_fwd), "bwd": timed(ours_bwd)},
               "max_abs_difference": agree}
    res["speedup"] = {p: res["reference_cuda_us"][p] / res["this_library_us"][p] for p in ("fwd", "bwd")}
    print(json.dumps(res))


if __name__ == "__main__":
    main()
