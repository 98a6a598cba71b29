#!/usr/bin/env python
"""Benchmark of the DSQG attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg1|cfg2|cfg2_4k|cfg3|cfg4]
    python bench.py --impl reference ...      # the reference's PyTorch path on the host cores

A "step" is one forward+backward pass of the DSQG op over one batch of synthetic input
(cfg3: one decode token across 10 layers).  Prints ONE JSON line on rank 0.

  value      whole-job tokens/s, inputs resident in HBM, CUDA-event timed, MAX over ranks
  e2e        same metric through the public Python API with pinned HOST buffers: the H2D copy
             of q,k,v,dout and the D2H copy of out,dq,dk,dv are inside the timed region
  roofline   the longest kernel of the step: algorithmic bytes per launch / its CUDA-event
             duration, against the measured HBM copy bandwidth in MEASURED_PEAKS.json
  cpu_baseline  the PyTorch restatement of the reference (oracle/) timed on the host cores on
             a bounded sample of the same workload (rank 0, N=1 only)

Multi-GPU: one process per GPU (torchrun); the batch is replicated per rank (weak scaling),
there is no data-path collective; torch.distributed only carries the barrier and the MAX of
the timings.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return FALLBACK_HBM_GBS, "fallback (no MEASURED_PEAKS.json)"


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the GPU works."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(5)
        except Exception:
            self.proc.kill()
        self.file.flush(); self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        self.file.close()
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        # "under load": the upper half of the samples (idle samples before/after sit at low clocks)
        load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- op workloads
def op_bytes(cfg):
    esz = 2 if cfg.dtype == torch.bfloat16 else 4
    return cfg.B * cfg.H * cfg.N * cfg.D * esz          # T: one [B,H,N,D] tensor


class OpProblem:
    """Device-resident tensors of one op workload and direct C-ABI calls on them."""

    def __init__(self, cfg, dev, x, scale_embed=False):
        import dwarf_b200  # noqa: F401  (loads the library)
        from dwarf_b200 import _lib
        self.lib, self._lib = _lib.load(), _lib
        self.cfg, self.dev = cfg, dev
        self.host = {nm: x[nm].pin_memory() for nm in ("q", "k", "v", "dout")}
        self.q, self.k, self.v, self.dout = (self.host[nm].to(dev, non_blocking=True) for nm in ("q", "k", "v", "dout"))
        self.pb = x["pos_bias"].to(dev); self.gain = x["head_gain"].to(dev)
        B, H, N, D = cfg.B, cfg.H, cfg.N, cfg.D
        self.off, self.J = _lib.offsets_array(cfg.offsets)
        J = self.J
        self.out = torch.empty_like(self.q); self.lse = torch.empty(B, H, N, device=dev)
        self.dq, self.dk, self.dv = (torch.empty_like(self.q) for _ in range(3))
        self.dpb = torch.empty(J, H, device=dev); self.dg = torch.empty(H, device=dev)
        self.se = (torch.randn(J, D, generator=torch.Generator().manual_seed(1234)) * 0.05).to(dev) if scale_embed else None
        self.dse = None if self.se is None else torch.empty(J, D, device=dev)
        self.nbytes = self.lib.dsqg_bwd_scratch_bytes(J, B, H, N, D, int(self.se is not None))
        self.scratch = torch.empty(self.nbytes, dtype=torch.uint8, device=dev)
        self.stream = torch.cuda.current_stream()
        self.dt = 0 if cfg.dtype == torch.bfloat16 else 1

    def fwd(self):
        c = self.cfg
        self._lib.check(self.lib.dsqg_fwd(self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.pb.data_ptr(),
                                          None if self.se is None else self.se.data_ptr(), self.gain.data_ptr(),
                                          self.off, self.J, self.out.data_ptr(), self.lse.data_ptr(),
                                          c.B, c.H, c.N, c.D, self.dt, self.stream.cuda_stream), "dsqg_fwd")

    def bwd(self, stages):
        c = self.cfg
        self._lib.check(self.lib.dsqg_bwd_stages(
            self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.pb.data_ptr(),
            None if self.se is None else self.se.data_ptr(), self.gain.data_ptr(), self.off, self.J,
            self.out.data_ptr(), self.lse.data_ptr(), self.dout.data_ptr(), self.dq.data_ptr(), self.dk.data_ptr(),
            self.dv.data_ptr(), self.dpb.data_ptr(), None if self.dse is None else self.dse.data_ptr(),
            self.dg.data_ptr(), self.scratch.data_ptr(), self.nbytes, c.B, c.H, c.N, c.D, self.dt,
            self.stream.cuda_stream, stages), "dsqg_bwd_stages")

    def timed(self, steps, warmup, world):
        """W warm-up steps, then exactly `steps` timed steps (CUDA events on the launching stream around
        every kernel, barrier + synchronize on both sides).  Returns (ms per step, MAX over ranks; this
        rank's ms per kernel; wall ms; whether L2 was flushed between steps)."""
        from dwarf_b200 import dist as ddist
        for _ in range(warmup):
            self.fwd(); self.bwd(1); self.bwd(6)
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
        # A step touches 12 T bytes; when that does not clearly exceed the 126 MB L2 (small per-GPU
        # batches, e.g. --scaling strong at 8 GPUs) a 256 MB buffer is overwritten between steps and
        # the step time is the sum of the kernels' event intervals instead of the whole span.
        flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev) if 12 * op_bytes(self.cfg) < (256 << 20) else None
        stream = self.stream
        ddist.barrier(); torch.cuda.synchronize()
        t_wall = time.perf_counter()
        for i in range(steps):
            if flush_buf is not None:
                flush_buf.fill_(i & 0xff)
            ev[i][0].record(stream); self.fwd()
            ev[i][1].record(stream); self.bwd(1)
            ev[i][2].record(stream); self.bwd(6)       # dK/dV kernel; its first CTAs also reduce dpos_bias / dhead_gain
            ev[i][3].record(stream)
        torch.cuda.synchronize(); ddist.barrier()
        wall_ms = (time.perf_counter() - t_wall) * 1e3
        total_ms = ev[0][0].elapsed_time(ev[-1][3]) if flush_buf is None else \
            sum(ev[i][0].elapsed_time(ev[i][3]) for i in range(steps))
        kern_ms = [sum(ev[i][s].elapsed_time(ev[i][s + 1]) for i in range(steps)) / steps for s in range(3)]
        total_ms = ddist.max_over_ranks(total_ms, self.dev if world > 1 else "cpu")
        return total_ms / steps, kern_ms, wall_ms, flush_buf is not None


def profiled_traffic(workload):
    """DRAM bytes (read + write) per launch of the three default kernels, from the table in
    profiles/dram_traffic.md (ncu captures of the named kernel instantiations).  {} when the
    workload was not captured."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    res = {}
    if not os.path.exists(path):
        return res
    with open(path) as f:
        for line in f:
            cells = [c.strip() for c in line.strip().strip("|").split("|")]
            if len(cells) >= 4 and cells[0] == workload:
                try:
                    res[cells[1]] = {"kernel": cells[2], "bytes": float(cells[3]) * 1e6}
                except ValueError:
                    pass
    return res


def small_op_line(cfg, dev, world, steps, warmup, x=None):
    """ms/step, tokens/s and roofline fraction of one more op workload (device-resident, fewer steps)."""
    from dwarf_b200 import synth
    prob = OpProblem(cfg, dev, synth.make_op_inputs(cfg) if x is None else x)
    ms, kern_ms, _, flushed = prob.timed(steps, warmup, world)
    peak, _ = measured_peaks()
    T = op_bytes(cfg)
    del prob
    torch.cuda.empty_cache()
    return {"workload": cfg.name, "ms_per_step": ms, "tokens_per_s": cfg.B * cfg.N * world / (ms * 1e-3), "steps": steps,
            "kernels_ms": {"dsqg_fwd": kern_ms[0], "dsqg_bwd_dq": kern_ms[1], "dsqg_bwd_dkdv": kern_ms[2]},
            "frac": 12 * T / (ms * 1e-3) / 1e9 / peak, "l2_flushed": flushed}


def forward_paths_line(dev, restore_path, steps=20, warmup=5):
    """Forward only, default register-fed kernel (path 2) against the forward whose dense window runs on
    tcgen05 tensor cores with tensor-memory accumulators (path 4, csrc/dsqg_umma.cu): the dense window
    alone (offsets 0..31) at the cfg1 and cfg2 shapes, and the whole cfg1 forward.  CUDA events around
    every call, L2 flushed between calls; us per forward (median)."""
    import dataclasses
    from dwarf_b200 import _lib, synth
    lib = _lib.load()
    res = {"what": "forward only: path 2 = register-fed mma.sync kernel (default), path 4 = dense window on tcgen05 / "
                   "tensor memory; us per call, median, L2 flushed"}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    cases = [("cfg1_dense_window", "cfg1", True), ("cfg2_dense_window", "cfg2", True), ("cfg1_all_offsets", "cfg1", False)]
    try:
        for name, base, dense in cases:
            cfg = synth.OP_CONFIGS[base]
            if dense:
                cfg = dataclasses.replace(cfg, offsets=tuple(o for o in cfg.offsets if o <= 32))
            prob = OpProblem(cfg, dev, synth.make_op_inputs(cfg))
            row = {"offsets": len(cfg.offsets)}
            for path, key in ((2, "mma_sync_us"), (4, "tcgen05_us")):
                _lib.check(lib.dsqg_set_kernel_path(path), "dsqg_set_kernel_path")
                for _ in range(warmup):
                    prob.fwd()
                ts = []
                for i in range(steps):
                    flush.fill_(i & 0xff)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(prob.stream); prob.fwd(); e1.record(prob.stream)
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1) * 1e3)
                row[key] = sorted(ts)[len(ts) // 2]
            res[name] = row
            del prob
            torch.cuda.empty_cache()
        res["device_error"] = lib.dsqg_device_error(1)
    finally:
        lib.dsqg_set_kernel_path(restore_path)
    return res


def api_line(cfg, dev, world, steps, warmup, x):
    """fwd+bwd through the operator a reference script calls (dsqg_attention -> DSQGFunction, the
    replacement of kernels/dsqg_attention_v3.py:445-456): device-resident tensors, result tensors
    and scratch allocated by the autograd Function on every call."""
    import dwarf_b200
    from dwarf_b200 import dist as ddist
    q, k, v = (x[nm].to(dev).requires_grad_(True) for nm in ("q", "k", "v"))
    dout = x["dout"].to(dev)
    pb = x["pos_bias"].to(dev).requires_grad_(True); gain = x["head_gain"].to(dev).requires_grad_(True)

    def step():
        out = dwarf_b200.dsqg_attention(q, k, v, pb, gain, None, cfg.offsets)
        out.backward(dout)
        q.grad = k.grad = v.grad = pb.grad = gain.grad = None
    for _ in range(warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream = torch.cuda.current_stream()
    ddist.barrier(); torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize(); ddist.barrier()
    ms = ddist.max_over_ranks(e0.elapsed_time(e1), dev if world > 1 else "cpu") / steps
    peak, _ = measured_peaks()
    return {"entry": "dwarf_b200.dsqg_attention (autograd Function over the C ABI)", "workload": cfg.name,
            "ms_per_step": ms, "tokens_per_s": cfg.B * cfg.N * world / (ms * 1e-3), "steps": steps,
            "frac": 12 * op_bytes(cfg) / (ms * 1e-3) / 1e9 / peak}


def run_op_workload(args, cfg, rank, local_rank, world):
    import dwarf_b200
    from dwarf_b200 import _lib, dist as ddist, synth

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if args.batch > 0:                                  # a smaller case of the same workload (e.g. for an ncu capture)
        import dataclasses
        cfg = dataclasses.replace(cfg, B=args.batch, name=cfg.name.replace(f"B{cfg.B} ", f"B{args.batch} "))
    if args.dense_window_only:                          # kernel experiments on the dense window alone (offsets 0..32)
        import dataclasses
        dense = tuple(o for o in cfg.offsets if o <= 32)
        cfg = dataclasses.replace(cfg, offsets=dense, name=cfg.name.replace(f"J{len(cfg.offsets)}", f"J{len(dense)} dense window only"))
    x = synth.make_op_inputs(cfg)                       # CPU, seeded
    x_full, cfg_full = x, cfg
    strong = args.scaling == "strong" and world > 1
    global_B = cfg.B
    if strong:                                          # fixed problem: this rank's slice of the batch
        x, cfg = shard_inputs(x, cfg, rank, world)
    prob = OpProblem(cfg, dev, x, args.scale_embed)
    host, q, pb, gain, se = prob.host, prob.q, prob.pb, prob.gain, prob.se
    B, H, N, D = cfg.B, cfg.H, cfg.N, cfg.D
    stream = prob.stream

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- device-resident timing: W warm-up steps, then exactly K timed steps -------------
    ms_per_step, kern_ms, wall_ms, flushed = prob.timed(args.steps, args.warmup, world)
    tokens_per_step = global_B * N if strong else B * N * world       # what all ranks processed
    value = tokens_per_step / (ms_per_step * 1e-3)

    # ---- end to end: pinned host buffers in, pinned host buffers out ----------------------
    # dwarf_b200.DSQGHostPipeline: every step uploads q, k, v, dout from pinned host memory and
    # downloads out, dq, dk, dv into pinned host memory; the copies of neighbouring steps overlap
    # the kernels (three streams, two sets of device buffers), all inside the timed region.
    res_host = {nm: torch.empty(q.shape, dtype=q.dtype).pin_memory() for nm in ("out", "dq", "dk", "dv")}
    pipe = dwarf_b200.DSQGHostPipeline((B, H, N, D), q.dtype, cfg.offsets, dev, depth=2, scale_embed=se is not None)
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        pipe.submit(host["q"], host["k"], host["v"], host["dout"], pb, gain,
                    res_host["out"], res_host["dq"], res_host["dk"], res_host["dv"], scale_embed=se)

    for _ in range(3):
        e2e_step()
    pipe.synchronize(); ddist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    pipe.join(stream)
    e1.record(stream)
    torch.cuda.synchronize(); ddist.barrier()
    e2e_ms = ddist.max_over_ranks(e0.elapsed_time(e1), dev if world > 1 else "cpu") / e2e_steps
    # what the host side delivers when every rank copies at the same time, one direction at a time:
    # the e2e figure is bounded by these (4 T bytes each way per step)
    pcie = {}
    for name, src, dst in (("h2d", host["q"], q), ("d2h", q, res_host["out"])):
        ddist.barrier(); torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(10):
            dst.copy_(src, non_blocking=True)
        e1.record(stream)
        torch.cuda.synchronize(); ddist.barrier()
        gbs = 10 * src.numel() * src.element_size() / (e0.elapsed_time(e1) * 1e-3) / 1e9
        pcie[name + "_gbs_per_gpu_min"] = -ddist.max_over_ranks(-gbs, dev if world > 1 else "cpu")
        pcie[name + "_gbs_all_gpus"] = ddist.sum_over_ranks(gbs, dev if world > 1 else "cpu")
    clocks = sampler.stop() if rank == 0 else None

    T = op_bytes(cfg)
    peak, peak_src = measured_peaks()
    # DRAM bytes (read + write) per launch from the ncu captures listed in profiles/dram_traffic.md,
    # reported together with the kernel instantiation they were taken on; only known for the
    # workloads that were captured (full batch, automatic kernel choice, no scale_embed).
    names = ["dsqg_fwd", "dsqg_bwd_dq", "dsqg_bwd_dkdv"]
    prof = profiled_traffic("" if se is not None or strong or args.batch > 0 or args.kernel_path or args.dense_window_only else args.workload)
    ncu_traffic = [prof.get(nm, {}).get("bytes") for nm in names]
    ncu_kernel = [prof.get(nm, {}).get("kernel") for nm in names]
    alg = [4 * T, 6 * T, 6 * T]           # per launch: fwd Q,K,V->O ; dq Q,K,V,O,dO->dQ ; dkdv Q,K,V,dO->dK,dV
    top = max(range(3), key=lambda s: kern_ms[s])
    achieved = alg[top] / (kern_ms[top] * 1e-3) / 1e9
    step_achieved = 12 * T / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": "DSQG fwd+bwd tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": "bf16" if cfg.dtype == torch.bfloat16 else "f32", "data": "synthetic",
        "config": {"workload": cfg.name + (" +scale_embed" if se is not None else ""), "tokens_per_step_per_gpu": B * N,
                   "l2": (f"inputs+outputs per step ({12 * T / 1e6:.0f} MB) exceed the 126 MB L2; no flush" if not flushed
                          else f"inputs+outputs per step are {12 * T / 1e6:.0f} MB: L2 flushed by a 256 MB write between steps"),
                   "parallelism": (f"batch of {global_B} split over {world} GPUs, no collective" if strong
                                   else f"batch replicated x{world}, no collective")},
        "e2e": {"value": tokens_per_step / (e2e_ms * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": 4 * T, "d2h_bytes_per_step": 4 * T, "ms_per_step": e2e_ms,
                "steps": e2e_steps, "host_copy_bandwidth": pcie},
        "gpu_launches": ((3 if args.kernel_path in (0, 2, 4) else 4) + (2 if se is not None and args.kernel_path in (0, 2, 4) else 0)) * args.steps,   # paths 1 and 3 reduce in a 4th kernel
        "roofline": {"bound": "hbm", "kernel": names[top], "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": ncu_traffic[top], "traffic_from": (
                         None if ncu_traffic[top] is None else f"profiles/dram_traffic.md, ncu capture of {ncu_kernel[top]}"),
                     "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": alg[top], "ms_per_launch": kern_ms[top]},
        "step_roofline": {"algorithmic_bytes_per_step": 12 * T, "achieved": step_achieved,
                          "frac": step_achieved / peak, "unit": "GB/s"},
        "kernels": [{"name": names[s], "ms": kern_ms[s], "algorithmic_bytes": alg[s], "traffic": ncu_traffic[s],
                     "profiled_kernel": ncu_kernel[s], "gbs": alg[s] / (kern_ms[s] * 1e-3) / 1e9} for s in range(3)],
        "wall_ms_timed_region": wall_ms,
        "clocks": clocks,
    }
    del prob, pipe, res_host
    torch.cuda.empty_cache()
    if args.extras and not strong and args.batch <= 0 and se is None:
        # The rest of the metric in the same record: the operator API on the same workload, the other
        # op configurations, the decode step, and (N > 1) the same batch split over the ranks.
        xs = min(args.steps, 50)
        sampler2 = ClockSampler(local_rank)
        if rank == 0:
            sampler2.start()
        line["api"] = api_line(cfg, dev, world, xs, 5, x)
        if world > 1:
            xs_, cfg_s = shard_inputs(x_full, cfg_full, rank, world)
            sl = small_op_line(cfg_s, dev, world, xs, 5, xs_)
            sl["tokens_per_s"] = cfg_full.B * cfg_full.N / (sl["ms_per_step"] * 1e-3)
            sl["workload"] = f"{cfg_full.name}: batch of {cfg_full.B} split over {world} GPUs, no collective"
            sl["speedup_vs_one_rank_of_the_weak_run"] = ms_per_step / sl["ms_per_step"]
            line["strong"] = sl
        for other in ("cfg2", "cfg2_4k"):
            if other != args.workload:
                line[other] = small_op_line(synth.OP_CONFIGS[other], dev, world, min(args.steps, 30), 5)
        dargs = argparse.Namespace(**vars(args))
        dargs.steps, dargs.warmup, dargs.decode_layers = min(args.steps, 100), 5, 0
        d = run_decode_workload(dargs, rank, local_rank, world, sample_clocks=False, device_rings=True)
        line["decode"] = {"workload": d["config"]["workload"], "tokens_per_s": d["value"], "ms_per_step": d["ms_per_step"],
                          "ms_per_step_eager": d["ms_per_step_eager"], "ring_gbs": d["roofline"]["achieved"],
                          "frac": d["roofline"]["frac"], "steps": dargs.steps, "launch": d["config"]["launch"]}
        if world == 1:
            line["forward_paths"] = forward_paths_line(dev, args.kernel_path)
        if rank == 0:
            line["extras_clocks"] = sampler2.stop()      # clocks while api / strong / cfg2 / cfg2_4k / decode / forward paths ran
    return line


def shard_inputs(x, cfg, rank, world):
    """This rank's contiguous slice of the batch (strong scaling: the configuration's batch split over the ranks)."""
    import dataclasses
    from dwarf_b200 import dist as ddist
    b0, b1 = ddist.shard_range(cfg.B, rank, world)
    if b1 <= b0:
        raise SystemExit(f"strong scaling: batch {cfg.B} has no entry for rank {rank} of {world}")
    y = dict(x)
    for nm in ("q", "k", "v", "dout"):
        y[nm] = x[nm][b0:b1].contiguous()
    return y, dataclasses.replace(cfg, B=b1 - b0)


def run_decode_workload(args, rank, local_rank, world, sample_clocks=True, device_rings=False):
    import dwarf_b200
    from dwarf_b200 import dist as ddist, synth

    cfg = synth.DecodeConfig()
    if args.decode_layers > 0:
        cfg.layers = args.decode_layers
        cfg.name = cfg.name.replace("L10", f"L{cfg.layers}")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    # device_rings: the 12 GB of ring contents are drawn on the GPU (same distribution, another
    # stream of random numbers) instead of on the host, which takes most of a minute
    inter = args.ring_layout == "interleaved"
    x = synth.make_decode_inputs(cfg, device="cpu", rings_on="meta" if inter else (dev if device_rings else None))
    host = {nm: x[nm].pin_memory() for nm in ("q", "k_new", "v_new")}
    if inter:
        # one ring per layer with key and value of a slot side by side, drawn on the device
        gd = torch.Generator(device=dev).manual_seed(cfg.seed + 1)
        kv = torch.randn(cfg.layers, cfg.S, cfg.H, cfg.R, 2, cfg.D, generator=gd, device=dev, dtype=cfg.dtype)
        kr = vr = None
    else:
        kr, vr = x["k_ring"].to(dev), x["v_ring"].to(dev)
    q, kn, vn = (host[nm].to(dev) for nm in ("q", "k_new", "v_new"))
    head = x["head"].to(dev); pb = x["pos_bias"].to(dev); gain = x["head_gain"].to(dev)
    out = torch.empty_like(q)
    L = cfg.layers
    stream = torch.cuda.current_stream()

    def step():
        for l in range(L):
            # from the second layer of a token on, the kernel ahead in the stream is another layer's
            # step (its own rings), so the overlapped launch is allowed
            if inter:
                dwarf_b200.dsqg_decode_step_kv(q[l], kn[l], vn[l], kv[l], head, pb, gain, None, cfg.offsets,
                                               None, out[l], overlap=args.decode_overlap and l > 0)
            else:
                dwarf_b200.dsqg_decode_step(q[l], kn[l], vn[l], kr[l], vr[l], head, pb, gain, None, cfg.offsets,
                                            None, out[l], overlap=args.decode_overlap and l > 0)

    sampler = ClockSampler(local_rank)
    if rank == 0 and sample_clocks:
        sampler.start()
    for _ in range(args.warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ddist.barrier(); torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize(); ddist.barrier()
    eager_ms = ddist.max_over_ranks(e0.elapsed_time(e1), dev if world > 1 else "cpu") / args.steps
    # The 10 launches of a step are latency-bound: replay them as one CUDA graph (the library
    # neither allocates nor synchronises, so its calls can be captured as they are).
    graph = torch.cuda.CUDAGraph()
    gs = torch.cuda.Stream()
    gs.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(gs):
        step()
        gs.synchronize()
        with torch.cuda.graph(graph, stream=gs):
            step()
    torch.cuda.current_stream().wait_stream(gs)
    for _ in range(args.warmup):
        graph.replay()
    ddist.barrier(); torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(args.steps):
        graph.replay()
    e1.record(stream)
    torch.cuda.synchronize(); ddist.barrier()
    ms = ddist.max_over_ranks(e0.elapsed_time(e1), dev if world > 1 else "cpu") / args.steps

    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    e2e_steps = max(3, min(args.steps, 50))

    def e2e_step():
        for nm, dst in (("q", q), ("k_new", kn), ("v_new", vn)):
            dst.copy_(host[nm], non_blocking=True)
        step()
        out_host.copy_(out, non_blocking=True)
    e2e_step()
    torch.cuda.synchronize(); ddist.barrier()
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    torch.cuda.synchronize(); ddist.barrier()
    e2e_ms = ddist.max_over_ranks(e0.elapsed_time(e1), dev if world > 1 else "cpu") / e2e_steps
    clocks = sampler.stop() if rank == 0 and sample_clocks else None

    J = len(cfg.offsets)
    esz = 2
    per_pair = 2 * J * cfg.D * esz + 2 * cfg.D * esz + 2 * cfg.D * esz   # taps K+V, ring write, q + out
    layer_bytes = per_pair * cfg.S * cfg.H
    peak, peak_src = measured_peaks()
    achieved = layer_bytes * L / (ms * 1e-3) / 1e9
    tokens = cfg.S * world
    small = 3 * cfg.S * cfg.H * cfg.D * esz * L
    return {
        "metric": "DSQG decode tokens/s", "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg.name, "l2": f"ring footprint {2 * L * cfg.S * cfg.H * cfg.R * cfg.D * esz / 1e9:.1f} GB >> L2",
                   "rings": ("one ring per layer, key and value of a slot side by side [S,H,R,2,D]" if inter
                             else "separate K and V rings per layer [S,H,R,D]"),
                   "launch": f"one CUDA graph of the {L} per-layer launches per step"
                             + ("; layers after the first launched with programmatic dependent launch "
                                "(ring gather overlaps the layer before)" if args.decode_overlap else ""),
                   "parallelism": f"sequences replicated x{world}, no collective"},
        "ms_per_step_eager": eager_ms,
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": small,
                "d2h_bytes_per_step": small // 3, "ms_per_step": e2e_ms, "steps": e2e_steps},
        "gpu_launches": L * args.steps,
        "roofline": {"bound": "hbm", "kernel": "dsqg_decode", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     # DRAM read+write of one launch from the committed ncu capture of this shape
                     "frac": achieved / peak, "traffic": 34.27e6 if cfg.name.startswith("cfg3") else None,
                     "peak_source": peak_src, "algorithmic_bytes_per_launch": layer_bytes, "ms_per_launch": ms / L},
        "clocks": clocks,
    }


def run_train_workload(args, rank, local_rank, world):
    """cfg4: end-to-end training step of the condM-shaped LM (fwd + bwd + AdamW), bf16 autocast,
    DDP gradient all-reduce over NCCL when world > 1.  Token ids come from pinned host memory
    every step and the loss is read back: the whole step is the end-to-end path."""
    import torch.nn.functional as F
    from dwarf_b200 import dist as ddist
    from dwarf_b200.model import CondMLM

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    B, N, V = 32, 2048, 32000
    torch.manual_seed(1234)
    model = CondMLM(vocab=V, seq_len=N, attention=args.lm_attention).to(dev)
    if not args.packed_layout:          # A/B: the reference's permute copies and separate gate multiply
        for blk in model.blocks:
            if hasattr(blk.attn, "_packed"):
                blk.attn._packed = False
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank])
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, fused=True)
    g = torch.Generator().manual_seed(4321 + rank)
    host_ids = torch.randint(0, V, (B, N + 1), generator=g).pin_memory()
    loss_host = torch.zeros((), dtype=torch.float32).pin_memory()
    stream = torch.cuda.current_stream()

    def step():
        ids = host_ids.to(dev, non_blocking=True)
        with torch.amp.autocast("cuda", dtype=torch.bfloat16):
            logits = model(ids[:, :-1])
        loss = F.cross_entropy(logits.float().view(-1, V), ids[:, 1:].reshape(-1))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        loss_host.copy_(loss.detach(), non_blocking=True)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ddist.barrier(); torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize(); ddist.barrier()
    ms = ddist.max_over_ranks(e0.elapsed_time(e1), dev if world > 1 else "cpu") / args.steps
    allreduce = None
    if world > 1:
        # the same steps with DDP's gradient all-reduce switched off (no_sync): the difference is what the
        # all-reduce adds to the step after its overlap with the backward pass
        with model.no_sync():
            for _ in range(2):
                step()
            ddist.barrier(); torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(args.steps):
                step()
            e1.record(stream)
            torch.cuda.synchronize(); ddist.barrier()
        ms_ns = ddist.max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
        grad_bytes = sum(p.numel() * 4 for p in model.parameters() if p.requires_grad)
        allreduce = {"ms_per_step_without_allreduce": ms_ns, "exposed_ms": ms - ms_ns, "share_of_step": (ms - ms_ns) / ms,
                     "gradient_bytes": grad_bytes, "backend": "nccl"}
    clocks = sampler.stop() if rank == 0 else None
    tokens = B * N * world
    val = tokens / (ms * 1e-3)
    n_params = sum(p.numel() for p in model.parameters())
    return {
        "metric": "condM-shaped LM training tokens/s", "value": val, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "cfg4 condM-shaped LM train step: 6 layers d256 8x32 heads FFN1024 vocab32000, "
                               "DSQG layers 0-4 + full attention layer 5, B32/GPU N2048, AdamW",
                   "dsqg_layers": args.lm_attention + (", q/k/v read in place, gate folded (strided entry points)"
                                                       if args.packed_layout and args.lm_attention == "condM"
                                                       else ", permute copies + separate gate multiply"),
                   "parameters": n_params, "final_loss": float(loss_host),
                   "parallelism": f"dp{world} (DDP, NCCL gradient all-reduce)" if world > 1 else "single GPU"},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": B * (N + 1) * 8, "d2h_bytes_per_step": 4,
                "note": "the timed step already starts from pinned host token ids and ends with the loss on the host"},
        "gpu_launches": 3 * 5 * args.steps,      # DSQG forward + dQ + dK/dV kernels of the 5 DSQG layers (others are library GEMMs)
        "allreduce": allreduce,
        "clocks": clocks,
    }


# ----------------------------------------------------------------------------- CPU legs
def cpu_reference_time(cfg, sample_B, repeats, fwd_bwd=True, with_se=False):
    """Times the PyTorch restatement of the reference's DSQG path (oracle/dsqg_oracle.py, a
    line-for-line generalisation of kernels/dsqg_attention_v3.py:543-561) on the host cores.
    This is the one place outside tests/ where oracle/ is executed: as the measured baseline."""
    from dwarf_b200 import synth
    from oracle import dsqg_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    x = synth.make_op_inputs(cfg, B=sample_B)
    se = None
    if with_se:
        se = torch.randn(len(cfg.offsets), cfg.D, generator=torch.Generator().manual_seed(1234)) * 0.05
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        if fwd_bwd:
            O.dsqg_reference_grads(x["q"], x["k"], x["v"], x["pos_bias"], x["dout"], se, x["head_gain"],
                                   cfg.offsets, chunk=1)
        else:
            O.dsqg_reference_chunked(x["q"], x["k"], x["v"], x["pos_bias"], se, x["head_gain"], cfg.offsets, 1)
        best = min(best, time.perf_counter() - t0)
    return sample_B * cfg.N / best, best


def run_reference_arm(args, cfg):
    """--impl reference: the reference's own (CPU, PyTorch) implementation of the path.  The
    reference checkout does not travel with the repository, so its restatement in oracle/ is
    timed (bit-identical to the reference functions on their 44-offset set)."""
    sample_B = 2
    from dwarf_b200 import synth
    from oracle import dsqg_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    x = synth.make_op_inputs(cfg, B=sample_B)
    se = None
    if args.scale_embed:
        se = torch.randn(len(cfg.offsets), cfg.D, generator=torch.Generator().manual_seed(1234)) * 0.05

    def step():
        O.dsqg_reference_grads(x["q"], x["k"], x["v"], x["pos_bias"], x["dout"], se, x["head_gain"],
                               cfg.offsets, chunk=1)
    for _ in range(min(args.warmup, 1)):
        step()
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    el = (time.perf_counter() - t0) / steps
    val = sample_B * cfg.N / el
    sample = f"{sample_B} of {cfg.B} batch entries per step ({sample_B * cfg.N} tokens), fwd+bwd via autograd, fp32"
    return {
        "impl": "reference", "metric": "DSQG fwd+bwd tokens/s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": el * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg.name, "tokens_per_step_per_gpu": cfg.B * cfg.N},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=["cfg1", "cfg2", "cfg2_4k", "cfg3", "cfg4"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scale-embed", action="store_true",
                    help="op workloads: add the condU scale_embed term (seeded N(0, 0.05) [J,D]) and its gradient")
    ap.add_argument("--batch", type=int, default=0, help="op workloads: batch size instead of the configuration's")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="op workloads at N > 1: weak = every GPU runs the configuration's batch (default); "
                         "strong = the configuration's batch is split over the GPUs")
    ap.add_argument("--no-decode-overlap", dest="decode_overlap", action="store_false",
                    help="cfg3: launch every layer as an ordinary kernel (default: layers after the first overlap the one before)")
    ap.add_argument("--ring-layout", choices=["interleaved", "separate"], default="interleaved",
                    help="cfg3: one K/V ring per layer with key and value of a slot side by side (default) or two rings")
    ap.add_argument("--decode-layers", type=int, default=0, help="cfg3: number of layers (default: the 10 of the configuration)")
    ap.add_argument("--kernel-path", type=int, default=0,
                    help="dsqg_set_kernel_path value for A/B runs: 0 automatic (default), 1 generic, 2 tensor-core, "
                         "3 forward with TMA-staged V, 4 forward with the dense window on tcgen05 and tensor memory")
    ap.add_argument("--dense-window-only", action="store_true",
                    help="op workloads: keep only the offsets 0..32 of the configuration's set (A/B measurement of the "
                         "dense-window part of the kernels; not a configuration of the specification)")
    ap.add_argument("--lm-attention", choices=["condM", "condU"], default="condM",
                    help="cfg4: DSQG layers with the position bias only (condM, the configuration's shape) or with "
                         "scale_embed and the per-head gain (condU)")
    ap.add_argument("--no-packed-layout", dest="packed_layout", action="store_false",
                    help="cfg4: make the permute copies before / after the op and the gate multiply in PyTorch, as the "
                         "reference does, instead of the strided entry points (A/B measurement)")
    ap.add_argument("--no-extras", dest="extras", action="store_false",
                    help="op workloads: only the headline measurement (default: the line also carries the operator "
                         "API, the other op configurations, the decode step and, at N > 1, the strong-scaling split)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    # stdout carries exactly one JSON line: whatever libraries write to file descriptor 1 while
    # the benchmark runs (NCCL's version banner, for one) is sent to stderr instead
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    from dwarf_b200 import dist as ddist, synth
    rank, local_rank, world = ddist.env_world()

    if args.impl == "reference":
        if rank == 0:
            cfg = synth.OP_CONFIGS["cfg1" if args.workload in ("cfg3", "cfg4") else args.workload]
            print(json.dumps(run_reference_arm(args, cfg)), file=json_out, flush=True)
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the DSQG kernels have no CPU fallback")
    ddist.init_process_group("nccl")
    if args.kernel_path:
        from dwarf_b200 import _lib
        _lib.check(_lib.load().dsqg_set_kernel_path(args.kernel_path), "dsqg_set_kernel_path")
    if args.workload == "cfg3":
        line = run_decode_workload(args, rank, local_rank, world)
    elif args.workload == "cfg4":
        line = run_train_workload(args, rank, local_rank, world)
    else:
        cfg = synth.OP_CONFIGS[args.workload]
        line = run_op_workload(args, cfg, rank, local_rank, world)
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            sample_B = min(cfg.B, 32)
            val, secs = cpu_reference_time(cfg, sample_B, repeats=4, with_se=args.scale_embed)
            line["cpu_baseline"] = {"value": val, "unit": "tokens/s", "cores": torch.get_num_threads(),
                                    "kind": "port",
                                    "sample": f"{sample_B} of {cfg.B} batch entries ({sample_B * cfg.N} tokens), "
                                              f"fwd+bwd via autograd in fp32, best of 4 ({secs:.2f} s)"}
    if rank == 0:
        print(json.dumps(line), file=json_out, flush=True)
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
