#!/usr/bin/env python
"""Benchmark of the tensor-transpose hot path (cuttPlanMeasure -> cuttExecute).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

For N > 1 launch it under torch.distributed.run (one rank per GPU); RANK / LOCAL_RANK /
WORLD_SIZE are read from the environment.

Workloads (all data synthetic, seeded or closed-form):
  c5a  (default, every N) rank-4 fp32 (1024,1024,32,256), permutation (1,0,2,3), sharded on the
       last dimension over the N ranks: slab mode, no communication.  The 34 GB tensor is fixed,
       so this is strong scaling; at N = 1 the whole tensor is transposed by one GPU.  The same
       line also carries
         * at N >= 2: block "c5b" - the same tensor with permutation (3,2,0,1): the sharded
           dimension moves, every rank stores its tiles into the peers' output slabs from
           inside the kernel (NVLink all-to-all, no NCCL in the data path);
         * at N = 1: block "extras" - the single-GPU workloads c2, c3 (measured, model-only,
           and a hold-out suite the cost model never saw), c4, c1 and the original cuTT on the
           same GPU.
  c5b  headline = the all-to-all permutation.
  c2   one step = the 14142 x 14142 matrix transpose in fp32 and then in fp64 (two launches).
       With N > 1 every rank transposes its own pair (independent replicas, weak scaling).
  c4   rank-6 fp32 tensor with tiny leading dimensions.   c1  the 0.8 MB README tensor.
  c3   the 100-case random rank 2-7 suite (fp64 and fp32); value = median over cases.

Every timed plan's output is verified once, outside the timed region, against the permutation's
index formula (oracle/device_check.py: the 64-bit restatement of the reference's checker); the
line is only printed with "bit_exact": true when every check found zero mismatches, and every
cuttExecute return code inside the timed loops is checked.

Metric: effective GB/s = 2 * volume * sizeofType / time  (the reference's definition,
src/cuttTimer.cpp:92,134-138), whole job over all ranks.  One JSON line on stdout (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "effective_transpose_bandwidth"
UNIT = "GB/s"


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            with open(p) as f:
                return float(json.load(f)["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def _vol(dims):
    v = 1
    for d in dims:
        v *= int(d)
    return v


def _c5_dims(args):
    from cutt_b200 import workloads as W
    dims = list(W.C5_DIMS)
    if args.c5_scale > 1:           # smaller stand-in for quick checks: shrink dim 2
        dims[2] = max(1, dims[2] // args.c5_scale)
    return dims


def workload_config(args, world):
    """Static description of the workload; both arms print exactly this dictionary."""
    from cutt_b200 import workloads as W
    w = args.workload
    if w in ("c5a", "c5b"):
        dims = _c5_dims(args)
        perm = W.C5A_PERM if w == "c5a" else W.C5B_PERM
        mode = ("slab mode, no communication" if w == "c5a"
                else "all-to-all by peer stores from inside the kernel")
        return {"workload": "%s: rank-4 fp32 %s perm %s sharded on the last dim over %d GPU(s), %s"
                            % (w, tuple(dims), tuple(perm), world, mode),
                "dims": dims, "perm": list(perm), "elt": [4],
                "l2": "inputs larger than L2 (%.1f GB per side over all ranks)" % (_vol(dims) * 4 / 1e9)}
    if w == "c2":
        return {"workload": "c2: rank-2 transpose (14142,14142) perm (1,0), fp32 then fp64 per step",
                "dims": list(W.C2[0]), "perm": list(W.C2[1]), "elt": [4, 8],
                "l2": "inputs larger than L2 (0.8 GB and 1.6 GB per side)"}
    if w == "c4":
        return {"workload": "c4: rank-6 fp32 (4,3,5,400,7,2400) perm (4,1,5,0,3,2)",
                "dims": list(W.C4[0]), "perm": list(W.C4[1]), "elt": [4],
                "l2": "inputs larger than L2 (1.6 GB per side)"}
    if w == "c1":
        return {"workload": "c1: rank-4 fp64 (31,549,2,3) perm (3,0,2,1)",
                "dims": list(W.C1[0]), "perm": list(W.C1[1]), "elt": [8],
                "l2": "0.8 MB tensor: L2 is flushed between timed launches"}
    if w == "c3":
        return {"workload": "c3: %d seeded random rank 2-7 tensors of ~2e8 elements, fp64 and fp32; median over cases"
                            % args.suite_cases,
                "dims": None, "perm": None, "elt": [8, 4], "l2": "inputs larger than L2"}
    raise ValueError(w)


def _cases_of(args):
    """(name, dims, perm, elt) list of one step of a single-GPU workload."""
    from cutt_b200 import workloads as W
    w = args.workload
    if w == "c2":
        return [("c2_f32", W.C2[0], W.C2[1], 4), ("c2_f64", W.C2[0], W.C2[1], 8)]
    if w == "c4":
        return [("c4_f32", W.C4[0], W.C4[1], 4)]
    if w == "c1":
        return [("c1_f64", W.C1[0], W.C1[1], 8)]
    raise ValueError(w)


def _cpu_sample_cases(args):
    """Bounded sample of the workload for the legs that run on the host cores."""
    from cutt_b200 import workloads as W
    w = args.workload
    if w in ("c5a", "c5b"):
        dims = list(W.C5_SAMPLE_DIMS)
        if args.c5_scale > 1:
            dims[2] = max(1, dims[2] // args.c5_scale)
        perm = W.C5A_PERM if w == "c5a" else W.C5B_PERM
        return [(w + "_sample", dims, perm, 4)], \
            "the same permutation on a slab of %d positions of the sharded dimension, dims %s (%.2f GB per side)" \
            % (dims[3], dims, _vol(dims) * 4 / 1e9)
    if w == "c3":
        cases = []
        for i, (d, p) in enumerate(W.c3_cases(4)):
            cases += [("c3_%d_f64" % i, d, p, 8), ("c3_%d_f32" % i, d, p, 4)]
        return cases, "the first 4 of the suite's cases, fp64 and fp32"
    return _cases_of(args), "the full workload"


# ----------------------------------------------------------------------------------------
# CPU legs: the restatement of the permutation (oracle/host_transpose.c, blocked OpenMP loop
# nest) on the host cores.  The original library has no CPU implementation and no sm_100 build.
def _cpu_buffers(cases):
    import numpy as np
    bufs = []
    for i, (name, dims, perm, elt) in enumerate(cases):
        a = np.random.default_rng(5 + i).random(_vol(dims), dtype=np.float32 if elt == 4 else np.float64)
        bufs.append((dims, perm, a, np.empty_like(a)))
    nbytes = sum(2 * a.size * a.dtype.itemsize for _, _, a, _ in bufs)
    return bufs, nbytes


def cpu_baseline(args):
    """About 10 s of the CPU restatement on a bounded sample of the workload, all host cores."""
    import oracle
    cores = oracle.use_all_cores()
    cases, sample = _cpu_sample_cases(args)
    bufs, nbytes = _cpu_buffers(cases)
    for dims, perm, a, o in bufs:  # warm (page faults of the output buffer)
        oracle.transpose_blocked(dims, perm, a, o)
    n = 0
    t0 = time.perf_counter()
    while True:
        for dims, perm, a, o in bufs:
            oracle.transpose_blocked(dims, perm, a, o)
        n += 1
        if time.perf_counter() - t0 > 10.0 or n >= 64:
            break
    dt = (time.perf_counter() - t0) / n
    return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "%d steps of: %s; blocked OpenMP loop nest (oracle/host_transpose.c)" % (n, sample)}


def run_reference(args):
    """Reference arm: the CPU restatement with every host thread, --warmup untimed and --steps
    timed steps, each step one pass over the bounded sample.  Rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import oracle
    cores = oracle.use_all_cores()   # launchers export OMP_NUM_THREADS=1 to their children
    cases, sample = _cpu_sample_cases(args)
    bufs, nbytes = _cpu_buffers(cases)

    def step():
        for dims, perm, a, o in bufs:
            oracle.transpose_blocked(dims, perm, a, o)

    warm = max(3, args.warmup)   # the GPU arm warms up at least three times as well
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    val = nbytes / dt / 1e9
    sharded = args.workload in ("c5a", "c5b")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": warm, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong" if sharded else "weak", "vs_baseline": None,
        "dtype": _dtype_of(args), "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "each step: %s; one process on the host cores whatever N is" % sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the original cuTT has no CPU implementation and no sm_100 build; this arm times "
                "the CPU restatement of its permutation (oracle/host_transpose.c) on the host cores",
    }
    print(json.dumps(line))
    return 0


def _dtype_of(args):
    return {"c5a": "b32 (bit moves)", "c5b": "b32 (bit moves)", "c4": "b32 (bit moves)",
            "c1": "b64 (bit moves)"}.get(args.workload, "b32+b64 (bit moves)")


# ----------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.dev = device_index
        self.proc = None
        self.path = "/tmp/cutt_bench_clocks_%d.csv" % os.getpid()

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for ln in f:
                    p = [x.strip() for x in ln.split(",")]
                    if len(p) < 9 or not p[0].isdigit() or int(p[0]) != self.dev:
                        continue
                    try:
                        sm.append(float(p[1])); mx.append(float(p[2]))
                    except ValueError:
                        continue
                    for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                        if v.lower().startswith("active"):
                            reasons.add(name)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            # samples under load: the upper half of the observed clocks
            sm.sort()
            out["sm_mhz"] = statistics.median(sm[len(sm) // 2:])
            out["sm_max_mhz"] = max(mx)
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def _physical_gpu_index(local_device: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_device])
        except Exception:
            return local_device
    return local_device


class Ctx:
    """Per-process state of the GPU arm."""

    def __init__(self, args):
        import torch
        import cutt_b200 as C
        from cutt_b200 import workloads as W
        from oracle import device_check as DC   # checker only: never inside a timed region
        self.args, self.torch, self.C, self.W, self.DC = args, torch, C, W, DC
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the transpose path has no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist
        C.lib()
        if args.plan_cache and os.path.exists(args.plan_cache):
            C.plan_cache_load(args.plan_cache)
        self.peak, self.peak_kind = _peaks()
        self.stream = torch.cuda.current_stream().cuda_stream
        self.checks = {}          # name -> mismatches found by the verification steps

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.dist is None:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, x: int) -> int:
        if self.dist is None:
            return x
        t = self.torch.tensor([x], dtype=self.torch.int64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return int(t.item())

    def check(self, name, dims, perm, tout, tin=None, **kw):
        """Verifies one output against the index formula; records the mismatch count."""
        torch = self.torch
        it = torch.int32 if tout.element_size() == 4 else torch.int64
        bad = self.DC.count_mismatches(dims, perm, tout.view(it), None if tin is None else tin.view(it), **kw)
        self.checks[name] = self.checks.get(name, 0) + bad
        return bad

    def finish(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


def base_line(args, value, ms_per_step, world, scaling):
    return {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": _dtype_of(args), "data": "synthetic"}


def _traffic(key, algorithmic_bytes):
    """DRAM bytes per launch of the dominant kernel from the committed ncu captures
    (profiles/traffic.json).  An entry is either a byte count for the full-size launch or
    {"dram_bytes", "algorithmic_bytes"} of a smaller capture of the same kernel, which is scaled
    to this launch by the bytes moved."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            e = json.load(f).get(key)
    except Exception:
        return None
    if isinstance(e, dict):
        try:
            return float(e["dram_bytes"]) / float(e["algorithmic_bytes"]) * algorithmic_bytes
        except Exception:
            return None
    return e


# ----------------------------------------------------------------------------------------
def time_sharded(ctx, which, steps, warmup, sample_clocks):
    """One sharded workload (c5a / c5b) on all ranks: plan by measurement, timed steps, full
    verification of this rank's output slab.  Returns a dictionary of results."""
    torch, C, W = ctx.torch, ctx.C, ctx.W
    from cutt_b200.multigpu import ShardedTranspose
    args = ctx.args
    dims = _c5_dims(args)
    perm = W.C5A_PERM if which == "c5a" else W.C5B_PERM
    elt = 4
    vol = _vol(dims)
    loc = vol // ctx.world
    # closed-form content (a hash of the global element index): every rank can verify its output
    # slab without reading another GPU's input
    inp = torch.empty(loc, dtype=torch.int32, device="cuda")
    ctx.DC.fill_pattern(inp, first_index=ctx.rank * loc)
    st = ShardedTranspose(dims, perm, elt, measure_input=inp)
    for _ in range(max(3, warmup)):
        st.execute(inp)
    st.finish()
    sampler = ClockSampler(_physical_gpu_index(ctx.local))
    if sample_clocks and ctx.rank == 0:
        sampler.start()
        time.sleep(0.3)
    ctx.barrier()
    st.execute(inp)   # untimed: the GPU idled while the clock sampler started
    l0 = C.launch_count()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        st.execute(inp)          # raises on a non-zero return code
    e1.record()
    ctx.barrier()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / steps
    launches = C.launch_count() - l0
    clocks = sampler.stop() if (sample_clocks and ctx.rank == 0) else None
    # verification: wipe the slab, run once more, compare every element of the slab
    st.out.fill_(-1)
    st.finish()
    st.execute(inp)
    st.finish()
    bad = ctx.check(which, dims, perm, st.out, None, out_first=ctx.rank * loc)
    bad = ctx.sum_over_ranks(bad)
    ctx.checks[which] = bad
    total_bytes = 2 * vol * elt
    value = total_bytes / (ms * 1e-3) / 1e9
    res = {"value": value, "ms_per_step": ms, "per_gpu_gbs": value / ctx.world, "launches": launches,
           "clocks": clocks, "mode": "slab" if st.mode == 0 else "all-to-all by peer stores",
           "plan": json.loads(C.plan_describe(st.handle))["label"], "mismatches": bad,
           "bytes_per_gpu_per_launch": total_bytes // ctx.world,
           "per_gpu_frac_of_peak": value / ctx.world / ctx.peak}
    if st.mode == 1 and ctx.world > 1:
        remote = (ctx.world - 1) / ctx.world * loc * elt      # bytes each GPU sends over NVLink per step
        nv = remote / (ms * 1e-3) / 1e9
        res["nvlink"] = {"remote_gbs_per_gpu_per_direction": nv, "frac_of_770_measured_peer_copy": nv / 770.0,
                         "frac_of_900_nominal": nv / 900.0,
                         "destination_run_bytes": dims[3] // ctx.world * elt}
    st.close()
    del inp, st
    torch.cuda.empty_cache()
    return res


def run_emulated(ctx):
    """--emulate-world N on ONE GPU: the N ranks' parts of a sharded workload run back to back on
    this device, every "peer" slab being another local buffer (the kernels never wait for each
    other, so this is legitimate).  It exists to profile the peer-store kernel's instruction and
    DRAM behaviour without NVLink; the GB/s it prints say nothing about a multi-GPU job."""
    torch, C, W = ctx.torch, ctx.C, ctx.W
    from cutt_b200 import multigpu as mg
    args = ctx.args
    world = args.emulate_world
    dims = _c5_dims(args)
    perm = W.C5A_PERM if args.workload == "c5a" else W.C5B_PERM
    vol = _vol(dims)
    loc = vol // world
    ins, outs = [], []
    for g in range(world):
        t = torch.empty(loc, dtype=torch.int32, device="cuda")
        ctx.DC.fill_pattern(t, first_index=g * loc)
        ins.append(t)
        outs.append(torch.full((loc,), -1, dtype=torch.int32, device="cuda"))
    ptrs = [o.data_ptr() for o in outs]
    handles = []
    for g in range(world):
        rc, h = mg.mg_plan_measure(dims, perm, 4, world, g, ctx.stream, ins[g].data_ptr(), ptrs)
        if rc != 0:
            raise SystemExit("cutt_mg_plan_measure failed: %d" % rc)
        handles.append(h)

    def step():
        for g, h in enumerate(handles):
            rc = mg.mg_execute(h, ins[g].data_ptr(), ptrs)
            if rc != 0:
                raise SystemExit("cutt_mg_execute failed: %d" % rc)

    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    l0 = C.launch_count()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    launches = C.launch_count() - l0
    for o in outs:
        o.fill_(-1)
    step()
    torch.cuda.synchronize()
    for g in range(world):
        ctx.check("%s_emulated" % args.workload, dims, perm, outs[g], None, out_first=g * loc)
    value = 2 * vol * 4 / (ms * 1e-3) / 1e9
    line = base_line(args, value, ms, 1, "weak")
    line["config"] = workload_config(args, world)
    line["config"]["workload"] += " - EMULATED: all %d ranks run back to back on one GPU" % world
    line["detail"] = {"plans": [json.loads(C.plan_describe(h))["label"] for h in handles[:2]],
                      "mode": "slab" if mg.mg_mode(handles[0]) == 0 else "all-to-all by stores into %d local slabs" % world}
    line["roofline"] = {"bound": "hbm", "achieved": value, "peak": ctx.peak, "unit": UNIT, "frac": value / ctx.peak,
                        "traffic": None, "peak_kind": ctx.peak_kind}
    line["gpu_launches"] = launches
    line["e2e"] = None
    for h in handles:
        C.cuttDestroy(h)
    return line


def e2e_host_leg(ctx, cases, steps):
    """The same metric through cutt_c_transpose_host: pinned host buffers in, pinned host buffers
    out, the uploads and downloads inside the timed region.  Every rank runs its own copy."""
    torch, C = ctx.torch, ctx.C
    hbufs = []
    for i, (name, dims, perm, elt) in enumerate(cases):
        vol = _vol(dims)
        dt = torch.int32 if elt == 4 else torch.int64
        hin = torch.empty(vol, dtype=dt, pin_memory=True)
        dtmp = torch.empty(vol, dtype=dt, device="cuda")
        ctx.DC.fill_pattern(dtmp, first_index=0)
        hin.copy_(dtmp)
        del dtmp
        hout = torch.empty(vol, dtype=dt, pin_memory=True)
        hbufs.append((name, dims, perm, elt, hin, hout))
    torch.cuda.synchronize()
    nbytes = sum(2 * _vol(d) * e for _, d, _, e, _, _ in hbufs)

    def step():
        for name, dims, perm, elt, hin, hout in hbufs:
            rc = C.transpose_host(dims, perm, elt, hin.data_ptr(), hout.data_ptr())
            if rc != 0:
                raise SystemExit("cutt_c_transpose_host failed: %d" % rc)

    step()
    ctx.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    ctx.barrier()
    secs = ctx.max_over_ranks((time.perf_counter() - t0) / steps)
    bad = 0
    for name, dims, perm, elt, hin, hout in hbufs:
        bad += ctx.check("e2e", dims, perm, hout.cuda(), None)
    bad = ctx.sum_over_ranks(bad)
    ctx.checks["e2e"] = bad
    del hbufs
    return {"value": ctx.world * nbytes / secs / 1e9, "unit": UNIT, "h2d_bytes_per_step": nbytes // 2,
            "d2h_bytes_per_step": nbytes // 2, "steps": steps, "mismatches": bad}


def run_default(ctx):
    """c5a (or c5b) headline at every N; c5b block at N >= 2; single-GPU extras at N = 1."""
    args = ctx.args
    head = time_sharded(ctx, args.workload, args.steps, args.warmup, True)
    line = base_line(args, head["value"], head["ms_per_step"], ctx.world, "strong")
    line["config"] = workload_config(args, ctx.world)
    line["detail"] = {"mode": head["mode"], "plan": head["plan"], "per_gpu_gbs": head["per_gpu_gbs"],
                      "whole_job_gbs": head["value"]}
    line["roofline"] = {"bound": "hbm", "achieved": head["per_gpu_gbs"], "peak": ctx.peak, "unit": UNIT,
                        "frac": head["per_gpu_gbs"] / ctx.peak,
                        "traffic": _traffic(args.workload, head["bytes_per_gpu_per_launch"]),
                        "kernel": "permute_tiles_kernel (one launch per GPU per step)",
                        "peak_kind": ctx.peak_kind, "per": "GPU"}
    if "nvlink" in head:
        line["nvlink"] = head["nvlink"]
    line["gpu_launches"] = head["launches"]
    line["clocks"] = head["clocks"]
    # end to end through host buffers: a bounded sample of the same permutation per rank
    if not args.no_e2e:
        cases, sample = _cpu_sample_cases(args)
        e2e = e2e_host_leg(ctx, cases, max(1, min(args.steps, 3)))
        e2e["sample"] = "every rank: " + sample
        line["e2e"] = e2e
    else:
        line["e2e"] = None
    if ctx.world > 1 and args.workload == "c5a" and not args.no_extras:
        b = time_sharded(ctx, "c5b", args.steps, args.warmup, False)
        line["c5b"] = {"workload": "same tensor, perm %s: all-to-all by peer stores over NVLink" % (tuple(ctx.W.C5B_PERM),),
                       "value": b["value"], "ms_per_step": b["ms_per_step"], "per_gpu_gbs": b["per_gpu_gbs"],
                       "per_gpu_frac_of_hbm_peak": b["per_gpu_frac_of_peak"], "plan": b["plan"],
                       "nvlink": b.get("nvlink"), "mismatches": b["mismatches"]}
    if ctx.rank == 0 and ctx.world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args)
    if ctx.rank == 0 and ctx.world == 1 and not args.no_extras:
        line["extras"] = single_gpu_extras(ctx)
    return line


# ----------------------------------------------------------------------------------------
def time_cases(ctx, cases, steps, warmup, sample_clocks, flush_l2=False):
    """Device-resident timing of a list of (name, dims, perm, elt): cuttPlanMeasure, warm-up,
    `steps` timed steps of one cuttExecute per case, verification of every output."""
    torch, C = ctx.torch, ctx.C
    plans = []
    for ci, (name, dims, perm, elt) in enumerate(cases):
        vol = _vol(dims)
        g = torch.Generator(device="cuda")
        g.manual_seed(2 + ci + 100 * ctx.rank)
        tin = torch.rand(vol, dtype=torch.float32 if elt == 4 else torch.float64, device="cuda", generator=g)
        tout = torch.empty_like(tin)
        rc, h = C.cuttPlanMeasure(len(dims), dims, perm, elt, ctx.stream, tin.data_ptr(), tout.data_ptr())
        if rc != 0:
            raise SystemExit("cuttPlanMeasure failed: %d" % rc)
        plans.append((name, dims, perm, elt, vol, tin, tout, h))
    step_bytes = sum(2 * p[4] * p[3] for p in plans)
    flush = torch.empty(1 << 28, dtype=torch.uint8, device="cuda") if flush_l2 else None

    def step():
        for p in plans:
            if flush is not None:
                flush.fill_(1)
            rc = C.cuttExecute(p[7], p[5].data_ptr(), p[6].data_ptr())
            if rc != 0:
                raise SystemExit("cuttExecute failed: %d" % rc)

    for _ in range(max(3, warmup)):
        step()
    sampler = ClockSampler(_physical_gpu_index(ctx.local))
    if sample_clocks and ctx.rank == 0:
        sampler.start()
        time.sleep(0.3)
    ctx.barrier()
    step()   # the GPU idled while the clock sampler started: one more untimed step
    launches_t0 = C.launch_count()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2 * len(plans))] for _ in range(steps)]
    for k in range(steps):
        for i, p in enumerate(plans):
            if flush is not None:
                flush.fill_(1)
            ev[k][2 * i].record()
            rc = C.cuttExecute(p[7], p[5].data_ptr(), p[6].data_ptr())
            ev[k][2 * i + 1].record()
            if rc != 0:
                raise SystemExit("cuttExecute failed inside the timed loop: %d" % rc)
    ctx.barrier()
    launches = C.launch_count() - launches_t0
    if flush is None:
        total_ms = ev[0][0].elapsed_time(ev[-1][-1])
    else:   # the flush launches sit between the timed ones: add up the launches
        total_ms = sum(ev[k][2 * i].elapsed_time(ev[k][2 * i + 1]) for k in range(steps) for i in range(len(plans)))
    total_ms = ctx.max_over_ranks(total_ms)
    clocks = sampler.stop() if (sample_clocks and ctx.rank == 0) else None
    per_case = {}
    for i, p in enumerate(plans):
        ms = statistics.mean(ev[k][2 * i].elapsed_time(ev[k][2 * i + 1]) for k in range(steps))
        bad = ctx.check(p[0], p[1], p[2], p[6], p[5])
        gbs = 2 * p[4] * p[3] / (ms * 1e-3) / 1e9
        per_case[p[0]] = {"ms": ms, "gbs": gbs, "frac_of_peak": gbs / ctx.peak, "mismatches": bad,
                          "plan": json.loads(C.plan_describe(p[7]))["label"]}
    ms_per_step = total_ms / steps
    return {"plans": plans, "per_case": per_case, "ms_per_step": ms_per_step, "step_bytes": step_bytes,
            "value": ctx.world * step_bytes / (ms_per_step * 1e-3) / 1e9, "launches": launches, "clocks": clocks}


def d2d_context(ctx, src, nbytes):
    """Same-GPU device-to-device copies of `nbytes`, for context: the driver's copy and this
    library's own copy kernel (the plan an identity permutation gets)."""
    torch, C = ctx.torch, ctx.C
    dst = torch.empty_like(src)

    def timed(fn, n=5):
        for _ in range(2):
            fn()
        a0 = torch.cuda.Event(enable_timing=True); a1 = torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(n):
            fn()
        a1.record()
        torch.cuda.synchronize()
        return 2 * nbytes / (a0.elapsed_time(a1) / n * 1e-3) / 1e9

    d2d = timed(lambda: dst.copy_(src))
    own = None
    n_el = src.numel()
    rc, hc = C.plan_params([n_el // 2, 2], [0, 1], src.element_size(), ctx.stream, method=0)
    if rc == 0:
        own = timed(lambda: C.cuttExecute(hc, src.data_ptr(), dst.data_ptr()))
        C.cuttDestroy(hc)
    return d2d, own


def run_single(ctx):
    """c2 / c4 / c1 as the headline (device-resident value, host-buffer e2e)."""
    args = ctx.args
    cases = _cases_of(args)
    r = time_cases(ctx, cases, args.steps, args.warmup, True, flush_l2=(args.workload == "c1"))
    plans = r["plans"]
    line = base_line(args, r["value"], r["ms_per_step"], ctx.world, "weak")
    line["config"] = workload_config(args, ctx.world)
    dom = max(range(len(plans)), key=lambda i: plans[i][4] * plans[i][3])
    dname = plans[dom][0]
    dom_bytes = 2 * plans[dom][4] * plans[dom][3]
    d2d, own = d2d_context(ctx, plans[dom][5], dom_bytes // 2)
    line["detail"] = {"per_case": r["per_case"], "d2d_copy_gbs": d2d, "own_copy_kernel_gbs": own}
    ach = r["per_case"][dname]["gbs"]
    line["roofline"] = {"bound": "hbm", "achieved": ach, "peak": ctx.peak, "unit": UNIT, "frac": ach / ctx.peak,
                        "traffic": _traffic(dname, dom_bytes), "kernel": "permute_tiles_kernel (%s)" % dname,
                        "peak_kind": ctx.peak_kind, "frac_of_same_run_d2d_copy": ach / d2d}
    line["gpu_launches"] = r["launches"]
    line["clocks"] = r["clocks"]
    for p in plans:
        ctx.C.cuttDestroy(p[7])
    del plans, r
    ctx.torch.cuda.empty_cache()
    line["e2e"] = None if args.no_e2e else e2e_host_leg(ctx, cases, max(1, min(args.steps, 3)))
    if ctx.rank == 0 and ctx.world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args)
    return line


def run_suite(ctx, cases, reps=5, measure=True, name="c3"):
    """cuttPlanMeasure (or cuttPlan: the cost model's first pick) + timed cuttExecute for every
    case, fp64 then fp32; every output verified against the index formula."""
    torch, C = ctx.torch, ctx.C
    out = []
    maxvol = max(_vol(d) for d, _ in cases)
    buf_in = torch.rand(maxvol, dtype=torch.float64, device="cuda")
    buf_out = torch.empty_like(buf_in)
    for ci, (dims, perm) in enumerate(cases):
        vol = _vol(dims)
        for elt in (8, 4):
            if measure:
                rc, h = C.cuttPlanMeasure(len(dims), dims, perm, elt, ctx.stream, buf_in.data_ptr(), buf_out.data_ptr())
            else:
                rc, h = C.cuttPlan(len(dims), dims, perm, elt, ctx.stream)
            if rc != 0:
                raise RuntimeError("plan failed %s %s" % (dims, perm))
            if C.cuttExecute(h, buf_in.data_ptr(), buf_out.data_ptr()) != 0:
                raise RuntimeError("execute failed %s %s" % (dims, perm))
            ts = []
            for _ in range(reps):
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
                rc = C.cuttExecute(h, buf_in.data_ptr(), buf_out.data_ptr())
                e1.record()
                torch.cuda.synchronize()
                if rc != 0:
                    raise RuntimeError("execute failed %s %s" % (dims, perm))
                ts.append(e0.elapsed_time(e1))
            ms = statistics.median(ts)
            label = json.loads(C.plan_describe(h))["label"]
            C.cuttDestroy(h)
            it = torch.int32 if elt == 4 else torch.int64
            bad = ctx.check(name, dims, perm, buf_out.view(it)[:vol], buf_in.view(it)[:vol])
            out.append({"case": ci, "dims": dims, "perm": perm, "elt": elt, "ms": ms,
                        "gbs": 2 * vol * elt / (ms * 1e-3) / 1e9, "plan": label, "mismatches": bad})
    del buf_in, buf_out
    return out


def _suite_summary(ctx, res):
    g = [r["gbs"] for r in res]
    med = statistics.median(g)
    return {"runs": len(res), "median_gbs": med, "frac_of_peak": med / ctx.peak, "frac_of_8000": med / 8000.0,
            "min_gbs": min(g), "max_gbs": max(g), "mismatches": sum(r["mismatches"] for r in res)}


def run_c3(ctx):
    args = ctx.args
    res = run_suite(ctx, ctx.W.c3_cases(args.suite_cases), reps=max(3, args.steps))
    med = statistics.median(r["gbs"] for r in res)
    t_ms = statistics.median(r["ms"] for r in res)
    line = base_line(args, med * ctx.world, t_ms, ctx.world, "weak")
    line["config"] = workload_config(args, ctx.world)
    line["roofline"] = {"bound": "hbm", "achieved": med, "peak": ctx.peak, "unit": UNIT, "frac": med / ctx.peak,
                        "traffic": None, "peak_kind": ctx.peak_kind}
    line["suite"] = _suite_summary(ctx, res)
    if args.verbose:
        line["suite"]["cases"] = res
    line["gpu_launches"] = len(res) * max(3, args.steps)
    line["e2e"] = None
    return line


def c1_back_to_back(ctx, launches=400):
    """Microseconds per launch of the cuttPlan plan for C1 with the tensor resident in L2."""
    C, W, torch, DC = ctx.C, ctx.W, ctx.torch, ctx.DC
    dims, perm = list(W.C1[0]), list(W.C1[1])
    vol = _vol(dims)
    tin = torch.empty(vol, dtype=torch.int64, device="cuda")
    DC.fill_pattern(tin, first_index=0)
    tout = torch.zeros_like(tin)
    C.clear_plan_cache()
    rc, h = C.cuttPlan(len(dims), dims, perm, 8)
    if rc != 0:
        raise RuntimeError("cuttPlan failed: %d" % rc)
    try:
        plan = json.loads(C.plan_describe(h))["label"]
        for _ in range(20):
            C.cuttExecute(h, tin.data_ptr(), tout.data_ptr())
        torch.cuda.synchronize()
        best = None
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(launches):
                if C.cuttExecute(h, tin.data_ptr(), tout.data_ptr()) != 0:
                    raise RuntimeError("cuttExecute failed")
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / launches
            best = us if best is None else min(best, us)
        bad = ctx.check("c1_back_to_back", dims, perm, tout, None)
    finally:
        C.cuttDestroy(h)
    return {"us_per_launch": best, "gbs": 2 * vol * 8 / best / 1e3, "plan": plan, "launches": launches,
            "mismatches": bad, "note": "tensor resident in L2, launches queued back to back on one stream"}


def single_gpu_extras(ctx):
    """The single-GPU workloads beside the sharded headline (N = 1 only).  Nothing here can fail
    the headline: errors are reported inside the block."""
    args, C, W, torch = ctx.args, ctx.C, ctx.W, ctx.torch
    extras = {}
    saved_workload = args.workload
    # c2: the matrix transpose, fp32 + fp64 per step
    try:
        args.workload = "c2"
        cases = _cases_of(args)
        r = time_cases(ctx, cases, args.steps, args.warmup, False)
        plans = r["plans"]
        d2d, own = d2d_context(ctx, plans[1][5], plans[1][4] * plans[1][3])
        extras["c2"] = {"workload": workload_config(args, 1)["workload"], "value": r["value"],
                        "ms_per_step": r["ms_per_step"], "per_case": r["per_case"],
                        "d2d_copy_gbs": d2d, "own_copy_kernel_gbs": own,
                        "traffic": {k: _traffic(k, 0) for k in r["per_case"]}}
        for p in plans:
            C.cuttDestroy(p[7])
        del plans, r
        torch.cuda.empty_cache()
        e = e2e_host_leg(ctx, cases, max(1, min(args.steps, 3)))
        extras["c2"]["e2e"] = e
    except Exception as e:
        extras["c2"] = {"error": repr(e)}
    # c4 and c1
    for w in ("c4", "c1"):
        try:
            args.workload = w
            r = time_cases(ctx, _cases_of(args), args.steps, args.warmup, False, flush_l2=(w == "c1"))
            extras[w] = {"workload": workload_config(args, 1)["workload"], "per_case": r["per_case"]}
            for p in r["plans"]:
                C.cuttDestroy(p[7])
            del r
            torch.cuda.empty_cache()
        except Exception as e:
            extras[w] = {"error": repr(e)}
    # c1 again the way a caller with a small, cache-resident tensor sees it: the same plan
    # (cuttPlan) launched back to back, no flush in between
    try:
        extras["c1"]["back_to_back"] = c1_back_to_back(ctx)
    except Exception as e:
        extras["c1_back_to_back"] = {"error": repr(e)}
    args.workload = saved_workload
    # c3: the cost model alone first (cuttPlan would otherwise find the measured winners in the
    # plan cache), then the measured plans; then a hold-out suite the model never saw
    suite = W.c3_cases(args.suite_cases)
    per_case = None
    try:
        C.clear_plan_cache()
        res0 = run_suite(ctx, suite, reps=5, measure=False, name="c3_cuttPlan")
        extras["c3_suite_cuttPlan"] = _suite_summary(ctx, res0)
        extras["c3_suite_cuttPlan"]["note"] = "cost model's first pick; in-sample: the model was fitted to timings of these shapes"
        res = run_suite(ctx, suite, reps=5, name="c3_cuttPlanMeasure")
        extras["c3_suite"] = _suite_summary(ctx, res)
        per_case = [r["gbs"] for r in res]
        ratios = sorted(a["gbs"] / b["gbs"] for a, b in zip(res0, res))
        extras["c3_suite_cuttPlan"]["over_measured"] = {"median": statistics.median(ratios), "min": ratios[0]}
    except Exception as e:
        extras["c3_suite"] = {"error": repr(e)}
    try:
        hold = W.c3_holdout_cases(args.holdout_cases)
        C.clear_plan_cache()
        h0 = run_suite(ctx, hold, reps=5, measure=False, name="c3_holdout_cuttPlan")
        h1 = run_suite(ctx, hold, reps=5, name="c3_holdout_cuttPlanMeasure")
        ratios = sorted(a["gbs"] / b["gbs"] for a, b in zip(h0, h1))
        extras["c3_holdout"] = {
            "note": "same generator, seeds 2000 and up: shapes the cost model was never fitted to",
            "cuttPlan": _suite_summary(ctx, h0), "cuttPlanMeasure": _suite_summary(ctx, h1),
            "cuttPlan_over_measured": {"median": statistics.median(ratios), "mean": statistics.mean(ratios),
                                       "min": ratios[0]}}
    except Exception as e:
        extras["c3_holdout"] = {"error": repr(e)}
    # the ORIGINAL cuTT on this GPU (PTX-JIT build), same shapes
    try:
        args.workload = "c2"
        extras["reference_cutt_gpu"] = reference_gpu_baseline(_cases_of(args))
        d1, p1 = W.C1
        ref1 = reference_gpu_baseline([("c1", d1, p1, 8), ("c1", d1, p1, 4)],
                                      modes=(("cuttPlanMeasure", ["--measure"]),), reps=20)
        extras["reference_cutt_gpu"]["c1_gbs"] = ref1.get("cuttPlanMeasure", {}).get("per_case_gbs")
        if per_case is not None:
            suite_cases = [("c3", d, p, e) for d, p in suite for e in (8, 4)]
            ref = reference_gpu_baseline(suite_cases, modes=(("cuttPlanMeasure", ["--measure"]),), reps=3)
            rr = ref.get("cuttPlanMeasure", {})
            if "per_case_gbs" in rr:
                ratios = sorted(o / max(x, 1e-9) for o, x in zip(per_case, rr["per_case_gbs"]))
                behind = sorted(((o / max(x, 1e-9), i) for i, (o, x) in enumerate(zip(per_case, rr["per_case_gbs"]))))[:10]
                behind = [{"case": i // 2, "elt": 8 if i % 2 == 0 else 4, "ours_gbs": round(per_case[i], 1),
                           "reference_gbs": rr["per_case_gbs"][i]} for q, i in behind if q < 1.0]
                extras["reference_cutt_gpu"]["c3_suite_cuttPlanMeasure"] = {
                    "median_gbs": statistics.median(rr["per_case_gbs"]), "min_gbs": min(rr["per_case_gbs"]),
                    "max_gbs": max(rr["per_case_gbs"]),
                    "ours_over_reference": {"median": statistics.median(ratios), "min": ratios[0], "max": ratios[-1],
                                            "cases_where_reference_is_faster": sum(1 for x in ratios if x < 1.0),
                                            "slowest_relative_cases": behind}}
            else:
                extras["reference_cutt_gpu"]["c3_suite_cuttPlanMeasure"] = rr
    except Exception as e:
        extras["reference_cutt_gpu"] = {"error": repr(e)}
    args.workload = saved_workload
    return extras


def reference_gpu_baseline(cases, modes=(("cuttPlan", []), ("cuttPlanMeasure", ["--measure"])), reps=5):
    """The original cuTT on this GPU (PTX-JIT build, see oracle/build_ref.py), same shapes,
    both planning modes; runs in a child process because the original exits on CUDA errors."""
    try:
        from oracle import ref_runner
        if not ref_runner.available():
            return {"unavailable": "oracle/_ref/libcutt_ref.so not built (original sources not on this machine)"}
        import tempfile
        spec = [{"dims": list(d), "perm": list(p), "elt": e} for _, d, p, e in cases]
        out = {}
        with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as f:
            json.dump(spec, f)
            path = f.name
        for mode, flag in modes:
            res = subprocess.run([sys.executable, "-m", "oracle.ref_runner", path, "--reps", str(reps), "--device-input"] + flag,
                                 cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
            recs = [json.loads(ln) for ln in res.stdout.splitlines() if ln.startswith("{")]
            if res.returncode != 0 or len(recs) != len(spec):
                out[mode] = {"error": (res.stderr or "no output")[-300:]}
                continue
            tot_bytes = sum(2 * _vol(r["dims"]) * r["elt"] for r in recs)
            tot_ms = sum(r["ms"] for r in recs)
            out[mode] = {"gbs": tot_bytes / (tot_ms * 1e-3) / 1e9,
                         "per_case_gbs": [round(r["gbs"], 1) for r in recs]}
        os.remove(path)
        out["build"] = "unmodified sources, nvcc -gencode arch=compute_60,code=compute_60 (PTX only), driver JIT"
        return out
    except Exception as e:
        return {"error": repr(e)}


def run_ours(args):
    ctx = Ctx(args)
    if args.workload in ("c5a", "c5b") and args.emulate_world > 1:
        if ctx.world != 1:
            raise SystemExit("--emulate-world is a single-process, single-GPU mode")
        line = run_emulated(ctx)
    elif args.workload in ("c5a", "c5b"):
        line = run_default(ctx)
    elif args.workload == "c3":
        line = run_c3(ctx)
    else:
        line = run_single(ctx)
    bad = {k: v for k, v in ctx.checks.items() if v}
    line["bit_exact"] = not bad
    line["verified"] = {"how": "every timed plan's output compared once, outside the timed region, with the "
                               "64-bit index formula of the permutation (oracle/device_check.py)",
                        "outputs_checked": sorted(ctx.checks), "mismatches": sum(ctx.checks.values())}
    if args.plan_cache and ctx.rank == 0:
        ctx.C.plan_cache_save(args.plan_cache)
    rc = 0
    if bad:
        line["error"] = "outputs differ from the permutation: %s" % bad
        rc = 1
    if ctx.rank == 0:
        print(json.dumps(line))
    ctx.finish()
    return rc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5a", choices=["c1", "c2", "c3", "c4", "c5a", "c5b"])
    ap.add_argument("--c5-scale", type=int, default=1, help="divide dim 2 of the C5 tensor (quick checks)")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="c5a/c5b on ONE GPU with this many emulated ranks run back to back (profiling aid)")
    ap.add_argument("--suite-cases", type=int, default=100)
    ap.add_argument("--holdout-cases", type=int, default=50)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--plan-cache", default=None,
                    help="text file of measured plan choices: loaded if present, written at the end")
    args = ap.parse_args()
    if args.steps < 1:
        args.steps = 1
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
