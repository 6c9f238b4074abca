#!/usr/bin/env python
"""Benchmark of the tensor-transpose hot path (cuttPlanMeasure -> cuttExecute).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads (all data synthetic, seeded):
  c2   (default) one step = the 14142 x 14142 matrix transpose in fp32 and then in fp64
       (two launches).  With N > 1 every rank transposes its own pair: independent
       objects, no collective, weak scaling.
  c4   rank-6 fp32 tensor with tiny leading dimensions.
  c3   the 100-case random rank 2-7 suite (fp64 and fp32); value = median over cases.
  c5a  rank-4 fp32 (1024,1024,32,256), permutation (1,0,2,3), sharded on the last dimension over
       the N ranks: slab mode, no communication (strong scaling: the 34 GB tensor is fixed).
  c5b  same tensor, permutation (3,2,0,1): the sharded dimension moves, every rank stores its
       tiles into the peers' output slabs from inside the kernel (NVLink all-to-all).

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
C2_WORKLOAD = "c2: rank-2 transpose (14142,14142) perm (1,0), fp32 then fp64 per step"


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            with open(p) as f:
                return float(json.load(f)["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def _workload_cases(name):
    from cutt_b200 import workloads as W
    if name == "c2":
        return [("c2_f32", W.C2[0], W.C2[1], 4), ("c2_f64", W.C2[0], W.C2[1], 8)]
    if name == "c4":
        return [("c4_f32", W.C4[0], W.C4[1], 4)]
    if name == "c1":
        return [("c1_f64", W.C1[0], W.C1[1], 8)]
    raise ValueError(name)


def _vol(dims):
    v = 1
    for d in dims:
        v *= int(d)
    return v


# ----------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the path (the original library has no CPU code and
# no sm_100 build), all host threads, on bounded samples of the same workload.
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import numpy as np
    import oracle
    cases = _workload_cases(args.workload if args.workload != "c3" else "c2")
    cores = oracle.num_threads()
    bufs = []
    for name, dims, perm, elt in cases:
        vol = _vol(dims)
        rng = np.random.default_rng(2 if elt == 4 else 3)
        a = rng.random(vol, dtype=np.float32 if elt == 4 else np.float64)
        bufs.append((dims, perm, elt, a))
    nbytes = sum(2 * _vol(d) * e for d, _, e, _ in bufs)

    def step():
        for dims, perm, elt, a in bufs:
            oracle.transpose_blocked(dims, perm, a)

    for _ in range(min(args.warmup, 1)):
        step()
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    val = nbytes / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "b32+b64 (bit moves)", "data": "synthetic",
        "config": {"workload": C2_WORKLOAD if args.workload == "c2" else args.workload,
                   "cases": [[n, d, p, e] for n, d, p, e in cases]},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": "%d full steps of the workload (blocked OpenMP loop nest)" % steps},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the original cuTT has no CPU implementation and no sm_100 build; this arm times "
                "the CPU restatement of its permutation (oracle/host_transpose.c) on the host cores",
    }
    print(json.dumps(line))
    return 0


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


def run_ours(args):
    import numpy as np
    import torch
    import cutt_b200 as C
    from cutt_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the transpose path has no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    C.lib()
    if args.plan_cache and os.path.exists(args.plan_cache):
        C.plan_cache_load(args.plan_cache)
    peak, peak_kind = _peaks()
    stream = torch.cuda.current_stream().cuda_stream

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    launches0 = C.launch_count()
    extras = {}

    if args.workload == "c3":
        res = run_suite(C, W.c3_cases(args.suite_cases), stream, reps=max(3, args.steps))
        med = statistics.median(r["gbs"] for r in res)
        t_ms = statistics.median(r["ms"] for r in res)
        val = max_over_ranks(med) if world == 1 else med * world
        line = base_line(args, val, t_ms, world)
        line["config"] = {"workload": "c3: %d seeded random rank 2-7 tensors of ~2e8 elements, fp64 and fp32; median over cases" % len(res),
                          "l2": "inputs larger than L2"}
        line["roofline"] = {"bound": "hbm", "achieved": med, "peak": peak, "unit": UNIT, "frac": med / peak,
                            "traffic": None, "peak_kind": peak_kind}
        line["suite"] = {"median_gbs": med, "min_gbs": min(r["gbs"] for r in res), "max_gbs": max(r["gbs"] for r in res),
                         "cases": res if args.verbose else len(res)}
        line["gpu_launches"] = C.launch_count() - launches0
        if rank == 0:
            print(json.dumps(line))
        return 0

    if args.workload in ("c5a", "c5b"):
        return run_sharded(args, C, W, dist, world, rank, local, peak, peak_kind, barrier, max_over_ranks)

    cases = _workload_cases(args.workload)
    # device-resident inputs (seeded uniform values), one pair of buffers per case
    plans = []
    for ci, (name, dims, perm, elt) in enumerate(cases):
        vol = _vol(dims)
        g = torch.Generator(device="cuda")
        g.manual_seed(2 + ci + 100 * rank)
        tin = torch.rand(vol, dtype=torch.float32 if elt == 4 else torch.float64, device="cuda", generator=g)
        tout = torch.empty_like(tin)
        rc, h = C.cuttPlanMeasure(len(dims), dims, perm, elt, stream, tin.data_ptr(), tout.data_ptr())
        if rc != 0:
            raise SystemExit("cuttPlanMeasure failed: %d" % rc)
        plans.append((name, dims, perm, elt, vol, tin, tout, h))
    step_bytes = sum(2 * vol * elt for _, _, _, elt, vol, _, _, _ in plans)

    def step():
        for _, _, _, _, _, tin, tout, h in plans:
            rc = C.cuttExecute(h, tin.data_ptr(), tout.data_ptr())
            if rc != 0:
                raise SystemExit("cuttExecute failed: %d" % rc)

    for _ in range(max(3, args.warmup)):
        step()
    sampler = ClockSampler(_physical_gpu_index(local))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    step()   # the GPU idled while the clock sampler started: one more untimed step before the timed ones
    launches_t0 = C.launch_count()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(plans) + 1)] for _ in range(args.steps)]
    for k in range(args.steps):
        ev[k][0].record()
        for i, (_, _, _, _, _, tin, tout, h) in enumerate(plans):
            rc = C.cuttExecute(h, tin.data_ptr(), tout.data_ptr())
            ev[k][i + 1].record()
    barrier()
    launches_timed = C.launch_count() - launches_t0
    total_ms = ev[0][0].elapsed_time(ev[-1][-1])
    total_ms = max_over_ranks(total_ms)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = total_ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # dominant kernel: the launch moving the most bytes
    dom = max(range(len(plans)), key=lambda i: plans[i][4] * plans[i][3])
    dom_ms = statistics.mean(ev[k][dom].elapsed_time(ev[k][dom + 1]) for k in range(args.steps))
    dom_bytes = 2 * plans[dom][4] * plans[dom][3]
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    per_case = {}
    for i, p in enumerate(plans):
        ms = statistics.mean(ev[k][i].elapsed_time(ev[k][i + 1]) for k in range(args.steps))
        per_case[p[0]] = {"ms": ms, "gbs": 2 * p[4] * p[3] / (ms * 1e-3) / 1e9, "plan": json.loads(C.plan_describe(p[7]))["label"]}

    # same-GPU device-to-device copies of the dominant case's bytes, for context: the driver's
    # copy (torch copy_ = cudaMemcpyAsync D2D) and this library's own copy kernel (the plan an
    # identity permutation gets), which also puts a plain copy into the profiler's launch list
    torch.cuda.synchronize()
    src = plans[dom][5]
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
        return dom_bytes / (a0.elapsed_time(a1) / n * 1e-3) / 1e9

    d2d = timed(lambda: dst.copy_(src))
    own_copy = None
    n_el = plans[dom][4]
    rc, hc = C.plan_params([n_el // 2, 2], [0, 1], plans[dom][3], stream, method=0)
    if rc == 0:
        own_copy = timed(lambda: C.cuttExecute(hc, src.data_ptr(), dst.data_ptr()))
        C.cuttDestroy(hc)
    del dst

    # end to end: host buffers in, host buffers out, through the C ABI
    e2e_steps = 0 if args.no_e2e else max(1, min(args.steps, 3))
    e2e = None
    if e2e_steps:
        hbufs = []
        for (name, dims, perm, elt, vol, tin, tout, h) in plans:
            hin = torch.empty(vol, dtype=tin.dtype, pin_memory=True)
            hin.copy_(tin)
            hout = torch.empty(vol, dtype=tin.dtype, pin_memory=True)
            hbufs.append((dims, perm, elt, hin, hout))
        torch.cuda.synchronize()

        def e2e_step():
            for dims, perm, elt, hin, hout in hbufs:
                rc = C.transpose_host(dims, perm, elt, hin.data_ptr(), hout.data_ptr())
                if rc != 0:
                    raise SystemExit("cutt_c_transpose_host failed: %d" % rc)

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_s = max_over_ranks((time.perf_counter() - t0) / e2e_steps)
        # the host round trip must reproduce the device result
        for (dims, perm, elt, hin, hout), p in zip(hbufs, plans):
            if not torch.equal(hout, p[6].cpu()):
                raise SystemExit("end-to-end result differs from the device-resident result")
        e2e = {"value": world * step_bytes / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": step_bytes // 2,
               "d2h_bytes_per_step": step_bytes // 2, "steps": e2e_steps}
        del hbufs

    line = base_line(args, value, ms_per_step, world)
    line["config"] = {"workload": C2_WORKLOAD if args.workload == "c2" else args.workload,
                      "cases": [[p[0], p[1], p[2], p[3]] for p in plans],
                      "l2": "inputs larger than L2 (0.8 GB and 1.6 GB per side)", "per_case": per_case,
                      "d2d_copy_gbs": d2d, "own_copy_kernel_gbs": own_copy}
    line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT,
                        "frac": achieved / peak, "traffic": _traffic_note(plans[dom][0]),
                        "kernel": "permute_tiles_kernel (%s)" % plans[dom][0], "peak_kind": peak_kind,
                        "frac_of_same_run_d2d_copy": achieved / d2d}
    line["e2e"] = e2e
    line["gpu_launches"] = launches_timed
    line["clocks"] = clocks

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(cases)
    if rank == 0 and not args.no_extras and world == 1:
        try:
            # the cost model alone first (cuttPlan would otherwise find the measured winners in the plan cache)
            C.clear_plan_cache()
            res0 = run_suite(C, W.c3_cases(args.suite_cases), stream, reps=5, measure=False)
            med0 = statistics.median(r["gbs"] for r in res0)
            extras["c3_suite_cuttPlan"] = {"cases": len(res0), "median_gbs": med0, "frac_of_peak": med0 / peak,
                                           "min_gbs": min(r["gbs"] for r in res0)}
        except Exception as e:
            extras["c3_suite_cuttPlan"] = {"error": repr(e)}
        try:
            res = run_suite(C, W.c3_cases(args.suite_cases), stream, reps=5)
            med = statistics.median(r["gbs"] for r in res)
            extras["c3_suite"] = {"cases": len(res), "median_gbs": med, "frac_of_peak": med / peak,
                                  "frac_of_8000": med / 8000.0,
                                  "min_gbs": min(r["gbs"] for r in res), "max_gbs": max(r["gbs"] for r in res),
                                  "_per_case": [r["gbs"] for r in res]}
        except Exception as e:  # extras never fail the headline
            extras["c3_suite"] = {"error": repr(e)}
    if rank == 0 and not args.no_extras and world == 1:
        # the 0.8 MB README tensor (configs[0]): launch/latency-bound, reported beside the suites
        try:
            d1, p1 = W.C1
            res1 = run_suite(C, [(d1, p1)], stream, reps=20)
            extras["c1_readme_example"] = {"dims": d1, "perm": p1,
                                           "fp64_us": res1[0]["ms"] * 1e3, "fp64_gbs": res1[0]["gbs"],
                                           "fp32_us": res1[1]["ms"] * 1e3, "fp32_gbs": res1[1]["gbs"],
                                           "plan_fp64": res1[0]["plan"]}
            ref1 = reference_gpu_baseline([("c1", d1, p1, 8), ("c1", d1, p1, 4)],
                                          modes=(("cuttPlanMeasure", ["--measure"]),), reps=20)
            extras["c1_readme_example"]["reference_cutt_gpu_gbs"] = ref1.get("cuttPlanMeasure", {}).get("per_case_gbs")
        except Exception as e:
            extras["c1_readme_example"] = {"error": repr(e)}
        extras["reference_cutt_gpu"] = reference_gpu_baseline(cases)
        if "c3_suite" in extras and "error" not in extras["c3_suite"]:
            suite_cases = [("c3", d, p, e) for d, p in W.c3_cases(args.suite_cases) for e in (8, 4)]
            ref = reference_gpu_baseline(suite_cases, modes=(("cuttPlanMeasure", ["--measure"]),), reps=3)
            r = ref.get("cuttPlanMeasure", {})
            if "per_case_gbs" in r:
                ours = extras["c3_suite"].pop("_per_case")
                ratios = sorted(o / max(x, 1e-9) for o, x in zip(ours, r["per_case_gbs"]))
                behind = sorted(((o / max(x, 1e-9), i) for i, (o, x) in enumerate(zip(ours, r["per_case_gbs"]))))[:10]
                behind = [{"case": i // 2, "elt": 8 if i % 2 == 0 else 4, "ours_gbs": round(ours[i], 1),
                           "reference_gbs": r["per_case_gbs"][i]} for q, i in behind if q < 1.0]
                extras["reference_cutt_gpu"]["c3_suite_cuttPlanMeasure"] = {
                    "median_gbs": statistics.median(r["per_case_gbs"]), "min_gbs": min(r["per_case_gbs"]),
                    "max_gbs": max(r["per_case_gbs"]),
                    "ours_over_reference": {"median": statistics.median(ratios), "min": ratios[0], "max": ratios[-1],
                                            "cases_where_reference_is_faster": sum(1 for x in ratios if x < 1.0),
                                            "slowest_relative_cases": behind}}
            else:
                extras["reference_cutt_gpu"]["c3_suite_cuttPlanMeasure"] = r
        if "c3_suite" in extras:
            extras["c3_suite"].pop("_per_case", None)
    if extras:
        line["extras"] = extras
    for p in plans:
        C.cuttDestroy(p[7])
    if args.plan_cache and rank == 0:
        C.plan_cache_save(args.plan_cache)
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


def run_sharded(args, C, W, dist, world, rank, local, peak, peak_kind, barrier, max_over_ranks):
    """C5: the 2^33-element fp32 tensor sharded over the ranks (strong scaling)."""
    import torch
    from cutt_b200.multigpu import ShardedTranspose
    dims = list(W.C5_DIMS)
    if args.c5_scale > 1:           # smaller stand-in for quick checks: shrink dim 2
        dims[2] = max(1, dims[2] // args.c5_scale)
    perm = W.C5A_PERM if args.workload == "c5a" else W.C5B_PERM
    elt = 4
    vol = _vol(dims)
    loc = vol // world
    g = torch.Generator(device="cuda")
    g.manual_seed(5 + rank)
    inp = torch.rand(loc, dtype=torch.float32, device="cuda", generator=g)
    st = ShardedTranspose(dims, perm, elt, measure_input=inp)
    launches0 = C.launch_count()
    for _ in range(max(3, args.warmup)):
        st.execute(inp)
    st.finish()
    sampler = ClockSampler(_physical_gpu_index(local))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    st.execute(inp)   # untimed: the GPU idled while the clock sampler started
    l0 = C.launch_count()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        st.execute(inp)
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    launches = C.launch_count() - l0
    clocks = sampler.stop() if rank == 0 else None
    total_bytes = 2 * vol * elt
    value = total_bytes / (ms * 1e-3) / 1e9
    per_gpu = value / world
    line = base_line(args, value, ms, world)
    line["scaling"] = "strong"
    line["dtype"] = "b32 (bit moves)"
    line["config"] = {"workload": "%s: rank-4 fp32 %s perm %s sharded on the last dim over %d GPU(s), mode %s"
                      % (args.workload, dims, perm, world, "slab" if st.mode == 0 else "all-to-all by peer stores"),
                      "l2": "inputs larger than L2 (%.1f GB per side per GPU)" % (loc * elt / 1e9),
                      "per_gpu_gbs": per_gpu, "plan": json.loads(C.plan_describe(st.handle))["label"]}
    line["roofline"] = {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": UNIT, "frac": per_gpu / peak,
                        "traffic": None, "kernel": "permute_tiles_kernel (per GPU)", "peak_kind": peak_kind}
    if st.mode == 1 and world > 1:
        remote = (world - 1) / world * loc * elt          # bytes each GPU sends over NVLink per step
        nv = remote / (ms * 1e-3) / 1e9
        line["nvlink"] = {"remote_gbs_per_gpu_per_direction": nv, "frac_of_770_measured": nv / 770.0,
                          "frac_of_900_nominal": nv / 900.0}
    line["gpu_launches"] = launches
    line["clocks"] = clocks
    line["e2e"] = None
    st.close()
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


def _traffic_note(case_name):
    """DRAM bytes per launch of the dominant kernel from the committed ncu capture, if any."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(p) as f:
            return json.load(f).get(case_name)
    except Exception:
        return None


def base_line(args, value, ms_per_step, world):
    return {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "b32+b64 (bit moves)", "data": "synthetic"}


def run_suite(C, cases, stream, reps=5, measure=True):
    """cuttPlanMeasure (or cuttPlan: the cost model's first pick) + timed cuttExecute for every
    case, fp64 then fp32."""
    import torch
    out = []
    maxvol = max(_vol(d) for d, _ in cases)
    buf_in = torch.rand(maxvol, dtype=torch.float64, device="cuda")
    buf_out = torch.empty_like(buf_in)
    for ci, (dims, perm) in enumerate(cases):
        vol = _vol(dims)
        for elt in (8, 4):
            if measure:
                rc, h = C.cuttPlanMeasure(len(dims), dims, perm, elt, stream, buf_in.data_ptr(), buf_out.data_ptr())
            else:
                rc, h = C.cuttPlan(len(dims), dims, perm, elt, stream)
            if rc != 0:
                raise RuntimeError("plan failed %s %s" % (dims, perm))
            C.cuttExecute(h, buf_in.data_ptr(), buf_out.data_ptr())
            ts = []
            for _ in range(reps):
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
                C.cuttExecute(h, buf_in.data_ptr(), buf_out.data_ptr())
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            ms = statistics.median(ts)
            label = json.loads(C.plan_describe(h))["label"]
            C.cuttDestroy(h)
            out.append({"case": ci, "dims": dims, "perm": perm, "elt": elt, "ms": ms,
                        "gbs": 2 * vol * elt / (ms * 1e-3) / 1e9, "plan": label})
    return out


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


def cpu_baseline(cases):
    import numpy as np
    import oracle
    bufs = []
    for name, dims, perm, elt in cases:
        a = np.random.default_rng(5).random(_vol(dims), dtype=np.float32 if elt == 4 else np.float64)
        bufs.append((dims, perm, a))
    nbytes = sum(2 * a.size * a.dtype.itemsize for _, _, a in bufs)
    for dims, perm, a in bufs:  # warm (page faults of the output allocator)
        oracle.transpose_blocked(dims, perm, a)
    n = 0
    t0 = time.perf_counter()
    while True:
        for dims, perm, a in bufs:
            oracle.transpose_blocked(dims, perm, a)
        n += 1
        if time.perf_counter() - t0 > 10.0 or n >= 8:
            break
    dt = (time.perf_counter() - t0) / n
    return {"value": nbytes / dt / 1e9, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
            "sample": "%d full steps of the same workload, blocked OpenMP loop nest (oracle/host_transpose.c)" % n}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5a", "c5b"])
    ap.add_argument("--c5-scale", type=int, default=1, help="divide dim 2 of the C5 tensor (quick checks)")
    ap.add_argument("--suite-cases", type=int, default=100)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--plan-cache", default=None,
                    help="text file of measured plan choices: loaded if present, written at the end")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
