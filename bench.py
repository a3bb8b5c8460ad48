#!/usr/bin/env python
"""MSDA forward+backward benchmark on B200: samples/s and HBM roofline fraction.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--dtype D]
    python bench.py --impl reference ...        # the CPU implementation of the path

One "step" = one forward + one backward of multi-scale deformable attention
over one batch of synthetic inputs with the shapes of BEVFormer-base spatial
cross-attention (6 camera views x 2500 queries, 8 heads x 32 channels, 4 levels
x 8 points, 30825 keys); a "sample" is one batch entry (one camera view).
Prints ONE JSON line:

  value        samples/s over all ranks, operands resident in HBM, calls through the C ABI
  e2e          the same through the public Python API with HOST (pinned) operands:
               host->device copies of the inputs and device->host copies of all four
               results are inside the timed region
  roofline     the backward kernel (the dominant one): algorithmic bytes per launch /
               CUDA-event time of that kernel alone, against the measured copy bandwidth
  cpu_baseline the CPU restatement of the reference's path timed on the host cores

With N > 1 (under torchrun, one rank per GPU) the batch is sharded: every rank
holds its own 6 samples; there is no data-path collective, so scaling is weak.
`--shard query` instead splits ONE batch's queries over the ranks and all-reduces
grad_value with NCCL (strong scaling; reported with "scaling": "strong").
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "msda_fwd_bwd_samples_per_s"
UNIT = "samples/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=10,
                    help="how many times the timed region of exactly --steps steps is run; "
                         "ms_per_step is the median over these runs")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--op", default="msda", choices=["msda", "fused", "gka", "da", "dcn", "addrelu", "maxpool"],
                    help="msda (the headline path, default); fused: MSDA with its callers' softmax and "
                         "location arithmetic inside; gka / da: the sibling operators geometric "
                         "kernel attention / deformable aggregation; dcn / addrelu / maxpool: modulated "
                         "deformable convolution, add+ReLU, stem max pooling (the operators "
                         "behind the other default patches); all of these on one GPU")
    ap.add_argument("--tensor-cores", type=int, default=1, choices=[0, 1, 2],
                    help="--op dcn: 1 = tcgen05 3xTF32 products (default), 2 = tcgen05 single "
                         "TF32 product, 0 = fp32 FMA kernel")
    ap.add_argument("--workload", default="bevformer_sca")
    ap.add_argument("--dtype", default="float32", choices=["float32", "float16", "bfloat16"])
    ap.add_argument("--batch", type=int, default=None,
                    help="override the workload's batch size (smaller cases for profiler captures)")
    ap.add_argument("--shard", default="batch", choices=["batch", "query"])
    ap.add_argument("--stage", type=int, default=None, help="tuning: bulk-copy staging 0 off / 1 both directions / 2 backward only (default)")
    ap.add_argument("--ctas-per-sm", type=int, default=None, help="tuning: forward kernel")
    ap.add_argument("--ctas-per-sm-bwd", type=int, default=None, help="tuning: backward kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-strong", action="store_true",
                    help="N > 1: skip the planned splits of one batch (strong scaling, stress shapes)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0,
                    help="budget of the CPU baseline sample")
    return ap.parse_args()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None,
                "sm_max_mhz": max(mx) if mx else None,
                "samples": len(mhz), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU baseline
def cpu_baseline(workload, seconds):
    """Times the CPU restatements of the reference's path on a bounded sample: whole batch
    entries of the same workload, repeated until about `seconds` have passed. Two
    implementations are timed — the PyTorch port of the reference's golden
    (grid_sample + autograd, float32, all torch threads) and the threaded C oracle
    (float64) — and the faster one is reported."""
    import torch
    from drivingsdk_b200 import workloads
    from oracle import golden_torch, msda_oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    msda_oracle.set_threads(cores)
    sample_b = min(workload.B, 2)
    w = workload.with_batch(sample_b)
    inp = workloads.make_inputs(w)
    n = lambda k: inp[k].numpy()

    def run_torch():
        golden_torch.msda_forward_backward(inp["value"], inp["shapes"], inp["loc"], inp["attn"],
                                           inp["grad_out"])

    def run_c():
        msda_oracle.forward(n("value"), n("shapes"), n("starts"), n("loc"), n("attn"))
        msda_oracle.backward(n("value"), n("shapes"), n("starts"), n("loc"), n("attn"),
                             n("grad_out"))

    results = {}
    for name, fn in (("torch_port_f32", run_torch), ("c_oracle_f64", run_c)):
        fn()  # warm-up
        t0 = time.perf_counter()
        reps = 0
        while True:
            fn()
            reps += 1
            if time.perf_counter() - t0 > seconds / 2 or reps >= 50:
                break
        dt = time.perf_counter() - t0
        results[name] = sample_b * reps / dt
    best = max(results, key=results.get)
    return {"value": results[best], "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{sample_b} of {workload.B} batch entries of {workload.name}, fwd+bwd, "
                      f"fastest of {{{', '.join(f'{k}: {v:.2f}' for k, v in results.items())}}} "
                      f"({best})"}


def workload_config(w, w_local, query_shard):
    """The `config` object of the JSON line; identical for both arms."""
    return {"workload": w.name, "B_per_rank": w_local.B, "Q_per_rank": w_local.Q,
            "H": w.H, "D": w.D, "K": w.K, "L": w.L, "P": w.P,
            "sharding": ("query+allreduce" if query_shard else "batch"),
            "l2": "2 rotating input sets; one step moves more operand bytes than the 126 MB L2"}


def run_reference_arm(args):
    """--impl reference: the reference's CPU implementation of the path on the host cores.
    Its device kernels need the vendor's NPU toolchain and cannot run here, and its CPU
    golden is Python test code that does not travel with this tree, so the timed code is
    the committed restatement of that golden (oracle/golden_torch.py, oracle/msda_oracle.c)."""
    from drivingsdk_b200 import workloads
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = workloads.WORKLOADS[args.workload]
    if args.batch:
        w = w.with_batch(args.batch)
    seconds = max(4.0, min(60.0, 2.0 * (args.steps + args.warmup)))
    base = cpu_baseline(w, seconds)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * w.B / base["value"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, w, args.shard == "query" and args.gpus > 1),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- native arm
def run_native(args):
    import torch
    import torch.distributed as dist

    from drivingsdk_b200 import capi, workloads
    import drivingsdk_b200 as sdk

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the native arm has no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py: --gpus N > 1 must be launched with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    lib = capi.load()
    for knob, val in ((capi.TUNE_STAGE, args.stage), (capi.TUNE_CTAS_PER_SM, args.ctas_per_sm),
                      (capi.TUNE_CTAS_PER_SM_BWD, args.ctas_per_sm_bwd)):
        if val is not None:
            lib.msda_sm100_tune(knob, val)
    dtype = getattr(torch, args.dtype)
    code = capi.dtype_code(dtype)
    esize = 4 if dtype == torch.float32 else 2
    w = workloads.WORKLOADS[args.workload]
    if args.batch:
        w = w.with_batch(args.batch)
    query_shard = args.shard == "query" and world > 1
    if query_shard:
        from drivingsdk_b200 import dist as sdist
        q0, q1 = sdist.query_range(w.Q, world, rank)
        w_local = w.with_queries(q1 - q0)
    else:
        w_local = w

    # two rotating input sets; one step already touches far more than the 126 MB L2
    NSETS = 2
    sets, host_sets = [], []
    shapes_i32 = starts_i32 = None
    for i in range(NSETS):
        inp = workloads.make_inputs(w_local, dtype, seed_offset=1000 * rank + i)
        host = {k: inp[k].to(dtype).pin_memory() for k in ("value", "loc", "attn", "grad_out")}
        host_sets.append(host)
        sets.append({k: v.to(dev) for k, v in host.items()})
        if shapes_i32 is None:
            shapes_i32 = inp["shapes"].to(torch.int32).to(dev)
            starts_i32 = inp["starts"].to(torch.int32).to(dev)
    B, K, H, D, L, Q, P = w_local.B, w_local.K, w_local.H, w_local.D, w_local.L, w_local.Q, w_local.P
    dims = (B, K, H, D, L, Q, P)
    out = torch.empty(B, Q, H * D, device=dev, dtype=dtype)
    gv = torch.empty(B, K, H, D, device=dev, dtype=dtype)
    gl = torch.empty(B, Q, H, L, P, 2, device=dev, dtype=dtype)
    ga = torch.empty(B, Q, H, L, P, device=dev, dtype=dtype)
    ws_bytes = lib.msda_sm100_backward_workspace_bytes(B, K, H, D, code)
    ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
    stream = torch.cuda.current_stream()

    def step_c_abi(s):
        capi.check(lib.msda_sm100_forward(
            s["value"].data_ptr(), shapes_i32.data_ptr(), starts_i32.data_ptr(),
            s["loc"].data_ptr(), s["attn"].data_ptr(), out.data_ptr(), *dims, code,
            stream.cuda_stream), "forward")
        capi.check(lib.msda_sm100_backward_ws(
            s["value"].data_ptr(), shapes_i32.data_ptr(), starts_i32.data_ptr(),
            s["loc"].data_ptr(), s["attn"].data_ptr(), s["grad_out"].data_ptr(), gv.data_ptr(),
            gl.data_ptr(), ga.data_ptr(), ws.data_ptr(), ws_bytes, *dims, code,
            stream.cuda_stream), "backward")
        if query_shard:
            dist.all_reduce(gv)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- device-resident timing (the `value`) -------------------------
    for i in range(args.warmup):
        step_c_abi(sets[i % NSETS])
    barrier()
    K_steps = args.steps
    # The timed region is short (K steps of ~0.5 ms), so the clock sampler would mostly see an
    # idle GPU. Untimed steps of the same work run for ~0.4 s before and ~0.2 s after the timed
    # region while the sampler is on, so that its samples are taken under this load.
    def busy(seconds):
        t_end = time.perf_counter() + seconds
        i = 0
        while time.perf_counter() < t_end:
            step_c_abi(sets[i % NSETS])
            i += 1
            if i % 16 == 0:
                torch.cuda.synchronize()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    busy(0.4)
    # The timed region is exactly K steps between two barriers; it is run `repeats` times and
    # the median region is what the line reports (one region is only ~10 ms at K = 20).
    R = max(1, args.repeats)
    kev = [[[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(K_steps)]
           for _ in range(R)]
    for rep in kev:
        for quad in rep:
            for e in quad:
                e.record(stream)  # materialise the underlying cudaEvent_t
    region = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(R)]
    launches0 = lib.msda_sm100_launch_count()
    for r in range(R):
        barrier()
        region[r][0].record(stream)
        for i in range(K_steps):
            lib.msda_sm100_profile_events(*[e.cuda_event for e in kev[r][i]])
            step_c_abi(sets[i % NSETS])
        region[r][1].record(stream)
        lib.msda_sm100_profile_events(None, None, None, None)
        barrier()
    launches = (lib.msda_sm100_launch_count() - launches0) // R
    busy(0.2)
    clocks = sampler.stop() if rank == 0 else None
    region_ms = [a.elapsed_time(b) for a, b in region]
    fwd_all = sorted(q[0].elapsed_time(q[1]) for rep in kev for q in rep)
    bwd_all = sorted(q[2].elapsed_time(q[3]) for rep in kev for q in rep)
    fwd_ms = fwd_all[len(fwd_all) // 2]
    bwd_ms = bwd_all[len(bwd_all) // 2]

    t = torch.tensor(region_ms, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)     # per region, the slowest rank
    per_step = sorted(float(x) / K_steps for x in t.tolist())
    ms_per_step = per_step[len(per_step) // 2]
    timing = {"repeats": R, "ms_per_step_median": ms_per_step,
              "ms_per_step_p10": per_step[max(0, int(0.1 * (R - 1)))],
              "ms_per_step_min": per_step[0], "ms_per_step_max": per_step[-1]}
    global_samples = w.B if query_shard else w.B * world
    value = global_samples / (ms_per_step * 1e-3)

    # ---------------- one batch spread over the ranks, and the large-head-dim shapes -------
    extra = {}
    if world > 1 and not query_shard and not args.no_strong:
        extra = run_planned_splits(lib, dist, dev, rank, world, w, dtype, ms_per_step, barrier)

    # ---------------- end-to-end through the Python API with host operands ----------
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(sdk, host_sets, shapes_i32, starts_i32, dev, dtype, world, query_shard,
                      max(4, min(K_steps, 20)), global_samples, barrier)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = load_peaks()
    fb, bb = workloads.compulsory_bytes(w_local, esize)
    bwd_gbs = bb / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = fb / (fwd_ms * 1e-3) / 1e9
    step_gbs = (fb + bb) / (ms_per_step * 1e-3) / 1e9
    bwd_kernel = backward_kernel_name(lib, capi, w.D, esize)
    # what actually bounds the two kernels: rows moved between L2 and the SMs, against the
    # rates the library's probe measures on this device in this run
    rows = count_corner_rows(sets[0]["loc"], shapes_i32)
    ceil = measured_row_ceilings(lib, capi, dev, w_local.D, esize)
    fwd_rows_s = rows / (fwd_ms * 1e-3)
    bwd_rows_s = rows / (bwd_ms * 1e-3)
    row_roofline = {
        "rows_per_launch": rows, "measured": ceil,
        "forward": {"bound": "16-byte vector loads of gathered value rows (L2 -> SM)",
                    "achieved_rows_per_s": fwd_rows_s,
                    "frac": fwd_rows_s / ceil["gather_rows_per_s"]},
        "backward": {"bound": "vector reductions of grad_value rows in L2 (it also gathers "
                              "as many value rows)",
                     "achieved_rows_per_s": bwd_rows_s,
                     "frac": bwd_rows_s / ceil["red_rows_per_s"]},
    }
    roofline = {
        "bound": "hbm", "kernel": bwd_kernel, "achieved": bwd_gbs, "peak": peak,
        "unit": "GB/s", "frac": bwd_gbs / peak,
        "traffic": TRAFFIC_BYTES.get((bwd_kernel, w.name, args.dtype)),
        "peak_kind": peak_kind, "algorithmic_bytes": bb, "kernel_ms": bwd_ms,
        "forward": {"kernel": "msda_fwd_kernel", "achieved": fwd_gbs, "frac": fwd_gbs / peak,
                    "algorithmic_bytes": fb, "kernel_ms": fwd_ms},
        "step": {"achieved": step_gbs, "frac": step_gbs / peak, "algorithmic_bytes": fb + bb},
        "rows": row_roofline,
    }
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K_steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if query_shard else "weak", "vs_baseline": None,
        "dtype": {"float32": "f32", "float16": "f16", "bfloat16": "bf16"}[args.dtype],
        "data": "synthetic",
        "config": workload_config(w, w_local, query_shard),
        "roofline": roofline, "clocks": clocks, "gpu_launches": int(launches) * world,
        "timing": timing,
        "tuning": {"stage": lib.msda_sm100_tune(capi.TUNE_STAGE, -1),
                   "ctas_per_sm": lib.msda_sm100_tune(capi.TUNE_CTAS_PER_SM, -1),
                   "ctas_per_sm_bwd": lib.msda_sm100_tune(capi.TUNE_CTAS_PER_SM_BWD, -1)},
    }
    if e2e is not None:
        line["e2e"] = e2e
    line.update(extra)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(w, args.cpu_seconds)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (ncu: dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the dominant
# kernel, keyed by (kernel, workload, dtype). An entry applies only while the kernel of that
# name is the one launched, so a number captured for an older kernel is never reported for a
# newer one; combinations without a capture report null.
TRAFFIC_BYTES = {
    ("msda_bwd_kernel", "bevformer_sca", "float32"): 630_341_376,
}


def count_corner_rows(loc, shapes):
    """How many value rows one forward gathers (and one backward gathers and reduces): the
    bilinear corners that exist, over all samples (kernels/multi_scale_deformable_attn/
    op_kernel/msda.h:367-390 for which samples count; a corner outside the level is skipped).
    loc [B,Q,H,L,P,2] on the device, shapes [L,2] (H, W)."""
    import torch
    hw = shapes.to(loc.device).to(torch.float32)
    Hl = hw[:, 0].view(1, 1, 1, -1, 1)
    Wl = hw[:, 1].view(1, 1, 1, -1, 1)
    x = loc[..., 0].float() * Wl - 0.5
    y = loc[..., 1].float() * Hl - 0.5
    valid = (x > -1) & (y > -1) & (x < Wl) & (y < Hl)
    x0, y0 = torch.floor(x), torch.floor(y)
    cx = (x0 >= 0).int() + (x0 + 1 <= Wl - 1).int()
    cy = (y0 >= 0).int() + (y0 + 1 <= Hl - 1).int()
    return int((valid.int() * cx * cy).sum().item())


def measured_row_ceilings(lib, capi, dev, D, esize):
    """L2 <-> SM row rates measured on this device right now by the library's own probe:
    (gathers of value rows, reductions of fp32 accumulation rows) in rows per second."""
    import ctypes
    import torch
    pow2 = lambda b: max(64, min(512, 1 << (max(1, b) - 1).bit_length()))
    g_row, r_row = pow2(D * esize), pow2(D * 4)
    buf = torch.empty(32 << 20, device=dev, dtype=torch.uint8)
    g, r = ctypes.c_double(0), ctypes.c_double(0)
    capi.check(lib.msda_sm100_probe_row_rates(buf.data_ptr(), buf.numel(), g_row, r_row,
                                              ctypes.byref(g), ctypes.byref(r),
                                              torch.cuda.current_stream().cuda_stream), "probe")
    return {"gather_row_bytes": g_row, "gather_rows_per_s": g.value,
            "red_row_bytes": r_row, "red_rows_per_s": r.value}


def backward_kernel_name(lib, capi, D, dtype_size):
    """Name of the kernel msda_sm100_backward_ws launches (one template, msda_bwd_kernel)."""
    return "msda_bwd_kernel"


def run_planned_splits(lib, dist, dev, rank, world, w, dtype, replica_ms_per_step, barrier):
    """N > 1, after the replica timing: ONE batch spread over the ranks by the planner
    (drivingsdk_b200.dist.plan with a cost model built from one entry's time measured here), for
    the headline workload ("strong") and for the large-head-dim shape with 8 batch entries
    ("config5a", bf16) and with one entry whose queries are split over all ranks and whose
    grad_value is summed with NCCL ("config5b", bf16). Every rank draws only the entries it
    works on (seeded per entry). Timing: CUDA events, max over ranks; the reduction's own
    time is reported as allreduce_ms. A few steps each, so that the whole thing adds seconds."""
    import torch
    from drivingsdk_b200 import capi, workloads
    from drivingsdk_b200 import dist as sdist

    stream = torch.cuda.current_stream()

    def one(label, wl, dt, force_kind=None):
        esize = 4 if dt == torch.float32 else 2
        code = capi.dtype_code(dt)
        # per-entry cost for the planner: ONE batch entry of this workload, forward + backward,
        # timed here on every rank (median of 3 after a warm-up; the slowest rank counts)
        e1 = workloads.make_inputs(wl.with_batch(1), dt, seed_offset=49)
        dv = {k: e1[k].to(dt).to(dev).contiguous() for k in ("value", "loc", "attn", "grad_out")}
        sh1 = e1["shapes"].to(torch.int32).to(dev)
        st1 = e1["starts"].to(torch.int32).to(dev)
        d1 = (1, wl.K, wl.H, wl.D, wl.L, wl.Q, wl.P)
        o1 = torch.empty(1, wl.Q, wl.H * wl.D, device=dev, dtype=dt)
        g1 = [torch.empty_like(dv[k]) for k in ("value", "loc", "attn")]
        wsb = lib.msda_sm100_backward_workspace_bytes(1, wl.K, wl.H, wl.D, code)
        ws1 = torch.empty(max(wsb, 16), device=dev, dtype=torch.uint8)
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        single = []
        for it in range(4):
            ea.record(stream)
            capi.check(lib.msda_sm100_forward(
                dv["value"].data_ptr(), sh1.data_ptr(), st1.data_ptr(), dv["loc"].data_ptr(),
                dv["attn"].data_ptr(), o1.data_ptr(), *d1, code, stream.cuda_stream), "forward")
            capi.check(lib.msda_sm100_backward_ws(
                dv["value"].data_ptr(), sh1.data_ptr(), st1.data_ptr(), dv["loc"].data_ptr(),
                dv["attn"].data_ptr(), dv["grad_out"].data_ptr(), g1[0].data_ptr(),
                g1[1].data_ptr(), g1[2].data_ptr(), ws1.data_ptr(), wsb, *d1, code,
                stream.cuda_stream), "backward")
            eb.record(stream)
            eb.synchronize()
            if it > 0:
                single.append(ea.elapsed_time(eb))
        tt = torch.tensor([sorted(single)[1]], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        entry_s = float(tt.item()) * 1e-3
        del dv, o1, g1, ws1
        cost = sdist.CostModel(entry_s, float(wl.K * wl.H * wl.D * esize),
                               fixed_seconds=sdist.fixed_entry_seconds(wl.K, wl.H, wl.D, esize))
        plan = sdist.plan(wl.B, wl.Q, world, cost=cost)
        if force_kind == "hybrid" and plan.kind != "hybrid":
            plan = sdist.candidate_plans(wl.B, wl.Q, world)[1]
        groups = sdist.make_groups(plan)
        group = groups.get(plan.group_of(rank))
        b0, b1 = plan.ranges[rank]
        if plan.kind == "hybrid":
            q0, q1 = plan.query_ranges[rank]
        elif plan.kind == "query":
            (q0, q1), (b0, b1) = plan.ranges[rank], (0, wl.B)
        else:
            q0, q1 = 0, wl.Q
        nb, nq = max(0, b1 - b0), max(0, q1 - q0)
        times, red_times = [], []
        if nb > 0 and nq > 0:
            ents = [workloads.make_inputs(wl.with_batch(1), dt, seed_offset=50 + b)
                    for b in range(b0, b1)]
            cat = lambda k, qs: torch.cat([e[k][:, q0:q1] if qs else e[k] for e in ents]) \
                .to(dt).to(dev).contiguous()
            value, loc, attn, go = cat("value", False), cat("loc", True), cat("attn", True), \
                cat("grad_out", True)
            shapes = ents[0]["shapes"].to(torch.int32).to(dev)
            starts = ents[0]["starts"].to(torch.int32).to(dev)
            dims = (nb, wl.K, wl.H, wl.D, wl.L, nq, wl.P)
            out = torch.empty(nb, nq, wl.H * wl.D, device=dev, dtype=dt)
            gv, gl, ga = torch.empty_like(value), torch.empty_like(loc), torch.empty_like(attn)
            ws_bytes = lib.msda_sm100_backward_workspace_bytes(nb, wl.K, wl.H, wl.D, code)
            ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]

        def step(timed):
            if timed:
                e[0].record(stream)
            if nb > 0 and nq > 0:
                capi.check(lib.msda_sm100_forward(
                    value.data_ptr(), shapes.data_ptr(), starts.data_ptr(), loc.data_ptr(),
                    attn.data_ptr(), out.data_ptr(), *dims, code, stream.cuda_stream), "forward")
                capi.check(lib.msda_sm100_backward_ws(
                    value.data_ptr(), shapes.data_ptr(), starts.data_ptr(), loc.data_ptr(),
                    attn.data_ptr(), go.data_ptr(), gv.data_ptr(), gl.data_ptr(), ga.data_ptr(),
                    ws.data_ptr(), ws_bytes, *dims, code, stream.cuda_stream), "backward")
            if timed:
                e[1].record(stream)
            if plan.needs_allreduce and nb > 0:
                dist.all_reduce(gv, group=group)
            if timed:
                e[2].record(stream)

        for _ in range(3):
            step(False)
        STEPS = 8
        for _ in range(STEPS):
            barrier()
            step(True)
            barrier()
            times.append(e[0].elapsed_time(e[2]))
            red_times.append(e[1].elapsed_time(e[2]))
        t = torch.tensor([times, red_times], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms = sorted(t[0].tolist())[STEPS // 2]
        red_ms = sorted(t[1].tolist())[STEPS // 2]
        return {"workload": wl.name, "B": wl.B, "dtype": str(dt)[6:], "plan": plan.kind,
                "ranges": [list(r) for r in plan.ranges],
                "query_ranges": [list(r) for r in plan.query_ranges],
                "idle_ranks": sum(plan.is_idle(r) for r in range(world)),
                "ms_per_step": step_ms, "allreduce_ms": red_ms if plan.needs_allreduce else 0.0,
                "value": wl.B / (step_ms * 1e-3), "unit": UNIT, "scaling": "strong",
                "predicted_ms": None if plan.predicted_seconds is None
                else plan.predicted_seconds * 1e3,
                "one_entry_one_gpu_ms": entry_s * 1e3,
                "single_gpu_ms": entry_s * wl.B * 1e3,
                "efficiency_ceiling": plan.efficiency_ceiling()}

    stress = workloads.WORKLOADS["stress_d128"]
    out = {"strong": one("strong", w, dtype)}
    out["config5a"] = one("config5a", stress, torch.bfloat16)
    out["config5b"] = one("config5b", stress.with_batch(1), torch.bfloat16, force_kind="hybrid")
    return out


def run_e2e(sdk, host_sets, shapes_i32, starts_i32, dev, dtype, world, query_shard, steps,
            global_samples, barrier):
    """Public API, host operands. Every step copies value / locations / weights / grad_output
    from pinned host memory to the device, runs forward and backward through the autograd
    function, and copies output and all three gradients back to pinned host memory — all
    inside the timed region. The three stages run on three streams with three buffer slots, so
    the upload of step i+1 and the download of step i-1 overlap the kernels of step i (PCIe
    is full duplex); per step the same bytes move as without the overlap."""
    import torch
    import torch.distributed as dist
    h0 = host_sets[0]
    NSLOT = 3
    s_comp = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    d_in = [{k: torch.empty_like(v, device=dev) for k, v in h0.items()} for _ in range(NSLOT)]
    ev_in = [torch.cuda.Event() for _ in range(NSLOT)]
    ev_comp = [torch.cuda.Event() for _ in range(NSLOT)]
    ev_out = [torch.cuda.Event() for _ in range(NSLOT)]
    used = [False] * NSLOT
    keep = [None] * NSLOT       # device results of a slot: referenced until the host has seen
                                # their download finish, so the allocator cannot reuse them early
    h_out = [None] * NSLOT
    h2d = sum(v.numel() * v.element_size() for v in h0.values())

    def one_step(i, host):
        slot = i % NSLOT
        if used[slot]:
            ev_out[slot].synchronize()      # slot's previous results are on the host now
        with torch.cuda.stream(s_in):
            if used[slot]:
                s_in.wait_event(ev_comp[slot])      # its inputs are no longer being read
            for k in d_in[slot]:
                d_in[slot][k].copy_(host[k], non_blocking=True)
            ev_in[slot].record(s_in)
        s_comp.wait_event(ev_in[slot])
        value = d_in[slot]["value"].detach().requires_grad_(True)
        loc = d_in[slot]["loc"].detach().requires_grad_(True)
        attn = d_in[slot]["attn"].detach().requires_grad_(True)
        out = sdk.multi_scale_deformable_attn(value, shapes_i32, starts_i32, loc, attn)
        out.backward(d_in[slot]["grad_out"])
        gvalue = value.grad
        if query_shard:
            dist.all_reduce(gvalue)
        res = (out.detach(), gvalue, loc.grad, attn.grad)
        ev_comp[slot].record(s_comp)
        if h_out[slot] is None:
            h_out[slot] = [torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in res]
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[slot])
            for h, r in zip(h_out[slot], res):
                h.copy_(r, non_blocking=True)
            ev_out[slot].record(s_out)
        keep[slot] = res
        used[slot] = True

    def drain():
        for slot in range(NSLOT):
            if used[slot]:
                s_comp.wait_event(ev_out[slot])
                s_comp.wait_event(ev_in[slot])

    for i in range(4):
        one_step(i, host_sets[i % len(host_sets)])
    drain()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_comp)
    s_in.wait_event(e0)
    s_out.wait_event(e0)
    for i in range(steps):
        one_step(i, host_sets[i % len(host_sets)])
    drain()
    e1.record(s_comp)
    barrier()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    d2h = sum(h.numel() * h.element_size() for h in h_out[0])
    return {"value": global_samples / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms,
            "steps": steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "overlap": "3 streams, 3 slots: upload, kernels and download of neighbouring steps overlap"}


# --------------------------------------------------------------------------- sibling operators
def run_sibling(args):
    """One-GPU fwd+bwd timing of geometric kernel attention (--op gka) or deformable
    aggregation (--op da) through the C ABI, operands in HBM, with the same roofline
    accounting (every operand once, every result once) and a CPU-oracle baseline."""
    import numpy as np
    import torch
    from drivingsdk_b200 import capi
    from oracle import msda_oracle

    lib = capi.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(4321)
    stream = torch.cuda.current_stream()
    if args.op == "gka":
        # MapTR-style call of the reference's unit test (tests/torch/
        # test_geometric_kernel_attention.py:109): 24 views, 7156 queries, 4 heads x 64
        # channels, one 15x25 level, 15 points per query
        B, Q, H, D, L, P, hw = 24, 7156, 4, 64, 1, 15, (15, 25)
        K = hw[0] * hw[1] * L
        value = (torch.rand(B, K, H, D, generator=g) * 3).to(dev)
        loc = torch.empty(B, Q, H, L, P, 2)
        loc[..., 0] = torch.randint(-3, hw[1] + 3, (B, Q, H, L, P), generator=g).float()
        loc[..., 1] = torch.randint(-3, hw[0] + 3, (B, Q, H, L, P), generator=g).float()
        loc = loc.to(dev)
        attn = torch.rand(B, Q, H, L, P, generator=g).to(dev)
        go = (torch.rand(B, Q, H * D, generator=g) * 10).to(dev)
        shapes = torch.tensor([list(hw)] * L, dtype=torch.int32, device=dev)
        starts = torch.arange(L, dtype=torch.int32, device=dev) * (hw[0] * hw[1])
        out = torch.empty(B, Q, H * D, device=dev)
        gv, ga = torch.empty_like(value), torch.empty_like(attn)
        dims = (B, K, H, D, L, Q, P)
        samples = B
        nv, ns, no = value.numel(), attn.numel(), out.numel()
        fwd_bytes, bwd_bytes = 4 * (nv + 3 * ns + no), 4 * (2 * nv + 4 * ns + no)

        def fwd():
            capi.check(lib.gka_sm100_forward(value.data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                             loc.data_ptr(), attn.data_ptr(), out.data_ptr(), *dims,
                                             capi.F32, stream.cuda_stream), "gka fwd")

        def bwd():
            capi.check(lib.gka_sm100_backward_ws(
                value.data_ptr(), shapes.data_ptr(), starts.data_ptr(), loc.data_ptr(),
                attn.data_ptr(), go.data_ptr(), gv.data_ptr(), ga.data_ptr(), None, 0, *dims,
                capi.F32, stream.cuda_stream), "gka bwd")

        def cpu_once(nb):
            n = lambda t: t[:nb].cpu().numpy()
            msda_oracle.gka_forward(n(value), shapes.cpu().numpy(), starts.cpu().numpy(), n(loc), n(attn))
            msda_oracle.gka_backward(n(value), shapes.cpu().numpy(), starts.cpu().numpy(), n(loc),
                                     n(attn), n(go))
        config = {"workload": "gka_maptr_test_shape", "B": B, "Q": Q, "H": H, "D": D, "K": K,
                  "L": L, "P": P}
    elif args.op == "fused":
        # BEVFormer-base shape, fed by reference points, offsets (pixels) and logits
        from drivingsdk_b200 import workloads
        w = workloads.WORKLOADS["bevformer_sca"]
        B, Q, H, D, L, P, K = w.B, w.Q, w.H, w.D, w.L, w.P, w.K
        shapes64, starts64 = workloads.level_tensors(w.levels)
        shapes, starts = shapes64.int().to(dev), starts64.int().to(dev)
        value = torch.randn(B, K, H, D, generator=g).to(dev)
        ref = torch.rand(B, Q, L, 2, generator=g).to(dev)
        off = (torch.randn(B, Q, H, L, P, 2, generator=g) * 20).to(dev)
        logits = torch.randn(B, Q, H, L, P, generator=g).to(dev)
        go = torch.randn(B, Q, H * D, generator=g).to(dev)
        out = torch.empty(B, Q, H * D, device=dev)
        gv, goff, glog = torch.empty_like(value), torch.empty_like(off), torch.empty_like(logits)
        gref = torch.empty(B, Q, L, 2, device=dev)
        dims = (B, K, H, D, L, Q, P)
        samples = B
        nv, ns, no, nr = value.numel(), logits.numel(), out.numel(), ref.numel()
        fwd_bytes = 4 * (nv + 3 * ns + nr + no)
        bwd_bytes = 4 * (2 * nv + 6 * ns + 2 * nr + no)

        def fwd():
            capi.check(lib.msda_sm100_fused_forward(
                value.data_ptr(), shapes.data_ptr(), starts.data_ptr(), ref.data_ptr(),
                off.data_ptr(), logits.data_ptr(), out.data_ptr(), *dims, capi.F32,
                stream.cuda_stream), "fused fwd")

        def bwd():
            capi.check(lib.msda_sm100_fused_backward_ws(
                value.data_ptr(), shapes.data_ptr(), starts.data_ptr(), ref.data_ptr(),
                off.data_ptr(), logits.data_ptr(), go.data_ptr(), gv.data_ptr(), gref.data_ptr(),
                goff.data_ptr(), glog.data_ptr(), None, 0, *dims, capi.F32, stream.cuda_stream),
                "fused bwd")

        def cpu_once(nb):
            from drivingsdk_b200.ops.msda_fused import compose_unfused
            loc, attn = compose_unfused(ref[:nb].cpu(), off[:nb].cpu(), logits[:nb].cpu(), shapes64)
            n = lambda t: t[:nb].cpu().numpy()
            msda_oracle.forward(n(value), shapes64.numpy(), starts64.numpy(), loc.numpy(), attn.numpy())
            msda_oracle.backward(n(value), shapes64.numpy(), starts64.numpy(), loc.numpy(),
                                 attn.numpy(), n(go))
        config = {"workload": "bevformer_sca_fused", "B": B, "Q": Q, "H": H, "D": D, "K": K,
                  "L": L, "P": P}
    else:
        # Sparse4D-style call: 6 cameras x 4 scales (64x176 ... 8x22), 256 channels in 8 groups,
        # 900 anchors x 13 points, batch 6; locations uniform in (0, 1): every sample counts
        B, C, A, Pts, G = 6, 256, 900, 13, 8
        maps = [[(64, 176), (32, 88), (16, 44), (8, 22)]] * 6
        cams, scales = len(maps), len(maps[0])
        shapes_np = np.array(maps, dtype=np.int32).reshape(cams, scales, 2)
        sizes = (shapes_np[..., 0] * shapes_np[..., 1]).reshape(-1)
        starts_np = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int32).reshape(cams, scales)
        F = int(sizes.sum())
        feat = torch.randn(B, F, C, generator=g).to(dev)
        loc = torch.rand(B, A, Pts, cams, 2, generator=g).clamp_(1e-4, 1 - 1e-4).to(dev)
        wts = torch.rand(B, A, Pts, cams, scales, G, generator=g).to(dev)
        go = torch.randn(B, A, C, generator=g).to(dev)
        shapes = torch.from_numpy(shapes_np).to(dev)
        starts = torch.from_numpy(starts_np).to(dev)
        out = torch.empty(B, A, C, device=dev)
        gf, gl, gw = torch.empty_like(feat), torch.empty_like(loc), torch.empty_like(wts)
        dims = (B, F, C, A, Pts, cams, scales, G)
        samples = B
        nf, nl, nw, no = feat.numel(), loc.numel(), wts.numel(), out.numel()
        fwd_bytes, bwd_bytes = 4 * (nf + nl + nw + no), 4 * (2 * nf + 2 * nl + 2 * nw + no)

        def fwd():
            capi.check(lib.da_sm100_forward(feat.data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                            loc.data_ptr(), wts.data_ptr(), out.data_ptr(), *dims,
                                            stream.cuda_stream), "da fwd")

        def bwd():
            capi.check(lib.da_sm100_backward(feat.data_ptr(), shapes.data_ptr(), starts.data_ptr(),
                                             loc.data_ptr(), wts.data_ptr(), go.data_ptr(),
                                             gf.data_ptr(), gl.data_ptr(), gw.data_ptr(), *dims,
                                             stream.cuda_stream), "da bwd")

        def cpu_once(nb):
            n = lambda t: t[:nb].cpu().numpy()
            msda_oracle.da_forward(n(feat), shapes_np, starts_np, n(loc), n(wts))
            msda_oracle.da_backward(n(feat), shapes_np, starts_np, n(loc), n(wts), n(go))
        config = {"workload": "da_sparse4d_shape", "B": B, "C": C, "anchors": A, "pts": Pts,
                  "cams": cams, "scales": scales, "groups": G, "F": F}

    for _ in range(max(3, args.warmup)):
        fwd(); bwd()
    torch.cuda.synchronize()
    K_steps = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K_steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.msda_sm100_launch_count()
    e0.record(stream)
    for i in range(K_steps):
        ev[i][0].record(stream); fwd(); ev[i][1].record(stream); bwd(); ev[i][2].record(stream)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / K_steps
    fwd_ms = sum(q[0].elapsed_time(q[1]) for q in ev) / K_steps
    bwd_ms = sum(q[1].elapsed_time(q[2]) for q in ev) / K_steps
    peak, peak_kind = load_peaks()
    line = {
        "metric": f"{args.op}_fwd_bwd_samples_per_s", "value": samples / (ms * 1e-3), "unit": UNIT,
        "n_gpus": 1, "steps": K_steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config,
        "roofline": {"bound": "hbm", "kernel": f"{args.op} backward call (zero-fill + kernel)",
                     "achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak, "traffic": None,
                     "peak_kind": peak_kind, "algorithmic_bytes": bwd_bytes, "kernel_ms": bwd_ms,
                     "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                                 "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak,
                                 "algorithmic_bytes": fwd_bytes, "kernel_ms": fwd_ms},
                     "step": {"frac": (fwd_bytes + bwd_bytes) / (ms * 1e-3) / 1e9 / peak,
                              "algorithmic_bytes": fwd_bytes + bwd_bytes}},
        "gpu_launches": int(lib.msda_sm100_launch_count() - launches0),
    }
    if args.op == "gka":
        # row-rate roofline, as for the headline operator: every sample is exactly one row
        # (clamped pixel), gathered in the forward, gathered and reduced in the backward
        ceil = measured_row_ceilings(lib, capi, dev, D, 4)
        rows = B * Q * H * L * P
        line["roofline"]["rows"] = {
            "rows_per_launch": rows, "measured": ceil,
            "forward": {"achieved_rows_per_s": rows / (fwd_ms * 1e-3),
                        "frac": rows / (fwd_ms * 1e-3) / ceil["gather_rows_per_s"]},
            "backward": {"achieved_rows_per_s": rows / (bwd_ms * 1e-3),
                         "frac": rows / (bwd_ms * 1e-3) / ceil["red_rows_per_s"]}}
    if not args.no_cpu_baseline:
        msda_oracle.set_threads(os.cpu_count() or 1)
        t0 = time.perf_counter()
        cpu_once(1)
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 1.0 / dt, "unit": UNIT, "cores": 1, "kind": "port",
                                "sample": "1 batch entry, fwd+bwd, C oracle (float64, one thread)"}
    print(json.dumps(line))


def load_tensor_peak():
    """Dense TF32 TFLOP/s for the roofline of the tensor-core products: half the measured
    bf16 burst figure (TF32 issues at half the bf16 rate), else half the fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]) / 2, "measured bf16 / 2"
    except Exception:
        return 1590.0 / 2, "fallback bf16 / 2"


def run_conv_side(args):
    """One-GPU timing, through the C ABI with operands in HBM, of the operators behind the
    other default patches: modulated deformable convolution (--op dcn, forward + backward at
    the shape of the reference's unit test, tests/torch/test_deformable_conv2d.py:59), add+ReLU
    with its gradient (--op addrelu, tests/torch/test_add_relu.py:42) and the ResNet stem's
    max pooling (--op maxpool, tests/torch/test_npu_max_pool2d.py:33)."""
    import ctypes
    import numpy as np
    import torch
    from drivingsdk_b200 import capi

    lib = capi.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(2468)
    stream = torch.cuda.current_stream()
    st = stream.cuda_stream
    u = lambda lo, hi, *shape: (torch.rand(*shape, generator=g) * (hi - lo) + lo).to(dev)
    hbm_peak, hbm_kind = load_peaks()
    bwd = None
    if args.op == "dcn":
        from oracle import dcn_oracle
        N, C, Co, H, W, k = 18, 512, 512, 29, 50, 3
        shape = capi.DcnShape(N, H, W, C, H, W, Co, k, k, 1, 1, 1, 1, 1, 1, 1, 1)
        M, Kd = N * H * W, k * k * C
        x, off = u(-5, 5, N, H, W, C), u(-2, 2, N, H, W, 2 * k * k)
        mask, w = u(-5, 5, N, H, W, k * k), u(-0.05, 0.05, Co, k, k, C)
        go = u(-5, 5, N, H, W, Co)
        out = torch.empty(N, H, W, Co, device=dev)
        cols = torch.empty(lib.dcn_sm100_columns_bytes(ctypes.byref(shape)) // 4, device=dev)
        ws_bytes = lib.dcn_sm100_backward_workspace_bytes(ctypes.byref(shape))
        ws = torch.empty(ws_bytes // 4 + 4, device=dev)
        gx, goff, gmask, gw = (torch.empty_like(t) for t in (x, off, mask, w))
        old_tc = lib.dcn_sm100_use_tensor_cores(args.tensor_cores)

        def fwd():
            capi.check(lib.dcn_sm100_forward(x.data_ptr(), off.data_ptr(), mask.data_ptr(),
                                             w.data_ptr(), None, out.data_ptr(), cols.data_ptr(),
                                             ctypes.byref(shape), st), "dcn fwd")

        def bwd():
            capi.check(lib.dcn_sm100_backward(
                x.data_ptr(), off.data_ptr(), mask.data_ptr(), w.data_ptr(), cols.data_ptr(),
                go.data_ptr(), gx.data_ptr(), goff.data_ptr(), gmask.data_ptr(), gw.data_ptr(), None,
                ws.data_ptr(), ws_bytes, ctypes.byref(shape), st), "dcn bwd")

        def cpu_once():
            nchw = lambda t, n=1: t[:n].permute(0, 3, 1, 2).cpu().numpy()
            wn = w.permute(0, 3, 1, 2).cpu().numpy()
            dcn_oracle.forward(nchw(x), nchw(off), nchw(mask), wn, None, 1, 1, 1)
            dcn_oracle.backward(nchw(x), nchw(off), nchw(mask), wn, nchw(go), 1, 1, 1)
        samples, cpu_samples = N, 1
        gemm_flops = 2.0 * M * Co * Kd
        peak, peak_kind = load_tensor_peak()
        bound, roof_unit, scale = "tensor", "TFLOP/s", 1e12
        work_fwd, work_bwd = gemm_flops, 2 * gemm_flops
        # operands and results once; the columns tensor once out (forward), once in (backward)
        nx, no, nw, nc, ns = x.numel(), out.numel(), w.numel(), cols.numel(), off.numel() + mask.numel()
        hbm_bytes = {"forward": 4 * (nx + ns + nw + no + nc),
                     "backward": 4 * (2 * nx + 2 * ns + 2 * nw + no + nc)}
        config = {"workload": "modulated_dcn_test_shape", "N": N, "C": C, "Co": Co, "H": H, "W": W,
                  "kernel": k, "groups": 1, "deform_groups": 1,
                  "products": ["fp32 FMA", "tcgen05 3xTF32", "tcgen05 1xTF32"][args.tensor_cores]}
        kernel_name = "three matrix products (forward, grad_columns, grad_weight)"
    elif args.op == "addrelu":
        shape_t = (18, 256, 232, 100)
        x, y = u(-1, 1, *shape_t), u(-1, 1, *shape_t)
        go, gi = u(-1, 1, *shape_t), torch.empty(shape_t, device=dev)
        n = x.numel()

        def fwd():
            capi.check(lib.addrelu_sm100_forward(x.data_ptr(), y.data_ptr(), n, capi.F32, st), "addrelu")

        def bwd():
            capi.check(lib.addrelu_sm100_backward(x.data_ptr(), go.data_ptr(), gi.data_ptr(), n,
                                                  capi.F32, st), "addrelu grad")

        def cpu_once():
            a, b = x[:1].cpu().numpy(), y[:1].cpu().numpy()
            r = np.maximum(a + b, 0)
            np.where(r > 0, go[:1].cpu().numpy(), 0)
        samples, cpu_samples = shape_t[0], 1
        peak, peak_kind = hbm_peak, hbm_kind
        bound, roof_unit, scale = "hbm", "GB/s", 1e9
        work_fwd, work_bwd = 12.0 * n, 12.0 * n
        hbm_bytes = {"forward": 12 * n, "backward": 12 * n}
        config = {"workload": "add_relu_test_shape", "shape": list(shape_t)}
        kernel_name = "add+relu gradient kernel"
    else:
        shape_t = (18, 64, 464, 800)
        x = u(0, 1, *shape_t)
        y = torch.empty(shape_t[0], shape_t[1], (shape_t[2] + 1) // 2, (shape_t[3] + 1) // 2, device=dev)

        def fwd():
            capi.check(lib.maxpool_sm100_forward(x.data_ptr(), y.data_ptr(), *shape_t, capi.F32, st),
                       "maxpool")

        def cpu_once():
            torch.nn.functional.max_pool2d(x[:1].cpu(), 3, 2, 1)
        samples, cpu_samples = shape_t[0], 1
        peak, peak_kind = hbm_peak, hbm_kind
        bound, roof_unit, scale = "hbm", "GB/s", 1e9
        work_fwd, work_bwd = 4.0 * (x.numel() + y.numel()), 0.0
        hbm_bytes = {"forward": 4 * (x.numel() + y.numel())}
        config = {"workload": "resnet_stem_maxpool_test_shape", "shape": list(shape_t),
                  "note": "inference only, as in the reference"}
        kernel_name = "maxpool3s2 kernel"

    def step():
        fwd()
        if bwd is not None:
            bwd()
    for _ in range(max(3, args.warmup)):
        step()
    torch.cuda.synchronize()
    K_steps = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K_steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.msda_sm100_launch_count()
    e0.record(stream)
    for i in range(K_steps):
        ev[i][0].record(stream)
        fwd()
        ev[i][1].record(stream)
        if bwd is not None:
            bwd()
        ev[i][2].record(stream)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / K_steps
    fwd_ms = sum(q[0].elapsed_time(q[1]) for q in ev) / K_steps
    bwd_ms = sum(q[1].elapsed_time(q[2]) for q in ev) / K_steps
    main_ms, main_work = (bwd_ms, work_bwd) if bwd is not None else (fwd_ms, work_fwd)
    roof = {"bound": bound, "kernel": kernel_name,
            "achieved": main_work / (main_ms * 1e-3) / scale, "peak": peak, "unit": roof_unit,
            "frac": main_work / (main_ms * 1e-3) / scale / peak, "traffic": None,
            "peak_kind": peak_kind, "kernel_ms": main_ms,
            "forward": {"achieved": work_fwd / (fwd_ms * 1e-3) / scale,
                        "frac": work_fwd / (fwd_ms * 1e-3) / scale / peak, "kernel_ms": fwd_ms},
            "step": {"frac": (work_fwd + work_bwd) / (ms * 1e-3) / scale / peak},
            "hbm_algorithmic_bytes": hbm_bytes}
    if args.op == "dcn":
        roof["note"] = ("achieved counts each fp32 product once (2*M*N*K); with --tensor-cores 1 "
                        "the tensor cores execute three TF32 products for it")
        lib.dcn_sm100_use_tensor_cores(old_tc)
    line = {
        "metric": f"{args.op}_samples_per_s", "value": samples / (ms * 1e-3), "unit": UNIT,
        "n_gpus": 1, "steps": K_steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config, "roofline": roof,
        "gpu_launches": int(lib.msda_sm100_launch_count() - launches0),
        "device_status": int(lib.msda_sm100_device_status(1)),
    }
    if not args.no_cpu_baseline:
        t0 = time.perf_counter()
        cpu_once()
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": cpu_samples / dt, "unit": UNIT, "cores": os.cpu_count() or 1,
                                "kind": "port",
                                "sample": "1 batch entry through the numpy/torch CPU restatement"}
    print(json.dumps(line))


def main():
    args = parse_args()
    if args.op in ("dcn", "addrelu", "maxpool"):
        run_conv_side(args)
    elif args.op != "msda":
        run_sibling(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
