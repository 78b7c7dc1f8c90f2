"""Benchmark of the AUSSM selective-scan operators on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (the largest point of the benchmark's scaling sweep): unitary
scan, forward + backward, batch 16, d_inner 1024, d_state 16, sequence length
16384, float32 inputs / complex64 state, synthetic seeded inputs (u, z ~ N(0,1),
dt = softplus(N(0,1)), theta ~ U(-pi, pi), B and C with N(0, 1/n) parts).
A step is one forward and one backward pass of the scan over that batch.

  value     scan core (phase tensor resident in HBM), Gelem/s with elem = B*L*D*N,
            timed with CUDA events; with N GPUs every rank runs the same per-GPU
            workload on its own shard (weak scaling, no collective on the data path)
  strong    the same scan with the GLOBAL batch of 16 split over the ranks (16/N rows each)
  e2e       the drop-in operator through ssm_adaptive_interface with HOST buffers:
            pinned-memory inputs copied in and results copied out inside the timed region;
            copy_floor_ms is the same pipeline with the copies alone
  roofline  the backward scan kernel against the measured HBM copy bandwidth
  extras    the other benchmark configurations: the sweep's shorter sequences, the three
            scan variants at batch 8 x d_inner 2048 x 4096 steps, and the two training steps
  cpu_baseline / --impl reference
            the CPU restatement of the reference's PyTorch oracle on a bounded sample

    python bench.py --only scan|complex|real|gemm [shape flags]     one kernel family on a small case
                                                                     (what the profiler captures run)
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(batch=16, d_inner=1024, d_state=16, seq_len=16384)
CONFIG2 = dict(batch=8, d_inner=2048, d_state=16, seq_len=4096)
CPU_SAMPLE = dict(batch=1, seq_len=1024)          # slice of the workload the CPU oracle is timed on
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per algorithmic byte of the backward scan kernel, from the profiler capture named below; the
# capture is only valid for the kernel source it was taken from, so its hash travels with the number.
TRAFFIC_PROFILE = dict(file="profiles/scan_unitary_one_wave.md", ratio=0.98,
                       kernel_source="aussm_b200/csrc/scan_unitary.cu")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # smaller cases for profiler captures; the defaults are the benchmark workload
    ap.add_argument("--batch", type=int, default=WORKLOAD["batch"])
    ap.add_argument("--d-inner", type=int, default=WORKLOAD["d_inner"])
    ap.add_argument("--d-state", type=int, default=WORKLOAD["d_state"])
    ap.add_argument("--seq-len", type=int, default=WORKLOAD["seq_len"])
    ap.add_argument("--only", default="", choices=["", "scan", "complex", "preal", "real", "gemm", "dropin"],
                    help="time one kernel family on the given shape and print a short line")
    ap.add_argument("--gemm-shape", type=int, nargs=3, metavar=("M", "N", "K"), default=(8192, 8192, 1024))
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--e2e-chunk", type=int, default=0, help="batch entries per pipeline chunk of the e2e leg (0: batch/8)")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def source_hash(rel):
    import hashlib
    try:
        with open(os.path.join(ROOT, rel), "rb") as f:
            return hashlib.sha256(f.read()).hexdigest()[:16]
    except OSError:
        return None


def traffic_ratio():
    """(DRAM bytes / algorithmic bytes, where it comes from) for the backward scan kernel, or (None, why) when the
    committed capture was taken from a different version of the kernel source."""
    want = None
    try:
        with open(os.path.join(ROOT, TRAFFIC_PROFILE["file"])) as f:
            for line in f:
                if "kernel source sha256/16:" in line:
                    want = line.split("kernel source sha256/16:")[1].split()[0].strip("` .")
    except OSError:
        return None, f"{TRAFFIC_PROFILE['file']} missing"
    have = source_hash(TRAFFIC_PROFILE["kernel_source"])
    if want is None or have != want:
        return None, (f"{TRAFFIC_PROFILE['file']} was captured from another version of "
                      f"{TRAFFIC_PROFILE['kernel_source']} (capture {want}, now {have})")
    return TRAFFIC_PROFILE["ratio"], (f"ncu one-wave capture ({TRAFFIC_PROFILE['file']}): dram bytes = "
                                      f"{TRAFFIC_PROFILE['ratio']} x algorithmic, scaled by units; kernel source {have}")


# ---------------------------------------------------------------------------
# clocks sampling during the timed region
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        if sm:
            sm.sort()
            out["sm_mhz"] = sm[len(sm) // 2]
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------
def make_scan_inputs(b, d, n, l, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, device=device)
    inp = dict(
        theta=(torch.rand(b, d, n, l, generator=g, device=device) * 2 - 1) * math.pi,
        u=r(b, d, l), dt=torch.nn.functional.softplus(r(b, d, l)), z=r(b, d, l), gy=r(b, d, l),
        B_r=torch.nn.functional.softplus(r(n) / math.sqrt(n)), B_theta=r(n) / math.sqrt(n),
        C_r=torch.nn.functional.softplus(r(n) / math.sqrt(n)), C_theta=r(n) / math.sqrt(n), D=r(d))
    return inp


def make_op_inputs_cpu(b, d, n, l, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    sc = 1.0 / math.sqrt(n)
    return dict(u=r(b, d, l), dt=torch.nn.functional.softplus(r(b, d, l)), x=r(d, n, d) / math.sqrt(d),
                x_bias=(torch.rand(d, n, generator=g) * 2 - 1) * math.pi, B=torch.complex(r(n) * sc, r(n) * sc),
                C=torch.complex(r(n) * sc, r(n) * sc), D=r(d), z=r(b, d, l), gy=r(b, d, l))


# ---------------------------------------------------------------------------
# CPU oracle timing (cpu_baseline and the reference arm)
# ---------------------------------------------------------------------------
def _time_cpu(fn, steps, warmup):
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        fn()
        t1 = time.perf_counter()
        if it >= warmup:
            times.append(t1 - t0)
    return sum(times) / len(times)


def time_cpu_oracle(d, n, steps, warmup, what="dropin"):
    """The CPU port of the reference's PyTorch oracle, float32, all host threads, on a slice of the workload.
    what = "dropin": the operator as the reference defines it (phase projection + scan);
    what = "scan": its scan part alone on a given phase tensor (the same arithmetic as the GPU arm's `value`)."""
    from oracle import unitary as O          # the checker, timed here as the CPU baseline only
    b, l = CPU_SAMPLE["batch"], CPU_SAMPLE["seq_len"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    inp = make_op_inputs_cpu(b, d, n, l, 99)
    if what == "dropin":
        names = ["u", "dt", "x", "x_bias", "B", "C", "D", "z"]
        args = [inp[k].clone().requires_grad_(True) for k in names]

        def run():
            for a in args:
                a.grad = None
            (O.polar_cumsum_unitary(*args) * inp["gy"]).sum().backward()
        label = "drop-in operator (phase projection + scan)"
    else:
        sp = torch.nn.functional.softplus
        theta = O.phase_projection(inp["u"], inp["x"], inp["x_bias"]).detach()
        theta = torch.remainder(theta + math.pi, 2 * math.pi) - math.pi
        args = [theta.requires_grad_(True)] + [inp[k].clone().requires_grad_(True) for k in ("u", "dt", "z")]
        par = [sp(inp["B"].real), inp["B"].imag.clone(), sp(inp["C"].real), inp["C"].imag.clone(), inp["D"]]

        def run():
            for a in args:
                a.grad = None
            y, _, _ = O.scan_unitary_cumsum(*args, *par)
            (y * inp["gy"]).sum().backward()
        label = "scan core (phase tensor given)"
    sec = _time_cpu(run, steps, warmup)
    elems = b * l * d * n
    sample = (f"{label} fwd+bwd in float32 on a slice of the workload: batch {b}, seq {l}, d_inner {d}, "
              f"d_state {n}; mean of {steps} runs after {warmup} warm-up")
    return dict(value=elems / sec / 1e9, unit="Gelem/s", cores=cores, kind="port", sample=sample), sec


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(1, min(args.warmup, 3))
    scan, sec = time_cpu_oracle(args.d_inner, args.d_state, steps, warmup, "scan")
    drop, _ = time_cpu_oracle(args.d_inner, args.d_state, steps, warmup, "dropin")
    cfg = workload_config(args)
    cfg["workload"] = (f"CPU slice of the unitary selective scan fwd+bwd: batch {CPU_SAMPLE['batch']} x d_inner "
                       f"{args.d_inner} x d_state {args.d_state} x seq {CPU_SAMPLE['seq_len']} (the GPU arm runs batch "
                       f"{args.batch} x seq {args.seq_len}; throughput in the same unit)")
    cfg["batch_per_gpu"], cfg["seq_len"] = CPU_SAMPLE["batch"], CPU_SAMPLE["seq_len"]
    line = {
        "impl": "reference", "metric": "AUSSM unitary scan fwd+bwd throughput", "value": scan["value"],
        "unit": "Gelem/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": cfg, "cpu_baseline": scan,
        # like for like with the GPU arm: `value` = scan core alone, `e2e` = the operator with its phase projection
        "e2e": {"value": drop["value"], "unit": "Gelem/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "sample": drop["sample"]},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args):
    return {"workload": (f"unitary selective scan fwd+bwd, batch {args.batch} x d_inner {args.d_inner} x d_state "
                         f"{args.d_state} x seq {args.seq_len} per GPU, float32 / complex64 state"),
            "batch_per_gpu": args.batch, "d_inner": args.d_inner, "d_state": args.d_state, "seq_len": args.seq_len,
            "sharding": "batch shards, one per GPU, no data-path collective",
            "l2": "inputs larger than L2 (no flush needed)"}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class ScanCore:
    """Buffers and the two C-ABI calls of the unitary scan core for one shape."""

    def __init__(self, lib, b, d, n, l, dev, seed):
        self.lib, self.shape = lib, (b, d, n, l)
        self.inp = make_scan_inputs(b, d, n, l, dev, seed)
        i = self.inp
        self.y = torch.empty_like(i["u"])
        self.h_re = torch.empty(b, d, n, device=dev)
        self.h_im = torch.empty_like(self.h_re)
        self.dtheta = torch.empty_like(i["theta"])
        self.du, self.ddt, self.dz = (torch.empty_like(i["u"]) for _ in range(3))
        self.small = [torch.empty(n, device=dev) for _ in range(4)] + [torch.empty(d, device=dev)]
        self.ws = torch.empty(lib.aussm_b200_scan_unitary_bwd_workspace_bytes(b, d, n, l), dtype=torch.uint8,
                              device=dev)
        # non-empty only when the launch is cut into time segments (few channels)
        self.fws = torch.empty(max(16, lib.aussm_b200_scan_unitary_fwd_workspace_bytes(b, d, n, l)), dtype=torch.uint8,
                               device=dev)
        self.stream = torch.cuda.current_stream().cuda_stream

    def fwd(self):
        from aussm_b200 import _lib
        i, P = self.inp, (lambda t: t.data_ptr())
        b, d, n, l = self.shape
        rc = self.lib.aussm_b200_scan_unitary_fwd_ws(P(i["theta"]), P(i["u"]), P(i["dt"]), P(i["z"]), P(i["B_r"]),
                                                     P(i["B_theta"]), P(i["C_r"]), P(i["C_theta"]), P(i["D"]), None,
                                                     None, P(self.y), P(self.h_re), P(self.h_im), b, d, n, l,
                                                     P(self.fws), self.fws.numel(), self.stream)
        _lib.check(rc, "scan forward")

    def bwd(self):
        from aussm_b200 import _lib
        i, P = self.inp, (lambda t: t.data_ptr())
        b, d, n, l = self.shape
        s = self.small
        rc = self.lib.aussm_b200_scan_unitary_bwd(P(i["gy"]), None, None, P(i["theta"]), P(i["u"]), P(i["dt"]),
                                                  P(i["z"]), P(i["B_r"]), P(i["B_theta"]), P(i["C_r"]),
                                                  P(i["C_theta"]), P(i["D"]), P(self.h_re), P(self.h_im),
                                                  P(self.dtheta), P(self.du), P(self.ddt), P(self.dz), P(s[0]),
                                                  P(s[1]), P(s[2]), P(s[3]), P(s[4]), None, None, b, d, n, l,
                                                  P(self.ws), self.ws.numel(), self.stream)
        _lib.check(rc, "scan backward")

    def time(self, steps, warmup, barrier):
        """(ms per step, ms forward, ms backward, launches in the timed region) with CUDA events on the launching stream."""
        for _ in range(warmup):
            self.fwd()
            self.bwd()
        barrier()
        launches0 = self.lib.aussm_b200_kernel_launches()      # the library counts its own kernel launches
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * steps + 1)]
        ev[0].record()
        for k in range(steps):
            self.fwd()
            ev[2 * k + 1].record()
            self.bwd()
            ev[2 * k + 2].record()
        barrier()
        total = ev[0].elapsed_time(ev[2 * steps])
        f = sum(ev[2 * k].elapsed_time(ev[2 * k + 1]) for k in range(steps)) / steps
        bw = sum(ev[2 * k + 1].elapsed_time(ev[2 * k + 2]) for k in range(steps)) / steps
        return total / steps, f, bw, int(self.lib.aussm_b200_kernel_launches() - launches0)


def _time_events(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def variant_case(kind, b, d, n, l, steps, warmup=3, seed=7):
    """Forward and forward+backward time of one scan family through its autograd wrapper (scan cores, inputs
    resident in HBM).  Algorithmic bytes per (b, i, t): unitary 4N+16 / 8N+28, complex 8N+16 / 16N+28,
    positive real 4N+16 / 8N+28 (+ the (b, N, L) B and C streams, negligible for d_inner >> 1), real (Mamba)
    16 / 28."""
    import aussm_b200
    from aussm_b200.s6 import selective_scan_fn
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed + b + d + n + l)
    r = lambda *s: torch.randn(*s, generator=g, device=dev)
    sp = torch.nn.functional.softplus
    u, z, gy = r(b, d, l).requires_grad_(True), r(b, d, l).requires_grad_(True), r(b, d, l)
    dt = sp(r(b, d, l)).requires_grad_(True)
    D = r(d)
    sc = 1 / math.sqrt(n)
    if kind == "unitary":
        theta = ((torch.rand(b, d, n, l, generator=g, device=dev) * 2 - 1) * math.pi).requires_grad_(True)
        Br, Bt, Cr, Ct = sp(r(n) * sc), r(n) * sc, sp(r(n) * sc), r(n) * sc
        leaves = [theta, u, dt, z]
        fwd = lambda: aussm_b200.scan_unitary(theta, u, dt, z, Br, Bt, Cr, Ct, D)[0]
        bytes_f, bytes_b, bound = 4 * n + 16, 8 * n + 28, "hbm"
    elif kind in ("complex", "preal"):
        cplx = kind == "complex"
        rho = (-sp(r(b, d, n, l))).requires_grad_(True)
        theta = ((torch.rand(b, d, n, l, generator=g, device=dev) * 2 - 1) * math.pi).requires_grad_(True) if cplx else None
        Bre, Cre = r(b, n, l) * sc, r(b, n, l) * sc
        Bim, Cim = (r(b, n, l) * sc, r(b, n, l) * sc) if cplx else (None, None)
        leaves = [t for t in (rho, theta, u, dt, z) if t is not None]
        fwd = lambda: aussm_b200.scan_complex(rho, theta, u, dt, z, Bre, Bim, Cre, Cim, D)
        k = 2 if cplx else 1
        bytes_f, bytes_b, bound = 4 * k * n + 16, 8 * k * n + 28, "hbm"
    elif kind == "real":
        A = -torch.exp(r(d, n))
        Bm, Cm = r(b, n, l) * sc, r(b, n, l) * sc
        leaves = [u, dt, z]
        fwd = lambda: selective_scan_fn(u, dt, A, Bm, Cm, D, z=z, delta_softplus=True)
        bytes_f, bytes_b, bound = 16, 28, ("instruction issue and dependent-chain latency (issue slots 0.44 / 0.41 busy, shared-memory "
                                          "pipe 0.62 / 0.60: profiles/scan_s6_small.md), not HBM")
    else:
        raise ValueError(kind)
    ms_f = _time_events(lambda: fwd(), steps, warmup)

    def both():
        for t in leaves:
            t.grad = None
        fwd().backward(gy)

    ms_fb = _time_events(both, steps, warmup)
    peak, _src = measured_peak()
    units = b * d * l
    gbs = units * (bytes_f + bytes_b) / ms_fb / 1e6
    return {"kind": kind, "batch": b, "d_inner": d, "d_state": n, "seq_len": l, "ms_fwd": round(ms_f, 4),
            "ms_fwd_bwd": round(ms_fb, 4), "gelem_s": round(units * n / ms_fb / 1e6, 2),
            "algorithmic_gb_s": round(gbs, 1), "hbm_frac": round(gbs / peak, 4), "bound": bound,
            "note": "through the autograd wrappers (output allocation included)"}


def gemm_case(M, N, K, steps, warmup=3):
    """C (M x N) = A (M x K, K contiguous) * B (K x N, N contiguous) through aussm_b200_gemm_split3."""
    import aussm_b200
    from aussm_b200 import _lib
    lib = _lib.load()
    A = torch.randn(M, K, device="cuda")
    B = torch.randn(K, N, device="cuda")
    C = torch.empty(M, N, device="cuda")
    ws = torch.empty(lib.aussm_b200_gemm_split3_workspace_bytes(M, N, K, 1, 0, 0, 1, 0), dtype=torch.uint8, device="cuda")

    def call():
        _lib.check(lib.aussm_b200_gemm_split3(A.data_ptr(), 0, 0, B.data_ptr(), 1, 0, C.data_ptr(), M, N, K, 1, 0, 0,
                                              ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream),
                   "gemm_split3")

    ms = _time_events(call, steps, warmup)
    return {"kind": "split gemm", "M": M, "N": N, "K": K, "ms": ms,
            "tflops_float32_equivalent": 2.0 * M * N * K / ms / 1e9, "device_status": aussm_b200.device_status(),
            "note": "includes the two hi/lo split passes of the operands"}


def dropin_case(b, d, n, l, steps, warmup=2):
    """The drop-in operator fwd+bwd with inputs resident in HBM (no host copies)."""
    import aussm_b200
    inp = {k: v.cuda() for k, v in make_op_inputs_cpu(b, d, n, l, 5).items()}
    names = ["u", "dt", "x", "x_bias", "B", "C", "D", "z"]
    args = [inp[k].requires_grad_(True) for k in names]

    def both():
        for a in args:
            a.grad = None
        aussm_b200.ssm_adaptive_interface(*args, unitary=True).backward(inp["gy"])

    ms = _time_events(both, steps, warmup)
    return {"kind": "drop-in operator", "batch": b, "d_inner": d, "d_state": n, "seq_len": l, "ms_fwd_bwd": ms,
            "gelem_s": b * d * n * l / ms / 1e6, "device_status": aussm_b200.device_status()}


def run_only(args):
    torch.cuda.set_device(0)
    b, d, n, l = args.batch, args.d_inner, args.d_state, args.seq_len
    if args.only == "scan":
        from aussm_b200 import _lib
        lib = _lib.load()
        out = {"kind": "unitary scan core", "batch": b, "d_inner": d, "d_state": n, "seq_len": l}
        # with and without the time-axis split (it only engages when the channels under-fill the GPU)
        for tag, on in (("", 1), ("_no_time_split", 0)):
            _lib.set_option("time_split", on)
            split = lib.aussm_b200_scan_unitary_fwd_workspace_bytes(b, d, n, l) > 0
            if not on and "time_split" in out and not out["time_split"]:
                break
            core = ScanCore(lib, b, d, n, l, torch.device("cuda", 0), 1234)
            ms, f, bw, _ = core.time(args.steps, args.warmup, torch.cuda.synchronize)
            out.update({"ms_fwd" + tag: f, "ms_bwd" + tag: bw, "ms_fwd_bwd" + tag: ms})
            if on:
                out["time_split"] = split
            del core
        _lib.set_option("time_split", 1)
    elif args.only == "gemm":
        out = gemm_case(*args.gemm_shape, args.steps, args.warmup)
    elif args.only == "dropin":
        out = dropin_case(b, d, n, l, args.steps, args.warmup)
    else:
        out = variant_case(args.only, b, d, n, l, args.steps, args.warmup)
    print(json.dumps(out), flush=True)


def run_extras(args, dev, world, rank, barrier):
    """The other benchmark configurations, short runs.  One GPU: the sweep's shorter sequences and the three
    variants of configuration 2.  Every N: the two end-to-end training steps (batch sharded over the ranks,
    NCCL all-reduce of the weight gradients)."""
    from aussm_b200 import _lib
    from aussm_b200.train import make_config, max_over_ranks, train_step
    out = {}
    if world == 1:
        lib = _lib.load()
        sweep = []
        b, d, n = WORKLOAD["batch"], WORKLOAD["d_inner"], WORKLOAD["d_state"]
        peak, _ = measured_peak()
        for l in (256, 1024, 4096):
            core = ScanCore(lib, b, d, n, l, dev, 77 + l)
            ms, f, bw, _ = core.time(5, 3, torch.cuda.synchronize)
            units = b * d * l
            sweep.append({"seq_len": l, "ms_fwd": round(f, 4), "ms_bwd": round(bw, 4), "ms_fwd_bwd": round(ms, 4),
                          "gelem_s": round(units * n / ms / 1e6, 2),
                          "hbm_frac": round(units * (12 * n + 44) / ms / 1e6 / peak, 4)})
            del core
        out["config1_sweep"] = {"shape": f"batch {b} x d_inner {d} x d_state {n}", "points": sweep}
        torch.cuda.empty_cache()
        c2 = CONFIG2
        out["config2_variants"] = [variant_case(k, c2["batch"], c2["d_inner"], c2["d_state"], c2["seq_len"], 3, 2)
                                   for k in ("real", "complex", "preal", "unitary")]
        torch.cuda.empty_cache()
    train = []
    for config, micro, steps, warm in ((3, 0, 5, 3), (4, 4, 2, 1)):
        model, batch, loss_fn, tokens, local_batch, gb = make_config(config, dev, rank, world)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
        x, y = batch()
        for _ in range(warm):
            train_step(model, opt, x, y, loss_fn, world, micro, global_batch=gb)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            loss, ncoll = train_step(model, opt, x, y, loss_fn, world, micro, global_batch=gb)
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1) / steps, dev, world)
        rec = {"config": config, "ms_per_step": round(ms, 3), "tokens_per_s": round(tokens / ms * 1e3, 1),
               "local_batch": local_batch, "micro_batch": micro, "steps": steps, "warmup": warm,
               "allreduce_calls_per_step": ncoll, "loss": loss}
        if world == 1 and config == 3:
            # the same step captured once into a CUDA graph and replayed (the small configuration is bound by the
            # host's launch rate; one process only: the all-reduce variant is not captured)
            try:
                rec.update(_graphed_step(config, dev, x, y, micro, gb, warm, steps, tokens))
            except Exception as exc:          # the eager figure above stands on its own
                rec["cuda_graph_error"] = f"{type(exc).__name__}: {exc}"[:300]
        train.append(rec)
        del model, opt, x, y
        torch.cuda.empty_cache()
    out["training_steps"] = train
    return out


def _graphed_step(config, dev, x, y, micro, gb, warm, steps, tokens):
    """The training step of `config` captured once into a CUDA graph and replayed: its time per step."""
    from aussm_b200.train import GraphedTrainStep, make_config
    model_g, _b, loss_g, _t, _l, _g = make_config(config, dev, 0, 1)
    opt_g = torch.optim.AdamW(model_g.parameters(), lr=1e-3, capturable=True)
    graphed = GraphedTrainStep(model_g, opt_g, x, y, loss_g, micro_batch=micro, global_batch=gb)
    for _ in range(warm):
        graphed.step()
    torch.cuda.synchronize()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(steps):
        gl = graphed.step()
    g1.record()
    torch.cuda.synchronize()
    gms = g0.elapsed_time(g1) / steps
    return {"ms_per_step_cuda_graph": round(gms, 3), "tokens_per_s_cuda_graph": round(tokens / gms * 1e3, 1),
            "loss_cuda_graph": float(gl)}


def run_ours(args):
    import torch.distributed as dist

    import aussm_b200
    from aussm_b200 import _lib

    if args.only:
        return run_only(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def rank_max(ms):
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    b, d, n, l = args.batch, args.d_inner, args.d_state, args.seq_len
    elems = b * d * n * l
    core = ScanCore(lib, b, d, n, l, dev, 1234 + rank)
    # warm-up outside the sampled region, then the timed steps with the clocks sampled
    for _ in range(args.warmup):
        core.fwd()
        core.bwd()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_local, fwd_ms, bwd_ms, launches = core.time(args.steps, 0, barrier)
    clocks = sampler.stop() if rank == 0 else None
    status = lib.aussm_b200_device_status(core.stream)
    if status != 0:
        raise RuntimeError(f"device status {status} after the timed region")
    ms_per_step = rank_max(ms_local)
    value = elems * world / (ms_per_step * 1e-3) / 1e9

    # roofline of the dominant kernel (backward scan): algorithmic bytes per (b, i, t) = 8N + 28
    peak, peak_src = measured_peak()
    bwd_bytes = (8 * n + 28) * b * d * l
    fwd_bytes = (4 * n + 16) * b * d * l
    achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    ratio, traffic_src = traffic_ratio()
    mhz = clocks.get("sm_mhz") if clocks else None
    roofline = {"bound": "hbm", "kernel": "scan_unitary_bwd_kernel", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak,
                "traffic": int(ratio * bwd_bytes) if ratio is not None else None, "traffic_source": traffic_src,
                "peak_source": peak_src, "bytes_per_launch": bwd_bytes, "ms_per_launch": bwd_ms,
                # the kernel is close to FP32-issue-bound, so its time follows the SM clock: cycles compare runs
                "mcycles_per_launch": bwd_ms * mhz * 1e-3 if mhz else None,
                "forward": {"kernel": "scan_unitary_fwd_kernel", "achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                            "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak, "ms_per_launch": fwd_ms,
                            "bytes_per_launch": fwd_bytes,
                            "mcycles_per_launch": fwd_ms * mhz * 1e-3 if mhz else None},
                "fwd_bwd_frac": (fwd_bytes + bwd_bytes) / (ms_per_step * 1e-3) / 1e9 / peak}
    del core
    torch.cuda.empty_cache()

    # strong scaling: the global batch of the workload split over the ranks (batch/N rows per GPU)
    strong = None
    if b % world == 0:
        if world == 1:
            strong = {"value": value, "unit": "Gelem/s", "ms_per_step": ms_per_step, "batch_per_gpu": b,
                      "global_batch": b}
        else:
            sb = b // world
            score = ScanCore(lib, sb, d, n, l, dev, 4321 + rank)
            s_ms, _, _, _ = score.time(args.steps, args.warmup, barrier)
            s_ms = rank_max(s_ms)
            strong = {"value": elems / (s_ms * 1e-3) / 1e9, "unit": "Gelem/s", "ms_per_step": s_ms,
                      "batch_per_gpu": sb, "global_batch": b,
                      "note": "total work fixed: the workload's batch split over the ranks, no collective"}
            del score
            torch.cuda.empty_cache()

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, dev, world, rank)
    extras = None
    if not args.no_extras:
        if world == 1:
            try:
                extras = run_extras(args, dev, world, rank, barrier)
            except Exception as exc:          # the headline line does not depend on the extra configurations
                extras = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        else:
            extras = run_extras(args, dev, world, rank, barrier)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu, _ = time_cpu_oracle(d, n, 3, 2, "scan")

    if rank == 0:
        line = {
            "metric": "AUSSM unitary scan fwd+bwd throughput", "value": value, "unit": "Gelem/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args), "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "roofline": roofline, "cpu_baseline": cpu, "strong": strong, "extras": extras,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_e2e(args, dev, world, rank):
    """Drop-in operator with host buffers: H2D of u, dt, z, grad_y and the parameters, forward and
    backward through ssm_adaptive_interface, D2H of y and of every gradient, all inside the timed region."""
    import torch.distributed as dist

    import aussm_b200

    b, d, n, l = args.batch, args.d_inner, args.d_state, args.seq_len
    # pinned buffers on the GPU's own NUMA node (matters when several ranks share a two-socket host)
    saved_affinity = os.sched_getaffinity(0)
    host = make_op_inputs_cpu(b, d, n, l, 4321 + rank)
    numa_cpus = aussm_b200.bind_process_to_gpu_cpus(dev)
    pin = {k: v.pin_memory() for k, v in host.items()}
    out_host = {k: torch.empty_like(v).pin_memory() for k, v in host.items() if k != "gy"}
    out_host["y"] = torch.empty_like(host["u"]).pin_memory()
    os.sched_setaffinity(0, saved_affinity)          # only the allocations above needed the binding
    h2d = sum(v.numel() * v.element_size() for v in pin.values())
    d2h = sum(v.numel() * v.element_size() for v in out_host.values())

    pipe = aussm_b200.HostBatchStep(dev, chunk=args.e2e_chunk or None)
    steps = max(1, min(args.steps, 3))

    def timed(fn, warm):
        for _ in range(warm):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    ms = timed(lambda: pipe.step(pin, out_host), 2)
    launches = pipe.kernel_launches_last_step
    # the same pipeline with the copies alone (same pinned buffers, same chunks, no arithmetic): what the host
    # and the PCIe links give this step at this number of ranks
    floor_ms = timed(lambda: pipe.step(pin, out_host, copies_only=True), 1)
    if aussm_b200.device_status() != 0:
        raise RuntimeError("device status non-zero after the end-to-end leg")
    elems = b * d * n * l * world
    return {"value": elems / (ms * 1e-3) / 1e9, "unit": "Gelem/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": ms, "steps": steps, "copy_floor_ms": floor_ms,
            "copy_floor_gb_s_per_rank_each_way": (h2d + d2h) / 2 / (floor_ms * 1e-3) / 1e9,
            "host_cpus_bound": numa_cpus, "gpu_launches_per_step": launches,
            "api": "aussm_b200.HostBatchStep (chunks of batch/8 through ssm_adaptive_interface, the extension_cpp "
                   "drop-in; three-stream copy-in / compute / copy-out pipeline: parameters first, forward as soon "
                   "as u, dt, z are there, y out during the backward pass), host pinned buffers"}


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
