"""Benchmark of the AUSSM unitary selective scan on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE configs[1], largest point of the sweep): unitary scan,
forward + backward, batch 16, d_inner 1024, d_state 16, sequence length 16384,
float32 inputs / complex64 state, synthetic seeded inputs (u, z ~ N(0,1),
dt = softplus(N(0,1)), theta ~ U(-pi, pi), B and C with N(0, 1/n) parts).
A step is one forward and one backward pass of the scan over that batch.

  value     scan core (phase tensor resident in HBM), Gelem/s with elem = B*L*D*N,
            timed with CUDA events; with N GPUs every rank runs the same per-GPU
            workload on its own shard (weak scaling, no collective on the data path)
  e2e       the drop-in operator through ssm_adaptive_interface with HOST buffers:
            pinned-memory inputs copied in and results copied out inside the timed region
  roofline  the backward scan kernel against the measured HBM copy bandwidth
  cpu_baseline / --impl reference
            the CPU restatement of the reference's PyTorch oracle on a bounded sample
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
CPU_SAMPLE = dict(batch=1, seq_len=1024)          # slice of the workload the CPU oracle is timed on
FALLBACK_HBM_GBS = 6650.0


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
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-chunk", type=int, default=0, help="batch entries per pipeline chunk of the e2e leg (0: batch/8)")
    ap.add_argument("--e2e-streams", type=int, default=1, help="compute streams of the e2e pipeline (1 or 2)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--fast-trig", type=int, default=0)
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--blocks-per-sm", type=int, default=0)
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


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
def time_cpu_oracle(d, n, steps, warmup):
    from oracle import unitary as O          # the checker, timed here as the CPU baseline only
    b, l = CPU_SAMPLE["batch"], CPU_SAMPLE["seq_len"]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    inp = make_op_inputs_cpu(b, d, n, l, 99)
    names = ["u", "dt", "x", "x_bias", "B", "C", "D", "z"]
    args = [inp[k].clone().requires_grad_(True) for k in names]
    times = []
    for it in range(warmup + steps):
        for a in args:
            a.grad = None
        t0 = time.perf_counter()
        y = O.polar_cumsum_unitary(*args)
        (y * inp["gy"]).sum().backward()
        t1 = time.perf_counter()
        if it >= warmup:
            times.append(t1 - t0)
    sec = sum(times) / len(times)
    elems = b * l * d * n
    sample = (f"drop-in operator (phase projection + scan) fwd+bwd in float32 on a slice of the workload: batch {b}, "
              f"seq {l}, d_inner {d}, d_state {n}; mean of {steps} runs after {warmup} warm-up")
    return dict(value=elems / sec / 1e9, unit="Gelem/s", cores=cores, kind="port", sample=sample), sec


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb, sec = time_cpu_oracle(args.d_inner, args.d_state, max(1, args.steps), max(1, min(args.warmup, 2)))
    line = {
        "impl": "reference", "metric": "AUSSM unitary scan fwd+bwd throughput", "value": cb["value"],
        "unit": "Gelem/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args), "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "Gelem/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
def run_ours(args):
    import torch.distributed as dist

    import aussm_b200
    from aussm_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    _lib.set_option("fast_trig", args.fast_trig)
    _lib.set_option("variant", args.variant)
    _lib.set_option("blocks_per_sm", args.blocks_per_sm)

    b, d, n, l = args.batch, args.d_inner, args.d_state, args.seq_len
    elems = b * d * n * l
    inp = make_scan_inputs(b, d, n, l, dev, 1234 + rank)
    y = torch.empty_like(inp["u"])
    h_re = torch.empty(b, d, n, device=dev)
    h_im = torch.empty_like(h_re)
    dtheta = torch.empty_like(inp["theta"])
    du, ddt, dz = (torch.empty_like(inp["u"]) for _ in range(3))
    dB_r, dB_t, dC_r, dC_t = (torch.empty(n, device=dev) for _ in range(4))
    dD = torch.empty(d, device=dev)
    ws = torch.empty(lib.aussm_b200_scan_unitary_bwd_workspace_bytes(b, d, n, l), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    P = lambda t: t.data_ptr()

    def fwd():
        rc = lib.aussm_b200_scan_unitary_fwd(P(inp["theta"]), P(inp["u"]), P(inp["dt"]), P(inp["z"]), P(inp["B_r"]),
                                             P(inp["B_theta"]), P(inp["C_r"]), P(inp["C_theta"]), P(inp["D"]), None,
                                             None, P(y), P(h_re), P(h_im), b, d, n, l, stream)
        _lib.check(rc, "scan forward")

    def bwd():
        rc = lib.aussm_b200_scan_unitary_bwd(P(inp["gy"]), None, None, P(inp["theta"]), P(inp["u"]), P(inp["dt"]),
                                             P(inp["z"]), P(inp["B_r"]), P(inp["B_theta"]), P(inp["C_r"]),
                                             P(inp["C_theta"]), P(inp["D"]), P(h_re), P(h_im), P(dtheta), P(du),
                                             P(ddt), P(dz), P(dB_r), P(dB_t), P(dC_r), P(dC_t), P(dD), None, None, b,
                                             d, n, l, P(ws), ws.numel(), stream)
        _lib.check(rc, "scan backward")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        fwd()
        bwd()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3 * args.steps + 1)]
    ev[0].record()
    for k in range(args.steps):
        fwd()
        ev[3 * k + 1].record()
        bwd()
        ev[3 * k + 2].record()
        ev[3 * k + 3].record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = ev[0].elapsed_time(ev[3 * args.steps])
    fwd_ms = sum(ev[3 * k].elapsed_time(ev[3 * k + 1]) for k in range(args.steps)) / args.steps
    bwd_ms = sum(ev[3 * k + 1].elapsed_time(ev[3 * k + 2]) for k in range(args.steps)) / args.steps
    status = lib.aussm_b200_device_status(stream)
    if status != 0:
        raise RuntimeError(f"device status {status} after the timed region")
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_ms = float(t.item())
    ms_per_step = max_ms / args.steps
    value = elems * world / (ms_per_step * 1e-3) / 1e9

    # roofline of the dominant kernel (backward scan): algorithmic bytes per (b, i, t) = 8N + 28
    peak, peak_src = measured_peak()
    bwd_bytes = (8 * n + 28) * b * d * l
    fwd_bytes = (4 * n + 16) * b * d * l
    achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "scan_unitary_bwd_kernel", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "traffic": int(0.98 * bwd_bytes), "traffic_source": "ncu one-wave capture (profiles/scan_unitary_one_wave.md): dram bytes = 0.98 x algorithmic, scaled by units", "peak_source": peak_src,
                "bytes_per_launch": bwd_bytes, "ms_per_launch": bwd_ms,
                "forward": {"kernel": "scan_unitary_fwd_kernel", "achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                            "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak, "ms_per_launch": fwd_ms,
                            "bytes_per_launch": fwd_bytes},
                "fwd_bwd_frac": (fwd_bytes + bwd_bytes) / (ms_per_step * 1e-3) / 1e9 / peak}

    # free the scan-core buffers before the end-to-end leg
    del dtheta, du, ddt, dz, y, ws
    inp.clear()
    torch.cuda.empty_cache()

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, dev, world, rank)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu, _ = time_cpu_oracle(d, n, 2, 1)

    if rank == 0:
        line = {
            "metric": "AUSSM unitary scan fwd+bwd throughput", "value": value, "unit": "Gelem/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args), "clocks": clocks, "e2e": e2e, "gpu_launches": 3 * args.steps,
            "roofline": roofline, "cpu_baseline": cpu,
            "options": {"fast_trig": args.fast_trig, "variant": args.variant},
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

    pipe = aussm_b200.HostBatchStep(dev, chunk=args.e2e_chunk or None, compute_streams=args.e2e_streams)

    def step():
        pipe.step(pin, out_host)

    steps = max(1, min(args.steps, 3))
    for _ in range(2):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if aussm_b200.device_status() != 0:
        raise RuntimeError("device status non-zero after the end-to-end leg")
    elems = b * d * n * l * world
    return {"value": elems / (float(ms.item()) * 1e-3) / 1e9, "unit": "Gelem/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": float(ms.item()), "steps": steps,
            "host_cpus_bound": numa_cpus,
            "api": "aussm_b200.HostBatchStep (chunks of batch/8 through ssm_adaptive_interface, the extension_cpp "
                   "drop-in; three-stream copy-in / compute / copy-out pipeline), host pinned buffers",
            "gpu_launches_per_step": "per chunk and window: 3 tcgen05 GEMMs, 3 TF32 splits, 1 fwd + 1 bwd scan; "
                                     "1 reduce per chunk (phases kept between forward and backward)"}


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
