"""Timing sweep of the scan operators (CUDA events, scan cores with inputs resident in HBM).

    python -m aussm_b200.sweep [--config 1|2] [--steps K]
    python -m aussm_b200.sweep --gemm M N K [--steps K]      (the split GEMM alone, theta-like operand layouts)

config 1: unitary scan core, batch 16, d_inner 1024, d_state 16, seq in {256, 1024, 4096, 16384}
config 2: real (Mamba S6), complex and unitary scan cores at batch 8, d_inner 2048, d_state 16, seq 4096
Prints one JSON line per case: ms forward, ms backward, Gelem/s (elem = B*L*D*N) and algorithmic GB/s.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

import aussm_b200
from aussm_b200.s6 import selective_scan_fn


def _time(fn, steps, warmup=2):
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


def _case(kind, b, d, n, l, steps):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(b + d + n + l)
    r = lambda *s: torch.randn(*s, generator=g, device=dev)
    sp = torch.nn.functional.softplus
    u, z, gy = r(b, d, l), r(b, d, l), r(b, d, l)
    dt = sp(r(b, d, l))
    D = r(d)
    if kind == "unitary":
        theta = ((torch.rand(b, d, n, l, generator=g, device=dev) * 2 - 1) * math.pi).requires_grad_(True)
        Br, Bt, Cr, Ct = sp(r(n)), r(n), sp(r(n)), r(n)
        leaves = [theta, u.requires_grad_(True), dt.requires_grad_(True), z.requires_grad_(True)]
        fwd = lambda: aussm_b200.scan_unitary(theta, u, dt, z, Br, Bt, Cr, Ct, D)[0]
        bytes_f, bytes_b = (4 * n + 16), (8 * n + 28)
    elif kind == "complex":
        rho = (-sp(r(b, d, n, l))).requires_grad_(True)
        theta = ((torch.rand(b, d, n, l, generator=g, device=dev) * 2 - 1) * math.pi).requires_grad_(True)
        s = 1 / math.sqrt(n)
        Bre, Bim, Cre, Cim = (r(b, n, l) * s for _ in range(4))
        leaves = [rho, theta, u.requires_grad_(True), dt.requires_grad_(True), z.requires_grad_(True)]
        fwd = lambda: aussm_b200.scan_complex(rho, theta, u, dt, z, Bre, Bim, Cre, Cim, D)
        bytes_f, bytes_b = (8 * n + 16), (16 * n + 28)
    else:  # real: Mamba S6
        A = -torch.exp(r(d, n))
        s = 1 / math.sqrt(n)
        Bm, Cm = r(b, n, l) * s, r(b, n, l) * s
        delta = r(b, d, l).requires_grad_(True)
        leaves = [u.requires_grad_(True), delta, z.requires_grad_(True)]
        fwd = lambda: selective_scan_fn(u, delta, A, Bm, Cm, D, z=z, delta_softplus=True)
        bytes_f, bytes_b = 16, 28
    ms_f = _time(lambda: fwd(), steps)

    def both():
        for t in leaves:
            t.grad = None
        fwd().backward(gy)

    ms_fb = _time(both, steps)
    units = b * d * l
    elems = units * n
    print(json.dumps({"kind": kind, "batch": b, "d_inner": d, "d_state": n, "seq": l, "ms_fwd": round(ms_f, 4),
                      "ms_fwd_bwd": round(ms_fb, 4), "gelem_s": round(elems / ms_fb / 1e6, 2),
                      "algorithmic_gb_s_fwd": round(units * bytes_f / ms_f / 1e6, 1),
                      "algorithmic_gb_s_fwd_bwd": round(units * (bytes_f + bytes_b) / ms_fb / 1e6, 1),
                      "note": "through the autograd wrappers (output allocation included)"}), flush=True)


def _gemm_case(M, N, K, steps):
    """C (M x N) = A (M x K, K contiguous) * B (K x N, N contiguous) through aussm_b200_gemm_tf32x3."""
    from aussm_b200 import _lib
    lib = _lib.load()
    A = torch.randn(M, K, device="cuda")
    B = torch.randn(K, N, device="cuda")
    C = torch.empty(M, N, device="cuda")
    ws = torch.empty(lib.aussm_b200_gemm_tf32x3_workspace_bytes(M, N, K, 1, 0, 0), dtype=torch.uint8, device="cuda")

    def call():
        _lib.check(lib.aussm_b200_gemm_tf32x3(A.data_ptr(), 0, 0, B.data_ptr(), 1, 0, C.data_ptr(), M, N, K, 1, 0, 0,
                                              ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream),
                   "gemm_tf32x3")

    ms = _time(call, steps, warmup=3)
    print(json.dumps({"kind": "split gemm", "M": M, "N": N, "K": K, "ms": ms,
                      "tflops_float32_equivalent": 2.0 * M * N * K / ms / 1e9,
                      "device_status": aussm_b200.device_status(),
                      "note": "includes the two hi/lo split passes of the operands"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--gemm", type=int, nargs=3, metavar=("M", "N", "K"))
    a = ap.parse_args()
    if a.gemm:
        _gemm_case(*a.gemm, a.steps)
    elif a.config == 1:
        for l in (256, 1024, 4096, 16384):
            _case("unitary", 16, 1024, 16, l, a.steps)
    else:
        for kind in ("real", "complex", "unitary"):
            _case(kind, 8, 2048, 16, 4096, a.steps)


if __name__ == "__main__":
    main()
