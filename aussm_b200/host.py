"""Forward + backward of the adaptive unitary operator for a batch that lives in pinned HOST memory.

The operator is independent across batch entries (only the parameter gradients sum over the batch), so a batch
that arrives from the host does not have to be resident on the device as a whole: ``HostBatchStep`` cuts it into
chunks of a few batch entries and runs three CUDA streams as a pipeline,

    copy-in stream   the parameters, then host -> device of chunk c+1 (u, dt, z; grad_y last)
    compute stream   ssm_adaptive_interface forward (as soon as u, dt, z are there) and backward of chunk c
                     (parameter gradients accumulate)
    copy-out stream  device -> host of y of chunk c while its backward pass runs, then du, ddt, dz

with two sets of device buffers, so that the PCIe transfers of one chunk hide behind the arithmetic of another.
The result is the same as one ``ssm_adaptive_interface`` call on the whole batch followed by ``backward`` (the
parameter gradients are summed chunk by chunk in a fixed order, so they are reproducible, but the order of that
sum differs from the single call's).

There is no counterpart in the reference, which keeps its batches on the device
(extension-cpp/extension_cpp/ops.py:28-93 is the call this wraps).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
from torch import Tensor

from . import ops

__all__ = ["HostBatchStep", "bind_process_to_gpu_cpus"]


def bind_process_to_gpu_cpus(device) -> int:
    """Restrict the calling process to the CPU cores next to `device` (NVML's ideal CPU affinity of that GPU), so that
    pinned host buffers allocated afterwards land on the GPU's own NUMA node.  With one process per GPU on a
    two-socket host this keeps the host<->device copies of all ranks off the inter-socket link.  Returns the number
    of cores in the new affinity set, or 0 if nothing was changed (NVML missing, no affinity information)."""
    import os
    try:
        import pynvml
        dev = torch.device(device)
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(idx).uuid)
            handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (ncpu + 63) // 64)
        cpus = {64 * w + b for w, mask in enumerate(words) for b in range(64) if (int(mask) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        cpus &= allowed
        if not cpus or cpus == allowed:
            return 0
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return 0

_SEQ = ("u", "dt", "z", "gy")                    # (b, d, l) tensors that travel per chunk
_PARAMS = ("x", "x_bias", "B", "C", "D")


class HostBatchStep:
    """Pipelined forward+backward over a host-resident batch.

    ``step(inputs, outputs)``: ``inputs`` maps ``u, dt, z, gy`` to pinned float32 host tensors ``(b, d, l)`` and
    ``x, x_bias, B, C, D`` to the parameters (host or device); ``outputs`` maps ``y, u, dt, z`` to pinned host
    tensors that receive the output and the gradients of ``u, dt, z``, and ``x, x_bias, B, C, D`` to host tensors
    that receive the parameter gradients.  The call returns after queueing everything; the caller's current
    stream waits for the last copy, so a synchronize (or an event recorded on it) covers the whole step.
    """

    def __init__(self, device, chunk: Optional[int] = None, short_edges: bool = True, timeline: bool = False):
        self.device = torch.device(device)
        self.chunk = chunk
        self.short_edges = short_edges
        self.timeline = timeline          # record the start and end of every stage of every chunk (last_timeline())
        self._marks = []
        self.s_in = torch.cuda.Stream(self.device)
        # one compute stream: two streams taking the chunks in turn measured slower (146 against 136 ms on the
        # benchmark step)
        self.s_cmp = [torch.cuda.Stream(self.device)]
        self.s_out = torch.cuda.Stream(self.device)
        self._bufs = None
        self._shape = None
        self.kernel_launches_last_step = 0     # this library's kernels queued by the last step() call

    def _prepare(self, b, d, l, chunk):
        key = (b, d, l, chunk)
        if self._shape == key:
            return
        self._shape = key
        mk = lambda: torch.empty(chunk, d, l, device=self.device, dtype=torch.float32)
        self._bufs = [{k: mk() for k in _SEQ} for _ in range(2)]

    def _mark(self, stream, chunk: int, what: str) -> None:
        if self.timeline:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            self._marks.append((chunk, what, ev))

    def last_timeline(self):
        """Milliseconds from the start of the last ``step`` (recorded with ``timeline=True``) at which each chunk's
        copy-in, compute and copy-out began and ended: a list of ``(chunk, label, ms)`` with labels ``in0 in1 cmp0
        cmp1 out0 out1`` (chunk -1: ``start`` / ``end`` of the step).  Synchronizes the device."""
        if not self._marks:
            return []
        torch.cuda.synchronize(self.device)
        t0 = self._marks[0][2]
        return [(c, what, t0.elapsed_time(ev)) for c, what, ev in self._marks]

    def step(self, inputs: Dict[str, Tensor], outputs: Dict[str, Tensor], copies_only: bool = False) -> None:
        """``copies_only=True`` queues the same host<->device copies in the same chunks and order but no
        arithmetic (the outputs then hold copies of the inputs): the time of that is what the host and the
        links allow this step, whatever the kernels do."""
        from . import _lib
        launches0 = _lib.load().aussm_b200_kernel_launches()
        u = inputs["u"]
        b, d, l = u.shape
        chunk = self.chunk or max(1, b // 8)
        self._prepare(b, d, l, chunk)
        for k in _SEQ:
            if not inputs[k].is_pinned():
                raise RuntimeError(f"HostBatchStep: input '{k}' must be in pinned host memory")
        cur = torch.cuda.current_stream(self.device)
        self._marks = []
        mark = self._mark
        mark(cur, -1, "start")
        for s in (self.s_in, self.s_out, *self.s_cmp):
            s.wait_stream(cur)

        # The parameters travel first, on the copy-in stream: copies of one direction are served in the order they
        # were queued whatever their stream, so a parameter copy queued on the compute stream would wait behind
        # the first two chunks.  One set of parameter leaves per compute stream (each accumulates its own
        # gradients), added at the end.
        params = []
        with torch.cuda.stream(self.s_in):
            for sc in self.s_cmp:
                params.append([inputs[k].to(self.device, non_blocking=True).detach().requires_grad_(True)
                               for k in _PARAMS])
            params_ready = self.s_in.record_event()
        for sc in self.s_cmp:
            sc.wait_event(params_ready)
            for par in params:
                for t in par:
                    t.record_stream(sc)

        # chunk boundaries: a short first and last chunk (the copy-in of the first and the copy-out of the last are
        # the two transfers nothing can hide)
        edge = 1 if (chunk >= 2 and b >= 2 * chunk + 2 and self.short_edges) else 0
        bounds = [0]
        if edge:
            bounds.append(edge)
        while bounds[-1] < b - edge:
            bounds.append(min(b - edge, bounds[-1] + chunk))
        if edge:
            bounds.append(b)
        in_free = [None, None]        # the compute stream no longer reads buffer set i
        for c in range(len(bounds) - 1):
            lo, hi = bounds[c], bounds[c + 1]
            i = c % 2
            buf = self._bufs[i]
            with torch.cuda.stream(self.s_in):
                if in_free[i] is not None:
                    self.s_in.wait_event(in_free[i])
                mark(self.s_in, c, "in0")
                for k in ("u", "dt", "z"):
                    buf[k][: hi - lo].copy_(inputs[k][lo:hi], non_blocking=True)
                fwd_ready = self.s_in.record_event()          # the forward pass can start
                buf["gy"][: hi - lo].copy_(inputs["gy"][lo:hi], non_blocking=True)
                in_ready = self.s_in.record_event()
                mark(self.s_in, c, "in1")
            sc = self.s_cmp[c % len(self.s_cmp)]
            par = params[c % len(self.s_cmp)]
            with torch.cuda.stream(sc):
                sc.wait_event(fwd_ready)
                mark(sc, c, "cmp0")
                if copies_only:
                    sc.wait_event(in_ready)
                    fwd_done = sc.record_event()
                    y_out = buf["gy"][: hi - lo]
                    res = {"u": buf["u"][: hi - lo], "dt": buf["dt"][: hi - lo], "z": buf["z"][: hi - lo]}
                else:
                    leaves = [buf[k][: hi - lo].detach().requires_grad_(True) for k in ("u", "dt", "z")]
                    y = ops.ssm_adaptive_interface(leaves[0], leaves[1], par[0], par[1], par[2], par[3], par[4],
                                                   leaves[2], unitary=True)
                    fwd_done = sc.record_event()              # y can leave while the backward pass runs
                    sc.wait_event(in_ready)
                    y.backward(buf["gy"][: hi - lo])
                    y_out = y.detach()
                    res = {"u": leaves[0].grad, "dt": leaves[1].grad, "z": leaves[2].grad}
                done = sc.record_event()
                mark(sc, c, "cmp1")
                in_free[i] = done
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(fwd_done)
                mark(self.s_out, c, "out0")
                y_out.record_stream(self.s_out)
                outputs["y"][lo:hi].copy_(y_out, non_blocking=True)
                self.s_out.wait_event(done)
                for k, t in res.items():
                    t.record_stream(self.s_out)
                    outputs[k][lo:hi].copy_(t, non_blocking=True)
                mark(self.s_out, c, "out1")
                if copies_only:
                    # the copies out must finish before the next copy in reuses this buffer set
                    in_free[i] = self.s_out.record_event()
        with torch.cuda.stream(self.s_out):
            for sc in self.s_cmp:
                self.s_out.wait_stream(sc)
            for j, k in enumerate(_PARAMS):
                if copies_only:
                    outputs[k].copy_(params[0][j].detach(), non_blocking=True)
                    continue
                grads = [par[j].grad for par in params if par[j].grad is not None]
                for g in grads:
                    g.record_stream(self.s_out)
                total = grads[0] if len(grads) == 1 else grads[0] + grads[1]
                outputs[k].copy_(total, non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_in)
        mark(cur, -1, "end")
        self.kernel_launches_last_step = int(_lib.load().aussm_b200_kernel_launches() - launches0)
