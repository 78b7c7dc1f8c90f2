"""Data-parallel training step for the end-to-end benchmark configurations.

    python -m aussm_b200.train --config 3 [--steps K] [--warmup W]            (one GPU)
    python -m torch.distributed.run --nproc-per-node N -m aussm_b200.train --config 4 --micro-batch 1

config 3: SSMTS, layers 'a|m|a|m', d_model 128, d_state 16, input/output dim 21, seq 720, global batch 64,
          MSE against N(0,1) targets (the reference's regression task, task/sequence_mse_regression.py:119-168)
config 4: SSMSequenceClassifier, six AUSSM blocks, d_model 512, d_state 16, vocab 256, seq 65536, global batch 32,
          10-class cross-entropy (task/sequence_classification.py:94-125)

One process per GPU; the batch is sharded over ranks, the scan needs no communication, and the only collective
is the all-reduce of the weight gradients (NCCL over NVLink), done here on flat buckets after the backward pass.
Synthetic seeded data and random-init weights stand in for the datasets (none ships with the reference).
"""
from __future__ import annotations

import argparse
import json
import math
import os
from typing import Iterable, List

import torch
import torch.distributed as dist

__all__ = ["shard_range", "allreduce_gradients", "max_over_ranks", "make_config", "train_step", "GraphedTrainStep"]


def shard_range(total: int, rank: int, world: int):
    """Contiguous shard [lo, hi) of `total` items for `rank`; the first total % world ranks get one more."""
    base, rem = divmod(total, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def allreduce_gradients(params: Iterable[torch.nn.Parameter], world: int, bucket_bytes: int = 64 << 20,
                        group=None, average: bool = True) -> int:
    """Sum the gradients over ranks with one all-reduce per flat bucket and, with ``average``, divide by the
    number of ranks; returns the number of collectives.  Parameters without a gradient contribute zeros, so
    that every rank issues the same collectives."""
    if world <= 1:
        return 0
    params = [p for p in params if p.requires_grad]
    calls = 0
    bucket: List[torch.nn.Parameter] = []
    size = 0

    def flush():
        nonlocal bucket, size, calls
        if not bucket:
            return
        flats = []
        for p in bucket:
            g = p.grad if p.grad is not None else torch.zeros_like(p)
            flats.append(torch.view_as_real(g).reshape(-1) if g.is_complex() else g.reshape(-1))
        flat = torch.cat([f.float() for f in flats])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= world
        off = 0
        for p, f in zip(bucket, flats):
            n = f.numel()
            piece = flat[off:off + n]
            off += n
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            if p.grad.is_complex():
                p.grad.copy_(torch.view_as_complex(piece.view(-1, 2)).view_as(p.grad))
            else:
                p.grad.copy_(piece.view_as(p.grad))
        calls += 1
        bucket, size = [], 0

    for p in params:
        nbytes = p.numel() * p.element_size()
        if size and size + nbytes > bucket_bytes:
            flush()
        bucket.append(p)
        size += nbytes
    flush()
    return calls


def max_over_ranks(value: float, device, world: int) -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def make_config(config: int, device, rank: int, world: int, scale: float = 1.0):
    """Model, a data generator for this rank's shard, and the loss of one benchmark configuration."""
    from .models import SSMTS, SSMSequenceClassifier
    torch.manual_seed(1234)                       # identical initial weights on every rank
    if config == 3:
        gb, l, dim = 64, max(16, int(720 * scale)), 21
        model = SSMTS(d_model=128, input_dim=dim, output_dim=dim, layers="a|m|a|m", d_state=16).to(device)
        lo, hi = shard_range(gb, rank, world)
        g = torch.Generator(device="cpu").manual_seed(99 + rank)

        def batch():
            t = torch.arange(l, dtype=torch.float32)[None, :, None]
            period = torch.randint(4, 169, (hi - lo, 1, dim), generator=g).float()
            x = torch.randn(hi - lo, l, dim, generator=g) + torch.sin(2 * math.pi * t / period)
            return x.to(device), torch.randn(hi - lo, l, dim, generator=g).to(device)

        loss_fn = lambda out, y: torch.mean((out - y) ** 2)
        tokens = gb * l
    elif config == 4:
        gb, l = 32, max(64, int(65536 * scale))
        model = SSMSequenceClassifier(d_model=512, vocab_size=256, output_dim=10, layers="a|a|a|a|a|a",
                                      d_state=16).to(device)
        lo, hi = shard_range(gb, rank, world)
        g = torch.Generator(device="cpu").manual_seed(99 + rank)

        def batch():
            return (torch.randint(0, 256, (hi - lo, l), generator=g).to(device),
                    torch.randint(0, 10, (hi - lo,), generator=g).to(device))

        loss_fn = torch.nn.functional.cross_entropy
        tokens = gb * l
    else:
        raise ValueError("config must be 3 or 4")
    return model, batch, loss_fn, tokens, hi - lo, gb


def train_step(model, opt, x, y, loss_fn, world: int, micro_batch: int = 0, clip: float = 1.0,
               global_batch: int = 0):
    """Forward, backward (optionally in micro-batches that accumulate gradients), gradient all-reduce,
    clipping at `clip` (the reference's gradient_clip_val, experiments/all/weather.yaml:63) and optimizer step.

    Every sample weighs 1 / global_batch in the loss whatever shard it is in, and the ranks' gradients are
    summed: the result equals the single-process gradient of the mean loss also when the shards are uneven
    (global batch not divisible by the number of ranks).  ``global_batch = 0`` means local batch x world."""
    opt.zero_grad(set_to_none=True)
    n = x.shape[0]
    gb = global_batch if global_batch > 0 else n * world
    mb = n if micro_batch <= 0 else min(micro_batch, n)
    total = 0.0
    for s in range(0, n, mb):
        out = model(x[s:s + mb])
        loss = loss_fn(out, y[s:s + mb]) * (min(s + mb, n) - s) / gb
        loss.backward()
        total += float(loss.detach())
    from . import ops
    if ops.check_device_status and x.is_cuda:
        ops._poll_status("train_step", x.device)
    ncoll = allreduce_gradients(model.parameters(), world, average=False)
    torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
    opt.step()
    return total, ncoll


class GraphedTrainStep:
    """One-process training step (forward, backward in micro-batches, clipping, optimizer) of a fixed-shape batch,
    captured once into a CUDA graph and replayed.

    The small configurations are bound by the host: a step of configuration 3 is several hundred kernels of a few
    microseconds each, and the Python and launch overhead between them is most of its time.  The operators take
    their workspaces from the caller's allocator and never synchronise, so the whole step records into one graph.
    The optimizer must be built with ``capturable=True``.  ``step(x, y)`` copies a new batch of the same shape
    into the static inputs, replays the graph and returns the loss as a device tensor (reading it synchronises).
    With more than one rank the gradient all-reduce sits between backward and clipping; that variant is not
    captured here: use ``train_step``."""

    def __init__(self, model, opt, x, y, loss_fn, micro_batch: int = 0, clip: float = 1.0, global_batch: int = 0,
                 warmup: int = 3):
        from . import ops
        self.model, self.opt, self.loss_fn, self.clip = model, opt, loss_fn, clip
        self.x, self.y = x.clone(), y.clone()
        n = x.shape[0]
        self.gb = global_batch if global_batch > 0 else n
        self.mb = n if micro_batch <= 0 else min(micro_batch, n)
        saved = ops.keep_phases
        if saved == "auto":
            ops.keep_phases = True          # the free-memory query of "auto" is not a call to make while capturing
        try:
            cur = torch.cuda.current_stream()
            side = torch.cuda.Stream()
            side.wait_stream(cur)
            with torch.cuda.stream(side):   # warm-up off the capturing stream: lazy initialisation, allocator state
                for _ in range(max(1, warmup)):
                    opt.zero_grad(set_to_none=True)
                    self._body()
            cur.wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            opt.zero_grad(set_to_none=True)
            with torch.cuda.graph(self.graph):
                self.loss = self._body()
        finally:
            ops.keep_phases = saved

    def _body(self):
        n = self.x.shape[0]
        total = torch.zeros((), device=self.x.device)
        for s in range(0, n, self.mb):
            out = self.model(self.x[s:s + self.mb])
            loss = self.loss_fn(out, self.y[s:s + self.mb]) * ((min(s + self.mb, n) - s) / self.gb)
            loss.backward()
            total = total + loss.detach()
        torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.clip, foreach=True)
        self.opt.step()
        return total

    def step(self, x=None, y=None):
        if x is not None:
            self.x.copy_(x, non_blocking=True)
        if y is not None:
            self.y.copy_(y, non_blocking=True)
        self.graph.replay()
        return self.loss


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=3)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--scale", type=float, default=1.0, help="shrinks the sequence length (smoke runs)")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    model, batch, loss_fn, tokens, local_batch, gb = make_config(a.config, dev, rank, world, a.scale)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    x, y = batch()
    for _ in range(a.warmup):
        train_step(model, opt, x, y, loss_fn, world, a.micro_batch, global_batch=gb)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    loss = ncoll = 0
    for _ in range(a.steps):
        loss, ncoll = train_step(model, opt, x, y, loss_fn, world, a.micro_batch, global_batch=gb)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = max_over_ranks(e0.elapsed_time(e1) / a.steps, dev, world)
    if rank == 0:
        print(json.dumps({"config": a.config, "n_gpus": world, "ms_per_step": ms, "tokens_per_s": tokens / ms * 1e3,
                          "global_batch": gb, "local_batch": local_batch, "loss": loss,
                          "allreduce_calls_per_step": ncoll, "micro_batch": a.micro_batch, "scale": a.scale,
                          "parameters": sum(p.numel() for p in model.parameters()), "data": "synthetic"}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
