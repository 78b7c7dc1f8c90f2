"""Host-side logic of the multi-GPU path, run as two gloo ranks on the CPU:
batch sharding, flat-bucket gradient all-reduce (real and complex parameters,
parameters without a gradient), max-over-ranks timing."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aussm_b200.train import allreduce_gradients, max_over_ranks, shard_range, train_step


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        params = [torch.nn.Parameter(torch.zeros(5, 3)), torch.nn.Parameter(torch.zeros(4, dtype=torch.complex64)),
                  torch.nn.Parameter(torch.zeros(7)), torch.nn.Parameter(torch.zeros(2, 2))]
        g = torch.Generator().manual_seed(100 + rank)
        params[0].grad = torch.randn(5, 3, generator=g)
        params[1].grad = torch.complex(torch.randn(4, generator=g), torch.randn(4, generator=g))
        params[2].grad = torch.randn(7, generator=g) if rank == 0 else None      # missing on rank 1
        params[3].grad = torch.randn(2, 2, generator=g)
        mine = [None if p.grad is None else p.grad.clone() for p in params]
        calls = allreduce_gradients(params, world, bucket_bytes=64)             # small buckets: several collectives
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        for i, p in enumerate(params):
            parts = [torch.zeros_like(p.grad) if gathered[r][i] is None else gathered[r][i] for r in range(world)]
            torch.testing.assert_close(p.grad, sum(parts) / world)
        slow = max_over_ranks(10.0 + rank, torch.device("cpu"), world)
        ret[rank] = (calls, slow)
    finally:
        dist.destroy_process_group()


def test_two_rank_gradient_allreduce_and_timing():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert ret[0][0] == ret[1][0] and ret[0][0] >= 2
        assert ret[0][1] == ret[1][1] == 11.0


def test_shards_cover_the_batch_without_overlap():
    for total in (1, 7, 16, 64):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _uneven_worker(rank, world, port, ret):
    """Three ranks share a global batch of 7 (shards of 3, 2, 2): the reduced gradient of one step must equal
    the single-process gradient of the mean loss over all 7 samples."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gb = 7
        g = torch.Generator().manual_seed(5)
        x, y = torch.randn(gb, 4, generator=g), torch.randn(gb, 2, generator=g)
        torch.manual_seed(3)
        model = torch.nn.Linear(4, 2)
        single = torch.nn.Linear(4, 2)
        single.load_state_dict(model.state_dict())
        loss_fn = lambda out, t: torch.mean((out - t) ** 2)
        torch.mean((single(x) - y) ** 2).backward()
        lo, hi = shard_range(gb, rank, world)

        class NoStep:                      # keep the weights: only the gradient is compared
            def zero_grad(self, set_to_none=True):
                model.zero_grad(set_to_none=set_to_none)

            def step(self):
                pass

        train_step(model, NoStep(), x[lo:hi], y[lo:hi], loss_fn, world, micro_batch=2, clip=1e9, global_batch=gb)
        for p, q in zip(model.parameters(), single.parameters()):
            torch.testing.assert_close(p.grad, q.grad, rtol=1e-5, atol=1e-6)
        ret[rank] = hi - lo
    finally:
        dist.destroy_process_group()


def test_uneven_shards_give_the_single_process_gradient():
    world = 3
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_uneven_worker, args=(world, port, ret), nprocs=world, join=True)
        assert sorted(ret.values()) == [2, 2, 3]
