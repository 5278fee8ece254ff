"""The N>1 path on CPU: two gloo ranks shard the batch, compute their slice and all-gather.
The per-shard op is the oracle's broadcast expression (the CUDA kernels need a GPU); what is
tested is the sharding and gathering logic that bench.py --gpus N and callers rely on."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from genbmm_b200 import sharded
    gen = torch.Generator().manual_seed(0)
    a = torch.rand(batch, 6, 5, generator=gen)
    b = torch.rand(batch, 5, 4, generator=gen)
    full = oracle.expr_forward(0, a, b)
    got = sharded.sharded_apply(lambda x, y: oracle.expr_forward(0, x, y), a, b)
    lo, hi = sharded.shard_bounds(batch, rank, world)
    ok = torch.equal(got, full) and sharded.shard_batch(a).shape[0] == hi - lo
    out_q.put((rank, bool(ok), lo, hi))
    dist.destroy_process_group()


def _run(world, batch):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, batch, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    return res


def test_two_ranks_even_and_ragged_batches():
    for batch in (8, 5):
        res = _run(2, batch)
        assert all(ok for _, ok, _, _ in res)
        assert res[0][2] == 0 and res[0][3] == res[1][2] and res[1][3] == batch


def test_shard_bounds_cover_the_batch():
    from genbmm_b200.sharded import shard_bounds
    for batch in (0, 1, 7, 8, 64):
        for world in (1, 2, 4, 8):
            spans = [shard_bounds(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
