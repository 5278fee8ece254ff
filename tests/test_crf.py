"""The chain/tree driver of benchmark configuration 4 (linear-chain CRF log-partition)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def cpu_bmm(a, b):
    return oracle.expr_forward(0, a, b)


@pytest.mark.parametrize("B,L,C", [(2, 1, 3), (2, 2, 4), (3, 7, 5), (2, 8, 3), (1, 13, 4), (2, 15, 3), (1, 31, 2)])
def test_tree_equals_sequential_chain_on_cpu(B, L, C):
    from genbmm_b200 import crf
    gen = torch.Generator().manual_seed(B * 100 + L)
    pot = torch.randn(B, L, C, C, generator=gen, dtype=torch.float64)
    logz, marg = crf.marginals(pot, bmm=cpu_bmm)
    want_z, want_m = oracle.crf_log_partition(pot)
    assert torch.allclose(logz, want_z, rtol=1e-10, atol=1e-10)
    assert torch.allclose(marg, want_m, rtol=1e-8, atol=1e-10)
    assert torch.allclose(marg.sum((2, 3)), torch.ones(B, L, dtype=torch.float64))


@pytest.mark.parametrize("L,C", [(1, 3), (2, 4), (13, 5), (40, 7)])
def test_alpha_beta_recursions_equal_autograd_of_the_chain_product(L, C):
    """The memory-light float64 checker used at the full benchmark size against the autograd one."""
    gen = torch.Generator().manual_seed(L * 10 + C)
    pot = torch.randn(2, L, C, C, generator=gen, dtype=torch.float64)
    want_z, want_m = oracle.crf_log_partition(pot)
    for b in range(2):
        z, m = oracle.crf_alpha_beta(pot[b])
        assert abs(z - float(want_z[b])) <= 1e-12 * max(1.0, abs(z))
        assert np.allclose(m, want_m[b].numpy(), rtol=1e-10, atol=1e-14)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from genbmm_b200 import crf
    gen = torch.Generator().manual_seed(7)
    pot = torch.randn(2, 12, 4, 4, generator=gen, dtype=torch.float64)
    want_z, want_m = oracle.crf_log_partition(pot)
    lo, hi = rank * 12 // world, (rank + 1) * 12 // world
    chunk = pot[:, lo:hi].clone().requires_grad_(True)
    logz = crf.sharded_log_partition(chunk, bmm=cpu_bmm)
    grad, = torch.autograd.grad(logz.sum(), chunk)
    ok = torch.allclose(logz, want_z, rtol=1e-10, atol=1e-10) and torch.allclose(grad, want_m[:, lo:hi], rtol=1e-8,
                                                                                    atol=1e-10)
    q.put((rank, bool(ok)))
    dist.destroy_process_group()


def test_chain_chunk_sharding_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True), (1, True)]


@pytest.mark.gpu
@pytest.mark.parametrize("B,L,C", [(2, 7, 5), (3, 16, 33), (2, 31, 64)])
def test_crf_on_gpu_matches_oracle(B, L, C):
    from genbmm_b200 import crf
    gen = torch.Generator().manual_seed(3)
    pot = torch.randn(B, L, C, C, generator=gen)
    logz, marg = crf.marginals(pot.cuda())
    want_z, want_m = oracle.crf_log_partition(pot)
    assert np.allclose(logz.cpu().numpy(), want_z.numpy(), rtol=1e-5, atol=1e-5)
    assert np.allclose(marg.cpu().numpy(), want_m.numpy(), rtol=2e-4, atol=1e-7)


@pytest.mark.gpu
def test_config4_full_size_properties():
    """T=512, C=256, B=16: potentials (16,511,256,256).  Checked against the float64 chain on one
    batch element's log-partition and through properties of the marginals at full size."""
    from genbmm_b200 import crf
    gen = torch.Generator().manual_seed(3)
    pot = torch.randn(16, 511, 256, 256, generator=gen)
    logz, marg = crf.marginals(pot.cuda())
    # sequential float64 chain for one element (forward only, numpy): alpha_t = alpha_{t-1} (x) pot_t
    p = pot[0].double().numpy()
    alpha = p[0]
    for t in range(1, 511):
        s = alpha[:, :, None] + p[t][None, :, :]
        m = s.max(1)
        alpha = m + np.log(np.exp(s - m[:, None, :]).sum(1))
    want = np.log(np.exp(alpha - alpha.max()).sum()) + alpha.max()
    assert abs(float(logz[0]) - want) <= 1e-5 * abs(want)
    # every position's edge marginals are a distribution over (i, j)
    sums = marg.sum((2, 3))
    assert torch.allclose(sums, torch.ones_like(sums), rtol=0, atol=2e-3)
    assert (marg >= 0).all()
    # consecutive positions agree on the state marginal they share
    right = marg[:, :-1].sum(2)     # state at the right end of edge t
    left = marg[:, 1:].sum(3)       # state at the left end of edge t+1
    assert torch.allclose(right, left, rtol=0, atol=2e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("B,L,C", [(2, 15, 64), (2, 63, 256)])
def test_graphed_marginals_replay_matches_eager(B, L, C):
    """One capture, two replays on different potentials: each must reproduce the eager driver."""
    from genbmm_b200 import crf
    run = crf.GraphedMarginals((B, L, C, C), "cuda")
    gen = torch.Generator().manual_seed(11)
    for _ in range(2):
        pot = torch.randn(B, L, C, C, generator=gen).cuda()
        logz, marg = run(pot)
        want_z, want_m = crf.marginals(pot)
        assert torch.allclose(logz, want_z, rtol=1e-6, atol=0)
        assert torch.allclose(marg, want_m, rtol=1e-5, atol=1e-9)
    with pytest.raises(RuntimeError):
        run(torch.zeros(B, L + 1, C, C, device="cuda"))


@pytest.mark.gpu
def test_sharded_log_partition_over_nccl_on_cuda_tensors():
    """The chain-chunk path with its NCCL all-gather carrying CUDA tensors (a one-rank group: the collective,
    its autograd node and the redundant upper levels all run; with one rank the result must equal the unsharded
    driver), forward and gradient."""
    from genbmm_b200 import crf
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        gen = torch.Generator().manual_seed(5)
        pot = torch.randn(3, 31, 128, 128, generator=gen).cuda()
        x = pot.clone().requires_grad_(True)
        logz = crf.sharded_log_partition(x)
        grad, = torch.autograd.grad(logz.sum(), x)
        want_z, want_m = crf.marginals(pot)
        assert torch.allclose(logz, want_z, rtol=1e-6, atol=0)
        assert torch.allclose(grad, want_m, rtol=1e-5, atol=1e-9)
        oz, om = oracle.crf_alpha_beta(pot[1].cpu())
        assert abs(float(logz[1].detach()) - oz) <= 1e-5 * abs(oz)
        assert np.allclose(grad[1].cpu().numpy(), om, rtol=2e-4, atol=1e-9)
    finally:
        dist.destroy_process_group()
