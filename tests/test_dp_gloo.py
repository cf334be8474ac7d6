"""CPU tests of the data-parallel host logic with a world_size-2 gloo group: sharding M and
all-reducing grad_w reproduces the single-process result.  The per-shard compute is the CPU oracle
here (the product kernels need a GPU); what is under test is the sharding and the exchange step."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, M, K, N, bits, ret):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "appmult-aware-retraining_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lutgemm_dp import allreduce_grads_bucketed, allreduce_weight_grad, shard_rows
    from oracle import OracleC, oracle_np as O
    oc = OracleC(); oc.set_num_threads(2)
    lf, la, lw = O.to_wire(*O.synthetic_tables(bits, seed=0), bits)
    rng = np.random.default_rng(42)  # every rank draws the same full problem
    a = rng.integers(0, 1 << bits, (M, K)).astype(np.uint8)
    w = rng.integers(0, 1 << bits, (K, N)).astype(np.uint8)
    gc = rng.standard_normal((M, N)).astype(np.float32)
    lo, hi = shard_rows(M, rank, world)
    c = oc.forward(a[lo:hi], w, lf, bits) if hi > lo else np.zeros((0, N), np.uint32)
    if hi > lo:
        ga, gw = oc.backward(gc[lo:hi], a[lo:hi], w, la, lw, bits)
    else:
        ga, gw = np.zeros((0, K), np.float32), np.zeros((K, N), np.float32)
    gw_t = torch.from_numpy(gw.copy())
    work = allreduce_weight_grad(gw_t, async_op=True)
    work.wait()
    # bucketed averaging of parameter gradients
    p1, p2 = torch.nn.Parameter(torch.zeros(5, 3)), torch.nn.Parameter(torch.zeros(7))
    p1.grad = torch.full((5, 3), float(rank + 1)); p2.grad = torch.arange(7.0) * (rank + 1)
    ncoll = allreduce_grads_bucketed([p1, p2], bucket_bytes=32)
    if rank == 0:
        ret["ncoll"] = ncoll
        ret["p1"] = p1.grad.clone().numpy(); ret["p2"] = p2.grad.clone().numpy()
    ret[f"c{rank}"] = c; ret[f"ga{rank}"] = ga; ret[f"gw{rank}"] = gw_t.numpy().copy(); ret[f"range{rank}"] = (lo, hi)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("M", [37, 1, 64])
def test_m_sharding_with_gw_allreduce_matches_single_process(M):
    from oracle import OracleC, oracle_np as O
    world, K, N, bits = 2, 24, 19, 7
    port = 29500 + (os.getpid() + M) % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, M, K, N, bits, ret), nprocs=world, join=True)
        ret = dict(ret)
    oc = OracleC()
    lf, la, lw = O.to_wire(*O.synthetic_tables(bits, seed=0), bits)
    rng = np.random.default_rng(42)
    a = rng.integers(0, 1 << bits, (M, K)).astype(np.uint8)
    w = rng.integers(0, 1 << bits, (K, N)).astype(np.uint8)
    gc = rng.standard_normal((M, N)).astype(np.float32)
    c_full = oc.forward(a, w, lf, bits)
    ga_full, gw_full = oc.backward(gc, a, w, la, lw, bits)
    assert ret["range0"][0] == 0 and ret["range0"][1] == ret["range1"][0] and ret["range1"][1] == M
    assert np.array_equal(np.concatenate([ret["c0"], ret["c1"]]), c_full)
    assert np.array_equal(np.concatenate([ret["ga0"], ret["ga1"]]), ga_full)  # rows are independent
    for r in range(world):  # every rank ends with the same, complete weight gradient
        assert np.abs(ret[f"gw{r}"] - gw_full).max() <= 1e-5 * max(np.abs(gw_full).max(), 1e-30)
    assert np.array_equal(ret["gw0"], ret["gw1"])
    assert ret["ncoll"] == 2 and np.allclose(ret["p1"], 1.5) and np.allclose(ret["p2"], np.arange(7.0) * 1.5)


def test_shard_rows_partitions():
    from lutgemm_dp import shard_rows
    for M in (0, 1, 7, 8, 1000):
        for world in (1, 2, 3, 8):
            spans = [shard_rows(M, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == M
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_rows(4, 2, 2)


def _hook_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "appmult-aware-retraining_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lutgemm_dp import OverlappedGradReducer
    torch.manual_seed(0)  # same initial weights on every rank
    model = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh(), torch.nn.Linear(8, 5), torch.nn.Tanh(),
                                torch.nn.Linear(5, 3))
    reducer = OverlappedGradReducer(model.parameters(), bucket_bytes=200)  # several buckets
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    steps = []
    for step in range(3):
        x = torch.randn(4, 6, generator=torch.Generator().manual_seed(10 * step + rank))
        if step == 1:
            opt.zero_grad(set_to_none=True)  # a caller that detaches .grad from the buffer is folded back in
        else:
            reducer.zero_grad()
        model(x).square().sum().backward()
        local = [p.grad.clone() for p in model.parameters()]  # not yet final: collectives may be in flight
        ncoll = reducer.finish()
        steps.append((ncoll, [p.grad.clone().numpy() for p in model.parameters()]))
        assert all(p.grad.data_ptr() >= reducer.flat.data_ptr() for p in model.parameters())
        opt.step()
    # reference: the same three steps with gradients averaged by plain per-tensor all-reduce
    torch.manual_seed(0)
    model2 = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh(), torch.nn.Linear(8, 5), torch.nn.Tanh(),
                                 torch.nn.Linear(5, 3))
    opt2 = torch.optim.SGD(model2.parameters(), lr=0.1)
    want = []
    for step in range(3):
        x = torch.randn(4, 6, generator=torch.Generator().manual_seed(10 * step + rank))
        opt2.zero_grad(set_to_none=True)
        model2(x).square().sum().backward()
        for p in model2.parameters():
            dist.all_reduce(p.grad)
            p.grad.div_(world)
        want.append([p.grad.clone().numpy() for p in model2.parameters()])
        opt2.step()
    ret[f"steps{rank}"] = steps
    ret[f"want{rank}"] = want
    ret[f"buckets{rank}"] = len(reducer.buckets)
    reducer.close()
    dist.barrier()
    dist.destroy_process_group()


def test_overlapped_grad_reducer_matches_per_tensor_allreduce():
    """Hook-driven bucketed all-reduce into the persistent flat gradient buffer (world size 2, gloo) against a
    plain per-tensor all-reduce after backward, over three optimizer steps."""
    world = 2
    port = 31500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_hook_worker, args=(world, port, ret), nprocs=world, join=True)
        ret = dict(ret)
    assert ret["buckets0"] >= 2
    for r in range(world):
        for (ncoll, got), want in zip(ret[f"steps{r}"], ret[f"want{r}"]):
            assert ncoll == ret["buckets0"]
            for g_, w_ in zip(got, want):
                assert np.allclose(g_, w_, rtol=1e-6, atol=1e-7)
    for (_, g0), (_, g1) in zip(ret["steps0"], ret["steps1"]):  # both ranks hold the same averaged gradients
        for a_, b_ in zip(g0, g1):
            assert np.array_equal(a_, b_)
