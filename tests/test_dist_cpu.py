"""Collectives, point-to-point, object broadcast, multi-rank checkpoints and failure detection on CPU ranks (gloo)."""
import os

import pytest
import torch

from dist_utils import run_distributed


def body_collectives():
    import bmtrain_b200 as bmt
    from bmtrain_b200 import nccl

    rank, world = bmt.rank(), bmt.world_size()
    comm = bmt.config["comm"]
    # gather_result, also on a non-contiguous slice (test_synchronize)
    ref = torch.rand(world * 4, 6, generator=torch.Generator().manual_seed(0))
    part = ref[rank * 4:(rank + 1) * 4]
    assert torch.equal(bmt.gather_result(part), ref)
    assert torch.equal(bmt.gather_result(part[:, ::2]), ref[:, ::2])
    # autograd through all_reduce("prod") and reduce_scatter (test_nccl_backward)
    x = torch.tensor([float(rank + 2)], requires_grad=True)
    y = bmt.distributed.all_reduce(x, "prod")
    expect = 1.0
    for r in range(world):
        expect *= r + 2
    assert abs(y.item() - expect) < 1e-5
    y.backward()
    assert abs(x.grad.item() - expect / (rank + 2)) < 1e-5
    z = torch.arange(world * 2, dtype=torch.float32).view(world * 2, 1).clone().requires_grad_()
    out = bmt.distributed.reduce_scatter(z, "sum")
    assert torch.equal(out, z.detach()[rank * 2:(rank + 1) * 2] * world)
    out.sum().backward()
    assert torch.equal(z.grad, torch.ones_like(z))
    g = bmt.distributed.all_gather(torch.full((3,), float(rank), requires_grad=True))
    assert g.shape == (world, 3) and g[world - 1, 0].item() == world - 1
    b = bmt.distributed.broadcast(torch.full((2,), float(rank + 5)), world - 1)
    assert b[0].item() == world - 1 + 5
    for op, fn in (("max", max), ("min", min)):
        v = bmt.distributed.all_reduce(torch.tensor([float(rank)]), op)
        assert v.item() == fn(range(world))
    assert abs(bmt.sum_loss(torch.tensor(float(rank))).item() - (world - 1) / 2) < 1e-6
    # tensor-level API with the historical names
    t = torch.full((4,), float(rank + 1))
    o = torch.empty(4)
    nccl.allReduce(t, o, "sum", comm)
    assert o[0].item() == sum(range(1, world + 1))
    big = torch.empty(4 * world)
    nccl.allGather(t, big, comm)
    assert big[4 * (world - 1)].item() == world
    small = torch.empty(4)
    nccl.reduceScatter(big, small, "avg", comm)
    assert abs(small[0].item() - (rank + 1)) < 1e-6
    nccl.broadcast(t, o, 0, comm)
    assert o[0].item() == 1.0
    assert nccl.commCount(comm) == world and nccl.commRank(comm) == rank
    # point to point with and without cached shapes (test_send_recv)
    if world >= 2:
        nccl.groupStart()
        if rank == 0:
            nccl.send(torch.arange(5.0), 1, comm)
        elif rank == 1:
            r = torch.empty(5)
            nccl.recv(r, 0, comm)
        nccl.groupEnd()
        if rank == 1:
            assert torch.equal(r, torch.arange(5.0))
        for rep in range(2):
            if rank == 0:
                bmt.distributed.send_activations(torch.full((2, 3), 7.0 + rep, dtype=torch.float16), 1, comm, static=True).wait()
            elif rank == 1:
                got = bmt.distributed.recv_activations(0, comm, static=True)
                assert got.dtype == torch.float16 and got.shape == (2, 3) and got[0, 0].item() == 7.0 + rep
    # pickled objects (test_store)
    objs = bmt.store.allgather_objects({"rank": rank, "pad": "x" * rank})
    assert [o["rank"] for o in objs] == list(range(world))
    assert bmt.store.broadcast_object({"hello": rank}, comm, src=world - 1)["hello"] == world - 1
    sub = nccl.commInitRank(nccl.getUniqueId() if rank % 2 == 0 else nccl.getUniqueId(), 1, 0)
    assert sub.size == 1


@pytest.mark.parametrize("world", [2, 4])
def test_collectives_and_p2p(world):
    run_distributed("test_dist_cpu", "body_collectives", world)


def body_checkpoint(path):
    import bmtrain_b200 as bmt

    rank = bmt.rank()
    torch.manual_seed(0)

    class Net(bmt.DistributedModule):
        def __init__(self):
            super().__init__()
            self.emb = bmt.nn.Embedding(37, 12, dtype=torch.float32)
            self.layers = bmt.TransformerBlockList([bmt.Block(bmt.nn.Linear(12, 12, dtype=torch.float32)) for _ in range(3)])

        def forward(self, ids):
            return self.layers(self.emb(ids)).sum()

    net = Net()
    bmt.init_parameters(net)
    opt = bmt.optim.AdamOffloadOptimizer(net.parameters(), lr=1e-2)
    om = bmt.optim.OptimManager(loss_scale=None)
    om.add_optimizer(opt)
    ids = torch.randint(0, 37, (4, 5), generator=torch.Generator().manual_seed(rank))
    for _ in range(2):
        om.zero_grad(); om.backward(net(ids)); om.step()
    bmt.save(net, path)
    before = bmt.store._save_to_rank0(net)
    whole = om.state_dict(gather_opt=True)
    net2 = Net()
    res = bmt.load(net2, path)
    assert not res.missing_keys and not res.unexpected_keys
    after = bmt.store._save_to_rank0(net2)
    if rank == 0:
        plain = torch.load(path)
        assert list(plain.keys()) == ["emb.weight"] + [f"layers.{i}.{n}" for i in range(3) for n in ("weight", "bias")]
        assert plain["emb.weight"].shape == (37, 12)
        for k in before:
            assert torch.equal(before[k], after[k]) and torch.equal(before[k], plain[k])
    # resuming from the gathered (layout independent) optimizer state continues identically
    opt2 = bmt.optim.AdamOffloadOptimizer(net2.parameters(), lr=1e-2)
    om2 = bmt.optim.OptimManager(loss_scale=None)
    om2.add_optimizer(opt2)
    om2.load_state_dict(whole)
    for o, n in ((om, net), (om2, net2)):
        o.zero_grad(); o.backward(n(ids)); o.step()
    a, b = bmt.store._save_to_rank0(net), bmt.store._save_to_rank0(net2)
    if rank == 0:
        for k in a:
            assert torch.equal(a[k], b[k]), k
    stats = bmt.inspect.inspect_model(net, "*")
    assert len(stats) == 7 and stats[0]["shape"] == (37, 12)


def test_multi_rank_checkpoint_and_optimizer_gather(tmp_path):
    run_distributed("test_dist_cpu", "body_checkpoint", 2, path=str(tmp_path / "ckpt.pt"))


# ------------------------------------------------------------------------------------------------ failure detection
def body_rank_failure():
    """A rank that raises between steps: the survivor's next collective ends with an error within the group timeout."""
    import bmtrain_b200 as bmt

    if bmt.rank() == 1:
        raise RuntimeError("injected failure on rank 1")
    try:
        for _ in range(3):
            bmt.distributed.all_reduce(torch.ones(4))
    except Exception as exc:  # the collective reports the lost peer instead of hanging
        os._exit(17)
    os._exit(3)


def test_peer_failure_is_detected_not_hung():
    import torch.multiprocessing as mp
    from dist_utils import _worker, free_port

    ctx = mp.get_context("spawn")
    port = free_port()
    os.environ["BMT_TIMEOUT"] = "8"
    try:
        errq = ctx.Queue()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, "test_dist_cpu", "body_rank_failure", {}, {}, "cpu", errq))
                 for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(60)
        assert not any(p.is_alive() for p in procs), "a rank hung after its peer failed"
        assert procs[0].exitcode == 17, procs[0].exitcode
        assert procs[1].exitcode != 0
    finally:
        os.environ.pop("BMT_TIMEOUT", None)
        for p in procs:
            if p.is_alive():
                p.kill()


def body_heartbeat():
    """A rank whose heartbeat stops is reported by the others within the timeout, and forgiven when it comes back."""
    import time

    import bmtrain_b200 as bmt

    rank = bmt.rank()
    fired = []
    hb = bmt.watchdog.start(interval=0.1, timeout=0.8, on_failure=lambda lost: fired.extend(lost))
    time.sleep(0.5)
    bmt.watchdog.check()  # everybody alive
    if rank == 1:
        hb.pause()        # looks hung to the others; the process itself stays healthy
        time.sleep(3.0)
        hb.resume()
        time.sleep(1.0)
    else:
        deadline = time.time() + 5.0
        while not hb.lost_ranks() and time.time() < deadline:
            time.sleep(0.05)
        assert hb.lost_ranks() == [1], hb.lost_ranks()
        assert fired == [1]
        try:
            bmt.watchdog.check()
        except RuntimeError as exc:
            assert "rank(s) [1]" in str(exc)
        else:
            raise AssertionError("check() did not raise")
        deadline = time.time() + 6.0
        while hb.lost_ranks() and time.time() < deadline:
            time.sleep(0.05)
        assert hb.lost_ranks() == []  # rank 1 resumed
    x = torch.ones(1)
    assert float(bmt.distributed.all_reduce(x, "sum")) == bmt.world_size()
    # phases of a step, reduced as the maximum over ranks
    timer = bmt.utils.StepTimer()
    with timer.phase("a"):
        time.sleep(0.02 * (rank + 1))
    with timer.phase("b"):
        time.sleep(0.01)
    out = timer.finish_step()
    assert out["a"] >= 0.02 * bmt.world_size() * 1e3 * 0.9 and abs(out["total"] - out["a"] - out["b"]) < 30.0
    assert set(timer.averages()) == {"a", "b", "total"}


def test_heartbeat_and_step_timer():
    run_distributed("test_dist_cpu", "body_heartbeat", 2)


def body_shm():
    """The shared-memory transport against gloo on the same data: sizes below and above one slot, every dtype and op."""
    import bmtrain_b200 as bmt
    import torch.distributed as dist

    comm = bmt.config["comm"]
    r, W = comm.rank, comm.size
    g = torch.Generator().manual_seed(11 + r)
    for n in (1, 7, 1000, 3 * 1024 * 1024 + 5):
        for dtype in (torch.float32, torch.float64, torch.int32, torch.int64):
            x = (torch.randn(n, generator=g) * 4).to(dtype)
            for op in ("sum", "max", "min"):
                want = x.clone()
                dist.all_reduce(want, op={"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op], group=comm.group)
                got = x.clone()
                comm.all_reduce(got, op)
                assert comm._shm is not None
                if dtype.is_floating_point:
                    assert torch.allclose(got, want, rtol=1e-6, atol=1e-6), (n, dtype, op)
                else:
                    assert torch.equal(got, want), (n, dtype, op)
        x = torch.randn(n, generator=g)
        out = torch.empty(W * n)
        comm.all_gather_into(out, x)
        ref = [torch.empty(n) for _ in range(W)]
        dist.all_gather(ref, x, group=comm.group)
        assert torch.equal(out, torch.cat(ref))
        y = torch.randn(W * n, generator=g)
        part = torch.empty(n)
        comm.reduce_scatter_into(part, y, "sum")
        tot = y.clone()
        dist.all_reduce(tot, group=comm.group)
        assert torch.allclose(part, tot[r * n:(r + 1) * n], rtol=1e-5, atol=1e-5)
        b = torch.full((n,), float(r)).half()
        comm.broadcast(b, W - 1)
        assert float(b.float().min()) == float(b.float().max()) == W - 1
    h = torch.full((33,), 1.5, dtype=torch.bfloat16)
    comm.all_reduce(h, "avg")
    assert torch.all(h == 1.5)


def test_shared_memory_transport(monkeypatch):
    monkeypatch.setenv("BMT_CPU_COMM", "shm")
    run_distributed("test_dist_cpu", "body_shm", 3)
    # the engine on top of it: the ZeRO / checkpoint test body gives the same results as over gloo
    run_distributed("test_dist_cpu", "body_collectives", 2)
