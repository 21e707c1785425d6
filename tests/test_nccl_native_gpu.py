"""The C++ NCCL wrapper (non-blocking communicators, error polling, abort) on one and two GPUs."""
import pytest
import torch

from dist_utils import run_distributed

pytestmark = pytest.mark.gpu


def test_native_communicator_single_rank(bmt_gpu):
    from bmtrain_b200.nccl import native

    if native.lib() is None:
        pytest.skip("_nccl.so not built")
    assert native.lib().bmt_nccl_version() >= 21400
    comm = native.NativeCommunicator([0], 0, name="solo", watchdog_ms=20)
    x = torch.arange(1024, device="cuda", dtype=torch.float32)
    comm.all_reduce(x, "sum")
    out = torch.empty(1024, device="cuda")
    comm.all_gather_into(out, x)
    comm.reduce_scatter_into(out, x, "max")
    torch.cuda.synchronize()
    assert torch.equal(out, torch.arange(1024, device="cuda", dtype=torch.float32))
    assert comm.async_error() == 0
    comm.check()
    comm.abort()
    assert comm.async_error() == -2000
    with pytest.raises(native.NCCLError):
        comm.all_reduce(x)
    comm.destroy()


def body_native_pair():
    import bmtrain_b200 as bmt
    from bmtrain_b200.nccl import native

    world = bmt.config["comm"]
    comm = native.from_communicator(world, watchdog_ms=50)
    r, n = comm.rank, comm.size
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        x = (torch.arange(4096, device="cuda") % 97 + r).to(dtype)
        y = x.clone()
        comm.all_reduce(y, "sum")
        ref = x.clone()
        world.all_reduce(ref, "sum")
        assert torch.equal(y, ref)
        g = torch.empty(n * 4096, device="cuda", dtype=dtype)
        comm.all_gather_into(g, x)
        g2 = torch.empty_like(g)
        world.all_gather_into(g2, x)
        assert torch.equal(g, g2)
        s = torch.empty(4096 // n, device="cuda", dtype=dtype)
        comm.reduce_scatter_into(s, x, "sum")
        s2 = torch.empty_like(s)
        world.reduce_scatter_into(s2, x, "sum")
        assert torch.equal(s, s2)
    b = torch.full((16,), float(r), device="cuda")
    comm.broadcast(b, root=1)
    assert float(b[0]) == 1.0
    msg = torch.full((32,), 7.0 + r, device="cuda")
    if r == 0:
        comm.send(msg, 1)
    elif r == 1:
        got = torch.empty(32, device="cuda")
        comm.recv(got, 0)
        torch.cuda.synchronize()
        assert float(got[0]) == 7.0
    comm.barrier()
    assert comm.async_error() == 0
    comm.destroy()


def test_native_communicator_2gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from bmtrain_b200.nccl import native

    if native.lib() is None:
        pytest.skip("_nccl.so not built")
    run_distributed("test_nccl_native_gpu", "body_native_pair", 2, device="cuda")
