"""Multi-GPU paths (2 B200s, one process per GPU, NCCL + peer memory).  Skipped with fewer than two GPUs."""
import pytest
import torch

from dist_utils import run_distributed

pytestmark = pytest.mark.gpu


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def body_fused_rs(fused: bool):
    """ZeRO-3 training of a small fp16 GPT on 2 ranks: gradients through the fused NVLink reduce-scatter must match
    the NCCL path and a single-process fp32 oracle."""
    import os

    import bmtrain_b200 as bmt
    from bmtrain_b200.parallel import symm
    from oracle import OracleGPT
    from bmtrain_b200.store import _save_to_rank0

    rank, world = bmt.rank(), bmt.world_size()
    cfg = dict(num_layers=3, vocab=2048, d=256, dh=64, h=4, dff=1024, max_distance=128)
    torch.manual_seed(7)
    ref = OracleGPT(cfg["num_layers"], cfg["vocab"], cfg["d"], cfg["dh"], cfg["h"], cfg["dff"], cfg["max_distance"], activation="gelu")
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, 0.02)
        for blk in ref.transformers:
            blk.ln_attn.weight.add_(1.0)
            blk.ln_ff.weight.add_(1.0)
        ref.layernorm.weight.add_(1.0)
    model = bmt.models.GPT(cfg["num_layers"], cfg["vocab"], cfg["d"], cfg["dh"], cfg["h"], cfg["dff"], cfg["max_distance"],
                           dtype=torch.float16, activation="gelu")
    model.load_state_dict(ref.state_dict())
    assert symm.peer_runtime(bmt.config["zero_comm"]) is not None or not fused
    loss_fn = bmt.loss.FusedCrossEntropy()
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, cfg["vocab"], (2, 65), generator=g).cuda()
    all_ids = [torch.randint(0, cfg["vocab"], (2, 65), generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
    pos = torch.arange(64, device="cuda")[None].expand(2, -1).contiguous()
    mask = torch.ones(2, 64, dtype=torch.bool, device="cuda")
    scale = 1024.0
    for it in range(2):  # second pass: gradient accumulation on top of the first
        logits = model(ids[:, :-1].contiguous(), pos, mask)
        loss = loss_fn(logits.view(-1, logits.shape[-1]), ids[:, 1:].contiguous().view(-1))
        (loss * scale / world).backward()
    bmt.synchronize()
    from bmtrain_b200.parallel import fused_ops
    if fused:
        # first block in forward and last block in backward were not prefetched: their QKV weight came through the fused kernel
        assert fused_ops.calls["zero_gather_gemm"] == 4, fused_ops.calls
    for rt in symm._runtimes.values():
        if rt is not None:
            rt.check()
            assert int(rt.overflow.item()) == 0
    # oracle gradients: mean over ranks, two accumulated passes
    for r in range(world):
        rid = all_ids[r]
        lg = ref(rid[:, :-1], pos.cpu(), mask.cpu())
        l = torch.nn.functional.cross_entropy(lg.view(-1, cfg["vocab"]), rid[:, 1:].reshape(-1))
        (l * 2 / world).backward()
    got = {r["name"]: r for r in bmt.inspect.inspect_model(model, "*")}
    for name, p in ref.named_parameters():
        key = name
        ref_std = (p.grad * scale).std().item()
        assert abs(got[key]["grad_std"] - ref_std) <= 0.03 * ref_std + 1e-4, (name, got[key]["grad_std"], ref_std)


@pytest.mark.parametrize("fused", [True, False])
def test_zero3_fused_reduce_scatter_2gpu(fused, monkeypatch):
    _need(2)
    monkeypatch.setenv("BMT_PEER", "1" if fused else "0")
    monkeypatch.setenv("BMT_FUSED_GATHER", "1")  # exercise the fused gather in forward as well (default: backward only)
    run_distributed("test_multi_gpu", "body_fused_rs", 2, device="cuda", fused=fused)


def body_tp_fused():
    """Fused all-gather->GEMM and GEMM->reduce-scatter against NCCL + plain GEMM on the same data (2 ranks)."""
    import bmtrain_b200 as bmt
    from bmtrain_b200.ops import gemm as G
    from bmtrain_b200.parallel import fused_ops, symm

    comm = bmt.config["comm"]
    rank, W = comm.rank, comm.size
    rt = symm.peer_runtime(comm)
    assert rt is not None
    for dtype in (torch.float16, torch.bfloat16):
        tol = 2e-2 if dtype == torch.bfloat16 else 3e-3
        for (m, K, N) in ((256, 512, 1024), (1024, 2560, 3840), (128, 8192, 2560)):
            for rep in range(3):  # ring of two buffers: the third call reuses the first slot
                torch.manual_seed(1000 * rep + rank)
                x_local = torch.randn(m, K, device="cuda", dtype=dtype)
                torch.manual_seed(5)
                w = (torch.randn(N, K, device="cuda") * 0.05).to(dtype)
                bias = torch.randn(N, device="cuda").to(dtype)
                x_all = torch.empty(W * m, K, device="cuda", dtype=dtype)
                comm.all_gather_into(x_all, x_local)
                ref = G.gemm_nt(x_all, w, bias).float()
                got = fused_ops.ag_gemm(x_local, w, bias, comm, False, True)
                assert got is not None
                out, gathered = got
                assert torch.equal(gathered, x_all)
                assert ((out.float() - ref).abs().max() / ref.abs().max()).item() < tol
                # GEMM -> reduce-scatter: every rank holds different activations, same weight
                xs = torch.randn(W * m, K, device="cuda", dtype=dtype)
                full = G.gemm_nt(xs, w).float()
                comm.all_reduce(full, "sum")
                ref_rs = full[rank * m:(rank + 1) * m] + bias.float()
                got_rs = fused_ops.gemm_rs(xs, w, bias, comm, False)
                assert got_rs is not None
                assert ((got_rs.float() - ref_rs).abs().max() / ref_rs.abs().max()).item() < tol, (m, K, N, rep)
                # K x N weight layout (dgrad form)
                wkn = (torch.randn(K, N, device="cuda") * 0.05).to(dtype) if rank >= 0 else None
                torch.manual_seed(6)
                wkn = (torch.randn(K, N, device="cuda") * 0.05).to(dtype)
                full = G.gemm_nn(xs, wkn).float()
                comm.all_reduce(full, "sum")
                got_kn = fused_ops.gemm_rs(xs, wkn, None, comm, True)
                assert ((got_kn.float() - full[rank * m:(rank + 1) * m]).abs().max() / full.abs().max()).item() < tol
    # same activation shape feeding weights of different widths and layouts back to back (the projections of one
    # transformer block): every combination keeps its own buffers and counters
    torch.manual_seed(77 + rank)
    x_local = torch.randn(256, 1024, device="cuda", dtype=torch.bfloat16)
    x_all = torch.empty(W * 256, 1024, device="cuda", dtype=torch.bfloat16)
    comm.all_gather_into(x_all, x_local)
    torch.manual_seed(8)
    ws = [(torch.randn(n, 1024, device="cuda") * 0.05).to(torch.bfloat16) for n in (512, 4096, 1536)]
    wk = (torch.randn(1024, 2048, device="cuda") * 0.05).to(torch.bfloat16)
    for rep in range(3):
        for w in ws:
            out = fused_ops.ag_gemm(x_local, w, None, comm, False, False)
            ref = G.gemm_nt(x_all, w).float()
            assert ((out.float() - ref).abs().max() / ref.abs().max()).item() < 2e-2
        out, gathered = fused_ops.ag_gemm(x_local, wk, None, comm, True, True)
        ref = G.gemm_nn(x_all, wk).float()
        assert torch.equal(gathered, x_all)
        assert ((out.float() - ref).abs().max() / ref.abs().max()).item() < 2e-2
    torch.cuda.synchronize()
    rt.check()
    from bmtrain_b200.ops import _native
    assert _native.cuda_lib().bmt_gemm_status() == 0


def test_tp_fused_kernels_2gpu():
    _need(2)
    run_distributed("test_multi_gpu", "body_tp_fused", 2, device="cuda")


def test_tp_fused_kernels_4gpu():
    """Groups of four: rows of three other ranks per kernel (tile rotation, early "delivered", push order)."""
    _need(4)
    run_distributed("test_multi_gpu", "body_tp_fused", 4, device="cuda")


def body_tp_model_gpu():
    """bf16 GPT with tp_size=2 on 2 GPUs (column/row parallel layers on the fused kernels, vocab-parallel embedding and
    loss) against the fp32 single-process oracle: loss and gradient statistics."""
    import bmtrain_b200 as bmt
    from oracle import OracleGPT

    rank = bmt.rank()
    cfg = dict(num_layers=2, vocab=2048, d=256, dh=64, h=4, dff=1024, max_distance=256)
    torch.manual_seed(3)
    ref = OracleGPT(cfg["num_layers"], cfg["vocab"], cfg["d"], cfg["dh"], cfg["h"], cfg["dff"], cfg["max_distance"], activation="gelu")
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, 0.03)
        for blk in ref.transformers:
            blk.ln_attn.weight.add_(1.0)
            blk.ln_ff.weight.add_(1.0)
        ref.layernorm.weight.add_(1.0)
    model = bmt.models.GPT(cfg["num_layers"], cfg["vocab"], cfg["d"], cfg["dh"], cfg["h"], cfg["dff"], cfg["max_distance"],
                           dtype=torch.bfloat16, activation="gelu")
    model.load_state_dict(ref.state_dict())
    ids = torch.randint(0, cfg["vocab"], (2, 257), generator=torch.Generator().manual_seed(9))
    pos = torch.arange(256)[None].expand(2, -1).contiguous()
    mask = torch.ones(2, 256, dtype=torch.bool)
    logits = model(ids[:, :-1].cuda(), pos.cuda(), mask.cuda())      # (s, b, vocab / 2)
    loss = bmt.loss.FusedCrossEntropy(parallel=True)(logits.reshape(-1, logits.shape[-1]), ids[:, 1:].t().reshape(-1).cuda())
    (loss * 256.0).backward()
    bmt.synchronize()
    rl = torch.nn.functional.cross_entropy(ref(ids[:, :-1], pos, mask).view(-1, cfg["vocab"]), ids[:, 1:].reshape(-1))
    (rl * 256.0).backward()
    assert abs(loss.item() - rl.item()) < 3e-2, (loss.item(), rl.item())
    got = {r["name"]: r for r in bmt.inspect.inspect_model(model, "*")}
    for name, p in ref.named_parameters():
        if name not in got:
            continue
        ref_std = p.grad.std().item()
        if tuple(got[name]["shape"]) == tuple(p.shape):   # tensor-parallel shards report their own slice: compare the replicated ones
            assert abs(got[name]["grad_std"] - ref_std) <= 0.08 * ref_std + 1e-4, (name, got[name]["grad_std"], ref_std)
    from bmtrain_b200.parallel import symm
    rt = symm.peer_runtime(bmt.config["tp_comm"])
    assert rt is not None
    rt.check()


def test_tensor_parallel_model_2gpu():
    _need(2)
    run_distributed("test_multi_gpu", "body_tp_model_gpu", 2, device="cuda", init_kwargs=dict(tp_size=2))


def _oracle_gpt(cfg, seed, std=0.03, activation="gelu"):
    from oracle import OracleGPT

    torch.manual_seed(seed)
    ref = OracleGPT(cfg["num_layers"], cfg["vocab"], cfg["d"], cfg["dh"], cfg["h"], cfg["dff"], cfg["max_distance"], activation=activation)
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, std)
        for blk in ref.transformers:
            blk.ln_attn.weight.add_(1.0)
            blk.ln_ff.weight.add_(1.0)
        ref.layernorm.weight.add_(1.0)
    return ref


def _compare_grads(bmt, model, ref, rel):
    got = {r["name"]: r for r in bmt.inspect.inspect_model(model, "*")}
    checked = 0
    for name, p in ref.named_parameters():
        if name not in got or tuple(got[name]["shape"]) != tuple(p.shape):
            continue   # tensor-parallel shards report their own slice
        ref_std = p.grad.std().item()
        assert abs(got[name]["grad_std"] - ref_std) <= rel * ref_std + 1e-4, (name, got[name]["grad_std"], ref_std)
        assert abs(got[name]["grad_mean"] - p.grad.mean().item()) <= rel * ref_std + 1e-4, name
        checked += 1
    assert checked > 0


def body_tp_zero_gpu():
    """bf16 GPT with tensor parallel 2 x ZeRO 2 on 4 GPUs, two accumulated backward passes, next to the ZeRO gathers and the
    fused gradient reduce-scatter; loss and gradients follow the fp32 single-process model.  By default the tensor-parallel
    pairs take NCCL + separate GEMMs in this layout; with BMT_TP_FUSED_WITH_ZERO=1 they run on the fused kernels in their
    non-spinning form."""
    import os

    import bmtrain_b200 as bmt
    from bmtrain_b200.parallel import fused_ops, symm

    rank, world = bmt.rank(), bmt.world_size()
    tp = bmt.config["tp_size"]
    dp, dp_rank = world // tp, rank // tp
    assert symm.no_spin()
    cfg = dict(num_layers=3, vocab=2048, d=256, dh=64, h=4, dff=1024, max_distance=256)
    ref = _oracle_gpt(cfg, 3)
    model = bmt.models.GPT(cfg["num_layers"], cfg["vocab"], cfg["d"], cfg["dh"], cfg["h"], cfg["dff"], cfg["max_distance"],
                           dtype=torch.bfloat16, activation="gelu")
    model.load_state_dict(ref.state_dict())
    all_ids = torch.randint(0, cfg["vocab"], (dp, 2, 2, 257), generator=torch.Generator().manual_seed(9))
    pos = torch.arange(256)[None].expand(2, -1).contiguous()
    mask = torch.ones(2, 256, dtype=torch.bool)
    loss_fn = bmt.loss.FusedCrossEntropy(parallel=True)
    losses = []
    for it in range(2):
        ids = all_ids[dp_rank, it]
        logits = model(ids[:, :-1].cuda(), pos.cuda(), mask.cuda())      # (s, b, vocab / tp)
        loss = loss_fn(logits.reshape(-1, logits.shape[-1]), ids[:, 1:].t().reshape(-1).cuda())
        (loss * 256.0 / dp).backward()
        losses.append(loss.item())
    bmt.synchronize()
    if os.environ.get("BMT_TP_FUSED_WITH_ZERO") == "1":
        assert fused_ops.calls["ag_gemm"] > 0 and fused_ops.calls["gemm_rs"] > 0, fused_ops.calls
    else:
        assert fused_ops.calls["ag_gemm"] == 0 and fused_ops.calls["gemm_rs"] == 0, fused_ops.calls
    for d in range(dp):
        for it in range(2):
            ids = all_ids[d, it]
            rl = torch.nn.functional.cross_entropy(ref(ids[:, :-1], pos, mask).view(-1, cfg["vocab"]), ids[:, 1:].reshape(-1))
            (rl * 256.0 / dp).backward()
            if d == dp_rank:
                assert abs(losses[it] - rl.item()) < 3e-2, (it, losses[it], rl.item())
    _compare_grads(bmt, model, ref, 0.08)
    for rt in symm._runtimes.values():
        if rt is not None:
            rt.check()
    from bmtrain_b200.ops import _native
    assert _native.cuda_lib().bmt_gemm_status() == 0


@pytest.mark.parametrize("fused", [False, True])
def test_tensor_parallel_with_zero_4gpu(fused, monkeypatch):
    _need(4)
    monkeypatch.setenv("BMT_TP_FUSED_WITH_ZERO", "1" if fused else "0")
    run_distributed("test_multi_gpu", "body_tp_zero_gpu", 4, device="cuda", init_kwargs=dict(tp_size=2))


def test_tp_fused_kernels_nonspinning_2gpu(monkeypatch):
    """The deliver / wait / sum form of GEMM -> reduce-scatter and the fused reduce-scatter with an external hand-shake."""
    _need(2)
    monkeypatch.setenv("BMT_NO_SPIN", "1")
    run_distributed("test_multi_gpu", "body_tp_fused", 2, device="cuda")


def body_pipe_zero_gpu():
    """fp16 GPT, pipeline 2 x ZeRO 2 on 4 GPUs, 4 layers (two per stage), 4 micro-batches: every block of a stage keeps its
    full gradients across the micro-batches in peer-visible staging memory, so each needs staging of its own."""
    import bmtrain_b200 as bmt
    from bmtrain_b200.parallel import symm

    rank, world = bmt.rank(), bmt.world_size()
    cfg = dict(num_layers=4, vocab=1024, d=256, dh=64, h=4, dff=512, max_distance=64)
    ref = _oracle_gpt(cfg, 5, activation="relu")
    model = bmt.models.GPT(cfg["num_layers"], cfg["vocab"], cfg["d"], cfg["dh"], cfg["h"], cfg["dff"], cfg["max_distance"],
                           dtype=torch.float16, activation="relu")
    assert isinstance(model.transformers, bmt.PipelineTransformerBlockList)
    assert len(model.transformers.layer_ids) == 2
    model.load_state_dict(ref.state_dict())
    all_ids = torch.randint(0, cfg["vocab"], (world, 2, 65), generator=torch.Generator().manual_seed(60))
    ids = all_ids[rank]
    pos = torch.arange(64)[None].expand(2, -1).contiguous()
    mask = torch.ones(2, 64, dtype=torch.bool)
    loss_fn = bmt.loss.FusedCrossEntropy()
    scale = 512.0
    logits = model(ids[:, :-1].cuda(), pos.cuda(), mask.cuda())
    loss = loss_fn(logits.view(-1, logits.shape[-1]), ids[:, 1:].reshape(-1).cuda())
    (loss * scale / world).backward()
    bmt.synchronize()
    ref_loss = None
    for d in range(world):
        rl = torch.nn.functional.cross_entropy(ref(all_ids[d][:, :-1], pos, mask).view(-1, cfg["vocab"]), all_ids[d][:, 1:].reshape(-1))
        (rl * scale / world).backward()
        if d == rank:
            ref_loss = rl.item()
    assert abs(loss.item() - ref_loss) < 2e-2, (loss.item(), ref_loss)
    got = {r["name"]: r for r in bmt.inspect.inspect_model(model, "*")}
    for name, p in ref.named_parameters():
        if name not in got:
            continue
        ref_std = p.grad.std().item()
        assert abs(got[name]["grad_std"] - ref_std) <= 0.05 * ref_std + 1e-4, (name, got[name]["grad_std"], ref_std)
    for rt in symm._runtimes.values():
        if rt is not None:
            rt.check()


def test_pipeline_with_zero_4gpu():
    _need(4)
    run_distributed("test_multi_gpu", "body_pipe_zero_gpu", 4, device="cuda", init_kwargs=dict(pipe_size=2, num_micro_batches=4))


def test_pipeline_2gpu():
    """Two pipeline stages on two GPUs (NCCL send / recv between the stages, no ZeRO sharding inside a stage)."""
    _need(2)
    run_distributed("test_multi_gpu", "body_pipe_zero_gpu", 2, device="cuda", init_kwargs=dict(pipe_size=2, num_micro_batches=4))
