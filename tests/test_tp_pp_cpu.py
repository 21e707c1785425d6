"""Tensor-parallel and pipeline-parallel paths on CPU ranks (gloo) against a single-process PyTorch model."""
import pytest
import torch

from dist_utils import run_distributed

CFG = dict(num_layers=2, vocab=512, d=64, dh=16, h=4, dff=256, max_distance=32)


def _oracle(activation="relu"):
    from oracle import OracleGPT

    torch.manual_seed(3)
    ref = OracleGPT(CFG["num_layers"], CFG["vocab"], CFG["d"], CFG["dh"], CFG["h"], CFG["dff"], CFG["max_distance"], activation=activation)
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, 0.05)
        for blk in ref.transformers:
            blk.ln_attn.weight.add_(1.0)
            blk.ln_ff.weight.add_(1.0)
        ref.layernorm.weight.add_(1.0)
    return ref


def _tp_state_dict(ref, tp):
    """The oracle's state dict re-ordered for the tensor-parallel QKV layout.

    Under tensor parallelism the fused QKV projection is split by output rows, and each rank's rows are laid out
    (head, {q,k,v}, dim); the full matrix is therefore the concatenation of the per-rank head groups, which for the
    oracle's (head, {q,k,v}, dim) ordering is the identity.  Nothing to permute: kept as a hook for other layouts."""
    return ref.state_dict()


def body_tp(world_tp=2):
    import bmtrain_b200 as bmt
    from bmtrain_b200.store import _save_to_rank0

    rank, world = bmt.rank(), bmt.world_size()
    tp = bmt.config["tp_size"]
    ref = _oracle()
    model = bmt.models.GPT(CFG["num_layers"], CFG["vocab"], CFG["d"], CFG["dh"], CFG["h"], CFG["dff"], CFG["max_distance"],
                           dtype=torch.float32)
    res = model.load_state_dict(_tp_state_dict(ref, tp))
    assert not res.missing_keys and not res.unexpected_keys
    # checkpoint round trip re-assembles the tensor-parallel shards
    sd = _save_to_rank0(model)
    if rank == 0:
        for k, v in ref.state_dict().items():
            assert torch.allclose(sd[k], v), k
    dp = world // tp
    dp_rank = rank // tp
    g = torch.Generator().manual_seed(50)
    all_ids = torch.randint(0, CFG["vocab"], (dp, 2, 17), generator=g)
    ids = all_ids[dp_rank]
    pos = torch.arange(16)[None].expand(2, -1).contiguous()
    mask = torch.ones(2, 16, dtype=torch.bool)
    loss_fn = bmt.loss.FusedCrossEntropy(parallel=True)
    opt = bmt.optim.AdamOptimizer(model.parameters(), lr=1e-2)
    om = bmt.optim.OptimManager(loss_scale=None, grad_scale=dp)
    om.add_optimizer(opt)
    ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-2)
    for step in range(3):
        logits = model(ids[:, :-1].contiguous(), pos, mask)          # (s, b, vocab / tp), sequence first
        target = ids[:, 1:].t().contiguous()                          # (s, b)
        loss = loss_fn(logits.reshape(-1, logits.shape[-1]), target.reshape(-1))
        om.zero_grad()
        om.backward(loss)
        om.step()
        ref_opt.zero_grad()
        ref_loss = 0.0
        for d in range(dp):
            rl = torch.nn.functional.cross_entropy(ref(all_ids[d][:, :-1], pos, mask).view(-1, CFG["vocab"]),
                                                   all_ids[d][:, 1:].reshape(-1)) / dp
            rl.backward()
            ref_loss += rl.item()
        ref_opt.step()
        mean_loss = bmt.sum_loss(loss.detach()).item()
        assert abs(mean_loss - ref_loss) < 2e-3 * max(1.0, ref_loss), (step, mean_loss, ref_loss)
    sd = _save_to_rank0(model)
    if rank == 0:
        for k, v in ref.state_dict().items():
            assert torch.allclose(sd[k], v, atol=2e-3, rtol=1e-2), k


def test_tensor_parallel_gpt_cpu():
    run_distributed("test_tp_pp_cpu", "body_tp", 2, init_kwargs=dict(tp_size=2))


def test_tensor_parallel_with_zero_cpu():
    run_distributed("test_tp_pp_cpu", "body_tp", 4, init_kwargs=dict(tp_size=2))


def body_pipe():
    import bmtrain_b200 as bmt
    from bmtrain_b200.store import _save_to_rank0

    rank, world = bmt.rank(), bmt.world_size()
    ref = _oracle()
    model = bmt.models.GPT(CFG["num_layers"], CFG["vocab"], CFG["d"], CFG["dh"], CFG["h"], CFG["dff"], CFG["max_distance"],
                           dtype=torch.float32)
    assert isinstance(model.transformers, bmt.PipelineTransformerBlockList)
    model.load_state_dict(ref.state_dict())
    g = torch.Generator().manual_seed(60)
    all_ids = torch.randint(0, CFG["vocab"], (world, 2, 17), generator=g)
    ids = all_ids[rank]
    pos = torch.arange(16)[None].expand(2, -1).contiguous()
    mask = torch.ones(2, 16, dtype=torch.bool)
    opt = bmt.optim.AdamOptimizer(model.parameters(), lr=1e-2)
    om = bmt.optim.OptimManager(loss_scale=None, grad_scale=world)
    om.add_optimizer(opt)
    ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-2)
    for step in range(3):
        logits = model(ids[:, :-1].contiguous(), pos, mask)
        loss = torch.nn.functional.cross_entropy(logits.view(-1, CFG["vocab"]), ids[:, 1:].reshape(-1))
        om.zero_grad()
        om.backward(loss)
        om.step()
        ref_opt.zero_grad()
        ref_loss = 0.0
        for d in range(world):
            rl = torch.nn.functional.cross_entropy(ref(all_ids[d][:, :-1], pos, mask).view(-1, CFG["vocab"]),
                                                   all_ids[d][:, 1:].reshape(-1)) / world
            rl.backward()
            ref_loss += rl.item()
        ref_opt.step()
        mean_loss = bmt.sum_loss(loss.detach()).item()
        assert abs(mean_loss - ref_loss) < 2e-3 * max(1.0, ref_loss), (step, mean_loss, ref_loss)
    sd = _save_to_rank0(model)
    if rank == 0:
        for k, v in ref.state_dict().items():
            assert torch.allclose(sd[k], v, atol=2e-3, rtol=1e-2), k


def test_pipeline_gpt_cpu():
    run_distributed("test_tp_pp_cpu", "body_pipe", 2, init_kwargs=dict(pipe_size=2, num_micro_batches=2))


def test_pipeline_with_zero_cpu():
    run_distributed("test_tp_pp_cpu", "body_pipe", 4, init_kwargs=dict(pipe_size=2, num_micro_batches=4))


def body_tp_helpers():
    """The reference-named helper functions of the tensor-parallel linear core against plain collectives + matmul."""
    import bmtrain_b200 as bmt
    from bmtrain_b200.nn import parallel_linear_func as P

    comm = bmt.config["tp_comm"]
    tp, r = comm.size, comm.rank
    torch.manual_seed(3)
    x_all = torch.randn(tp * 6, 10)
    w = torch.randn(8, 10, requires_grad=True)
    b = torch.randn(8, requires_grad=True)
    x_loc = x_all[r * 6:(r + 1) * 6].clone().requires_grad_()
    out = P.async_all_gather_linear_func(x_loc, w, b)
    assert torch.allclose(out, x_all @ w.t() + b, atol=1e-5)
    # row-parallel: every rank holds a slice of the features, the sum over ranks is scattered over the tokens
    torch.manual_seed(5 + r)
    xr = torch.randn(tp * 6, 10)
    wr = torch.randn(8, 10)
    full = xr @ wr.t()
    tot = bmt.distributed.all_reduce(full.clone(), "sum")
    got = P.async_reduce_scatter_linear_func(xr, wr, None)
    assert torch.allclose(got, tot[r * 6:(r + 1) * 6], atol=1e-4)
    # backward helper: gathers the output gradient
    g_loc = torch.randn(6, 8)
    g_all = torch.cat(bmt.distributed.all_gather(g_loc).unbind(0), dim=0)
    xin = torch.randn(tp * 6, 10, requires_grad=True)
    wk = torch.randn(8, 10, requires_grad=True)
    gi, gw, gb = P.async_all_gather_linear_backward_func(g_loc, xin, wk, b)
    assert torch.allclose(gi, g_all @ wk, atol=1e-4) and torch.allclose(gw, g_all.t() @ xin, atol=1e-4)
    assert torch.allclose(gb, g_all.sum(0), atol=1e-4)


def test_tp_helper_functions_cpu():
    run_distributed("test_tp_pp_cpu", "body_tp_helpers", 2, init_kwargs=dict(tp_size=2))


def body_tp_linear_modules():
    """Column- and row-parallel linears, every flag combination, inside a Block and bare, against ``torch.nn.Linear`` with
    the full weight (the intent of the reference's ``tests/test_column_parallel_linear.py:6-75`` and
    ``tests/test_row_parallel_linear.py:6-54``): output, weight / bias gradient of this rank's shard, input gradient."""
    import bmtrain_b200 as bmt

    tp, r = bmt.config["tp_size"], bmt.config["topology"].tp_id
    torch.manual_seed(100)
    full = torch.nn.Linear(8, 8)
    x = torch.randn(8, 4, 8, requires_grad=True)
    y_ref = full(x)
    y_ref.sum().backward()
    w_ref, b_ref, gx_ref = full.weight.grad.clone(), full.bias.grad.clone(), x.grad.clone()

    def build(cls, blocked, **kw):
        mod = cls(8, 8, dtype=torch.float32, **kw)
        if blocked:
            mod = bmt.Block(mod)
        bmt.init_parameters(mod)
        mod.load_state_dict(full.state_dict())
        return mod

    for blocked in (False, True):
        for gather_input, gather_output in ((True, True), (True, False), (False, True)):
            mod = build(bmt.nn.ColumnParallelLinear, blocked, gather_input=gather_input, gather_output=gather_output)
            xin = (x.detach().chunk(tp, dim=0)[r] if gather_input else x.detach()).clone().requires_grad_()
            y = mod(xin)
            want = y_ref if gather_output else y_ref.chunk(tp, dim=-1)[r]
            tag = ("column", blocked, gather_input, gather_output)
            assert torch.allclose(y, want, atol=1e-5), tag
            y.sum().backward()
            bmt.synchronize()
            inner = mod._module if blocked else mod
            gw, gb = _local_grad(bmt, mod, inner, "weight"), _local_grad(bmt, mod, inner, "bias")
            # a gathered output is a replicated quantity: its backward hands every rank the gradient of its own slice
            assert torch.allclose(gw, w_ref.chunk(tp, dim=0)[r].reshape(-1), atol=1e-4), ("dW",) + tag
            assert torch.allclose(gb, b_ref.chunk(tp, dim=0)[r].reshape(-1), atol=1e-4), ("db",) + tag
            want_gx = gx_ref.chunk(tp, dim=0)[r] if gather_input else gx_ref
            assert torch.allclose(xin.grad, want_gx, atol=1e-4), ("dx",) + tag
        for split_input in (True, False):
            mod = build(bmt.nn.RowParallelLinear, blocked, split_input=split_input, all_reduce_output=True)
            xin = x.detach().chunk(tp, dim=0 if split_input else 2)[r].clone().requires_grad_()
            y = mod(xin)
            assert torch.allclose(y, y_ref, atol=1e-5), ("row", blocked, split_input)
            y.sum().backward()
            bmt.synchronize()
            inner = mod._module if blocked else mod
            gw = _local_grad(bmt, mod, inner, "weight")
            gb = _local_grad(bmt, mod, inner, "bias")
            assert torch.allclose(gw, w_ref.chunk(tp, dim=1)[r].reshape(-1), atol=1e-4), ("row dW", blocked, split_input)
            assert torch.allclose(gb, b_ref.reshape(-1), atol=1e-4), ("row db", blocked, split_input)


def _local_grad(bmt, mod, inner, name):
    """Gradient of this rank's shard of ``inner.<name>``, flattened (attribute access on a distributed module returns the
    gathered tensor; the parameter itself, with its gradient, sits in ``_parameters``)."""
    p = inner._parameters[name]
    assert p.grad is not None, f"no gradient on {name}"
    return p.grad.detach().reshape(-1).clone()


def test_tp_linear_modules_cpu():
    run_distributed("test_tp_pp_cpu", "body_tp_linear_modules", 2, init_kwargs=dict(tp_size=2))


def body_inspect_in_pipeline():
    """``record_tensor`` inside the blocks of a pipeline (the intent of the reference's ``tests/test_inspector_hidden.py``):
    every rank lists every layer in order, statistics and gradient statistics equal those of the same network run in one
    process on the batches of all ranks."""
    import bmtrain_b200 as bmt

    rank, world = bmt.rank(), bmt.world_size()
    torch.manual_seed(21)
    weights = [torch.randn(8, 8) * 0.5 for _ in range(4)]

    class Layer(bmt.DistributedModule):
        def __init__(self, w):
            super().__init__()
            self.fc = bmt.nn.Linear(8, 8, bias=False, dtype=torch.float32)
            self._w = w

        def forward(self, x):
            bmt.inspect.record_tensor(x, "hidden")
            return torch.tanh(self.fc(x))

    layers = [Layer(w) for w in weights]
    net = bmt.PipelineTransformerBlockList(layers)
    bmt.init_parameters(net)
    net.load_state_dict({f"{i}.fc.weight": w for i, w in enumerate(weights)})
    data = torch.randn(world, 4, 8, generator=torch.Generator().manual_seed(5))
    x = data[rank].clone().requires_grad_()
    with bmt.inspect.inspect_tensor() as insp:
        out = net(x)
        (out * out).sum().backward()
    summary = insp.get_summary()
    assert [s["name"] for s in summary] == [f"{i}.hidden" for i in range(4)], [s["name"] for s in summary]

    # one process, all data
    ref_x = data.reshape(-1, 8).clone().requires_grad_()
    hidden, h = [], ref_x
    for w in weights:
        h.retain_grad()
        hidden.append(h)
        h = torch.tanh(h @ w.t())
    (h * h).sum().backward()
    for got, want in zip(summary, hidden):
        assert got["shape"][1:] == (8,), got["shape"]
        assert abs(got["mean"] - want.mean().item()) < 1e-5, (got["name"], got["mean"], want.mean().item())
        assert abs(got["max"] - want.max().item()) < 1e-5 and abs(got["min"] - want.min().item()) < 1e-5
        assert got["grad_mean"] is not None
        assert abs(got["grad_mean"] - want.grad.mean().item()) < 1e-5, (got["name"], got["grad_mean"], want.grad.mean().item())
    t = insp.get_tensor("hidden", index=3)
    assert t is not None and t.shape[1:] == (8,)


def test_inspect_inside_pipeline_cpu():
    run_distributed("test_tp_pp_cpu", "body_inspect_in_pipeline", 2, init_kwargs=dict(pipe_size=2, num_micro_batches=2))


def test_inspect_inside_pipeline_with_zero_cpu():
    run_distributed("test_tp_pp_cpu", "body_inspect_in_pipeline", 4, init_kwargs=dict(pipe_size=2, num_micro_batches=2))


def body_init_parameters_in_lists(tmp):
    """``init_parameters`` draws what a single process draws under the same seed, whichever list type holds the layers and
    whichever stage owns them (the intent of the reference's ``tests/test_init_parameters_multi_gpu.py:98-141``)."""
    import os

    import bmtrain_b200 as bmt

    class Lin(bmt.DistributedModule):
        def __init__(self):
            super().__init__()
            self.weight = bmt.DistributedParameter(torch.empty(5, 3), init_method=torch.nn.init.xavier_normal_)
            self.bias = bmt.DistributedParameter(torch.empty(5), init_method=torch.nn.init.zeros_)

        def forward(self, x):
            return torch.nn.functional.linear(x, self.weight, self.bias)

    torch.manual_seed(33)
    want = {}
    for i in range(2):
        w = torch.empty(5, 3)
        torch.nn.init.xavier_normal_(w)
        want[f"l.{i}.weight"], want[f"l.{i}.bias"] = w, torch.zeros(5)

    def holder(make_list):
        class Net(bmt.DistributedModule):
            def __init__(self):
                super().__init__()
                self.l = make_list([Lin(), Lin()])

        return Net()

    kinds = {
        "pipeline": lambda layers: bmt.PipelineTransformerBlockList(layers),
        "block list": lambda layers: bmt.TransformerBlockList(layers),
        "checkpoint blocks": lambda layers: torch.nn.ModuleList([bmt.CheckpointBlock(layer) for layer in layers]),
    }
    path = os.path.join(tmp, "init.pt")
    for kind, make_list in kinds.items():
        torch.manual_seed(33)
        net = holder(make_list)
        bmt.init_parameters(net)
        bmt.save(net, path)
        bmt.synchronize()
        if bmt.rank() == 0:
            got = torch.load(path)
            assert list(got.keys()) == list(want.keys()), (kind, list(got.keys()))
            for k, v in want.items():
                assert torch.equal(got[k], v), (kind, k)
        bmt.synchronize()


def test_init_parameters_in_lists_cpu(tmp_path):
    run_distributed("test_tp_pp_cpu", "body_init_parameters_in_lists", 2, init_kwargs=dict(pipe_size=2, num_micro_batches=2),
                    tmp=str(tmp_path))


def body_pipeline_hidden_states():
    """``return_hidden_states=True`` through a pipeline with several micro-batches: the stacked per-layer inputs equal those
    of a single process, and a loss that also uses the middle hidden states gives the single-process gradients (the intent
    of the reference's ``tests/test_middle_hidden.py:120-190`` for its pipeline model)."""
    import bmtrain_b200 as bmt

    rank, world = bmt.rank(), bmt.world_size()
    torch.manual_seed(8)
    weights = [torch.randn(6, 6) * 0.4 for _ in range(4)]

    class Lin(bmt.DistributedModule):
        def __init__(self):
            super().__init__()
            self.fc = bmt.nn.Linear(6, 6, bias=False, dtype=torch.float32)

        def forward(self, x):
            return torch.tanh(self.fc(x))

    net = bmt.PipelineTransformerBlockList([Lin() for _ in weights])
    bmt.init_parameters(net)
    net.load_state_dict({f"{i}.fc.weight": w for i, w in enumerate(weights)})
    data = torch.randn(world, 4, 6, generator=torch.Generator().manual_seed(2))
    x = data[rank].clone().requires_grad_()
    last, hidden = net(x, return_hidden_states=True)
    assert hidden.shape == (4, 4, 6), hidden.shape          # (layers, this rank's batch, features)
    loss = (last * last).sum() + sum((i + 1) * hidden[i].sum() for i in range(4))
    loss.backward()
    bmt.synchronize()

    ws = [w.clone().requires_grad_() for w in weights]
    grads_x = []
    for d in range(world):
        xr = data[d].clone().requires_grad_()
        h, seen = xr, []
        for w in ws:
            seen.append(h)
            h = torch.tanh(h @ w.t())
        ((h * h).sum() + sum((i + 1) * seen[i].sum() for i in range(4))).backward()
        grads_x.append(xr.grad)
        if d == rank:
            assert torch.allclose(last, h, atol=1e-5)
            for i in range(4):
                assert torch.allclose(hidden[i], seen[i], atol=1e-5), i
    assert torch.allclose(x.grad, grads_x[rank], atol=1e-5)
    # weight gradients: the sum over the data of every rank that shares the layer's ZeRO group and pipeline group
    got = {r["name"]: r for r in bmt.inspect.inspect_model(net, "*")}
    for i, w in enumerate(ws):
        name = f"{i}.fc.weight"
        if name in got:
            assert abs(got[name]["grad_std"] - w.grad.std().item()) < 1e-4 * max(1.0, w.grad.std().item()), name


def test_pipeline_hidden_states_cpu():
    run_distributed("test_tp_pp_cpu", "body_pipeline_hidden_states", 2, init_kwargs=dict(pipe_size=2, num_micro_batches=2))


def test_pipeline_hidden_states_with_zero_cpu():
    run_distributed("test_tp_pp_cpu", "body_pipeline_hidden_states", 4, init_kwargs=dict(pipe_size=2, num_micro_batches=4))


def body_vp_cross_entropy():
    """Cross-entropy over a vocabulary sharded across the tensor-parallel group equals ``F.cross_entropy`` on the full
    logits: loss, ignored rows, and the gradient of this rank's slice (intent of ``tests/test_parallel_projection.py``)."""
    import bmtrain_b200 as bmt

    tp, r = bmt.config["tp_size"], bmt.config["topology"].tp_id
    torch.manual_seed(4)
    full = (torch.randn(37, 16 * tp) * 3).requires_grad_()
    target = torch.randint(0, 16 * tp, (37,))
    target[5] = target[20] = -100
    want = torch.nn.functional.cross_entropy(full, target, ignore_index=-100)
    want.backward()
    mine = full.detach()[:, r * 16:(r + 1) * 16].clone().requires_grad_()
    loss = bmt.loss.FusedCrossEntropy(ignore_index=-100, parallel=True)(mine, target)
    loss.backward()
    assert abs(loss.item() - want.item()) < 1e-5, (loss.item(), want.item())
    assert torch.allclose(mine.grad, full.grad[:, r * 16:(r + 1) * 16], atol=1e-6)
    none = bmt.loss.FusedCrossEntropy(ignore_index=-100, parallel=True, reduction="none")(mine.detach(), target)
    assert none[5].item() == 0.0 and none[20].item() == 0.0
    ref_rows = torch.nn.functional.cross_entropy(full.detach(), target, ignore_index=-100, reduction="none")
    assert torch.allclose(none, ref_rows, atol=1e-5)


def test_vp_cross_entropy_cpu():
    run_distributed("test_tp_pp_cpu", "body_vp_cross_entropy", 2, init_kwargs=dict(tp_size=2))
