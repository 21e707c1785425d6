"""Behavioural contract of the sharding engine, optimizers, checkpoint I/O and inspection on one CPU rank.

Each test states which behaviour of the reference it pins down (reference test file in parentheses)."""
import math
import os

import pytest
import torch
import torch.nn as nn


class Lin(torch.nn.Module):
    """Linear on sharded parameters built from the package's own layers."""

    def __new__(cls, bmt, i, o, bias=True):
        return bmt.nn.Linear(i, o, bias=bias, dtype=torch.float32)


def _mlp(bmt, d=16, n=3):
    class Layer(bmt.DistributedModule):
        def __init__(self):
            super().__init__()
            self.fc = bmt.nn.Linear(d, d, dtype=torch.float32)
            self.calls = 0

        def forward(self, x):
            self.calls += 1
            return torch.tanh(self.fc(x))

    return [Layer() for _ in range(n)]


def _torch_mlp(d=16, n=3):
    return nn.ModuleList([nn.Linear(d, d) for _ in range(n)])


def _copy_into(bmt_layers, torch_layers):
    for b, t in zip(bmt_layers, torch_layers):
        inner = b._module if hasattr(b, "_module") else b
        inner.load_state_dict({"fc.weight": t.weight.detach(), "fc.bias": t.bias.detach()})


# ------------------------------------------------------------------------------------------------ block transparency
@pytest.mark.parametrize("zero_level,ckpt", [(3, True), (3, False), (2, True), (2, False)])
def test_block_matches_inner_module(bmt_cpu, zero_level, ckpt):
    """A Block / TransformerBlockList is numerically identical to the plain modules (test_model_wrapper, test_training)."""
    bmt = bmt_cpu
    torch.manual_seed(0)
    ref = _torch_mlp()
    layers = _mlp(bmt)
    _copy_into(layers, ref)
    tbl = bmt.TransformerBlockList([bmt.Block(l, use_checkpoint=ckpt, zero_level=zero_level) for l in layers])
    x = torch.randn(4, 16, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    y = tbl(x)
    yr = xr
    for l in ref:
        yr = torch.tanh(l(yr))
    assert torch.allclose(y, yr, atol=1e-6)
    y.sum().backward()
    yr.sum().backward()
    assert torch.allclose(x.grad, xr.grad, atol=1e-6)
    for blk, l in zip(tbl, ref):
        g = {n: p.grad for n, p in blk.named_parameters()}
        assert torch.allclose(g["fc.weight"].view_as(l.weight), l.weight.grad, atol=1e-6)
        assert torch.allclose(g["fc.bias"], l.bias.grad, atol=1e-6)


def test_different_output_shapes(bmt_cpu):
    """A Block returns a tensor for tensor outputs and tuples of the same arity for tuple outputs (test_different_output_shape)."""
    bmt = bmt_cpu

    class One(bmt.DistributedModule):
        def forward(self, x):
            return x * 2

    class TupleOne(bmt.DistributedModule):
        def forward(self, x):
            return (x * 2,)

    class Two(bmt.DistributedModule):
        def forward(self, x):
            return x * 2, x + 1

    x = torch.randn(3, requires_grad=True)
    assert isinstance(bmt.Block(One())(x), torch.Tensor)
    out = bmt.Block(TupleOne())(x)
    assert isinstance(out, tuple) and len(out) == 1
    out = bmt.Block(Two())(x)
    assert isinstance(out, tuple) and len(out) == 2


def test_multi_return_and_hidden_states(bmt_cpu):
    """num_hidden threads several outputs; return_hidden_states stacks the per-layer inputs and supports losses on them
    (test_multi_return, test_middle_hidden)."""
    bmt = bmt_cpu

    class Layer(bmt.DistributedModule):
        def __init__(self):
            super().__init__()
            self.fc = bmt.nn.Linear(8, 8, dtype=torch.float32)

        def forward(self, a, b, scale):
            return torch.tanh(self.fc(a)) + b * scale, b + a

    torch.manual_seed(1)
    layers = [Layer() for _ in range(3)]
    bmt.init_parameters(torch.nn.ModuleList(layers))
    tbl = bmt.TransformerBlockList([bmt.Block(l) for l in layers], num_hidden=2)
    a = torch.randn(2, 8, requires_grad=True)
    b = torch.randn(2, 8, requires_grad=True)
    out = tbl(a, b, 0.5, return_hidden_states=True)
    assert len(out) == 4 and out[2].shape == (3, 2, 8) and out[3].shape == (3, 2, 8)
    # reference: run the same layers as plain modules
    ra, rb = a.detach().clone().requires_grad_(), b.detach().clone().requires_grad_()
    ha, hb, seen = ra, rb, []
    for blk in tbl:
        seen.append(ha)
        w = blk.state_dict()
        ha, hb = torch.tanh(torch.nn.functional.linear(ha, w["fc.weight"], w["fc.bias"])) + hb * 0.5, hb + ha
    assert torch.allclose(out[0], ha, atol=1e-6) and torch.allclose(out[1], hb, atol=1e-6)
    assert torch.allclose(out[2], torch.stack(seen), atol=1e-6)
    (out[0].sum() + out[2][1].pow(2).sum()).backward()
    (ha.sum() + seen[1].pow(2).sum()).backward()
    assert torch.allclose(a.grad, ra.grad, atol=1e-5) and torch.allclose(b.grad, rb.grad, atol=1e-5)
    plain = tbl(a.detach(), b.detach(), 0.5)
    assert isinstance(plain, tuple) and len(plain) == 2


def test_no_grad_and_frozen_blocks(bmt_cpu):
    """Frozen blocks with no-grad inputs run forward exactly once and are skipped in backward; trainable blocks with
    no-grad inputs are recomputed exactly once (test_no_grad)."""
    bmt = bmt_cpu
    torch.manual_seed(2)
    layers = _mlp(bmt)
    bmt.init_parameters(torch.nn.ModuleList(layers))
    for p in layers[0].parameters():
        p.requires_grad_(False)
    tbl = bmt.TransformerBlockList([bmt.Block(l) for l in layers])
    x = torch.randn(4, 16)  # does not require grad
    y = tbl(x)
    y.sum().backward()
    assert layers[0].calls == 1          # frozen + no-grad input: never recomputed
    assert layers[1].calls == 2 and layers[2].calls == 2  # checkpoint recompute
    assert all(p.grad is None for p in layers[0].parameters())
    assert all(p.grad is not None for p in layers[1].parameters())
    with torch.no_grad():
        for l in layers:
            l.calls = 0
        tbl(x)
        assert [l.calls for l in layers] == [1, 1, 1]
    with pytest.raises(AssertionError):
        blk = bmt.Block(_mlp(bmt, n=1)[0])
        bmt.TransformerBlockList([blk, blk])


def test_requires_grad_toggle(bmt_cpu):
    """requires_grad of parameters inside a block can change between steps (test_requires_grad)."""
    bmt = bmt_cpu
    torch.manual_seed(3)
    layers = _mlp(bmt, n=2)
    bmt.init_parameters(torch.nn.ModuleList(layers))
    tbl = bmt.TransformerBlockList([bmt.Block(l) for l in layers])
    x = torch.randn(4, 16)
    tbl(x).sum().backward()
    w = dict(tbl[0].named_parameters())["fc.weight"]
    assert w.grad is not None and w.grad.abs().sum() > 0
    for blk in tbl:
        for p in blk.parameters():
            p.grad = None
    for _, b in tbl[0]._buckets.items():
        b.storage.grad = None
    w.requires_grad_(False)
    tbl(x).sum().backward()
    assert w.grad is None
    bias = dict(tbl[0].named_parameters())["fc.bias"]
    assert bias.grad is not None and bias.grad.abs().sum() > 0
    w.requires_grad_(True)


def test_dropout_train_eval(bmt_cpu):
    """train()/eval() reach the wrapped module (test_dropout)."""
    bmt = bmt_cpu

    class Drop(bmt.DistributedModule):
        def __init__(self):
            super().__init__()
            self.drop = torch.nn.Dropout(0.5)

        def forward(self, x):
            return self.drop(x)

    tbl = bmt.TransformerBlockList([bmt.Block(Drop())])
    x = torch.ones(1000)
    tbl.train()
    assert (tbl(x) == 0).any()
    tbl.eval()
    assert torch.equal(tbl(x), x)


def test_grad_accumulation(bmt_cpu):
    """Two backward calls without zero_grad double the gradients (test_grad_accu)."""
    bmt = bmt_cpu
    torch.manual_seed(4)
    layers = _mlp(bmt, n=2)
    bmt.init_parameters(torch.nn.ModuleList(layers))
    tbl = bmt.TransformerBlockList([bmt.Block(l) for l in layers])
    x = torch.randn(4, 16)
    tbl(x).sum().backward()
    g1 = [b.storage.grad.clone() for blk in tbl for b in blk._buckets.values()]
    tbl(x).sum().backward()
    g2 = [b.storage.grad for blk in tbl for b in blk._buckets.values()]
    for a, b in zip(g1, g2):
        assert torch.allclose(b, 2 * a, atol=1e-6)


# ----------------------------------------------------------------------------------------- init / checkpoints / wrapper
def test_init_parameters_matches_torch(bmt_cpu):
    """init_parameters draws the same values as a single-process torch init under the same seed (test_init_parameters)."""
    bmt = bmt_cpu
    torch.manual_seed(123)
    a = torch.empty(32, 16)
    torch.nn.init.xavier_normal_(a)
    b = torch.empty(32)
    torch.nn.init.zeros_(b)
    lin = bmt.nn.Linear(16, 32, dtype=torch.float32)
    torch.manual_seed(123)
    bmt.init_parameters(lin)
    sd = bmt.store._save_to_rank0(lin)
    assert torch.equal(sd["weight"], a) and torch.equal(sd["bias"], b)
    blk = bmt.Block(bmt.nn.Linear(16, 32, dtype=torch.float32))
    torch.manual_seed(123)
    bmt.init_parameters(blk)
    sd = blk.state_dict()
    assert torch.equal(sd["weight"], a) and torch.equal(sd["bias"], b)


def test_checkpoint_roundtrip_with_plain_torch(bmt_cpu, tmp_path):
    """bmt.save writes a file a plain torch model loads, and bmt.load reads a plain torch checkpoint (test_load_ckpt)."""
    bmt = bmt_cpu
    torch.manual_seed(5)

    class Net(bmt.DistributedModule):
        def __init__(self):
            super().__init__()
            self.head = bmt.nn.Linear(16, 4, dtype=torch.float32)
            self.layers = bmt.TransformerBlockList([bmt.Block(bmt.nn.Linear(16, 16, dtype=torch.float32)) for _ in range(2)])

    class TorchNet(nn.Module):
        def __init__(self):
            super().__init__()
            self.head = nn.Linear(16, 4)
            self.layers = nn.ModuleList([nn.Linear(16, 16) for _ in range(2)])

    net, tnet = Net(), TorchNet()
    bmt.init_parameters(net)
    path = str(tmp_path / "ckpt.pt")
    bmt.save(net, path)
    assert not tnet.load_state_dict(torch.load(path)).missing_keys
    for k, v in tnet.state_dict().items():
        assert torch.equal(v, bmt.store._save_to_rank0(net)[k])
    with torch.no_grad():
        for p in tnet.parameters():
            p.add_(1.0)
    torch.save(tnet.state_dict(), path)
    res = bmt.load(net, path)
    assert not res.missing_keys and not res.unexpected_keys
    for k, v in tnet.state_dict().items():
        assert torch.equal(v, bmt.store._save_to_rank0(net)[k])
    bmt.save(net, path, non_blocking=True)
    bmt.config["save_thread"].join()
    assert set(torch.load(path).keys()) == set(tnet.state_dict().keys())


def test_model_wrapper(bmt_cpu):
    """BMTrainModelWrapper converts a plain torch model in place; outputs are exactly equal (test_model_wrapper)."""
    bmt = bmt_cpu
    torch.manual_seed(6)

    class TorchNet(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(50, 16)
            self.layers = nn.ModuleList([nn.Sequential(nn.Linear(16, 16), nn.Tanh()) for _ in range(2)])
            self.norm = nn.LayerNorm(16)

        def forward(self, ids):
            x = self.emb(ids)
            for l in self.layers:
                x = l(x)
            return self.norm(x)

    ref = TorchNet()
    sd = {k: v.clone() for k, v in ref.state_dict().items()}
    ids = torch.randint(0, 50, (3, 7))
    expect = ref(ids)
    wrapped = bmt.BMTrainModelWrapper(TorchNet())
    wrapped.load_state_dict(sd)
    got = wrapped(ids)
    assert torch.equal(got, expect)
    assert all(isinstance(m, bmt.Block) for m in wrapped.layers)
    got.sum().backward()


# ------------------------------------------------------------------------------------------------------- optimizers
def test_adam_variants_agree(bmt_cpu):
    """bmt Adam (fp32) equals torch Adam exactly; the offloaded variant stays within 1e-5 (test_optim)."""
    bmt = bmt_cpu
    torch.manual_seed(7)
    ref = nn.Linear(32, 32)
    m1, m2 = nn.Linear(32, 32), nn.Linear(32, 32)
    m1.load_state_dict(ref.state_dict())
    m2.load_state_dict(ref.state_dict())
    o_ref = torch.optim.Adam(ref.parameters(), lr=1e-2)
    o1 = bmt.optim.AdamOptimizer(m1.parameters(), lr=1e-2)
    o2 = bmt.optim.AdamOffloadOptimizer(m2.parameters(), lr=1e-2)
    for _ in range(20):
        g = [torch.randn_like(p) for p in ref.parameters()]
        for m in (ref, m1, m2):
            for p, gg in zip(m.parameters(), g):
                p.grad = gg.clone()
        o_ref.step(); o1.step(); o2.step()
    for a, b, c in zip(ref.parameters(), m1.parameters(), m2.parameters()):
        assert torch.equal(a, b)
        assert (a - c).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_half_adam_tracks_fp32(bmt_cpu, dtype):
    """Half-precision Adam (scaled fp16 state / bf16) and the offloaded variant follow an fp32 AdamW run (test_optim)."""
    bmt = bmt_cpu
    torch.manual_seed(8)
    w0 = torch.randn(64, 64) * 0.1
    ref = w0.clone().requires_grad_()
    o_ref = torch.optim.AdamW([ref], lr=1e-2, weight_decay=1e-2)
    pa = torch.nn.Parameter(w0.to(dtype))
    pb = torch.nn.Parameter(w0.to(dtype))
    oa = bmt.optim.AdamOptimizer([pa], lr=1e-2, weight_decay=1e-2)
    ob = bmt.optim.AdamOffloadOptimizer([pb], lr=1e-2, weight_decay=1e-2)
    scale = 128.0
    for _ in range(30):
        g = torch.randn(64, 64)
        ref.grad = g.clone()
        pa.grad = (g * scale).to(dtype)
        pb.grad = (g * scale).to(dtype)
        o_ref.step(); oa.step(scale=scale); ob.step(scale=scale)
    tol = 3e-2 if dtype == torch.bfloat16 else 5e-3
    assert (pa.float() - ref).abs().max() < tol and (pb.float() - ref).abs().max() < tol
    assert (oa.state[pa]["_param_fp32"] - ref).abs().max() < tol


def test_loss_scale_state_machine(bmt_cpu):
    """Overflow halves the scale, zeroes the gradients and skips the step (fp16 moments are rescaled); clean steps grow
    the scale after loss_scale_steps (optim_manager semantics)."""
    bmt = bmt_cpu
    p = torch.nn.Parameter(torch.ones(8, dtype=torch.float16))
    opt = bmt.optim.AdamOptimizer([p], lr=1e-2)
    sched = bmt.lr_scheduler.NoDecay(opt, start_lr=1e-2, warmup_iter=2, end_iter=100)
    om = bmt.optim.OptimManager(loss_scale=1024, loss_scale_factor=2, loss_scale_steps=2, min_loss_scale=512)
    om.add_optimizer(opt, sched)
    p.grad = torch.ones(8, dtype=torch.float16)
    om.step()
    assert om.loss_scale == 1024 and sched.num_iter == 1
    m_before = opt.state[p]["exp_avg"].clone()
    p.grad = torch.full((8,), float("inf"), dtype=torch.float16)
    before = p.detach().clone()
    om.step()
    assert om.loss_scale == 512 and torch.equal(p.detach(), before) and sched.num_iter == 1
    assert p.grad.abs().sum() == 0
    assert torch.allclose(opt.state[p]["exp_avg"].float(), m_before.float() * 0.5)
    p.grad = torch.full((8,), float("nan"), dtype=torch.float16)
    om.step()
    assert om.loss_scale == 512  # already at the minimum
    for _ in range(2):
        p.grad = torch.ones(8, dtype=torch.float16)
        om.step()
    assert om.loss_scale == 1024
    sd = om.state_dict()
    assert sd["loss_scale"] == 1024 and sd["loss_scale_enabled"] and len(sd["optimizers"]) == 1


def test_clip_grad_norm(bmt_cpu):
    bmt = bmt_cpu
    ps = [torch.nn.Parameter(torch.zeros(10)), torch.nn.Parameter(torch.zeros(5))]
    opt = bmt.optim.AdamOptimizer(ps)
    om = bmt.optim.OptimManager(loss_scale=4.0)
    om.add_optimizer(opt)
    ps[0].grad = torch.full((10,), 4.0)
    ps[1].grad = torch.full((5,), 8.0)
    norm = om.clip_grad_norm(opt.param_groups, max_norm=1.0)
    expect = math.sqrt(10 * 16 + 5 * 64) / 4.0
    assert abs(float(norm) - expect) < 1e-4
    total = math.sqrt(sum(float(p.grad.pow(2).sum()) for p in ps)) / 4.0
    assert abs(total - 1.0) < 1e-3
    inf_norm = om.clip_grad_norm(opt.param_groups, max_norm=100.0, norm_type="inf")
    assert float(inf_norm) > 0


@pytest.mark.parametrize("kind", ["adam", "offload"])
def test_optimizer_resume_is_bit_identical(bmt_cpu, kind, tmp_path):
    """Saving (model, optim_manager.state_dict()) and resuming gives bit-identical parameters (test_optim_state)."""
    bmt = bmt_cpu

    def make():
        torch.manual_seed(9)
        layers = _mlp(bmt, n=2)
        bmt.init_parameters(torch.nn.ModuleList(layers))
        model = bmt.TransformerBlockList([bmt.Block(l) for l in layers])
        cls = bmt.optim.AdamOptimizer if kind == "adam" else bmt.optim.AdamOffloadOptimizer
        opt = cls(model.parameters(), lr=1e-2, weight_decay=1e-2)
        sched = bmt.lr_scheduler.Noam(opt, start_lr=1e-2, warmup_iter=3, end_iter=50)
        om = bmt.optim.OptimManager(loss_scale=None)
        om.add_optimizer(opt, sched)
        return model, om

    def run(model, om, steps, start=0):
        for s in range(start, start + steps):
            torch.manual_seed(100 + s)
            x = torch.randn(4, 16)
            loss = model(x).pow(2).mean()
            om.zero_grad()
            om.backward(loss)
            om.step()

    m1, om1 = make()
    run(m1, om1, 6)
    m2, om2 = make()
    run(m2, om2, 3)
    path = str(tmp_path / "m.pt")
    bmt.save(m2, path)
    torch.save(om2.state_dict(), str(tmp_path / "o.pt"))
    m3, om3 = make()
    bmt.load(m3, path)
    om3.load_state_dict(torch.load(str(tmp_path / "o.pt"), weights_only=False))
    run(m3, om3, 3, start=3)
    for a, b in zip(bmt.store._save_to_rank0(m1).values(), bmt.store._save_to_rank0(m3).values()):
        assert torch.equal(a, b)
    whole = om3.state_dict(gather_opt=True)
    assert whole["optimizers"][0]["is_whole"]


def test_lr_schedulers(bmt_cpu):
    bmt = bmt_cpu
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.0)
    L = bmt.lr_scheduler
    s = L.Noam(opt, start_lr=1.0, warmup_iter=4, end_iter=100)
    s.step(2)
    assert abs(s.current_lr - 1.0 / 2.0 * 2 / 4) < 1e-9
    s.step(16)
    assert abs(s.current_lr - 0.25) < 1e-9 and opt.param_groups[0]["lr"] == s.current_lr
    s = L.Linear(opt, 1.0, 10, 110)
    s.step(60)
    assert abs(s.current_lr - 0.5) < 1e-9
    s = L.Cosine(opt, 1.0, 10, 110)
    s.step(60)
    assert abs(s.current_lr - 0.5) < 1e-9
    s = L.Exponential(opt, 1.0, 10, 110, gamma=0.5)
    s.step(12)
    assert abs(s.current_lr - 0.25) < 1e-9
    s = L.NoDecay(opt, 1.0, 10, 110)
    s.step(5)
    assert abs(s.current_lr - 0.5) < 1e-9
    s.step()
    assert s.num_iter == 6
    s2 = L.NoDecay(opt, 3.0, 1, 2)
    s2.load_state_dict(s.state_dict())
    assert s2.num_iter == 6 and s2.start_lr == 1.0


# ------------------------------------------------------------------------------------------------------ loss / inspect
def test_fused_cross_entropy_cpu(bmt_cpu):
    """FusedCrossEntropy equals torch CE incl. class weights, ignore_index and reductions (test_loss_func)."""
    bmt = bmt_cpu
    torch.manual_seed(10)
    for classes in (10, 1000):
        x = torch.randn(33, classes).to(torch.bfloat16).requires_grad_()
        t = torch.randint(0, classes, (33,))
        t[::5] = -100
        w = torch.rand(classes)
        for weight in (None, w):
            for red in ("mean", "sum", "none"):
                got = bmt.loss.FusedCrossEntropy(weight=weight, reduction=red)(x, t)
                ref = torch.nn.functional.cross_entropy(x.float(), t, weight=weight, reduction=red)
                assert torch.allclose(got, ref, atol=1e-4, rtol=1e-4)
        bmt.loss.FusedCrossEntropy()(x, t).backward()
        xr = x.detach().float().requires_grad_()
        torch.nn.functional.cross_entropy(xr, t).backward()
        assert (x.grad.float() - xr.grad).abs().max() < 1e-3


def test_has_inf_nan_cpu(bmt_cpu):
    from bmtrain_b200.loss._function import has_inf_nan

    for dtype in (torch.float16, torch.bfloat16):
        x = torch.randn(1000).to(dtype)
        flag = torch.zeros(1, dtype=torch.uint8)
        has_inf_nan(x, flag)
        assert flag.item() == 0
        x[17] = float("nan")
        has_inf_nan(x, flag)
        assert flag.item() == 1


def test_inspect_model_and_tensor(bmt_cpu):
    """inspect_model reports parameter and gradient statistics; record_tensor keeps hidden states and their gradients
    (test_inspector_hidden, test_other_hidden)."""
    bmt = bmt_cpu
    torch.manual_seed(11)

    class Layer(bmt.DistributedModule):
        def __init__(self):
            super().__init__()
            self.fc = bmt.nn.Linear(8, 8, dtype=torch.float32)

        def forward(self, x):
            bmt.inspect.record_tensor(x, "hidden")
            return torch.tanh(self.fc(x))

    class Net(bmt.DistributedModule):
        def __init__(self):
            super().__init__()
            self.layers = bmt.TransformerBlockList([bmt.Block(Layer()) for _ in range(2)])
            self.head = bmt.nn.Linear(8, 2, dtype=torch.float32)

        def forward(self, x):
            y = self.head(self.layers(x))
            bmt.inspect.record_tensor(y, "out", group="final")
            return y

    net = Net()
    bmt.init_parameters(net)
    x = torch.randn(5, 8)
    with bmt.inspect.inspect_tensor() as insp:
        net(x).sum().backward()
    summary = insp.get_summary()
    names = [s["name"] for s in summary]
    assert names == ["0.hidden", "1.hidden", "final.0.out"]
    assert summary[1]["grad_std"] is not None and summary[0]["shape"] == (5, 8)
    assert insp.get_tensor("hidden", index=1).shape == (5, 8)
    assert insp.get_tensor("out", group="final") is not None
    stats = bmt.inspect.inspect_model(net, "*weight")
    assert [s["name"] for s in stats] == ["layers.0.fc.weight", "layers.1.fc.weight", "head.weight"]
    assert all(s["grad_std"] > 0 for s in stats)
    text = bmt.inspect.format_summary(stats)
    lines = text.split("\n")
    assert lines[0].split() == ["name", "shape", "max", "min", "std", "mean", "grad_std", "grad_mean"]
    assert len(lines) == 4 and lines[1].startswith(" layers.0.fc.weight")
    text2 = bmt.inspect.format_summary(summary)
    assert "final.0.out" in text2


def test_misc_utils(bmt_cpu, capsys):
    bmt = bmt_cpu
    from bmtrain_b200.utils import AverageRecorder, round_up, check_torch_version

    assert round_up(10, 4) == 12 and check_torch_version("1.0.0") > 0
    rec = AverageRecorder(alpha=0.5)
    rec.record(2.0); rec.record(2.0)
    assert abs(rec.value - 2.0) < 1e-9
    bmt.print_rank("hello"); bmt.print_block("t", "c"); bmt.see_memory("mem")
    assert "hello" in capsys.readouterr().out
    bmt.debug.set("k", 1); bmt.debug.append("l", 2)
    assert bmt.debug.get("k") == 1 and bmt.debug.get("l") == [2]
    assert bmt.world_size() == 1 and bmt.rank() == 0 and bmt.CheckpointBlock is bmt.Block
    groups = dict(bmt.grouped_parameters(bmt.nn.Linear(4, 4, dtype=torch.float32)))
    assert None in groups and len(groups[None]) == 2


def test_reference_named_internals(bmt_cpu):
    """Module paths and helper names of the reference that user code may import: ZeroContext gathers a block by hand,
    the hook functions bracket a module, formatting / header / enum helpers give the reference's values."""
    bmt = bmt_cpu
    from bmtrain_b200.benchmark import all_gather, reduce_scatter, send_recv, shape, utils  # noqa: F401
    from bmtrain_b200.hook_func import OneStepNoGradFunc, PostHookFunc, PreHookFunc  # noqa: F401
    from bmtrain_b200.inspect.format import align_str, format_line, item_formater
    from bmtrain_b200.inspect.model import _gather_value
    from bmtrain_b200.nccl import dtype2nccl, op2nccl
    from bmtrain_b200.zero_context import ZeroContext

    assert shape.SHAPES[0] == 1024 and shape.SHAPES[-1] == 2 ** 32
    assert utils.format_size_(512) == "512B" and utils.format_size_(3 * 1024 * 1024) == "3.00MB" and len(utils.format_size(10 ** 10)) <= 6
    assert align_str("ab", 4, True) == "ab  " and align_str("ab", 4, False) == "  ab"
    assert format_line(["name", "toolongvalue"], [6, 5]) == " name  tool" and item_formater(0.5) == "0.5000" and item_formater(3) == "3"
    assert dtype2nccl(torch.float16) == 6 and dtype2nccl(torch.bfloat16) == 9 and op2nccl("max") == 2
    full = _gather_value(torch.arange(5.0), 6, (5,))
    assert torch.equal(full, torch.arange(5.0))

    lin = bmt.nn.Linear(6, 4)
    bmt.init_parameters(lin)
    blk = bmt.Block(lin)
    x = torch.randn(3, 6)
    want = blk(x)
    with ZeroContext(blk):
        assert blk._module.weight.shape == (4, 6)
        got = blk._module(x)
    assert torch.allclose(got, want)
    # bracketing by hand with the identity functions gathers / releases around the inner module as well
    (xin,) = PreHookFunc.apply(blk, x.clone().requires_grad_())
    out = blk._module(xin)
    (out,) = PostHookFunc.apply(blk, out)
    assert torch.allclose(out, want)


def test_offload_optimizer_host_memory_sizing(bmt_cpu, monkeypatch):
    """The offloading optimizer states what it needs in host memory and refuses, before allocating anything, when the
    machine cannot hold the state of all its ranks."""
    bmt = bmt_cpu
    p = torch.nn.Parameter(torch.zeros(1000, dtype=torch.float32))
    opt = bmt.optim.AdamOffloadOptimizer([p], lr=1e-3)
    assert opt.host_bytes() == 1000 * 16
    monkeypatch.setattr(opt, "host_bytes", lambda: 1 << 60)
    p.grad = torch.ones_like(p)
    with pytest.raises(MemoryError):
        opt.step()
    assert len(opt.state[p]) == 0


def test_known_gradient_norms_are_only_used_when_they_apply(bmt_cpu):
    """``fused_sq_norms`` hands ``clip_grad_norm`` the sum of squares a reduce-scatter kernel left behind: only for buckets
    all of whose gradient holders are asked for, and only until gradients are rewritten in place."""
    from bmtrain_b200 import block_layer as BL

    class Slot:
        def __init__(self, p):
            self.param = p

    def bucket(n_params, value):
        b = BL._Bucket("k", torch.float32, None, bmt_cpu.config["comm"])
        b.storage = torch.nn.Parameter(torch.zeros(4))
        b.storage.grad = torch.ones(4)
        b.slots = [Slot(torch.nn.Parameter(torch.zeros(2))) for _ in range(n_params)]
        b.sqsum = torch.tensor([value])
        b.sq_tag = BL._grad_epoch[0]
        BL._fused_buckets.add(b)
        return b

    b1, b2 = bucket(2, 3.0), bucket(2, 5.0)
    inner1 = [s.param for s in b1.slots]
    other = torch.nn.Parameter(torch.zeros(3))
    # all holders of b1 asked for, only one of b2: b1 counts, b2 does not
    known, parts = BL.fused_sq_norms(inner1 + [b2.slots[0].param, other])
    assert known == {id(p) for p in inner1} and [float(t) for t in parts] == [3.0]
    # the flat storage parameter stands for its bucket as well
    known, parts = BL.fused_sq_norms([b2.storage])
    assert known == {id(b2.storage)} and [float(t) for t in parts] == [5.0]
    # dropped gradients and in-place rewrites invalidate the figures
    b1.storage.grad = None
    assert BL.fused_sq_norms(inner1)[1] == []
    BL.grads_modified()
    assert BL.fused_sq_norms([b2.storage]) == (set(), [])
    BL._fused_buckets.discard(b1)
    BL._fused_buckets.discard(b2)


def test_cpu_partition_follows_numa_nodes():
    """Ranks share out the cores of the NUMA node their GPU is attached to; without a layout the split is even."""
    from bmtrain_b200.init import _read_cpu_list, _split_cpus

    assert _read_cpu_list("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    cpus = list(range(32))
    assert _split_cpus(cpus, 1, 4) == list(range(8, 16))
    nodes = {0: list(range(0, 16)), 1: list(range(16, 32))}
    layout = (nodes, [0, 0, 0, 1])                       # three GPUs on node 0, one on node 1
    assert _split_cpus(cpus, 0, 4, layout) == [0, 1, 2, 3, 4]
    assert _split_cpus(cpus, 2, 4, layout) == [10, 11, 12, 13, 14]
    assert _split_cpus(cpus, 3, 4, layout) == list(range(16, 32))
    # a rank whose node is unknown, or whose node has fewer usable cores than ranks, keeps the even split
    assert _split_cpus(cpus, 1, 4, (nodes, [0, -1, 0, 1])) == list(range(8, 16))
    assert _split_cpus(list(range(16, 32)), 0, 2, (nodes, [0, 1])) == list(range(16, 24))
